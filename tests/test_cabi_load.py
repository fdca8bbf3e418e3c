"""CPU-side checks of the C-ABI library: it loads without a GPU, exports every symbol the header
declares, refuses compute without a device, and its tiled weight layout is a bijection."""
import ctypes as C
import struct

import numpy as np
import pytest

import tl_b200
from tl_b200 import _lib, synth


def test_library_exports_every_declared_symbol():
    L = C.CDLL(_lib.SO_PATH)
    names = _lib.declared_symbols()
    assert len(names) > 80
    missing = [n for n in names if not hasattr(L, n)]
    assert not missing, missing


def test_binding_covers_header():
    L = _lib.lib()
    for n in _lib.declared_symbols():
        assert getattr(L, n).argtypes is not None, "no ctypes signature for " + n


def test_no_device_is_a_loud_error():
    L = _lib.lib()
    st = L.tlb_init(-1)
    if st == 0:
        pytest.skip("a CUDA device is present")
    assert st == 2  # DeviceError
    assert b"no CPU fallback" in L.tlb_last_error()
    with pytest.raises(tl_b200.TlbError) as e:
        tl_b200.Tensor.from_numpy(np.zeros(4, dtype=np.float32))
    assert e.value.code in (2, 3)
    with pytest.raises(tl_b200.TlbError):
        tl_b200.QTensor.from_gguf_bytes(synth.Q4_K, 16, 256, np.zeros(16 * 144, dtype=np.uint8))


@pytest.mark.parametrize("t,seg", [(synth.Q4_0, 8 * 18), (synth.Q8_0, 8 * 34), (synth.Q4_K, 144), (synth.Q6_K, 210)])
def test_tiled_layout_is_a_bijection(t, seg):
    L = _lib.lib()
    ub = L.tlb_layout_unit_bytes(t)
    assert ub == 16 * seg  # same bytes as GGUF: no padding inside a unit
    offs = [L.tlb_layout_unit_offset(t, i, o) for i in range(16) for o in range(seg)]
    assert min(offs) == 0 and max(offs) == ub - 1 and len(set(offs)) == ub
    assert L.tlb_layout_unit_offset(t, 16, 0) == -1 and L.tlb_layout_unit_offset(t, 0, seg) == -1
    assert ub % 16 == 0  # bulk copies move whole 16-byte lines


def test_argument_errors_need_no_device():
    L = _lib.lib()
    assert L.tlb_tensor_release(None) == 0       # release_safe: null is ignored
    assert L.tlb_qtensor_release(None) == 0
    assert L.tlb_tensor_retain(None) == 4        # NullPointer
    assert L.tlb_kvcache_len(None) == -1
    out = C.c_void_p()
    assert L.tlb_kvcache_new(C.byref(out), 3) == 0 and L.tlb_kvcache_len(out) == 3
    assert L.tlb_kvcache_resize(out, 5) == 0 and L.tlb_kvcache_len(out) == 5
    g = C.c_void_p()
    assert L.tlb_kvcache_get_k(C.byref(g), out, 7) == 6   # IndexOutOfBounds
    assert L.tlb_kvcache_get_k(C.byref(g), out, 1) == 4   # empty layer
    assert L.tlb_kvcache_free(out) == 0
    assert L.tlb_gguf_load(C.byref(out), b"/nonexistent.gguf") == 8


def test_gguf_writer_layout(tmp_path):
    """write_gguf produces the v3 header the reference's loader test writes by hand
    (crates/tl_runtime/tests/gguf_test.rs:10-62): one F32 tensor [10], data at offset 64."""
    data = np.arange(10, dtype=np.float32)
    p = tmp_path / "t.gguf"
    synth.write_gguf(p, {"tensor1": (synth.F32, data.view(np.uint8), (10,))})
    raw = p.read_bytes()
    assert raw[:4] == b"GGUF" and struct.unpack_from("<IQQ", raw, 4) == (3, 1, 0)
    assert struct.unpack_from("<Q", raw, 24)[0] == 7 and raw[32:39] == b"tensor1"
    assert struct.unpack_from("<IQIQ", raw, 39) == (1, 10, 0, 0)
    assert len(raw) == 64 + 40 + 24  # header padded 63 -> 64, 40 data bytes padded to 64
    np.testing.assert_array_equal(np.frombuffer(raw, dtype=np.float32, count=10, offset=64), data)
    # 2-D tensors store dimensions fastest-first
    w = synth.random_quant(synth.Q4_K, 32, 512, np.random.default_rng(0))
    synth.write_gguf(p, {"w": (synth.Q4_K, w.reshape(-1), (32, 512))}, metadata={"general.alignment": 64})
    raw = p.read_bytes()
    i = raw.index(b"\x01\x00\x00\x00\x00\x00\x00\x00w") + 9
    assert struct.unpack_from("<IQQI", raw, i) == (2, 512, 32, 12)


def _gguf_header(n_tensors, kvs=b"", n_kv=0, infos=b""):
    return b"GGUF" + struct.pack("<IQQ", 3, n_tensors, n_kv) + kvs + infos


def _load(tmp_path, raw):
    p = tmp_path / "h.gguf"
    p.write_bytes(raw)
    out = C.c_void_p()
    st = _lib.lib().tlb_gguf_load(C.byref(out), str(p).encode())
    n = _lib.lib().tlb_map_count(out) if st == 0 else None
    if st == 0:
        _lib.lib().tlb_map_free(out)
    return st, n


def test_gguf_hostile_headers_are_clean_errors(tmp_path):
    """Lengths and offsets of an untrusted file can neither wrap the bounds checks nor reach an allocation: truncated
    files and absurd string / array lengths give TLB_ERR_ARG; tensors whose data lies outside the file are skipped, as the
    reference skips them (crates/tl_runtime/src/gguf.rs:183-186).  None of this needs a device."""
    s = lambda b: struct.pack("<Q", len(b)) + b
    huge = 0xFFFFFFFFFFFFFFF0
    assert _load(tmp_path, b"GGUF")[0] == 8                                    # ends after the magic
    assert _load(tmp_path, b"GGUF" + struct.pack("<I", 3))[0] == 8             # truncated counts
    assert _load(tmp_path, b"GGML" + b"\0" * 40)[0] == 8                       # bad magic
    assert _load(tmp_path, _gguf_header(0, struct.pack("<Q", huge) + b"k", 1))[0] == 8        # key length wraps off + len
    kv_str = s(b"general.name") + struct.pack("<I", 8) + struct.pack("<Q", huge)
    assert _load(tmp_path, _gguf_header(0, kv_str, 1))[0] == 8                                # string value length
    kv_arr = s(b"tokens") + struct.pack("<IIQ", 9, 4, huge)
    assert _load(tmp_path, _gguf_header(0, kv_arr + b"\0" * 64, 1))[0] == 8                   # cnt * element size wraps
    kv_sarr = s(b"tokens") + struct.pack("<IIQ", 9, 8, huge)
    assert _load(tmp_path, _gguf_header(0, kv_sarr + b"\0" * 64, 1))[0] == 8                  # array of strings, absurd count
    assert _load(tmp_path, _gguf_header(5))[0] == 8                                           # tensor infos missing
    info = s(b"t") + struct.pack("<I", 1) + struct.pack("<Q", 8) + struct.pack("<IQ", 0, huge)
    assert _load(tmp_path, _gguf_header(1, infos=info) + b"\0" * 128) == (0, 0)               # offset beyond the file: skipped
    info = s(b"t") + struct.pack("<I", 2) + struct.pack("<QQ", 1 << 40, 1 << 40) + struct.pack("<IQ", 0, 0)
    assert _load(tmp_path, _gguf_header(1, infos=info) + b"\0" * 128) == (0, 0)               # shape product leaves int64: skipped
    info = s(b"t") + struct.pack("<I", 1) + struct.pack("<Q", 1 << 63) + struct.pack("<IQ", 0, 0)
    assert _load(tmp_path, _gguf_header(1, infos=info) + b"\0" * 128)[0] == 8                 # dimension above int64
    info = s(b"t") + struct.pack("<I", 1) + struct.pack("<Q", 64) + struct.pack("<IQ", 2, 0)
    assert _load(tmp_path, _gguf_header(1, infos=info) + b"\0" * 16) == (0, 0)                # Q4_0 data cut short: skipped
    kv_al = s(b"general.alignment") + struct.pack("<II", 4, 0x80000000)
    assert _load(tmp_path, _gguf_header(0, kv_al, 1))[0] == 8                                 # absurd alignment
