"""Entry points that keep the reference's own raw signatures (tl_cuda_mul_mv_q4_k / _q6_k on raw GGUF bytes) and the
TL-specific argument forms (shape as a tensor, path as pointer + length)."""
import ctypes as C

import numpy as np
import pytest

import tl_b200 as tl
from tl_b200 import synth

pytestmark = pytest.mark.gpu
T = tl.Tensor.from_numpy


@pytest.mark.parametrize("t,fn", [(synth.Q4_K, "tl_cuda_mul_mv_q4_k"), (synth.Q6_K, "tl_cuda_mul_mv_q6_k")])
def test_raw_bytes_matvec_with_the_reference_signature(orc, t, fn):
    """(x, w_raw U8 tensor, n, k) -> tensor, as crates/tl_runtime/src/system.rs:316-360 calls it; the raw bytes are
    repacked once (cache keyed by the raw tensor, which it keeps alive) and the fused kernel runs on the tiled copy."""
    L = tl.lib()
    rng = np.random.default_rng(70 + t)
    n, k = 96, 1024
    raw = synth.random_quant(t, n, k, rng).reshape(-1)
    w = T(raw)                                      # U8 device tensor with the raw GGUF bytes
    assert L.tlb_raw_weight_cache_clear() >= 0
    rc0 = w.refcount()
    for m in (1, 3, 40):
        x = rng.standard_normal((m, k), dtype=np.float32)
        xt = T(x)                                   # kept in a variable: a temporary's handle would be released before the call
        h = getattr(L, fn)(xt.h, w.h, n, k)
        assert h, L.tlb_last_error()
        got = tl.Tensor(h).numpy()
        want = orc.qmatmul(t, raw, n, k, x)
        assert got.shape == (m, n)
        assert float(np.max(np.abs(got - want)) / np.max(np.abs(want))) < (1e-4 if m <= 4 else 2e-3)
    assert w.refcount() == rc0 + 1                  # one cache entry, made by the first call
    x1 = T(rng.standard_normal(k, dtype=np.float32))
    one = getattr(L, fn)(x1.h, w.h, n, k)
    assert tl.Tensor(one).shape == (n,)             # a 1-D activation gives a 1-D result
    assert not getattr(L, fn)(None, w.h, n, k)      # null -> NULL + message, as the reference's null checks
    assert b"null" in L.tlb_last_error()
    notu8 = T(np.zeros(8, dtype=np.float32))
    assert not getattr(L, fn)(x1.h, notu8.h, n, k)  # not a U8 tensor
    assert L.tlb_raw_weight_cache_clear() == 1
    assert w.refcount() == rc0


def test_tl_specific_argument_forms(orc, tmp_path):
    L = tl.lib()
    a, shp = T(np.arange(24, dtype=np.float32)), T(np.array([2, 3, 4], dtype=np.float32))
    out = C.c_void_p()
    tl.check(L.tlb_reshape_new(C.byref(out), a.h, shp.h))      # shape as an f32 tensor
    assert tl.Tensor(out).shape == (2, 3, 4)
    out = C.c_void_p()
    toks, nxt = T(np.array([1, 2], dtype=np.float32)), T(np.array([7], dtype=np.float32))
    tl.check(L.tlb_cat_i64(C.byref(out), toks.h, nxt.h, 0))   # tokens.cat_i64(nxt, 0)
    np.testing.assert_array_equal(tl.Tensor(out).numpy(), [1, 2, 7])
    tens = {"n.weight": (synth.F32, np.arange(8, dtype=np.float32).view(np.uint8), (8,))}
    path = tmp_path / "one.gguf"
    synth.write_gguf(path, tens)
    raw_path = str(path).encode()
    buf = C.create_string_buffer(raw_path + b"#trailing-bytes-not-part-of-the-string")

    class Str(C.Structure):
        _fields_ = [("ptr", C.c_char_p), ("len", C.c_int64)]
    s = Str(C.cast(buf, C.c_char_p), len(raw_path))           # TL strings carry their length; no terminator at `len`
    m = C.c_void_p()
    tl.check(L.tlb_gguf_load_str(C.byref(m), C.byref(s)))
    out = C.c_void_p()
    tl.check(L.tlb_map_get_1d(C.byref(out), m, b"n.weight"))
    np.testing.assert_array_equal(tl.Tensor(out).numpy(), np.arange(8, dtype=np.float32))
    L.tlb_map_free(m)


def test_fused_rotary_emb_uses_one_table_for_cos_and_sin():
    """crates/tl_cuda/src/ops/fused.rs:129-185 hands the same table to the rotate-half kernel as cos and as sin."""
    L = tl.lib()
    rng = np.random.default_rng(9)
    x = rng.standard_normal((5, 3, 16), dtype=np.float32)
    f = rng.standard_normal((5, 8), dtype=np.float32)
    xt, ft = T(x), T(f)
    out = C.c_void_p()
    tl.check(L.tlb_fused_rotary_emb(C.byref(out), xt.h, ft.h, 16))
    got = tl.Tensor(out).numpy()
    x0, x1, ff = x[..., :8], x[..., 8:], f[:, None, :]
    np.testing.assert_allclose(got[..., :8], x0 * ff - x1 * ff, rtol=0, atol=1e-6)
    np.testing.assert_allclose(got[..., 8:], x0 * ff + x1 * ff, rtol=0, atol=1e-6)
    bad = C.c_void_p()
    assert L.tlb_fused_rotary_emb(C.byref(bad), xt.h, ft.h, 12) == 1
