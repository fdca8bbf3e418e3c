"""Seeded synthetic GGUF tensors and a GGUF v3 writer.

Real model files are not needed to exercise the path: every tensor is drawn from the value
distributions the benchmark configurations specify (random quants, f16 scales drawn as
|N(0, s)|), written in genuine GGUF block layouts, so the same bytes feed the CPU oracle and
the GPU library.  Layout facts follow the reference loader and dequantisers:
crates/tl_runtime/src/gguf.rs:61-190 (header, 32-byte data alignment, reversed dims) and
crates/tl_runtime/src/quantized.rs:182-415 (block layouts).
"""
import struct
import zlib

import numpy as np

F32, F16, Q4_0, Q8_0, Q4_K, Q6_K = 0, 1, 2, 8, 12, 14
Q4_1, Q5_0, Q5_1, Q8_1 = 3, 6, 7, 9
TYPE_NAMES = {F32: "F32", F16: "F16", Q4_0: "Q4_0", Q8_0: "Q8_0", Q4_K: "Q4_K", Q6_K: "Q6_K",
              Q4_1: "Q4_1", Q5_0: "Q5_0", Q5_1: "Q5_1", Q8_1: "Q8_1"}
BLOCK = {F32: (1, 4), F16: (1, 2), Q4_0: (32, 18), Q8_0: (32, 34), Q4_K: (256, 144), Q6_K: (256, 210),
         Q4_1: (32, 20), Q5_0: (32, 22), Q5_1: (32, 24), Q8_1: (32, 36)}


def type_nbytes(t, nelem):
    blk, nb = BLOCK[t]
    assert nelem % blk == 0
    return nelem // blk * nb


def bytes_per_weight(t):
    blk, nb = BLOCK[t]
    return nb / blk


def _rng(seed, name):
    return np.random.Generator(np.random.PCG64([seed & 0xFFFFFFFF, zlib.crc32(name.encode())]))


def _f16_abs_normal(rng, n, sigma, div=1.0):
    return (np.abs(rng.standard_normal(n, dtype=np.float32)) * np.float32(sigma) / np.float32(div)).astype(np.float16)


def random_quant(t, n, k, rng, scale_sigma=None):
    """Random tensor [n, k] of GGML type t as a uint8 array [n, row_bytes]."""
    nelem = n * k
    blk, nb = BLOCK[t]
    nblocks = nelem // blk
    if t == F32:
        return rng.standard_normal(nelem, dtype=np.float32).view(np.uint8).reshape(n, -1)
    if t == F16:
        return (rng.standard_normal(nelem, dtype=np.float32) * np.float32(scale_sigma or 0.02)).astype(np.float16).view(np.uint8).reshape(n, -1)
    if nblocks * nb >= (16 << 20):
        # large tensors: whole 64-bit draws viewed as bytes (five times faster than drawing bytes one by one); small
        # tensors keep the byte-wise draw the committed fixtures were made with
        words = rng.integers(0, 1 << 64, size=(nblocks * nb + 7) // 8, dtype=np.uint64, endpoint=False)
        out = words.view(np.uint8)[:nblocks * nb].reshape(nblocks, nb)
    else:
        out = rng.integers(0, 256, size=(nblocks, nb), dtype=np.uint8)
    if t == Q4_0:
        d = _f16_abs_normal(rng, nblocks, scale_sigma or 0.02, 8.0)
        out[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
    elif t == Q8_0:
        d = _f16_abs_normal(rng, nblocks, scale_sigma or 0.01)
        out[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
        q = out[:, 2:].view(np.int8)
        q[q == -128] = -127  # quants uniform in -127..127
    elif t == Q4_K:
        out[:, 0:2] = _f16_abs_normal(rng, nblocks, scale_sigma or 0.01).view(np.uint8).reshape(-1, 2)
        out[:, 2:4] = _f16_abs_normal(rng, nblocks, scale_sigma or 0.01).view(np.uint8).reshape(-1, 2)
    elif t == Q6_K:
        out[:, 208:210] = _f16_abs_normal(rng, nblocks, scale_sigma or 0.01).view(np.uint8).reshape(-1, 2)
    elif t in (Q4_1, Q5_0, Q5_1, Q8_1):  # f16 scale first; Q4_1 / Q5_1 / Q8_1 carry a second f16 (min, or d * sum)
        out[:, 0:2] = _f16_abs_normal(rng, nblocks, scale_sigma or 0.01).view(np.uint8).reshape(-1, 2)
        if t != Q5_0:
            out[:, 2:4] = (rng.standard_normal(nblocks, dtype=np.float32) * np.float32(scale_sigma or 0.01)).astype(np.float16).view(np.uint8).reshape(-1, 2)
    else:
        raise ValueError(t)
    return out.reshape(n, -1)


LLAMA3_8B = dict(n_layers=32, d_model=4096, n_heads=32, n_kv_heads=8, head_dim=128, ffn=14336,
                 vocab=128256, eps=1e-5, rope_base=500000.0, attn_scale=0.08839)
TINYLLAMA = dict(n_layers=22, d_model=2048, n_heads=32, n_kv_heads=4, head_dim=64, ffn=5632,
                 vocab=32000, eps=1e-5, rope_base=10000.0, attn_scale=0.125)
LLAMA3_70B = dict(n_layers=80, d_model=8192, n_heads=64, n_kv_heads=8, head_dim=128, ffn=28672,
                  vocab=128256, eps=1e-5, rope_base=500000.0, attn_scale=0.08839)


def llama_tensor_specs(cfg, linear_type, head_type=None, embd_type=F32):
    """Ordered list of (name, type, (n_out, k_in)) for a Llama-shaped decoder, named as the TL
    programs look them up (examples/apps/tinyllama/chatbot.tl:24-26,44-47,95-99,153-155)."""
    d, qd = cfg["d_model"], cfg["n_heads"] * cfg["head_dim"]
    kvd, f, v = cfg["n_kv_heads"] * cfg["head_dim"], cfg["ffn"], cfg["vocab"]
    specs = [("token_embd.weight", embd_type, (v, d))]
    for i in range(cfg["n_layers"]):
        p = "blk.%d." % i
        specs += [(p + "attn_norm.weight", F32, (d,)), (p + "attn_q.weight", linear_type, (qd, d)),
                  (p + "attn_k.weight", linear_type, (kvd, d)), (p + "attn_v.weight", linear_type, (kvd, d)),
                  (p + "attn_output.weight", linear_type, (d, qd)), (p + "ffn_norm.weight", F32, (d,)),
                  (p + "ffn_gate.weight", linear_type, (f, d)), (p + "ffn_up.weight", linear_type, (f, d)),
                  (p + "ffn_down.weight", linear_type, (d, f))]
    specs += [("output_norm.weight", F32, (d,)),
              ("output.weight", head_type if head_type is not None else linear_type, (v, d))]
    return specs


def make_tensor(name, t, shape, seed, scale_sigma=None):
    rng = _rng(seed, name)
    if len(shape) == 1:  # norm weights are 1.0
        return np.ones(shape[0], dtype=np.float32).view(np.uint8)
    n, k = shape
    if t == F32:  # embeddings N(0, 0.02)
        return (rng.standard_normal(n * k, dtype=np.float32) * np.float32(0.02)).view(np.uint8)
    return random_quant(t, n, k, rng, scale_sigma).reshape(-1)


def llama_tensors(cfg, seed, linear_type, head_type=None, embd_type=F32, scale_sigma=None, overrides=None):
    """dict name -> (type, uint8 bytes, row-major shape).  overrides: name -> GGML type for single tensors
    (mixed files such as Q4_K_M keep attn_v / ffn_down of some layers in Q6_K)."""
    out = {}
    for name, t, shape in llama_tensor_specs(cfg, linear_type, head_type, embd_type):
        t = (overrides or {}).get(name, t)
        out[name] = (t, make_tensor(name, t, shape, seed, scale_sigma), shape)
    return out


# ---------------------------------------------------------------- GGUF v3 writer

def _gguf_str(s):
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def write_gguf(path, tensors, metadata=None, alignment=32):
    """tensors: dict name -> (type, bytes ndarray, row-major shape).  Dimensions are stored
    reversed (GGML order: fastest first), as the loader expects (gguf.rs:129-136)."""
    metadata = dict(metadata or {})
    head = bytearray(b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(metadata)))
    for key, val in metadata.items():
        head += _gguf_str(key)
        if isinstance(val, str):
            head += struct.pack("<I", 8) + _gguf_str(val)
        elif isinstance(val, float):
            head += struct.pack("<If", 6, val)
        elif isinstance(val, bool):
            head += struct.pack("<IB", 7, int(val))
        elif isinstance(val, int):
            head += struct.pack("<II", 4, val)
        elif isinstance(val, (list, tuple)):  # array of u32
            head += struct.pack("<IIQ", 9, 4, len(val)) + b"".join(struct.pack("<I", x) for x in val)
        else:
            raise TypeError(type(val))
    offsets, off = {}, 0
    for name, (t, data, shape) in tensors.items():
        offsets[name] = off
        off += (data.size + alignment - 1) // alignment * alignment
    for name, (t, data, shape) in tensors.items():
        head += _gguf_str(name) + struct.pack("<I", len(shape))
        for dim in reversed(shape):
            head += struct.pack("<Q", dim)
        head += struct.pack("<IQ", t, offsets[name])
    pad = (alignment - len(head) % alignment) % alignment
    with open(path, "wb") as f:
        f.write(bytes(head) + b"\0" * pad)
        for name, (t, data, shape) in tensors.items():
            f.write(data.tobytes())
            f.write(b"\0" * ((alignment - data.size % alignment) % alignment))
