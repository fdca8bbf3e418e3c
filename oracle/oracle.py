"""ctypes front end of the CPU oracle (oracle/tl_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the CPU-baseline
legs of bench.py.  The product package never imports this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

F32, F16, Q4_0, Q8_0, Q4_K, Q6_K = 0, 1, 2, 8, 12, 14
Q4_1, Q5_0, Q5_1, Q8_1 = 3, 6, 7, 9


def build(force=False):
    """Compile liboracle.so in place (gcc, a second or two)."""
    so = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "tl_oracle.c")
    hdr = os.path.join(_HERE, "tl_oracle.h")
    if force or not os.path.exists(so) or os.path.getmtime(so) < max(os.path.getmtime(src), os.path.getmtime(hdr)):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return so


class LlamaCfg(C.Structure):
    _fields_ = [("n_layers", C.c_int32), ("d_model", C.c_int32), ("n_heads", C.c_int32),
                ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("ffn", C.c_int32),
                ("vocab", C.c_int32), ("eps", C.c_float), ("rope_base", C.c_float),
                ("attn_scale", C.c_float), ("kv_f16", C.c_int32), ("max_seq", C.c_int32)]


def lib():
    global _LIB
    if _LIB is None:
        L = C.CDLL(build())
        fp, u8p, sz = C.POINTER(C.c_float), C.POINTER(C.c_uint8), C.c_size_t
        L.orc_f16_to_f32.restype = C.c_float
        L.orc_f16_to_f32.argtypes = [C.c_uint16]
        L.orc_f32_to_f16.restype = C.c_uint16
        L.orc_f32_to_f16.argtypes = [C.c_float]
        L.orc_type_nbytes.restype = sz
        L.orc_type_nbytes.argtypes = [C.c_int, sz]
        L.orc_dequantize.argtypes = [C.c_int, u8p, sz, sz, fp]
        L.orc_matmul.argtypes = [fp, fp, fp, sz, sz, sz, sz, C.c_int]
        L.orc_matmul.restype = None
        L.orc_qmatmul.argtypes = [C.c_int, u8p, sz, sz, fp, sz, fp]
        L.orc_matmul_wt.argtypes = [fp, sz, sz, fp, sz, fp]
        L.orc_matmul_wt.restype = None
        L.orc_matmul_cached_t.argtypes = [fp, sz, sz, fp, sz, fp]
        L.orc_matmul_cached_t.restype = None
        L.orc_matmul_cached_t_cols.argtypes = [fp, sz, sz, fp, sz, sz, sz, fp]
        L.orc_matmul_cached_t_cols.restype = None
        L.orc_rms_norm.argtypes = [fp, fp, C.c_float, sz, sz, fp]
        L.orc_rms_norm.restype = None
        L.orc_rope_table_cpu.argtypes = [sz, sz, C.c_float, fp, fp]
        L.orc_rope_table_cpu.restype = None
        L.orc_apply_rope_cpu.argtypes = [fp, sz, sz, fp, sz, fp, sz, fp]
        L.orc_apply_rope_cpu.restype = None
        L.orc_rope_table_half.argtypes = [sz, sz, C.c_float, fp, fp]
        L.orc_rope_table_half.restype = None
        L.orc_apply_rope_rotate_half.argtypes = [fp, sz, sz, sz, fp, fp, fp]
        L.orc_apply_rope_rotate_half.restype = None
        L.orc_softmax.argtypes = [fp, sz, sz, sz, fp]
        L.orc_softmax.restype = None
        L.orc_silu.argtypes = [fp, sz, fp]
        L.orc_silu.restype = None
        for n in ("orc_add", "orc_mul"):
            getattr(L, n).argtypes = [fp, fp, sz, sz, fp]
            getattr(L, n).restype = None
        L.orc_scale.argtypes = [fp, C.c_float, sz, fp]
        L.orc_scale.restype = None
        L.orc_embedding.argtypes = [fp, sz, sz, fp, sz, fp]
        L.orc_repeat_interleave.argtypes = [fp, sz, sz, sz, sz, fp]
        L.orc_repeat_interleave.restype = None
        L.orc_causal_mask.argtypes = [sz, fp]
        L.orc_causal_mask.restype = None
        L.orc_argmax_last.argtypes = [fp, sz]
        L.orc_argmax_last.restype = sz
        L.orc_argmax_first.argtypes = [fp, sz]
        L.orc_argmax_first.restype = sz
        L.orc_sample_top_p.argtypes = [fp, sz, C.c_float, C.c_float, C.c_double]
        L.orc_sample_top_p.restype = sz
        L.orc_sample_top_k_top_p.argtypes = [fp, sz, C.c_float, C.c_long, C.c_float, C.c_double]
        L.orc_sample_top_k_top_p.restype = sz
        L.orc_philox4x32_10.argtypes = [C.POINTER(C.c_uint32), C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]
        L.orc_philox4x32_10.restype = None
        L.orc_rng_uniform.argtypes = [C.c_uint64, C.c_uint64]
        L.orc_rng_uniform.restype = C.c_double
        L.orc_repetition_penalty.argtypes = [fp, sz, fp, sz, C.c_float, fp]
        L.orc_repetition_penalty.restype = None
        L.orc_sdpa_cpu.argtypes = [fp, fp, fp, fp, sz, sz, sz, sz, fp]
        L.orc_sdpa_cpu.restype = None
        L.orc_llama_new.argtypes = [C.POINTER(LlamaCfg)]
        L.orc_llama_new.restype = C.c_void_p
        L.orc_llama_free.argtypes = [C.c_void_p]
        L.orc_llama_free.restype = None
        L.orc_llama_set_tensor.argtypes = [C.c_void_p, C.c_char_p, C.c_int, u8p, sz]
        L.orc_llama_kv_write.argtypes = [C.c_void_p, C.c_int, C.c_int, fp, fp]
        L.orc_llama_kv_write.restype = None
        L.orc_llama_kv_clear.argtypes = [C.c_void_p]
        L.orc_llama_kv_clear.restype = None
        L.orc_llama_forward.argtypes = [C.c_void_p, C.POINTER(C.c_int32), C.c_int, C.c_int, fp]
        L.orc_llama_last_hidden.argtypes = [C.c_void_p]
        L.orc_llama_last_hidden.restype = fp
        _LIB = L
    return _LIB


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(C.POINTER(C.c_float))


def _b(a):
    a = np.ascontiguousarray(a, dtype=np.uint8)
    return a, a.ctypes.data_as(C.POINTER(C.c_uint8))


def type_nbytes(t, nelem):
    return lib().orc_type_nbytes(t, nelem)


def dequantize(t, data, nelem):
    data, dp = _b(np.frombuffer(data, dtype=np.uint8) if not isinstance(data, np.ndarray) else data)
    out = np.empty(nelem, dtype=np.float32)
    rc = lib().orc_dequantize(t, dp, data.size, nelem, out.ctypes.data_as(C.POINTER(C.c_float)))
    if rc:
        raise ValueError("orc_dequantize failed (type %d, %d bytes, %d elems)" % (t, data.size, nelem))
    return out


def matmul(a, b):
    a, ap = _f(a)
    b, bp = _f(b)
    batch = int(np.prod(a.shape[:-2])) if a.ndim > 2 else 1
    m, k = (a.shape[-2], a.shape[-1]) if a.ndim >= 2 else (1, a.shape[0])
    n = b.shape[-1]
    out = np.empty(a.shape[:-2] + (m, n) if a.ndim >= 2 else (n,), dtype=np.float32)
    lib().orc_matmul(ap, bp, out.ctypes.data_as(C.POINTER(C.c_float)), batch, m, k, n, int(b.ndim > 2))
    return out


def qmatmul(t, w, n, k, x):
    w, wp = _b(w)
    x, xp = _f(x)
    m = x.size // k
    out = np.empty((m, n), dtype=np.float32)
    rc = lib().orc_qmatmul(t, wp, n, k, xp, m, out.ctypes.data_as(C.POINTER(C.c_float)))
    if rc:
        raise ValueError("orc_qmatmul failed")
    return out


def matmul_cached_t_cols(w_kn, x, j0, j1):
    """x [k] . w_kn[:, j0:j1] with the reference's strided inner loop; w_kn is [k, n] f32."""
    k, n = w_kn.shape
    x, xp = _f(x)
    out = np.empty(j1 - j0, dtype=np.float32)
    lib().orc_matmul_cached_t_cols(w_kn.ctypes.data_as(C.POINTER(C.c_float)), n, k, xp, 1, j0, j1,
                                   out.ctypes.data_as(C.POINTER(C.c_float)))
    return out


def rms_norm(x, w, eps):
    x, xp = _f(x)
    d = x.shape[-1]
    out = np.empty_like(x)
    wp = None
    if w is not None:
        w, wp = _f(w)
    lib().orc_rms_norm(xp, wp, eps, x.size // d, d, out.ctypes.data_as(C.POINTER(C.c_float)))
    return out


def rope_table_cpu(seq_len, dim, base):
    c = np.empty((seq_len, dim), dtype=np.float32)
    s = np.empty((seq_len, dim), dtype=np.float32)
    lib().orc_rope_table_cpu(seq_len, dim, base, c.ctypes.data_as(C.POINTER(C.c_float)),
                             s.ctypes.data_as(C.POINTER(C.c_float)))
    return c, s


def rope_table_half(seq_len, dim, base):
    c = np.empty((seq_len, dim // 2), dtype=np.float32)
    s = np.empty((seq_len, dim // 2), dtype=np.float32)
    lib().orc_rope_table_half(seq_len, dim, base, c.ctypes.data_as(C.POINTER(C.c_float)),
                              s.ctypes.data_as(C.POINTER(C.c_float)))
    return c, s


def apply_rope_cpu(x, cos_t, sin_t):
    x, xp = _f(x)
    cos_t, cp = _f(cos_t)
    sin_t, sp = _f(sin_t)
    out = np.empty_like(x)
    lib().orc_apply_rope_cpu(xp, x.size, x.shape[-1], cp, cos_t.size, sp, sin_t.size,
                             out.ctypes.data_as(C.POINTER(C.c_float)))
    return out


def apply_rope_rotate_half(x, cos_t, sin_t):
    """x: [tokens, heads, head_dim]"""
    x, xp = _f(x)
    cos_t, cp = _f(cos_t)
    sin_t, sp = _f(sin_t)
    out = np.empty_like(x)
    lib().orc_apply_rope_rotate_half(xp, x.shape[0], x.shape[1], x.shape[2], cp, sp,
                                     out.ctypes.data_as(C.POINTER(C.c_float)))
    return out


def softmax(x, axis):
    x, xp = _f(x)
    axis %= x.ndim
    outer = int(np.prod(x.shape[:axis]))
    inner = int(np.prod(x.shape[axis + 1:]))
    out = np.empty_like(x)
    lib().orc_softmax(xp, outer, x.shape[axis], inner, out.ctypes.data_as(C.POINTER(C.c_float)))
    return out


def silu(x):
    x, xp = _f(x)
    out = np.empty_like(x)
    lib().orc_silu(xp, x.size, out.ctypes.data_as(C.POINTER(C.c_float)))
    return out


def _binop(fn, a, b):
    a, ap = _f(a)
    b, bp = _f(b)
    out = np.empty_like(a)
    fn(ap, bp, a.size, b.size, out.ctypes.data_as(C.POINTER(C.c_float)))
    return out


def add(a, b):
    return _binop(lib().orc_add, a, b)


def mul(a, b):
    return _binop(lib().orc_mul, a, b)


def scale(a, s):
    a, ap = _f(a)
    out = np.empty_like(a)
    lib().orc_scale(ap, s, a.size, out.ctypes.data_as(C.POINTER(C.c_float)))
    return out


def embedding(table, idx):
    table, tp = _f(table)
    idx, ip = _f(idx)
    out = np.empty(idx.shape + (table.shape[1],), dtype=np.float32)
    rc = lib().orc_embedding(tp, table.shape[0], table.shape[1], ip, idx.size,
                             out.ctypes.data_as(C.POINTER(C.c_float)))
    if rc:
        raise IndexError("embedding index out of range")
    return out


def repeat_interleave(x, repeats, axis):
    x, xp = _f(x)
    outer = int(np.prod(x.shape[:axis]))
    inner = int(np.prod(x.shape[axis + 1:]))
    shp = list(x.shape)
    shp[axis] *= repeats
    out = np.empty(shp, dtype=np.float32)
    lib().orc_repeat_interleave(xp, outer, x.shape[axis], inner, repeats,
                                out.ctypes.data_as(C.POINTER(C.c_float)))
    return out


def causal_mask(n):
    out = np.empty((n, n), dtype=np.float32)
    lib().orc_causal_mask(n, out.ctypes.data_as(C.POINTER(C.c_float)))
    return out


def argmax_last(x):
    x, xp = _f(x)
    return int(lib().orc_argmax_last(xp, x.size))


def sample_top_p(x, temp, top_p, u):
    """sample_impl of the reference CPU back end with the random number u in [0, 1) supplied."""
    x, xp = _f(x)
    return int(lib().orc_sample_top_p(xp, x.size, temp, top_p, u))


def sample_top_k_top_p(x, temp, top_k, top_p, u):
    x, xp = _f(x)
    return int(lib().orc_sample_top_k_top_p(xp, x.size, temp, top_k, top_p, u))


def philox4x32_10(ctr, key):
    c = (C.c_uint32 * 4)(*ctr)
    k = (C.c_uint32 * 2)(*key)
    o = (C.c_uint32 * 4)()
    lib().orc_philox4x32_10(c, k, o)
    return [int(v) for v in o]


def rng_uniform(seed, counter):
    return float(lib().orc_rng_uniform(seed, counter))


def argmax_first(x):
    x, xp = _f(x)
    return int(lib().orc_argmax_first(xp, x.size))


def repetition_penalty(logits, tokens, penalty):
    logits, lp = _f(logits)
    tokens, tp = _f(tokens)
    out = np.empty_like(logits)
    lib().orc_repetition_penalty(lp, logits.size, tp, tokens.size, penalty,
                                 out.ctypes.data_as(C.POINTER(C.c_float)))
    return out


def sdpa_cpu(q, k, v, mask=None):
    q, qp = _f(q)
    k, kp = _f(k)
    v, vp = _f(v)
    mp = None
    if mask is not None:
        mask, mp = _f(mask)
    bh = int(np.prod(q.shape[:-2])) if q.ndim > 2 else 1
    out = np.empty_like(q)
    lib().orc_sdpa_cpu(qp, kp, vp, mp, bh, q.shape[-2], k.shape[-2], q.shape[-1],
                       out.ctypes.data_as(C.POINTER(C.c_float)))
    return out


class Llama:
    """Oracle Llama forward over GGUF-typed tensors; `tensors` maps name -> (type, bytes ndarray)."""

    def __init__(self, cfg, tensors):
        self.cfg = LlamaCfg(**cfg)
        self._keep = []
        self.h = lib().orc_llama_new(C.byref(self.cfg))
        if not self.h:
            raise MemoryError("orc_llama_new")
        for name, (t, data) in tensors.items():
            data, dp = _b(data.view(np.uint8).reshape(-1))
            self._keep.append(data)
            if lib().orc_llama_set_tensor(self.h, name.encode(), t, dp, data.size):
                raise KeyError(name)

    def kv_write(self, layer, pos, k, v):
        k, kp = _f(k)
        v, vp = _f(v)
        lib().orc_llama_kv_write(self.h, layer, pos, kp, vp)

    def forward(self, tokens, start_pos):
        tok = np.ascontiguousarray(tokens, dtype=np.int32)
        out = np.empty(self.cfg.vocab, dtype=np.float32)
        rc = lib().orc_llama_forward(self.h, tok.ctypes.data_as(C.POINTER(C.c_int32)), tok.size,
                                     start_pos, out.ctypes.data_as(C.POINTER(C.c_float)))
        if rc:
            raise RuntimeError("orc_llama_forward rc=%d" % rc)
        return out

    def last_hidden(self):
        p = lib().orc_llama_last_hidden(self.h)
        return np.ctypeslib.as_array(p, shape=(self.cfg.d_model,)).copy()

    def close(self):
        if self.h:
            lib().orc_llama_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
