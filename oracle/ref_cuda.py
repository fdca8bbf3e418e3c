"""ctypes front end of oracle/_ref/libtlref.so: the reference's OWN CUDA kernels
(crates/tl_cuda/src/cuda_kernels/autograd.cu, compiled unmodified by `make -C oracle ref`).

TEST INFRASTRUCTURE ONLY.  The GPU tests run these kernels on the inputs they give the oracle and
libtlb200, which pins the oracle's restatement (K-quant bit layouts, RMSNorm, rotate-half RoPE, softmax,
argmax, attention, ...) on outputs of the reference itself.  The product package never imports this
module or loads that library.  Device memory comes from torch; every launch goes to the NULL stream,
as the reference does (crates/tl_cuda/src/stream.rs:17-22), followed by a device synchronisation.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.path.join(_HERE, "_ref", "libtlref.so")
_LIB = None


def build():
    """Compile the reference kernels where a TL checkout is present; returns the path or None."""
    src_root = os.environ.get("TL_REFERENCE", "/root/reference")
    cu = os.path.join(src_root, "crates", "tl_cuda", "src", "cuda_kernels", "autograd.cu")
    if os.path.exists(cu) and (not os.path.exists(SO_PATH) or os.path.getmtime(SO_PATH) < os.path.getmtime(cu)):
        subprocess.check_call(["make", "-C", _HERE, "-s", "ref", "TL_REFERENCE=" + src_root])
    return SO_PATH if os.path.exists(SO_PATH) else None


def available():
    return os.path.exists(SO_PATH)


def lib():
    global _LIB
    if _LIB is None:
        if not available():
            raise FileNotFoundError(SO_PATH + " is not built (make -C oracle ref, on a machine holding the TL checkout)")
        _LIB = C.CDLL(SO_PATH)
    return _LIB


def _dev(a, dtype=np.float32):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a, dtype=dtype)).cuda()


def _run(name, *args):
    """Calls launch_<name>(args..., stream 0) and waits.  torch tensors among `args` are passed as device pointers and
    stay referenced here until the kernel has finished (a temporary freed earlier would hand its memory to the next)."""
    import torch
    fn = getattr(lib(), name)
    fn.restype = None
    conv = [C.c_void_p(a.data_ptr()) if isinstance(a, torch.Tensor) else (C.c_void_p(0) if a is None else a) for a in args]
    fn(*conv, C.c_void_p(0))
    torch.cuda.synchronize()
    del args


def _out(shape):
    import torch
    return torch.full(tuple(shape), float("nan"), dtype=torch.float32, device="cuda")


def mul_mv(t, w_bytes, n, k, x):
    """launch_mul_mv_q4_k_kernel / _q6_k_kernel (autograd.cu:2904-2946): x [m, k] . W[n, k]^T on the raw GGUF bytes."""
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, k)
    m = x.shape[0]
    xd, wd, out = _dev(x), _dev(np.frombuffer(w_bytes, dtype=np.uint8) if not isinstance(w_bytes, np.ndarray) else w_bytes.reshape(-1), np.uint8), _out((m, n))
    _run({12: "launch_mul_mv_q4_k_kernel", 14: "launch_mul_mv_q6_k_kernel"}[t], xd, wd, out, C.c_int(m), C.c_int(n), C.c_int(k))
    return out.cpu().numpy()


def matmul(a, b):
    """launch_matmul_kernel (autograd.cu:1428): a [batch, m, k] . b [k, n] or [batch, k, n]."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    a3 = a.reshape((-1,) + a.shape[-2:])
    batch, m, k = a3.shape
    n = b.shape[-1]
    out = _out((batch, m, n))
    _run("launch_matmul_kernel", _dev(a3), _dev(b), out, C.c_int(m), C.c_int(k), C.c_int(n), C.c_int(batch), C.c_int(int(b.ndim > 2)))
    return out.cpu().numpy().reshape(a.shape[:-1] + (n,))


def softmax(x, axis):
    x = np.ascontiguousarray(x, dtype=np.float32)
    axis %= x.ndim
    outer, inner = int(np.prod(x.shape[:axis])), int(np.prod(x.shape[axis + 1:]))
    out = _out(x.shape)
    _run("launch_softmax_kernel", _dev(x), out, C.c_int(outer), C.c_int(x.shape[axis]), C.c_int(inner))
    return out.cpu().numpy()


def rms_norm(x, eps):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = _out(x.shape)
    _run("launch_rms_norm_kernel", _dev(x), out, C.c_int(x.size // x.shape[-1]), C.c_int(x.shape[-1]), C.c_float(eps))
    return out.cpu().numpy()


def fused_rms_norm(x, w, eps):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = _out(x.shape)
    _run("launch_fused_rms_norm_kernel", _dev(x), _dev(w), out, C.c_int(x.size // x.shape[-1]), C.c_int(x.shape[-1]), C.c_float(eps))
    return out.cpu().numpy()


def fused_add_rms_norm(x, res, w, eps):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = _out(x.shape)
    _run("launch_fused_add_rms_norm_kernel", _dev(x), _dev(res), _dev(w), out, C.c_int(x.size // x.shape[-1]),
         C.c_int(x.shape[-1]), C.c_float(eps))
    return out.cpu().numpy()


def fused_silu_mul(x, up):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = _out(x.shape)
    _run("launch_fused_silu_mul_kernel", _dev(x), _dev(up), out, C.c_int(x.size))
    return out.cpu().numpy()


def apply_rope(x, cos_t, sin_t):
    """launch_apply_rope_kernel (autograd.cu:1731; rotate-half): x [tokens, heads, dim], tables [seq, dim / 2]."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    tokens, heads, dim = x.shape
    out = _out(x.shape)
    _run("launch_apply_rope_kernel", _dev(x), _dev(cos_t), _dev(sin_t), out, C.c_int(tokens), C.c_int(heads), C.c_int(dim),
         C.c_int(dim // 2), C.c_int(cos_t.shape[1]), C.c_int(cos_t.shape[0]))
    return out.cpu().numpy()


def argmax_all(x):
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    out = _out((1,))
    _run("launch_argmax_all_kernel", _dev(x), out, C.c_int(x.size))
    return int(out.cpu().numpy()[0])


def causal_mask(n):
    out = _out((n, n))
    _run("launch_causal_mask_kernel", out, C.c_int(n))
    return out.cpu().numpy()


def repeat_interleave(x, repeats, axis):
    x = np.ascontiguousarray(x, dtype=np.float32)
    outer, inner = int(np.prod(x.shape[:axis])), int(np.prod(x.shape[axis + 1:]))
    shp = list(x.shape)
    shp[axis] *= repeats
    out = _out(shp)
    _run("launch_repeat_interleave_kernel", _dev(x), out, C.c_int(outer), C.c_int(inner), C.c_int(x.shape[axis]), C.c_int(repeats))
    return out.cpu().numpy()


def embedding_f32(table, idx):
    table = np.ascontiguousarray(table, dtype=np.float32)
    idx = np.ascontiguousarray(idx, dtype=np.float32).reshape(-1)
    out = _out((idx.size, table.shape[1]))
    _run("launch_embedding_f32_kernel", _dev(table), _dev(idx), out, C.c_int(idx.size), C.c_int(table.shape[1]), C.c_int(table.shape[0]))
    return out.cpu().numpy()


def repetition_penalty(logits, tokens, penalty):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    tokens = np.ascontiguousarray(tokens, dtype=np.float32).reshape(-1)
    out = _out(logits.shape)
    _run("launch_repetition_penalty_kernel", _dev(logits), _dev(tokens), out, C.c_int(logits.shape[-1]), C.c_int(tokens.size),
         C.c_float(penalty), C.c_int(logits.size))
    return out.cpu().numpy()


def sdpa(q, k, v, mask=None):
    """launch_sdpa_kernel (autograd.cu:2710; flash_attention_kernel, additive mask [sq, sk]): q [b, h, sq, d], k, v [b, h, sk, d]."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    b, h, sq, d = q.shape
    sk = k.shape[-2]
    out = _out(q.shape)
    md = _dev(mask) if mask is not None else None
    _run("launch_sdpa_kernel", _dev(q), _dev(k), _dev(v), md, out, C.c_int(b), C.c_int(h),
         C.c_int(sq), C.c_int(sk), C.c_int(d), C.c_int(int(mask is not None)))
    return out.cpu().numpy()
