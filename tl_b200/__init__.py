"""tl_b200 - host-side mirror of TL's tensor / quantized-LLM FFI over libtlb200 (sm_100a).

Names follow the reference's runtime symbols (crates/tl_runtime/src/device_ffi.rs,
system.rs, llm.rs): Tensor.matmul_quantized = tl_qtensor_matmul, Tensor.rms_norm =
tl_tensor_rms_norm, KVCache.update = tl_kvcache_update, TensorMap.load = tl_gguf_load, ...
Every call goes through the C ABI; there is no CPU path in this package.
"""
import ctypes as C
import gc

import numpy as np

from . import synth  # noqa: F401
from ._lib import DecoderCfg, TlbError, check, declared_symbols, lib  # noqa: F401

F32, F16, Q4_0, Q8_0, Q4_K, Q6_K = 0, 1, 2, 8, 12, 14
Q4_1, Q5_0, Q5_1, Q8_1 = 3, 6, 7, 9
ROPE_CPU, ROPE_HALF = 0, 1
TIE_LAST, TIE_FIRST = 0, 1
_NP_DT = {0: np.float32, 1: np.float64, 2: np.float16, 4: np.int32, 5: np.int64, 6: np.uint8, 7: np.uint32}
_DT_NP = {np.dtype(v): k for k, v in _NP_DT.items()}


def init(device=-1):
    check(lib().tlb_init(device))


def sync():
    check(lib().tlb_sync())


def kernel_launches():
    return int(lib().tlb_kernel_launches())


# ---- tensor parallelism (one process per GPU) ---------------------------------------------------------------
def rng_uniform(seed, counter):
    """The number in [0, 1) a session draws at step `counter` under `seed` (Philox-4x32-10)."""
    return float(lib().tlb_rng_uniform(int(seed), int(counter)))


def tp_unique_id():
    """128-byte communicator id; rank 0 makes it and the host passes it to the other ranks."""
    buf = (C.c_uint8 * 128)()
    check(lib().tlb_tp_unique_id(buf, 128))
    return bytes(buf)


def tp_init(uid, rank, size, join_timeout_s=60.0):
    check(lib().tlb_tp_init(uid, len(uid), rank, size, float(join_timeout_s)))


def tp_poll():
    check(lib().tlb_tp_poll())


def tp_shutdown():
    check(lib().tlb_tp_shutdown())


def tp_p2p_export():
    buf = (C.c_uint8 * 64)()
    check(lib().tlb_tp_p2p_export(buf, 64))
    return bytes(buf)


def tp_p2p_attach(handles):
    """handles: the 64-byte export of every rank, in rank order."""
    blob = b"".join(handles)
    check(lib().tlb_tp_p2p_attach(blob, len(handles)))


def tp_p2p_disable():
    check(lib().tlb_tp_p2p_disable())


def tp_p2p_enable():
    check(lib().tlb_tp_p2p_enable())


def tp_exchange_in_launch(on):
    """Decode sessions created afterwards exchange partial sums inside the matvec launches (True) or through an
    all-reduce launch of their own (False); needs attached peer memory, the same setting on all ranks."""
    check(lib().tlb_tp_exchange_in_launch(1 if on else 0))


def tp_split_kind(name):
    return int(lib().tlb_tp_split_kind(name.encode()))


def tp_shard_bytes(kind, t, n, k, data, rank, size):
    """Host-side shard of a row-major [n, k] GGUF tensor: (bytes ndarray, (n_shard, k_shard)).  Needs no device."""
    data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
    sn, sk, sb = C.c_int64(), C.c_int64(), C.c_size_t()
    src = data.ctypes.data_as(C.c_void_p)
    check(lib().tlb_tp_shard_bytes(kind, t, n, k, src, data.size, rank, size, None, 0, C.byref(sn), C.byref(sk), C.byref(sb)))
    out = np.empty(sb.value, dtype=np.uint8)
    check(lib().tlb_tp_shard_bytes(kind, t, n, k, src, data.size, rank, size, out.ctypes.data_as(C.c_void_p), out.size,
                                   C.byref(sn), C.byref(sk), C.byref(sb)))
    return out, (sn.value, sk.value)


def _shape_arg(shape):
    arr = (C.c_int64 * max(1, len(shape)))(*shape)
    return arr, len(shape)


class Tensor:
    """Reference-counted device tensor handle (one reference owned by this object)."""

    def __init__(self, handle):
        self.h = C.c_void_p(handle) if not isinstance(handle, C.c_void_p) else handle

    @staticmethod
    def _wrap(fn, *args):
        out = C.c_void_p()
        check(fn(C.byref(out), *args))
        return Tensor(out)

    @staticmethod
    def from_numpy(a):
        a = np.ascontiguousarray(a)
        if a.dtype not in _DT_NP:
            a = a.astype(np.float32)
        shp, rank = _shape_arg(a.shape)
        return Tensor._wrap(lib().tlb_tensor_from_host, a.ctypes.data_as(C.c_void_p), _DT_NP[a.dtype], shp, rank)

    @staticmethod
    def zeros(shape, dtype=F32):
        shp, rank = _shape_arg(shape)
        return Tensor._wrap(lib().tlb_tensor_zeros, dtype, shp, rank)

    @property
    def shape(self):
        r = lib().tlb_tensor_rank(self.h)
        buf = (C.c_int64 * max(1, r))()
        check(lib().tlb_tensor_shape(self.h, buf, r))
        return tuple(buf[i] for i in range(r))

    def numel(self):
        return int(lib().tlb_tensor_numel(self.h))

    def refcount(self):
        return int(lib().tlb_tensor_refcount(self.h))

    def numpy(self):
        dt = _NP_DT[lib().tlb_tensor_dtype(self.h)]
        out = np.empty(self.shape, dtype=dt)
        check(lib().tlb_tensor_to_host(self.h, out.ctypes.data_as(C.c_void_p), out.nbytes))
        return out

    def item_i64(self):
        v = C.c_int64()
        check(lib().tlb_tensor_item_i64(self.h, C.byref(v)))
        return v.value

    def clone(self):
        return Tensor._wrap(lib().tlb_tensor_clone, self.h)

    # elementwise / shape
    def add(self, o): return Tensor._wrap(lib().tlb_add, self.h, o.h)
    def mul(self, o): return Tensor._wrap(lib().tlb_mul, self.h, o.h)
    def silu(self): return Tensor._wrap(lib().tlb_silu, self.h)
    def scale(self, s): return Tensor._wrap(lib().tlb_scale, self.h, float(s))
    def softmax(self, dim): return Tensor._wrap(lib().tlb_softmax, self.h, dim)
    def matmul(self, o): return Tensor._wrap(lib().tlb_matmul, self.h, o.h)
    matmul_4d = matmul
    add_4d = add
    def narrow(self, dim, start, length): return Tensor._wrap(lib().tlb_narrow, self.h, dim, start, length)
    def transpose(self, d0, d1): return Tensor._wrap(lib().tlb_transpose, self.h, d0, d1)

    def reshape(self, shape):
        shp, rank = _shape_arg(shape)
        return Tensor._wrap(lib().tlb_reshape, self.h, shp, rank)

    def cat(self, o, dim): return Tensor._wrap(lib().tlb_cat, self.h, o.h, dim)
    cat_4d = cat
    def repeat_interleave(self, repeats, dim): return Tensor._wrap(lib().tlb_repeat_interleave, self.h, repeats, dim)
    @staticmethod
    def new_causal_mask(n): return Tensor._wrap(lib().tlb_new_causal_mask, n)
    def embedding(self, table): return Tensor._wrap(lib().tlb_embedding, table.h, self.h)

    # LLM ops
    def rms_norm(self, w, eps): return Tensor._wrap(lib().tlb_rms_norm, self.h, w.h if w is not None else None, float(eps))
    @staticmethod
    def rope_new_cos(dim, seq_len, base, mode=ROPE_CPU): return Tensor._wrap(lib().tlb_rope_new_cos, dim, seq_len, float(base), mode)
    @staticmethod
    def rope_new_sin(dim, seq_len, base, mode=ROPE_CPU): return Tensor._wrap(lib().tlb_rope_new_sin, dim, seq_len, float(base), mode)
    def apply_rope(self, cos, sin, mode=ROPE_CPU): return Tensor._wrap(lib().tlb_apply_rope, self.h, cos.h, sin.h, mode)
    def argmax(self, tie=TIE_LAST): return Tensor._wrap(lib().tlb_argmax, self.h, tie)
    def argmax_into(self, out, tie=TIE_LAST):
        """Allocation-free argmax: writes the index (as f32) into element 0 of the existing tensor `out`."""
        check(lib().tlb_argmax_into(out.h, self.h, tie))
        return out
    def sample(self, temp, top_p, tie=TIE_LAST): return Tensor._wrap(lib().tlb_sample, self.h, float(temp), float(top_p), tie)
    def sample_top_p(self, temp, top_p, u, tie=TIE_LAST):
        return Tensor._wrap(lib().tlb_sample_top_p, self.h, float(temp), float(top_p), float(u), tie)
    def sample_top_k_top_p(self, temp, top_k, top_p, u, tie=TIE_LAST):
        return Tensor._wrap(lib().tlb_sample_top_k_top_p, self.h, float(temp), int(top_k), float(top_p), float(u), tie)
    def repetition_penalty(self, tokens, p): return Tensor._wrap(lib().tlb_repetition_penalty, self.h, tokens.h, float(p))
    def sdpa(self, k, v, mask=None, mask_mode=0):
        return Tensor._wrap(lib().tlb_sdpa, self.h, k.h, v.h, mask.h if mask is not None else None, mask_mode)
    def fused_silu_mul(self, up): return Tensor._wrap(lib().tlb_fused_silu_mul, self.h, up.h)
    def fused_rms_norm(self, w, eps): return Tensor._wrap(lib().tlb_fused_rms_norm, self.h, w.h, float(eps))
    def fused_add_rms_norm(self, res, w, eps): return Tensor._wrap(lib().tlb_fused_add_rms_norm, self.h, res.h, w.h, float(eps))
    def matmul_quantized(self, qw): return Tensor._wrap(lib().tlb_qtensor_matmul, self.h, qw.h)

    def release(self):
        if self.h:
            lib().tlb_tensor_release(self.h)
            self.h = None

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


class QTensor:
    """Quantized weight in the tiled device layout (QTensor of crates/tl_runtime/src/quantized.rs:29-40)."""

    def __init__(self, handle):
        self.h = handle

    @staticmethod
    def from_gguf_bytes(t, n, k, data):
        data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        out = C.c_void_p()
        check(lib().tlb_qtensor_from_gguf_bytes(C.byref(out), t, n, k, data.ctypes.data_as(C.c_void_p), data.size))
        return QTensor(out)

    def info(self):
        t, n, k, b = C.c_int(), C.c_int64(), C.c_int64(), C.c_uint64()
        check(lib().tlb_qtensor_info(self.h, C.byref(t), C.byref(n), C.byref(k), C.byref(b)))
        return dict(type=t.value, n=n.value, k=k.value, device_bytes=b.value)

    def dequantize(self):
        return Tensor._wrap(lib().tlb_qtensor_dequantize, self.h)

    def release(self):
        if self.h:
            lib().tlb_qtensor_release(self.h)
            self.h = None

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


class TensorMap:
    """Map name -> tensor as tl_gguf_load returns it (crates/tl_runtime/src/tensor_map.rs:19-22)."""

    def __init__(self, handle):
        self.h = handle

    @staticmethod
    def load(path):
        out = C.c_void_p()
        check(lib().tlb_gguf_load(C.byref(out), str(path).encode()))
        return TensorMap(out)

    @staticmethod
    def new():
        out = C.c_void_p()
        check(lib().tlb_map_new(C.byref(out)))
        return TensorMap(out)

    def meta_number(self, key):
        v = C.c_double()
        check(lib().tlb_map_meta_number(self.h, key.encode(), C.byref(v)))
        return v.value

    def meta_string(self, key):
        v = lib().tlb_map_meta_string(self.h, key.encode())
        return v.decode() if v is not None else None

    def decoder_cfg(self):
        """Model sizes from the file's metadata, as a dict a Decoder takes."""
        c = DecoderCfg()
        check(lib().tlb_decoder_cfg_from_map(self.h, C.byref(c)))
        return {k: getattr(c, k) for k in ("n_layers", "d_model", "n_heads", "n_kv_heads", "head_dim", "ffn", "vocab",
                                           "eps", "rope_base", "attn_scale")}

    def add(self, name, t, shape, data):
        data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        shp, rank = _shape_arg(shape)
        check(lib().tlb_map_add(self.h, name.encode(), t, shp, rank, data.ctypes.data_as(C.c_void_p), data.size))

    def add_tp(self, name, t, shape, data, tp_rank, tp_size):
        """Adds only shard tp_rank of tp_size of a split tensor (whole tensor for replicated ones)."""
        data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        shp, rank = _shape_arg(shape)
        check(lib().tlb_map_add_tp(self.h, name.encode(), t, shp, rank, data.ctypes.data_as(C.c_void_p), data.size, tp_rank, tp_size))

    @staticmethod
    def load_tp(path, tp_rank, tp_size):
        out = C.c_void_p()
        check(lib().tlb_gguf_load_tp(C.byref(out), str(path).encode(), tp_rank, tp_size))
        return TensorMap(out)

    def names(self):
        return [lib().tlb_map_name(self.h, i).decode() for i in range(lib().tlb_map_count(self.h))]

    def get_quantized(self, name):
        out = C.c_void_p()
        check(lib().tlb_map_get_quantized(C.byref(out), self.h, name.encode()))
        return QTensor(out)

    def get(self, name):
        return Tensor._wrap(lib().tlb_map_get, self.h, name.encode())

    get_1d = get

    def free(self):
        if self.h:
            lib().tlb_map_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class KVCache:
    """Per-layer (K, V) handle table (crates/tl_runtime/src/llm.rs:105-174)."""

    def __init__(self, layers):
        self.h = C.c_void_p()
        check(lib().tlb_kvcache_new(C.byref(self.h), layers))

    def len(self): return int(lib().tlb_kvcache_len(self.h))
    def clear(self): check(lib().tlb_kvcache_clear(self.h))
    def resize(self, n): check(lib().tlb_kvcache_resize(self.h, n))
    def get_k(self, layer): return Tensor._wrap(lib().tlb_kvcache_get_k, self.h, layer)
    def get_v(self, layer): return Tensor._wrap(lib().tlb_kvcache_get_v, self.h, layer)
    def update(self, layer, k, v): check(lib().tlb_kvcache_update(self.h, layer, k.h, v.h))

    def free(self):
        if self.h:
            lib().tlb_kvcache_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Graph:
    """Captured stream work (GpuStream::begin_capture/end_capture + GpuGraph::replay)."""

    def __init__(self):
        self.h = None

    def __enter__(self):
        # A capture does not survive a synchronising call, and the finalisers of this module's objects make such calls
        # (a decoder's destroy, a weight's free).  Garbage that is only waiting for the cycle collector goes now, and the
        # collector stays off until the capture has ended.
        self._gc_was_on = gc.isenabled()
        gc.collect()
        gc.disable()
        try:
            check(lib().tlb_stream_begin_capture())
        except Exception:
            if self._gc_was_on:
                gc.enable()
            raise
        return self

    def __exit__(self, *exc):
        out = C.c_void_p()
        try:
            check(lib().tlb_stream_end_capture(C.byref(out)))
        finally:
            if self._gc_was_on:
                gc.enable()
        self.h = out
        return False

    def replay(self): check(lib().tlb_graph_replay(self.h))
    def node_count(self): return int(lib().tlb_graph_node_count(self.h))

    def destroy(self):
        if self.h:
            lib().tlb_graph_destroy(self.h)
            self.h = None


class Tokenizer:
    """tokenizer.json reader + BPE encoder / decoder (crates/tl_runtime/src/tokenizer.rs).  encode_ids / decode_ids work on the
    host alone; encode / encode_chat / encode_chat_zephyr return f32 id tensors on the device, as TL holds them."""

    def __init__(self, path):
        self.h = C.c_void_p()
        check(lib().tlb_tokenizer_new(C.byref(self.h), str(path).encode()))

    def vocab_size(self): return int(lib().tlb_tokenizer_vocab_size(self.h))

    def id_to_token(self, i):
        r = lib().tlb_tokenizer_id_to_token(self.h, i)
        return None if r is None else r.decode("utf-8")

    def encode_ids(self, text):
        n = C.c_int64()
        raw = text.encode("utf-8")
        check(lib().tlb_tokenizer_encode_ids(self.h, raw, None, 0, C.byref(n)))
        buf = (C.c_int32 * max(1, n.value))()
        check(lib().tlb_tokenizer_encode_ids(self.h, raw, buf, n.value, C.byref(n)))
        return [int(buf[i]) for i in range(n.value)]

    def decode_ids(self, ids):
        buf = (C.c_int32 * max(1, len(ids)))(*ids)
        return lib().tlb_tokenizer_decode_ids(self.h, buf, len(ids)).decode("utf-8", errors="replace")

    def encode(self, text): return Tensor._wrap(lib().tlb_tokenizer_encode, self.h, text.encode("utf-8"))
    def encode_chat(self, text): return Tensor._wrap(lib().tlb_tokenizer_encode_chat, self.h, text.encode("utf-8"))
    def encode_chat_zephyr(self, text): return Tensor._wrap(lib().tlb_tokenizer_encode_chat_zephyr, self.h, text.encode("utf-8"))
    def decode(self, ids): return lib().tlb_tokenizer_decode(self.h, ids.h).decode("utf-8", errors="replace")

    def free(self):
        if self.h:
            lib().tlb_tokenizer_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Decoder:
    """Fused decode session over a TensorMap holding a Llama-shaped model."""

    def __init__(self, cfg, weights, kv_f16=True, max_seq=4096, tie_rule=TIE_LAST, tp_size=1, tp_rank=0, batch=1):
        self.cfg = DecoderCfg(n_layers=cfg["n_layers"], d_model=cfg["d_model"], n_heads=cfg["n_heads"],
                              n_kv_heads=cfg["n_kv_heads"], head_dim=cfg["head_dim"], ffn=cfg["ffn"],
                              vocab=cfg["vocab"], eps=cfg["eps"], rope_base=cfg["rope_base"],
                              attn_scale=cfg["attn_scale"], kv_f16=int(kv_f16), max_seq=max_seq,
                              tie_rule=tie_rule, tp_size=tp_size, tp_rank=tp_rank, batch=batch)
        self.batch = max(1, batch)
        self.h = C.c_void_p()
        check(lib().tlb_decoder_create(C.byref(self.h), C.byref(self.cfg), weights.h))

    def kv_write(self, layer, pos0, k, v):
        k = np.ascontiguousarray(k, dtype=np.float32)
        v = np.ascontiguousarray(v, dtype=np.float32)
        check(lib().tlb_decoder_kv_write(self.h, layer, pos0, k.shape[0], k.ctypes.data_as(C.c_void_p),
                                         v.ctypes.data_as(C.c_void_p)))

    def step(self, token, pos, rope_pos=None, read=True):
        nxt = C.c_int32(-1)
        check(lib().tlb_decoder_step(self.h, token, pos, pos if rope_pos is None else rope_pos,
                                     C.byref(nxt) if read else None))
        return nxt.value

    def prefill(self, tokens, pos0=0, rope_pos0=None, rope_step=1, read=True):
        """All prompt tokens at once (cache rows pos0.., rotation rows rope_pos0 + i * rope_step); returns the greedy next token."""
        toks = (C.c_int32 * max(1, len(tokens)))(*[int(t) for t in tokens])
        nxt = C.c_int32(-1)
        check(lib().tlb_decoder_prefill(self.h, toks, len(tokens), pos0, pos0 if rope_pos0 is None else rope_pos0, rope_step,
                                        C.byref(nxt) if read else None))
        return nxt.value

    def sample_top_p(self, temp, top_p, u):
        """Sample from the logits of the last step / prompt on the device; returns the token id."""
        tok = C.c_int32(-1)
        check(lib().tlb_decoder_sample_top_p(self.h, float(temp), float(top_p), float(u), C.byref(tok)))
        return tok.value

    def generate(self, first_token, start_pos, n, read=True):
        out = (C.c_int32 * max(1, n))()
        check(lib().tlb_decoder_generate(self.h, first_token, start_pos, n, out if read else None))
        return [out[i] for i in range(n)] if read else None

    # ---- batch sessions (batch > 1): arrays are indexed by sequence
    def kv_write_seq(self, seq, layer, pos0, k, v):
        k = np.ascontiguousarray(k, dtype=np.float32)
        v = np.ascontiguousarray(v, dtype=np.float32)
        check(lib().tlb_decoder_kv_write_seq(self.h, seq, layer, pos0, k.shape[0], k.ctypes.data_as(C.c_void_p), v.ctypes.data_as(C.c_void_p)))

    def prefill_seq(self, seq, tokens, pos0=0, rope_pos0=None, rope_step=1, read=True):
        toks = (C.c_int32 * max(1, len(tokens)))(*[int(t) for t in tokens])
        nxt = C.c_int32(-1)
        check(lib().tlb_decoder_prefill_seq(self.h, seq, toks, len(tokens), pos0, pos0 if rope_pos0 is None else rope_pos0, rope_step,
                                            C.byref(nxt) if read else None))
        return nxt.value

    def step_batch(self, tokens, pos, rope_pos=None, read=True):
        B = self.batch
        t = (C.c_int32 * B)(*[int(x) for x in tokens])
        p = (C.c_int32 * B)(*[int(x) for x in pos])
        r = (C.c_int32 * B)(*[int(x) for x in rope_pos]) if rope_pos is not None else None
        out = (C.c_int32 * B)()
        check(lib().tlb_decoder_step_batch(self.h, t, p, r, out if read else None))
        return [out[i] for i in range(B)] if read else None

    def generate_batch(self, first_tokens, start_pos, n, read=True):
        B = self.batch
        t = (C.c_int32 * B)(*[int(x) for x in first_tokens])
        p = (C.c_int32 * B)(*[int(x) for x in start_pos])
        out = (C.c_int32 * max(1, n * B))()
        check(lib().tlb_decoder_generate_batch(self.h, t, p, n, out if read else None))
        return np.array(out[:n * B], dtype=np.int64).reshape(n, B) if read else None

    def logits_batch(self):
        out = np.empty((self.batch, self.cfg.vocab), dtype=np.float32)
        check(lib().tlb_decoder_logits_batch(self.h, out.ctypes.data_as(C.c_void_p)))
        return out

    def generate_sampled(self, first_token, start_pos, n, temp, top_k, top_p, seed):
        out = (C.c_int32 * max(1, n))()
        check(lib().tlb_decoder_generate_sampled(self.h, first_token, start_pos, n, float(temp), int(top_k), float(top_p), int(seed), out))
        return [out[i] for i in range(n)]

    def logits(self):
        out = np.empty(self.cfg.vocab, dtype=np.float32)
        check(lib().tlb_decoder_logits(self.h, out.ctypes.data_as(C.c_void_p)))
        return out

    def hidden(self):
        out = np.empty(self.cfg.d_model, dtype=np.float32)
        check(lib().tlb_decoder_hidden(self.h, out.ctypes.data_as(C.c_void_p)))
        return out

    def stats(self, ctx):
        w, kv, n = C.c_uint64(), C.c_uint64(), C.c_int32()
        check(lib().tlb_decoder_stats(self.h, ctx, C.byref(w), C.byref(kv), C.byref(n)))
        return dict(weight_bytes=w.value, kv_bytes=kv.value, kernels_per_step=n.value)

    def time_kernel(self, which, copies, iters):
        us, b = C.c_float(), C.c_uint64()
        check(lib().tlb_decoder_time_kernel(self.h, which.encode(), copies, iters, C.byref(us), C.byref(b)))
        return us.value, b.value

    def destroy(self):
        if self.h:
            lib().tlb_decoder_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


def map_from_tensors(tensors, tp_rank=0, tp_size=1):
    """TensorMap from the dict synth.llama_tensors returns (name -> (type, bytes, shape)); with tp_size > 1 only this
    rank's shard of every split tensor goes to the device."""
    m = TensorMap.new()
    for name, (t, data, shape) in tensors.items():
        if tp_size > 1:
            m.add_tp(name, t, shape, data, tp_rank, tp_size)
        else:
            m.add(name, t, shape, data)
    return m
