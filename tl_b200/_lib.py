"""ctypes binding of libtlb200.so: loads the in-tree shared library and declares every entry point
of include/tlb200.h.  Loading needs no GPU; compute calls fail with TLB_ERR_DEVICE without one."""
import ctypes as C
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.path.join(HERE, "libtlb200.so")
HEADER = os.path.join(HERE, "..", "include", "tlb200.h")

_lib = None


class TlbError(RuntimeError):
    """Raised when an entry point returns a non-zero status (codes of crates/tl_runtime/src/error.rs:7-18)."""

    NAMES = {1: "ShapeMismatch", 2: "DeviceError", 3: "Allocation", 4: "NullPointer", 5: "Internal",
             6: "IndexOutOfBounds", 7: "TypeMismatch", 8: "Argument", 999: "Unknown"}

    def __init__(self, code, msg):
        super().__init__("%s (%d): %s" % (self.NAMES.get(code, "?"), code, msg))
        self.code = code


class DecoderCfg(C.Structure):
    _fields_ = [("n_layers", C.c_int32), ("d_model", C.c_int32), ("n_heads", C.c_int32),
                ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("ffn", C.c_int32), ("vocab", C.c_int32),
                ("eps", C.c_float), ("rope_base", C.c_float), ("attn_scale", C.c_float),
                ("kv_f16", C.c_int32), ("max_seq", C.c_int32), ("tie_rule", C.c_int32),
                ("tp_size", C.c_int32), ("tp_rank", C.c_int32), ("batch", C.c_int32)]


def declared_symbols():
    """Names of all functions declared in include/tlb200.h (tlb_* and the reference's own tl_cuda_mul_mv_* names)."""
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b((?:tlb|tl_cuda)_[a-z0-9_]+)\s*\(", src)))


def lib():
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(SO_PATH):
        raise ImportError("libtlb200.so is not built: run `python -m tl_b200.build` (there is no CPU fallback)")
    L = C.CDLL(SO_PATH)
    vp, i64, i32, f32, u64, sz = C.c_void_p, C.c_int64, C.c_int32, C.c_float, C.c_uint64, C.c_size_t
    pvp, pi64 = C.POINTER(C.c_void_p), C.POINTER(C.c_int64)
    S = C.c_int  # tlb_status

    def d(name, res, *args):
        f = getattr(L, name)
        f.restype = res
        f.argtypes = list(args)

    d("tlb_init", S, C.c_int); d("tlb_shutdown", S); d("tlb_last_error", C.c_char_p); d("tlb_device_id", C.c_int)
    d("tlb_sync", S); d("tlb_kernel_launches", u64); d("tlb_mem_stats", S, C.POINTER(u64), C.POINTER(u64))
    d("tlb_event_create", S, pvp); d("tlb_event_record", S, vp); d("tlb_event_elapsed_ms", S, vp, vp, C.POINTER(f32))
    d("tlb_event_destroy", S, vp); d("tlb_flush_l2", S)
    d("tlb_tensor_from_host", S, pvp, vp, C.c_int, pi64, C.c_int); d("tlb_tensor_zeros", S, pvp, C.c_int, pi64, C.c_int)
    d("tlb_tensor_to_host", S, vp, vp, sz); d("tlb_tensor_retain", S, vp); d("tlb_tensor_release", S, vp)
    d("tlb_tensor_refcount", C.c_int, vp); d("tlb_tensor_rank", C.c_int, vp); d("tlb_tensor_numel", i64, vp)
    d("tlb_tensor_shape", S, vp, pi64, C.c_int); d("tlb_tensor_dtype", C.c_int, vp); d("tlb_tensor_data", vp, vp)
    d("tlb_tensor_clone", S, pvp, vp); d("tlb_tensor_item_i64", S, vp, pi64)
    for n in ("tlb_add", "tlb_mul", "tlb_matmul", "tlb_fused_silu_mul", "tlb_embedding"):
        d(n, S, pvp, vp, vp)
    d("tlb_silu", S, pvp, vp); d("tlb_scale", S, pvp, vp, f32); d("tlb_softmax", S, pvp, vp, i64)
    d("tlb_narrow", S, pvp, vp, i64, i64, i64); d("tlb_transpose", S, pvp, vp, i64, i64)
    d("tlb_reshape", S, pvp, vp, pi64, C.c_int); d("tlb_cat", S, pvp, vp, vp, i64)
    d("tlb_repeat_interleave", S, pvp, vp, i64, i64); d("tlb_new_causal_mask", S, pvp, i64)
    d("tlb_rms_norm", S, pvp, vp, vp, f32); d("tlb_fused_rms_norm", S, pvp, vp, vp, f32)
    d("tlb_fused_add_rms_norm", S, pvp, vp, vp, vp, f32)
    d("tlb_rope_new_cos", S, pvp, i64, i64, f32, C.c_int); d("tlb_rope_new_sin", S, pvp, i64, i64, f32, C.c_int)
    d("tlb_apply_rope", S, pvp, vp, vp, vp, C.c_int); d("tlb_argmax", S, pvp, vp, C.c_int)
    d("tlb_argmax_into", S, vp, vp, C.c_int)
    d("tlb_sample", S, pvp, vp, f32, f32, C.c_int); d("tlb_repetition_penalty", S, pvp, vp, vp, f32)
    d("tlb_sample_top_p", S, pvp, vp, f32, f32, C.c_double, C.c_int)
    d("tlb_sdpa", S, pvp, vp, vp, vp, vp, C.c_int)
    d("tlb_qtensor_from_gguf_bytes", S, pvp, C.c_int, i64, i64, vp, sz); d("tlb_qtensor_retain", S, vp)
    d("tlb_qtensor_release", S, vp)
    d("tlb_qtensor_info", S, vp, C.POINTER(C.c_int), pi64, pi64, C.POINTER(u64))
    d("tlb_qtensor_dequantize", S, pvp, vp); d("tlb_qtensor_matmul", S, pvp, vp, vp)
    d("tlb_layout_unit_offset", C.c_int, C.c_int, C.c_int, C.c_int); d("tlb_layout_unit_bytes", C.c_int, C.c_int)
    d("tlb_gguf_load", S, pvp, C.c_char_p); d("tlb_map_new", S, pvp)
    d("tlb_map_meta_number", S, vp, C.c_char_p, C.POINTER(C.c_double)); d("tlb_map_meta_string", C.c_char_p, vp, C.c_char_p)
    d("tlb_decoder_cfg_from_map", S, vp, vp)
    d("tlb_tokenizer_new", S, vp, C.c_char_p); d("tlb_tokenizer_free", S, vp); d("tlb_tokenizer_vocab_size", C.c_int64, vp)
    d("tlb_tokenizer_id_to_token", C.c_char_p, vp, C.c_int64)
    d("tlb_tokenizer_encode_ids", S, vp, C.c_char_p, vp, C.c_int64, vp)
    d("tlb_tokenizer_encode", S, vp, vp, C.c_char_p); d("tlb_tokenizer_encode_chat", S, vp, vp, C.c_char_p)
    d("tlb_tokenizer_encode_chat_zephyr", S, vp, vp, C.c_char_p)
    d("tlb_tokenizer_decode", C.c_char_p, vp, vp); d("tlb_tokenizer_decode_ids", C.c_char_p, vp, vp, C.c_int64)
    d("tlb_chatbot_step_per_op", S, vp, vp, vp, vp, vp, vp, C.c_int64, C.c_int64, vp, vp)
    d("tlb_map_add", S, vp, C.c_char_p, C.c_int, pi64, C.c_int, vp, sz); d("tlb_map_free", S, vp)
    d("tlb_map_count", i64, vp); d("tlb_map_name", C.c_char_p, vp, i64)
    d("tlb_map_get_quantized", S, pvp, vp, C.c_char_p); d("tlb_map_get", S, pvp, vp, C.c_char_p)
    d("tlb_kvcache_new", S, pvp, i64); d("tlb_kvcache_free", S, vp); d("tlb_kvcache_clear", S, vp)
    d("tlb_kvcache_len", i64, vp); d("tlb_kvcache_resize", S, vp, i64)
    d("tlb_kvcache_get_k", S, pvp, vp, i64); d("tlb_kvcache_get_v", S, pvp, vp, i64)
    d("tlb_kvcache_update", S, vp, i64, vp, vp)
    d("tlb_stream_begin_capture", S); d("tlb_stream_end_capture", S, pvp); d("tlb_stream_is_capturing", C.c_int)
    d("tlb_graph_replay", S, vp); d("tlb_graph_node_count", i64, vp); d("tlb_graph_destroy", S, vp)
    d("tlb_decoder_create", S, pvp, C.POINTER(DecoderCfg), vp); d("tlb_decoder_destroy", S, vp)
    d("tlb_decoder_kv_write", S, vp, C.c_int, C.c_int, C.c_int, vp, vp)
    d("tlb_decoder_step", S, vp, i32, i32, i32, C.POINTER(i32))
    d("tlb_decoder_generate", S, vp, i32, i32, i32, C.POINTER(i32))
    d("tlb_decoder_prefill", S, vp, C.POINTER(i32), i32, i32, i32, i32, C.POINTER(i32))
    d("tlb_decoder_sample_top_p", S, vp, f32, f32, C.c_double, C.POINTER(i32))
    d("tlb_decoder_logits", S, vp, vp); d("tlb_decoder_hidden", S, vp, vp)
    d("tlb_decoder_stats", S, vp, i32, C.POINTER(u64), C.POINTER(u64), C.POINTER(i32))
    d("tlb_decoder_time_kernel", S, vp, C.c_char_p, C.c_int, C.c_int, C.POINTER(f32), C.POINTER(u64))
    d("tlb_sample_top_k_top_p", S, pvp, vp, f32, i32, f32, C.c_double, C.c_int); d("tlb_rng_uniform", C.c_double, u64, u64)
    d("tlb_decoder_generate_sampled", S, vp, i32, i32, i32, f32, i32, f32, u64, C.POINTER(i32))
    d("tl_cuda_mul_mv_q4_k", vp, vp, vp, i64, i64); d("tl_cuda_mul_mv_q6_k", vp, vp, vp, i64, i64); d("tlb_raw_weight_cache_clear", i64)
    d("tlb_reshape_new", S, pvp, vp, vp); d("tlb_cat_i64", S, pvp, vp, vp, i64); d("tlb_map_get_1d", S, pvp, vp, C.c_char_p)
    d("tlb_gguf_load_str", S, pvp, vp); d("tlb_fused_rotary_emb", S, pvp, vp, vp, i64)
    pi32 = C.POINTER(i32)
    d("tlb_decoder_kv_write_seq", S, vp, C.c_int, C.c_int, C.c_int, C.c_int, vp, vp)
    d("tlb_decoder_prefill_seq", S, vp, i32, pi32, i32, i32, i32, i32, pi32)
    d("tlb_decoder_step_batch", S, vp, pi32, pi32, pi32, pi32)
    d("tlb_decoder_generate_batch", S, vp, pi32, pi32, i32, pi32)
    d("tlb_decoder_logits_batch", S, vp, vp)
    d("tlb_tp_unique_id", S, vp, sz); d("tlb_tp_init", S, vp, sz, C.c_int, C.c_int, C.c_double); d("tlb_tp_poll", S)
    d("tlb_tp_shutdown", S); d("tlb_tp_rank", C.c_int); d("tlb_tp_size", C.c_int); d("tlb_allreduce", S, vp)
    d("tlb_tp_p2p_export", S, vp, sz); d("tlb_tp_p2p_attach", S, vp, C.c_int); d("tlb_tp_p2p_disable", S); d("tlb_tp_p2p_enable", S); d("tlb_tp_exchange_in_launch", S, C.c_int)
    d("tlb_tp_split_kind", C.c_int, C.c_char_p)
    d("tlb_tp_shard_bytes", S, C.c_int, C.c_int, i64, i64, vp, sz, C.c_int, C.c_int, vp, sz, pi64, pi64, C.POINTER(sz))
    d("tlb_map_add_tp", S, vp, C.c_char_p, C.c_int, pi64, C.c_int, vp, sz, C.c_int, C.c_int)
    d("tlb_gguf_load_tp", S, pvp, C.c_char_p, C.c_int, C.c_int)
    _lib = L
    return L


def check(status):
    if status != 0:
        raise TlbError(status, lib().tlb_last_error().decode(errors="replace"))
