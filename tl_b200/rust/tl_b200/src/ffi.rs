//! The C ABI of libtlb200 (include/tlb200.h), declaration for declaration: 138 entry points.
//! Handles are opaque; status codes are the values of RuntimeErrorCode (crates/tl_runtime/src/error.rs:7-18).
#![allow(non_camel_case_types)]
use std::ffi::{c_char, c_int, c_void};

pub type TlbStatus = c_int;
pub const TLB_OK: TlbStatus = 0;
pub type TlbDtype = c_int;
pub const TLB_F32: TlbDtype = 0;
pub const TLB_F16: TlbDtype = 2;
pub const TLB_I32: TlbDtype = 4;
pub const TLB_I64: TlbDtype = 5;
pub const TLB_U8: TlbDtype = 6;
pub const TLB_ROPE_CPU: c_int = 0;
pub const TLB_ROPE_HALF: c_int = 1;
pub const TLB_TIE_LAST: c_int = 0;
pub const TLB_TIE_FIRST: c_int = 1;

macro_rules! opaque { ($($n:ident),*) => { $( #[repr(C)] pub struct $n { _private: [u8; 0] } )* } }
opaque!(TlbTensor, TlbQTensor, TlbMap, TlbKvCache, TlbGraph, TlbDecoder, TlbTokenizer);

/// StringStruct of crates/tl_runtime/src/string_ffi.rs:7-11
#[repr(C)]
pub struct TlbString {
    pub ptr: *mut c_char,
    pub len: i64,
}

#[repr(C)]
#[derive(Clone, Copy, Default)]
pub struct TlbDecoderCfg {
    pub n_layers: i32,
    pub d_model: i32,
    pub n_heads: i32,
    pub n_kv_heads: i32,
    pub head_dim: i32,
    pub ffn: i32,
    pub vocab: i32,
    pub eps: f32,
    pub rope_base: f32,
    pub attn_scale: f32,
    pub kv_f16: i32,
    pub max_seq: i32,
    pub tie_rule: i32,
    pub tp_size: i32,
    pub tp_rank: i32,
    pub batch: i32,
}

#[link(name = "tlb200")]
extern "C" {
    pub fn tlb_init(device: c_int) -> TlbStatus;
    pub fn tlb_shutdown() -> TlbStatus;
    pub fn tlb_last_error() -> *const c_char;
    pub fn tlb_device_id() -> c_int;
    pub fn tlb_sync() -> TlbStatus;
    pub fn tlb_kernel_launches() -> u64;
    pub fn tlb_mem_stats(bytes_in_use: *mut u64, bytes_reserved: *mut u64) -> TlbStatus;
    pub fn tlb_event_create(ev: *mut *mut c_void) -> TlbStatus;
    pub fn tlb_event_record(ev: *mut c_void) -> TlbStatus;
    pub fn tlb_event_elapsed_ms(start: *mut c_void, stop: *mut c_void, ms: *mut f32) -> TlbStatus;
    pub fn tlb_event_destroy(ev: *mut c_void) -> TlbStatus;
    pub fn tlb_flush_l2() -> TlbStatus;
    pub fn tlb_tensor_from_host(out: *mut *mut TlbTensor, data: *const c_void, dt: TlbDtype, shape: *const i64, rank: c_int) -> TlbStatus;
    pub fn tlb_tensor_zeros(out: *mut *mut TlbTensor, dt: TlbDtype, shape: *const i64, rank: c_int) -> TlbStatus;
    pub fn tlb_tensor_to_host(t: *const TlbTensor, dst: *mut c_void, dst_bytes: usize) -> TlbStatus;
    pub fn tlb_tensor_retain(t: *mut TlbTensor) -> TlbStatus;
    pub fn tlb_tensor_release(t: *mut TlbTensor) -> TlbStatus;
    pub fn tlb_tensor_refcount(t: *const TlbTensor) -> c_int;
    pub fn tlb_tensor_rank(t: *const TlbTensor) -> c_int;
    pub fn tlb_tensor_numel(t: *const TlbTensor) -> i64;
    pub fn tlb_tensor_shape(t: *const TlbTensor, shape_out: *mut i64, max_rank: c_int) -> TlbStatus;
    pub fn tlb_tensor_dtype(t: *const TlbTensor) -> TlbDtype;
    pub fn tlb_tensor_data(t: *const TlbTensor) -> *mut c_void;
    pub fn tlb_tensor_clone(out: *mut *mut TlbTensor, t: *const TlbTensor) -> TlbStatus;
    pub fn tlb_tensor_item_i64(t: *const TlbTensor, value: *mut i64) -> TlbStatus;
    pub fn tlb_add(out: *mut *mut TlbTensor, a: *const TlbTensor, b: *const TlbTensor) -> TlbStatus;
    pub fn tlb_mul(out: *mut *mut TlbTensor, a: *const TlbTensor, b: *const TlbTensor) -> TlbStatus;
    pub fn tlb_silu(out: *mut *mut TlbTensor, a: *const TlbTensor) -> TlbStatus;
    pub fn tlb_scale(out: *mut *mut TlbTensor, a: *const TlbTensor, s: f32) -> TlbStatus;
    pub fn tlb_softmax(out: *mut *mut TlbTensor, a: *const TlbTensor, dim: i64) -> TlbStatus;
    pub fn tlb_matmul(out: *mut *mut TlbTensor, a: *const TlbTensor, b: *const TlbTensor) -> TlbStatus;
    pub fn tlb_narrow(out: *mut *mut TlbTensor, a: *const TlbTensor, dim: i64, start: i64, len: i64) -> TlbStatus;
    pub fn tlb_transpose(out: *mut *mut TlbTensor, a: *const TlbTensor, d0: i64, d1: i64) -> TlbStatus;
    pub fn tlb_reshape(out: *mut *mut TlbTensor, a: *const TlbTensor, shape: *const i64, rank: c_int) -> TlbStatus;
    pub fn tlb_cat(out: *mut *mut TlbTensor, a: *const TlbTensor, b: *const TlbTensor, dim: i64) -> TlbStatus;
    pub fn tlb_repeat_interleave(out: *mut *mut TlbTensor, a: *const TlbTensor, repeats: i64, dim: i64) -> TlbStatus;
    pub fn tlb_reshape_new(out: *mut *mut TlbTensor, a: *const TlbTensor, shape: *const TlbTensor) -> TlbStatus;
    pub fn tlb_cat_i64(out: *mut *mut TlbTensor, a: *const TlbTensor, b: *const TlbTensor, dim: i64) -> TlbStatus;
    pub fn tlb_new_causal_mask(out: *mut *mut TlbTensor, size: i64) -> TlbStatus;
    pub fn tlb_embedding(out: *mut *mut TlbTensor, table: *const TlbTensor, idx: *const TlbTensor) -> TlbStatus;
    pub fn tlb_rms_norm(out: *mut *mut TlbTensor, x: *const TlbTensor, weight: *const TlbTensor, eps: f32) -> TlbStatus;
    pub fn tlb_rope_new_cos(out: *mut *mut TlbTensor, dim: i64, seq_len: i64, base: f32, mode: c_int) -> TlbStatus;
    pub fn tlb_rope_new_sin(out: *mut *mut TlbTensor, dim: i64, seq_len: i64, base: f32, mode: c_int) -> TlbStatus;
    pub fn tlb_apply_rope(out: *mut *mut TlbTensor, x: *const TlbTensor, cos_t: *const TlbTensor, sin_t: *const TlbTensor, mode: c_int) -> TlbStatus;
    pub fn tlb_argmax(out: *mut *mut TlbTensor, x: *const TlbTensor, tie: c_int) -> TlbStatus;
    pub fn tlb_argmax_into(out: *mut TlbTensor, x: *const TlbTensor, tie: c_int) -> TlbStatus;
    pub fn tlb_sample(out: *mut *mut TlbTensor, logits: *const TlbTensor, temp: f32, top_p: f32, tie: c_int) -> TlbStatus;
    pub fn tlb_sample_top_p(out: *mut *mut TlbTensor, logits: *const TlbTensor, temp: f32, top_p: f32, u: f64, tie: c_int) -> TlbStatus;
    pub fn tlb_sample_top_k_top_p(out: *mut *mut TlbTensor, logits: *const TlbTensor, temp: f32, top_k: i32, top_p: f32, u: f64, tie: c_int) -> TlbStatus;
    pub fn tlb_rng_uniform(seed: u64, counter: u64) -> f64;
    pub fn tlb_repetition_penalty(out: *mut *mut TlbTensor, logits: *const TlbTensor, tokens: *const TlbTensor, penalty: f32) -> TlbStatus;
    pub fn tlb_sdpa(out: *mut *mut TlbTensor, q: *const TlbTensor, k: *const TlbTensor, v: *const TlbTensor, mask: *const TlbTensor, mask_mode: c_int) -> TlbStatus;
    pub fn tlb_fused_silu_mul(out: *mut *mut TlbTensor, gate: *const TlbTensor, up: *const TlbTensor) -> TlbStatus;
    pub fn tlb_fused_rms_norm(out: *mut *mut TlbTensor, x: *const TlbTensor, w: *const TlbTensor, eps: f32) -> TlbStatus;
    pub fn tlb_fused_add_rms_norm(out: *mut *mut TlbTensor, x: *const TlbTensor, residual: *const TlbTensor, w: *const TlbTensor, eps: f32) -> TlbStatus;
    pub fn tlb_fused_rotary_emb(out: *mut *mut TlbTensor, x: *const TlbTensor, freqs: *const TlbTensor, head_dim: i64) -> TlbStatus;
    pub fn tlb_qtensor_from_gguf_bytes(out: *mut *mut TlbQTensor, type_: c_int, n: i64, k: i64, bytes: *const c_void, nbytes: usize) -> TlbStatus;
    pub fn tlb_qtensor_retain(q: *mut TlbQTensor) -> TlbStatus;
    pub fn tlb_qtensor_release(q: *mut TlbQTensor) -> TlbStatus;
    pub fn tlb_qtensor_info(q: *const TlbQTensor, type_: *mut c_int, n: *mut i64, k: *mut i64, device_bytes: *mut u64) -> TlbStatus;
    pub fn tlb_qtensor_dequantize(out: *mut *mut TlbTensor, q: *const TlbQTensor) -> TlbStatus;
    pub fn tlb_qtensor_matmul(out: *mut *mut TlbTensor, x: *const TlbTensor, w: *const TlbQTensor) -> TlbStatus;
    pub fn tl_cuda_mul_mv_q4_k(x: *mut c_void, w_raw: *mut c_void, n: i64, k: i64) -> *mut c_void;
    pub fn tl_cuda_mul_mv_q6_k(x: *mut c_void, w_raw: *mut c_void, n: i64, k: i64) -> *mut c_void;
    pub fn tlb_raw_weight_cache_clear() -> i64;
    pub fn tlb_layout_unit_offset(ggml_type: c_int, row16: c_int, raw_off: c_int) -> c_int;
    pub fn tlb_layout_unit_bytes(ggml_type: c_int) -> c_int;
    pub fn tlb_gguf_load(out: *mut *mut TlbMap, path: *const c_char) -> TlbStatus;
    pub fn tlb_gguf_load_str(out: *mut *mut TlbMap, path: *const TlbString) -> TlbStatus;
    pub fn tlb_map_new(out: *mut *mut TlbMap) -> TlbStatus;
    pub fn tlb_map_add(m: *mut TlbMap, name: *const c_char, type_: c_int, shape: *const i64, rank: c_int, bytes: *const c_void, nbytes: usize) -> TlbStatus;
    pub fn tlb_map_free(m: *mut TlbMap) -> TlbStatus;
    pub fn tlb_map_count(m: *const TlbMap) -> i64;
    pub fn tlb_map_name(m: *const TlbMap, i: i64) -> *const c_char;
    pub fn tlb_map_meta_number(m: *const TlbMap, key: *const c_char, out: *mut f64) -> TlbStatus;
    pub fn tlb_map_meta_string(m: *const TlbMap, key: *const c_char) -> *const c_char;
    pub fn tlb_map_get_quantized(out: *mut *mut TlbQTensor, m: *mut TlbMap, name: *const c_char) -> TlbStatus;
    pub fn tlb_map_get(out: *mut *mut TlbTensor, m: *mut TlbMap, name: *const c_char) -> TlbStatus;
    pub fn tlb_map_get_1d(out: *mut *mut TlbTensor, m: *mut TlbMap, name: *const c_char) -> TlbStatus;
    pub fn tlb_kvcache_new(out: *mut *mut TlbKvCache, layers: i64) -> TlbStatus;
    pub fn tlb_kvcache_free(c: *mut TlbKvCache) -> TlbStatus;
    pub fn tlb_kvcache_clear(c: *mut TlbKvCache) -> TlbStatus;
    pub fn tlb_kvcache_len(c: *const TlbKvCache) -> i64;
    pub fn tlb_kvcache_resize(c: *mut TlbKvCache, layers: i64) -> TlbStatus;
    pub fn tlb_kvcache_get_k(out: *mut *mut TlbTensor, c: *mut TlbKvCache, layer: i64) -> TlbStatus;
    pub fn tlb_kvcache_get_v(out: *mut *mut TlbTensor, c: *mut TlbKvCache, layer: i64) -> TlbStatus;
    pub fn tlb_kvcache_update(c: *mut TlbKvCache, layer: i64, k: *mut TlbTensor, v: *mut TlbTensor) -> TlbStatus;
    pub fn tlb_stream_begin_capture() -> TlbStatus;
    pub fn tlb_stream_end_capture(out: *mut *mut TlbGraph) -> TlbStatus;
    pub fn tlb_stream_is_capturing() -> c_int;
    pub fn tlb_graph_replay(g: *mut TlbGraph) -> TlbStatus;
    pub fn tlb_graph_node_count(g: *const TlbGraph) -> i64;
    pub fn tlb_graph_destroy(g: *mut TlbGraph) -> TlbStatus;
    pub fn tlb_tp_unique_id(id_out: *mut c_void, id_bytes: usize) -> TlbStatus;
    pub fn tlb_tp_init(id: *const c_void, id_bytes: usize, rank: c_int, size: c_int, join_timeout_s: f64) -> TlbStatus;
    pub fn tlb_tp_poll() -> TlbStatus;
    pub fn tlb_tp_shutdown() -> TlbStatus;
    pub fn tlb_tp_rank() -> c_int;
    pub fn tlb_tp_size() -> c_int;
    pub fn tlb_allreduce(t: *mut TlbTensor) -> TlbStatus;
    pub fn tlb_tp_p2p_export(handle_out: *mut c_void, handle_bytes: usize) -> TlbStatus;
    pub fn tlb_tp_p2p_attach(handles: *const c_void, n_handles: c_int) -> TlbStatus;
    pub fn tlb_tp_p2p_disable() -> TlbStatus;
    pub fn tlb_tp_p2p_enable() -> TlbStatus;
    pub fn tlb_tp_exchange_in_launch(on: c_int) -> TlbStatus;
    pub fn tlb_tp_split_kind(name: *const c_char) -> c_int;
    pub fn tlb_tp_shard_bytes(kind: c_int, type_: c_int, n: i64, k: i64, bytes: *const c_void, nbytes: usize, rank: c_int, size: c_int, out: *mut c_void, out_cap: usize, n_out: *mut i64, k_out: *mut i64, out_bytes: *mut usize) -> TlbStatus;
    pub fn tlb_map_add_tp(m: *mut TlbMap, name: *const c_char, type_: c_int, shape: *const i64, rank: c_int, bytes: *const c_void, nbytes: usize, tp_rank: c_int, tp_size: c_int) -> TlbStatus;
    pub fn tlb_gguf_load_tp(out: *mut *mut TlbMap, path: *const c_char, tp_rank: c_int, tp_size: c_int) -> TlbStatus;
    pub fn tlb_decoder_cfg_from_map(m: *const TlbMap, cfg: *mut TlbDecoderCfg) -> TlbStatus;
    pub fn tlb_tokenizer_new(out: *mut *mut TlbTokenizer, path: *const c_char) -> TlbStatus;
    pub fn tlb_tokenizer_free(t: *mut TlbTokenizer) -> TlbStatus;
    pub fn tlb_tokenizer_vocab_size(t: *const TlbTokenizer) -> i64;
    pub fn tlb_tokenizer_id_to_token(t: *const TlbTokenizer, id: i64) -> *const c_char;
    pub fn tlb_tokenizer_encode_ids(t: *const TlbTokenizer, text: *const c_char, ids: *mut i32, cap: i64, n: *mut i64) -> TlbStatus;
    pub fn tlb_tokenizer_encode(out: *mut *mut TlbTensor, t: *const TlbTokenizer, text: *const c_char) -> TlbStatus;
    pub fn tlb_tokenizer_encode_chat(out: *mut *mut TlbTensor, t: *const TlbTokenizer, user_text: *const c_char) -> TlbStatus;
    pub fn tlb_tokenizer_encode_chat_zephyr(out: *mut *mut TlbTensor, t: *const TlbTokenizer, user_text: *const c_char) -> TlbStatus;
    pub fn tlb_tokenizer_decode(t: *mut TlbTokenizer, ids: *const TlbTensor) -> *const c_char;
    pub fn tlb_tokenizer_decode_ids(t: *mut TlbTokenizer, ids: *const i32, n: i64) -> *const c_char;
    pub fn tlb_chatbot_step_per_op(weights: *mut TlbMap, cache: *mut TlbKvCache, cos_t: *const TlbTensor, sin_t: *const TlbTensor, cfg: *const TlbDecoderCfg, tokens: *const f32, n_tokens: i64, start_pos: i64, next_token: *mut i64, logits_out: *mut *mut TlbTensor) -> TlbStatus;
    pub fn tlb_decoder_create(out: *mut *mut TlbDecoder, cfg: *const TlbDecoderCfg, weights: *mut TlbMap) -> TlbStatus;
    pub fn tlb_decoder_destroy(d: *mut TlbDecoder) -> TlbStatus;
    pub fn tlb_decoder_kv_write(d: *mut TlbDecoder, layer: c_int, pos0: c_int, n: c_int, k: *const f32, v: *const f32) -> TlbStatus;
    pub fn tlb_decoder_step(d: *mut TlbDecoder, token: i32, pos: i32, rope_pos: i32, next: *mut i32) -> TlbStatus;
    pub fn tlb_decoder_generate(d: *mut TlbDecoder, first_token: i32, start_pos: i32, n: i32, tokens_out: *mut i32) -> TlbStatus;
    pub fn tlb_decoder_prefill(d: *mut TlbDecoder, tokens: *const i32, n: i32, pos0: i32, rope_pos0: i32, rope_step: i32, next: *mut i32) -> TlbStatus;
    pub fn tlb_decoder_kv_write_seq(d: *mut TlbDecoder, seq: c_int, layer: c_int, pos0: c_int, n: c_int, k: *const f32, v: *const f32) -> TlbStatus;
    pub fn tlb_decoder_prefill_seq(d: *mut TlbDecoder, seq: i32, tokens: *const i32, n: i32, pos0: i32, rope_pos0: i32, rope_step: i32, next: *mut i32) -> TlbStatus;
    pub fn tlb_decoder_step_batch(d: *mut TlbDecoder, tokens: *const i32, pos: *const i32, rope_pos: *const i32, next: *mut i32) -> TlbStatus;
    pub fn tlb_decoder_generate_batch(d: *mut TlbDecoder, first_tokens: *const i32, start_pos: *const i32, n: i32, tokens_out: *mut i32) -> TlbStatus;
    pub fn tlb_decoder_logits_batch(d: *mut TlbDecoder, logits_out: *mut f32) -> TlbStatus;
    pub fn tlb_decoder_sample_top_p(d: *mut TlbDecoder, temp: f32, top_p: f32, u: f64, token: *mut i32) -> TlbStatus;
    pub fn tlb_decoder_generate_sampled(d: *mut TlbDecoder, first_token: i32, start_pos: i32, n: i32, temp: f32, top_k: i32, top_p: f32, seed: u64, tokens_out: *mut i32) -> TlbStatus;
    pub fn tlb_decoder_logits(d: *mut TlbDecoder, logits_out: *mut f32) -> TlbStatus;
    pub fn tlb_decoder_hidden(d: *mut TlbDecoder, hidden_out: *mut f32) -> TlbStatus;
    pub fn tlb_decoder_stats(d: *const TlbDecoder, ctx: i32, weight_bytes: *mut u64, kv_bytes: *mut u64, kernels_per_step: *mut i32) -> TlbStatus;
    pub fn tlb_decoder_time_kernel(d: *mut TlbDecoder, which: *const c_char, copies: c_int, iters: c_int, us_per_launch: *mut f32, bytes_per_launch: *mut u64) -> TlbStatus;
}
