/*
 * tlb200.h - C ABI of libtlb200, a B200 (sm_100a) implementation of TL's quantized
 * Llama inference path.  Plain pointers and sizes only; no C++ or torch types.
 *
 * Each entry point names the reference interface it replaces (path within the TL
 * repository : line).  Conventions follow the reference's FFI rules
 * (docs/dev/FFI_IMPLEMENTATION_GUIDE.md:7-23, docs/dev/MEMORY_MANAGEMENT_OVERVIEW.md:36-58):
 *   - every op returns a NEW tensor handle with reference count 1 in *out;
 *   - inputs are never consumed or modified;
 *   - retain = RC+1, release = RC-1 (storage is returned to the stream-ordered pool at 0);
 *   - integers that travel inside tensors (token ids, indices) are f32 values.
 * Status codes are the reference's RuntimeErrorCode values
 * (crates/tl_runtime/src/error.rs:7-18).  On failure *out is NULL and
 * tlb_last_error() returns a thread-local message (error.rs:161-182).
 * There is no CPU fallback: every compute entry point fails with TLB_ERR_DEVICE when no
 * CUDA device is usable.
 */
#ifndef TLB200_H
#define TLB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    TLB_OK = 0, TLB_ERR_SHAPE = 1, TLB_ERR_DEVICE = 2, TLB_ERR_ALLOC = 3, TLB_ERR_NULL = 4,
    TLB_ERR_INTERNAL = 5, TLB_ERR_INDEX = 6, TLB_ERR_TYPE = 7, TLB_ERR_ARG = 8, TLB_ERR_UNKNOWN = 999
} tlb_status;

/* crates/tl_backend/src/dtype.rs:5-14 (F32, F64, F16, BF16, I32, I64, U8, U32) */
typedef enum { TLB_F32 = 0, TLB_F64 = 1, TLB_F16 = 2, TLB_BF16 = 3, TLB_I32 = 4, TLB_I64 = 5,
               TLB_U8 = 6, TLB_U32 = 7 } tlb_dtype;

/* GGML type ids as stored in GGUF (crates/tl_runtime/src/quantized.rs:10-22) */
typedef enum { TLB_GGML_F32 = 0, TLB_GGML_F16 = 1, TLB_GGML_Q4_0 = 2, TLB_GGML_Q4_1 = 3, TLB_GGML_Q5_0 = 6, TLB_GGML_Q5_1 = 7,
               TLB_GGML_Q8_0 = 8, TLB_GGML_Q8_1 = 9, TLB_GGML_Q4_K = 12, TLB_GGML_Q6_K = 14 } tlb_ggml_type;

typedef struct tlb_tensor tlb_tensor;     /* CudaTensor handle (crates/tl_cuda/src/tensor.rs:39-99) */
typedef struct tlb_qtensor tlb_qtensor;   /* QTensor (crates/tl_runtime/src/quantized.rs:29-40) */
typedef struct tlb_map tlb_map;           /* OpaqueTensorMap (crates/tl_runtime/src/tensor_map.rs:19-22) */
typedef struct tlb_kvcache tlb_kvcache;   /* OpaqueKVCache (crates/tl_runtime/src/system.rs:387-615) */
typedef struct tlb_graph tlb_graph;       /* GpuGraph (crates/tl_backend/src/graph.rs:22-31) */
typedef struct tlb_decoder tlb_decoder;   /* fused decode session; see below */
typedef struct tlb_tokenizer tlb_tokenizer; /* OpaqueTokenizer (crates/tl_runtime/src/tokenizer.rs:8-11) */

/* ---- runtime ------------------------------------------------------------------------- */
/* crates/tl_cuda/src/device.rs:79-86 get_device(): lazily binds one CUDA device and one
 * non-blocking stream.  device < 0 selects the LOCAL_RANK / 0 default. */
tlb_status  tlb_init(int device);
tlb_status  tlb_shutdown(void);
const char *tlb_last_error(void);                       /* crates/tl_runtime/src/error.rs:161-182 */
int         tlb_device_id(void);                        /* crates/tl_cuda/src/ffi_ops.rs:1243-1246 */
tlb_status  tlb_sync(void);                             /* GpuStream::synchronize, crates/tl_backend/src/stream.rs:12-31 */
uint64_t    tlb_kernel_launches(void);                  /* kernels launched (or replayed in graphs) so far */
/* pool statistics, crates/tl_cuda/src/buffer_pool.rs:58-76 */
tlb_status  tlb_mem_stats(uint64_t *bytes_in_use, uint64_t *bytes_reserved);
/* CUDA-event timing on the library's stream */
tlb_status  tlb_event_create(void **ev);
tlb_status  tlb_event_record(void *ev);
tlb_status  tlb_event_elapsed_ms(void *start, void *stop, float *ms);  /* synchronises on stop */
tlb_status  tlb_event_destroy(void *ev);
/* write `bytes` of zeros to a scratch buffer larger than L2 (evicts cached weights between timed runs) */
tlb_status  tlb_flush_l2(void);

/* ---- tensors (crates/tl_runtime/src/device_ffi.rs:684-746; crates/tl_backend/src/tensor.rs:7-55) ---- */
tlb_status tlb_tensor_from_host(tlb_tensor **out, const void *data, tlb_dtype dt, const int64_t *shape, int rank);
tlb_status tlb_tensor_zeros(tlb_tensor **out, tlb_dtype dt, const int64_t *shape, int rank);
tlb_status tlb_tensor_to_host(const tlb_tensor *t, void *dst, size_t dst_bytes);       /* syncs */
tlb_status tlb_tensor_retain(tlb_tensor *t);            /* tl_tensor_acquire */
tlb_status tlb_tensor_release(tlb_tensor *t);           /* tl_tensor_release / _release_safe / _free */
int        tlb_tensor_refcount(const tlb_tensor *t);
int        tlb_tensor_rank(const tlb_tensor *t);        /* tl_tensor_dim */
int64_t    tlb_tensor_numel(const tlb_tensor *t);       /* tl_tensor_numel / tl_tensor_len */
tlb_status tlb_tensor_shape(const tlb_tensor *t, int64_t *shape_out, int max_rank);
tlb_dtype  tlb_tensor_dtype(const tlb_tensor *t);
void      *tlb_tensor_data(const tlb_tensor *t);        /* device pointer; tl_tensor_data */
tlb_status tlb_tensor_clone(tlb_tensor **out, const tlb_tensor *t);    /* deep copy (tl_tensor_clone copies on CPU) */
tlb_status tlb_tensor_item_i64(const tlb_tensor *t, int64_t *value);   /* crates/tl_cuda/src/ffi_ops.rs:340, syncs */

/* ---- elementwise / shape ops (crates/tl_runtime/src/device_ffi.rs, line per op) ------- */
tlb_status tlb_add(tlb_tensor **out, const tlb_tensor *a, const tlb_tensor *b);          /* :809 tl_tensor_add, :1526 add_4d; numpy broadcast */
tlb_status tlb_mul(tlb_tensor **out, const tlb_tensor *a, const tlb_tensor *b);          /* :819 */
tlb_status tlb_silu(tlb_tensor **out, const tlb_tensor *a);                              /* :1070 */
tlb_status tlb_scale(tlb_tensor **out, const tlb_tensor *a, float s);                    /* :925 */
tlb_status tlb_softmax(tlb_tensor **out, const tlb_tensor *a, int64_t dim);              /* :1097 */
tlb_status tlb_matmul(tlb_tensor **out, const tlb_tensor *a, const tlb_tensor *b);       /* :834 tl_tensor_matmul, :1521 matmul_4d */
tlb_status tlb_narrow(tlb_tensor **out, const tlb_tensor *a, int64_t dim, int64_t start, int64_t len); /* :1235 */
tlb_status tlb_transpose(tlb_tensor **out, const tlb_tensor *a, int64_t d0, int64_t d1); /* :1207 */
tlb_status tlb_reshape(tlb_tensor **out, const tlb_tensor *a, const int64_t *shape, int rank); /* :1198 zero-copy view */
tlb_status tlb_cat(tlb_tensor **out, const tlb_tensor *a, const tlb_tensor *b, int64_t dim); /* :1264 cat_4d, :1259 cat2 */
tlb_status tlb_repeat_interleave(tlb_tensor **out, const tlb_tensor *a, int64_t repeats, int64_t dim); /* :1275 */
tlb_status tlb_reshape_new(tlb_tensor **out, const tlb_tensor *a, const tlb_tensor *shape);   /* :1193 tl_tensor_reshape_new: the shape as a tensor of f32 (reads it back: syncs) */
tlb_status tlb_cat_i64(tlb_tensor **out, const tlb_tensor *a, const tlb_tensor *b, int64_t dim); /* :1250 tl_tensor_cat_i64: integers travel as f32, so tlb_cat */
tlb_status tlb_new_causal_mask(tlb_tensor **out, int64_t size);                          /* :170 */
tlb_status tlb_embedding(tlb_tensor **out, const tlb_tensor *table, const tlb_tensor *idx); /* :1300; out-of-range id -> TLB_ERR_INDEX */

/* ---- LLM ops --------------------------------------------------------------------------- */
tlb_status tlb_rms_norm(tlb_tensor **out, const tlb_tensor *x, const tlb_tensor *weight /* may be NULL */, float eps); /* device_ffi.rs:1314 */
/* RoPE conventions: the CPU and CUDA back ends of the reference disagree, both are provided.
 * TLB_ROPE_CPU  (crates/tl_cpu/src/ffi.rs:2589-2685): tables [seq, dim] pair-duplicated; adjacent
 *   pairs (x[i], x[i+1]); row 0 of the table passed in rotates EVERY vector.
 * TLB_ROPE_HALF (crates/tl_cuda/src/ops/llm.rs:96-177): tables [seq, dim/2]; rotate-half
 *   (x[i], x[i+dim/2]); x is [.., tokens, heads, dim] and token t uses table row t.
 * Tables are built on the host with libm powf/cosf/sinf, as both back ends do. */
typedef enum { TLB_ROPE_CPU = 0, TLB_ROPE_HALF = 1 } tlb_rope_mode;
tlb_status tlb_rope_new_cos(tlb_tensor **out, int64_t dim, int64_t seq_len, float base, tlb_rope_mode mode); /* device_ffi.rs:1323 */
tlb_status tlb_rope_new_sin(tlb_tensor **out, int64_t dim, int64_t seq_len, float base, tlb_rope_mode mode); /* device_ffi.rs:1332 */
tlb_status tlb_apply_rope(tlb_tensor **out, const tlb_tensor *x, const tlb_tensor *cos_t, const tlb_tensor *sin_t, tlb_rope_mode mode); /* device_ffi.rs:1342 */
/* Tie rule: TLB_TIE_LAST is tl_cpu (crates/tl_cpu/src/tensor.rs:841-846), TLB_TIE_FIRST is the CUDA kernel
 * (crates/tl_cuda/src/cuda_kernels/autograd.cu:1119-1132). Result: [1] f32 holding the index. */
typedef enum { TLB_TIE_LAST = 0, TLB_TIE_FIRST = 1 } tlb_tie_rule;
tlb_status tlb_argmax(tlb_tensor **out, const tlb_tensor *x, tlb_tie_rule tie);           /* device_ffi.rs:1138 (dim ignored, scans all) */
/* No counterpart in the reference.  tlb_argmax for callers that must not allocate device memory (a
 * sampling loop on a thread that may not take the allocator's locks or fail for lack of memory, a
 * process whose memory was handed out completely at start-up): the index is written, as f32, into
 * element 0 of `out`, an f32 tensor the caller already owns, and the kernel's partial results live in a
 * fixed 16 KB array inside the library, so nothing is allocated or freed.  Limits: x holds at most
 * 4,194,304 elements (TLB_ERR_ARG beyond that; tlb_argmax has no limit); tlb_init must have run
 * (TLB_ERR_DEVICE otherwise).  The first call on a device looks up the array's address and should
 * be made outside any stream capture.  All calls share the array and each call is two launches: they go
 * to the library's one stream under a host lock, so calls from one thread or from several never interleave;
 * GPU work that touched the array from any other stream would race with them.  Nothing in the array needs
 * clearing between calls. */
tlb_status tlb_argmax_into(tlb_tensor *out, const tlb_tensor *x, tlb_tie_rule tie);
/* temp <= 0: greedy.  temp > 0: the reference CUDA path ignores temp/top_p and returns the argmax
 * (crates/tl_cuda/src/ffi_ops.rs:880-884); this entry point does the same. */
tlb_status tlb_sample(tlb_tensor **out, const tlb_tensor *logits, float temp, float top_p, tlb_tie_rule tie); /* device_ffi.rs:1158 */
/* What the reference CPU back end's sampler computes (crates/tl_cpu/src/tensor.rs:1625-1680: softmax(logits / temp),
 * stable descending order, prefix up to the first running sum above top_p, draw inside it), with the random number
 * u in [0, 1) given by the caller instead of rand::thread_rng(); temp <= 0 is the greedy branch.  Result: [1] f32. */
tlb_status tlb_sample_top_p(tlb_tensor **out, const tlb_tensor *logits, float temp, float top_p, double u, tlb_tie_rule tie);
/* The same sampler with a top-k limit as well: the kept prefix ends at the top-p cutoff or after top_k tokens, whichever comes
 * first (top_k <= 0: no limit; the reference's top_k_sample_kernel, autograd.cu:2370-2415, masks to the k best and takes
 * their argmax, which is tlb_argmax). */
tlb_status tlb_sample_top_k_top_p(tlb_tensor **out, const tlb_tensor *logits, float temp, int32_t top_k, float top_p, double u, tlb_tie_rule tie);
/* The number in [0, 1) the session generator gives for (seed, counter): Philox-4x32-10 keyed by the seed, first output word.
 * tlb_decoder_generate_sampled draws these on the device (the reference draws from rand::thread_rng(), unseeded). */
double     tlb_rng_uniform(uint64_t seed, uint64_t counter);
tlb_status tlb_repetition_penalty(tlb_tensor **out, const tlb_tensor *logits, const tlb_tensor *tokens, float penalty); /* device_ffi.rs:563 */
/* softmax(q k^T / sqrt(d) + mask) v.  mask_mode 0: none; 1: additive (CUDA, autograd.cu:2263-2367);
 * 2: zero entries become -1e9 (CPU, crates/tl_cpu/src/device_impl.rs:775-870). */
tlb_status tlb_sdpa(tlb_tensor **out, const tlb_tensor *q, const tlb_tensor *k, const tlb_tensor *v, const tlb_tensor *mask, int mask_mode); /* device_ffi.rs:535 */
/* GpuFusedOps, crates/tl_backend/src/fused_ops.rs:15-57 */
tlb_status tlb_fused_silu_mul(tlb_tensor **out, const tlb_tensor *gate, const tlb_tensor *up);
tlb_status tlb_fused_rms_norm(tlb_tensor **out, const tlb_tensor *x, const tlb_tensor *w, float eps);
tlb_status tlb_fused_add_rms_norm(tlb_tensor **out, const tlb_tensor *x, const tlb_tensor *residual, const tlb_tensor *w, float eps);
/* fused_rotary_emb(freqs, head_dim) as crates/tl_cuda/src/ops/fused.rs:129-185 computes it: rotate-half with the one table
 * [tokens, head_dim / 2] used as both cos and sin; x is [b, tokens, heads, d], [tokens, heads, d] or [tokens, d]. */
tlb_status tlb_fused_rotary_emb(tlb_tensor **out, const tlb_tensor *x, const tlb_tensor *freqs, int64_t head_dim);

/* ---- quantized weights ------------------------------------------------------------------ */
/* Upload GGUF bytes of a row-major [n, k] tensor and repack them ONCE into the tiled,
 * 16-byte-vectorised device layout (same byte count).  Replaces the raw-byte upload cached
 * in QTensor::gpu_raw_cache (crates/tl_runtime/src/system.rs:316-331).
 * Q4_0 / Q8_0 / Q4_K / Q6_K with k a multiple of 256 take the tiled layout and the fused kernels.  Every other
 * case the reference wraps in a QTensor (crates/tl_runtime/src/gguf.rs:157-177) - F32, F16, Q4_1, Q5_0, Q5_1, Q8_1,
 * and Q4_0 / Q8_0 with k only a multiple of 32 - is kept DENSE: dequantised once to f32 and multiplied through
 * the f32 matmul, the reference's own route for types without a fused kernel (system.rs:236-264).  The reference's
 * dequantiser rejects Q4_1 / Q5_0 / Q5_1 / Q8_1 (crates/tl_runtime/src/quantized.rs:108); here they follow the
 * published GGML block definitions. */
tlb_status tlb_qtensor_from_gguf_bytes(tlb_qtensor **out, tlb_ggml_type type, int64_t n, int64_t k, const void *bytes, size_t nbytes);
tlb_status tlb_qtensor_retain(tlb_qtensor *q);          /* tl_qtensor_retain, system.rs:142 */
tlb_status tlb_qtensor_release(tlb_qtensor *q);         /* tl_qtensor_release_safe / _free, system.rs:150-172 */
tlb_status tlb_qtensor_info(const tlb_qtensor *q, int *type, int64_t *n, int64_t *k, uint64_t *device_bytes);
/* QTensor::dequantize_to_tensor (quantized.rs:117-165): f32 [n, k], bit-identical to the
 * reference's CPU dequantisers (quantized.rs:167-415) */
tlb_status tlb_qtensor_dequantize(tlb_tensor **out, const tlb_qtensor *q);
/* tl_qtensor_matmul (system.rs:180-382) == tl_cuda_mul_mv_q4_k/_q6_k (crates/tl_cuda/src/ffi_ops.rs:1314-1391)
 * plus the Q4_0/Q8_0 kernels the reference lacks: y[M,N] = x[M,K] . W^T, x 1-D [K] or 2-D [M,K].
 * Up to 4 rows: the streaming matvec (int8 MMA, max-abs-rel ~1e-5).  More than 16 rows, and 5-16 rows where it is
 * the faster of the two: the tensor-core GEMM with f16 operands and f32 accumulation (~5e-4 of the row maximum). */
tlb_status tlb_qtensor_matmul(tlb_tensor **out, const tlb_tensor *x, const tlb_qtensor *w);

/* The reference's raw-bytes entry points, under the reference's own names and signatures
 * (crates/tl_runtime/src/device_ffi.rs:1805-1833; crates/tl_cuda/src/ffi_ops.rs:1314-1391): x is a tensor handle, w_raw a
 * U8 tensor handle holding the raw GGUF bytes of a [n, k] Q4_K / Q6_K weight on the device.  The bytes are repacked into
 * the tiled layout once per distinct raw tensor (a cache keyed by its device address that keeps a reference to it) and
 * every call runs the fused kernels.  NULL on failure (tlb_last_error tells why). */
void *tl_cuda_mul_mv_q4_k(void *x, void *w_raw, int64_t n, int64_t k);
void *tl_cuda_mul_mv_q6_k(void *x, void *w_raw, int64_t n, int64_t k);
int64_t tlb_raw_weight_cache_clear(void);      /* drops the repacked copies; returns how many there were */

/* Tiled-layout introspection (no counterpart in the reference; used by the layout tests): byte offset
 * inside a 16-row unit of byte raw_off of the GGUF bytes of row row16's 256-weight segment; unit size. */
int tlb_layout_unit_offset(int ggml_type, int row16, int raw_off);
int tlb_layout_unit_bytes(int ggml_type);

/* ---- GGUF loader and tensor map --------------------------------------------------------- */
tlb_status tlb_gguf_load(tlb_map **out, const char *path);                                /* crates/tl_runtime/src/gguf.rs:34 */
/* the same with the path as TL passes strings: StringStruct { ptr, len } (crates/tl_runtime/src/string_ffi.rs:7-11) */
typedef struct { char *ptr; int64_t len; } tlb_string;
tlb_status tlb_gguf_load_str(tlb_map **out, const tlb_string *path);
/* In-memory form of the loader: an empty map, then one tensor at a time from host bytes in GGUF
 * block layout with a row-major shape (what gguf.rs:129-190 builds per tensor). */
tlb_status tlb_map_new(tlb_map **out);
tlb_status tlb_map_add(tlb_map *m, const char *name, tlb_ggml_type type, const int64_t *shape, int rank, const void *bytes, size_t nbytes);
tlb_status tlb_map_free(tlb_map *m);                                                      /* tensor_map.rs tl_tensor_map_free */
int64_t    tlb_map_count(const tlb_map *m);
const char *tlb_map_name(const tlb_map *m, int64_t i);
/* Scalar (integer, float, bool) and string metadata of a loaded GGUF file, by key (gguf.rs:61-110 reads and drops them
 * except general.alignment).  TLB_ERR_INDEX / NULL when the key is absent or of another kind. */
tlb_status tlb_map_meta_number(const tlb_map *m, const char *key, double *out);
const char *tlb_map_meta_string(const tlb_map *m, const char *key);
tlb_status tlb_map_get_quantized(tlb_qtensor **out, tlb_map *m, const char *name);        /* tensor_map.rs:279 (retained clone) */
tlb_status tlb_map_get(tlb_tensor **out, tlb_map *m, const char *name);                   /* tensor_map.rs:110 dequantised f32, cached */
tlb_status tlb_map_get_1d(tlb_tensor **out, tlb_map *m, const char *name);                /* tl_tensor_map_get_1d (src/compiler/codegen/builtins.rs:2687): same lookup */

/* ---- KV cache handle table (crates/tl_runtime/src/system.rs:387-615, llm.rs:105-174) ----- */
tlb_status tlb_kvcache_new(tlb_kvcache **out, int64_t layers);
tlb_status tlb_kvcache_free(tlb_kvcache *c);
tlb_status tlb_kvcache_clear(tlb_kvcache *c);
int64_t    tlb_kvcache_len(const tlb_kvcache *c);
tlb_status tlb_kvcache_resize(tlb_kvcache *c, int64_t layers);
tlb_status tlb_kvcache_get_k(tlb_tensor **out, tlb_kvcache *c, int64_t layer);           /* retained */
tlb_status tlb_kvcache_get_v(tlb_tensor **out, tlb_kvcache *c, int64_t layer);
tlb_status tlb_kvcache_update(tlb_kvcache *c, int64_t layer, tlb_tensor *k, tlb_tensor *v);

/* ---- stream capture / graphs (crates/tl_backend/src/stream.rs:12-31, graph.rs:22-31) ----
 * Between begin and end, entry points that wait for the device return TLB_ERR_ARG and leave the capture usable.  A
 * tlb_decoder_destroy made in between takes effect when the capture ends.  Freeing weights (tlb_qtensor_release of the
 * last reference, tlb_map_free) in between is the caller's to avoid: it synchronises and the capture does not survive it
 * (a host language with finalisers keeps its collector off for the duration, as the Python mirror's Graph does). */
tlb_status tlb_stream_begin_capture(void);
tlb_status tlb_stream_end_capture(tlb_graph **out);
int        tlb_stream_is_capturing(void);
tlb_status tlb_graph_replay(tlb_graph *g);
int64_t    tlb_graph_node_count(const tlb_graph *g);
tlb_status tlb_graph_destroy(tlb_graph *g);

/* ---- tensor parallelism over the GPUs of one node (no counterpart in the reference: crates/tl_cuda/src/device.rs:21-27
 * binds one device, the collectives of crates/tl_cuda/src/ffi_ops.rs:726-730 are stubs) ---------------------------------
 * One process per GPU.  Rank 0 makes a 128-byte id (tlb_tp_unique_id), the host passes it to the other processes, and
 * every rank joins with tlb_tp_init after tlb_init.  Joining is bounded: a rank that never arrives makes the others return
 * TLB_ERR_DEVICE after join_timeout_s (<= 0: 60 s) with the communicator aborted.  tlb_tp_poll reports an asynchronous
 * failure of an earlier collective (a peer that died) without blocking. */
tlb_status tlb_tp_unique_id(void *id_out, size_t id_bytes);
tlb_status tlb_tp_init(const void *id, size_t id_bytes, int rank, int size, double join_timeout_s);
tlb_status tlb_tp_poll(void);
tlb_status tlb_tp_shutdown(void);
int        tlb_tp_rank(void);
int        tlb_tp_size(void);
/* f32 sum over the ranks, in place, on the library's stream */
tlb_status tlb_allreduce(tlb_tensor *t);
/* Optional second transport for the small sums of decoding (up to 65,536 floats): a one-shot all-reduce in which every
 * rank stores its share into a slot of every peer's memory over NVLink and then reads only its own memory.  Each rank
 * exports a 64-byte CUDA IPC handle, the host gathers them in rank order, each rank attaches; all ranks must have
 * exported before any attaches and attached before the next all-reduce.  Sums are bitwise equal on every rank.  A peer
 * that does not write within about a second makes the kernel give up (TLB_ERR_DEVICE at the next tlb_sync). */
tlb_status tlb_tp_p2p_export(void *handle_out, size_t handle_bytes);
tlb_status tlb_tp_p2p_attach(const void *handles, int n_handles);
tlb_status tlb_tp_p2p_disable(void);   /* back to NCCL for every size (all ranks together, between steps) */
tlb_status tlb_tp_p2p_enable(void);    /* and on again, without re-attaching */
/* With peer memory attached, batch-1 decode sessions created afterwards exchange their partial sums inside the matvec
 * launches (on, the default: o_proj / ffn_down push their tiles to every rank, the next launch adds them while it
 * loads) or through an all-reduce launch of their own between the matvecs (off).  All ranks the same setting. */
tlb_status tlb_tp_exchange_in_launch(int on);
/* Which way a tensor is split, by its GGUF name: 0 replicated, 1 along rows (attn_q/k/v, ffn_gate/up, output.weight),
 * 2 along columns (attn_output, ffn_down). */
int        tlb_tp_split_kind(const char *name);
/* Host-side byte slice of a row-major [n, k] GGUF tensor for shard `rank` of `size`: rows [rank n/size, ...) for kind 1
 * (one contiguous range), for kind 2 the blocks of columns [rank k/size, ...) of every row (k/size must hold whole blocks).
 * out == NULL only reports the shard's shape and byte count.  No device is needed. */
tlb_status tlb_tp_shard_bytes(int kind, tlb_ggml_type type, int64_t n, int64_t k, const void *bytes, size_t nbytes, int rank, int size,
                              void *out, size_t out_cap, int64_t *n_out, int64_t *k_out, size_t *out_bytes);
/* tlb_map_add / tlb_gguf_load keeping only this rank's shard of every split tensor */
tlb_status tlb_map_add_tp(tlb_map *m, const char *name, tlb_ggml_type type, const int64_t *shape, int rank, const void *bytes, size_t nbytes,
                          int tp_rank, int tp_size);
tlb_status tlb_gguf_load_tp(tlb_map **out, const char *path, int tp_rank, int tp_size);

/* ---- fused decode session ---------------------------------------------------------------
 * Runs the op sequence of examples/apps/llama3/chatbot_llama3.tl:66-125,220-236 (and
 * examples/apps/tinyllama/chatbot.tl:50-113) for one new token as a chain of fused kernels
 * inside one CUDA graph: norm+QKV, RoPE+KV-append+split-K attention, o_proj, norm+gate/up,
 * silu*up+down, norm+head, argmax.  KV lives in a preallocated [L][KVH][max_seq][D] cache. */
typedef struct {
    int32_t n_layers, d_model, n_heads, n_kv_heads, head_dim, ffn, vocab;
    float   eps, rope_base, attn_scale;   /* attn_scale: the f32 literal the TL program passes to scale() */
    int32_t kv_f16;                       /* 1: f16 KV cache; 0: f32 (reference) */
    int32_t max_seq;
    int32_t tie_rule;                     /* tlb_tie_rule for the greedy token */
    /* tensor parallelism (one process per GPU): this process holds shard tp_rank of tp_size - whole heads of
     * q / k / v, hidden units of gate / up and vocabulary rows of the head (row split), the matching inner-dimension
     * slices of attn_output / ffn_down (column split) - loaded with tlb_gguf_load_tp / tlb_map_add_tp, after
     * tlb_tp_init; the model sizes above stay those of the WHOLE model.  0 or 1 / 0 for a single GPU. */
    int32_t tp_size, tp_rank;
    /* sequences the session holds (0 or 1: one).  Every sequence has its own cache rows and position; sequence 0 is the
     * one the single-sequence entry points (tlb_decoder_step, _generate, _prefill, _kv_write) work on. */
    int32_t batch;
} tlb_decoder_cfg;

/* Fills the model sizes of *cfg from the GGUF metadata of a loaded file (<arch>.block_count, .embedding_length, ...;
 * the reference programs hard-code them, examples/apps/llama3/chatbot_llama3.tl:67-71,95,106,196); kv_f16, max_seq, tie_rule and
 * the tp fields stay as the caller set them. */
tlb_status tlb_decoder_cfg_from_map(const tlb_map *m, tlb_decoder_cfg *cfg);

/* ---- tokenizer (host code; crates/tl_runtime/src/tokenizer.rs, which wraps the `tokenizers` crate 0.22.2).  Reads a Hugging
 * Face tokenizer.json of a BPE model in one of the two styles the reference's programs load: byte-level (Llama-3: Split
 * with the Llama-3 or GPT-2 pattern + ByteLevel) or SentencePiece-style (TinyLlama / Llama-2: Prepend + Replace normalizer,
 * byte fallback).  Anything else in the file is refused with TLB_ERR_TYPE.  Ids travel as f32 tensors, as TL holds them. */
tlb_status tlb_tokenizer_new(tlb_tokenizer **out, const char *path);                                 /* :16 tl_tokenizer_new */
tlb_status tlb_tokenizer_free(tlb_tokenizer *t);
int64_t    tlb_tokenizer_vocab_size(const tlb_tokenizer *t);                                           /* added tokens included */
const char *tlb_tokenizer_id_to_token(const tlb_tokenizer *t, int64_t id);                             /* NULL outside the vocabulary */
/* encode(text, add_special_tokens = false): ids into a host buffer (ids may be NULL to ask for the count), no device needed */
tlb_status tlb_tokenizer_encode_ids(const tlb_tokenizer *t, const char *text, int32_t *ids, int64_t cap, int64_t *n);
tlb_status tlb_tokenizer_encode(tlb_tensor **out, const tlb_tokenizer *t, const char *text);           /* :44 BOS = 1 in front */
tlb_status tlb_tokenizer_encode_chat(tlb_tensor **out, const tlb_tokenizer *t, const char *user_text); /* :136 Llama-3 template, special ids 128000 / 128006 / 128007 / 128009 */
tlb_status tlb_tokenizer_encode_chat_zephyr(tlb_tensor **out, const tlb_tokenizer *t, const char *user_text); /* :210 */
/* decode: one id -> its vocabulary text (byte tokens as their byte, <|...|> as nothing, U+2581 / U+0120 as a space, U+010A as a
 * line break); several -> decode(ids, skip_special_tokens = true).  The string lives until the next decode on this tokenizer. */
const char *tlb_tokenizer_decode(tlb_tokenizer *t, const tlb_tensor *ids);                              /* :73 */
const char *tlb_tokenizer_decode_ids(tlb_tokenizer *t, const int32_t *ids, int64_t n);

/* The TL chatbot's forward pass over `tokens` (f32-encoded ids, as TL holds them) from cache row start_pos, issued op by
 * op through the per-op entry points above, in the program's order (examples/apps/llama3/chatbot_llama3.tl:48-125,220-236):
 * the route an unmodified TL program takes, from native code.  cos_t / sin_t: Tensor::rope_new_cos / _sin tables; the
 * cache grows by concatenation (tlb_kvcache_*).  *next_token: lo.narrow(last).sample(0.0, 0.9).item_i64(); the last row
 * of the logits when logits_out is not NULL.  Uses cfg's sizes, eps, attn_scale and tie_rule. */
tlb_status tlb_chatbot_step_per_op(tlb_map *weights, tlb_kvcache *cache, const tlb_tensor *cos_t, const tlb_tensor *sin_t,
                                   const tlb_decoder_cfg *cfg, const float *tokens, int64_t n_tokens, int64_t start_pos,
                                   int64_t *next_token, tlb_tensor **logits_out);
tlb_status tlb_decoder_create(tlb_decoder **out, const tlb_decoder_cfg *cfg, tlb_map *weights);
tlb_status tlb_decoder_destroy(tlb_decoder *d);
/* overwrite cached K/V rows [pos0, pos0+n) of one layer from host f32 [n, n_kv_heads*head_dim] */
tlb_status tlb_decoder_kv_write(tlb_decoder *d, int layer, int pos0, int n, const float *k, const float *v);
/* One token through the model: the token's K/V go to cache row `pos`, attention spans rows [0, pos],
 * RoPE uses angle position `rope_pos` (the reference CPU path rotates a whole prompt at the position
 * of its first token; pass rope_pos = pos for plain decoding).  Host in, host out: the token id is
 * copied to the device, the greedy next token is copied back (*next may be NULL to skip the read). */
tlb_status tlb_decoder_step(tlb_decoder *d, int32_t token, int32_t pos, int32_t rope_pos, int32_t *next);
/* n greedy steps with the token fed back on the device, no host round trip in between;
 * tokens_out (host, n entries, may be NULL) is read back once at the end. */
tlb_status tlb_decoder_generate(tlb_decoder *d, int32_t first_token, int32_t start_pos, int32_t n, int32_t *tokens_out);
/* A whole prompt at once: token i goes to cache row pos0 + i and is rotated by table row rope_pos0 + i * rope_step
 * (rope_step 1: every token at its own position; rope_step 0: the whole prompt at rope_pos0, which is what the
 * reference CPU path does, crates/tl_cpu/src/ffi.rs:2661-2674).  Same result as n calls of tlb_decoder_step within
 * the f16 operand rounding of the tensor-core GEMMs (examples/apps/llama3/chatbot_llama3.tl:220-236 runs the same
 * layers on the whole prompt); *next (may be NULL) receives the greedy token after the last prompt token, and
 * tlb_decoder_logits / tlb_decoder_hidden then describe that last token.  Prompts of 16 tokens or fewer, and
 * shapes the GEMM does not take, run token by token through the fused chain. */
tlb_status tlb_decoder_prefill(tlb_decoder *d, const int32_t *tokens, int32_t n, int32_t pos0, int32_t rope_pos0, int32_t rope_step, int32_t *next);
/* ---- a batch of sequences in one session (cfg.batch > 1) ----
 * The reference's matmul entry takes any number of activation rows (crates/tl_runtime/src/system.rs:180-222) and the TL
 * program's layers are batch-agnostic (examples/apps/llama3/chatbot_llama3.tl:220-236).  Here one token per sequence goes
 * through every linear layer as one pass over the weights (tensor-core GEMM, so the session needs the shapes that path
 * takes), and through attention as independent sequences.  Arrays are indexed by sequence. */
tlb_status tlb_decoder_kv_write_seq(tlb_decoder *d, int seq, int layer, int pos0, int n, const float *k, const float *v);
/* a prompt for ONE sequence of the batch (arguments as tlb_decoder_prefill); *next: the greedy token after it */
tlb_status tlb_decoder_prefill_seq(tlb_decoder *d, int32_t seq, const int32_t *tokens, int32_t n, int32_t pos0, int32_t rope_pos0, int32_t rope_step, int32_t *next);
/* one token per sequence: tokens[b] at cache row pos[b] (rotation row rope_pos[b]; NULL: pos); next (may be NULL): [batch] */
tlb_status tlb_decoder_step_batch(tlb_decoder *d, const int32_t *tokens, const int32_t *pos, const int32_t *rope_pos, int32_t *next);
/* n greedy steps of the whole batch, tokens fed back on the device; tokens_out (may be NULL): [n][batch] */
tlb_status tlb_decoder_generate_batch(tlb_decoder *d, const int32_t *first_tokens, const int32_t *start_pos, int32_t n, int32_t *tokens_out);
tlb_status tlb_decoder_logits_batch(tlb_decoder *d, float *logits_out /* host, [batch, vocab] */);

/* tlb_sample_top_p on the logits of the last step or prompt, without bringing them to the host; temp <= 0 returns the
 * greedy token the step chose.  The caller feeds *token to the next tlb_decoder_step. */
tlb_status tlb_decoder_sample_top_p(tlb_decoder *d, float temp, float top_p, double u, int32_t *token);
/* n sampled steps with the token fed back on the device (temperature, top-k, top-p; one draw per step from
 * tlb_rng_uniform(seed, step)); temp <= 0 is tlb_decoder_generate.  Single-GPU sessions. */
tlb_status tlb_decoder_generate_sampled(tlb_decoder *d, int32_t first_token, int32_t start_pos, int32_t n, float temp, int32_t top_k, float top_p,
                                        uint64_t seed, int32_t *tokens_out);
tlb_status tlb_decoder_logits(tlb_decoder *d, float *logits_out /* host, vocab floats */);
tlb_status tlb_decoder_hidden(tlb_decoder *d, float *hidden_out /* host, d_model floats: residual stream before output_norm */);
/* algorithmic bytes one decode step reads at context length ctx (weights + KV), kernels per step */
tlb_status tlb_decoder_stats(const tlb_decoder *d, int32_t ctx, uint64_t *weight_bytes, uint64_t *kv_bytes, int32_t *kernels_per_step);
/* time `iters` launches of one named matvec of layer 0 ("qkv", "o", "gate_up", "down", "head") over a
 * rotating pool of `copies` weight copies; returns mean microseconds per launch and bytes per launch */
tlb_status tlb_decoder_time_kernel(tlb_decoder *d, const char *which, int copies, int iters, float *us_per_launch, uint64_t *bytes_per_launch);

#ifdef __cplusplus
}
#endif
#endif
