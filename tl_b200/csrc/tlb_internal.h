// Internal declarations shared by the translation units of libtlb200.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/tlb200.h"

namespace tlb {

constexpr int kMaxRank = 8;

// One device, one non-blocking stream (the reference uses the legacy NULL stream and a
// device-wide sync after every launch, crates/tl_cuda/src/stream.rs:17-22,63-73).
struct Context {
    int device = -1;
    cudaStream_t stream = nullptr;
    cudaMemPool_t pool = nullptr;
    int sm_count = 0;
    size_t smem_optin = 0;
    std::atomic<uint64_t> launches{0};
    std::atomic<int64_t> bytes_in_use{0};
    void *flush_buf = nullptr;
    size_t flush_bytes = 0;
    int *err_flag = nullptr;  // device word set by kernels whose bounded waits ran out
    // scratch of the streaming matvec (launches are ordered on `stream`, so one set serves all):
    // partial results per K-slice, and per-tile counts of finished slices (zero between launches)
    float *mv_part = nullptr;
    size_t mv_part_floats = 0;
    float *mv_part1 = nullptr;       // one activation row: slice scratch that rests at a sentinel bit pattern between launches
    size_t mv_part1_floats = 0;
    int *mv_cnt = nullptr;
    size_t mv_cnt_n = 0;
    bool capturing = false;
    uint64_t capture_launches = 0;
};
Context *ctx();          // nullptr + error set when no device
void run_deferred_destroys();   // decoder.cu: sessions whose destruction was asked for during a stream capture
bool ensure_init();

tlb_status fail(tlb_status code, const char *fmt, ...);
tlb_status cuda_fail(cudaError_t e, const char *what);
#define TLB_CUDA(expr)                                                   \
    do {                                                                 \
        cudaError_t _e = (expr);                                         \
        if (_e != cudaSuccess) return ::tlb::cuda_fail(_e, #expr);       \
    } while (0)
#define TLB_TRY(expr)                                \
    do {                                             \
        tlb_status _s = (expr);                      \
        if (_s != TLB_OK) return _s;                 \
    } while (0)

inline void count_launch(int n = 1) { Context *c = ctx(); if (c) c->launches += n; }

// Reference-counted device storage (Arc<CudaBuffer>, crates/tl_cuda/src/tensor.rs:39-99).
struct Storage {
    std::atomic<int> rc{1};
    void *ptr = nullptr;
    size_t bytes = 0;
};
Storage *storage_alloc(size_t bytes);   // nullptr on failure (error set)
void storage_release(Storage *s);

size_t dtype_size(tlb_dtype dt);

}  // namespace tlb

struct tlb_tensor {
    std::atomic<int> rc{1};
    tlb::Storage *st = nullptr;
    size_t offset = 0;  // bytes into st->ptr (always contiguous row-major)
    tlb_dtype dt = TLB_F32;
    int rank = 0;
    int64_t shape[tlb::kMaxRank] = {0};
    int64_t numel() const { int64_t n = 1; for (int i = 0; i < rank; i++) n *= shape[i]; return n; }
    void *data() const { return st ? (char *)st->ptr + offset : nullptr; }
    float *f32() const { return (float *)data(); }
};

namespace tlb {

tlb_status new_tensor(tlb_tensor **out, tlb_dtype dt, const int64_t *shape, int rank);
tlb_status new_view(tlb_tensor **out, const tlb_tensor *src, const int64_t *shape, int rank, size_t extra_off);

// ---- quantized weights ---------------------------------------------------------------
// Device layout: the [n, k] tensor is cut into units of 16 rows x 256 weights, stored
// [n/16][k/256][unit bytes]; unit bytes = 16 * 256 * bytes-per-weight (2304 / 4352 / 3360).
struct QFormat { int type; int unit_bytes; int raw_block; int raw_block_bytes; };
const QFormat *qformat(int ggml_type);

}  // namespace tlb

struct tlb_qtensor {
    std::atomic<int> rc{1};
    int type = 0;
    int64_t n = 0, k = 0;       // logical rows / cols
    int64_t n_tiles = 0, upt = 0; // 16-row tiles, units per tile (k/256)
    tlb::Storage *st = nullptr; // tiled device bytes; null for a dense tensor
    // Dense form, for what the tiled kernels do not take (F32, F16, Q4_1, Q5_0, Q5_1, Q8_1, and Q4_0 / Q8_0 rows that
    // are not a multiple of 256 long): the weight dequantised once to f32 [n, k], and its transpose [k, n] built by
    // the first matmul - the two caches QTensor keeps on the reference's fallback route
    // (crates/tl_runtime/src/system.rs:195-217,236-264).
    tlb_tensor *dense = nullptr;
    tlb_tensor *dense_t = nullptr;
    std::mutex mu;              // guards the lazy dense_t
    bool tiled() const { return st != nullptr; }
    uint8_t *dev() const { return (uint8_t *)st->ptr; }
    uint64_t nbytes() const { return tiled() ? (uint64_t)n_tiles * upt * tlb::qformat(type)->unit_bytes : (uint64_t)n * k * 4; }
};

namespace tlb {

// ---- kernel launchers (all on ctx()->stream) ------------------------------------------
// quant.cu
// qgemm_tc.cu: Y[m, n] = X[m, k] . W^T on the tensor cores, for more rows than the matvec's four (tcgen05 with the weights
// in tensor memory; up to 16 rows: a streaming kernel on mma.sync)
bool qgemm_supported(int ggml_type);
tlb_status launch_qgemm(const tlb_qtensor *w, const float *x, int64_t m, float *out);
// K-splits the tensor-core GEMM uses for m activation rows on `tiles` row tiles of `units` 256-wide K units each and
// n_all output columns (1 = none)
int qgemm_k_splits(int64_t m, int64_t tiles, int64_t units, int64_t n_all, int sm_count);
// activation row counts that qgemm_run_multi hands to its streaming kernel for few rows instead of the tensor-memory GEMM
bool qrows_rows(int64_t m);
// the same in steps, so that several weights can share one conversion of the activations:
// f32 rows (optionally silu(x) * x2, optionally RMS-normalised with norm_w) -> scaled f16 rows; then out = [resid +] act . W^T
struct GemmAct { Storage *xh = nullptr, *inv = nullptr, *sums = nullptr; int64_t m = 0, k = 0; };
tlb_status qgemm_prepare(GemmAct *a, const float *x, const float *x2, int64_t m, int64_t k, const float *norm_w, float eps);
tlb_status qgemm_run(const tlb_qtensor *w, const GemmAct &a, float *out, const float *resid);
// up to three weights of one type and K (q | k | v, gate | up) in one launch: outs[i] = act . ws[i]^T
tlb_status qgemm_run_multi(const tlb_qtensor *const *ws, int n_w, const GemmAct &a, float *const *outs, const float *resid);
void qgemm_release(GemmAct *a);
// sampling.cu: temperature / top-p sampling of n logits with the draw u in [0, 1); the token id as f32 into out[0]
tlb_status launch_sample_top_p(const float *logits, int64_t n, float temp, float top_p, float u, float *out, int top_k = 0);
size_t sample_workspace_bytes(int64_t n);
tlb_status launch_sample_into(const float *logits, int64_t n, float temp, float top_p, int top_k, float u, float *out, void *workspace,
                              int *state, int *tokens_out, int tokens_cap, unsigned long long *counter, unsigned long long seed);
// prefill.cu: the other kernels of prompt processing
tlb_status launch_embed_rows(const int *tokens, const float *table, float *x, int n_tokens, int dm);
tlb_status launch_rope_append(float *q, const float *k, const float *v, void *kcache, void *vcache, int kv_f16, const float *cos_t,
                              const float *sin_t, int n_tokens, int H, int KVH, int D, int max_seq, int pos0, int rope0, int rope_step);
bool prefill_attention_supported(int head_dim);
bool prefill_attention_tc_supported(int D, int kv_f16, int n_tokens);
tlb_status launch_prefill_attention_tc(const float *q, const void *kcache, const void *vcache, float *out, int n_tokens, int H, int KVH,
                                       int max_seq, int pos0, float scale);
tlb_status launch_prefill_attention(const float *q, const void *kcache, const void *vcache, int kv_f16, float *out, int n_tokens, int H,
                                    int KVH, int D, int max_seq, int pos0, float scale);
tlb_status launch_repack(int type, const uint8_t *raw, uint8_t *tiled, int64_t n, int64_t k);
tlb_status launch_dequant_tiled(int type, const uint8_t *tiled, float *out, int64_t n, int64_t k);
// raw GGUF blocks of any supported type -> f32, same expressions as the tiled dequantiser; nelem weights
size_t ggml_raw_nbytes(int type, int64_t nelem);   // 0: unknown type or nelem not a whole number of blocks
tlb_status launch_dequant_raw(int type, const uint8_t *raw, float *out, int64_t nelem);
tlb_status launch_interleave8(int type, const uint8_t *a, const uint8_t *b, uint8_t *dst, int64_t n, int64_t k);

// qmatvec.cu ---------------------------------------------------------------------------
// How the activation vector of a streaming matvec is produced inside the kernel.
enum Prologue { PRO_PLAIN = 0, PRO_ADD_NORM = 1, PRO_SILU_MUL = 2, PRO_ATTN_MERGE = 3 };
enum Finish { FIN_PLAIN = 0, FIN_RESID = 1, FIN_SILU = 2 };

// Tensor-parallel partial sums added inside the matvec launch that produces them (tp.cu owns the memory).  The warp
// that finishes a tile (16 output rows) stores its 16 partial sums into slot [buffer][own rank] of EVERY rank's region
// (peer stores over NVLink, own memory included), each as one 8-byte word {value, sequence number}.  It then reads the
// tile's words of all ranks from its OWN region, waiting (bounded) for those that do not carry the current sequence
// number yet - all ranks run the same schedule, so a tile's partial sums arrive from everywhere at about the same time
// - and adds the values in rank order, so every rank forms the same sum.  An aligned 8-byte store is indivisible: a
// word with the right number has its value, and neither a fence nor a separate flag is involved.  The exchange of
// early tiles overlaps the streaming of later ones.  The warp that finishes the launch's last tile advances the
// sequence number; buffers alternate with it (a rank can be one exchange ahead of a peer, never two).
constexpr int kTpMaxRanks = 8;
struct TpFuse {
    unsigned long long *peer_ll[kTpMaxRanks];   // rank p's words[0][own rank]
    const unsigned long long *mine_ll;          // own words[0][0]
    unsigned *seq;                              // device: sequence number of the exchange in progress
    int *done;                                  // device: tiles of the running launch finished so far
    int size, buf_stride, rank_stride;          // strides in words
};
bool tp_allreduce_is_kernel(int64_t n);   // tp_allreduce of n floats runs this library's peer-memory kernel (not NCCL)
bool tp_fuse_args(TpFuse *out);           // false: no peer memory attached (or switched off): use tp_allreduce
constexpr int kMaxSlices = 16;   // most K-slices a matvec may cut its launch into
struct MatvecJob {
    // up to 3 weight tensors sharing K and the same activation (q|k|v, gate|up)
    int n_w = 0;
    const uint8_t *w[3] = {nullptr, nullptr, nullptr};
    int64_t n_tiles[3] = {0, 0, 0};
    int64_t n_rows[3] = {0, 0, 0};                 // valid output rows (<= n_tiles*16)
    // Output of tensor i: [M, n_rows], every element written (no clearing needed).
    float *out[3] = {nullptr, nullptr, nullptr};
    int slices = 0;                  // K-slices the launch is cut into; 0: chosen by qmatvec_plan_slices()
    int type = 0;
    int64_t k = 0;
    int m = 1;
    // prologue inputs
    int prologue = PRO_PLAIN;
    const float *x = nullptr;        // PLAIN: x [M,K]; ADD_NORM: residual [K]; SILU_MUL: gate [M,K]
    const float *x2 = nullptr;       // ADD_NORM: delta added to x (may be null); SILU_MUL: up
    const float *norm_w = nullptr;   // ADD_NORM: weight [K]
    float eps = 0.f;
    float *x_out = nullptr;          // ADD_NORM: x + x2 written here by block 0 (may be null)
    const float *emb_table = nullptr; // ADD_NORM with token lookup: x = emb_table[*token * K ...]
    const int *token = nullptr;
    bool pdl = false;                // launch with programmatic stream serialization
    // ADD_NORM without the statistics pass: x already holds the whole residual and ssq_parts[0 .. n_parts)
    // are partial sums of its squares left by the launch that produced it (finish == FIN_RESID there)
    const float *ssq_parts = nullptr;
    int n_parts = 0;
    // PRO_ATTN_MERGE: the activation is the output of decode attention still split over the keys: per
    // (kv head, split, query head of the group) att_dim weighted sums, the split's score maximum and its sum
    // of exponentials, rows of att_dim + 4 floats; splits = ceil((*att_pos + 1) / att_keys).  The prologue
    // combines them (softmax over all keys) while it loads.
    const float *att_part = nullptr;
    const int *att_pos = nullptr;
    int att_max_splits = 0, att_rep = 0, att_dim = 0, att_keys = 0;
    // What the warp that completes a tile does with its 16 results (m == 1, one tensor, for the fused forms):
    //   FIN_PLAIN  out[row] = y
    //   FIN_RESID  out[row] = resid[row] + y, and ssq_out[tile] = sum of the squares of those 16 values
    //   FIN_SILU   rows 0..7 of a tile are gate, rows 8..15 up of the same 8 units (launch_interleave8):
    //              out[8 * tile + i] = silu(y[i]) * y[8 + i]
    int finish = 0;
    bool tp_reduce = false;          // y is this rank's partial sum: added over the tensor-parallel ranks inside the launch (FIN_PLAIN / FIN_RESID)
    const float *resid = nullptr;
    float *ssq_out = nullptr;
    bool dry_run = false;            // validate and plan only: tells whether the launch would be accepted
    bool last_of_chain = false;      // no matvec follows closely: take half an SM's shared memory instead of a third
};
tlb_status launch_qmatvec(const MatvecJob &job);
// K-slices the kernel wants for a launch of `tiles` 16-row tiles (all tensors) over inner dimension k,
// at most max_slices; a pure function of its arguments, so producer and consumer agree without talking.
int qmatvec_plan_slices(int type, int64_t k, int m, int64_t tiles, int max_slices);
size_t qmatvec_max_k(int m);   // largest K the single-pass kernel supports for m activation rows

// ops.cu
tlb_status launch_binary(int op, const float *a, const float *b, float *out, const int64_t *oshape,
                         const int64_t *astr, const int64_t *bstr, int rank, int64_t n);
tlb_status launch_unary(int op, const float *a, float *out, int64_t n, float s);
tlb_status launch_softmax(const float *a, float *out, int64_t outer, int64_t axis, int64_t inner);
tlb_status launch_matmul(const float *a, const float *b, float *out, int64_t batch, int64_t m,
                         int64_t k, int64_t n, bool b_batched);
tlb_status launch_copy_strided(const float *a, float *out, const int64_t *oshape, const int64_t *astr,
                               int rank, int64_t n, int64_t a_off);
tlb_status launch_rms_norm(const float *x, const float *res, const float *w, float eps, float *out,
                           int64_t rows, int64_t d);
tlb_status launch_rope_cpu(const float *x, const float *cos_t, const float *sin_t, int64_t tab_len,
                           float *out, int64_t nvec, int64_t d);
tlb_status launch_rope_half(const float *x, const float *cos_t, const float *sin_t, float *out,
                            int64_t tokens, int64_t heads, int64_t d);
tlb_status launch_embedding(const float *table, const float *idx, float *out, int64_t n, int64_t vocab,
                            int64_t dim, int *oob_flag);
tlb_status launch_argmax(const float *x, int64_t n, int tie_first, float *out_f32, int *out_i32);
tlb_status launch_causal_mask(float *out, int64_t size);
tlb_status launch_rep_penalty(float *logits, const float *tokens, int64_t rows, int64_t vocab, int64_t nt,
                              float penalty);
tlb_status launch_silu_mul(const float *g, const float *u, float *out, int64_t n);
tlb_status launch_f32_to_f16(const float *a, __half *out, int64_t n);

// tp.cu: tensor-parallel ranks of this process's communicator (1 / 0 before tlb_tp_init)
int tp_rank();
int tp_size();
int tp_live_sessions();        // decode sessions created with tp_size > 1 and not yet destroyed (decoder.cu)
tlb_status tp_allreduce(float *x, int64_t n);                                     // x := sum over ranks, in place, on ctx()->stream
tlb_status tp_allgather(const void *send, void *recv, size_t bytes_per_rank);     // recv[rank] := every rank's send

// attention.cu
constexpr int kAttnKeysPerSplit = 128;   // keys one CTA of the decode attention covers; splits = ceil((pos + 1) / this)
struct DecodeAttnJob {
    const float *qkv = nullptr;      // one sequence: [q (H*D) | k (KVH*D) | v (KVH*D)] raw projections of the new token
    // a batch of sequences (batch > 1; merged in the kernel, defer_merge must be false): dense rows q [batch, H*D],
    // k, v [batch, KVH*D]; caches cache_seq_bytes apart; pos / rope_pos entries state_stride ints apart; partial,
    // counters and out hold batch * KVH heads
    const float *q = nullptr, *k = nullptr, *v = nullptr;
    int batch = 1;
    size_t cache_seq_bytes = 0;
    int state_stride = 0;
    void *kcache, *vcache; // [KVH][max_seq][D] of this layer, f16 or f32
    int kv_f16;
    int H, KVH, D, max_seq;
    const int *pos;        // device: cache row of the new token (attend to rows 0..pos)
    const int *rope_pos;   // device: angle position
    const float *cos_t, *sin_t; // [max_seq, D] pair-duplicated tables (CPU convention)
    float scale;
    float *partial;        // scratch [KVH][splits][rep][D+4]
    bool defer_merge = false;   // leave the per-split results in `partial`; the o_proj launch merges them in its prologue
    int *counters;         // [KVH], zero on entry, reset by the kernel
    int splits;
    float *out;            // [H*D]
    bool pdl;
};
tlb_status launch_decode_attention(const DecodeAttnJob &j);
tlb_status launch_sdpa(const float *q, const float *k, const float *v, const float *mask, int mask_mode,
                       float *out, int64_t bh, int64_t sq, int64_t sk, int64_t d, int64_t mask_bh);

}  // namespace tlb
