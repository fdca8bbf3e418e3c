// Fused decode session: one token through a Llama-shaped decoder as a chain of 5 kernels per layer
// inside one CUDA graph.  The op order is that of the TL programs
// (examples/apps/llama3/chatbot_llama3.tl:66-125,220-236; examples/apps/tinyllama/chatbot.tl:50-113),
// which issue ~40 single-op FFI calls per layer per token, each followed by a device-wide sync
// (crates/tl_cuda/src/stream.rs:69-73).  Here:
//   K1  RMSNorm*w (prologue)  ->  q|k|v matvec        (layer 0: embedding lookup + sum of squares here too)
//   K2  RoPE(q, k) + KV append + attention split over the keys (per-split results are left as they are)
//   K3  softmax over the splits (prologue)  ->  o_proj matvec  ->  residual add, per-tile sums of squares (tile finishing)
//   K4  RMSNorm*w (prologue)  ->  gate|up matvec over interleaved rows  ->  SiLU(gate)*up (tile finishing)
//   K5  down matvec           ->  residual add, per-tile sums of squares (tile finishing)
//   ... output_norm (prologue) -> lm_head matvec, argmax + position advance.
// A residual add thus happens where the projection's rows are finished, and the RMSNorm that follows
// adds up d_model/16 partial sums instead of re-reading the row in every CTA.  Every buffer of the chain
// is written in full by its producer (no accumulation, no clearing).  The residual stream ping-pongs
// between two buffers so no kernel updates memory that another CTA of the same launch reads.  All
// kernels are launched with programmatic dependent launch: what a kernel can fetch without its
// predecessor's results (weights, norm weights, RoPE tables, older KV rows) is requested before it waits.
#include "tlb_internal.h"

#include <cstdlib>
#include <mutex>
#include <vector>

using namespace tlb;

static std::atomic<int> g_tp_sessions{0};
namespace tlb { int tp_live_sessions() { return g_tp_sessions.load(); } }

// Sessions given up while a stream capture is in progress: destroying one synchronises with the device, which would
// invalidate the capture, so it waits until the capture has ended.
static std::vector<tlb_decoder *> g_deferred_destroy;
static std::mutex g_deferred_mu;
namespace tlb {
void run_deferred_destroys()
{
    std::vector<tlb_decoder *> todo;
    {
        std::lock_guard<std::mutex> lk(g_deferred_mu);
        todo.swap(g_deferred_destroy);
    }
    for (tlb_decoder *d : todo) tlb_decoder_destroy(d);
}
}  // namespace tlb

struct LayerW {
    tlb_qtensor *q = nullptr, *k = nullptr, *v = nullptr, *o = nullptr, *gate = nullptr, *up = nullptr, *down = nullptr;
    tlb_tensor *attn_norm = nullptr, *ffn_norm = nullptr;
    tlb_qtensor *gu = nullptr;   // gate and up interleaved by groups of 8 rows (launch_interleave8): [2 * ffn, d_model]
};

struct tlb_decoder {
    tlb_decoder_cfg cfg;
    std::vector<LayerW> layers;
    tlb_tensor *emb = nullptr, *out_norm = nullptr;
    tlb_qtensor *head = nullptr;
    // device state
    float *xa = nullptr, *xb = nullptr;   // residual stream, ping-pong: xb enters a layer and leaves it, xa holds it after o_proj
    float *qkv = nullptr, *attn = nullptr, *logits = nullptr, *cos_t = nullptr, *sin_t = nullptr, *partial = nullptr;
    void *kcache = nullptr, *vcache = nullptr;
    int *state = nullptr;        // [0] token, [1] pos, [2] rope_pos, [3] output index
    int *counters = nullptr;     // attention merge counters [KVH], argmax counter at [KVH]
    int *tokens_out = nullptr;   // device ring of generated tokens
    int tokens_cap = 0;
    float *amax_v = nullptr;
    long long *amax_i = nullptr;
    int *h_state = nullptr;      // pinned host staging [4]
    float *hbuf = nullptr;       // silu(gate) * up, written by the gate|up launch
    float *ssq_o = nullptr, *ssq_d = nullptr;   // per-tile sums of squares of the residual after o_proj / down
    int max_splits = 1;
    cudaGraphExec_t graph = nullptr;
    uint64_t graph_kernels = 0;
    bool pdl = true;
    bool tp_pdl_ar = false;          // tensor-parallel chain with all-reduce launches of this library between the matvecs: they keep the dependent-launch chain
    bool dry = false;            // enqueue_step only validates the matvec launches
    std::vector<void *> allocs;
    size_t kv_layer_elems = 0;
    // tensor parallelism: this process holds shard tp_r of tp.  H, KVH, F, V below are the LOCAL sizes (heads, KV heads,
    // hidden units, vocabulary rows of this shard); they equal the model's sizes for tp == 1.
    int tp = 1, tp_r = 0;
    int H = 0, KVH = 0, F = 0, V = 0;
    // batch of sequences (cfg.batch > 1): caches [batch][layer][KV head][max_seq][D]; sequence 0 is also the sequence the
    // single-sequence entry points work on.  Rows of the b* buffers are sequences.
    int B = 1;
    size_t kv_seq_bytes = 0;      // bytes between the caches of consecutive sequences
    int *btok = nullptr, *bpos = nullptr, *brope = nullptr, *bidx = nullptr;   // per-sequence token / cache row / rotation row; output index
    float *bx = nullptr, *bx2 = nullptr, *bq = nullptr, *bk = nullptr, *bv = nullptr, *battn = nullptr, *bg = nullptr, *bu = nullptr, *bt = nullptr;
    float *blogits = nullptr, *blogits_all = nullptr, *bpartial = nullptr, *bpair = nullptr;
    int *bcounters = nullptr, *btokens_out = nullptr;
    cudaGraphExec_t bgraph = nullptr;
    uint64_t bgraph_kernels = 0;
    // sampled generation: the same chain with the sampler in place of the argmax, as a graph of its own
    struct { bool on = false; float temp = 0.f, top_p = 1.f; int top_k = 0; unsigned long long seed = 0; } samp;
    void *samp_ws = nullptr;
    unsigned long long *samp_counter = nullptr;
    cudaGraphExec_t sgraph = nullptr;
    uint64_t sgraph_kernels = 0;
    float *part = nullptr;        // tp > 1: this rank's partial o_proj / ffn_down result, summed over the ranks in place
    float *pair = nullptr;        // tp > 1: (best logit, its global index) of this shard, then of every shard [1 + tp][2]
    float *logits_all = nullptr;  // tp > 1: the gathered logits of all shards (tlb_decoder_logits)
};

namespace {

constexpr int kArgmaxBlocks = 148;

// argmax over the logits + advance of the decode state, in one launch.  Tie rule as tlb_argmax.
__global__ void argmax_advance_kernel(const float *__restrict__ x, int n, int tie_first, float *pv, long long *pi, int *counter,
                                      int *state, int *tokens_out, int tokens_cap, int use_pdl)
{
    if (use_pdl) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }
    __shared__ float sv[32];
    __shared__ long long si[32];
    __shared__ int last;
    float bv = 0.f;
    long long bi = -1;
    auto better = [&](float v, long long i, float cv, long long ci) {
        if (ci < 0) return true;
        if (v > cv) return true;
        if (v < cv) return false;
        return tie_first ? i < ci : i > ci;
    };
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const float v = __ldcg(x + i);
        if (better(v, i, bv, bi)) { bv = v; bi = i; }
    }
    for (int o = 16; o; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        long long oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi >= 0 && better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    if (lane == 0) { sv[w] = bv; si[w] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < (int)(blockDim.x >> 5); i++)
            if (si[i] >= 0 && better(sv[i], si[i], bv, bi)) { bv = sv[i]; bi = si[i]; }
        pv[blockIdx.x] = bv;
        pi[blockIdx.x] = bi;
        __threadfence();
        last = (atomicAdd(counter, 1) == (int)gridDim.x - 1);
    }
    __syncthreads();
    if (!last || threadIdx.x >= 32) return;
    // the last block's first warp folds the per-block winners: one round of loads, then shuffles
    __threadfence();
    bv = 0.f; bi = -1;
    for (int i = lane; i < (int)gridDim.x; i += 32) {
        float v = __ldcg(pv + i);
        long long ix = __ldcg(pi + i);
        if (ix >= 0 && better(v, ix, bv, bi)) { bv = v; bi = ix; }
    }
    for (int o = 16; o; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        long long oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi >= 0 && better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if (lane != 0) return;
    if (bi < 0) bi = 0;
    int idx = state[3];
    if (tokens_out && idx < tokens_cap) tokens_out[idx] = (int)bi;
    state[0] = (int)bi;
    state[1] += 1;
    state[2] += 1;
    state[3] = idx + 1;
    *counter = 0;
}

// Vocabulary-split head: each rank has the (best logit, global index) pair of its shard, gathered in rank order into
// pairs[tp][2]; one warp picks the winner under the tie rule and advances the decode state, identically on every rank.
__global__ void argmax_pick_kernel(const float *__restrict__ pairs, int tp, int tie_first, int *state, int *tokens_out, int tokens_cap)
{
    if (threadIdx.x != 0) return;
    float bv = pairs[0];
    long long bi = (long long)pairs[1];
    for (int r = 1; r < tp; r++) {
        const float v = pairs[2 * r];
        const long long i = (long long)pairs[2 * r + 1];
        if (v > bv || (v == bv && (tie_first ? i < bi : i > bi))) { bv = v; bi = i; }
    }
    const int idx = state[3];
    if (tokens_out && idx < tokens_cap) tokens_out[idx] = (int)bi;
    state[0] = (int)bi;
    state[1] += 1;
    state[2] += 1;
    state[3] = idx + 1;
}

// One block: the best logit of this shard and its global index (< 2^24, exact in f32) as two floats.
__global__ void __launch_bounds__(1024) argmax_pair_kernel(const float *__restrict__ x, int n, int tie_first, int offset, float *pair)
{
    __shared__ float sv[32];
    __shared__ int si[32];
    float bv = 0.f;
    int bi = -1;
    auto better = [&](float v, int i, float cv, int ci) { return ci < 0 || v > cv || (v == cv && (tie_first ? i < ci : i > ci)); };
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = __ldcg(x + i);
        if (better(v, i, bv, bi)) { bv = v; bi = i; }
    }
    for (int o = 16; o; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi >= 0 && better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); w++)
            if (si[w] >= 0 && better(sv[w], si[w], bv, bi)) { bv = sv[w]; bi = si[w]; }
        pair[0] = bv;
        pair[1] = (float)(max(bi, 0) + offset);
    }
}

template <typename T>
tlb_status dalloc(tlb_decoder *d, T **p, size_t count, bool zero = true)
{
    TLB_CUDA(cudaMalloc((void **)p, count * sizeof(T) ? count * sizeof(T) : 16));
    d->allocs.push_back(*p);
    if (zero) TLB_CUDA(cudaMemsetAsync(*p, 0, count * sizeof(T), ctx()->stream));
    return TLB_OK;
}

tlb_status get_q(tlb_map *m, const std::string &name, tlb_qtensor **q, int64_t n, int64_t k, int want_type)
{
    TLB_TRY(tlb_map_get_quantized(q, m, name.c_str()));
    if (!(*q)->tiled())
        return fail(TLB_ERR_TYPE, "tensor '%s' (GGML type %d, K = %lld) has no fused kernel: the decode session takes Q4_0 / Q8_0 / Q4_K / Q6_K with K a multiple of 256",
                    name.c_str(), (*q)->type, (long long)(*q)->k);
    if ((*q)->n != n || (*q)->k != k)
        return fail(TLB_ERR_SHAPE, "tensor '%s' is [%lld, %lld], expected [%lld, %lld]", name.c_str(), (long long)(*q)->n,
                    (long long)(*q)->k, (long long)n, (long long)k);
    if (want_type >= 0 && (*q)->type != want_type)
        return fail(TLB_ERR_TYPE, "tensor '%s' has GGML type %d; the tensors fused into one launch must share type %d", name.c_str(),
                    (*q)->type, want_type);
    return TLB_OK;
}

tlb_status get_f(tlb_map *m, const std::string &name, tlb_tensor **t, int64_t numel)
{
    TLB_TRY(tlb_map_get(t, m, name.c_str()));
    if ((*t)->numel() != numel) return fail(TLB_ERR_SHAPE, "tensor '%s' has %lld elements, expected %lld", name.c_str(), (long long)(*t)->numel(), (long long)numel);
    return TLB_OK;
}

void set_w(MatvecJob &j, int i, const tlb_qtensor *q, float *out)
{
    j.w[i] = q->dev();
    j.n_tiles[i] = q->n_tiles;
    j.n_rows[i] = q->n;
    j.out[i] = out;
}

// the kernel chain of one decode step (launched eagerly or into a capturing stream)
// output_norm + head + greedy token (with the advance of the decode state) on the residual in xb.
// ssq_parts: per-tile sums of squares of xb left by the launch that wrote it, or null (the head launch sums itself).
tlb_status enqueue_head(tlb_decoder *d, const float *ssq_parts, const float *x = nullptr, const float *x2 = nullptr, float *x_out = nullptr)
{
    const tlb_decoder_cfg &c = d->cfg;
    const int dm = c.d_model;
    {   // output_norm + head (tp > 1: this rank's rows of the vocabulary)
        MatvecJob j;
        j.n_w = 1;
        set_w(j, 0, d->head, d->logits);
        j.type = d->head->type; j.k = dm; j.m = 1;
        j.prologue = PRO_ADD_NORM; j.x = x ? x : d->xb; j.x2 = x2; j.x_out = x_out;
        j.ssq_parts = ssq_parts; j.n_parts = ssq_parts ? (dm + 15) / 16 : 0;
        j.norm_w = d->out_norm->f32(); j.eps = c.eps;
        j.last_of_chain = true;
        j.pdl = d->pdl && (!x2 || d->tp_pdl_ar);     // behind an NCCL collective: a plain stream dependency
        j.dry_run = d->dry;
        TLB_TRY(launch_qmatvec(j));
    }
    if (d->dry) return TLB_OK;
    if (d->samp.on) {
        // temperature / top-k / top-p sampling on the device, the random number drawn from (seed, step counter); the token
        // and the advance of the positions go where the argmax would have put them
        return launch_sample_into(d->logits, c.vocab, d->samp.temp, d->samp.top_p, d->samp.top_k, 0.f, nullptr, d->samp_ws, d->state, d->tokens_out,
                                  d->tokens_cap, d->samp_counter, d->samp.seed);
    }
    if (d->tp > 1) {
        argmax_pair_kernel<<<1, 1024, 0, ctx()->stream>>>(d->logits, d->V, (int)(c.tie_rule == TLB_TIE_FIRST), d->tp_r * d->V, d->pair);
        TLB_CUDA(cudaGetLastError());
        TLB_TRY(tp_allgather(d->pair, d->pair + 2, 2 * sizeof(float)));
        argmax_pick_kernel<<<1, 32, 0, ctx()->stream>>>(d->pair + 2, d->tp, (int)(c.tie_rule == TLB_TIE_FIRST), d->state, d->tokens_out, d->tokens_cap);
        TLB_CUDA(cudaGetLastError());
        count_launch(2);
        return TLB_OK;
    }
    {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(kArgmaxBlocks);
        cfg.blockDim = dim3(256);
        cfg.stream = ctx()->stream;
        cudaLaunchAttribute at[1];
        if (d->pdl) {
            at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            at[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = at;
            cfg.numAttrs = 1;
        }
        static bool carveout_set = false;
        if (!carveout_set) {
            TLB_CUDA(cudaFuncSetAttribute(argmax_advance_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
            carveout_set = true;
        }
        TLB_CUDA(cudaLaunchKernelEx(&cfg, argmax_advance_kernel, (const float *)d->logits, (int)c.vocab, (int)(c.tie_rule == TLB_TIE_FIRST), d->amax_v, d->amax_i, d->counters + c.n_kv_heads,
                                    d->state, d->tokens_out, d->tokens_cap, (int)d->pdl));
        count_launch();
    }
    return TLB_OK;
}

// The chain of one decode step on one shard of a tensor-parallel group (Megatron split): q | k | v and gate | up hold
// this rank's heads / hidden units, o_proj and ffn_down this rank's slice of their inner dimension, so their results
// are partial sums: they are written plain, summed over the ranks (tp_allreduce, in place), and the launch that
// consumes them adds the sum to the residual while it normalises (the PRO_ADD_NORM prologue with a delta; CTA 0 stores
// the new residual).  Two collectives per layer and nothing else crosses the ranks until the (maximum, index) pairs of
// the vocabulary-split head.  Launches behind a collective take a plain stream dependency.
tlb_status enqueue_step_tp(tlb_decoder *d)
{
    const tlb_decoder_cfg &c = d->cfg;
    const int dm = c.d_model, qd = d->H * c.head_dim, kvd = d->KVH * c.head_dim, F = d->F;
    d->tp_pdl_ar = tp_allreduce_is_kernel(dm);   // this library's all-reduce launch takes part in the dependent-launch chain
    for (int l = 0; l < c.n_layers; l++) {
        const LayerW &w = d->layers[l];
        {   // K1: residual (+ the summed ffn_down of the layer before) -> RMSNorm -> q | k | v of this rank's heads
            if (w.k->type != w.q->type || w.v->type != w.q->type) return fail(TLB_ERR_TYPE, "tensor-parallel sessions take q, k, v of one GGML type per layer");
            MatvecJob j;
            j.n_w = 3;
            set_w(j, 0, w.q, d->qkv); set_w(j, 1, w.k, d->qkv + qd); set_w(j, 2, w.v, d->qkv + qd + kvd);
            j.type = w.q->type; j.k = dm; j.m = 1;
            j.prologue = PRO_ADD_NORM; j.norm_w = w.attn_norm->f32(); j.eps = c.eps;
            if (l == 0) { j.emb_table = d->emb->f32(); j.token = d->state; j.x_out = d->xb; j.pdl = d->pdl; }
            else { j.x = d->xa; j.x2 = d->part; j.x_out = d->xb; j.pdl = d->pdl && d->tp_pdl_ar; }
            j.dry_run = d->dry;
            TLB_TRY(launch_qmatvec(j));
        }
        {   // K2: attention over this rank's KV heads
            DecodeAttnJob a;
            a.qkv = d->qkv;
            a.kcache = (char *)d->kcache + (size_t)l * d->kv_layer_elems * (c.kv_f16 ? 2 : 4);
            a.vcache = (char *)d->vcache + (size_t)l * d->kv_layer_elems * (c.kv_f16 ? 2 : 4);
            a.kv_f16 = c.kv_f16; a.H = d->H; a.KVH = d->KVH; a.D = c.head_dim; a.max_seq = c.max_seq;
            a.pos = d->state + 1; a.rope_pos = d->state + 2; a.cos_t = d->cos_t; a.sin_t = d->sin_t; a.scale = c.attn_scale;
            a.partial = d->partial; a.counters = d->counters; a.splits = d->max_splits; a.out = d->attn; a.pdl = d->pdl;
            a.defer_merge = true;
            if (!d->dry) TLB_TRY(launch_decode_attention(a));
        }
        {   // K3: this rank's slice of o_proj -> partial sum
            MatvecJob j;
            j.n_w = 1;
            set_w(j, 0, w.o, d->part);
            j.type = w.o->type; j.k = qd; j.m = 1;
            j.prologue = PRO_ATTN_MERGE;
            j.att_part = d->partial; j.att_pos = d->state + 1; j.att_max_splits = d->max_splits;
            j.att_rep = d->H / d->KVH; j.att_dim = c.head_dim; j.att_keys = kAttnKeysPerSplit;
            j.pdl = d->pdl;
            j.dry_run = d->dry;
            TLB_TRY(launch_qmatvec(j));
        }
        if (!d->dry) TLB_TRY(tp_allreduce(d->part, dm));
        {   // K4: xa = xb + sum; RMSNorm; gate | up of this rank's hidden units; SiLU(gate) * up
            MatvecJob j;
            j.n_w = 1;
            set_w(j, 0, w.gu, d->hbuf);
            j.type = w.gu->type; j.k = dm; j.m = 1;
            j.prologue = PRO_ADD_NORM; j.x = d->xb; j.x2 = d->part; j.x_out = d->xa;
            j.norm_w = w.ffn_norm->f32(); j.eps = c.eps;
            j.finish = FIN_SILU;
            j.pdl = d->pdl && d->tp_pdl_ar;
            j.dry_run = d->dry;
            TLB_TRY(launch_qmatvec(j));
        }
        {   // K5: this rank's slice of ffn_down -> partial sum
            MatvecJob j;
            j.n_w = 1;
            set_w(j, 0, w.down, d->part);
            j.type = w.down->type; j.k = F; j.m = 1;
            j.prologue = PRO_PLAIN; j.x = d->hbuf;
            j.pdl = d->pdl;
            j.dry_run = d->dry;
            TLB_TRY(launch_qmatvec(j));
        }
        if (!d->dry) TLB_TRY(tp_allreduce(d->part, dm));
    }
    return enqueue_head(d, nullptr, d->xa, d->part, d->xb);   // xb = xa + sum: the residual before output_norm
}

tlb_status enqueue_step(tlb_decoder *d)
{
    // A tensor-parallel shard with peer memory attached runs the single-GPU chain on its own heads / hidden units: o_proj
    // and ffn_down add their partial sums over the ranks inside the launch, tile by tile (MatvecJob::tp_reduce), so what
    // they leave - the residual and the per-tile sums of its squares - is what the next launch expects anyway.  Without
    // peer memory the partial sums go through collective launches between the matvecs (enqueue_step_tp).
    TpFuse probe;
    const bool tpr = d->tp > 1 && tp_fuse_args(&probe) && d->cfg.d_model <= probe.rank_stride;
    if (d->tp > 1 && !tpr) return enqueue_step_tp(d);
    const tlb_decoder_cfg &c = d->cfg;
    const int dm = c.d_model, qd = d->H * c.head_dim, kvd = d->KVH * c.head_dim, F = d->F;
    const int L = c.n_layers;
    for (int l = 0; l < L; l++) {
        const LayerW &w = d->layers[l];
        {   // K1: q | k | v in one launch when they share a type, else one launch per type
            const tlb_qtensor *ws[3] = {w.q, w.k, w.v};
            float *outs[3] = {d->qkv, d->qkv + qd, d->qkv + qd + kvd};
            bool done[3] = {false, false, false};
            bool first = true;
            for (int a = 0; a < 3; a++) {
                if (done[a]) continue;
                MatvecJob j;
                j.n_w = 0;
                for (int b = a; b < 3; b++)
                    if (!done[b] && ws[b]->type == ws[a]->type) { set_w(j, j.n_w++, ws[b], outs[b]); done[b] = true; }
                j.type = ws[a]->type; j.k = dm; j.m = 1;
                j.prologue = PRO_ADD_NORM;
                j.norm_w = w.attn_norm->f32(); j.eps = c.eps;
                // the residual lives in xb here: the embedding row for layer 0 (the first launch stores it), else what
                // the last down launch left
                if (l == 0 && first) { j.emb_table = d->emb->f32(); j.token = d->state; j.x_out = d->xb; }
                else if (l == 0) { j.x = d->xb; }
                else { j.x = d->xb; j.ssq_parts = d->ssq_d; j.n_parts = (dm + 15) / 16; }
                j.pdl = d->pdl;
                j.dry_run = d->dry;
                TLB_TRY(launch_qmatvec(j));
                first = false;
            }
        }
        {   // K2
            DecodeAttnJob a;
            a.qkv = d->qkv;
            a.kcache = (char *)d->kcache + (size_t)l * d->kv_layer_elems * (c.kv_f16 ? 2 : 4);
            a.vcache = (char *)d->vcache + (size_t)l * d->kv_layer_elems * (c.kv_f16 ? 2 : 4);
            a.kv_f16 = c.kv_f16; a.H = d->H; a.KVH = d->KVH; a.D = c.head_dim; a.max_seq = c.max_seq;
            a.pos = d->state + 1; a.rope_pos = d->state + 2; a.cos_t = d->cos_t; a.sin_t = d->sin_t; a.scale = c.attn_scale;
            a.partial = d->partial; a.counters = d->counters; a.splits = d->max_splits; a.out = d->attn; a.pdl = d->pdl;
            a.defer_merge = true;
            if (!d->dry) TLB_TRY(launch_decode_attention(a));
        }
        {   // K3
            MatvecJob j;
            j.n_w = 1;
            set_w(j, 0, w.o, d->xa);
            j.type = w.o->type; j.k = qd; j.m = 1;
            // the attention launch leaves its per-split results; they are combined here, as the activation is loaded
            j.prologue = PRO_ATTN_MERGE;
            j.att_part = d->partial; j.att_pos = d->state + 1; j.att_max_splits = d->max_splits;
            j.att_rep = c.n_heads / c.n_kv_heads; j.att_dim = c.head_dim; j.att_keys = kAttnKeysPerSplit;
            j.finish = FIN_RESID; j.resid = d->xb; j.ssq_out = d->ssq_o;   // xa = xb + o_proj(attn)
            j.tp_reduce = tpr;
            j.pdl = d->pdl;
            j.dry_run = d->dry;
            TLB_TRY(launch_qmatvec(j));
        }
        {   // K4
            MatvecJob j;
            j.n_w = 1;
            set_w(j, 0, w.gu, d->hbuf);
            j.type = w.gu->type; j.k = dm; j.m = 1;
            j.prologue = PRO_ADD_NORM; j.x = d->xa; j.ssq_parts = d->ssq_o; j.n_parts = (dm + 15) / 16;
            j.norm_w = w.ffn_norm->f32(); j.eps = c.eps;
            j.finish = FIN_SILU;
            j.pdl = d->pdl;
            j.dry_run = d->dry;
            TLB_TRY(launch_qmatvec(j));
        }
        {   // K5
            MatvecJob j;
            j.n_w = 1;
            set_w(j, 0, w.down, d->xb);
            j.type = w.down->type; j.k = F; j.m = 1;
            j.prologue = PRO_PLAIN; j.x = d->hbuf;
            j.finish = FIN_RESID; j.resid = d->xa; j.ssq_out = d->ssq_d;   // xb = xa + down(h)
            j.tp_reduce = tpr;
            j.pdl = d->pdl;
            j.dry_run = d->dry;
            TLB_TRY(launch_qmatvec(j));
        }
    }
    TLB_TRY(enqueue_head(d, d->ssq_d));
    return TLB_OK;
}


// ---- a batch of sequences, one new token each ------------------------------------------------------------------
// The reference's matmul entry takes any number of rows (crates/tl_runtime/src/system.rs:180-222) and the TL program's
// projections are batch-agnostic (examples/apps/llama3/chatbot_llama3.tl:220-236): here the B new tokens go through the
// linear layers as B rows of ONE pass over the weights (tensor-core GEMM with on-the-fly dequantisation; the weight
// stream, the cost of decoding, is shared by the batch), and through attention as B independent sequences, each with
// its own cache, position and split-K reduction (one grid plane per sequence).

// out[i] = a[i] + b[i]
__global__ void add_rows_kernel(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ out, int64_t n4)
{
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
        const float4 x = reinterpret_cast<const float4 *>(a)[i], y = reinterpret_cast<const float4 *>(b)[i];
        reinterpret_cast<float4 *>(out)[i] = make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w);
    }
}

// Block b: argmax of logits row b (n entries; tie rule as tlb_argmax).  pairs == null: the token goes straight to the
// sequence's state (rows [row0, row0 + gridDim.x)).  Otherwise (vocabulary split over ranks) the (value, global index)
// pair of this shard goes to pairs[b] for the exchange.
__global__ void __launch_bounds__(1024) argmax_rows_kernel(const float *__restrict__ logits, int n, int tie_first, int offset, float *pairs,
                                                            int *tok, int *pos, int *rope, const int *idx, int *tokens_out, int B, int cap, int row0)
{
    __shared__ float sv[32];
    __shared__ int si[32];
    const float *x = logits + (size_t)blockIdx.x * n;
    float bv = 0.f;
    int bi = -1;
    auto better = [&](float v, int i, float cv, int ci) { return ci < 0 || v > cv || (v == cv && (tie_first ? i < ci : i > ci)); };
    if ((n & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        // four 16-byte loads in flight per thread; a thread meets its indices in increasing order
        const float4 *x4 = reinterpret_cast<const float4 *>(x);
        const int n4 = n >> 2;
        for (int i = threadIdx.x; i < n4; i += 4 * blockDim.x) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int j = i + u * blockDim.x;
                v[u] = j < n4 ? __ldcg(x4 + j) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int j = i + u * blockDim.x;
                if (j >= n4) break;
                const float e[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
                for (int k = 0; k < 4; k++)
                    if (better(e[k], 4 * j + k, bv, bi)) { bv = e[k]; bi = 4 * j + k; }
            }
        }
    } else {
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            const float v = __ldcg(x + i);
            if (better(v, i, bv, bi)) { bv = v; bi = i; }
        }
    }
    for (int o = 16; o; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi >= 0 && better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x != 0) return;
    for (int w = 1; w < (int)(blockDim.x >> 5); w++)
        if (si[w] >= 0 && better(sv[w], si[w], bv, bi)) { bv = sv[w]; bi = si[w]; }
    bi = max(bi, 0) + offset;
    if (pairs) { pairs[2 * blockIdx.x] = bv; pairs[2 * blockIdx.x + 1] = (float)bi; return; }
    const int b = row0 + blockIdx.x;
    if (tokens_out && *idx < cap) tokens_out[(size_t)*idx * B + b] = bi;
    tok[b] = bi; pos[b] += 1; rope[b] += 1;
}

// After the exchange: pairs[rank][row][2]; thread `row` picks the winner over the ranks and updates the state.
__global__ void argmax_rows_pick_kernel(const float *__restrict__ pairs, int tp, int rows, int tie_first, int *tok, int *pos, int *rope,
                                        const int *idx, int *tokens_out, int B, int cap, int row0)
{
    const int r = threadIdx.x;
    if (r >= rows) return;
    float bv = pairs[2 * r];
    int bi = (int)pairs[2 * r + 1];
    for (int k = 1; k < tp; k++) {
        const float v = pairs[((size_t)k * rows + r) * 2];
        const int i = (int)pairs[((size_t)k * rows + r) * 2 + 1];
        if (v > bv || (v == bv && (tie_first ? i < bi : i > bi))) { bv = v; bi = i; }
    }
    const int b = row0 + r;
    if (tokens_out && *idx < cap) tokens_out[(size_t)*idx * B + b] = bi;
    tok[b] = bi; pos[b] += 1; rope[b] += 1;
}

__global__ void bump_index_kernel(int *idx) { *idx += 1; }

tlb_status add_rows(const float *a, const float *b, float *out, int64_t n)
{
    add_rows_kernel<<<(unsigned)std::min<int64_t>(1184, (n / 4 + 255) / 256), 256, 0, ctx()->stream>>>(a, b, out, n / 4);
    TLB_CUDA(cudaGetLastError());
    count_launch();
    return TLB_OK;
}

// out = [resid +] act . W^T; with tensor parallelism W is this rank's slice of the inner dimension, the result a partial
// sum: summed over the ranks first, the residual added afterwards.
tlb_status row_parallel(tlb_decoder *d, const tlb_qtensor *w, const GemmAct &a, float *out, const float *resid, float *scratch, int64_t rows)
{
    if (d->tp <= 1) return qgemm_run(w, a, out, resid);
    TLB_TRY(qgemm_run(w, a, scratch, nullptr));
    TLB_TRY(tp_allreduce(scratch, rows * d->cfg.d_model));
    return add_rows(resid, scratch, out, rows * d->cfg.d_model);
}

// output_norm + head + greedy tokens for `rows` residual rows x (sequences row0 ..): logits to blogits[row0 ..]
tlb_status batch_head(tlb_decoder *d, const float *x, int rows, int row0)
{
    const tlb_decoder_cfg &c = d->cfg;
    const int tie_first = c.tie_rule == TLB_TIE_FIRST;
    GemmAct a;
    TLB_TRY(qgemm_prepare(&a, x, nullptr, rows, c.d_model, d->out_norm->f32(), c.eps));
    float *lg = d->blogits + (size_t)row0 * d->V;
    tlb_status st = qgemm_run(d->head, a, lg, nullptr);
    qgemm_release(&a);
    TLB_TRY(st);
    if (d->tp > 1) {
        argmax_rows_kernel<<<rows, 1024, 0, ctx()->stream>>>(lg, d->V, tie_first, d->tp_r * d->V, d->bpair, nullptr, nullptr, nullptr, nullptr, nullptr, d->B, 0, row0);
        TLB_CUDA(cudaGetLastError());
        TLB_TRY(tp_allgather(d->bpair, d->bpair + 2 * d->B, (size_t)rows * 2 * sizeof(float)));
        argmax_rows_pick_kernel<<<1, 32, 0, ctx()->stream>>>(d->bpair + 2 * d->B, d->tp, rows, tie_first, d->btok, d->bpos, d->brope, d->bidx, d->btokens_out, d->B, d->tokens_cap, row0);
        TLB_CUDA(cudaGetLastError());
        count_launch(2);
    } else {
        argmax_rows_kernel<<<rows, 1024, 0, ctx()->stream>>>(lg, d->V, tie_first, 0, nullptr, d->btok, d->bpos, d->brope, d->bidx, d->btokens_out, d->B, d->tokens_cap, row0);
        TLB_CUDA(cudaGetLastError());
        count_launch();
    }
    return TLB_OK;
}

bool prefill_batched_ok(const tlb_decoder *d);

tlb_status enqueue_step_batch(tlb_decoder *d)
{
    const tlb_decoder_cfg &c = d->cfg;
    const int B = d->B, dm = c.d_model, qd = d->H * c.head_dim, kvd = d->KVH * c.head_dim, F = d->F;
    const size_t esz = c.kv_f16 ? 2 : 4;
    TLB_TRY(launch_embed_rows(d->btok, d->emb->f32(), d->bx, B, dm));
    float *x = d->bx, *x2 = d->bx2;
    for (int l = 0; l < c.n_layers; l++) {
        const LayerW &w = d->layers[l];
        GemmAct a;
        tlb_status st = TLB_OK;
        TLB_TRY(qgemm_prepare(&a, x, nullptr, B, dm, w.attn_norm->f32(), c.eps));
        {
            const tlb_qtensor *ws3[3] = {w.q, w.k, w.v};
            float *outs3[3] = {d->bq, d->bk, d->bv};
            bool done3[3] = {false, false, false};
            for (int i = 0; i < 3 && st == TLB_OK; i++) {
                if (done3[i]) continue;
                const tlb_qtensor *gw[3];
                float *go[3];
                int gn = 0;
                for (int b = i; b < 3; b++)
                    if (!done3[b] && ws3[b]->type == ws3[i]->type) { gw[gn] = ws3[b]; go[gn++] = outs3[b]; done3[b] = true; }
                st = qgemm_run_multi(gw, gn, a, go, nullptr);
            }
        }
        qgemm_release(&a);
        TLB_TRY(st);
        {   // RoPE, cache append and split-K attention of every sequence over its own cache
            DecodeAttnJob j;
            j.q = d->bq; j.k = d->bk; j.v = d->bv; j.batch = B;
            j.cache_seq_bytes = d->kv_seq_bytes; j.state_stride = 1;
            j.kcache = (char *)d->kcache + (size_t)l * d->kv_layer_elems * esz;
            j.vcache = (char *)d->vcache + (size_t)l * d->kv_layer_elems * esz;
            j.kv_f16 = c.kv_f16; j.H = d->H; j.KVH = d->KVH; j.D = c.head_dim; j.max_seq = c.max_seq;
            j.pos = d->bpos; j.rope_pos = d->brope; j.cos_t = d->cos_t; j.sin_t = d->sin_t; j.scale = c.attn_scale;
            j.partial = d->bpartial; j.counters = d->bcounters; j.splits = d->max_splits; j.out = d->battn; j.pdl = false;
            j.defer_merge = false;
            TLB_TRY(launch_decode_attention(j));
        }
        TLB_TRY(qgemm_prepare(&a, d->battn, nullptr, B, qd, nullptr, 0.f));
        st = row_parallel(d, w.o, a, x2, x, d->bt, B);        // x2 = x + o_proj(attention)
        qgemm_release(&a);
        TLB_TRY(st);
        TLB_TRY(qgemm_prepare(&a, x2, nullptr, B, dm, w.ffn_norm->f32(), c.eps));
        {
            const tlb_qtensor *ws2[2] = {w.gate, w.up};
            float *outs2[2] = {d->bg, d->bu};
            st = qgemm_run_multi(ws2, 2, a, outs2, nullptr);
        }
        qgemm_release(&a);
        TLB_TRY(st);
        TLB_TRY(qgemm_prepare(&a, d->bg, d->bu, B, F, nullptr, 0.f));   // silu(gate) * up inside the f16 conversion
        st = row_parallel(d, w.down, a, x, x2, d->bt, B);     // x = x2 + down(silu(gate) * up)
        qgemm_release(&a);
        TLB_TRY(st);
    }
    TLB_TRY(batch_head(d, x, B, 0));
    bump_index_kernel<<<1, 1, 0, ctx()->stream>>>(d->bidx);
    TLB_CUDA(cudaGetLastError());
    count_launch();
    return TLB_OK;
}

tlb_status ensure_batch_graph(tlb_decoder *d)
{
    if (d->bgraph) return TLB_OK;
    Context *cx = ctx();
    uint64_t before = cx->launches.load();
    TLB_CUDA(cudaStreamBeginCapture(cx->stream, cudaStreamCaptureModeThreadLocal));
    tlb_status st = enqueue_step_batch(d);
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamEndCapture(cx->stream, &g);
    d->bgraph_kernels = cx->launches.load() - before;
    cx->launches = before;
    if (st != TLB_OK) { if (g) cudaGraphDestroy(g); return st; }
    if (e != cudaSuccess) return cuda_fail(e, "cudaStreamEndCapture");
    e = cudaGraphInstantiate(&d->bgraph, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGraphInstantiate");
    return TLB_OK;
}

tlb_status ensure_graph(tlb_decoder *d)
{
    if (d->graph) return TLB_OK;
    Context *cx = ctx();
    uint64_t before = cx->launches.load();
    TLB_CUDA(cudaStreamBeginCapture(cx->stream, cudaStreamCaptureModeThreadLocal));
    tlb_status st = enqueue_step(d);
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamEndCapture(cx->stream, &g);
    d->graph_kernels = cx->launches.load() - before;
    cx->launches = before;
    if (st != TLB_OK) { if (g) cudaGraphDestroy(g); return st; }
    if (e != cudaSuccess) return cuda_fail(e, "cudaStreamEndCapture");
    e = cudaGraphInstantiate(&d->graph, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGraphInstantiate");
    return TLB_OK;
}

tlb_status set_state(tlb_decoder *d, int token, int pos, int rope_pos, int out_idx)
{
    // pageable source: the runtime stages the 16 bytes before returning, so the next call may reuse the stack
    int hs[4] = {token, pos, rope_pos, out_idx};
    TLB_CUDA(cudaMemcpyAsync(d->state, hs, sizeof hs, cudaMemcpyHostToDevice, ctx()->stream));
    return TLB_OK;
}

}  // namespace

extern "C" {


tlb_status tlb_decoder_destroy(tlb_decoder *d)
{
    if (!d) return TLB_OK;
    if (ctx() && ctx()->capturing) {
        std::lock_guard<std::mutex> lk(g_deferred_mu);
        g_deferred_destroy.push_back(d);
        return TLB_OK;
    }
    if (ctx()) cudaStreamSynchronize(ctx()->stream);
    if (d->graph) cudaGraphExecDestroy(d->graph);
    if (d->bgraph) cudaGraphExecDestroy(d->bgraph);
    if (d->sgraph) cudaGraphExecDestroy(d->sgraph);
    for (LayerW &w : d->layers) {
        tlb_qtensor_release(w.q); tlb_qtensor_release(w.k); tlb_qtensor_release(w.v); tlb_qtensor_release(w.o);
        tlb_qtensor_release(w.gate); tlb_qtensor_release(w.up); tlb_qtensor_release(w.down); tlb_qtensor_release(w.gu);
        tlb_tensor_release(w.attn_norm); tlb_tensor_release(w.ffn_norm);
    }
    tlb_tensor_release(d->emb); tlb_tensor_release(d->out_norm); tlb_qtensor_release(d->head);
    for (void *p : d->allocs) cudaFree(p);
    if (d->h_state) cudaFreeHost(d->h_state);
    if (d->tp > 1) g_tp_sessions--;
    delete d;
    return TLB_OK;
}

tlb_status tlb_decoder_create(tlb_decoder **out, const tlb_decoder_cfg *cfg, tlb_map *m)
{
    if (!out) return fail(TLB_ERR_NULL, "null out");
    *out = nullptr;
    if (!cfg || !m) return fail(TLB_ERR_NULL, "null argument");
    if (!ensure_init()) return TLB_ERR_DEVICE;
    const tlb_decoder_cfg &c = *cfg;
    if (c.n_layers < 1 || c.d_model < 1 || c.n_heads < 1 || c.n_kv_heads < 1 || c.head_dim < 1 || c.ffn < 1 || c.vocab < 1 || c.max_seq < 1)
        return fail(TLB_ERR_ARG, "decoder config has a non-positive size");
    if (c.n_heads % c.n_kv_heads) return fail(TLB_ERR_SHAPE, "n_heads must be a multiple of n_kv_heads");
    const int tp = c.tp_size > 1 ? c.tp_size : 1, tp_r = tp > 1 ? c.tp_rank : 0;
    if (tp > 1) {
        // one process per GPU: the weights in the map are this rank's shards (tlb_gguf_load_tp / tlb_map_add_tp) and the
        // communicator of tlb_tp_init carries the two sums per layer
        if (tp != tp_size() || tp_r != tp_rank())
            return fail(TLB_ERR_ARG, "decoder config names shard %d of %d, the communicator of tlb_tp_init is rank %d of %d", c.tp_rank, c.tp_size, tp_rank(), tp_size());
        if (c.n_heads % tp || c.n_kv_heads % tp || c.ffn % tp || c.vocab % tp)
            return fail(TLB_ERR_SHAPE, "heads (%d / %d), ffn %d and vocab %d must divide over %d ranks", c.n_heads, c.n_kv_heads, c.ffn, c.vocab, tp);
        if ((c.ffn / tp) % 256 || ((c.n_heads / tp) * c.head_dim) % 256)
            return fail(TLB_ERR_SHAPE, "a rank's slice of ffn (%d) and of the attention width (%d) must be multiples of 256", c.ffn / tp, (c.n_heads / tp) * c.head_dim);
        if ((int64_t)c.vocab >= (1 << 24)) return fail(TLB_ERR_SHAPE, "vocabulary too large for the index exchange");
    }
    if (c.batch < 0 || c.batch > 64) return fail(TLB_ERR_ARG, "batch %d: a session holds 1 to 64 sequences", c.batch);
    tlb_decoder *d = new tlb_decoder();
    d->cfg = c;
    d->B = c.batch > 1 ? c.batch : 1;
    d->tp = tp; d->tp_r = tp_r;
    if (tp > 1) g_tp_sessions++;
    d->H = c.n_heads / tp; d->KVH = c.n_kv_heads / tp; d->F = c.ffn / tp; d->V = c.vocab / tp;
    // local sizes: the shapes this rank's tensors must have
    const int64_t dm = c.d_model, qd = (int64_t)d->H * c.head_dim, kvd = (int64_t)d->KVH * c.head_dim, F = d->F;
    tlb_status st = TLB_OK;
#define TRY_D(expr) do { st = (expr); if (st != TLB_OK) { tlb_decoder_destroy(d); return st; } } while (0)
    d->layers.resize(c.n_layers);
    for (int l = 0; l < c.n_layers; l++) {
        std::string p = "blk." + std::to_string(l) + ".";
        LayerW &w = d->layers[l];
        TRY_D(get_q(m, p + "attn_q.weight", &w.q, qd, dm, -1));
        TRY_D(get_q(m, p + "attn_k.weight", &w.k, kvd, dm, -1));
        TRY_D(get_q(m, p + "attn_v.weight", &w.v, kvd, dm, -1));
        TRY_D(get_q(m, p + "attn_output.weight", &w.o, dm, qd, -1));
        TRY_D(get_q(m, p + "ffn_gate.weight", &w.gate, F, dm, -1));
        TRY_D(get_q(m, p + "ffn_up.weight", &w.up, F, dm, w.gate->type));
        TRY_D(get_q(m, p + "ffn_down.weight", &w.down, dm, F, -1));
        TRY_D(get_f(m, p + "attn_norm.weight", &w.attn_norm, dm));
        TRY_D(get_f(m, p + "ffn_norm.weight", &w.ffn_norm, dm));
    }
    TRY_D(get_f(m, "token_embd.weight", &d->emb, (int64_t)c.vocab * dm));
    TRY_D(get_f(m, "output_norm.weight", &d->out_norm, dm));
    TRY_D(get_q(m, "output.weight", &d->head, d->V, dm, -1));
    {
        // Types may differ from tensor to tensor and from layer to layer (Q4_K_M files keep attn_v and ffn_down of
        // some layers in Q6_K); only gate and up of one layer must agree, since they are interleaved into one tensor.
        if (dm % 4 || F % 16 || (qd + 2 * kvd) % 4) {
            tlb_decoder_destroy(d);
            return fail(TLB_ERR_SHAPE, "d_model and the q|k|v width must be multiples of 4, ffn a multiple of 16");
        }
        // gate | up of every layer, interleaved by groups of 8 rows into one tensor of its own
        for (LayerW &w : d->layers) {
            tlb_qtensor *g = new tlb_qtensor();
            g->type = w.gate->type; g->n = 2 * F; g->k = dm; g->n_tiles = 2 * F / 16; g->upt = dm / 256;
            g->st = storage_alloc((size_t)g->n_tiles * g->upt * qformat(g->type)->unit_bytes);
            w.gu = g;
            if (!g->st) { tlb_decoder_destroy(d); return TLB_ERR_ALLOC; }
            TRY_D(launch_interleave8(g->type, w.gate->dev(), w.up->dev(), g->dev(), F, dm));
        }
    }
    TRY_D(dalloc(d, &d->xa, dm)); TRY_D(dalloc(d, &d->xb, dm));
    TRY_D(dalloc(d, &d->qkv, qd + 2 * kvd)); TRY_D(dalloc(d, &d->attn, qd));
    TRY_D(dalloc(d, &d->hbuf, F));
    TRY_D(dalloc(d, &d->ssq_o, (dm + 15) / 16)); TRY_D(dalloc(d, &d->ssq_d, (dm + 15) / 16));
    TRY_D(dalloc(d, &d->logits, d->V));
    if (tp > 1) {
        TRY_D(dalloc(d, &d->part, dm));
        TRY_D(dalloc(d, &d->pair, 2 * (1 + tp)));
        TRY_D(dalloc(d, &d->logits_all, c.vocab));
    }
    d->kv_layer_elems = (size_t)kvd * c.max_seq;
    d->kv_seq_bytes = d->kv_layer_elems * c.n_layers * (c.kv_f16 ? 2 : 4);
    const size_t kv_bytes = d->kv_seq_bytes * d->B;      // [sequence][layer][KV head][row][D]
    TRY_D(dalloc(d, (char **)&d->kcache, kv_bytes)); TRY_D(dalloc(d, (char **)&d->vcache, kv_bytes));
    d->max_splits = (c.max_seq + kAttnKeysPerSplit - 1) / kAttnKeysPerSplit;
    int rep = c.n_heads / c.n_kv_heads;
    TRY_D(dalloc(d, &d->partial, (size_t)d->KVH * d->max_splits * rep * (c.head_dim + 4)));
    TRY_D(dalloc(d, &d->counters, c.n_kv_heads + 1));
    TRY_D(dalloc(d, &d->state, 4));
    d->tokens_cap = c.max_seq;
    TRY_D(dalloc(d, &d->tokens_out, d->tokens_cap));
    TRY_D(dalloc(d, &d->amax_v, kArgmaxBlocks)); TRY_D(dalloc(d, &d->amax_i, kArgmaxBlocks));
    // RoPE tables on the host with libm, pair-duplicated [max_seq, D] (crates/tl_cpu/src/ffi.rs:2589-2627)
    {
        tlb_tensor *ct = nullptr, *sn = nullptr;
        TRY_D(tlb_rope_new_cos(&ct, c.head_dim, c.max_seq, c.rope_base, TLB_ROPE_CPU));
        st = tlb_rope_new_sin(&sn, c.head_dim, c.max_seq, c.rope_base, TLB_ROPE_CPU);
        if (st == TLB_OK) st = dalloc(d, &d->cos_t, (size_t)c.max_seq * c.head_dim, false);
        if (st == TLB_OK) st = dalloc(d, &d->sin_t, (size_t)c.max_seq * c.head_dim, false);
        if (st == TLB_OK) {
            size_t b = (size_t)c.max_seq * c.head_dim * 4;
            cudaMemcpyAsync(d->cos_t, ct->data(), b, cudaMemcpyDeviceToDevice, ctx()->stream);
            cudaMemcpyAsync(d->sin_t, sn->data(), b, cudaMemcpyDeviceToDevice, ctx()->stream);
        }
        tlb_tensor_release(ct); tlb_tensor_release(sn);
        if (st != TLB_OK) { tlb_decoder_destroy(d); return st; }
    }
    if (d->B > 1) {
        const size_t B = d->B;
        if (!prefill_batched_ok(d)) {
            tlb_decoder_destroy(d);
            return fail(TLB_ERR_SHAPE, "a batch session runs its linear layers on the tensor-core GEMM: d_model, the attention width and ffn must be multiples of 256, head_dim 64 or 128");
        }
        TRY_D(dalloc(d, &d->btok, B)); TRY_D(dalloc(d, &d->bpos, B)); TRY_D(dalloc(d, &d->brope, B)); TRY_D(dalloc(d, &d->bidx, 1));
        TRY_D(dalloc(d, &d->bx, B * dm)); TRY_D(dalloc(d, &d->bx2, B * dm)); TRY_D(dalloc(d, &d->bt, B * dm));
        TRY_D(dalloc(d, &d->bq, B * qd)); TRY_D(dalloc(d, &d->bk, B * kvd)); TRY_D(dalloc(d, &d->bv, B * kvd)); TRY_D(dalloc(d, &d->battn, B * qd));
        TRY_D(dalloc(d, &d->bg, B * F)); TRY_D(dalloc(d, &d->bu, B * F));
        TRY_D(dalloc(d, &d->blogits, B * (size_t)d->V));
        if (tp > 1) { TRY_D(dalloc(d, &d->blogits_all, B * (size_t)c.vocab * 2)); TRY_D(dalloc(d, &d->bpair, 2 * B * (1 + tp))); }
        TRY_D(dalloc(d, &d->bpartial, B * (size_t)d->KVH * d->max_splits * (c.n_heads / c.n_kv_heads) * (c.head_dim + 4)));
        TRY_D(dalloc(d, &d->bcounters, B * (size_t)d->KVH));
        TRY_D(dalloc(d, &d->btokens_out, (size_t)d->tokens_cap * B));
    }
    cudaError_t e = cudaMallocHost((void **)&d->h_state, 4 * sizeof(int));
    if (e != cudaSuccess) { tlb_decoder_destroy(d); return cuda_fail(e, "cudaMallocHost"); }
    d->dry = true;                 // every matvec shape of the chain must be launchable
    st = enqueue_step(d);
    d->dry = false;
    if (st != TLB_OK) { tlb_decoder_destroy(d); return st; }
    TRY_D(tlb_sync());
#undef TRY_D
    *out = d;
    return TLB_OK;
}

tlb_status tlb_decoder_kv_write(tlb_decoder *d, int layer, int pos0, int n, const float *k, const float *v)
{
    if (!d || !k || !v) return fail(TLB_ERR_NULL, "null argument");
    const tlb_decoder_cfg &c = d->cfg;
    if (layer < 0 || layer >= c.n_layers || pos0 < 0 || n < 0 || pos0 + n > c.max_seq)
        return fail(TLB_ERR_INDEX, "kv_write: layer %d rows [%d, %d) out of range", layer, pos0, pos0 + n);
    if (n == 0) return TLB_OK;
    const int D = c.head_dim, KVH = d->KVH, KVH_all = c.n_kv_heads, h0 = d->tp_r * d->KVH;   // host rows hold all heads; this rank keeps its own
    const size_t es = c.kv_f16 ? 2 : 4;
    // host layout [n][KVH*D] -> cache layout [KVH][max_seq][D]: staged whole, one copy per head, one wait at the end
    const size_t head_bytes = (size_t)n * D * es;
    std::vector<uint8_t> buf(2 * (size_t)KVH * head_bytes);
    for (int which = 0; which < 2; which++) {
        const float *src = which ? v : k;
        char *dst = (char *)(which ? d->vcache : d->kcache) + (size_t)layer * d->kv_layer_elems * es;
        for (int h = 0; h < KVH; h++) {
            uint8_t *hb = buf.data() + ((size_t)which * KVH + h) * head_bytes;
            for (int t = 0; t < n; t++)
                for (int e = 0; e < D; e++) {
                    float f = src[((size_t)t * KVH_all + h0 + h) * D + e];
                    if (c.kv_f16) ((__half *)hb)[(size_t)t * D + e] = __float2half_rn(f);
                    else ((float *)hb)[(size_t)t * D + e] = f;
                }
            TLB_CUDA(cudaMemcpyAsync(dst + ((size_t)h * c.max_seq + pos0) * D * es, hb, head_bytes, cudaMemcpyHostToDevice, ctx()->stream));
        }
    }
    TLB_CUDA(cudaStreamSynchronize(ctx()->stream));   // the staging buffer goes away on return
    return TLB_OK;
}

tlb_status tlb_decoder_step(tlb_decoder *d, int32_t token, int32_t pos, int32_t rope_pos, int32_t *next)
{
    if (!d) return fail(TLB_ERR_NULL, "null decoder");
    if (token < 0 || token >= d->cfg.vocab) return fail(TLB_ERR_INDEX, "Embedding index %d out of range for vocab size %d", token, d->cfg.vocab);
    if (pos < 0 || pos >= d->cfg.max_seq || rope_pos < 0 || rope_pos >= d->cfg.max_seq)
        return fail(TLB_ERR_INDEX, "position %d / %d outside the cache of %d rows", pos, rope_pos, d->cfg.max_seq);
    TLB_TRY(ensure_graph(d));
    TLB_TRY(set_state(d, token, pos, rope_pos, 0));
    TLB_CUDA(cudaGraphLaunch(d->graph, ctx()->stream));
    ctx()->launches += d->graph_kernels;
    if (next) {
        TLB_CUDA(cudaMemcpyAsync(d->h_state, d->state, sizeof(int), cudaMemcpyDeviceToHost, ctx()->stream));
        TLB_TRY(tlb_sync());
        *next = d->h_state[0];
    }
    return TLB_OK;
}

tlb_status tlb_decoder_generate(tlb_decoder *d, int32_t first_token, int32_t start_pos, int32_t n, int32_t *tokens_out)
{
    if (!d) return fail(TLB_ERR_NULL, "null decoder");
    if (first_token < 0 || first_token >= d->cfg.vocab) return fail(TLB_ERR_INDEX, "Embedding index %d out of range", first_token);
    if (n < 0 || start_pos < 0 || start_pos + n > d->cfg.max_seq) return fail(TLB_ERR_INDEX, "positions [%d, %d) outside the cache of %d rows", start_pos, start_pos + n, d->cfg.max_seq);
    TLB_TRY(ensure_graph(d));
    TLB_TRY(set_state(d, first_token, start_pos, start_pos, 0));
    for (int i = 0; i < n; i++) TLB_CUDA(cudaGraphLaunch(d->graph, ctx()->stream));
    ctx()->launches += d->graph_kernels * (uint64_t)n;
    if (tokens_out && n) {
        TLB_CUDA(cudaMemcpyAsync(tokens_out, d->tokens_out, (size_t)n * sizeof(int), cudaMemcpyDeviceToHost, ctx()->stream));
        TLB_TRY(tlb_sync());
    }
    return TLB_OK;
}

tlb_status tlb_decoder_logits(tlb_decoder *d, float *logits_out)
{
    if (!d || !logits_out) return fail(TLB_ERR_NULL, "null argument");
    const float *src = d->logits;
    if (d->tp > 1) {   // every rank calls this: the shards' rows are gathered in rank order = vocabulary order
        TLB_TRY(tp_allgather(d->logits, d->logits_all, (size_t)d->V * sizeof(float)));
        src = d->logits_all;
    }
    TLB_CUDA(cudaMemcpyAsync(logits_out, src, (size_t)d->cfg.vocab * 4, cudaMemcpyDeviceToHost, ctx()->stream));
    return tlb_sync();
}

tlb_status tlb_decoder_hidden(tlb_decoder *d, float *hidden_out)
{
    if (!d || !hidden_out) return fail(TLB_ERR_NULL, "null argument");
    TLB_CUDA(cudaMemcpyAsync(hidden_out, d->xb, (size_t)d->cfg.d_model * 4, cudaMemcpyDeviceToHost, ctx()->stream));
    return tlb_sync();
}

tlb_status tlb_decoder_stats(const tlb_decoder *d, int32_t ctx_len, uint64_t *weight_bytes, uint64_t *kv_bytes, int32_t *kernels_per_step)
{
    if (!d) return fail(TLB_ERR_NULL, "null decoder");
    uint64_t wb = d->head->nbytes() + (uint64_t)d->cfg.d_model * 4 * (2 * d->cfg.n_layers + 2);
    for (const LayerW &w : d->layers)
        wb += w.q->nbytes() + w.k->nbytes() + w.v->nbytes() + w.o->nbytes() + w.gate->nbytes() + w.up->nbytes() + w.down->nbytes();
    if (weight_bytes) *weight_bytes = wb;
    if (kv_bytes) *kv_bytes = 2ull * d->cfg.n_layers * d->KVH * d->cfg.head_dim * (uint64_t)ctx_len * (d->cfg.kv_f16 ? 2 : 4);
    if (kernels_per_step) {   // per layer: one q | k | v launch per weight type among the three, and four more; then head + argmax
        int nk = d->tp > 1 ? 3 : 2;
        for (const LayerW &w : d->layers) nk += 5 + (w.k->type != w.q->type) + (w.v->type != w.q->type && w.v->type != w.k->type);
        *kernels_per_step = nk;
    }
    return TLB_OK;
}

tlb_status tlb_decoder_time_kernel(tlb_decoder *d, const char *which, int copies, int iters, float *us_per_launch, uint64_t *bytes_per_launch)
{
    if (!d || !which || !us_per_launch) return fail(TLB_ERR_NULL, "null argument");
    const tlb_decoder_cfg &c = d->cfg;
    const int dm = c.d_model, qd = d->H * c.head_dim, kvd = d->KVH * c.head_dim, F = d->F;
    if (copies < 1) copies = 1;
    if (copies > c.n_layers) copies = c.n_layers;
    {   // the rotation below launches one kernel shape: only the leading layers typed like layer 0 take part
        const LayerW &a = d->layers[0];
        int same = 1;
        while (same < copies) {
            const LayerW &b = d->layers[same];
            if (b.q->type != a.q->type || b.k->type != a.q->type || b.v->type != a.q->type || a.k->type != a.q->type || a.v->type != a.q->type ||
                b.o->type != a.o->type || b.gu->type != a.gu->type || b.down->type != a.down->type) break;
            same++;
        }
        copies = same;
    }
    std::string w(which);
    int64_t out_n = w == "qkv" ? qd + 2 * kvd : (w == "o" || w == "down") ? dm : w == "gate_up" ? 2 * F : w == "head" ? d->V : -1;
    if (out_n < 0) return fail(TLB_ERR_ARG, "unknown kernel '%s' (qkv, o, gate_up, down, head)", which);
    int64_t kk = (w == "o") ? qd : (w == "down") ? F : dm;
    float *xin = nullptr, *outb = nullptr;
    TLB_CUDA(cudaMalloc(&xin, (size_t)std::max<int64_t>(kk, 2 * F) * 4));
    constexpr int kOutRot = 3;   // consecutive launches overlap (programmatic dependent launch): each writes a buffer of its own
    TLB_CUDA(cudaMalloc(&outb, (size_t)out_n * kOutRot * 4));
    {
        std::vector<float> hx((size_t)std::max<int64_t>(kk, 2 * F));
        uint32_t s = 12345u;
        for (float &v : hx) { s = s * 1664525u + 1013904223u; v = ((s >> 8) / 8388608.0f) - 1.0f; }
        cudaMemcpy(xin, hx.data(), hx.size() * 4, cudaMemcpyHostToDevice);
    }
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    uint64_t bytes = 0;
    tlb_status st = TLB_OK;
    for (int it = -3; it < iters && st == TLB_OK; it++) {   // 3 warm-up launches, then the timed ones
        if (it == 0) cudaEventRecord(e0, ctx()->stream);
        const LayerW &lw = d->layers[(it + 3) % copies];
        MatvecJob j;
        float *o = outb + (size_t)((it + 3) % kOutRot) * out_n;
        j.m = 1; j.prologue = PRO_PLAIN; j.x = xin;
        if (w == "qkv") {
            if (lw.k->type != lw.q->type || lw.v->type != lw.q->type) { st = fail(TLB_ERR_TYPE, "time_kernel(qkv): q, k, v of layer 0 differ in type"); break; }
            j.n_w = 3; set_w(j, 0, lw.q, o); set_w(j, 1, lw.k, o + qd); set_w(j, 2, lw.v, o + qd + kvd);
            j.type = lw.q->type; j.k = dm; bytes = lw.q->nbytes() + lw.k->nbytes() + lw.v->nbytes();
        } else if (w == "o") {
            j.n_w = 1; set_w(j, 0, lw.o, o); j.type = lw.o->type; j.k = qd; bytes = lw.o->nbytes();
        } else if (w == "gate_up") {
            j.n_w = 1; set_w(j, 0, lw.gu, o); j.type = lw.gu->type; j.k = dm; j.finish = FIN_SILU;
            bytes = lw.gu->nbytes();
        } else if (w == "down") {
            j.n_w = 1; set_w(j, 0, lw.down, o); j.type = lw.down->type; j.k = F; bytes = lw.down->nbytes();
        } else {
            j.n_w = 1; set_w(j, 0, d->head, o); j.type = d->head->type; j.k = dm; bytes = d->head->nbytes();
            j.last_of_chain = true;
        }
        j.pdl = d->pdl;   // as in the decode chain: a launch's set-up overlaps its predecessor
        st = launch_qmatvec(j);
    }
    cudaEventRecord(e1, ctx()->stream);
    cudaEventSynchronize(e1);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    cudaFree(xin); cudaFree(outb);
    if (st != TLB_OK) return st;
    *us_per_launch = ms * 1000.f / (float)std::max(1, iters);
    if (bytes_per_launch) *bytes_per_launch = bytes + (uint64_t)kk * 4 + (uint64_t)out_n * 4;
    return tlb_sync();
}

}  // extern "C"

// Prompt processing: `n` tokens at once.  Per layer: norm -> q, k, v GEMMs -> RoPE + cache append -> causal
// attention over the cache -> o GEMM (+ residual) -> norm -> gate, up GEMMs -> silu * up -> down GEMM (+ residual);
// then the decode head on the last token.  Prompts are cut into chunks so the f32 work space stays bounded.
namespace {
constexpr int kPrefillChunk = 2048;

bool prefill_batched_ok(const tlb_decoder *d)
{
    const tlb_decoder_cfg &c = d->cfg;
    const int qd = d->H * c.head_dim, kvd = d->KVH * c.head_dim;
    for (const LayerW &w : d->layers)
        if (!qgemm_supported(w.q->type) || !qgemm_supported(w.k->type) || !qgemm_supported(w.v->type) || !qgemm_supported(w.o->type) ||
            !qgemm_supported(w.gate->type) || !qgemm_supported(w.down->type))
            return false;
    return qgemm_supported(d->head->type) && prefill_attention_supported(c.head_dim) && c.d_model % 256 == 0 && qd % 256 == 0 && d->F % 256 == 0 && kvd % 4 == 0;
}

struct Scratch {
    std::vector<Storage *> all;
    template <typename T> tlb_status get(T **p, size_t count)
    {
        Storage *s = storage_alloc(count * sizeof(T));
        if (!s) return TLB_ERR_ALLOC;
        all.push_back(s);
        *p = (T *)s->ptr;
        return TLB_OK;
    }
    ~Scratch() { for (Storage *s : all) storage_release(s); }
};

// T prompt tokens of sequence `seq` (0 for a single-sequence session) into cache rows pos0 ..; the residual of the last
// token is copied to last_row_out when given.  With tensor parallelism every rank runs this on its shard.
tlb_status prefill_chunk(tlb_decoder *d, int seq, const int32_t *tokens, int T, int pos0, int rope0, int rope_step, float *last_row_out)
{
    const tlb_decoder_cfg &c = d->cfg;
    const int dm = c.d_model, qd = d->H * c.head_dim, kvd = d->KVH * c.head_dim, F = d->F;
    const size_t esz = c.kv_f16 ? 2 : 4;
    Scratch ws;
    int *tok_d;
    float *x, *x2, *q, *k, *v, *att, *g, *u, *part = nullptr;
    TLB_TRY(ws.get(&tok_d, (size_t)T));
    if (d->tp > 1) TLB_TRY(ws.get(&part, (size_t)T * dm));
    TLB_TRY(ws.get(&x, (size_t)T * dm)); TLB_TRY(ws.get(&x2, (size_t)T * dm));
    TLB_TRY(ws.get(&q, (size_t)T * qd)); TLB_TRY(ws.get(&k, (size_t)T * kvd)); TLB_TRY(ws.get(&v, (size_t)T * kvd));
    TLB_TRY(ws.get(&att, (size_t)T * qd));
    TLB_TRY(ws.get(&g, (size_t)T * F)); TLB_TRY(ws.get(&u, (size_t)T * F));
    TLB_CUDA(cudaMemcpyAsync(tok_d, tokens, (size_t)T * sizeof(int), cudaMemcpyHostToDevice, ctx()->stream));
    TLB_TRY(launch_embed_rows(tok_d, d->emb->f32(), x, T, dm));
    for (int l = 0; l < c.n_layers; l++) {
        const LayerW &w = d->layers[l];
        void *kc = (char *)d->kcache + (size_t)seq * d->kv_seq_bytes + (size_t)l * d->kv_layer_elems * esz;
        void *vc = (char *)d->vcache + (size_t)seq * d->kv_seq_bytes + (size_t)l * d->kv_layer_elems * esz;
        GemmAct a;
        tlb_status st;
        TLB_TRY(qgemm_prepare(&a, x, nullptr, T, dm, w.attn_norm->f32(), c.eps));
        {   // q | k | v: one launch per weight type (one launch when they agree)
            const tlb_qtensor *ws3[3] = {w.q, w.k, w.v};
            float *outs3[3] = {q, k, v};
            bool done3[3] = {false, false, false};
            st = TLB_OK;
            for (int i = 0; i < 3 && st == TLB_OK; i++) {
                if (done3[i]) continue;
                const tlb_qtensor *gw[3];
                float *go[3];
                int gn = 0;
                for (int b = i; b < 3; b++)
                    if (!done3[b] && ws3[b]->type == ws3[i]->type) { gw[gn] = ws3[b]; go[gn++] = outs3[b]; done3[b] = true; }
                st = qgemm_run_multi(gw, gn, a, go, nullptr);
            }
        }
        qgemm_release(&a);
        TLB_TRY(st);
        TLB_TRY(launch_rope_append(q, k, v, kc, vc, c.kv_f16, d->cos_t, d->sin_t, T, d->H, d->KVH, c.head_dim, c.max_seq, pos0, rope0, rope_step));
        TLB_TRY(launch_prefill_attention(q, kc, vc, c.kv_f16, att, T, d->H, d->KVH, c.head_dim, c.max_seq, pos0, c.attn_scale));
        TLB_TRY(qgemm_prepare(&a, att, nullptr, T, qd, nullptr, 0.f));
        st = row_parallel(d, w.o, a, x2, x, part, T);  // x2 = x + o_proj(attention)
        qgemm_release(&a);
        TLB_TRY(st);
        TLB_TRY(qgemm_prepare(&a, x2, nullptr, T, dm, w.ffn_norm->f32(), c.eps));
        {
            const tlb_qtensor *ws2[2] = {w.gate, w.up};
            float *outs2[2] = {g, u};
            st = qgemm_run_multi(ws2, 2, a, outs2, nullptr);
        }
        qgemm_release(&a);
        TLB_TRY(st);
        // silu(gate) * up as a pass of its own: fused into the conversion it was slower (the exponentials ran twice
        // or the row of 14336 had to stay in registers)
        TLB_TRY(launch_silu_mul(g, u, g, (int64_t)T * F));
        TLB_TRY(qgemm_prepare(&a, g, nullptr, T, F, nullptr, 0.f));
        st = row_parallel(d, w.down, a, x, x2, part, T);   // x = x2 + down(silu(gate) * up)
        qgemm_release(&a);
        TLB_TRY(st);
    }
    if (last_row_out) TLB_CUDA(cudaMemcpyAsync(last_row_out, x + (size_t)(T - 1) * dm, (size_t)dm * sizeof(float), cudaMemcpyDeviceToDevice, ctx()->stream));
    return TLB_OK;
}
}  // namespace

extern "C" tlb_status tlb_decoder_prefill(tlb_decoder *d, const int32_t *tokens, int32_t n, int32_t pos0, int32_t rope_pos0, int32_t rope_step, int32_t *next)
{
    if (!d || !tokens) return fail(TLB_ERR_NULL, "null argument");
    const tlb_decoder_cfg &c = d->cfg;
    if (n < 1) return fail(TLB_ERR_ARG, "prefill needs at least one token");
    for (int i = 0; i < n; i++)
        if (tokens[i] < 0 || tokens[i] >= c.vocab) return fail(TLB_ERR_INDEX, "Embedding index %d out of range for vocab size %d", tokens[i], c.vocab);
    const int64_t last_rope = (int64_t)rope_pos0 + (int64_t)(n - 1) * rope_step;
    if (pos0 < 0 || (int64_t)pos0 + n > c.max_seq || rope_pos0 < 0 || rope_step < 0 || last_rope >= c.max_seq)
        return fail(TLB_ERR_INDEX, "positions [%d, %d) / rotation rows up to %lld outside the cache of %d rows", pos0, pos0 + n, (long long)last_rope, c.max_seq);
    if (n <= 4 || !prefill_batched_ok(d)) {
        // few tokens, or a shape the GEMM path does not take: the fused single-token chain, token by token
        int32_t tok = 0;
        for (int i = 0; i < n; i++) TLB_TRY(tlb_decoder_step(d, tokens[i], pos0 + i, rope_pos0 + i * rope_step, i == n - 1 ? &tok : nullptr));
        if (next) *next = tok;
        return TLB_OK;
    }
    for (int off = 0; off < n; off += kPrefillChunk) {
        const int T = std::min(kPrefillChunk, n - off);
        TLB_TRY(prefill_chunk(d, 0, tokens + off, T, pos0 + off, rope_pos0 + off * rope_step, rope_step, off + T == n ? d->xb : nullptr));
    }
    // head on the last token; the state then names the next token and the row it will occupy
    TLB_TRY(set_state(d, tokens[n - 1], pos0 + n - 1, (int)last_rope, 0));
    TLB_TRY(enqueue_head(d, nullptr));
    if (next) {
        TLB_CUDA(cudaMemcpyAsync(d->h_state, d->state, sizeof(int), cudaMemcpyDeviceToHost, ctx()->stream));
        TLB_TRY(tlb_sync());
        *next = d->h_state[0];
    }
    return TLB_OK;
}

// n sampled steps with the token fed back on the device: softmax(logits / temp), the k most probable tokens, the top-p prefix,
// one draw per step from the counter-based generator keyed by `seed` (step i of this call uses counter i: the same seed
// gives the same tokens; tlb_rng_uniform(seed, i) is the number step i drew).  temp <= 0 is tlb_decoder_generate.
extern "C" tlb_status tlb_decoder_generate_sampled(tlb_decoder *d, int32_t first_token, int32_t start_pos, int32_t n, float temp, int32_t top_k, float top_p,
                                                   uint64_t seed, int32_t *tokens_out)
{
    if (!d) return fail(TLB_ERR_NULL, "null decoder");
    if (temp <= 0.f || top_k == 1) return tlb_decoder_generate(d, first_token, start_pos, n, tokens_out);
    if (d->tp > 1) return fail(TLB_ERR_ARG, "sampled generation needs the whole vocabulary on one GPU (tp_size 1)");
    if (first_token < 0 || first_token >= d->cfg.vocab) return fail(TLB_ERR_INDEX, "Embedding index %d out of range", first_token);
    if (n < 0 || start_pos < 0 || start_pos + n > d->cfg.max_seq) return fail(TLB_ERR_INDEX, "positions [%d, %d) outside the cache of %d rows", start_pos, start_pos + n, d->cfg.max_seq);
    if (!d->samp_ws) {
        TLB_CUDA(cudaMalloc(&d->samp_ws, sample_workspace_bytes(d->cfg.vocab)));
        d->allocs.push_back(d->samp_ws);
        TLB_CUDA(cudaMalloc((void **)&d->samp_counter, sizeof(unsigned long long)));
        d->allocs.push_back(d->samp_counter);
    }
    if (d->sgraph && (d->samp.temp != temp || d->samp.top_k != top_k || d->samp.top_p != top_p || d->samp.seed != seed)) {
        TLB_CUDA(cudaStreamSynchronize(ctx()->stream));
        cudaGraphExecDestroy(d->sgraph);
        d->sgraph = nullptr;
    }
    if (!d->sgraph) {
        d->samp.temp = temp; d->samp.top_k = top_k; d->samp.top_p = top_p; d->samp.seed = seed;
        Context *cx = ctx();
        const uint64_t before = cx->launches.load();
        d->samp.on = true;
        TLB_CUDA(cudaStreamBeginCapture(cx->stream, cudaStreamCaptureModeThreadLocal));
        tlb_status st = enqueue_step(d);
        cudaGraph_t g = nullptr;
        cudaError_t e = cudaStreamEndCapture(cx->stream, &g);
        d->samp.on = false;
        d->sgraph_kernels = cx->launches.load() - before;
        cx->launches = before;
        if (st != TLB_OK) { if (g) cudaGraphDestroy(g); return st; }
        if (e != cudaSuccess) return cuda_fail(e, "cudaStreamEndCapture");
        e = cudaGraphInstantiate(&d->sgraph, g, 0);
        cudaGraphDestroy(g);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGraphInstantiate");
    }
    const unsigned long long zero = 0;
    TLB_CUDA(cudaMemcpyAsync(d->samp_counter, &zero, sizeof zero, cudaMemcpyHostToDevice, ctx()->stream));
    TLB_TRY(set_state(d, first_token, start_pos, start_pos, 0));
    for (int i = 0; i < n; i++) TLB_CUDA(cudaGraphLaunch(d->sgraph, ctx()->stream));
    ctx()->launches += d->sgraph_kernels * (uint64_t)n;
    if (tokens_out && n) {
        TLB_CUDA(cudaMemcpyAsync(tokens_out, d->tokens_out, (size_t)n * sizeof(int), cudaMemcpyDeviceToHost, ctx()->stream));
        TLB_TRY(tlb_sync());
    }
    return TLB_OK;
}

// ---- batch sessions: per-sequence prompts and batched steps -------------------------------------------------------
namespace {
tlb_status need_batch(const tlb_decoder *d, int seq)
{
    if (!d) return fail(TLB_ERR_NULL, "null decoder");
    if (d->B <= 1) return fail(TLB_ERR_ARG, "the session was created with batch <= 1");
    if (seq < 0 || seq >= d->B) return fail(TLB_ERR_INDEX, "sequence %d outside the batch of %d", seq, d->B);
    return TLB_OK;
}
tlb_status put_ints(int *dst, const int32_t *src, size_t n)
{
    TLB_CUDA(cudaMemcpyAsync(dst, src, n * sizeof(int), cudaMemcpyHostToDevice, ctx()->stream));   // pageable source: staged before return
    return TLB_OK;
}
}  // namespace

extern "C" tlb_status tlb_decoder_kv_write_seq(tlb_decoder *d, int seq, int layer, int pos0, int n, const float *k, const float *v)
{
    if (!d) return fail(TLB_ERR_NULL, "null decoder");
    if (seq < 0 || seq >= d->B) return fail(TLB_ERR_INDEX, "sequence %d outside the batch of %d", seq, d->B);
    // the single-sequence writer on a cache pointer moved to the sequence's region
    void *k0 = d->kcache, *v0 = d->vcache;
    d->kcache = (char *)k0 + (size_t)seq * d->kv_seq_bytes;
    d->vcache = (char *)v0 + (size_t)seq * d->kv_seq_bytes;
    tlb_status st = tlb_decoder_kv_write(d, layer, pos0, n, k, v);
    d->kcache = k0; d->vcache = v0;
    return st;
}

extern "C" tlb_status tlb_decoder_prefill_seq(tlb_decoder *d, int32_t seq, const int32_t *tokens, int32_t n, int32_t pos0, int32_t rope_pos0, int32_t rope_step, int32_t *next)
{
    TLB_TRY(need_batch(d, seq));
    if (!tokens) return fail(TLB_ERR_NULL, "null tokens");
    const tlb_decoder_cfg &c = d->cfg;
    if (n < 1) return fail(TLB_ERR_ARG, "prefill needs at least one token");
    for (int i = 0; i < n; i++)
        if (tokens[i] < 0 || tokens[i] >= c.vocab) return fail(TLB_ERR_INDEX, "Embedding index %d out of range for vocab size %d", tokens[i], c.vocab);
    const int64_t last_rope = (int64_t)rope_pos0 + (int64_t)(n - 1) * rope_step;
    if (pos0 < 0 || (int64_t)pos0 + n > c.max_seq || rope_pos0 < 0 || rope_step < 0 || last_rope >= c.max_seq)
        return fail(TLB_ERR_INDEX, "positions [%d, %d) / rotation rows up to %lld outside the cache of %d rows", pos0, pos0 + n, (long long)last_rope, c.max_seq);
    float *row = d->bx2 + (size_t)seq * c.d_model;     // free between steps
    for (int off = 0; off < n; off += kPrefillChunk) {
        const int T = std::min(kPrefillChunk, n - off);
        TLB_TRY(prefill_chunk(d, seq, tokens + off, T, pos0 + off, rope_pos0 + off * rope_step, rope_step, off + T == n ? row : nullptr));
    }
    // the sequence's state: the last prompt token at its row; the head then names the next token and advances both
    const int32_t st3[3] = {tokens[n - 1], pos0 + n - 1, (int32_t)last_rope};
    TLB_TRY(put_ints(d->btok + seq, st3, 1)); TLB_TRY(put_ints(d->bpos + seq, st3 + 1, 1)); TLB_TRY(put_ints(d->brope + seq, st3 + 2, 1));
    int *keep = d->btokens_out;
    d->btokens_out = nullptr;                           // a prompt's token is not part of a generate() run
    tlb_status st = batch_head(d, row, 1, seq);
    d->btokens_out = keep;
    TLB_TRY(st);
    if (next) {
        TLB_CUDA(cudaMemcpyAsync(d->h_state, d->btok + seq, sizeof(int), cudaMemcpyDeviceToHost, ctx()->stream));
        TLB_TRY(tlb_sync());
        *next = d->h_state[0];
    }
    return TLB_OK;
}

// One token for every sequence: tokens[b] goes to cache row pos[b] of sequence b (rotation row rope_pos[b], or pos[b] when
// rope_pos is null); next (may be null) receives the greedy tokens.  One pass over the weights serves the whole batch.
extern "C" tlb_status tlb_decoder_step_batch(tlb_decoder *d, const int32_t *tokens, const int32_t *pos, const int32_t *rope_pos, int32_t *next)
{
    TLB_TRY(need_batch(d, 0));
    if (!tokens || !pos) return fail(TLB_ERR_NULL, "null argument");
    const tlb_decoder_cfg &c = d->cfg;
    for (int b = 0; b < d->B; b++) {
        const int rp = rope_pos ? rope_pos[b] : pos[b];
        if (tokens[b] < 0 || tokens[b] >= c.vocab) return fail(TLB_ERR_INDEX, "Embedding index %d out of range for vocab size %d", tokens[b], c.vocab);
        if (pos[b] < 0 || pos[b] >= c.max_seq || rp < 0 || rp >= c.max_seq) return fail(TLB_ERR_INDEX, "sequence %d: position %d / %d outside the cache of %d rows", b, pos[b], rp, c.max_seq);
    }
    TLB_TRY(ensure_batch_graph(d));
    const int32_t zero = 0;
    TLB_TRY(put_ints(d->btok, tokens, d->B)); TLB_TRY(put_ints(d->bpos, pos, d->B)); TLB_TRY(put_ints(d->brope, rope_pos ? rope_pos : pos, d->B));
    TLB_TRY(put_ints(d->bidx, &zero, 1));
    TLB_CUDA(cudaGraphLaunch(d->bgraph, ctx()->stream));
    ctx()->launches += d->bgraph_kernels;
    if (next) {
        TLB_CUDA(cudaMemcpyAsync(next, d->btok, (size_t)d->B * sizeof(int), cudaMemcpyDeviceToHost, ctx()->stream));
        TLB_TRY(tlb_sync());
    }
    return TLB_OK;
}

// n greedy steps of the whole batch with the tokens fed back on the device; tokens_out (may be null): [n][batch].
extern "C" tlb_status tlb_decoder_generate_batch(tlb_decoder *d, const int32_t *first_tokens, const int32_t *start_pos, int32_t n, int32_t *tokens_out)
{
    TLB_TRY(need_batch(d, 0));
    if (!first_tokens || !start_pos) return fail(TLB_ERR_NULL, "null argument");
    const tlb_decoder_cfg &c = d->cfg;
    if (n < 0 || n > d->tokens_cap) return fail(TLB_ERR_INDEX, "%d steps exceed the session's %d rows", n, d->tokens_cap);
    for (int b = 0; b < d->B; b++) {
        if (first_tokens[b] < 0 || first_tokens[b] >= c.vocab) return fail(TLB_ERR_INDEX, "Embedding index %d out of range", first_tokens[b]);
        if (start_pos[b] < 0 || (int64_t)start_pos[b] + n > c.max_seq) return fail(TLB_ERR_INDEX, "sequence %d: rows [%d, %d) outside the cache of %d rows", b, start_pos[b], start_pos[b] + n, c.max_seq);
    }
    TLB_TRY(ensure_batch_graph(d));
    const int32_t zero = 0;
    TLB_TRY(put_ints(d->btok, first_tokens, d->B)); TLB_TRY(put_ints(d->bpos, start_pos, d->B)); TLB_TRY(put_ints(d->brope, start_pos, d->B));
    TLB_TRY(put_ints(d->bidx, &zero, 1));
    for (int i = 0; i < n; i++) TLB_CUDA(cudaGraphLaunch(d->bgraph, ctx()->stream));
    ctx()->launches += d->bgraph_kernels * (uint64_t)n;
    if (tokens_out && n) {
        TLB_CUDA(cudaMemcpyAsync(tokens_out, d->btokens_out, (size_t)n * d->B * sizeof(int), cudaMemcpyDeviceToHost, ctx()->stream));
        TLB_TRY(tlb_sync());
    }
    return TLB_OK;
}

// logits of the last step (or prompt) of every sequence: [batch, vocab]
extern "C" tlb_status tlb_decoder_logits_batch(tlb_decoder *d, float *logits_out)
{
    TLB_TRY(need_batch(d, 0));
    if (!logits_out) return fail(TLB_ERR_NULL, "null argument");
    const size_t B = d->B, V = d->V, vocab = d->cfg.vocab;
    if (d->tp <= 1) {
        TLB_CUDA(cudaMemcpyAsync(logits_out, d->blogits, B * vocab * 4, cudaMemcpyDeviceToHost, ctx()->stream));
        return tlb_sync();
    }
    // gathered as [rank][batch][V]; rearranged to [batch][vocab] on the way out (every rank calls this)
    float *gath = d->blogits_all + B * vocab;
    TLB_TRY(tp_allgather(d->blogits, gath, B * V * sizeof(float)));
    for (int r = 0; r < d->tp; r++)
        TLB_CUDA(cudaMemcpy2DAsync(d->blogits_all + (size_t)r * V, vocab * 4, gath + (size_t)r * B * V, V * 4, V * 4, B, cudaMemcpyDeviceToDevice, ctx()->stream));
    TLB_CUDA(cudaMemcpyAsync(logits_out, d->blogits_all, B * vocab * 4, cudaMemcpyDeviceToHost, ctx()->stream));
    return tlb_sync();
}

// Temperature / top-p sampling from the logits of the last step or prompt, on the device: only the token id crosses
// to the host (the logits are 4 bytes x vocab).  The caller feeds the token to the next tlb_decoder_step.
extern "C" tlb_status tlb_decoder_sample_top_p(tlb_decoder *d, float temp, float top_p, double u, int32_t *token)
{
    if (!d || !token) return fail(TLB_ERR_NULL, "null argument");
    if (!(u >= 0.0 && u < 1.0)) return fail(TLB_ERR_ARG, "sample: the random number must lie in [0, 1)");
    if (temp <= 0.f) {   // greedy: what the step itself chose
        TLB_CUDA(cudaMemcpyAsync(d->h_state, d->state, sizeof(int), cudaMemcpyDeviceToHost, ctx()->stream));
        TLB_TRY(tlb_sync());
        *token = d->h_state[0];
        return TLB_OK;
    }
    TLB_TRY(launch_sample_top_p(d->logits, d->cfg.vocab, temp, top_p, (float)u, d->amax_v));   // amax_v: free between steps
    float h = 0.f;
    TLB_CUDA(cudaMemcpyAsync(&h, d->amax_v, sizeof(float), cudaMemcpyDeviceToHost, ctx()->stream));
    TLB_TRY(tlb_sync());
    *token = (int32_t)h;
    return TLB_OK;
}
