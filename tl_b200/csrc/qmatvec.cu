// Streaming dequant-fused matvec for GGUF Q4_K / Q6_K / Q8_0 / Q4_0 weights (decode path,
// 1..4 activation rows).  Replaces mul_mv_q4_k_kernel / mul_mv_q6_k_kernel
// (crates/tl_cuda/src/cuda_kernels/autograd.cu:2813-2900: one thread per output, byte loads, weights
// re-read once per activation row) and the dequantise-then-naive-matmul route the reference takes
// for Q4_0 / Q8_0 (crates/tl_runtime/src/system.rs:236-264).
//
// Shape of the kernel (persistent CTAs, one or two per SM):
//   * the weight bytes of all tensors of a launch form ONE linear stream of units (16 rows x 256
//     weights, quant.cu); CTA b takes the contiguous range [U*b/G, U*(b+1)/G): equal bytes per CTA
//     whatever the row count;
//   * a producer warp moves units global -> shared with 1-D bulk async copies (cp.async.bulk +
//     mbarrier complete_tx) through a ring of stages; it does not depend on the activations, so
//     the HBM stream starts while the prologue is still running (and, under programmatic dependent
//     launch, while the previous kernel is still finishing);
//   * the prologue quantises the activation to int8 levels in shared memory (qmv_common.cuh) and
//     can fuse what precedes the matvec in the decode chain: residual add + RMSNorm * weight,
//     SiLU(gate) * up, or the embedding lookup;
//   * consumer warps take one unit at a time: conflict-free 128-bit shared loads, one AND per four
//     weights, integer tensor-core MMAs (qmv_units.cuh);
//   * per output tile the warps' fragments are summed in fixed order in shared memory and added to
//     the output with one atomicAdd per row.  A tile is touched by at most two CTAs per
//     accumulation slot and a + b == b + a, so results do not depend on scheduling.
#include "qmv_prologue.cuh"
#include "qmv_units.cuh"

#include <map>

namespace tlb {

constexpr int kRedCols = 12;   // 8 MMA columns + 4 min-term columns (one per activation row)
constexpr int kProducerLanes = 8;

__device__ __forceinline__ const uint8_t *unit_src(const MvParams &p, int u)
{
    int tile = u / p.upt, uk = u - tile * p.upt;
    int wi = (tile >= p.tiles_end[0]) + (tile >= p.tiles_end[1]);
    int t0 = wi == 0 ? 0 : p.tiles_end[wi - 1];
    return p.w[wi] + ((size_t)(tile - t0) * p.upt + uk) * p.unit_bytes;
}

template <int FMT, int NW>
__global__ void __launch_bounds__(NW * 32 + 32, (NW <= 8) ? 2 : 1) qmatvec_kernel(const __grid_constant__ MvParams p)
{
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int NT = NW * 32;   // consumer threads
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nst = p.n_stages;
    float *red = reinterpret_cast<float *>(smem + p.off_red);            // [2][NW][kRedCols][16]
    MvShared *sh = reinterpret_cast<MvShared *>(smem + p.off_misc + p.m * (p.k / 128) * 4);
    const uint32_t full0 = smem_u32(smem + p.off_bars), empty0 = full0 + nst * 8;
    const uint32_t ring_u32 = smem_u32(smem);

    const int G = gridDim.x, b = blockIdx.x;
    const int u0 = (int)((long long)p.total_units * b / G), u1 = (int)((long long)p.total_units * (b + 1) / G);
    const int n_units = u1 - u0;
#define STAMP(i) do { if (p.trace && tid == 0) p.trace[(size_t)b * 10 + (i)] = clock64(); } while (0)
    STAMP(0);
    if (p.trace && tid == 0) p.trace[(size_t)b * 10 + 8] = (long long)global_ns();

    const uint32_t act_bar = full0 + 2 * nst * 8;   // completion of the activation-image copy
    if (tid < nst) {   // one thread per stage: the inits run in parallel
        mbar_init(full0 + tid * 8, 1);
        mbar_init(empty0 + tid * 8, 1);
        if (tid == 0) { sh->abort_flag = 0; mbar_init(act_bar, 1); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    volatile int *abortp = &sh->abort_flag;
    STAMP(1);

    if (warp == NW) {
        // ---- producer: lane i < kProducerLanes streams the units i, i + kProducerLanes, ... of this
        // CTA's range.  The stage count is a multiple of kProducerLanes, so every stage is always
        // armed by the same lane: a lane reuses a stage only after ITS previous use of that stage
        // was released, which keeps the parity waits unambiguous.  Weights do not depend on the
        // previous kernel, so there is no dependency wait here.
        if (lane >= kProducerLanes) return;
        int i = lane, slot = lane, use = 0;
        for (; i < n_units; i += kProducerLanes) {
            if (use > 0 && !mbar_wait(empty0 + slot * 8, (use - 1) & 1, abortp, p.err, 1)) break;
            mbar_expect_tx(full0 + slot * 8, p.unit_bytes);
            bulk_g2s(ring_u32 + slot * p.stage_bytes, unit_src(p, u0 + i), p.unit_bytes, full0 + slot * 8);
            slot += kProducerLanes;
            if (slot >= nst) { slot -= nst; use++; }
        }
        if (*abortp) {
            // give the copies this lane still has in flight a bounded time to land before the CTA exits
            for (int k = i - kProducerLanes, n = 0; k >= 0 && n < nst; k -= kProducerLanes, n++)
                mbar_wait_drain(full0 + (k % nst) * 8, (k / nst) & 1);
        }
        return;
    }

    // ---- consumers
    if (p.use_pdl) {
        pdl_wait();                // everything below may read what the previous kernel wrote
        // Released only after our own wait: a dependent's early part then runs with every kernel
        // before our predecessor complete, so it may read state those kernels wrote.
        pdl_launch_dependents();
    }
    for (int z = 0; z < 3; z++)
        if (p.zero_ptr[z])
            for (long long idx = (long long)b * NT + tid; idx < p.zero_n[z]; idx += (long long)G * NT) p.zero_ptr[z][idx] = 0.f;
    STAMP(2);
    const bool act_ok = build_activation<FMT>(p, sh, smem, tid, NT, act_bar, abortp);
    STAMP(3);
    if (!act_ok) return;   // a bounded wait gave up: the error word is set, outputs stay untouched
    const int ncols = p.m * p.nl;
    LaneCtx L;
    L.lane = lane; L.r = lane >> 2; L.c = lane & 3;
    {
        const int r = L.r, c = L.c;
        const int colr = r < ncols ? r : 0, c0 = 2 * c < ncols ? 2 * c : 0, c1 = 2 * c + 1 < ncols ? 2 * c + 1 : 0;
        L.xq_b = smem_u32(smem + p.off_xq) + colr * p.col_stride;
        L.alam_b = smem_u32(smem + p.off_alam) + 2 * c * 4;
        L.xsum_b = smem_u32(smem + p.off_xsum) + ((r < 2 * p.m) ? r : (r & 1)) * (p.k / 32) * 2;
        L.sa_b = smem_u32(smem + p.off_sa) + colr * 32;
        L.sa_c0 = smem_u32(smem + p.off_sa) + c0 * 4;
        L.sa_c1 = smem_u32(smem + p.off_sa) + c1 * 4;
        L.minv_b = smem_u32(smem + p.off_minv) + (c < p.m ? c : 0) * 4;
    }

    // Ring cursor of this warp, advanced incrementally (no integer division in the unit loop):
    // the unit with CTA-relative index cur_rel sits in stage `slot`, in use number `phase` (mod 2).
    int u = u0, par = 0, tile = u0 / p.upt;
    int cur_rel = 0, slot = 0, phase = 0;
    while (u < u1) {
        const int tile_first = tile * p.upt;
        const int seg_end = min(u1, tile_first + p.upt);
        float master[4] = {0.f, 0.f, 0.f, 0.f}, mm[4] = {0.f, 0.f, 0.f, 0.f};
        for (int uu = u + warp; uu < seg_end; uu += NW) {
            slot += (uu - u0) - cur_rel;
            cur_rel = uu - u0;
            while (slot >= nst) { slot -= nst; phase ^= 1; }
            if (!mbar_wait(full0 + slot * 8, phase, abortp, p.err, 2)) break;
            if (cur_rel == 0) STAMP(4);
            process_unit<FMT>(ring_u32 + slot * p.stage_bytes, uu - tile_first, L, master, mm);
            if (cur_rel == 0) STAMP(5);
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + slot * 8);
        }
        float *rp = red + ((size_t)par * NW + warp) * (kRedCols * 16);
        rp[(2 * L.c) * 16 + L.r] = master[0];
        rp[(2 * L.c + 1) * 16 + L.r] = master[1];
        rp[(2 * L.c) * 16 + L.r + 8] = master[2];
        rp[(2 * L.c + 1) * 16 + L.r + 8] = master[3];
        if (FMT == TLB_GGML_Q4_K) {   // min term of activation row c: columns (hi, lo) summed
            rp[(8 + L.c) * 16 + L.r] = -(mm[0] + mm[1]);
            rp[(8 + L.c) * 16 + L.r + 8] = -(mm[2] + mm[3]);
        }
        named_bar(1, NT);
        {
            // Every warp reduces its share of the 16 rows: lane = (source warp, column slot); the
            // butterfly adds in a fixed order, so the sum does not depend on timing.
            constexpr int RPW = 16 / NW, CSL = 32 / NW;   // rows per warp, column slots per pass
            const int w_src = lane % NW, cs = lane / NW;
            const int wi = (tile >= p.tiles_end[0]) + (tile >= p.tiles_end[1]);
            const int t0 = wi == 0 ? 0 : p.tiles_end[wi - 1];
            float *dst = (p.out_alt[wi] && (b & 1)) ? p.out_alt[wi] : p.out[wi];
            const float *rsrc = red + ((size_t)par * NW + w_src) * (kRedCols * 16);
#pragma unroll
            for (int rr = 0; rr < RPW; rr++) {
                const int row = warp * RPW + rr;
                for (int mi = 0; mi < p.m; mi++) {
                    float v = 0.f;
#pragma unroll
                    for (int c0 = 0; c0 < 4; c0 += CSL) {
                        const int slot = c0 + cs;
                        if (slot < p.nl) v += rsrc[(mi * p.nl + slot) * 16 + row];
                        else if (FMT == TLB_GGML_Q4_K && slot == p.nl) v += rsrc[(8 + mi) * 16 + row];
                    }
                    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                    const int grow = (tile - t0) * 16 + row;
                    if (lane == 0 && grow < p.n_rows[wi]) atomicAdd(dst + (size_t)mi * p.n_rows[wi] + grow, v);
                }
            }
        }
        u = seg_end;
        tile++;
        par ^= 1;
    }
    STAMP(6);
    if (p.trace && tid == 0) p.trace[(size_t)b * 10 + 9] = (long long)global_ns();
#undef STAMP
}

// ---------------------------------------------------------------- host side

struct SmemPlan { int off_xq, off_alam, off_xsum, off_sa, off_minv, off_red, off_bars, off_misc, col_stride; size_t fixed; };

static SmemPlan plan_smem(int type, int m, int nl, int64_t k, int nw)
{
    // everything except the ring; offsets are relative to the end of the ring
    SmemPlan s;
    size_t o = 0;
    auto take = [&](size_t bytes) { size_t at = o; o += (bytes + 127) / 128 * 128; return (int)at; };
    s.col_stride = (int)k + 64;   // == 64 mod 128: two columns never share a bank group
    s.off_xq = take((size_t)m * nl * s.col_stride);
    s.off_alam = take((size_t)(k / 256) * kMaxCols * 4);
    s.off_xsum = take(type == TLB_GGML_Q4_K ? (size_t)2 * m * (k / 32) * 2 : 0);
    s.off_sa = take(type == TLB_GGML_Q6_K ? (size_t)(k / 256) * kMaxCols * 32 : type == TLB_GGML_Q4_0 ? (size_t)(k / 32) * kMaxCols * 4 : 0);
    s.off_minv = take(type == TLB_GGML_Q4_K ? (size_t)(k / 256) * 4 * 4 : 0);
    s.off_red = take((size_t)2 * nw * kRedCols * 16 * 4);
    s.off_misc = take((size_t)m * (k / 128) * 4 + sizeof(MvShared));
    s.off_bars = take(0);
    s.fixed = o;
    return s;
}

size_t qmatvec_max_k(int m)
{
    Context *c = ctx();
    size_t budget = c ? c->smem_optin : 232448;
    int nl = m <= 2 ? 3 : 2;
    size_t k = 256;
    while (plan_smem(TLB_GGML_Q6_K, m, nl, (int64_t)(k + 256), 16).fixed + 16 * (4352 + 128 + 16) <= budget) k += 256;
    return k;
}

template <int FMT, int NW>
static tlb_status launch_fmt(const MvParams &p, int grid, size_t smem, bool pdl)
{
    static size_t set_bytes = 0;
    if (smem > set_bytes) {
        TLB_CUDA(cudaFuncSetAttribute(qmatvec_kernel<FMT, NW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        set_bytes = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(NW * 32 + 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx()->stream;
    cudaLaunchAttribute at[2];
    int na = 0;
    if (pdl) {
        at[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[na].val.programmaticStreamSerializationAllowed = 1;
        na++;
    }
    static const bool debug = getenv("TLB_DEBUG") != nullptr;
    if (debug)
        fprintf(stderr, "[tlb] qmatvec fmt %d warps %d grid %d stages %d smem %zu k %d units %d\n", FMT, NW, grid,
                p.n_stages, smem, p.k, p.total_units);
    cfg.attrs = at;
    cfg.numAttrs = na;
    TLB_CUDA(cudaLaunchKernelEx(&cfg, qmatvec_kernel<FMT, NW>, p));
    count_launch();
    return TLB_OK;
}

tlb_status launch_qmatvec(const MatvecJob &job)
{
    Context *c = ctx();
    if (!c) return fail(TLB_ERR_DEVICE, "no device");
    const QFormat *f = qformat(job.type);
    if (!f) return fail(TLB_ERR_TYPE, "unsupported GGML type %d", job.type);
    if (job.m < 1 || job.m > 4) return fail(TLB_ERR_ARG, "matvec kernel takes 1..4 activation rows, got %d", job.m);
    if (job.k <= 0 || job.k % 256) return fail(TLB_ERR_SHAPE, "K = %lld must be a positive multiple of 256", (long long)job.k);
    if (job.n_w < 1 || job.n_w > 3) return fail(TLB_ERR_ARG, "1..3 weight tensors per launch");
    if (job.prologue != PRO_PLAIN && job.m != 1) return fail(TLB_ERR_ARG, "fused prologues take one activation row");
    MvParams p = {};
    int64_t tiles = 0;
    for (int i = 0; i < 3; i++) {
        if (i < job.n_w) {
            if (!job.w[i] || !job.out[i]) return fail(TLB_ERR_NULL, "null weight or output");
            tiles += job.n_tiles[i];
            p.w[i] = job.w[i];
            p.out[i] = job.out[i];
            p.out_alt[i] = job.out_alt[i];
            p.n_rows[i] = (int)job.n_rows[i];
        }
        p.tiles_end[i] = (int)tiles;
    }
    if (tiles == 0) return TLB_OK;
    p.n_w = job.n_w;
    p.upt = (int)(job.k / 256);
    p.k = (int)job.k;
    p.m = job.m;
    p.nl = job.m <= 2 ? 3 : 2;
    if (tiles * p.upt > INT32_MAX) return fail(TLB_ERR_SHAPE, "too many units for one launch");
    p.total_units = (int)(tiles * p.upt);
    p.unit_bytes = f->unit_bytes;
    p.stage_bytes = (f->unit_bytes + 127) / 128 * 128;
    // Two CTAs of 8 consumer warps per SM when shared memory allows a useful ring for each, else one of 16.
    const bool two_slots = job.out_alt[0] != nullptr;
    // CTAs: every CTA must own at least one tile's worth of units per accumulation slot, so that a
    // tile gets at most two contributions per slot (deterministic sums).
    const int64_t max_ctas = two_slots ? 2 * tiles : tiles;
    int nw = 8;
    size_t budget = (c->smem_optin + 1024) / 2 - 1024;   // per-CTA share when two CTAs are resident
    SmemPlan sp = plan_smem(job.type, job.m, p.nl, job.k, nw);
    if (job.force_warps == 16 || max_ctas < 2 * (int64_t)c->sm_count || sp.fixed + 12 * (size_t)(p.stage_bytes + 16) > budget) {
        nw = 16;
        budget = c->smem_optin;
        sp = plan_smem(job.type, job.m, p.nl, job.k, nw);
        if (sp.fixed + 16 * (size_t)(p.stage_bytes + 16) > budget)
            return fail(TLB_ERR_SHAPE, "K = %lld with %d rows needs more shared memory than one SM has (max K %zu)",
                        (long long)job.k, job.m, qmatvec_max_k(job.m));
    }
    int nst = (int)((budget - sp.fixed - 16) / (p.stage_bytes + 16));
    if (nst > 64) nst = 64;
    // A multiple of the consumer-warp count (itself a multiple of kProducerLanes): a stage is then
    // always consumed by the same warp and armed by the same producer lane, so a parity wait can
    // never be satisfied by a phase two uses back.
    nst = nst / nw * nw;
    p.n_stages = nst;
    const size_t ring = (size_t)nst * p.stage_bytes;
    p.off_xq = (int)ring + sp.off_xq; p.off_alam = (int)ring + sp.off_alam; p.off_xsum = (int)ring + sp.off_xsum;
    p.off_sa = (int)ring + sp.off_sa; p.off_minv = (int)ring + sp.off_minv; p.off_red = (int)ring + sp.off_red;
    p.off_misc = (int)ring + sp.off_misc;
    p.off_bars = (int)ring + sp.off_bars;
    p.col_stride = sp.col_stride;
    const size_t smem = ring + sp.fixed + (size_t)nst * 16 + 16;   // ring barriers + the image-copy barrier
    if ((size_t)(sp.off_red - sp.off_xq) > c->act_bytes)
        return fail(TLB_ERR_SHAPE, "activation image of %d bytes exceeds the %zu-byte scratch", sp.off_red - sp.off_xq, c->act_bytes);
    p.act_img = c->act_img;
    p.grid_sync = c->grid_sync;
    p.prologue = job.prologue;
    p.x = job.x; p.x2 = job.x2; p.x3 = job.x3; p.norm_w = job.norm_w; p.eps = job.eps; p.x_out = job.x_out;
    p.emb_table = job.emb_table; p.token = job.token;
    for (int z = 0; z < 3; z++) { p.zero_ptr[z] = job.zero_ptr[z]; p.zero_n[z] = job.zero_n[z]; }
    p.err = c->err_flag;
    p.use_pdl = job.pdl ? 1 : 0;
    p.trace = job.trace;
    if (!p.x && !(p.prologue == PRO_ADD_NORM && p.token)) return fail(TLB_ERR_NULL, "null activation");
    const int grid = (int)std::min<int64_t>((int64_t)c->sm_count * (nw == 8 ? 2 : 1), max_ctas);
#define LAUNCH(FMTV)                                                                  \
    return nw == 8 ? launch_fmt<FMTV, 8>(p, grid, smem, job.pdl) : launch_fmt<FMTV, 16>(p, grid, smem, job.pdl)
    switch (job.type) {
    case TLB_GGML_Q4_K: LAUNCH(TLB_GGML_Q4_K);
    case TLB_GGML_Q6_K: LAUNCH(TLB_GGML_Q6_K);
    case TLB_GGML_Q8_0: LAUNCH(TLB_GGML_Q8_0);
    default: LAUNCH(TLB_GGML_Q4_0);
    }
#undef LAUNCH
}

}  // namespace tlb

using namespace tlb;

extern "C" tlb_status tlb_qtensor_matmul(tlb_tensor **out, const tlb_tensor *x, const tlb_qtensor *w)
{
    if (!out) return fail(TLB_ERR_NULL, "null out");
    *out = nullptr;
    if (!x || !w) return fail(TLB_ERR_NULL, "tl_qtensor_matmul received null argument");
    if (x->dt != TLB_F32) return fail(TLB_ERR_TYPE, "activation must be f32");
    if (x->rank < 1) return fail(TLB_ERR_SHAPE, "activation must have rank >= 1");
    int64_t k = x->shape[x->rank - 1];
    if (k != w->k) return fail(TLB_ERR_SHAPE, "Matmul shape mismatch: x inner dim %lld vs weight K %lld", (long long)k, (long long)w->k);
    int64_t m = k ? x->numel() / k : 0;
    int64_t oshape[kMaxRank];
    for (int i = 0; i < x->rank - 1; i++) oshape[i] = x->shape[i];
    oshape[x->rank - 1] = w->n;
    TLB_TRY(new_tensor(out, TLB_F32, oshape, x->rank));
    if (m * w->n == 0) return TLB_OK;
    tlb_status st = TLB_OK;
    cudaError_t e = cudaMemsetAsync((*out)->data(), 0, (size_t)m * w->n * 4, ctx()->stream);
    if (e != cudaSuccess) st = cuda_fail(e, "memset");
    for (int64_t m0 = 0; m0 < m && st == TLB_OK; m0 += 4) {   // the weight stream is repeated per group of 4 rows
        MatvecJob job;
        job.n_w = 1;
        job.w[0] = w->dev();
        job.n_tiles[0] = w->n_tiles;
        job.n_rows[0] = w->n;
        job.out[0] = (*out)->f32() + m0 * w->n;
        job.type = w->type;
        job.k = k;
        job.m = (int)std::min<int64_t>(4, m - m0);
        job.x = x->f32() + m0 * k;
        st = launch_qmatvec(job);
    }
    if (st != TLB_OK) { tlb_tensor_release(*out); *out = nullptr; }
    return st;
}
