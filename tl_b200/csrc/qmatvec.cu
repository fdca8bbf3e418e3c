// Streaming dequant-fused matvec for GGUF Q4_K / Q6_K / Q8_0 / Q4_0 weights (decode path,
// 1..4 activation rows).  Replaces mul_mv_q4_k_kernel / mul_mv_q6_k_kernel
// (crates/tl_cuda/src/cuda_kernels/autograd.cu:2813-2900: one thread per output, byte loads, weights
// re-read once per activation row) and the dequantise-then-naive-matmul route the reference takes
// for Q4_0 / Q8_0 (crates/tl_runtime/src/system.rs:236-264).
//
// Shape of the kernel (one persistent CTA of 16 warps per SM, the whole register file at 128 per thread;
// a variant of two 8-warp CTAs that leaves room for a CTA of the next kernel measured 35 % slower
// per step: at 80 registers the unit loop no longer keeps its shared loads in flight):
//   * work is cut into ITEMS: one tile of 16 output rows x one K-slice of `upi` consecutive units
//     (a unit = 16 rows x 256 weights, quant.cu).  Items are numbered slice-major and dealt out in
//     contiguous ranges, first to CTAs and then to the warps of a CTA, so every warp gets the same
//     number of bytes to within one item;
//   * a warp owns its items from the first byte to the stored result.  It streams their units
//     global -> shared itself with 1-D bulk async copies (cp.async.bulk + mbarrier complete_tx) through
//     a ring of stages that belongs to it alone: after consuming a stage the warp refills it with the
//     unit `spw` positions ahead.  No other warp is ever waited for - there is no block-wide barrier,
//     no shared-memory reduction and no atomic in the streaming phase;
//   * the copies do not depend on the activations, so the first `spw` are issued before the kernel
//     waits for its predecessor (programmatic dependent launch);
//   * the prologue quantises the activation to int8 levels in shared memory (qmv_prologue.cuh) -
//     only the 256-blocks the CTA's K-slices cover - and can fuse what precedes the matvec in the
//     decode chain: residual add + RMSNorm * weight, SiLU(gate) * up, or the embedding lookup;
//   * per unit: conflict-free 128-bit shared loads, one AND per four weights, integer tensor-core
//     MMAs (qmv_units.cuh);
//   * the 16 * m partial results of item (slice, tile) are written - not added - to a scratch slot of
//     their own; the warp that finishes the last slice of a tile (a per-tile counter tells) adds the
//     slices in index order and writes the output rows.  Nothing is accumulated atomically and nothing
//     has to be cleared beforehand, so results do not depend on scheduling;
//   * with a single K-slice ("local" mode, chosen for launches with many units per warp such as
//     gate|up and the head) a CTA's units are cut evenly over its warps whatever the tile borders, and
//     the pieces of each tile are added - in warp order - in shared memory after one block barrier:
//     no global scratch, fence or counter at all;
//   * finishing a tile can fuse what follows the matvec in the decode chain: the residual add with
//     per-tile sums of squares for the next RMSNorm, or SiLU(gate) * up over interleaved gate|up rows;
//   * a host-side cost model (slice_cost) picks the number of K-slices per launch shape.
#include "qmv_prologue.cuh"
#include "qmv_units.cuh"

#include <algorithm>

namespace tlb {

constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
constexpr int kCtasPerSm = 1;       // CTAs a launch brings per SM
constexpr int kResidentPerSm = 1;   // CTAs the register and shared-memory budgets allow per SM

struct ItemRef {
    const uint8_t *src;   // first unit of the item
    int wi, row0, slice;  // tensor, first output row within the tensor, K-slice
    int tile;             // tile index within the launch
};

// Position in the slice-major item order, advanced without divisions.
struct ItemCursor { int slice, tile; };

__device__ __forceinline__ ItemCursor cursor_at(const MvParams &p, int item)
{
    ItemCursor c;
    c.slice = item / p.tiles;
    c.tile = item - c.slice * p.tiles;
    return c;
}
__device__ __forceinline__ void cursor_next(const MvParams &p, ItemCursor &c)
{
    if (++c.tile == p.tiles) { c.tile = 0; c.slice++; }
}
__device__ __forceinline__ ItemRef item_ref(const MvParams &p, const ItemCursor &c)
{
    ItemRef r;
    r.slice = c.slice;
    r.tile = c.tile;
    r.wi = (c.tile >= p.tiles_end[0]) + (c.tile >= p.tiles_end[1]);
    const int t0 = r.wi == 0 ? 0 : p.tiles_end[r.wi - 1];
    r.row0 = (c.tile - t0) * 16;
    r.src = p.w[r.wi] + ((size_t)(c.tile - t0) * p.upt + (size_t)c.slice * p.upi) * p.unit_bytes;
    return r;
}

// The fused ways of finishing a tile (one activation row, one tensor).  Lane e < 16 holds the
// result y of row e of the tile; all 32 lanes call.
//   FIN_RESID  out[row] = resid[row] + y; the squares of the 16 sums, added in a fixed tree, go to
//              ssq_out[tile]: the next RMSNorm adds the tiles instead of re-reading the row
//              (crates/tl_cpu/src/ffi.rs:2444-2486 sums the squares of the whole row).
//   FIN_SILU   rows 0..7 are gate and rows 8..15 up of hidden units 8*tile .. 8*tile+7:
//              out[8*tile + e] = silu(gate) * up (crates/tl_cpu/src/ffi.rs:2083-2103 then an elementwise mul).
// `res` is the residual of row e, loaded by the caller (so that it can be in flight with other loads).
__device__ __forceinline__ void finish_tile_fused(const MvParams &p, const ItemRef &fr, float y, float res, int lane)
{
    float *out = p.out[0];
    const int nrows = p.n_rows[0];
    if (p.finish == FIN_RESID) {
        const int g = fr.row0 + lane;
        const bool valid = lane < 16 && g < nrows;
        const float xn = valid ? res + y : 0.f;
        if (valid) out[g] = xn;
        float s = xn * xn;
        s += __shfl_xor_sync(0xffffffffu, s, 8);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        if (lane == 0) p.ssq_out[fr.tile] = s;
    } else {   // FIN_SILU
        const float up = __shfl_down_sync(0xffffffffu, y, 8);
        const int h = fr.tile * 8 + lane;
        if (lane < 8 && 2 * h < nrows) out[h] = silu_f(y) * up;
    }
}

// ---- sum over tensor-parallel ranks, tile by tile (TpFuse).  Lane e < 16 holds row e of the tile; all 32 lanes call.
// Every value travels as one 8-byte word {value, sequence number}: an aligned 8-byte store is indivisible, so a
// reader that finds the sequence number it waits for has the value with it - no fence and no separate flag.
__device__ __forceinline__ void tp_push_tile(const MvParams &p, unsigned seq, int row0, int nrows, float y, int lane)
{
    const int g = row0 + lane;
    if (lane < 16 && g < nrows) {
        const size_t at = (size_t)(seq & 1u) * p.tp.buf_stride + g;
        const unsigned long long word = ((unsigned long long)seq << 32) | __float_as_uint(y);
        for (int r = 0; r < p.tp.size; r++)        // 128 consecutive bytes per rank, own memory included
            asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(p.tp.peer_ll[r] + at), "l"(word) : "memory");
    }
}
// The ranks' values of the tile from this GPU's own memory, added in rank order (the same sum on every rank).  Waits,
// bounded (about a second), for words that have not arrived; *ok turns false if one never does.
__device__ __forceinline__ float tp_sum_tile(const MvParams &p, unsigned seq, int row0, int nrows, int lane, bool *ok)
{
    const int g = row0 + lane;
    float a = 0.f;
    bool got = true;
    if (lane < 16 && g < nrows) {
        const unsigned long long *v = p.tp.mine_ll + (size_t)(seq & 1u) * p.tp.buf_stride + g;
        for (int r = 0; r < p.tp.size && got; r++) {
            unsigned long long word, t0 = 0;
            for (unsigned it = 0;; it++) {
                asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(word) : "l"(v + (size_t)r * p.tp.rank_stride) : "memory");
                if ((unsigned)(word >> 32) == seq) break;
                if ((it & 255) == 255) {
                    const unsigned long long t = global_ns();
                    if (!t0) t0 = t;
                    if (t - t0 > 1000000000ull) { got = false; break; }
                }
            }
            a += __uint_as_float((unsigned)word);
        }
    }
    if (!__all_sync(0xffffffffu, got)) *ok = false;
    return a;
}

template <int FMT>
__global__ void __launch_bounds__(kThreads, kResidentPerSm) qmatvec_kernel(const __grid_constant__ MvParams p)
{
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    MvShared *sh = reinterpret_cast<MvShared *>(smem + p.off_misc);
    const int spw = p.spw;
    const uint32_t ring = smem_u32(smem) + (uint32_t)(warp * spw) * p.stage_bytes;   // this warp's stages
    const uint32_t bars = smem_u32(smem + p.off_bars) + (uint32_t)(warp * spw) * 8;  // and their barriers
    const int b = blockIdx.x;

    // Work of this CTA: a contiguous range of items.  Work of this warp: a contiguous range [wu0, wu1) of
    // the CTA's units in item order.  With K-slices (kb > 1) the ranges are whole items; with one
    // slice (kb == 1, an item is a whole tile) they are cut to equal unit counts, may start and end
    // inside a tile, and the pieces of a tile meet in shared memory at the end ("local" mode).
    const int ci0 = b * p.ipc_q + min(b, p.ipc_r), nci = p.ipc_q + (b < p.ipc_r ? 1 : 0), ci1 = ci0 + nci;
    const bool local = p.kb == 1;
    const int cta_units = nci * p.upi;
    const int wu0 = local ? cta_units * warp / kWarps : (nci * warp / kWarps) * p.upi;
    const int wu1 = local ? cta_units * (warp + 1) / kWarps : (nci * (warp + 1) / kWarps) * p.upi;
    const int n_units = wu1 - wu0;
    // activation blocks the CTA's items cover
    const int s_first = nci > 0 ? ci0 / p.tiles : 0, s_last = nci > 0 ? (ci1 - 1) / p.tiles : 0;
    const int blk0 = s_first * p.upi, nb = nci > 0 ? (s_last + 1) * p.upi - blk0 : 0;

    // Ring set-up, one lane per stage so that it takes one round of latencies instead of `spw`:
    // lane s initialises the barrier of stage s and requests the warp's unit s.
    // Only the first kEarly units are requested before the prologue: the activation loads of the
    // prologue share the SM's path from L2 with these copies and would otherwise queue behind a whole
    // ring of weights.  The rest of the ring is requested once the activation values have arrived.
    constexpr int kEarly = 2;
    const int n_first = min(spw, n_units);
    const uint8_t *first_src = nullptr;
    if (lane < spw) {
        mbar_init(bars + lane * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        if (lane < n_first) {
            const int g = wu0 + lane, it = g / p.upi, uo = g - it * p.upi;
            first_src = item_ref(p, cursor_at(p, ci0 + it)).src + (size_t)uo * p.unit_bytes;
            if (lane < kEarly) {
                mbar_expect_tx(bars + lane * 8, p.unit_bytes);
                bulk_g2s(ring + lane * p.stage_bytes, first_src, p.unit_bytes, bars + lane * 8);
            }
        }
    }
    if (tid == 0) sh->abort_flag = 0;
    __syncwarp();

    // Copy cursor (used by lane 0 only): the next unit to request and how many remain.
    int pf_left_in_item = 0, pf_remaining = n_units - n_first, issued = n_first;
    const uint8_t *pf_src = nullptr;
    ItemCursor pf_cur;
    {
        const int g = wu0 + n_first, it = g / p.upi, uo = g - it * p.upi;
        pf_cur = cursor_at(p, ci0 + it);
        if (uo && pf_remaining > 0) {   // in the middle of an item
            pf_src = item_ref(p, pf_cur).src + (size_t)uo * p.unit_bytes;
            cursor_next(p, pf_cur);
            pf_left_in_item = p.upi - uo;
        }
    }
    auto issue_copy = [&](int stage) {
        if (pf_left_in_item == 0) { pf_src = item_ref(p, pf_cur).src; cursor_next(p, pf_cur); pf_left_in_item = p.upi; }
        mbar_expect_tx(bars + stage * 8, p.unit_bytes);
        bulk_g2s(ring + stage * p.stage_bytes, pf_src, p.unit_bytes, bars + stage * 8);
        pf_src += p.unit_bytes;
        pf_left_in_item--; pf_remaining--; issued++;
    };

    float4 wgt_first[kKeep];       // static inputs of the prologue, fetched while the previous kernel finishes
    load_norm_weights(p, tid, kThreads, blk0, nb, wgt_first);
    if (p.use_pdl) {
        pdl_wait();                // everything below may read what the previous kernel wrote
        // Released only after our own wait: a dependent's early part then runs with every kernel
        // before our predecessor complete, so it may read state those kernels wrote.
        pdl_launch_dependents();
    }
    const unsigned tp_seq = p.tp_reduce ? ld_volatile_u32(p.tp.seq) : 0u;   // the launch before has completed: its exchange is over
    __syncthreads();               // abort_flag initialised; also keeps the CTA together for the prologue
    build_activation<FMT>(p, sh, smem, tid, kThreads, blk0, nb, wgt_first, [&](float dep) {
        // the rest of the ring's first round; the test on `dep` only ties the requests to the arrival of the loads
        if (lane >= kEarly && lane < n_first && __float_as_uint(dep) != 0x7fedcba9u) {
            mbar_expect_tx(bars + lane * 8, p.unit_bytes);
            bulk_g2s(ring + lane * p.stage_bytes, first_src, p.unit_bytes, bars + lane * 8);
        }
    });
    volatile int *abortp = &sh->abort_flag;

    const int ncols = p.m * p.nl;
    LaneCtx L;
    L.lane = lane; L.r = lane >> 2; L.c = lane & 3;
    {
        const int r = L.r, c = L.c;
        const int colr = r < ncols ? r : 0, c0 = 2 * c < ncols ? 2 * c : 0, c1 = 2 * c + 1 < ncols ? 2 * c + 1 : 0;
        L.xq_b = smem_u32(smem + p.off_xq) + colr * p.col_stride;
        L.alam_b = smem_u32(smem + p.off_alam) + 2 * c * 4;
        L.xsum_b = smem_u32(smem + p.off_xsum) + ((r < 2 * p.m) ? r : (r & 1)) * (p.nb_max * 8) * 2;
        L.sa_b = smem_u32(smem + p.off_sa) + colr * 32;
        L.sa_c0 = smem_u32(smem + p.off_sa) + c0 * 4;
        L.sa_c1 = smem_u32(smem + p.off_sa) + c1 * 4;
        L.minv_b = smem_u32(smem + p.off_minv) + (c < p.m ? c : 0) * 4;
    }
    float *segbuf = reinterpret_cast<float *>(smem + p.off_seg);   // local mode: [warp][run][16 * m] partial results

    int stage = 0, phase = 0, consumed = 0;
    bool ok = true;
    int remaining = n_units, seg = 0;
    const int it0 = wu0 / p.upi;
    int uo0 = wu0 - it0 * p.upi;          // the first run may start inside an item (local mode)
    ItemCursor cur = cursor_at(p, ci0 + it0);
    while (remaining > 0 && ok) {
        const ItemRef ir = item_ref(p, cur);
        const int run = min(remaining, p.upi - uo0);
        const int lb0 = ir.slice * p.upi + uo0 - blk0;
        float master[4] = {0.f, 0.f, 0.f, 0.f}, mm[4] = {0.f, 0.f, 0.f, 0.f};
        int uo = 0;
        // two units per trip: the two bodies are independent, so one warp has two instruction streams
        // to interleave, and the loop bookkeeping is paid once
        for (; uo + 1 < run; uo += 2) {
            const int st1 = stage + 1 == spw ? 0 : stage + 1, ph1 = stage + 1 == spw ? phase ^ 1 : phase;
            bool got = mbar_try_wait(bars + stage * 8, phase);
            if (!got) got = mbar_wait_slow(bars + stage * 8, phase, abortp, p.err, 2);
            bool got1 = mbar_try_wait(bars + st1 * 8, ph1);
            if (!got1) got1 = mbar_wait_slow(bars + st1 * 8, ph1, abortp, p.err, 2);
            if (!__all_sync(0xffffffffu, got && got1)) { ok = false; break; }   // warp-uniform: all lanes leave together
            process_unit<FMT>(ring + stage * p.stage_bytes, lb0 + uo, L, master, mm);
            process_unit<FMT>(ring + st1 * p.stage_bytes, lb0 + uo + 1, L, master, mm);
            consumed += 2;
            __syncwarp();          // every lane has read the stages: they may be overwritten
            if (lane == 0) {
                if (pf_remaining > 0) issue_copy(stage);
                if (pf_remaining > 0) issue_copy(st1);
            }
            stage = st1 + 1 == spw ? 0 : st1 + 1;
            phase = st1 + 1 == spw ? ph1 ^ 1 : ph1;
        }
        if (ok && uo < run) {
            bool got = mbar_try_wait(bars + stage * 8, phase);
            if (!got) got = mbar_wait_slow(bars + stage * 8, phase, abortp, p.err, 2);
            if (!__all_sync(0xffffffffu, got)) ok = false;
            else {
                process_unit<FMT>(ring + stage * p.stage_bytes, lb0 + uo, L, master, mm);
                consumed++;
                __syncwarp();
                if (lane == 0 && pf_remaining > 0) issue_copy(stage);
                if (++stage == spw) { stage = 0; phase ^= 1; }
            }
        }
        if (!ok) break;
        // Fold the level columns of each activation row (they sit in the four lanes of a quad).  The
        // Q4_K min term of activation row mi lives in lane c == mi.  The 16 * m partial results of the run
        // go to this warp's slot in shared memory (local mode) or to the item's slot of the slice scratch.
        float *part = local ? segbuf + ((size_t)warp * p.max_seg + seg) * (16 * p.m)
                            : p.part + ((size_t)ir.slice * p.tiles + ir.tile) * (16 * p.m);
        for (int mi = 0; mi < p.m; mi++) {
            const int lo = mi * p.nl, hi = lo + p.nl, cA = 2 * L.c, cB = 2 * L.c + 1;
            const bool inA = cA >= lo && cA < hi, inB = cB >= lo && cB < hi;
            float v0 = (inA ? master[0] : 0.f) + (inB ? master[1] : 0.f);   // row r
            float v1 = (inA ? master[2] : 0.f) + (inB ? master[3] : 0.f);   // row r + 8
            v0 += __shfl_xor_sync(0xffffffffu, v0, 1); v0 += __shfl_xor_sync(0xffffffffu, v0, 2);
            v1 += __shfl_xor_sync(0xffffffffu, v1, 1); v1 += __shfl_xor_sync(0xffffffffu, v1, 2);
            if (L.c == mi) {
                if (FMT == TLB_GGML_Q4_K) { v0 -= mm[0] + mm[1]; v1 -= mm[2] + mm[3]; }
                part[mi * 16 + L.r] = v0;
                part[mi * 16 + L.r + 8] = v1;
            }
        }
        seg++;
        remaining -= run;
        uo0 = 0;
        cursor_next(p, cur);
    }
    const bool tpr = p.tp_reduce != 0;
    int tp_finished = 0;                               // tiles this warp has completed over the ranks
    bool tp_ok = true;
    // what a finished tile's 16 sums (lane e < 16: row e) turn into
    auto finish_rows = [&](const ItemRef &fr, float y) {
        if (p.finish == FIN_PLAIN) {
            const int g = fr.row0 + lane;
            if (lane < 16 && g < p.n_rows[fr.wi]) p.out[fr.wi][g] = y;
        } else {
            const float res = (p.finish == FIN_RESID && lane < 16 && fr.row0 + lane < p.n_rows[0]) ? __ldcg(p.resid + fr.row0 + lane) : 0.f;
            finish_tile_fused(p, fr, lane < 16 ? y : 0.f, res, lane);
        }
    };
    if (local) {
        // The pieces of every tile of this CTA are in shared memory.  Tile t (CTA-local) is finished by
        // warp t % kWarps: it adds the pieces in the order of the warps that produced them - a fixed
        // order - and writes the rows.  No global scratch, fence or counter is involved.
        __syncthreads();           // every warp gets here: its waits are bounded
        if (!*abortp) {
            for (int tl = warp; tl < nci; tl += kWarps) {
                const int a0 = tl * p.upi, a1 = a0 + p.upi;
                float acc0 = 0.f, acc1 = 0.f;   // elements lane and lane + 32 of the 16 * m results
                for (int w = 0; w < kWarps; w++) {
                    const int b0 = cta_units * w / kWarps, b1 = cta_units * (w + 1) / kWarps;
                    if (b1 <= a0 || b0 >= a1 || b1 == b0) continue;
                    const float *sp = segbuf + ((size_t)w * p.max_seg + (tl - b0 / p.upi)) * (16 * p.m);
                    if (lane < 16 * p.m) acc0 += sp[lane];
                    if (lane + 32 < 16 * p.m) acc1 += sp[lane + 32];
                }
                ItemCursor cf;
                cf.slice = 0;
                cf.tile = ci0 + tl;
                const ItemRef fr = item_ref(p, cf);
                if (tpr) {
                    tp_push_tile(p, tp_seq, fr.row0, p.n_rows[0], acc0, lane);
                } else if (p.finish == FIN_PLAIN) {
                    float *out = p.out[fr.wi];
                    const int nrows = p.n_rows[fr.wi];
                    const int g = fr.row0 + (lane & 15);
                    if (lane < 16 * p.m && g < nrows) out[(size_t)(lane >> 4) * nrows + g] = acc0;
                    if (lane + 32 < 16 * p.m && g < nrows) out[(size_t)((lane >> 4) + 2) * nrows + g] = acc1;
                } else {
                    finish_rows(fr, acc0);
                }
            }
            if (tpr) {
                // the warp's tiles are on their way to every rank; now the other ranks' shares of them
                for (int tl = warp; tl < nci; tl += kWarps) {
                    ItemCursor cf;
                    cf.slice = 0;
                    cf.tile = ci0 + tl;
                    const ItemRef fr = item_ref(p, cf);
                    finish_rows(fr, tp_sum_tile(p, tp_seq, fr.row0, p.n_rows[0], lane, &tp_ok));
                    tp_finished++;
                }
            }
        }
    } else if (ok && wu1 > wu0 && p.fold_poll) {
        // One activation row.  The slice scratch rests at kFoldEmpty between launches, so a value that is not kFoldEmpty is
        // a slice that has arrived: the warp that owns slice 0 of a tile reads the tile's slices (all requested at once,
        // re-read while some are missing; bounded), adds them in slice order, puts kFoldEmpty back and writes the rows.
        // No fence, counter or atomic: a 4-byte store is indivisible, and the next launch starts after this one is over.
        const int i0 = ci0 + it0, i1 = ci0 + wu1 / p.upi;
        const size_t sstride = (size_t)p.tiles * 16;
        for (int item = i0; item < i1 && item < p.tiles; item++) {     // items below `tiles` are slice 0
            ItemCursor cf;
            cf.slice = 0;
            cf.tile = item;
            const ItemRef fr = item_ref(p, cf);
            float *src = p.part + (size_t)fr.tile * 16 + (lane & 15);
            unsigned sl[kMaxSlices];
            bool got = true;
            if (lane < 16) {
#pragma unroll
                for (int s = 0; s < kMaxSlices; s++) sl[s] = s < p.kb ? ld_volatile_u32(reinterpret_cast<const unsigned *>(src + s * sstride)) : 0u;
                unsigned long long t0 = 0;
                for (unsigned it = 0;; it++) {
                    bool all = true;
#pragma unroll
                    for (int s = 0; s < kMaxSlices; s++)
                        if (s < p.kb && sl[s] == kFoldEmpty) {
                            sl[s] = ld_volatile_u32(reinterpret_cast<const unsigned *>(src + s * sstride));
                            all = all && sl[s] != kFoldEmpty;
                        }
                    if (all) break;
                    if ((it & 255) == 255) {
                        const unsigned long long t = global_ns();
                        if (!t0) t0 = t;
                        if (t - t0 > 1000000000ull) { got = false; break; }
                    }
                }
            }
            if (!__all_sync(0xffffffffu, got)) { if (lane == 0) atomicExch(p.err, 3); break; }
            float a = 0.f;
            if (lane < 16) {
                a = __uint_as_float(sl[0]);
#pragma unroll
                for (int s = 1; s < kMaxSlices; s++) a += s < p.kb ? __uint_as_float(sl[s]) : 0.f;
#pragma unroll
                for (int s = 0; s < kMaxSlices; s++)
                    if (s < p.kb) reinterpret_cast<unsigned *>(src + s * sstride)[0] = kFoldEmpty;
            }
            if (tpr) {
                tp_push_tile(p, tp_seq, fr.row0, p.n_rows[0], a, lane);
                finish_rows(fr, tp_sum_tile(p, tp_seq, fr.row0, p.n_rows[0], lane, &tp_ok));
                tp_finished++;
            } else {
                finish_rows(fr, a);
            }
        }
    } else if (ok && wu1 > wu0) {
        // All partial results of this warp are out.  One fence, then one count per item (lane j counts
        // item j); the warp that completes a tile's last K-slice adds the slices in index order and
        // writes the output rows, so the sum is the same whichever warp does it.  It also clears the
        // tile's counter for the next launch on this stream.
        const int i0 = ci0 + it0, i1 = ci0 + wu1 / p.upi;
        __threadfence();                                      // our slices are visible before the counts say so
        __syncwarp();
        for (int base = i0; base < i1; base += 32) {
            const int mine = base + lane;
            ItemCursor cj = cursor_at(p, mine < i1 ? mine : base);
            bool last = false;
            if (mine < i1) last = atomicAdd(p.tile_cnt + cj.tile, 1) == p.kb - 1;
            const unsigned lasts = __ballot_sync(0xffffffffu, last);
            if (lasts) __threadfence();                       // the other slices are visible once their counts are
            for (unsigned rest = lasts; rest; rest &= rest - 1) {
                const int j = __ffs(rest) - 1;
                ItemCursor cf;
                cf.slice = 0;
                cf.tile = __shfl_sync(0xffffffffu, cj.tile, j);
                const ItemRef fr = item_ref(p, cf);
                float *out = p.out[fr.wi];
                const int nrows = p.n_rows[fr.wi];
                const float *src = p.part + (size_t)fr.tile * (16 * p.m);
                const size_t sstride = (size_t)p.tiles * (16 * p.m);
                if (p.finish == FIN_PLAIN && !tpr) {
                    for (int e = lane; e < 16 * p.m; e += 32) {
                        float a = __ldcg(src + e);
                        for (int s = 1; s < p.kb; s++) a += __ldcg(src + s * sstride + e);
                        const int mi = e >> 4, g = fr.row0 + (e & 15);
                        if (g < nrows) out[(size_t)mi * nrows + g] = a;
                    }
                } else {   // m == 1: all slices are requested at once, then added in slice order
                    float sl[kMaxSlices];
#pragma unroll
                    for (int s = 0; s < kMaxSlices; s++) sl[s] = (lane < 16 && s < p.kb) ? __ldcg(src + s * sstride + lane) : 0.f;
                    float a = sl[0];
#pragma unroll
                    for (int s = 1; s < kMaxSlices; s++) a += sl[s];
                    if (tpr) tp_push_tile(p, tp_seq, fr.row0, nrows, a, lane);
                    else finish_rows(fr, a);
                }
                if (lane == 0) p.tile_cnt[fr.tile] = 0;
            }
            if (tpr && lasts) {
                for (unsigned rest = lasts; rest; rest &= rest - 1) {
                    ItemCursor cf;
                    cf.slice = 0;
                    cf.tile = __shfl_sync(0xffffffffu, cj.tile, __ffs(rest) - 1);
                    const ItemRef fr = item_ref(p, cf);
                    finish_rows(fr, tp_sum_tile(p, tp_seq, fr.row0, p.n_rows[0], lane, &tp_ok));
                    tp_finished++;
                }
            }
        }
    }
    if (tpr && tp_finished && lane == 0) {
        // the warp that completes the launch's last tile moves on to the next sequence number (every warp read this one
        // when it started)
        if (!tp_ok) atomicExch(p.err, 32);
        if (atomicAdd(p.tp.done, tp_finished) + tp_finished == p.tiles) {
            *p.tp.done = 0;
            *p.tp.seq = tp_seq + 1;
        }
    }
    if (!ok && lane == 0) {
        // a bounded wait gave up (error word set): give the copies still in flight a bounded time to land
        for (int q = consumed; q < issued; q++) mbar_wait_drain(bars + (q % spw) * 8, (q / spw) & 1);
    }
}

// ---------------------------------------------------------------- host side

struct SmemPlan { int off_xq, off_alam, off_xsum, off_sa, off_minv, off_misc, col_stride; size_t fixed; };

static SmemPlan plan_smem(int type, int m, int nl, int nb)
{
    // everything except the ring and its barriers; offsets are relative to the end of the ring
    SmemPlan s;
    size_t o = 0;
    auto take = [&](size_t bytes) { size_t at = o; o += (bytes + 127) / 128 * 128; return (int)at; };
    s.col_stride = nb * 256 + 64;   // == 64 mod 128: two neighbouring columns never share a bank group
    s.off_xq = take((size_t)m * nl * s.col_stride);
    s.off_alam = take((size_t)nb * kMaxCols * 4);
    s.off_xsum = take(type == TLB_GGML_Q4_K ? (size_t)2 * m * (nb * 8) * 2 : 0);
    s.off_sa = take(type == TLB_GGML_Q6_K ? (size_t)nb * kMaxCols * 32 : type == TLB_GGML_Q4_0 ? (size_t)(nb * 8) * kMaxCols * 4 : 0);
    s.off_minv = take(type == TLB_GGML_Q4_K ? (size_t)nb * 4 * 4 : 0);
    s.off_misc = take(sizeof(MvShared));
    s.fixed = o;
    return s;
}

static int stage_bytes_of(const QFormat *f) { return (f->unit_bytes + 127) / 128 * 128; }

size_t qmatvec_max_k(int m)
{
    // the unsplit worst case: all blocks of K resident with two ring stages per warp
    Context *c = ctx();
    size_t budget = c ? c->smem_optin : 232448;
    int nl = m <= 2 ? 3 : 2;
    size_t k = 256;
    while (plan_smem(TLB_GGML_Q6_K, m, nl, (int)(k / 256) + 1).fixed + (size_t)kWarps * 2 * (4352 + 8) + 128 <= budget) k += 256;
    return k;
}

// Blocks of 256 a CTA may have to quantise when `n_items` slice-major items are dealt to `grid` CTAs.
static int blocks_per_cta(int64_t n_items, int grid, int64_t tiles, int upi, int upt)
{
    const int64_t ipc = (n_items + grid - 1) / grid;
    const int64_t touched = (ipc + tiles - 2) / tiles + 1;   // a range of ipc items straddles at most this many slices
    return (int)std::min<int64_t>(upt, touched * upi);
}

// Relative cost (warp instructions on the critical path) of cutting K into upt / upi slices.
static double slice_cost(int type, int m, int64_t tiles, int upt, int upi, int sm_count)
{
    const int kb = upt / upi;
    const int64_t n_items = tiles * kb;
    const int grid = (int)std::min<int64_t>((int64_t)sm_count * kCtasPerSm, n_items);
    const int64_t ipc = (n_items + grid - 1) / grid, ipw = (ipc + kWarps - 1) / kWarps;
    const int nb = blocks_per_cta(n_items, grid, tiles, upi, upt);
    const double unit = type == TLB_GGML_Q6_K ? 300.0 : type == TLB_GGML_Q8_0 ? 150.0 : 210.0;
    // one slice: the CTA's units are cut evenly over its warps whatever the tile borders
    const double stream = kb == 1 ? (double)((ipc * upi + kWarps - 1) / kWarps) * unit + 60.0 * ((ipc + kWarps - 1) / kWarps + 1)
                                  : (double)ipw * (upi * unit + 60.0);
    const double quant = 300.0 * ((m * nb + kThreads / 64 - 1) / (kThreads / 64));
    // Measured on the Llama-3-8B shapes: the end of a sliced launch (fence, counts, reading the slices back)
    // costs ~3 us; assembling tiles in shared memory costs a block barrier, which shows (~2 us of waiting
    // for the slowest warp) only when warps have so few units that their skew matters.
    const bool few = (ipc * upi + kWarps - 1) / kWarps < 4;
    const double fold = kb > 1 ? 600.0 + 16.0 * kb : (few ? 600.0 : 100.0);
    return stream + quant + fold;
}

int qmatvec_plan_slices(int type, int64_t k, int m, int64_t tiles, int max_slices)
{
    Context *c = ctx();
    const int sm = c ? c->sm_count : 148;
    const int upt = (int)(k / 256);
    if (upt < 1 || tiles < 1) return 1;
    max_slices = std::max(1, std::min(max_slices, kMaxSlices));
    int best = 1;
    double best_cost = 0.0;
    for (int upi = upt; upi >= 1; upi--) {
        if (upt % upi) continue;
        const int kb = upt / upi;
        if (kb > max_slices) break;
        const double cost = slice_cost(type, m, tiles, upt, upi, sm);
        if (kb == 1 || cost < best_cost) { best = kb; best_cost = cost; }
    }
    return best;
}

template <int FMT>
static tlb_status launch_fmt(const MvParams &p, int grid, size_t smem, bool pdl)
{
    // Function attributes are set once, to their final values, before the first launch: a graph whose
    // kernel nodes were captured while the limit was still growing replayed 25 % slower than the same
    // launches issued one by one.  Always the largest shared-memory split, whatever a launch needs, so
    // that SMs do not re-partition between launches.
    static bool prepared = false;
    if (!prepared) {
        TLB_CUDA(cudaFuncSetAttribute(qmatvec_kernel<FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ctx()->smem_optin));
        TLB_CUDA(cudaFuncSetAttribute(qmatvec_kernel<FMT>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        prepared = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx()->stream;
    cudaLaunchAttribute at[1];
    int na = 0;
    if (pdl) {
        at[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[na].val.programmaticStreamSerializationAllowed = 1;
        na++;
    }
    cfg.attrs = at;
    cfg.numAttrs = na;
    TLB_CUDA(cudaLaunchKernelEx(&cfg, qmatvec_kernel<FMT>, p));
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
    if (((uintptr_t)job.x | (uintptr_t)job.x2 | (uintptr_t)job.norm_w | (uintptr_t)job.emb_table) & 15)
        return fail(TLB_ERR_ARG, "matvec activations and norm weights must be 16-byte aligned");
    MvParams p = {};
    int64_t tiles = 0;
    for (int i = 0; i < 3; i++) {
        if (i < job.n_w) {
            if (!job.w[i] || !job.out[i]) return fail(TLB_ERR_NULL, "null weight or output");
            tiles += job.n_tiles[i];
            p.w[i] = job.w[i];
            p.out[i] = job.out[i];
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
    if (tiles > INT32_MAX / (64 * kMaxSlices)) return fail(TLB_ERR_SHAPE, "too many tiles for one launch");
    // K-slices: as many as the cost model likes and the slice scratch and tile counters hold
    int max_slices = kMaxSlices;
    if (tiles > (int64_t)c->mv_cnt_n) max_slices = 1;
    while (max_slices > 1 && (size_t)max_slices * tiles * 16 * job.m > c->mv_part_floats) max_slices--;
    p.kb = job.slices > 0 ? std::min(job.slices, max_slices) : qmatvec_plan_slices(job.type, job.k, job.m, tiles, max_slices);
    if (p.kb < 1 || p.upt % p.kb) return fail(TLB_ERR_ARG, "%d slices do not divide the %d units of K", p.kb, p.upt);
    p.upi = p.upt / p.kb;
    p.fold_poll = (job.m == 1 && (size_t)p.kb * tiles * 16 <= c->mv_part1_floats) ? 1 : 0;
    p.part = p.fold_poll ? c->mv_part1 : c->mv_part;
    p.tile_cnt = c->mv_cnt;
    p.tiles = (int)tiles;
    p.n_items = (int)(tiles * p.kb);
    p.unit_bytes = f->unit_bytes;
    p.stage_bytes = stage_bytes_of(f);
    const int grid = (int)std::min<int64_t>((int64_t)c->sm_count * kCtasPerSm, p.n_items);
    p.ipc_q = p.n_items / grid;
    p.ipc_r = p.n_items % grid;
    p.nb_max = blocks_per_cta(p.n_items, grid, tiles, p.upi, p.upt);
    const SmemPlan sp = plan_smem(job.type, job.m, p.nl, p.nb_max);
    // Shared memory per CTA: a third of the SM (1 KB per CTA is reserved by the system), so that a CTA of
    // the next kernel can be resident beside this launch's two; a launch nothing worthwhile follows may
    // take half, and a shape whose tables need more takes what it needs.
    const size_t sm_total = c->smem_optin + 1024;
    size_t budget = sm_total / (job.last_of_chain ? kCtasPerSm : kResidentPerSm) - 1024;
    if (sp.fixed + 128 + 2 * (size_t)kWarps * (p.stage_bytes + 8) > budget) budget = sm_total / kCtasPerSm - 1024;
    if (sp.fixed + 128 + 2 * (size_t)kWarps * (p.stage_bytes + 8) > budget) budget = c->smem_optin;
    const size_t per_stage = (size_t)kWarps * (p.stage_bytes + 8);
    if (sp.fixed + 128 + 2 * per_stage > budget)
        return fail(TLB_ERR_SHAPE, "K = %lld with %d rows needs more shared memory than one SM has (max K %zu)",
                    (long long)job.k, job.m, qmatvec_max_k(job.m));
    // (room for the local-mode slots: at most ~6 per warp)
    const size_t seg_room = (p.kb == 1 ? (size_t)kWarps * 8 * 16 * job.m * sizeof(float) + 128 : 0) +
                            (job.prologue == PRO_ATTN_MERGE ? (size_t)p.nb_max * 4 * std::max(1, job.att_max_splits) * sizeof(float) + 128 : 0);
    int spw = (int)((budget - sp.fixed - 128 - seg_room) / per_stage);
    // no more stages than the longest warp has units, and no more than keeps ~1.5 us of HBM latency covered
    const int64_t ipc = (p.n_items + grid - 1) / grid;
    const int64_t upw = (ipc + kWarps - 1) / kWarps * p.upi;
    spw = (int)std::min<int64_t>(std::min(spw, 8), std::max<int64_t>(2, upw));
    p.spw = spw;
    const size_t ring = (size_t)kWarps * spw * p.stage_bytes;
    p.off_xq = (int)ring + sp.off_xq; p.off_alam = (int)ring + sp.off_alam; p.off_xsum = (int)ring + sp.off_xsum;
    p.off_sa = (int)ring + sp.off_sa; p.off_minv = (int)ring + sp.off_minv; p.off_misc = (int)ring + sp.off_misc;
    p.off_bars = (int)(ring + sp.fixed);
    p.col_stride = sp.col_stride;
    size_t smem = ring + sp.fixed + (size_t)kWarps * spw * 8;
    // local mode (one K-slice): per warp, one slot of 16 * m partial results per tile its unit range touches
    p.max_seg = 1;
    p.off_seg = 0;
    if (p.kb == 1) {
        const int64_t n_max = (ipc * p.upi + kWarps - 1) / kWarps;           // most units a warp gets
        p.max_seg = (int)((n_max + p.upi - 2) / p.upi + 1);
        p.off_seg = (int)((smem + 127) / 128 * 128);
        smem = (size_t)p.off_seg + (size_t)kWarps * p.max_seg * 16 * job.m * sizeof(float);
        if (smem > c->smem_optin) return fail(TLB_ERR_SHAPE, "launch needs %zu bytes of shared memory", smem);
    }
    p.prologue = job.prologue;
    p.x = job.x; p.x2 = job.x2; p.norm_w = job.norm_w; p.eps = job.eps; p.x_out = job.x_out;
    p.tp_reduce = job.tp_reduce ? 1 : 0;
    if (job.tp_reduce) {
        if (job.m != 1 || job.n_w != 1 || job.finish == FIN_SILU) return fail(TLB_ERR_ARG, "the in-launch sum over tensor-parallel ranks takes one tensor, one activation row, plain or residual finishing");
        if (!tp_fuse_args(&p.tp)) return fail(TLB_ERR_ARG, "the in-launch sum over tensor-parallel ranks needs attached peer memory");
        if (job.n_rows[0] > p.tp.rank_stride) return fail(TLB_ERR_SHAPE, "vector too long for the tensor-parallel slots");
    }
    p.emb_table = job.emb_table; p.token = job.token;
    p.ssq_parts = job.ssq_parts; p.n_parts = job.n_parts;
    p.att_part = job.att_part; p.att_pos = job.att_pos;
    p.att_max_splits = job.att_max_splits; p.att_rep = job.att_rep; p.att_dim = job.att_dim; p.att_keys = job.att_keys;
    if (job.prologue == PRO_ATTN_MERGE) {
        if (!job.att_part || !job.att_pos || job.att_max_splits < 1 || job.att_rep < 1 || job.att_keys < 1 ||
            (job.att_dim != 64 && job.att_dim != 128) || job.k % job.att_dim)
            return fail(TLB_ERR_ARG, "attention-merge prologue: incomplete or unsupported description of the split results");
        // softmax weights of the splits, one row per query head of the CTA's blocks, after everything else
        p.off_wtab = (int)((smem + 127) / 128 * 128);
        smem = (size_t)p.off_wtab + (size_t)p.nb_max * (256 / job.att_dim) * job.att_max_splits * sizeof(float);
        if (smem > c->smem_optin) return fail(TLB_ERR_SHAPE, "launch needs %zu bytes of shared memory", smem);
    }
    p.finish = job.finish; p.resid = job.resid; p.ssq_out = job.ssq_out;
    if (job.finish != FIN_PLAIN && (job.m != 1 || job.n_w != 1)) return fail(TLB_ERR_ARG, "fused tile finishing takes one tensor and one activation row");
    if (job.finish == FIN_RESID && (!job.resid || !job.ssq_out)) return fail(TLB_ERR_NULL, "null residual or statistics buffer");
    if (job.ssq_parts && (job.prologue != PRO_ADD_NORM || job.n_parts < 1)) return fail(TLB_ERR_ARG, "partial sums of squares go with the fused RMSNorm prologue");
    p.err = c->err_flag;
    p.use_pdl = job.pdl ? 1 : 0;
    if (!p.x && !(p.prologue == PRO_ADD_NORM && p.token) && p.prologue != PRO_ATTN_MERGE) return fail(TLB_ERR_NULL, "null activation");
    if (p.prologue == PRO_SILU_MUL && !p.x2) return fail(TLB_ERR_NULL, "null activation");
    if (job.dry_run) return TLB_OK;   // the shape is launchable
    switch (job.type) {
    case TLB_GGML_Q4_K: return launch_fmt<TLB_GGML_Q4_K>(p, grid, smem, job.pdl);
    case TLB_GGML_Q6_K: return launch_fmt<TLB_GGML_Q6_K>(p, grid, smem, job.pdl);
    case TLB_GGML_Q8_0: return launch_fmt<TLB_GGML_Q8_0>(p, grid, smem, job.pdl);
    default: return launch_fmt<TLB_GGML_Q4_0>(p, grid, smem, job.pdl);
    }
}

}  // namespace tlb

using namespace tlb;

// More than 4 activation rows: the matvec would re-stream the weight once per group of 4 rows; launch_qgemm reads it once
// (up to 16 rows: its streaming kernel on mma.sync; more: the tensor-memory GEMM).  Up to 4 rows stay with the matvec: one
// launch, activations at 14 bits instead of f16's 11 (with 3 or 4 rows the other route measured faster on some shapes of
// 16 MB and more and slower on others).
static bool prefer_gemm(int64_t m, const tlb_qtensor *w)
{
    return m > 4 && qgemm_supported(w->type) && w->k % 256 == 0;
}

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
    if (!w->tiled()) {
        // dense weight: x . W^T through the f32 matmul over the cached transpose, the reference's route for types
        // without a fused kernel (crates/tl_runtime/src/system.rs:236-264)
        tlb_qtensor *wm = const_cast<tlb_qtensor *>(w);
        {
            std::lock_guard<std::mutex> lk(wm->mu);
            if (!wm->dense_t) {
                const int64_t tshape[2] = {w->k, w->n}, tstr[2] = {1, w->k};
                st = new_tensor(&wm->dense_t, TLB_F32, tshape, 2);
                if (st == TLB_OK) st = launch_copy_strided(w->dense->f32(), wm->dense_t->f32(), tshape, tstr, 2, w->n * w->k, 0);
                if (st != TLB_OK) { tlb_tensor_release(wm->dense_t); wm->dense_t = nullptr; }
            }
        }
        if (st == TLB_OK) st = launch_matmul(x->f32(), w->dense_t->f32(), (*out)->f32(), 1, m, k, w->n, false);
        if (st != TLB_OK) { tlb_tensor_release(*out); *out = nullptr; }
        return st;
    }
    // The kernels read the activation with 16-byte loads; a view that starts at an odd element (tlb_narrow makes
    // zero-copy views at any offset) is first copied to an aligned buffer.
    const tlb_tensor *xa = x;
    tlb_tensor *xcopy = nullptr;
    if ((uintptr_t)x->f32() & 15) {
        st = tlb_tensor_clone(&xcopy, x);
        if (st != TLB_OK) { tlb_tensor_release(*out); *out = nullptr; return st; }
        xa = xcopy;
    }
    if (prefer_gemm(m, w)) {
        // more than four rows (batched decoding, prompt processing): the weight is read once per 256 rows
        st = launch_qgemm(w, xa->f32(), m, (*out)->f32());
    } else {
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
            job.x = xa->f32() + m0 * k;
            st = launch_qmatvec(job);
        }
    }
    tlb_tensor_release(xcopy);   // stream-ordered pool: the storage outlives the kernels already enqueued
    if (st != TLB_OK) { tlb_tensor_release(*out); *out = nullptr; }
    return st;
}
