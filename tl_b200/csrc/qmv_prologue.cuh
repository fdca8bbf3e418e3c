// Prologue of the streaming matvec: builds the int8 B operands of the MMAs in shared memory.
//
// int8 levels: per activation row m and per block of 256 k (one weight super-block) the values are
// written as  x ~ alpha * (l0 + l1/254 + l2/254^2),  l_i in [-127, 127], alpha = max|x| / 127 over the
// block; every level is the rounded residual of the previous ones, so three levels carry ~23 bits
// and the integer MMAs downstream are exact.  Level l of row m is column m*nl + l, stored at
//   xq[col][256*lb + 64*G + 16*c + 8*sub + 4*h + byte]   for k = 256*blk + 64*G + 32*sub + 16*h + 4*c + byte,
// i.e. the two words a lane needs for one m16n8k32 MMA are adjacent.  lb = blk - blk0 is the block
// index local to the CTA: a CTA quantises only the blocks its K-slices cover.  alam[lb][col] =
// alpha * 254^-l (0 for unused columns).  Also written: per-32 sums of x as an (hi, lo) pair of f16
// scaled by a per-block power of two whose inverse goes to minv[lb][m] (Q4_K mins), per-16 sums of
// the levels as f16 (Q6_K offset term) or per-32 sums as int32 (Q4_0 offset term).
//
// Rounding uses the 1.5 * 2^23 trick: t = x * inv + MAGIC rounds to the nearest integer in the
// FMA pipe, the level is the low byte of t's bit pattern, and no conversion instruction is issued.
#pragma once
#include "qmv_common.cuh"

namespace tlb {

#define MAGIC_RN 12582912.0f

// A block (mrow, blk) is quantised by a group of 64 threads (index j in the group) in two steps with a
// group barrier between them, so that a group can run the steps of two blocks side by side:
// warp_absmax() gives the largest magnitude among a warp's 128 values; quantise_block() takes the
// block's maximum and writes the shared tables at local block index lb.
__device__ __forceinline__ float warp_absmax(const float4 v)
{
    float mx = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    return mx;
}

template <int FMT>
__device__ __forceinline__ void quantise_block(const MvParams &p, uint8_t *smem, const float amax, const float4 v,
                                               int mrow, int lb, int j, int lane)
{
    // blocks whose largest magnitude is below 2^-100 (or not finite) quantise to zero levels: their
    // contribution is below f32 resolution of any realistic result, and 1 / alpha stays finite
    const float alpha = (amax > 7.9e-31f && amax < 3.0e38f) ? amax * (1.f / 127.f) : 1.f;
    float res[4] = {v.x, v.y, v.z, v.w};
    float scale = alpha, inv = __frcp_rn(alpha);
    uint32_t words[3] = {0u, 0u, 0u};
    float lsum[3] = {0.f, 0.f, 0.f};
#pragma unroll
    for (int l = 0; l < 3; l++) {
        if (l < p.nl) {
            uint32_t tb[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                // |res * inv| <= 127 by construction at every level (alpha = max / 127; a residual is at most
                // half a step of the level before), so no clamp is needed
                const float t = fmaf(res[e], inv, MAGIC_RN);
                const float qf = t - MAGIC_RN;
                res[e] = fmaf(-qf, scale, res[e]);
                lsum[l] += qf;
                tb[e] = __float_as_uint(t);     // low byte = the level as two's-complement int8
            }
            words[l] = prmt(prmt(tb[0], tb[1], 0x0040u), prmt(tb[2], tb[3], 0x0040u), 0x5410u);
            scale *= (1.f / 254.f);
            inv *= 254.f;
        }
    }
    // k = 256*blk + 4*j + byte  ->  G = j >> 4, t = j & 15: sub = t >> 3, h = (t >> 2) & 1, c = t & 3
    const int G = j >> 4, t = j & 15;
    const int off = lb * 256 + G * 64 + (t & 3) * 16 + (t >> 3) * 8 + ((t >> 2) & 1) * 4;
#pragma unroll
    for (int l = 0; l < 3; l++)
        if (l < p.nl) *reinterpret_cast<uint32_t *>(smem + p.off_xq + (size_t)(mrow * p.nl + l) * p.col_stride + off) = words[l];
    if (j < kMaxCols) {   // alam[lb][0..7]: this row's levels; other rows' columns are written by their own groups
        const int col = j, l = col - mrow * p.nl;
        float *alam = reinterpret_cast<float *>(smem + p.off_alam);
        if (l >= 0 && l < p.nl) {
            float a = alpha;
            for (int i = 0; i < l; i++) a *= (1.f / 254.f);
            alam[lb * kMaxCols + col] = a;
        } else if (col >= p.m * p.nl && mrow == 0) {
            alam[lb * kMaxCols + col] = 0.f;   // unused columns
        }
    }
    if (FMT == TLB_GGML_Q4_K) {   // sums of x over sub-blocks of 32 = 8 consecutive k4 = 8 consecutive lanes
        // S: power of two bringing the block maximum into [512, 1024): f16 sums of 32 stay finite
        float S = 1.f;
        if (amax > 0.f && amax < 3.0e38f) {
            const int e = (int)((__float_as_uint(amax) >> 23) & 0xFF);
            const int se = 127 + 9 - (e - 127);
            if (se > 0 && se < 255) S = __uint_as_float((uint32_t)se << 23);
        }
        float t4 = ((v.x + v.y) + (v.z + v.w)) * S;
        t4 += __shfl_xor_sync(0xffffffffu, t4, 1);
        t4 += __shfl_xor_sync(0xffffffffu, t4, 2);
        t4 += __shfl_xor_sync(0xffffffffu, t4, 4);
        __half *xsum = reinterpret_cast<__half *>(smem + p.off_xsum);
        if ((lane & 7) == 0) {
            const __half hi = __float2half_rn(t4);
            const __half lo = __float2half_rn(t4 - __half2float(hi));
            xsum[(size_t)(2 * mrow) * (p.nb_max * 8) + lb * 8 + (j >> 3)] = hi;
            xsum[(size_t)(2 * mrow + 1) * (p.nb_max * 8) + lb * 8 + (j >> 3)] = lo;
        }
        if (j == 0) reinterpret_cast<float *>(smem + p.off_minv)[lb * 4 + mrow] = 1.f / S;
    }
    if (FMT == TLB_GGML_Q6_K) {   // level sums over groups of 16 = 4 consecutive lanes, as f16 (|sum| <= 2032: exact); [lb][col][16]
        __half *sa = reinterpret_cast<__half *>(smem + p.off_sa);
#pragma unroll
        for (int l = 0; l < 3; l++)
            if (l < p.nl) {
                float s = lsum[l];
                s += __shfl_xor_sync(0xffffffffu, s, 1);
                s += __shfl_xor_sync(0xffffffffu, s, 2);
                if ((lane & 3) == 0) sa[((size_t)lb * kMaxCols + mrow * p.nl + l) * 16 + (j >> 2)] = __float2half_rn(s);
            }
    }
    if (FMT == TLB_GGML_Q4_0) {   // level sums over blocks of 32 = 8 consecutive lanes, int32; [lb*8 + j/8][8 cols]
        int *sa = reinterpret_cast<int *>(smem + p.off_sa);
#pragma unroll
        for (int l = 0; l < 3; l++)
            if (l < p.nl) {
                float s = lsum[l];
                s += __shfl_xor_sync(0xffffffffu, s, 1);
                s += __shfl_xor_sync(0xffffffffu, s, 2);
                s += __shfl_xor_sync(0xffffffffu, s, 4);
                if ((lane & 7) == 0) sa[(size_t)(lb * 8 + (j >> 3)) * kMaxCols + mrow * p.nl + l] = __float2int_rn(s);
            }
    }
}

// Fills the shared tables for activation blocks [blk0, blk0 + nb) of every row.  All `nthreads`
// threads of the CTA call it; it ends with a CTA-wide barrier.
//
// Groups of 64 threads take one block each.  Everything a group needs from global memory is
// requested up front - the values of its own blocks (kept in registers), their norm weights, and
// for the fused RMSNorm its share of the REST of the row, which enters only the sum of squares - so
// the prologue costs one round trip to L2, not one per step.
//
// `after_loads(dep)` is called once per thread when the values it requested have arrived (dep is
// computed from them): the caller uses it to start traffic that should not delay those loads.
//
// The norm weights are static, so the caller fetches those of the first pass with
// load_norm_weights() BEFORE it waits for the previous kernel: they are read once per token and
// always miss L2, which would otherwise be the longest latency of the prologue.
constexpr int kKeep = 2;   // blocks per group handled in one pass

__device__ __forceinline__ void load_norm_weights(const MvParams &p, int tid, int nthreads, int blk0, int nb, float4 (&wgt)[kKeep])
{
    const int ngroups = nthreads >> 6, grp = tid >> 6, j = tid & 63;
#pragma unroll
    for (int i = 0; i < kKeep; i++) {
        wgt[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        const int item = grp + i * ngroups;     // ADD_NORM has one activation row: item == local block
        if (p.prologue == PRO_ADD_NORM && item < nb) wgt[i] = __ldg(reinterpret_cast<const float4 *>(p.norm_w) + (blk0 + item) * 64 + j);
    }
}

template <int FMT, typename AfterLoads>
__device__ void build_activation(const MvParams &p, MvShared *sh, uint8_t *smem, int tid, int nthreads, int blk0, int nb,
                                 const float4 (&wgt_first)[kKeep], AfterLoads after_loads)
{
    const int lane = tid & 31, warp = tid >> 5, nwarps = nthreads >> 5;
    const int ngroups = nthreads >> 6, grp = tid >> 6, j = tid & 63;
    const int nblk = p.k / 256, n_mine = p.m * nb;
    const bool norm = p.prologue == PRO_ADD_NORM;
    const float *emb = nullptr;
    if (norm && p.token) emb = p.emb_table + (size_t)__ldg(p.token) * p.k;

    // Attention output still split over the keys: first the softmax weight of every split for each query
    // head this CTA needs - w[head][s] = exp(m_s - M) / sum_t l_t exp(m_t - M), one warp per head - then the
    // values are the weighted sums of the splits' rows (attn_value below).
    const bool attn = p.prologue == PRO_ATTN_MERGE;
    int nsplit = 1;
    float *wtab = reinterpret_cast<float *>(smem + p.off_wtab);   // [heads of this CTA][att_max_splits]
    if (attn) {
        const int hpb = 256 / p.att_dim;     // query heads per block of 256
        nsplit = (__ldcg(p.att_pos) + p.att_keys) / p.att_keys;   // ceil((pos + 1) / keys per split)
        const size_t sstride = (size_t)p.att_rep * (p.att_dim + 4);
        for (int hl = warp; hl < nb * hpb; hl += nwarps) {
            const int head = blk0 * hpb + hl, kvh = head / p.att_rep, hr = head - kvh * p.att_rep;
            const float *row0 = p.att_part + ((size_t)kvh * p.att_max_splits * p.att_rep + hr) * (p.att_dim + 4) + p.att_dim;
            // lane s holds split s (and s + 32, ... for very long contexts, re-read in the later passes)
            const float m0 = lane < nsplit ? __ldcg(row0 + lane * sstride) : -INFINITY;
            const float l0 = lane < nsplit ? __ldcg(row0 + lane * sstride + 1) : 0.f;
            float mx = m0;
            for (int sp = lane + 32; sp < nsplit; sp += 32) mx = fmaxf(mx, __ldcg(row0 + sp * sstride));
            for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            const float w0 = lane < nsplit ? expf(m0 - mx) : 0.f;
            float lsum = l0 * w0;
            for (int sp = lane + 32; sp < nsplit; sp += 32) lsum += __ldcg(row0 + sp * sstride + 1) * expf(__ldcg(row0 + sp * sstride) - mx);
            for (int o = 16; o; o >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, o);
            const float inv_l = 1.f / lsum;
            if (lane < nsplit) wtab[hl * p.att_max_splits + lane] = w0 * inv_l;
            for (int sp = lane + 32; sp < nsplit; sp += 32) wtab[hl * p.att_max_splits + sp] = expf(__ldcg(row0 + sp * sstride) - mx) * inv_l;
        }
        __syncthreads();
    }
    auto attn_value = [&](int lb) {   // elements 4j .. 4j+3 of local block lb
        const int e = ((blk0 + lb) * 64 + j) * 4;
        const int head = e / p.att_dim, d = e - head * p.att_dim;
        const int kvh = head / p.att_rep, hr = head - kvh * p.att_rep, hl = head - blk0 * (256 / p.att_dim);
        const float *row = p.att_part + ((size_t)kvh * p.att_max_splits * p.att_rep + hr) * (p.att_dim + 4) + d;
        const size_t sstride = (size_t)p.att_rep * (p.att_dim + 4);
        const float *wr = wtab + hl * p.att_max_splits;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
        for (int sp = 0; sp < nsplit; sp++) {
            const float4 v = __ldcg(reinterpret_cast<const float4 *>(row + sp * sstride));
            const float w = wr[sp];
            acc.x = fmaf(w, v.x, acc.x); acc.y = fmaf(w, v.y, acc.y); acc.z = fmaf(w, v.z, acc.z); acc.w = fmaf(w, v.w, acc.w);
        }
        return acc;
    };

    float inv_rms = 0.f;
    for (int first = 0; first < n_mine || (norm && first == 0); first += ngroups * kKeep) {
        float4 keep[kKeep], wgt[kKeep];
        float ssq = 0.f;
#pragma unroll
        for (int i = 0; i < kKeep; i++) {
            const int item = first + grp + i * ngroups;
            if (item < n_mine) {
                const int mrow = item / nb, lb = item - mrow * nb, k4 = (blk0 + lb) * 64 + j;
                keep[i] = attn ? attn_value(lb) : prologue_value(p, emb, mrow, k4, 0.f);
                if (norm) wgt[i] = first == 0 ? wgt_first[i] : __ldg(reinterpret_cast<const float4 *>(p.norm_w) + k4);
            }
        }
        if (norm && first == 0 && p.ssq_parts) {
            // The producer of x left partial sums of squares: every warp adds them itself, in one fixed
            // order, so no block-wide exchange is needed and nothing of the row is re-read.
            for (int i = lane; i < p.n_parts; i += 32) ssq += __ldcg(p.ssq_parts + i);
            float dep = ssq;
#pragma unroll
            for (int i = 0; i < kKeep; i++)
                if (grp + i * ngroups < n_mine) dep += keep[i].x;
            after_loads(dep);
            for (int o = 16; o; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
            inv_rms = 1.f / sqrtf(ssq / (float)p.k + p.eps);
        } else if (norm && first == 0) {
            // the blocks outside [blk0, blk0 + nb): only their squares are needed (m == 1 with this prologue)
            for (int o = grp; o < nblk - nb; o += ngroups) {
                const int k4 = (o < blk0 ? o : o + nb) * 64 + j;
                const float4 v = prologue_value(p, emb, 0, k4, 0.f);
                ssq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                if (p.x_out && blockIdx.x == 0) reinterpret_cast<float4 *>(p.x_out)[k4] = v;
            }
            for (int it = grp; it < n_mine; it += ngroups) {   // own blocks beyond the first pass, if any
                if (it < ngroups * kKeep) continue;
                const int k4 = (blk0 + it) * 64 + j;
                const float4 v = prologue_value(p, emb, 0, k4, 0.f);
                ssq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                if (p.x_out && blockIdx.x == 0) reinterpret_cast<float4 *>(p.x_out)[k4] = v;
            }
#pragma unroll
            for (int i = 0; i < kKeep; i++) {
                const int item = grp + i * ngroups;
                if (item < n_mine) {
                    const float4 v = keep[i];
                    ssq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                    if (p.x_out && blockIdx.x == 0) reinterpret_cast<float4 *>(p.x_out)[(blk0 + item) * 64 + j] = v;
                }
            }
            after_loads(ssq);
            for (int o = 16; o; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
            if (lane == 0) sh->red_sum[warp] = ssq;
            __syncthreads();
            ssq = 0.f;
            for (int w = 0; w < nwarps; w++) ssq += sh->red_sum[w];
            inv_rms = 1.f / sqrtf(ssq / (float)p.k + p.eps);
        }
        if (!norm && first == 0) {
            float dep = 0.f;
#pragma unroll
            for (int i = 0; i < kKeep; i++)
                if (grp + i * ngroups < n_mine) dep += keep[i].x;
            after_loads(dep);
        }
        // step 1 of this pass's blocks: final values and each warp's maximum
        float *pair_max = &sh->red_max[grp * 2 * kKeep];
#pragma unroll
        for (int i = 0; i < kKeep; i++) {
            const int item = first + grp + i * ngroups;
            if (item < n_mine) {
                float4 v = keep[i];
                if (norm) {   // (x / rms) * weight (crates/tl_cpu/src/ffi.rs:2444-2486), the division as a multiply by 1/rms
                    v.x = (v.x * inv_rms) * wgt[i].x; v.y = (v.y * inv_rms) * wgt[i].y;
                    v.z = (v.z * inv_rms) * wgt[i].z; v.w = (v.w * inv_rms) * wgt[i].w;
                }
                keep[i] = v;
                const float mx = warp_absmax(v);
                if (lane == 0) pair_max[2 * i + (j >> 5)] = mx;
            }
        }
        if (first + grp < n_mine) named_bar(2 + grp, 64);
        // step 2: the blocks are independent from here on, their instruction streams interleave
#pragma unroll
        for (int i = 0; i < kKeep; i++) {
            const int item = first + grp + i * ngroups;
            if (item < n_mine) {
                const int mrow = item / nb, lb = item - mrow * nb;
                quantise_block<FMT>(p, smem, fmaxf(pair_max[2 * i], pair_max[2 * i + 1]), keep[i], mrow, lb, j, lane);
            }
        }
        if (first + grp < n_mine && first + ngroups * kKeep < n_mine) named_bar(2 + grp, 64);   // pair_max is reused by the next pass
    }
    __syncthreads();
}

}  // namespace tlb
