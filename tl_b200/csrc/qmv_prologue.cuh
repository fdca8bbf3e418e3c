// Prologue of the streaming matvec: builds the int8 B operands in shared memory.
//
// int8 levels: per activation row m and per block of 256 k (one weight super-block) the values are
// written as  x ~ alpha * (l0 + l1/254 + l2/254^2),  l_i in [-127, 127], alpha = max|x| / 127 over the
// block; every level is the rounded residual of the previous ones, so three levels carry ~23 bits
// and the integer MMAs downstream are exact.  Level l of row m is column m*nl + l, stored at
//   xq[col][64*G + 16*c + 8*sub + 4*h + byte]   for k = 64*G + 32*sub + 16*h + 4*c + byte,
// i.e. the two words a lane needs for one m16n8k32 MMA are adjacent.  alam[u][col] = alpha * 254^-l
// (0 for unused columns).  Also written: per-32 sums of x as an (hi, lo) pair of f16 scaled by a
// power of two (Q4_K mins), per-16 sums of the levels as f16 (Q6_K offset term) or per-32 sums as
// int32 (Q4_0 offset term).
//
// Rounding uses the 1.5 * 2^23 trick: t = x * inv + MAGIC rounds to the nearest integer in the
// FMA pipe, the level is the low byte of t's bit pattern, and no conversion instruction is issued.
#pragma once
#include "qmv_common.cuh"

namespace tlb {

#define MAGIC_RN 12582912.0f

template <int FMT>
__device__ void build_activation(const MvParams &p, MvShared *sh, uint8_t *smem, int tid, int nthreads)
{
    const int lane = tid & 31, warp = tid >> 5, nwarps = nthreads >> 5;
    const int k4n = p.k / 4, nsb = p.k / 256;
    uint8_t *xq = smem + p.off_xq;
    float *alam = reinterpret_cast<float *>(smem + p.off_alam);
    __half *xsum = reinterpret_cast<__half *>(smem + p.off_xsum);
    float *wmax = reinterpret_cast<float *>(smem + p.off_misc);   // [m][k/128] block maxima
    const float *xbase = p.x;
    if (p.prologue == PRO_ADD_NORM && p.token) xbase = p.emb_table + (size_t)__ldg(p.token) * p.k;

    for (int i = tid; i < nsb * kMaxCols; i += nthreads) alam[i] = 0.f;
    // pass 1: sum of squares (norm), maxima per 128 elements
    float ssq = 0.f, gmax = 0.f;
    // Loads are issued in batches of kBatch before any of them is used: a shuffle or a shared store
    // between two loads would otherwise expose the full L2 latency once per element group.
    constexpr int kBatch = 4;
    for (int mrow = 0; mrow < p.m; mrow++)
        for (int base = tid; base < k4n; base += nthreads * kBatch) {   // k4n % 64 == 0: warps stay whole
            float4 vv[kBatch], ww[kBatch];
#pragma unroll
            for (int j = 0; j < kBatch; j++) {
                const int k4 = base + j * nthreads;
                if (k4 < k4n) {
                    vv[j] = prologue_value(p, xbase, mrow, k4, 0.f);
                    if (p.prologue == PRO_ADD_NORM) ww[j] = __ldg(reinterpret_cast<const float4 *>(p.norm_w) + k4);
                }
            }
#pragma unroll
            for (int j = 0; j < kBatch; j++) {
                const int k4 = base + j * nthreads;
                if (k4 < k4n) {
                    const float4 v = vv[j];
                    float mx;
                    if (p.prologue == PRO_ADD_NORM) {
                        const float4 w = ww[j];
                        ssq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                        mx = fmaxf(fmaxf(fabsf(v.x * w.x), fabsf(v.y * w.y)), fmaxf(fabsf(v.z * w.z), fabsf(v.w * w.w)));
                        if (p.x_out && blockIdx.x == 0) reinterpret_cast<float4 *>(p.x_out)[k4] = v;
                    } else {
                        mx = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
                    }
                    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                    if (lane == 0) wmax[mrow * (p.k / 128) + (k4 >> 5)] = mx;
                    gmax = fmaxf(gmax, mx);
                }
            }
        }
    if (p.prologue == PRO_ADD_NORM)
        for (int o = 16; o; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
    if (lane == 0) { sh->red_sum[warp] = ssq; sh->red_max[warp] = gmax; }
    named_bar(1, nthreads);
    ssq = 0.f; gmax = 0.f;
    for (int w = 0; w < nwarps; w++) { ssq += sh->red_sum[w]; gmax = fmaxf(gmax, sh->red_max[w]); }
    float inv_rms = 0.f, stat_scale = 1.f;
    if (p.prologue == PRO_ADD_NORM) {
        inv_rms = 1.f / sqrtf(ssq / (float)p.k + p.eps);
        stat_scale = inv_rms;   // block maxima were taken before the division by rms
    }
    gmax *= stat_scale;
    // S: power of two bringing max|x| into [512, 1024), so that f16 sums of 32 stay finite
    float S = 1.f;
    if (gmax > 0.f && gmax < 3.0e38f) {
        const int e = (int)((__float_as_uint(gmax) >> 23) & 0xFF);   // gmax in [2^(e-127), 2^(e-126))
        const int se = 127 + 9 - (e - 127);
        if (se > 0 && se < 255) S = __uint_as_float((uint32_t)se << 23);
    }
    if (tid == 0) sh->inv_scale = 1.f / S;
    // pass 2: quantise
    for (int mrow = 0; mrow < p.m; mrow++)
      for (int base = tid; base < k4n; base += nthreads * kBatch) {
        float4 vv[kBatch];
#pragma unroll
        for (int j = 0; j < kBatch; j++)
            if (base + j * nthreads < k4n) vv[j] = prologue_value(p, xbase, mrow, base + j * nthreads, inv_rms);
#pragma unroll
        for (int j = 0; j < kBatch; j++) {
            const int k4 = base + j * nthreads;
            if (k4 >= k4n) break;
            const int u = k4 >> 6;
            float amax = fmaxf(wmax[mrow * (p.k / 128) + 2 * u], wmax[mrow * (p.k / 128) + 2 * u + 1]) * stat_scale;
            amax *= 1.000001f;   // maxima of the norm path were taken on un-normalised products: keep |l0| <= 127
            const float alpha = amax > 0.f ? amax * (1.f / 127.f) : 1.f;
            const float4 v = vv[j];
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
                        float t = fmaf(res[e], inv, MAGIC_RN);
                        t = fminf(fmaxf(t, MAGIC_RN - 127.f), MAGIC_RN + 127.f);
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
            // k = 4*k4 + byte  ->  G = k4 >> 4, t = k4 & 15: sub = t >> 3, h = (t >> 2) & 1, c = t & 3
            const int G = k4 >> 4, t = k4 & 15;
            const int off = G * 64 + (t & 3) * 16 + (t >> 3) * 8 + ((t >> 2) & 1) * 4;
            for (int l = 0; l < p.nl; l++)
                *reinterpret_cast<uint32_t *>(xq + (size_t)(mrow * p.nl + l) * p.col_stride + off) = words[l];
            if ((k4 & 63) == 0) {
                float a = alpha;
                for (int l = 0; l < p.nl; l++) { alam[u * kMaxCols + mrow * p.nl + l] = a; a *= (1.f / 254.f); }
            }
            if (FMT == TLB_GGML_Q4_K) {   // sums of x over sub-blocks of 32 = 8 consecutive k4 = 8 consecutive lanes
                float t4 = ((v.x + v.y) + (v.z + v.w)) * S;
                t4 += __shfl_xor_sync(0xffffffffu, t4, 1);
                t4 += __shfl_xor_sync(0xffffffffu, t4, 2);
                t4 += __shfl_xor_sync(0xffffffffu, t4, 4);
                if ((lane & 7) == 0) {
                    const __half hi = __float2half_rn(t4);
                    const __half lo = __float2half_rn(t4 - __half2float(hi));
                    xsum[(size_t)(2 * mrow) * (p.k / 32) + (k4 >> 3)] = hi;
                    xsum[(size_t)(2 * mrow + 1) * (p.k / 32) + (k4 >> 3)] = lo;
                }
            }
            if (FMT == TLB_GGML_Q6_K) {   // level sums over groups of 16 = 4 consecutive lanes, as f16 (|sum| <= 2032: exact); [u][col][16]
                __half *sa = reinterpret_cast<__half *>(smem + p.off_sa);
                for (int l = 0; l < p.nl; l++) {
                    float s = lsum[l];
                    s += __shfl_xor_sync(0xffffffffu, s, 1);
                    s += __shfl_xor_sync(0xffffffffu, s, 2);
                    if ((lane & 3) == 0) sa[((size_t)u * kMaxCols + mrow * p.nl + l) * 16 + ((k4 >> 2) & 15)] = __float2half_rn(s);
                }
            }
            if (FMT == TLB_GGML_Q4_0) {   // level sums over blocks of 32 = 8 consecutive lanes, int32; [k/32][8 cols]
                int *sa = reinterpret_cast<int *>(smem + p.off_sa);
                for (int l = 0; l < p.nl; l++) {
                    float s = lsum[l];
                    s += __shfl_xor_sync(0xffffffffu, s, 1);
                    s += __shfl_xor_sync(0xffffffffu, s, 2);
                    s += __shfl_xor_sync(0xffffffffu, s, 4);
                    if ((lane & 7) == 0) sa[(size_t)(k4 >> 3) * kMaxCols + mrow * p.nl + l] = __float2int_rn(s);
                }
            }
        }
      }
    named_bar(1, nthreads);
}

}  // namespace tlb
