// Per-unit consumers of the streaming matvec: one warp turns one unit (16 rows x 256 weights, layout
// in qlayout.cuh) into 16 x 8 partial sums with integer tensor-core MMAs.
//
// Common frame.  `u` is the unit's block index local to the CTA (row of the activation tables).  Lane (r, c) = (lane >> 2, lane & 3) owns rows r and r+8; its C fragment holds
// columns 2c and 2c+1: acc[0], acc[1] for row r, acc[2], acc[3] for row r+8.  A column is one int8
// level of one activation row (see build_activation).  Quants enter the MMA as raw integers:
// nibbles are separated with one AND per four weights, nothing is converted to floating point
// until a whole super-block (Q4_K, Q6_K) or block (Q4_0, Q8_0) has been summed exactly in int32.
#pragma once
#include "qmv_common.cuh"

namespace tlb {

struct LaneCtx {
    int lane, r, c;
    uint32_t xq_b;     // int8 activation column read by this lane as MMA column r (clamped to a used column)
    uint32_t alam_b;   // &alam[0][2c]
    uint32_t xsum_b;   // Q4_K: f16 sub-block sums, column (hi / lo) read by this lane
    uint32_t sa_b;     // Q6_K: f16 level sums of column r (clamped)
    uint32_t sa_c0, sa_c1;  // Q4_0: int32 level sums of columns 2c and 2c+1 (clamped)
    uint32_t minv_b;   // Q4_K: inverse power-of-two scale of the sub-block sums of activation row c (clamped)
};

// B-operand loads.  Lanes whose MMA column carries no level read column 0 instead (xq_b is clamped):
// same address as the lanes of column 0, so the load costs no extra shared-memory wavefront, and
// what those columns accumulate is multiplied by alam == 0 at the end.
__device__ __forceinline__ uint4 ldb128(const LaneCtx &, uint32_t a) { return lds128(a); }
__device__ __forceinline__ uint2 ldb64(const LaneCtx &, uint32_t a) { return lds64(a); }

#define NIB 0x0F0F0F0Fu
#define NIBH 0xF0F0F0F0u
#define H2_1024 0x64006400u

__device__ __forceinline__ int byte_u(uint32_t w, int i) { return (int)prmt(w, 0u, 0x4440u + i); }
__device__ __forceinline__ int byte_s(uint32_t w, int i) { return (int)prmt(w, 0u, (0x8880u + 0x1110u * i) + i); }
// exact int -> float for |v| < 2^22 without the conversion unit
__device__ __forceinline__ float i2f_small(int v) { return __int_as_float(0x4B400000 + v) - 12582912.0f; }

// ---- Q4_K: w = d * sc_s * q - dmin * m_s (crates/tl_runtime/src/quantized.rs:337-415) ----------
// One MMA = one sub-block of 32; its exact integer sum is multiplied by the 6-bit sub-block scale
// with an integer multiply-add, so a single int32 accumulator serves the super-block and d is
// applied once per 256 weights.  The mins enter through one f16 MMA per unit: A = the pair of 6-bit
// mins of sub-blocks (2c, 2c+1), B = the activation sums over those sub-blocks (hi, lo).
__device__ __forceinline__ void unit_q4k(uint32_t up, int u, const LaneCtx &L, float (&master)[4], float (&mm)[4])
{
    const int r = L.r, c = L.c;
    const uint4 hA = lds128(up + 2048 + r * 16), hB = lds128(up + 2048 + (r + 8) * 16);
    uint4 q[4];
#pragma unroll
    for (int G = 0; G < 4; G++) q[G] = lds128(up + G * 512 + L.lane * 16);
    // 6-bit scales of the 8 sub-blocks as bytes: (scl: 0..3, sch: 4..7); get_scale_min_k4 packing
    const uint32_t sclA = hA.y & 0x3F3F3F3Fu, schA = and_or(hA.y >> 2, 0x30303030u, hA.w & NIB);
    const uint32_t sclB = hB.y & 0x3F3F3F3Fu, schB = and_or(hB.y >> 2, 0x30303030u, hB.w & NIB);
    const uint32_t mnwA = (c < 2) ? (hA.z & 0x3F3F3F3Fu) : and_or(hA.z >> 2, 0x30303030u, (hA.w >> 4) & NIB);
    const uint32_t mnwB = (c < 2) ? (hB.z & 0x3F3F3F3Fu) : and_or(hB.z >> 2, 0x30303030u, (hB.w >> 4) & NIB);
    const uint32_t sel = (c & 1) ? 0x5342u : 0x5140u;   // bytes (2,3) / (0,1) -> f16 pair 1024 + value
    float accm[4] = {0.f, 0.f, 0.f, 0.f};
    hmma16816(accm, hsub2(prmt(mnwA, 0x64646464u, sel), H2_1024), hsub2(prmt(mnwB, 0x64646464u, sel), H2_1024), 0u, 0u,
              lds32(L.xsum_b + (8 * u + 2 * c) * 2), 0u);
    uint4 xbs[4];
#pragma unroll
    for (int G = 0; G < 4; G++) xbs[G] = ldb128(L, L.xq_b + (4 * u + G) * 64 + c * 16);
    // The high nibbles enter their MMA in place (q << 4, still an exact u8): their sums are kept in a
    // second accumulator and scaled by 1/16 once per unit, which saves the shift per four weights.
    int acc[4] = {0, 0, 0, 0}, acch[4] = {0, 0, 0, 0};
#pragma unroll
    for (int G = 0; G < 4; G++) {
        const uint4 xb = xbs[G];
        const uint32_t sw_A = (G < 2) ? sclA : schA, sw_B = (G < 2) ? sclB : schB;
        int c4[4];
        imma16832<false>(c4, q[G].x & NIB, q[G].z & NIB, q[G].y & NIB, q[G].w & NIB, xb.x, xb.y);
        int sA = byte_u(sw_A, 2 * (G & 1)), sB = byte_u(sw_B, 2 * (G & 1));
        acc[0] += sA * c4[0]; acc[1] += sA * c4[1]; acc[2] += sB * c4[2]; acc[3] += sB * c4[3];
        imma16832<false>(c4, q[G].x & NIBH, q[G].z & NIBH, q[G].y & NIBH, q[G].w & NIBH, xb.z, xb.w);
        sA = byte_u(sw_A, 2 * (G & 1) + 1); sB = byte_u(sw_B, 2 * (G & 1) + 1);
        acch[0] += sA * c4[0]; acch[1] += sA * c4[1]; acch[2] += sB * c4[2]; acch[3] += sB * c4[3];
    }
    const uint2 alw = lds64(L.alam_b + u * (kMaxCols * 4));
    const float al0 = __uint_as_float(alw.x), al1 = __uint_as_float(alw.y);
    const float2 dA = h2_to_f2(hA.x), dB = h2_to_f2(hB.x);   // (d, dmin)
    master[0] = fmaf(dA.x * al0, fmaf((float)acch[0], 0.0625f, (float)acc[0]), master[0]);
    master[1] = fmaf(dA.x * al1, fmaf((float)acch[1], 0.0625f, (float)acc[1]), master[1]);
    master[2] = fmaf(dB.x * al0, fmaf((float)acch[2], 0.0625f, (float)acc[2]), master[2]);
    master[3] = fmaf(dB.x * al1, fmaf((float)acch[3], 0.0625f, (float)acc[3]), master[3]);
    const float minv = __uint_as_float(lds32(L.minv_b + u * 16));   // undoes the power-of-two scale of the sums
    const float mA = dA.y * minv, mB = dB.y * minv;
    mm[0] = fmaf(mA, accm[0], mm[0]); mm[1] = fmaf(mA, accm[1], mm[1]);
    mm[2] = fmaf(mB, accm[2], mm[2]); mm[3] = fmaf(mB, accm[3], mm[3]);
}

// ---- Q6_K: w = d * sc_j * (q - 32), sc_j int8 per 16 weights (quantized.rs:268-329) -------------
// q = low nibble | two high bits << 4 is assembled bytewise (0..63).  A k32 MMA spans two scale
// groups, so it is issued twice with one half of B zeroed.  The -32 offset becomes
// -32 * sum_j sc_j * S_j with S_j the level sums over 16 activations: one f16 MMA per unit
// (A = the 16 scales of the row, B = S_j, all exact).
template <int QUARTER>
__device__ __forceinline__ uint32_t q6k_bytes(uint32_t W, uint32_t H)
{
    const uint32_t lo = ((QUARTER >> 1) ? (W >> 4) : W) & NIB;
    const uint32_t hs = (QUARTER == 0) ? (H << 4) : (QUARTER == 1) ? (H << 2) : (QUARTER == 2) ? H : (H >> 2);
    return and_or(hs, 0x30303030u, lo);
}

template <int QUARTER>
__device__ __forceinline__ void q6k_pair(const LaneCtx &L, const uint4 &Pr, const uint4 &Pq, uint32_t Hr0, uint32_t Hr1, uint32_t Hq0, uint32_t Hq1,
                                         uint32_t xaddr, uint32_t scA, uint32_t scB, int (&acc)[4])
{
    // words: slot q1*2 + h with q1 = QUARTER & 1
    const uint32_t a0 = q6k_bytes<QUARTER>(word_of(Pr, (QUARTER & 1) * 2), Hr0), a2 = q6k_bytes<QUARTER>(word_of(Pr, (QUARTER & 1) * 2 + 1), Hr1);
    const uint32_t a1 = q6k_bytes<QUARTER>(word_of(Pq, (QUARTER & 1) * 2), Hq0), a3 = q6k_bytes<QUARTER>(word_of(Pq, (QUARTER & 1) * 2 + 1), Hq1);
    const uint2 xb = ldb64(L, xaddr);
    int c4[4];
    imma16832<false>(c4, a0, a1, 0u, 0u, xb.x, 0u);          // scale group 2*QUARTER (k 0..15 of the 32)
    int sA = byte_s(scA, (QUARTER & 1) * 2), sB = byte_s(scB, (QUARTER & 1) * 2);
    acc[0] += sA * c4[0]; acc[1] += sA * c4[1]; acc[2] += sB * c4[2]; acc[3] += sB * c4[3];
    imma16832<false>(c4, 0u, 0u, a2, a3, 0u, xb.y);          // scale group 2*QUARTER + 1
    sA = byte_s(scA, (QUARTER & 1) * 2 + 1); sB = byte_s(scB, (QUARTER & 1) * 2 + 1);
    acc[0] += sA * c4[0]; acc[1] += sA * c4[1]; acc[2] += sB * c4[2]; acc[3] += sB * c4[3];
}

__device__ __forceinline__ void unit_q6k(uint32_t up, int u, const LaneCtx &L, float (&master)[4])
{
    const int r = L.r, c = L.c;
    uint4 P[4];
#pragma unroll
    for (int p = 0; p < 4; p++) P[p] = lds128(up + p * 512 + L.lane * 16);   // ql: (row r, n=0), (row r, n=1), (row r+8, n=0), (row r+8, n=1)
    const uint4 H0 = lds128(up + 2048 + L.lane * 16), H1 = lds128(up + 2560 + L.lane * 16);  // qh: row r, row r+8; word n*2 + h
    const uint4 sA = lds128(up + 3072 + r * 16), sB = lds128(up + 3072 + (r + 8) * 16);      // 16 int8 scales
    const uint32_t dw = lds32(up + 3328 + (r >> 1) * 4), dw8 = lds32(up + 3328 + ((r + 8) >> 1) * 4);
    const float2 dpA = h2_to_f2(dw), dpB = h2_to_f2(dw8);
    const float dA = (r & 1) ? dpA.y : dpA.x, dB = (r & 1) ? dpB.y : dpB.x;
    // offset term: T[row][col] = sum_j sc_j * S_j[col]
    float accT[4] = {0.f, 0.f, 0.f, 0.f};
    {
        const uint32_t sel = (c & 1) ? 0x5342u : 0x5140u;
        const uint32_t k1152 = 0x64806480u;   // (sc + 128) + 1024 - 1152 = sc
        const uint32_t wA0 = word_of(sA, c >> 1) ^ 0x80808080u, wA1 = word_of(sA, 2 + (c >> 1)) ^ 0x80808080u;
        const uint32_t wB0 = word_of(sB, c >> 1) ^ 0x80808080u, wB1 = word_of(sB, 2 + (c >> 1)) ^ 0x80808080u;
        const uint32_t sbase = L.sa_b + u * (kMaxCols * 32) + c * 4;
        hmma16816(accT, hsub2(prmt(wA0, 0x64646464u, sel), k1152), hsub2(prmt(wB0, 0x64646464u, sel), k1152),
                  hsub2(prmt(wA1, 0x64646464u, sel), k1152), hsub2(prmt(wB1, 0x64646464u, sel), k1152),
                  lds32(sbase), lds32(sbase + 16));
    }
    int acc[4] = {0, 0, 0, 0};
#pragma unroll
    for (int n = 0; n < 2; n++) {
        const uint32_t Hr0 = word_of(H0, n * 2), Hr1 = word_of(H0, n * 2 + 1), Hq0 = word_of(H1, n * 2), Hq1 = word_of(H1, n * 2 + 1);
        // MMA (n, quarter) covers k = 128n + 32*quarter + [0, 32): activation group 4u + 2n + quarter/2, sub = quarter & 1
        const uint32_t xg = L.xq_b + (4 * u + 2 * n) * 64 + c * 16;
        q6k_pair<0>(L, P[n], P[2 + n], Hr0, Hr1, Hq0, Hq1, xg, word_of(sA, 2 * n), word_of(sB, 2 * n), acc);
        q6k_pair<1>(L, P[n], P[2 + n], Hr0, Hr1, Hq0, Hq1, xg + 8, word_of(sA, 2 * n), word_of(sB, 2 * n), acc);
        q6k_pair<2>(L, P[n], P[2 + n], Hr0, Hr1, Hq0, Hq1, xg + 64, word_of(sA, 2 * n + 1), word_of(sB, 2 * n + 1), acc);
        q6k_pair<3>(L, P[n], P[2 + n], Hr0, Hr1, Hq0, Hq1, xg + 72, word_of(sA, 2 * n + 1), word_of(sB, 2 * n + 1), acc);
    }
    const uint2 alw = lds64(L.alam_b + u * (kMaxCols * 4));
    const float al0 = __uint_as_float(alw.x), al1 = __uint_as_float(alw.y);
    master[0] = fmaf(dA * al0, fmaf(-32.f, accT[0], (float)acc[0]), master[0]);
    master[1] = fmaf(dA * al1, fmaf(-32.f, accT[1], (float)acc[1]), master[1]);
    master[2] = fmaf(dB * al0, fmaf(-32.f, accT[2], (float)acc[2]), master[2]);
    master[3] = fmaf(dB * al1, fmaf(-32.f, accT[3], (float)acc[3]), master[3]);
}

// ---- Q4_0: w = d * (q - 8), f16 d per 32 weights (quantized.rs:182-225) -------------------------
__device__ __forceinline__ void unit_q40(uint32_t up, int u, const LaneCtx &L, float (&master)[4])
{
    const int r = L.r, c = L.c;
    const uint4 hA = lds128(up + 2048 + r * 16), hB = lds128(up + 2048 + (r + 8) * 16);   // 8 f16 scales per row
    const uint2 alw = lds64(L.alam_b + u * (kMaxCols * 4));
    const float al0 = __uint_as_float(alw.x), al1 = __uint_as_float(alw.y);
#pragma unroll
    for (int p = 0; p < 4; p++) {
        const uint4 q = lds128(up + p * 512 + L.lane * 16);   // (row r, blk 2p), (row r, blk 2p+1), (row r+8, blk 2p), (row r+8, blk 2p+1)
        const uint4 xb = ldb128(L, L.xq_b + (4 * u + p) * 64 + c * 16);
        const float2 sA = h2_to_f2(word_of(hA, p)), sB = h2_to_f2(word_of(hB, p));
#pragma unroll
        for (int e = 0; e < 2; e++) {
            const uint32_t wr = e ? q.y : q.x, wq = e ? q.w : q.z;
            int c4[4];
            imma16832<false>(c4, wr & NIB, wq & NIB, (wr >> 4) & NIB, (wq >> 4) & NIB, e ? xb.z : xb.x, e ? xb.w : xb.y);
            const int blk = 8 * u + 2 * p + e;
            const int s0 = (int)lds32(L.sa_c0 + blk * (kMaxCols * 4)), s1 = (int)lds32(L.sa_c1 + blk * (kMaxCols * 4));
            const float dA = e ? sA.y : sA.x, dB = e ? sB.y : sB.x;
            master[0] = fmaf(dA * al0, i2f_small(c4[0] - 8 * s0), master[0]);
            master[1] = fmaf(dA * al1, i2f_small(c4[1] - 8 * s1), master[1]);
            master[2] = fmaf(dB * al0, i2f_small(c4[2] - 8 * s0), master[2]);
            master[3] = fmaf(dB * al1, i2f_small(c4[3] - 8 * s1), master[3]);
        }
    }
}

// ---- Q8_0: w = d * q, int8 q (quantized.rs:227-260): the bytes are the A operand as stored ------
__device__ __forceinline__ void unit_q80(uint32_t up, int u, const LaneCtx &L, float (&master)[4])
{
    const int r = L.r, c = L.c;
    const uint4 hA = lds128(up + 4096 + r * 16), hB = lds128(up + 4096 + (r + 8) * 16);
    const uint2 alw = lds64(L.alam_b + u * (kMaxCols * 4));
    const float al0 = __uint_as_float(alw.x), al1 = __uint_as_float(alw.y);
#pragma unroll
    for (int b = 0; b < 8; b++) {
        const uint4 q = lds128(up + b * 512 + L.lane * 16);   // (row r, k 4c..), (row r, k 16+4c..), (row r+8, ...), (row r+8, ...)
        const uint2 xb = ldb64(L, L.xq_b + (4 * u + (b >> 1)) * 64 + c * 16 + (b & 1) * 8);
        int c4[4];
        imma16832<true>(c4, q.x, q.z, q.y, q.w, xb.x, xb.y);
        const float2 sA = h2_to_f2(word_of(hA, b >> 1)), sB = h2_to_f2(word_of(hB, b >> 1));
        const float dA = (b & 1) ? sA.y : sA.x, dB = (b & 1) ? sB.y : sB.x;
        master[0] = fmaf(dA * al0, i2f_small(c4[0]), master[0]);
        master[1] = fmaf(dA * al1, i2f_small(c4[1]), master[1]);
        master[2] = fmaf(dB * al0, i2f_small(c4[2]), master[2]);
        master[3] = fmaf(dB * al1, i2f_small(c4[3]), master[3]);
    }
}

template <int FMT>
__device__ __forceinline__ void process_unit(uint32_t up, int u, const LaneCtx &L, float (&master)[4], float (&mm)[4])
{
    if (FMT == TLB_GGML_Q4_K) unit_q4k(up, u, L, master, mm);
    else if (FMT == TLB_GGML_Q4_0) unit_q40(up, u, L, master);
    else if (FMT == TLB_GGML_Q8_0) unit_q80(up, u, L, master);
    else unit_q6k(up, u, L, master);
}

}  // namespace tlb
