// Streaming dequant-fused matvec for GGUF Q4_K / Q6_K / Q8_0 / Q4_0 weights (decode path,
// 1..4 activation rows).  Replaces mul_mv_q4_k_kernel / mul_mv_q6_k_kernel
// (crates/tl_cuda/src/cuda_kernels/autograd.cu:2813-2900, one thread per output, byte loads)
// and the dequantise-then-naive-matmul route for Q4_0/Q8_0
// (crates/tl_runtime/src/system.rs:236-264).
//
// Shape of the kernel (one persistent CTA per SM):
//   * the weight bytes of all tensors of the job form ONE linear stream of units
//     (16 rows x 256 weights, see quant.cu); CTA b takes the contiguous range
//     [U*b/G, U*(b+1)/G) - equal bytes per SM whatever the row count;
//   * a producer warp moves units global -> shared with 1-D bulk async copies
//     (cp.async.bulk + mbarrier complete_tx) through a ring of stages, independent of the
//     activations, so the HBM stream starts before the prologue has finished;
//   * 16 consumer warps each take one unit at a time: 128-bit conflict-free shared loads,
//     nibbles -> f16 pairs with one LOP3 + one HFMA2 per two weights (the 6-bit sub-block
//     scale is folded in exactly: sc*q <= 945 is an integer f16 represents), then
//     mma.sync.m16n8k16 with the activation as the B operand.  The activation is split
//     x = hi + lo into two f16 columns, so the product keeps ~22 bits of x although the
//     tensor core multiplies f16;
//   * per output tile the warps' fragments are summed in fixed order in shared memory and
//     added to the output with one atomicAdd per row; a tile is touched by at most two CTAs,
//     and a + b == b + a, so the result does not depend on scheduling.
// The prologue builds the activation in shared memory and can fuse what precedes the matvec
// in the decode chain: residual add + RMSNorm * weight, SiLU(gate) * up, or an embedding lookup.
#include "tlb_internal.h"

namespace tlb {

constexpr int kConsumerWarps = 16;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;
constexpr int kGroupStride = 144;  // bytes per 64 activations per column: 128 data + 16 pad (bank spread)

// ---------------------------------------------------------------- PTX helpers

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait: gives up after ~2 s, records the reason and raises the CTA-wide abort flag.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *err, int code)
{
    if (mbar_try_wait(bar, parity)) return true;
    unsigned long long t0 = global_ns();
    for (int it = 0;; it++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 63) == 63) {
            if (*abort_flag) return false;
            if (global_ns() - t0 > 2000000000ull) {
                *abort_flag = 1;
                atomicExch(err, code);
                return false;
            }
        }
    }
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void consumer_bar() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ uint4 lds128(uint32_t a)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a)
{
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a)
{
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t hfma2(uint32_t a, uint32_t b, uint32_t c)
{
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t hmul2(uint32_t a, uint32_t b)
{
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t hsub2(uint32_t a, uint32_t b)
{
    uint32_t d;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel)
{
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ float2 h2_to_f2(uint32_t h)
{
    return __half22float2(*reinterpret_cast<const __half2 *>(&h));
}
// D = A(16x16 f16, row) * B(16x8 f16, col) + C, f32 accumulate
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---------------------------------------------------------------- kernel parameters

struct MvParams {
    const uint8_t *w[3];
    float *out[3];
    int tiles_end[3];   // cumulative tile counts
    int n_rows[3];      // valid output rows per tensor
    int n_w;
    int upt;            // units per tile = K / 256
    int k;
    int m;              // activation rows, 1..4
    int total_units;
    int unit_bytes, stage_bytes, n_stages;
    int col_stride;     // bytes between activation columns in shared memory
    int prologue;
    const float *x, *x2, *norm_w;
    float eps;
    float *x_out;
    const float *emb_table;
    const int *token;
    float *zero_ptr[2];
    long long zero_n[2];
    int *err;
    int use_pdl;
};

// shared-memory slot (8 bytes = 4 halves [x0, x2, x1, x3]) of the k4-group t (0..15) inside a 64-group
template <int FMT>
__device__ __forceinline__ int xs_slot(int t)
{
    if (FMT == TLB_GGML_Q4_K) return (t & 7) * 2 + (t >> 3);              // (j, sub) -> j*2 + sub
    if (FMT == TLB_GGML_Q6_K) return t;
    return (((t >> 3) * 4) + (t & 3)) * 2 + ((t >> 2) & 1);               // (block, half, c) -> (block*4+c)*2 + half
}

__device__ __forceinline__ float silu_f(float g) { return g * (1.0f / (1.0f + expf(-g))); }

// Activation elements 4*k4 .. 4*k4+3 of row `mrow` as the matvec consumes them.  rms == 0 selects
// the statistics pass of PRO_ADD_NORM (returns x + x2 unnormalised).
__device__ __forceinline__ float4 prologue_value(const MvParams &p, const float *xbase, int mrow, int k4, float rms)
{
    const size_t row4 = (size_t)mrow * (p.k / 4) + k4;
    float4 v = __ldg(reinterpret_cast<const float4 *>(xbase) + row4);
    if (p.prologue == PRO_ADD_NORM) {
        if (p.x2) {
            float4 d = __ldg(reinterpret_cast<const float4 *>(p.x2) + row4);
            v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
        }
        if (rms != 0.f) {  // x / rms, then * weight, in the reference's order (crates/tl_cpu/src/ffi.rs:2444-2486)
            float4 w = __ldg(reinterpret_cast<const float4 *>(p.norm_w) + k4);
            v.x = __fdiv_rn(v.x, rms) * w.x; v.y = __fdiv_rn(v.y, rms) * w.y;
            v.z = __fdiv_rn(v.z, rms) * w.z; v.w = __fdiv_rn(v.w, rms) * w.w;
        }
    } else if (p.prologue == PRO_SILU_MUL) {
        float4 u = __ldg(reinterpret_cast<const float4 *>(p.x2) + row4);
        v.x = silu_f(v.x) * u.x; v.y = silu_f(v.y) * u.y; v.z = silu_f(v.z) * u.z; v.w = silu_f(v.w) * u.w;
    }
    return v;
}

// Shared-memory bookkeeping written by the prologue.
struct MvShared {
    float red_sum[kConsumerWarps];
    float red_max[kConsumerWarps];
    float inv_scale;     // 1 / (power-of-two scale applied to the activation)
    int abort_flag;
};

// Builds the activation columns in shared memory: column 2m holds hi = f16(s*x), column 2m+1 holds
// lo = f16(s*x - hi); s is a power of two that brings max|x| into [512, 1024) so that neither half
// overflows and sub-block sums of 32 stay below 65504.  For Q4_K also the per-32 sums (hi/lo).
template <int FMT>
__device__ void build_activation(const MvParams &p, MvShared *sh, uint8_t *xs, __half *xsum, int tid)
{
    const int lane = tid & 31, warp = tid >> 5;
    const int k4n = p.k / 4;
    const float *xbase = p.x;
    if (p.prologue == PRO_ADD_NORM && p.token) {
        int tok = __ldg(p.token);
        xbase = p.emb_table + (size_t)tok * p.k;
    }
    // pass 1: statistics
    float ssq = 0.f, amax = 0.f;
    for (int mrow = 0; mrow < p.m; mrow++)
        for (int k4 = tid; k4 < k4n; k4 += kConsumerThreads) {
            float4 v = prologue_value(p, xbase, mrow, k4, 0.f);
            if (p.prologue == PRO_ADD_NORM) {
                ssq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                float4 w = __ldg(reinterpret_cast<const float4 *>(p.norm_w) + k4);
                amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x * w.x), fabsf(v.y * w.y)), fmaxf(fabsf(v.z * w.z), fabsf(v.w * w.w))));
                if (p.x_out && blockIdx.x == 0) reinterpret_cast<float4 *>(p.x_out)[k4] = v;
            } else {
                amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
            }
        }
    for (int o = 16; o; o >>= 1) {
        ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    }
    if (lane == 0) { sh->red_sum[warp] = ssq; sh->red_max[warp] = amax; }
    consumer_bar();
    ssq = 0.f; amax = 0.f;
    for (int w = 0; w < kConsumerWarps; w++) { ssq += sh->red_sum[w]; amax = fmaxf(amax, sh->red_max[w]); }
    float rms = 0.f;
    if (p.prologue == PRO_ADD_NORM) {
        rms = sqrtf(ssq / (float)p.k + p.eps);
        amax = amax / rms;
    }
    float s = 1.f;
    if (amax > 0.f && amax < 3.0e38f) {
        int ex;
        frexpf(amax, &ex);          // amax = f * 2^ex, f in [0.5, 1)
        s = ldexpf(1.f, 10 - ex);   // amax * s in [512, 1024)
    }
    if (tid == 0) sh->inv_scale = 1.f / s;
    // pass 2: split and store
    for (int mrow = 0; mrow < p.m; mrow++) {
        uint8_t *col_hi = xs + (size_t)(2 * mrow) * p.col_stride;
        uint8_t *col_lo = col_hi + p.col_stride;
        for (int k4 = tid; k4 < k4n; k4 += kConsumerThreads) {  // k4n is a multiple of 64: whole warps stay in the loop
            float4 v = prologue_value(p, xbase, mrow, k4, rms);
            float y[4] = {v.x * s, v.y * s, v.z * s, v.w * s};
            __half h[4], l[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                h[e] = __float2half_rn(y[e]);
                l[e] = __float2half_rn(y[e] - __half2float(h[e]));
            }
            int G = k4 >> 4, t = k4 & 15;
            int off = G * kGroupStride + xs_slot<FMT>(t) * 8;
            __half2 h02 = __halves2half2(h[0], h[2]), h13 = __halves2half2(h[1], h[3]);
            __half2 l02 = __halves2half2(l[0], l[2]), l13 = __halves2half2(l[1], l[3]);
            *reinterpret_cast<uint2 *>(col_hi + off) = make_uint2(*reinterpret_cast<uint32_t *>(&h02), *reinterpret_cast<uint32_t *>(&h13));
            *reinterpret_cast<uint2 *>(col_lo + off) = make_uint2(*reinterpret_cast<uint32_t *>(&l02), *reinterpret_cast<uint32_t *>(&l13));
            if (FMT == TLB_GGML_Q4_K) {  // sums over sub-blocks of 32 = 8 consecutive k4 groups = 8 consecutive lanes
                float t4 = (y[0] + y[1]) + (y[2] + y[3]);
                t4 += __shfl_xor_sync(0xffffffffu, t4, 1);
                t4 += __shfl_xor_sync(0xffffffffu, t4, 2);
                t4 += __shfl_xor_sync(0xffffffffu, t4, 4);
                if ((lane & 7) == 0) {
                    __half sh_ = __float2half_rn(t4);
                    __half sl_ = __float2half_rn(t4 - __half2float(sh_));
                    int sb = k4 >> 3;
                    xsum[(size_t)(2 * mrow) * (p.k / 32) + sb] = sh_;
                    xsum[(size_t)(2 * mrow + 1) * (p.k / 32) + sb] = sl_;
                }
            }
        }
    }
    consumer_bar();
}

// ---------------------------------------------------------------- per-unit consumers
// Common frame: lane (r, c) = (lane >> 2, lane & 3) owns rows r and r+8 of the 16-row tile.  In the
// MMA the B column index is also r, so `xb` points at activation column min(r, ...) (hi for even,
// lo for odd columns).  acc[0], acc[1] are row r columns 2c, 2c+1; acc[2], acc[3] row r+8.

#define H2_1024 0x64006400u

__device__ __forceinline__ uint32_t word_of(const uint4 &v, int i)
{
    return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w));
}

// Q4_K.  Lane c owns the 64-weight group c of the super-block.  The 6-bit scale is folded into the
// A operand: (1024 + q) * sc - 1024 * sc = sc * q exactly (<= 945), so one accumulator serves the
// whole super-block and is scaled by d once.  The mins enter through a 17th MMA whose A operand is
// the pair of 6-bit mins and whose B operand is the pair of 32-element activation sums.
__device__ __forceinline__ void q4k_scales(const uint4 &h, int c, uint32_t &SLO, uint32_t &SHI, uint32_t &BLO,
                                           uint32_t &BHI, uint32_t &MN)
{
    // bytes 4..15 of the header: get_scale_min_k4 packing (crates/tl_runtime/src/quantized.rs:404-415)
    uint32_t sc_lo4 = h.y & 0x3F3F3F3Fu, mn_lo4 = h.z & 0x3F3F3F3Fu;
    uint32_t sc_hi4 = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);
    uint32_t mn_hi4 = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
    uint32_t scw = (c < 2) ? sc_lo4 : sc_hi4, mnw = (c < 2) ? mn_lo4 : mn_hi4;
    uint32_t sel = (c & 1) ? 0x5342u : 0x5140u;       // bytes (2,3) or (0,1) -> f16 pair 0x64xx = 1024 + value
    uint32_t S = hsub2(prmt(scw, 0x64646464u, sel), H2_1024);   // (sc[2c], sc[2c+1])
    MN = hsub2(prmt(mnw, 0x64646464u, sel), H2_1024);           // (m[2c], m[2c+1])
    uint32_t T = hmul2(S, 0x2C003C00u);   // (sc_a, sc_b / 16)
    uint32_t U = hmul2(S, 0xD400E400u);   // (-1024 sc_a, -64 sc_b)
    SLO = prmt(T, T, 0x1010u); SHI = prmt(T, T, 0x3232u);
    BLO = prmt(U, U, 0x1010u); BHI = prmt(U, U, 0x3232u);
}

__device__ __forceinline__ void unit_q4k(uint32_t up, int ukg, uint32_t xb, uint32_t xsumb, int lane, float (&master)[4])
{
    const int r = lane >> 2, c = lane & 3;
    const uint4 hA = lds128(up + 2048 + r * 16), hB = lds128(up + 2048 + (r + 8) * 16);
    uint4 q[4];
#pragma unroll
    for (int p = 0; p < 4; p++) q[p] = lds128(up + p * 512 + lane * 16);
    uint32_t sloA, shiA, bloA, bhiA, mnA, sloB, shiB, bloB, bhiB, mnB;
    q4k_scales(hA, c, sloA, shiA, bloA, bhiA, mnA);
    q4k_scales(hB, c, sloB, shiB, bloB, bhiB, mnB);
    float accq[4] = {0.f, 0.f, 0.f, 0.f}, accm[4] = {0.f, 0.f, 0.f, 0.f};
    mma16816(accm, mnA, mnB, 0u, 0u, lds32(xsumb + (8 * ukg + 2 * c) * 2), 0u);
    const uint32_t xg = xb + (4 * ukg + c) * kGroupStride;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const uint32_t wr = word_of(q[j >> 2], j & 3), wq = word_of(q[2 + (j >> 2)], j & 3);
        const uint4 b = lds128(xg + j * 16);
        const uint32_t wr8 = wr >> 8, wq8 = wq >> 8;
        mma16816(accq,
                 hfma2((wr & 0x000F000Fu) | H2_1024, sloA, bloA), hfma2((wq & 0x000F000Fu) | H2_1024, sloB, bloB),
                 hfma2((wr8 & 0x000F000Fu) | H2_1024, sloA, bloA), hfma2((wq8 & 0x000F000Fu) | H2_1024, sloB, bloB),
                 b.x, b.y);
        mma16816(accq,
                 hfma2((wr & 0x00F000F0u) | H2_1024, shiA, bhiA), hfma2((wq & 0x00F000F0u) | H2_1024, shiB, bhiB),
                 hfma2((wr8 & 0x00F000F0u) | H2_1024, shiA, bhiA), hfma2((wq8 & 0x00F000F0u) | H2_1024, shiB, bhiB),
                 b.z, b.w);
    }
    const float2 dA = h2_to_f2(hA.x), dB = h2_to_f2(hB.x);  // (d, dmin)
    master[0] += dA.x * accq[0] - dA.y * accm[0];
    master[1] += dA.x * accq[1] - dA.y * accm[1];
    master[2] += dB.x * accq[2] - dB.y * accm[2];
    master[3] += dB.x * accq[3] - dB.y * accm[3];
}

// Q4_0.  One MMA = one half (16 weights) of one 32-block, all four c lanes inside the same block;
// the f16 block scale cannot be folded exactly, so each block gets a fresh accumulator scaled in f32.
__device__ __forceinline__ void unit_q40(uint32_t up, int ukg, uint32_t xb, int lane, float (&master)[4])
{
    const int r = lane >> 2, c = lane & 3;
    const uint4 hA = lds128(up + 2048 + r * 16), hB = lds128(up + 2048 + (r + 8) * 16);
    uint4 q[4];
#pragma unroll
    for (int p = 0; p < 4; p++) q[p] = lds128(up + p * 512 + lane * 16);
#pragma unroll
    for (int b = 0; b < 8; b++) {
        const int p = b >> 1, e = b & 1;
        const uint32_t wr = e ? q[p].y : q[p].x, wq = e ? q[p].w : q[p].z;
        const uint32_t wr8 = wr >> 8, wq8 = wq >> 8;
        const uint4 xv = lds128(xb + (4 * ukg + p) * kGroupStride + (e * 4 + c) * 16);
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        // low nibbles: (1024 + q) - 1032 = q - 8
        mma16816(acc, hsub2((wr & 0x000F000Fu) | H2_1024, 0x64086408u), hsub2((wq & 0x000F000Fu) | H2_1024, 0x64086408u),
                 hsub2((wr8 & 0x000F000Fu) | H2_1024, 0x64086408u), hsub2((wq8 & 0x000F000Fu) | H2_1024, 0x64086408u),
                 xv.x, xv.y);
        // high nibbles: (1024 + 16 q) / 16 - 72 = q - 8
        mma16816(acc, hfma2((wr & 0x00F000F0u) | H2_1024, 0x2C002C00u, 0xD480D480u), hfma2((wq & 0x00F000F0u) | H2_1024, 0x2C002C00u, 0xD480D480u),
                 hfma2((wr8 & 0x00F000F0u) | H2_1024, 0x2C002C00u, 0xD480D480u), hfma2((wq8 & 0x00F000F0u) | H2_1024, 0x2C002C00u, 0xD480D480u),
                 xv.z, xv.w);
        const float2 sA = h2_to_f2(word_of(hA, b >> 1)), sB = h2_to_f2(word_of(hB, b >> 1));
        const float dA = (b & 1) ? sA.y : sA.x, dB = (b & 1) ? sB.y : sB.x;
        master[0] += dA * acc[0]; master[1] += dA * acc[1];
        master[2] += dB * acc[2]; master[3] += dB * acc[3];
    }
}

// Q8_0.  int8 -> f16: flip the sign bit (q + 128 as unsigned), drop the byte into the mantissa of
// 1024.0 with PRMT, subtract 1152.
__device__ __forceinline__ void unit_q80(uint32_t up, int ukg, uint32_t xb, int lane, float (&master)[4])
{
    const int r = lane >> 2, c = lane & 3;
    const uint4 hA = lds128(up + 4096 + r * 16), hB = lds128(up + 4096 + (r + 8) * 16);
#pragma unroll
    for (int b = 0; b < 8; b++) {
        uint4 q = lds128(up + b * 512 + lane * 16);
        q.x ^= 0x80808080u; q.y ^= 0x80808080u; q.z ^= 0x80808080u; q.w ^= 0x80808080u;
        const uint4 xv = lds128(xb + (4 * ukg + (b >> 1)) * kGroupStride + ((b & 1) * 4 + c) * 16);
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        const uint32_t k1152 = 0x64806480u;
        mma16816(acc, hsub2(prmt(q.x, 0x64646464u, 0x6240u), k1152), hsub2(prmt(q.z, 0x64646464u, 0x6240u), k1152),
                 hsub2(prmt(q.x, 0x64646464u, 0x7341u), k1152), hsub2(prmt(q.z, 0x64646464u, 0x7341u), k1152), xv.x, xv.y);
        mma16816(acc, hsub2(prmt(q.y, 0x64646464u, 0x6240u), k1152), hsub2(prmt(q.w, 0x64646464u, 0x6240u), k1152),
                 hsub2(prmt(q.y, 0x64646464u, 0x7341u), k1152), hsub2(prmt(q.w, 0x64646464u, 0x7341u), k1152), xv.z, xv.w);
        const float2 sA = h2_to_f2(word_of(hA, b >> 1)), sB = h2_to_f2(word_of(hB, b >> 1));
        const float dA = (b & 1) ? sA.y : sA.x, dB = (b & 1) ? sB.y : sB.x;
        master[0] += dA * acc[0]; master[1] += dA * acc[1];
        master[2] += dB * acc[2]; master[3] += dB * acc[3];
    }
}

// Q6_K.  One MMA = one 16-weight scale group.  q = low nibble | two high bits << 4, minus 32.
template <int QUARTER>
__device__ __forceinline__ void q6k_pair(uint32_t W, uint32_t Hh, uint32_t &v02, uint32_t &v13)
{
    const uint32_t lo = (QUARTER >> 1) ? (W >> 4) : W;        // high nibbles for quarters 2, 3
    const int sh = 2 * QUARTER;                               // position of the 2 high bits in each qh byte
    const uint32_t h02 = (sh <= 4) ? (Hh << (4 - sh)) : (Hh >> (sh - 4));
    const uint32_t h13 = Hh >> (4 + sh);
    v02 = hsub2((lo & 0x000F000Fu) | (h02 & 0x00300030u) | H2_1024, 0x64206420u);
    v13 = hsub2(((lo >> 8) & 0x000F000Fu) | (h13 & 0x00300030u) | H2_1024, 0x64206420u);
}

template <int QUARTER>
__device__ __forceinline__ void q6k_mma(uint32_t Wr, uint32_t Hr, uint32_t Wq, uint32_t Hq, uint32_t xaddr,
                                        float sr, float sq, float (&master)[4])
{
    uint32_t a0, a2, a1, a3;
    q6k_pair<QUARTER>(Wr, Hr, a0, a2);
    q6k_pair<QUARTER>(Wq, Hq, a1, a3);
    const uint2 b = lds64(xaddr);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    mma16816(acc, a0, a1, a2, a3, b.x, b.y);
    master[0] += sr * acc[0]; master[1] += sr * acc[1];
    master[2] += sq * acc[2]; master[3] += sq * acc[3];
}

__device__ __forceinline__ float i8_of(const uint4 &v, int j)
{
    return (float)(int)(int8_t)((word_of(v, j >> 2) >> (8 * (j & 3))) & 0xFFu);
}

__device__ __forceinline__ void unit_q6k(uint32_t up, int ukg, uint32_t xb, int lane, float (&master)[4])
{
    const int r = lane >> 2, c = lane & 3;
    uint4 P[4];
#pragma unroll
    for (int p = 0; p < 4; p++) P[p] = lds128(up + p * 512 + lane * 16);   // ql: (row r, n=0), (row r, n=1), (row r+8, n=0), (row r+8, n=1)
    const uint4 H0 = lds128(up + 2048 + lane * 16), H1 = lds128(up + 2560 + lane * 16);  // qh: row r, row r+8
    const uint4 sA = lds128(up + 3072 + r * 16), sB = lds128(up + 3072 + (r + 8) * 16);
    const uint32_t dw = lds32(up + 3328 + (r >> 1) * 4), dw8 = lds32(up + 3328 + ((r + 8) >> 1) * 4);
    const float2 dpA = h2_to_f2(dw), dpB = h2_to_f2(dw8);
    const float dA = (r & 1) ? dpA.y : dpA.x, dB = (r & 1) ? dpB.y : dpB.x;
#pragma unroll
    for (int n = 0; n < 2; n++)
#pragma unroll
        for (int jj = 0; jj < 2; jj++) {
            const uint32_t Wr0 = word_of(P[n], jj), Wr1 = word_of(P[n], 2 + jj), Hr = word_of(H0, n * 2 + jj);
            const uint32_t Wq0 = word_of(P[2 + n], jj), Wq1 = word_of(P[2 + n], 2 + jj), Hq = word_of(H1, n * 2 + jj);
            // MMA index j = 8n + 2*quarter + jj; activation slot: group 4*ukg + j/4, k4 (j%4)*4 + c
#define Q6K_STEP(QUARTER, WR, WQ)                                                                       \
            {                                                                                           \
                const int j = 8 * n + 2 * QUARTER + jj;                                                 \
                q6k_mma<QUARTER>(WR, Hr, WQ, Hq, xb + (4 * ukg + (j >> 2)) * kGroupStride + ((j & 3) * 4 + c) * 8, \
                                 dA * i8_of(sA, j), dB * i8_of(sB, j), master);                          \
            }
            Q6K_STEP(0, Wr0, Wq0)
            Q6K_STEP(1, Wr1, Wq1)
            Q6K_STEP(2, Wr0, Wq0)
            Q6K_STEP(3, Wr1, Wq1)
#undef Q6K_STEP
        }
}

template <int FMT>
__device__ __forceinline__ void process_unit(uint32_t up, int ukg, uint32_t xb, uint32_t xsumb, int lane, float (&master)[4])
{
    if (FMT == TLB_GGML_Q4_K) unit_q4k(up, ukg, xb, xsumb, lane, master);
    else if (FMT == TLB_GGML_Q4_0) unit_q40(up, ukg, xb, lane, master);
    else if (FMT == TLB_GGML_Q8_0) unit_q80(up, ukg, xb, lane, master);
    else unit_q6k(up, ukg, xb, lane, master);
}

// ---------------------------------------------------------------- the kernel

__device__ __forceinline__ bool mbar_wait_drain(uint32_t bar, uint32_t parity)
{
    unsigned long long t0 = global_ns();
    for (int it = 0;; it++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 63) == 63 && global_ns() - t0 > 1000000000ull) return false;
    }
}

__device__ __forceinline__ const uint8_t *unit_src(const MvParams &p, int u)
{
    int tile = u / p.upt, uk = u - tile * p.upt;
    int wi = (tile >= p.tiles_end[0]) + (tile >= p.tiles_end[1]);
    int t0 = wi == 0 ? 0 : p.tiles_end[wi - 1];
    return p.w[wi] + ((size_t)(tile - t0) * p.upt + uk) * p.unit_bytes;
}

template <int FMT>
__global__ void __launch_bounds__(kThreads, 1) qmatvec_kernel(const __grid_constant__ MvParams p)
{
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nst = p.n_stages;
    uint8_t *ring = smem;
    uint8_t *xs = ring + (size_t)nst * p.stage_bytes;
    __half *xsum = reinterpret_cast<__half *>(xs + (size_t)2 * p.m * p.col_stride);
    const int xsum_bytes = (FMT == TLB_GGML_Q4_K) ? ((2 * p.m * (p.k / 32) * 2 + 15) & ~15) : 0;
    float *red = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(xsum) + xsum_bytes);  // [2][warps][4][16]
    uint64_t *bars = reinterpret_cast<uint64_t *>(red + 2 * kConsumerWarps * 64);
    MvShared *sh = reinterpret_cast<MvShared *>(bars + 2 * nst);
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + nst * 8;
    const uint32_t ring_u32 = smem_u32(ring);

    const int G = gridDim.x, b = blockIdx.x;
    const int u0 = (int)((long long)p.total_units * b / G), u1 = (int)((long long)p.total_units * (b + 1) / G);
    const int n_units = u1 - u0;

    if (tid == 0) {
        for (int s = 0; s < nst; s++) { mbar_init(full0 + s * 8, 1); mbar_init(empty0 + s * 8, 1); }
        sh->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    volatile int *abortp = &sh->abort_flag;

    if (warp == kConsumerWarps) {
        // ---- producer: each lane streams the units i = lane, lane + 32, ... of this CTA's range.
        // Weights do not depend on the previous kernel, so no dependency wait here.
        int i = lane;
        for (; i < n_units; i += 32) {
            const int slot = i % nst, use = i / nst;
            if (use > 0 && !mbar_wait(empty0 + slot * 8, (use - 1) & 1, abortp, p.err, 1)) break;
            mbar_expect_tx(full0 + slot * 8, p.unit_bytes);
            bulk_g2s(ring_u32 + slot * p.stage_bytes, unit_src(p, u0 + i), p.unit_bytes, full0 + slot * 8);
        }
        if (*abortp) {
            // give the copies this lane still has in flight a bounded time to land before the CTA exits
            for (int k = i - 32; k >= 0 && k > i - 32 - nst * 32; k -= 32) mbar_wait_drain(full0 + (k % nst) * 8, (k / nst) & 1);
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
    for (int z = 0; z < 2; z++)
        if (p.zero_ptr[z])
            for (long long idx = (long long)b * kConsumerThreads + tid; idx < p.zero_n[z]; idx += (long long)G * kConsumerThreads)
                p.zero_ptr[z][idx] = 0.f;
    build_activation<FMT>(p, sh, xs, xsum, tid);
    const float inv_s = sh->inv_scale;
    const int r = lane >> 2, c = lane & 3;
    const int col = (r < 2 * p.m) ? r : (r & 1);
    const uint32_t xb = smem_u32(xs) + col * p.col_stride;
    const uint32_t xsumb = smem_u32(xsum) + col * (p.k / 32) * 2;

    int u = u0, par = 0;
    while (u < u1) {
        const int tile = u / p.upt;
        const int seg_end = min(u1, (tile + 1) * p.upt);
        float master[4] = {0.f, 0.f, 0.f, 0.f};
        for (int uu = u + warp; uu < seg_end; uu += kConsumerWarps) {
            const int rel = uu - u0, slot = rel % nst, use = rel / nst;
            if (!mbar_wait(full0 + slot * 8, use & 1, abortp, p.err, 2)) break;
            process_unit<FMT>(ring_u32 + slot * p.stage_bytes, uu - tile * p.upt, xb, xsumb, lane, master);
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + slot * 8);
        }
        float *rp = red + (size_t)par * kConsumerWarps * 64 + warp * 64;
        if (c < p.m) {
            rp[c * 16 + r] = master[0] + master[1];       // hi column + lo column
            rp[c * 16 + r + 8] = master[2] + master[3];
        }
        consumer_bar();
        if (tid < p.m * 16) {
            const int mm = tid >> 4, row = tid & 15;
            const float *rq = red + (size_t)par * kConsumerWarps * 64 + mm * 16 + row;
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; w++) sum += rq[w * 64];
            const int wi = (tile >= p.tiles_end[0]) + (tile >= p.tiles_end[1]);
            const int t0 = wi == 0 ? 0 : p.tiles_end[wi - 1];
            const int grow = (tile - t0) * 16 + row;
            if (grow < p.n_rows[wi]) atomicAdd(p.out[wi] + (size_t)mm * p.n_rows[wi] + grow, sum * inv_s);
        }
        u = seg_end;
        par ^= 1;
    }
}

// ---------------------------------------------------------------- host side

static size_t smem_fixed_bytes(int type, int m, int64_t k, int *col_stride)
{
    int cs = (int)(((k / 64) * kGroupStride + 127) / 128 * 128) + 64;  // == 64 mod 128: hi and lo columns on different banks
    if (col_stride) *col_stride = cs;
    size_t xsum = type == TLB_GGML_Q4_K ? (size_t)((2 * m * (k / 32) * 2 + 15) & ~15) : 0;
    return (size_t)2 * m * cs + xsum + 2 * kConsumerWarps * 64 * sizeof(float) + sizeof(MvShared) + 64;
}

size_t qmatvec_max_k(int m)
{
    Context *c = ctx();
    size_t budget = c ? c->smem_optin : 232448;
    size_t k = 256;
    while (smem_fixed_bytes(TLB_GGML_Q4_K, m, (int64_t)(k + 256), nullptr) + 8 * (4352 + 128 + 16) <= budget) k += 256;
    return k;
}

template <int FMT>
static tlb_status launch_fmt(const MvParams &p, int grid, size_t smem, bool pdl)
{
    static bool attr_set = false;
    if (!attr_set) {
        TLB_CUDA(cudaFuncSetAttribute(qmatvec_kernel<FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ctx()->smem_optin));
        attr_set = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx()->stream;
    cudaLaunchAttribute at[1];
    if (pdl) {
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at;
        cfg.numAttrs = 1;
    }
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
    if (tiles * p.upt > INT32_MAX) return fail(TLB_ERR_SHAPE, "too many units for one launch");
    p.total_units = (int)(tiles * p.upt);
    p.unit_bytes = f->unit_bytes;
    p.stage_bytes = (f->unit_bytes + 127) / 128 * 128;
    size_t fixed = smem_fixed_bytes(job.type, job.m, job.k, &p.col_stride);
    size_t budget = c->smem_optin;
    if (fixed + 8 * (size_t)(p.stage_bytes + 16) > budget)
        return fail(TLB_ERR_SHAPE, "K = %lld with %d rows needs more shared memory than one SM has (max K %zu)",
                    (long long)job.k, job.m, qmatvec_max_k(job.m));
    int nst = (int)((budget - fixed) / (p.stage_bytes + 16));
    if (nst > 64) nst = 64;
    p.n_stages = nst;
    size_t smem = fixed + (size_t)nst * (p.stage_bytes + 16);
    p.prologue = job.prologue;
    p.x = job.x; p.x2 = job.x2; p.norm_w = job.norm_w; p.eps = job.eps; p.x_out = job.x_out;
    p.emb_table = job.emb_table; p.token = job.token;
    for (int z = 0; z < 2; z++) { p.zero_ptr[z] = job.zero_ptr[z]; p.zero_n[z] = job.zero_n[z]; }
    p.err = c->err_flag;
    p.use_pdl = job.pdl ? 1 : 0;
    if (!p.x && !(p.prologue == PRO_ADD_NORM && p.token)) return fail(TLB_ERR_NULL, "null activation");
    int grid = (int)std::min<int64_t>(c->sm_count, tiles);  // >= upt units per CTA: at most two CTAs touch a tile
    switch (job.type) {
    case TLB_GGML_Q4_K: return launch_fmt<TLB_GGML_Q4_K>(p, grid, smem, job.pdl);
    case TLB_GGML_Q6_K: return launch_fmt<TLB_GGML_Q6_K>(p, grid, smem, job.pdl);
    case TLB_GGML_Q8_0: return launch_fmt<TLB_GGML_Q8_0>(p, grid, smem, job.pdl);
    default: return launch_fmt<TLB_GGML_Q4_0>(p, grid, smem, job.pdl);
    }
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
