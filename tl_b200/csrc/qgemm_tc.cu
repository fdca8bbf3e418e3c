// Quantized-weight GEMM for many activation rows (prompt processing, M > 16), up to three weights per launch:
//     Y[M, N] = X[M, K] . W^T,   W = GGUF Q4_K / Q6_K / Q4_0 / Q8_0 bytes in the tiled unit layout.
// It stands behind the same entry point as the streaming matvec (tl_qtensor_matmul,
// crates/tl_runtime/src/system.rs:180-382, which dequantises the whole weight to f32, transposes it
// and calls a one-thread-per-output matmul); here the weight is read once per tile of 256 activation
// rows and never exists in f32.
//
// One CTA computes 128 weight rows x NT activation rows (NT <= 256) on the 5th-generation tensor cores:
//   * the weight tile is the A operand (MMA M = 128) and lives in TENSOR MEMORY, never in shared memory: sixteen
//     producer warps (two per 16 weight rows, each taking two of a unit's four 64-wide groups) read the quantized
//     units with coalesced 16-byte loads, dequantise in registers (f16 pair arithmetic on exact integers, see
//     store4) and write their 16 rows x 64 K of a stage with one tcgen05.st (eight stages of 32 columns beside the
//     accumulator's 256);
//   * the activation tile is the B operand (MMA N = NT): f16 rows, brought into a shared-memory ring by TMA
//     (cp.async.bulk.tensor.2d, 128-byte swizzle, rows past M filled with zeros).  The ring is as deep as shared
//     memory allows (6 stages of 32 KB at NT = 256, 16 for narrow tiles): a TMA load takes ~1.5 us from request to
//     arrival, so a K step can only be as short as that divided by the depth;
//   * one thread issues tcgen05.mma (kind::f16, A from tensor memory, B from shared memory, f32 accumulate) for each
//     64-wide K step as soon as its barrier has the eight producer warps' arrivals and the TMA bytes; one
//     tcgen05.commit per K step reports its completion, which frees the weight stage for the producers (8 K steps
//     later) and the activation stage for the TMA thread (ring depth later);
//   * the accumulator lives in tensor memory (128 lanes x NT columns f32); after the last K step the
//     producer warps read it back with tcgen05.ld, undo the per-row activation scaling and write
//     Y[token][row] (32 consecutive floats per warp store).
// Activations are converted to f16 once per call with a power-of-two scale per row (so the largest
// element sits near 2^14 and nothing overflows or underflows); the scale is removed exactly in the
// epilogue.  Operand rounding is therefore 2^-12 relative per element, accumulated in f32.
//
// Every wait on an mbarrier is bounded (qmv_common.cuh: mbar_wait); when one runs out the CTA sets the
// context's error word, lets its outstanding copies land (bounded), frees its tensor memory and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cudaTypedefs.h>

#include <algorithm>

#include "tc05.cuh"

namespace tlb {

namespace {

constexpr int kGemmRows = 128;      // weight rows per CTA (MMA M)
constexpr int kGemmBK = 64;         // K per stage: one 128-byte swizzle row of f16

constexpr int kGemmProducers = 16;  // dequantising warps: two per 16 weight rows, two 64-groups of every unit each
constexpr int kGemmThreads = (kGemmProducers + 2) * 32;   // + the TMA warp and the MMA / tensor-memory warp
// Tensor memory: accumulator in columns [0, 256), weight stages (128 lanes x 32 columns of f16 pairs each) above
constexpr int kTmemCols = 512;
constexpr int kTmemA0 = 256;
constexpr int kStageACols = kGemmBK / 2;
constexpr int kGemmAStages = 8;
// Shared memory: the activation ring.  One barrier pair per K step in flight: slot kt % slots, slots = max(8, ring depth)
constexpr int kGemmBBytes = 192 * 1024;
constexpr int kGemmMaxSlots = 16;
constexpr int kGemmSmemMax = kGemmBBytes + 1024 + 8 * (2 * kGemmMaxSlots + 1) + 64;   // ring + alignment slack + barriers
constexpr int kGemmMaxW = 3;        // weights of one launch (q | k | v share their activations)

struct GemmParams {
    const uint8_t *w[kGemmMaxW];   // tiled units of each weight
    float *out[kGemmMaxW];         // [m, n[i]]
    int n[kGemmMaxW];              // weight rows (output features)
    int n_tiles16[kGemmMaxW];      // 16-row tiles
    int rt_end[kGemmMaxW];         // CTA row tiles (128 rows) up to and including weight i
    int n_w;
    int64_t upt;            // units per 16-row tile (K / 256)
    int m;                  // activation rows
    int nt;                 // activation rows per CTA (MMA N)
    int nb;                 // depth of the activation ring (stages)
    int gs;                 // 64-wide K groups per stage: 1, or 4 (a whole 256-wide unit per barrier round) for tiles of up to 64 rows
    int kt_total;           // K / 64
    int unit_bytes;
    const float *inv_scale; // [m]
    const float *resid;     // [m, n] added to the result, or null
    int *err;
    // K-splits (few activation rows on a narrow weight: too few 128-row tiles to fill the SMs): grid.z CTAs share a tile,
    // each over kt_total / splits of the K steps, writing its partial product to part[split][m][n_all]; a second small
    // launch adds the splits (and the residual).  splits == 1: the result goes straight to out.
    int splits;
    float *part;
    int n_all;              // columns of one partial row: the sum of the weights' rows
    int col0[kGemmMaxW];    // first column of weight i inside a partial row
};

__device__ __forceinline__ uint32_t hfma2u(uint32_t a, uint32_t b, uint32_t c)
{
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t hmul2u(uint32_t a, uint32_t b)
{
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint32_t h2_of(float a)   // (a, a) rounded to f16
{
    __half2 h = __float2half2_rn(a);
    return *reinterpret_cast<uint32_t *>(&h);
}
// Byte i of `w` in both halves of an f16 pair, as the exact integer it is (0..255): 0x6400 | byte is 1024 + byte.
__device__ __forceinline__ uint32_t byte_h2(uint32_t w, int i)
{
    return hsub2(prmt(w, 0x64646464u, 0x4040u | (uint32_t)i | ((uint32_t)i << 8)), 0x64006400u);
}

// One warp's share of one weight stage: 16 rows x 64 K as the A operand of the MMA, in tensor memory.  tcgen05.st
// writes 16 lanes x 256 bits at a time: lane (r, c) = (lane / 4, lane % 4) of the warp gives, for each 16-wide K chunk
// j, two 32-bit columns (2 c and 2 c + 1 of the chunk's eight, i.e. K 16 j + 4 c .. + 3 as two f16 pairs) of row r and
// two of row r + 8 - the ownership the unit layout gives the lanes anyway.  The sixteen words of a 64-group are
// collected here and stored with one instruction: v[4 j + 2 rs + {0, 1}] = chunk j, row r + 8 rs.
struct AFrag {
    uint32_t v[16];
    __device__ __forceinline__ void flush(uint32_t taddr) const
    {
        asm volatile("tcgen05.st.sync.aligned.16x256b.x4.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                     ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
                       "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]) : "memory");
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    }
};
// Four weights from the four bytes b0..b3 of `bytes` (each 0..255), in f16 pair arithmetic:
//     w = (b * p1 + p2) * p3 + p4        (p1..p4: the same f16 value in both halves)
// The bytes enter as 1024 + b (0x6400 | b), which is exact, and both fused multiply-adds round once.
// The two words hold the weights in the order (b0, b2, b1, b3): inside every group of four the middle two K positions
// are exchanged, and the activation rows are written in the same order (x_to_f16_kernel), which leaves every dot
// product unchanged.  They become chunk j of row r + 8 rs.
__device__ __forceinline__ void store4(AFrag &f, int j, int rs, uint32_t bytes, uint32_t p1, uint32_t p2, uint32_t p3, uint32_t p4)
{
    const uint32_t x02 = prmt(bytes, 0x64646464u, 0x4240u), x13 = prmt(bytes, 0x64646464u, 0x4341u);   // (1024 + b0, 1024 + b2), (1024 + b1, 1024 + b3)
    f.v[4 * j + 2 * rs] = hfma2u(hfma2u(x02, p1, p2), p3, p4);
    f.v[4 * j + 2 * rs + 1] = hfma2u(hfma2u(x13, p1, p2), p3, p4);
}
constexpr uint32_t kH2One = 0x3C003C00u;    // (1, 1)
constexpr uint32_t kH2Zero = 0u;
// (-(1024 + off), ...) for off in {8, 32, 128}: 1024 + b - (1024 + off) = b - off, exactly
constexpr uint32_t kH2Neg1032 = 0xE408E408u, kH2Neg1056 = 0xE420E420u, kH2Neg1152 = 0xE480E480u;

// ---- Q4_K: w = d * sc * q - dmin * m (crates/tl_runtime/src/quantized.rs:337-415).  The 6-bit (scale, min)
// pairs of four sub-blocks at a time, one per byte, unpacked from the 12 packed bytes as get_scale_min_k4 does:
// sub-blocks 0..3 (upper = false) or 4..7 (upper = true).  h = [d | dmin, q[0..3], q[4..7], q[8..11]].
__device__ __forceinline__ void q4k_scales4(const uint4 &h, bool upper, uint32_t &scw, uint32_t &mw)
{
    if (!upper) {
        scw = h.y & 0x3F3F3F3Fu;
        mw = h.z & 0x3F3F3F3Fu;
    } else {
        scw = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);
        mw = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
    }
}
// store4 parameters of one sub-block: (1024 + q) * sc - 1024 sc = q sc exactly, then * d - dmin m
struct Q4KSub { uint32_t sc, c, ndm; };
__device__ __forceinline__ Q4KSub q4k_sub(uint32_t scw, uint32_t mw, int byte, uint32_t dmin2)
{
    Q4KSub o;
    o.sc = byte_h2(scw, byte);
    o.c = hmul2u(o.sc, 0xE400E400u);                             // -1024 sc, exact
    o.ndm = hmul2u(byte_h2(mw, byte), dmin2) ^ 0x80008000u;      // -(dmin m), rounded once
    return o;
}

// One warp's registers for one Q4_K unit (16 rows x 256 weights): lane (r, c) = (lane / 4, lane % 4)
// holds, per 64-group G, the words [row r: bytes 4c..4c+3 | row r: bytes 16+4c.. | row r+8: same two],
// plus the 16-byte headers (d, dmin, packed scales) of rows r and r + 8.
struct Q4KRegs {
    uint4 q[2];
    uint4 h[2];
};
// 16 bytes / 2 bytes of a unit: from global memory through the read-only path (G), or from wherever the generic pointer
// leads (a stage in shared memory)
template <bool G> __device__ __forceinline__ uint4 ldq(const uint8_t *p)
{
    return G ? __ldg(reinterpret_cast<const uint4 *>(p)) : *reinterpret_cast<const uint4 *>(p);
}
template <bool G> __device__ __forceinline__ __half ldh(const uint8_t *p)
{
    return G ? __ldg(reinterpret_cast<const __half *>(p)) : *reinterpret_cast<const __half *>(p);
}

template <int HALF, bool G = true>
__device__ __forceinline__ void unit_load(Q4KRegs &u, const uint8_t *unit, int lane)
{
    const int r = lane >> 2;
#pragma unroll
    for (int gg = 0; gg < 2; gg++) u.q[gg] = ldq<G>(unit + (HALF * 2 + gg) * 512 + lane * 16);
    u.h[0] = ldq<G>(unit + 2048 + r * 16);
    u.h[1] = ldq<G>(unit + 2048 + (r + 8) * 16);
}
// Dequantise 64-group g of the unit (rows r and r + 8 of the warp's sixteen): chunks 0, 1 are the low nibbles
// (k = byte index), chunks 2, 3 the high ones (k = 32 + byte index).
__device__ __forceinline__ void unit_emit(const Q4KRegs &u, int g, AFrag &f)
{
#pragma unroll
    for (int rs = 0; rs < 2; rs++) {
        uint32_t scw, mw;
        q4k_scales4(u.h[rs], g >= 2, scw, mw);
        const uint32_t d2 = prmt(u.h[rs].x, 0u, 0x1010u), dmin2 = prmt(u.h[rs].x, 0u, 0x3232u);
        const Q4KSub lo = q4k_sub(scw, mw, (2 * g) & 3, dmin2), hi = q4k_sub(scw, mw, (2 * g + 1) & 3, dmin2);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const Q4KSub &q = (j >> 1) ? hi : lo;
            const uint32_t wd = word_of(u.q[g & 1], rs * 2 + (j & 1));   // bytes 16 (j & 1) + 4c .. of the group's 32
            store4(f, j, rs, (wd >> (4 * (j >> 1))) & 0x0F0F0F0Fu, q.sc, q.c, d2, q.ndm);
        }
    }
}

// ---- Q6_K (crates/tl_runtime/src/quantized.rs:268-329): w = d * sc * (q6 - 32).  Per lane and unit: the four
// ql pieces (row half hi, block half n), the two qh pieces (hi), sixteen int8 scales and d of rows r, r + 8.
struct Q6KRegs {
    uint4 ql[2];
    uint4 qh[2];
    uint4 sc[2];
    float d[2];
};
template <int HALF, bool G = true>
__device__ __forceinline__ void unit_load(Q6KRegs &u, const uint8_t *unit, int lane)
{
    const int r = lane >> 2;
#pragma unroll
    for (int hi = 0; hi < 2; hi++) {
        u.ql[hi] = ldq<G>(unit + (hi * 2 + HALF) * 512 + lane * 16);
        u.qh[hi] = ldq<G>(unit + 2048 + hi * 512 + lane * 16);
        u.sc[hi] = ldq<G>(unit + 3072 + (r + 8 * hi) * 16);
        u.d[hi] = __half2float(ldh<G>(unit + 3328 + (r + 8 * hi) * 2));
    }
}
// 64-group g = (n, sub): k = 128 n + 64 sub + [0, 64).  sub 0 takes the low nibbles of ql and bits 0-3 of qh,
// sub 1 the high nibbles and bits 4-7; inside the group, q1 = 0 / 1 selects ql[l] / ql[l + 32].
__device__ __forceinline__ void unit_emit(const Q6KRegs &u, int g, AFrag &f)
{
    const int n = g >> 1, sub = g & 1;
#pragma unroll
    for (int hi = 0; hi < 2; hi++) {
#pragma unroll
        for (int st = 0; st < 4; st++) {
            const int h = st & 1, q1 = st >> 1;
            const uint32_t qlw = q1 ? word_of(u.ql[hi], 2 + h) : word_of(u.ql[hi], h);
            const uint32_t qhw = word_of(u.qh[hi], n * 2 + h);
            const uint32_t nib = (sub ? (qlw >> 4) : qlw) & 0x0F0F0F0Fu;
            const uint32_t two = (qhw >> (2 * (sub * 2 + q1))) & 0x03030303u;
            const int s0 = 8 * n + h + 4 * sub;   // scale index for q1 = 0; q1 = 1 is two further
            const uint32_t sb = q1 ? (word_of(u.sc[hi], (s0 + 2) >> 2) >> (8 * ((s0 + 2) & 3))) : (word_of(u.sc[hi], s0 >> 2) >> (8 * (s0 & 3)));
            const uint32_t ds2 = h2_of(u.d[hi] * (float)(int)(int8_t)(sb & 0xFFu));   // d * sc, rounded to f16 once
            store4(f, st, hi, nib | (two << 4), kH2One, kH2Neg1056, ds2, kH2Zero);   // (q - 32) * ds
        }
    }
}

// ---- Q4_0 (quantized.rs:182-225): blocks of 32, w = d * (nibble - 8); low nibble of byte j is k = j, high k = 16 + j
struct Q40Regs {
    uint4 q[2];
    uint4 d[2];   // eight f16 block scales of rows r and r + 8
};
template <int HALF, bool G = true>
__device__ __forceinline__ void unit_load(Q40Regs &u, const uint8_t *unit, int lane)
{
    const int r = lane >> 2;
#pragma unroll
    for (int gg = 0; gg < 2; gg++) u.q[gg] = ldq<G>(unit + (HALF * 2 + gg) * 512 + lane * 16);
    u.d[0] = ldq<G>(unit + 2048 + r * 16);
    u.d[1] = ldq<G>(unit + 2048 + (r + 8) * 16);
}
__device__ __forceinline__ uint32_t h2_pair(const uint4 &v, int i)   // i-th f16 of the 16 bytes, in both halves
{
    return prmt(word_of(v, i >> 1), 0u, (i & 1) ? 0x3232u : 0x1010u);
}
__device__ __forceinline__ void unit_emit(const Q40Regs &u, int g, AFrag &f)
{
#pragma unroll
    for (int hi = 0; hi < 2; hi++) {
        const uint32_t d0 = h2_pair(u.d[hi], 2 * g), d1 = h2_pair(u.d[hi], 2 * g + 1);   // blocks 2g and 2g + 1 of the row's eight
#pragma unroll
        for (int st = 0; st < 4; st++) {
            const int nib = st & 1, b = st >> 1;
            const uint32_t d = b ? d1 : d0;
            const uint32_t wd = b ? word_of(u.q[g & 1], hi * 2 + 1) : word_of(u.q[g & 1], hi * 2);
            const uint32_t nibs = (nib ? (wd >> 4) : wd) & 0x0F0F0F0Fu;
            store4(f, st, hi, nibs, kH2One, kH2Neg1032, d, kH2Zero);   // (q - 8) * d
        }
    }
}

// ---- Q8_0 (quantized.rs:227-260): blocks of 32 int8, w = d * q
struct Q80Regs {
    uint4 q[4];
    uint4 d[2];
};
template <int HALF, bool G = true>
__device__ __forceinline__ void unit_load(Q80Regs &u, const uint8_t *unit, int lane)
{
    const int r = lane >> 2;
#pragma unroll
    for (int i = 0; i < 4; i++) u.q[i] = ldq<G>(unit + (HALF * 4 + i) * 512 + lane * 16);
    u.d[0] = ldq<G>(unit + 4096 + r * 16);
    u.d[1] = ldq<G>(unit + 4096 + (r + 8) * 16);
}
__device__ __forceinline__ void unit_emit(const Q80Regs &u, int g, AFrag &f)
{
#pragma unroll
    for (int hi = 0; hi < 2; hi++) {
        const uint32_t d0 = h2_pair(u.d[hi], 2 * g), d1 = h2_pair(u.d[hi], 2 * g + 1);
#pragma unroll
        for (int st = 0; st < 4; st++) {   // q + 128 as an unsigned byte u, then w = (u - 128) * d
            const int h = st & 1, b = st >> 1;
            const uint32_t d = b ? d1 : d0;
            const uint32_t wd = b ? word_of(u.q[2 * (g & 1) + 1], hi * 2 + h) : word_of(u.q[2 * (g & 1)], hi * 2 + h);
            store4(f, st, hi, wd ^ 0x80808080u, kH2One, kH2Neg1152, d, kH2Zero);
        }
    }
}

template <int FMT> struct UnitRegs;
template <> struct UnitRegs<12> { using type = Q4KRegs; };
template <> struct UnitRegs<14> { using type = Q6KRegs; };
template <> struct UnitRegs<2> { using type = Q40Regs; };
template <> struct UnitRegs<8> { using type = Q80Regs; };

// ---- one dequantising warp: 64-groups 2 HALF and 2 HALF + 1 of every unit of its 16 rows.  `dst`: tensor-memory address
// (the warp's 16 lanes, first column) of weight stage 0.  A stage holds gs 64-wide groups (gs = 1: K step = group, the
// warp fills every other pair of K steps; gs = 4: K step = unit, both warps of a row tile fill the same stage).
// Barrier slot of K step kt: kt % slots; weight stage: kt % na.
template <int FMT, int HALF, int GS>
__device__ __forceinline__ bool produce(const GemmParams &p, const uint8_t *ub, bool have, int lane, uint32_t dst, int slots,
                                        uint32_t full0, uint32_t empty0, volatile int *abort_flag, int u0, int units)
{
    constexpr int na = GS == 4 ? 3 : kGemmAStages;
    typename UnitRegs<FMT>::type cur, nxt;
    ub += (size_t)u0 * p.unit_bytes;          // this CTA's K range starts at unit u0
    // Registers hold one unit ahead; one lane of the pair's first warp asks L2 for the units kAhead further on, so
    // that the register loads find them there.
    constexpr int kAhead = 4;
    constexpr bool wide = GS == 4;
    const bool fetcher = have && HALF == 0 && lane == 0;
    if (fetcher)
        for (int j = 1; j <= kAhead && j < units; j++) l2_prefetch(ub + (size_t)j * p.unit_bytes, (uint32_t)p.unit_bytes);
    if (have) unit_load<HALF>(nxt, ub, lane);
    for (int u = 0; u < units; u++) {
        if (have) {
            cur = nxt;
            if (u + 1 < units) unit_load<HALF>(nxt, ub + (size_t)(u + 1) * p.unit_bytes, lane);
        }
        if (fetcher && u + 1 + kAhead < units) l2_prefetch(ub + (size_t)(u + 1 + kAhead) * p.unit_bytes, (uint32_t)p.unit_bytes);
#pragma unroll
        for (int gg = 0; gg < 2; gg++) {
            const int g = HALF * 2 + gg;
            const int kt = wide ? u : u * 4 + g;                 // the K step this group belongs to
            if ((!wide || gg == 0) && kt >= na) {                  // its stage was last read by the MMAs of K step kt - na
                const int back = kt - na;
                if (!mbar_wait(empty0 + 8u * (uint32_t)(back % slots), (uint32_t)(back / slots) & 1u, abort_flag, p.err, 21)) return false;
                tc_fence_after();
            }
            if (have) {
                AFrag f;
                unit_emit(cur, g, f);
                f.flush(dst + (uint32_t)((kt % na) * (kStageACols * GS) + (wide ? g * kStageACols : 0)));
            }
            if (!wide || gg == 1) {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(full0 + 8u * (uint32_t)(kt % slots));
            }
        }
    }
    return true;
}

// ---- the kernel
template <int FMT, int GS>
__global__ void __launch_bounds__(kGemmThreads, 1)
qgemm_kernel(const __grid_constant__ CUtensorMap xmap, const GemmParams p)
{
    extern __shared__ uint8_t smem_raw[];
    __shared__ int abort_word;
    __shared__ uint32_t tmem_slot;
    volatile int *abort_flag = &abort_word;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t sB = (smem_u32(smem_raw) + 1023u) & ~1023u;   // swizzled tiles want 1024-byte alignment
    // gs = 4 (token tiles of up to 64 rows): a stage is a whole 256-wide unit - four TMA boxes, sixteen MMAs, one barrier
    // round - because with so little tensor work per group the round itself (arrive, wait, commit, wait) sets the pace.
    // The accumulator then takes columns [0, 64) and three weight stages of 128 columns follow from column 128.
    constexpr int gs = GS, na = GS == 4 ? 3 : kGemmAStages;
    constexpr uint32_t tmem_a0 = GS == 4 ? 128u : (uint32_t)kTmemA0;
    const int nb = p.nb, slots = max(na, nb);
    const uint32_t group_b = (uint32_t)p.nt * 128u;                // bytes of one 64-wide activation box (multiple of 2048)
    const uint32_t stage_b = group_b * (uint32_t)gs;
    const uint32_t bars = sB + (uint32_t)nb * stage_b;
    // Slot kt % slots serves K step kt.  full: eight producer warps + the TMA thread's expect_tx; empty: the commit
    // after the step's MMAs.  A waiter for K step kt - d (d = 8 for the weight stage, nb for the activation stage) asks
    // for phase (kt - d) / slots of that slot; the phase before it has always completed by then (K steps complete in
    // order and the waiter itself saw step kt - d - 1 ... complete earlier), so the parity test cannot alias.
    auto full_bar = [&](int i) { return bars + 8u * (uint32_t)i; };
    auto empty_bar = [&](int i) { return bars + 8u * (uint32_t)(kGemmMaxSlots + i); };
    const uint32_t accum_bar = bars + 8u * (2 * kGemmMaxSlots);

    const int tok0 = blockIdx.y * p.nt;
    // K range of this CTA: whole units (4 K steps each), split evenly over grid.z
    const int units_all = (int)p.upt, split = blockIdx.z;
    const int u0 = units_all * split / p.splits, u1 = units_all * (split + 1) / p.splits;
    const int KT = (u1 - u0) * (4 / gs), kt_base = u0 * 4;       // K steps of this CTA; first 64-wide group
    int wi = 0;
    while (wi + 1 < p.n_w && (int)blockIdx.x >= p.rt_end[wi]) wi++;
    const int rt = (int)blockIdx.x - (wi ? p.rt_end[wi - 1] : 0);   // 128-row tile inside weight wi
    const int n_rows = p.n[wi];

    if (tid == 0) {
        abort_word = 0;
        for (int i = 0; i < slots; i++) {
            mbar_init(full_bar(i), gs == 4 ? 17 : 9);    // the producer warps of a stage + the TMA thread's expect_tx
            mbar_init(empty_bar(i), 1);
        }
        mbar_init(accum_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == kGemmProducers + 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;

    if (warp < kGemmProducers) {
        // ------------------------------------------------ dequantise the weight tile, stage by stage
        // 16 rows per warp.  A warp reaches only the tensor-memory lanes of its quarter (warp % 4), so warps w and
        // w + 4 take the two halves of quarter w % 4, and w + 8, w + 12 the same rows' other two 64-groups.
        const int sub = 2 * (warp & 3) + ((warp >> 2) & 1);
        const int tile16 = rt * 8 + sub;
        const bool have = tile16 < p.n_tiles16[wi];
        const uint8_t *ub = p.w[wi] + (size_t)(have ? tile16 : 0) * p.upt * p.unit_bytes;
        const uint32_t dst = tmem + ((uint32_t)(sub * 16) << 16) + tmem_a0;
        const bool ok = warp < 8 ? produce<FMT, 0, GS>(p, ub, have, lane, dst, slots, full_bar(0), empty_bar(0), abort_flag, u0, u1 - u0)
                                 : produce<FMT, 1, GS>(p, ub, have, lane, dst, slots, full_bar(0), empty_bar(0), abort_flag, u0, u1 - u0);
        // ------------------------------------------------ epilogue: tensor memory -> Y[token][row]
        if (ok && mbar_wait(accum_bar, 0, abort_flag, p.err, 22)) {
            tc_fence_after();
            const int quad = warp & 3, part = warp >> 2;    // tensor-memory lanes 32 quad .., a quarter of the columns
            const int row = rt * kGemmRows + quad * 32 + lane;
            float *out = p.out[wi];
            const bool partial = p.splits > 1;   // partial products go to part[split][token][col0 + row], unscaled residual-free
            float *pout = partial ? p.part + (size_t)split * p.m * p.n_all + p.col0[wi] : nullptr;
            const int chunks = p.nt >> 3;
            const int c_begin = 8 * (part * chunks / 4), c_end = 8 * ((part + 1) * chunks / 4);
            for (int c0 = c_begin; c0 < c_end; c0 += 8) {
                // the residual and the row scales first (independent loads in flight together), then the accumulator
                float rs[8], sc[8];
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const int tok = tok0 + c0 + j;
                    const bool live = tok < p.m && row < n_rows;
                    sc[j] = tok < p.m ? __ldg(p.inv_scale + tok) : 0.f;
                    rs[j] = (live && p.resid && !partial) ? __ldg(p.resid + (size_t)tok * n_rows + row) : 0.f;
                }
                uint32_t v[8];
                tmem_ld8(tmem + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0, v);
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const int tok = tok0 + c0 + j;
                    if (tok < p.m && row < n_rows) {
                        if (partial) pout[(size_t)tok * p.n_all + row] = __uint_as_float(v[j]) * sc[j];
                        else out[(size_t)tok * n_rows + row] = rs[j] + __uint_as_float(v[j]) * sc[j];
                    }
                }
            }
        }
    } else if (warp == kGemmProducers) {
        // ------------------------------------------------ TMA: activation tile of each K step, nb steps ahead of the MMAs
        if (lane == 0) {
            int issued = 0;
            int st = 0, slot = 0, bslot = 0, bround = 0;       // kt % nb, kt % slots, (kt - nb) % slots, (kt - nb) / slots
            for (int kt = 0; kt < KT; kt++) {
                if (kt >= nb) {
                    if (!mbar_wait(empty_bar(bslot), (uint32_t)bround & 1u, abort_flag, p.err, 23)) break;
                    if (++bslot == slots) { bslot = 0; bround++; }
                }
                mbar_expect_tx(full_bar(slot), stage_b);
                for (int j = 0; j < gs; j++)
                    tma_load_2d(sB + (uint32_t)st * stage_b + (uint32_t)j * group_b, &xmap, (kt_base + kt * gs + j) * kGemmBK, tok0, full_bar(slot));
                issued = kt + 1;
                if (++st == nb) st = 0;
                if (++slot == slots) slot = 0;
            }
            if (*abort_flag) {
                // let copies that were already requested land before the CTA gives its shared memory back
                for (int kt = max(0, issued - nb); kt < issued; kt++)
                    mbar_wait_drain(full_bar(kt % slots), (uint32_t)(kt / slots) & 1u);
            }
        }
    } else {
        // ------------------------------------------------ MMA issue
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | ((uint32_t)(p.nt >> 3) << 17) | ((uint32_t)(kGemmRows >> 4) << 24);   // f32 D, f16 A/B, K-major both
            bool ok = true;
            int st = 0, slot = 0, round = 0;
            for (int kt = 0; kt < KT; kt++) {
                if (!mbar_wait(full_bar(slot), (uint32_t)round & 1u, abort_flag, p.err, 24)) { ok = false; break; }
                tc_fence_after();
                for (int j = 0; j < gs; j++) {
                    const uint64_t bd = smem_desc_sw128(sB + (uint32_t)st * stage_b + (uint32_t)j * group_b);
                    const uint32_t ta = tmem + tmem_a0 + (uint32_t)((kt % na) * (kStageACols * gs) + j * kStageACols);
#pragma unroll
                    for (int k16 = 0; k16 < kGemmBK / 16; k16++)   // 16 f16: 8 columns of tensor memory, 32 bytes along the swizzle row
                        umma_f16_ts(tmem, ta + 8u * k16, bd + 2u * k16, idesc, (kt | j | k16) != 0);
                }
                umma_commit(empty_bar(slot));   // arrives when the MMAs above have read both stages
                if (++st == nb) st = 0;
                if (++slot == slots) { slot = 0; round++; }
            }
            umma_commit(accum_bar);
            if (!ok) mbar_wait_drain(accum_bar, 0);   // MMAs already issued finish before the tensor memory is freed
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kGemmProducers + 1) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

// Adds the K-splits: out_i[tok][row] = [resid +] sum_s part[s][tok][col0_i + row], splits added in index order.
struct SplitSum {
    float *out[kGemmMaxW];
    int n[kGemmMaxW], col0[kGemmMaxW];
    int n_w, n_all, m, splits;
    const float *part, *resid;
};
__global__ void __launch_bounds__(256) qgemm_split_sum_kernel(const SplitSum a)
{
    const size_t total = (size_t)a.m * a.n_all, stride = total;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int tok = (int)(i / a.n_all), col = (int)(i - (size_t)tok * a.n_all);
        int w = 0;
        while (w + 1 < a.n_w && col >= a.col0[w + 1]) w++;
        const int row = col - a.col0[w];
        float acc = __ldcg(a.part + i);
        for (int s = 1; s < a.splits; s++) acc += __ldcg(a.part + s * stride + i);
        if (a.resid) acc += __ldg(a.resid + (size_t)tok * a.n[w] + row);
        a.out[w][(size_t)tok * a.n[w] + row] = acc;
    }
}

// ---------------------------------------------------------------- raw quants as MMA operands
// The streaming kernel for few activation rows below spends its time issuing instructions, so it does not dequantise: a
// quant u (0 .. 255) placed in the low bits of an f16 IS the number u * 2^-24 (subnormal, or the first normal binade, whose bit
// patterns continue the same line up to 2047), which one AND per two weights produces.  The MMA sums u * x exactly over
// the 16 or 32 weights that share a scale, and the scale - times 2^24 - multiplies that sum in f32.  High nibbles stay in
// place where their chunk has a scale of its own (u * 16, the scale times 2^20).  Constant offsets (-32, -8, -128) are
// subtracted in f16, exactly; the per-sub-block minima of Q4_K enter through one more MMA per unit and activation half:
// A = the 6-bit minima as bf16, B = the activations' sub-block sums as bf16 (high part, remainder) pairs.
struct RawScales { float s[2][4]; };     // [row r / r + 8][chunk, or pair of chunks where two share a scale]
constexpr float kTwo24 = 16777216.f, kTwo20 = 1048576.f;

// D(16x8 f32) = A(16x16 f16) * B(16x8 f16)
__device__ __forceinline__ void hmma16816_z(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ void bmma16816_z(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
// byte i (a runtime index) of w as a float
__device__ __forceinline__ float byte_f(uint32_t w, int i) { return (float)((w >> (8 * i)) & 0xFFu); }
// a small integer as a bf16 in both halves of a word
__device__ __forceinline__ uint32_t bf16_pair(float v) { return prmt(__float_as_uint(v), 0u, 0x3232u); }

template <int FMT> struct RawTraits;
template <> struct RawTraits<12> { static constexpr int kPair = 2; static constexpr bool kMins = true; };
template <> struct RawTraits<14> { static constexpr int kPair = 1; static constexpr bool kMins = false; };
template <> struct RawTraits<2> { static constexpr int kPair = 2; static constexpr bool kMins = false; };
template <> struct RawTraits<8> { static constexpr int kPair = 2; static constexpr bool kMins = false; };

// Q4_K: chunks 0, 1 = the low nibbles (sub-block 2 g), chunks 2, 3 = the high ones in place (sub-block 2 g + 1)
__device__ __forceinline__ void unit_raw(const Q4KRegs &u, int g, AFrag &f, RawScales &sc)
{
#pragma unroll
    for (int rs = 0; rs < 2; rs++) {
        uint32_t scw, mw;
        q4k_scales4(u.h[rs], g >= 2, scw, mw);
        const float d = h2_to_f2(u.h[rs].x).x;
        // (2^23 + sc) * d 2^24 - 2^23 d 2^24 = sc d 2^24, rounded once
        const float d24 = d * kTwo24, d20 = d * kTwo20;
        sc.s[rs][0] = fmaf(__uint_as_float(prmt(scw, 0x4B000000u, 0x7650u + ((2 * g) & 3))), d24, -8388608.f * d24);
        sc.s[rs][1] = fmaf(__uint_as_float(prmt(scw, 0x4B000000u, 0x7650u + ((2 * g + 1) & 3))), d20, -8388608.f * d20);
#pragma unroll
        for (int jl = 0; jl < 2; jl++) {
            const uint32_t wd = word_of(u.q[g & 1], rs * 2 + jl), w8 = wd >> 8;
            f.v[4 * jl + 2 * rs] = wd & 0x000F000Fu;
            f.v[4 * jl + 2 * rs + 1] = w8 & 0x000F000Fu;
            f.v[4 * (2 + jl) + 2 * rs] = wd & 0x00F000F0u;
            f.v[4 * (2 + jl) + 2 * rs + 1] = w8 & 0x00F000F0u;
        }
    }
}
// the minima of sub-blocks c and c + 4 of rows r, r + 8 as the A operand of the sums MMA, and dmin of both rows
__device__ __forceinline__ void q4k_mins(const Q4KRegs &u, int c, uint32_t (&a)[4], float (&dmin)[2])
{
#pragma unroll
    for (int rs = 0; rs < 2; rs++) {
        uint32_t scw, mlo, mhi;
        q4k_scales4(u.h[rs], false, scw, mlo);
        q4k_scales4(u.h[rs], true, scw, mhi);
        a[rs] = bf16_pair(byte_f(mlo, c));
        a[2 + rs] = bf16_pair(byte_f(mhi, c));
        dmin[rs] = h2_to_f2(u.h[rs].x).y;
    }
}

template <class R> __device__ __forceinline__ void q4k_mins(const R &, int, uint32_t (&)[4], float (&)[2]) {}   // the other formats have no minima

// Q6_K: every chunk has its own int8 scale; q - 32 in f16
__device__ __forceinline__ void unit_raw(const Q6KRegs &u, int g, AFrag &f, RawScales &sc)
{
    const int n = g >> 1, sub = g & 1;
#pragma unroll
    for (int hi = 0; hi < 2; hi++) {
        const float d24 = u.d[hi] * kTwo24;
#pragma unroll
        for (int st = 0; st < 4; st++) {
            const int h = st & 1, q1 = st >> 1;
            const uint32_t qlw = q1 ? word_of(u.ql[hi], 2 + h) : word_of(u.ql[hi], h);
            const uint32_t qhw = word_of(u.qh[hi], n * 2 + h);
            const uint32_t nib = (sub ? (qlw >> 4) : qlw) & 0x0F0F0F0Fu;
            const uint32_t two = (qhw >> (2 * (sub * 2 + q1))) & 0x03030303u;
            const uint32_t b6 = nib | (two << 4);
            const int s0 = 8 * n + h + 4 * sub + 2 * q1;
            sc.s[hi][st] = d24 * (float)(int)(int8_t)((word_of(u.sc[hi], s0 >> 2) >> (8 * (s0 & 3))) & 0xFFu);
            f.v[4 * st + 2 * hi] = hsub2(b6 & 0x00FF00FFu, 0x00200020u);
            f.v[4 * st + 2 * hi + 1] = hsub2((b6 >> 8) & 0x00FF00FFu, 0x00200020u);
        }
    }
}
// Q4_0: chunks 2 b, 2 b + 1 = the low and high nibbles of block 2 g + b; nibble - 8 in f16
__device__ __forceinline__ void unit_raw(const Q40Regs &u, int g, AFrag &f, RawScales &sc)
{
#pragma unroll
    for (int hi = 0; hi < 2; hi++) {
#pragma unroll
        for (int b = 0; b < 2; b++) {
            const uint32_t dw = word_of(u.d[hi], g);                       // f16 scales of blocks 2 g, 2 g + 1
            sc.s[hi][b] = (b ? h2_to_f2(dw).y : h2_to_f2(dw).x) * kTwo24;
            const uint32_t wd = word_of(u.q[g & 1], hi * 2 + b);
            f.v[8 * b + 2 * hi] = hsub2(wd & 0x000F000Fu, 0x00080008u);
            f.v[8 * b + 2 * hi + 1] = hsub2((wd >> 8) & 0x000F000Fu, 0x00080008u);
            f.v[8 * b + 4 + 2 * hi] = hsub2((wd >> 4) & 0x000F000Fu, 0x00080008u);
            f.v[8 * b + 4 + 2 * hi + 1] = hsub2((wd >> 12) & 0x000F000Fu, 0x00080008u);
        }
    }
}
// Q8_0: chunks 2 b, 2 b + 1 = the halves of block 2 g + b; (q + 128) - 128 in f16
__device__ __forceinline__ void unit_raw(const Q80Regs &u, int g, AFrag &f, RawScales &sc)
{
#pragma unroll
    for (int hi = 0; hi < 2; hi++) {
#pragma unroll
        for (int st = 0; st < 4; st++) {
            const int h = st & 1, b = st >> 1;
            const uint32_t dw = word_of(u.d[hi], g);
            if (h == 0) sc.s[hi][b] = (b ? h2_to_f2(dw).y : h2_to_f2(dw).x) * kTwo24;
            const uint32_t wd = (b ? word_of(u.q[2 * (g & 1) + 1], hi * 2 + h) : word_of(u.q[2 * (g & 1)], hi * 2 + h)) ^ 0x80808080u;
            f.v[4 * st + 2 * hi] = hsub2(wd & 0x00FF00FFu, 0x00800080u);
            f.v[4 * st + 2 * hi + 1] = hsub2((wd >> 8) & 0x00FF00FFu, 0x00800080u);
        }
    }
}

// ---------------------------------------------------------------- up to 16 activation rows: a streaming kernel
// Few rows leave the tensor-core GEMM above at its floor (a 128-row tile per CTA whatever the width, a fixed cost per CTA and
// per K step), so they get the streaming form of the matvec instead: persistent CTAs of 16 warps, a warp owns 16 weight rows
// and streams their units from HBM through a private ring of bulk copies, turns them into raw-quant A fragments (above: the
// sixteen words of a 64-group ARE the A operands of four mma.sync.m16n8k16, row r / r + 8, K 4c .. 4c+3 of every 16-chunk)
// and multiplies them with the activation rows - f16, scaled per row by x_to_f16_kernel, one 256-wide piece per unit that
// the CTA's warps share - as two MMAs per chunk (rows 0-7 and 8-15 of the activation).
// The activation piece of a unit is 512 bytes per row, copied row by row to a pitch of 528 bytes; x_to_f16_kernel writes
// these rows with the chunk index and the lane's index c exchanged inside every 64-group (order [c][j][4]), so that a lane's
// B operands of four chunks are 32 consecutive bytes: two conflict-free 128-bit loads per 64-group and activation half.
// A CTA works through items = 16 consecutive tiles x a range of K units; with several ranges per tile group (narrow
// weights) the partial products go to scratch and a second launch adds them in range order.
constexpr int kRowsWarps = 16;
constexpr int kRowsThreads = (kRowsWarps + 1) * 32;     // + the copy warp of the activations
constexpr int kRowsWBytes = 168 * 1024;                  // weight rings of all warps: 2 to 4 stages each, by the unit's size
constexpr int kRowsAStages = 4;                          // activation ring per CTA
constexpr int kRowsAPitch = 528;                         // bytes between activation rows of a stage
constexpr int kRowsABytes = 16 * kRowsAPitch;
constexpr int kRowsSumBytes = 16 * 8 * 4;                // their sums over the unit's eight 32-blocks, (high, remainder) bf16 pairs

struct RowsParams {
    const uint8_t *w[kGemmMaxW];
    float *out[kGemmMaxW];
    int n[kGemmMaxW], n_tiles16[kGemmMaxW], tg_end[kGemmMaxW], tile0[kGemmMaxW];   // tile groups / first tile of weight i among all
    int n_w, upt, unit_bytes, stage_w, wstages, m;
    int tgroups, total, maxp;       // total = tgroups x upt unit steps, cut evenly over the CTAs; maxp: tile groups a CTA can touch
    int64_t k;
    const __half *xh;               // [m][k], rows in the order described above
    const float *inv_scale, *resid;
    const uint8_t *sums;            // [K / 256][16][8] sub-block sums of the activation rows (x_to_f16_kernel)
    float *part;                    // [CTA][tile group of the CTA][16 tiles][16 rows][16 activation rows]: pieces of split tile groups
    int *cnt;                       // [tile group][16 tiles]: pieces of the tile that are written; zero between launches
    int *err;
};

// unit registers from a stage in shared memory (the layouts of unit_load above)
template <int HALF> __device__ __forceinline__ void unit_load_s(Q4KRegs &u, uint32_t unit, int lane)
{
    const int r = lane >> 2;
    for (int gg = 0; gg < 2; gg++) u.q[gg] = lds128(unit + (HALF * 2 + gg) * 512 + lane * 16);
    u.h[0] = lds128(unit + 2048 + r * 16);
    u.h[1] = lds128(unit + 2048 + (r + 8) * 16);
}
template <int HALF> __device__ __forceinline__ void unit_load_s(Q6KRegs &u, uint32_t unit, int lane)
{
    const int r = lane >> 2;
#pragma unroll
    for (int hi = 0; hi < 2; hi++) {
        u.ql[hi] = lds128(unit + (hi * 2 + HALF) * 512 + lane * 16);
        u.qh[hi] = lds128(unit + 2048 + hi * 512 + lane * 16);
        u.sc[hi] = lds128(unit + 3072 + (r + 8 * hi) * 16);
        const uint32_t dw = lds32(unit + 3328 + ((r + 8 * hi) >> 1) * 4);
        u.d[hi] = (r & 1) ? h2_to_f2(dw).y : h2_to_f2(dw).x;
    }
}
template <int HALF> __device__ __forceinline__ void unit_load_s(Q40Regs &u, uint32_t unit, int lane)
{
    const int r = lane >> 2;
    for (int gg = 0; gg < 2; gg++) u.q[gg] = lds128(unit + (HALF * 2 + gg) * 512 + lane * 16);
    u.d[0] = lds128(unit + 2048 + r * 16);
    u.d[1] = lds128(unit + 2048 + (r + 8) * 16);
}
template <int HALF> __device__ __forceinline__ void unit_load_s(Q80Regs &u, uint32_t unit, int lane)
{
    const int r = lane >> 2;
    for (int i = 0; i < 4; i++) u.q[i] = lds128(unit + (HALF * 4 + i) * 512 + lane * 16);
    u.d[0] = lds128(unit + 4096 + r * 16);
    u.d[1] = lds128(unit + 4096 + (r + 8) * 16);
}

// What the streaming kernel asks of a format: head() once per unit (what all four 64-groups share), raw<GRP>() per group.
template <int FMT> struct RowsFmt {
    struct Head {};
    __device__ static __forceinline__ void head(Head &, uint32_t, int, uint32_t (&)[4], float (&)[2]) {}
    template <int GRP> __device__ static __forceinline__ void raw(const Head &, uint32_t unit, int lane, AFrag &f, RawScales &sc)
    {
        typename UnitRegs<FMT>::type regs;
        unit_load_s<(GRP >> 1)>(regs, unit, lane);
        unit_raw(regs, GRP, f, sc);
    }
};
// Q4_K: the 6-bit scales of rows r, r + 8 (sub-blocks 0-3, 4-7), d 2^24, d 2^20 and -2^23 times those once per unit; the
// minima of sub-blocks c, c + 4 as the A operand of the sums MMA with dmin of both rows.
template <> struct RowsFmt<12> {
    struct Head { uint32_t scl[2], sch[2]; float d24[2], d20[2], nd24[2], nd20[2]; };
    __device__ static __forceinline__ void head(Head &h, uint32_t unit, int lane, uint32_t (&am)[4], float (&dmin)[2])
    {
        const int r = lane >> 2, c = lane & 3;
#pragma unroll
        for (int rs = 0; rs < 2; rs++) {
            const uint4 hw = lds128(unit + 2048 + (r + 8 * rs) * 16);
            uint32_t mlo, mhi;
            q4k_scales4(hw, false, h.scl[rs], mlo);
            q4k_scales4(hw, true, h.sch[rs], mhi);
            const float2 dd = h2_to_f2(hw.x);
            h.d24[rs] = dd.x * kTwo24; h.d20[rs] = dd.x * kTwo20;
            h.nd24[rs] = h.d24[rs] * -8388608.f; h.nd20[rs] = h.d20[rs] * -8388608.f;
            am[rs] = bf16_pair(byte_f(mlo, c));
            am[2 + rs] = bf16_pair(byte_f(mhi, c));
            dmin[rs] = dd.y;
        }
    }
    template <int GRP> __device__ static __forceinline__ void raw(const Head &h, uint32_t unit, int lane, AFrag &f, RawScales &sc)
    {
        const uint4 q = lds128(unit + GRP * 512 + lane * 16);
#pragma unroll
        for (int rs = 0; rs < 2; rs++) {
            const uint32_t scw = GRP >= 2 ? h.sch[rs] : h.scl[rs];
            // (2^23 + sc) * d 2^24 - 2^23 d 2^24 = sc d 2^24, rounded once
            sc.s[rs][0] = fmaf(__uint_as_float(prmt(scw, 0x4B000000u, 0x7650u + ((2 * GRP) & 3))), h.d24[rs], h.nd24[rs]);
            sc.s[rs][1] = fmaf(__uint_as_float(prmt(scw, 0x4B000000u, 0x7650u + ((2 * GRP + 1) & 3))), h.d20[rs], h.nd20[rs]);
#pragma unroll
            for (int jl = 0; jl < 2; jl++) {
                const uint32_t wd = word_of(q, rs * 2 + jl), w8 = wd >> 8;
                f.v[4 * jl + 2 * rs] = wd & 0x000F000Fu;
                f.v[4 * jl + 2 * rs + 1] = w8 & 0x000F000Fu;
                f.v[4 * (2 + jl) + 2 * rs] = wd & 0x00F000F0u;
                f.v[4 * (2 + jl) + 2 * rs + 1] = w8 & 0x00F000F0u;
            }
        }
    }
};

// NT: halves (8 rows) of the activation in use
template <int FMT, int NT>
__global__ void __launch_bounds__(kRowsThreads, 1) qrows_kernel(const RowsParams p)
{
    extern __shared__ uint8_t rows_smem[];
    __shared__ int abort_word;
    volatile int *abort_flag = &abort_word;
    constexpr bool kMins = RawTraits<FMT>::kMins;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wstages = p.wstages, upt = p.upt;
    const uint32_t base = (smem_u32(rows_smem) + 127u) & ~127u;
    const uint32_t sAct = base;                                                         // [kRowsAStages][16 rows, pitch 528]
    const uint32_t sSum = sAct + kRowsAStages * kRowsABytes;                            // [kRowsAStages][16 rows][8 sums as bf16 pairs]
    const uint32_t sW0 = sSum + kRowsAStages * kRowsSumBytes;
    const uint32_t sW = sW0 + (uint32_t)(warp * wstages) * (uint32_t)p.stage_w;         // this warp's stages
    const uint32_t bars = sW0 + kRowsWarps * wstages * (uint32_t)p.stage_w;
    const uint32_t a_full = bars, a_empty = bars + 8 * kRowsAStages, w_full = bars + 16 * kRowsAStages + (uint32_t)(warp * wstages) * 8;

    if (tid == 0) {
        abort_word = 0;
        for (int i = 0; i < kRowsAStages; i++) { mbar_init(a_full + 8 * i, 1); mbar_init(a_empty + 8 * i, kRowsWarps); }
        for (int i = 0; i < kRowsWarps * wstages; i++) mbar_init(bars + 16 * kRowsAStages + 8 * i, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    // activation rows m .. 15 of every stage are never copied: zero
    for (int i = tid; i < kRowsAStages * (16 - p.m) * (kRowsAPitch / 16); i += kRowsThreads) {
        const int per = (16 - p.m) * (kRowsAPitch / 16), st = i / per, off = i - st * per;
        asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(sAct + st * kRowsABytes + p.m * kRowsAPitch + off * 16), "r"(0u) : "memory");
    }
    __syncthreads();

    // this CTA's unit steps: [start, end) of tile group x unit, tile-group-major
    const int start = (int)((int64_t)p.total * blockIdx.x / gridDim.x), end = (int)((int64_t)p.total * (blockIdx.x + 1) / gridDim.x);
    const int tg_first = start / upt, u_first = start - tg_first * upt;

    if (warp == kRowsWarps) {
        // ------------------------------------------------ the activation piece of every unit step: lane l copies row l
        bool ok = true;
        const uint32_t bytes = (uint32_t)p.m * 512u + (kMins ? kRowsSumBytes : 0);
        const __half *row = p.xh + (size_t)min(lane, p.m - 1) * p.k;
        int g = 0, u = u_first;
        pdl_wait();                                          // the activations are the preceding kernel's
        for (int pos = start; pos < end; pos++, g++) {
            const int st = g & (kRowsAStages - 1);
            if (g >= kRowsAStages) {
                if (lane == 0) ok = mbar_wait(a_empty + 8 * st, (uint32_t)((g >> 2) - 1) & 1u, abort_flag, p.err, 51);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
            }
            if (lane == 0) {
                mbar_expect_tx(a_full + 8 * st, bytes);
                if (kMins) bulk_g2s(sSum + st * kRowsSumBytes, p.sums + (size_t)u * kRowsSumBytes, kRowsSumBytes, a_full + 8 * st);
            }
            __syncwarp();
            if (lane < p.m) bulk_g2s(sAct + st * kRowsABytes + lane * kRowsAPitch, row + (size_t)u * 256, 512u, a_full + 8 * st);
            if (++u == upt) u = 0;
        }
        if (*abort_flag && lane == 0)
            for (int k = max(0, g - kRowsAStages); k < g; k++) mbar_wait_drain(a_full + 8 * (k & (kRowsAStages - 1)), (uint32_t)(k >> 2) & 1u);
        return;
    }

    // ------------------------------------------------ sixteen streaming warps
    const int r = lane >> 2, c = lane & 3;
    const uint32_t b_lane = (uint32_t)(r * kRowsAPitch + c * 32);
    // this warp's tile of tile group tg
    auto tile_of = [&](int tg, int &wi, int &tile16, bool &have) {
        wi = 0;
        while (wi + 1 < p.n_w && tg >= p.tg_end[wi]) wi++;
        tile16 = (tg - (wi ? p.tg_end[wi - 1] : 0)) * kRowsWarps + warp;
        have = tile16 < p.n_tiles16[wi];
    };
    // the copies run wstages units ahead of the MMAs, across tile groups
    int pf_pos = start, pf_tg = tg_first, pf_left = min(upt - u_first, end - start), issued = 0;
    const uint8_t *pf_src;
    bool pf_have;
    {
        int wi, tile16;
        tile_of(pf_tg, wi, tile16, pf_have);
        pf_src = p.w[wi] + ((size_t)tile16 * upt + u_first) * p.unit_bytes;
    }
    auto issue = [&](int st) {                 // one unit of weights into stage st
        if (lane == 0) {
            if (pf_have) {
                mbar_expect_tx(w_full + 8 * st, (uint32_t)p.unit_bytes);
                bulk_g2s(sW + st * p.stage_w, pf_src, (uint32_t)p.unit_bytes, w_full + 8 * st);
            } else {
                mbar_arrive(w_full + 8 * st);    // rows past the weight's end: nothing to copy, the phase still turns
            }
        }
        issued++;
        pf_pos++;
        pf_src += p.unit_bytes;
        if (--pf_left == 0 && pf_pos < end) {
            int wi, tile16;
            tile_of(++pf_tg, wi, tile16, pf_have);
            pf_src = p.w[wi] + (size_t)tile16 * upt * p.unit_bytes;
            pf_left = min(upt, end - pf_pos);
        }
    };
    for (int i = 0; i < wstages && pf_pos < end; i++) issue(i);
    pdl_wait();                                // from here on: activations, scales, residual, outputs, scratch and counters

    int g = 0, ws = 0;                         // units consumed, their weight stage
    uint32_t wph = 0;
    bool ok = true;
    int tg = tg_first, u0 = u_first;
    for (int pos = start; pos < end && ok; tg++, u0 = 0) {
        const int len = min(upt - u0, end - pos);
        pos += len;
        int wi, tile16;
        bool have;
        tile_of(tg, wi, tile16, have);
        float acc[NT][4];
#pragma unroll
        for (int t = 0; t < NT; t++)
#pragma unroll
            for (int e = 0; e < 4; e++) acc[t][e] = 0.f;
        for (int ul = len; ul > 0; ul--, g++) {
            const int as = g & (kRowsAStages - 1);
            bool got = mbar_wait(w_full + 8 * ws, wph, abort_flag, p.err, 52);
            got = got && mbar_wait(a_full + 8 * as, (uint32_t)(g >> 2) & 1u, abort_flag, p.err, 53);
            if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
            if (have) {
                const uint32_t unit = sW + ws * p.stage_w;
                const uint32_t xs = sAct + as * kRowsABytes + b_lane;
                typename RowsFmt<FMT>::Head hd;
                uint32_t am[4] = {0u, 0u, 0u, 0u};
                float dmin[2] = {0.f, 0.f};
                RowsFmt<FMT>::head(hd, unit, lane, am, dmin);
                if constexpr (kMins) {                      // - dmin * sum over the sub-blocks of min * (sum of x)
#pragma unroll
                    for (int t = 0; t < NT; t++) {
                        const uint2 b = lds64(sSum + as * kRowsSumBytes + (8 * t + r) * 32 + c * 8);
                        float mm[4];
                        bmma16816_z(mm, am[0], am[1], am[2], am[3], b.x, b.y);
#pragma unroll
                        for (int e = 0; e < 4; e++) acc[t][e] = fmaf(-dmin[e >> 1], mm[e], acc[t][e]);
                    }
                }
                auto group = [&](auto grp_tag) {
                    constexpr int GRP = decltype(grp_tag)::value;      // 64-group of the unit
                    AFrag f;
                    RawScales sc;
                    RowsFmt<FMT>::template raw<GRP>(hd, unit, lane, f, sc);
                    constexpr int P = RawTraits<FMT>::kPair;           // chunks that share a scale
#pragma unroll
                    for (int t = 0; t < NT; t++) {                     // activation rows 8 t + r
                        // B operands of the group's four chunks: words (2 j, 2 j + 1) = chunk j
                        const uint4 b01 = lds128(xs + t * (8 * kRowsAPitch) + GRP * 128), b23 = lds128(xs + t * (8 * kRowsAPitch) + GRP * 128 + 16);
                        const uint32_t bw[8] = {b01.x, b01.y, b01.z, b01.w, b23.x, b23.y, b23.z, b23.w};
#pragma unroll
                        for (int pr = 0; pr < 4 / P; pr++) {
                            float sub[4];
#pragma unroll
                            for (int jj = 0; jj < P; jj++) {           // 16-chunk j: K 64 GRP + 16 j + 4 c .. + 3 of rows r, r + 8
                                const int j = pr * P + jj;
                                if (jj == 0) hmma16816_z(sub, f.v[4 * j], f.v[4 * j + 2], f.v[4 * j + 1], f.v[4 * j + 3], bw[2 * j], bw[2 * j + 1]);
                                else hmma16816(sub, f.v[4 * j], f.v[4 * j + 2], f.v[4 * j + 1], f.v[4 * j + 3], bw[2 * j], bw[2 * j + 1]);
                            }
#pragma unroll
                            for (int e = 0; e < 4; e++) acc[t][e] = fmaf(sc.s[e >> 1][pr], sub[e], acc[t][e]);
                        }
                    }
                };
                group(std::integral_constant<int, 0>());
                group(std::integral_constant<int, 1>());
                group(std::integral_constant<int, 2>());
                group(std::integral_constant<int, 3>());
            }
            __syncwarp();                      // every lane has read both stages
            if (lane == 0) mbar_arrive(a_empty + 8 * as);
            if (pf_pos < end) issue(ws);       // the stage just read takes the unit wstages further on
            if (++ws == wstages) { ws = 0; wph ^= 1u; }
        }
        if (!ok) break;
        // results: lane (r, c) holds weight rows r and r + 8 x activation rows 8 t + 2 c, + 1.  A tile group that lies
        // in one CTA goes to the output.  The pieces of a split one go to this CTA's scratch slot of the group; the warp that
        // writes a tile's last piece (a count per tile tells) adds them, CTAs in index order, and writes the output rows.
        if (have) {
            const bool whole = len == upt;
            float *slot = p.part + (((size_t)blockIdx.x * p.maxp + (tg - tg_first)) * kRowsWarps + warp) * 256;
#pragma unroll
            for (int t = 0; t < NT; t++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int rt = r + (e >> 1) * 8, row = tile16 * 16 + rt, tok = 8 * t + 2 * c + (e & 1);
                    if (tok >= p.m) continue;
                    if (!whole) slot[rt * 16 + tok] = acc[t][e];
                    else if (row < p.n[wi]) {
                        const float res = p.resid ? __ldg(p.resid + (size_t)tok * p.n[wi] + row) : 0.f;
                        p.out[wi][(size_t)tok * p.n[wi] + row] = res + acc[t][e] * __ldg(p.inv_scale + tok);
                    }
                }
            if (!whole) {
                // the CTA of unit step x is the last one whose range starts at or before x
                const int64_t x0 = (int64_t)tg * upt, x1 = x0 + upt - 1;
                const int b_lo = (int)(((x0 + 1) * gridDim.x - 1) / p.total), b_hi = (int)(((x1 + 1) * gridDim.x - 1) / p.total);
                __threadfence();
                __syncwarp();
                int before = 0;
                if (lane == 0) before = atomicAdd(p.cnt + tg * kRowsWarps + warp, 1);
                before = __shfl_sync(0xffffffffu, before, 0);
                if (before == b_hi - b_lo) {
                    __threadfence();
                    if (lane == 0) p.cnt[tg * kRowsWarps + warp] = 0;
                    const size_t cta_stride = (size_t)p.maxp * kRowsWarps * 256;
                    const int tgf_lo = (int)((int64_t)p.total * b_lo / gridDim.x) / upt;
                    const float *src = p.part + (size_t)warp * 256 + lane;
                    const float *first = src + b_lo * cta_stride + (size_t)(tg - tgf_lo) * kRowsWarps * 256;
#pragma unroll
                    for (int i = 0; i < 8; i++) {               // entry 32 i + lane of the tile's 16 x 16: (row, activation row)
                        const int idx = 32 * i + lane, rt = idx >> 4, tok = idx & 15, row = tile16 * 16 + rt;
                        float sum = __ldcg(first + 32 * i);
                        for (int cta = b_lo + 1; cta <= b_hi; cta++) sum += __ldcg(src + cta * cta_stride + 32 * i);
                        if (tok < p.m && row < p.n[wi]) {
                            const float res = p.resid ? __ldg(p.resid + (size_t)tok * p.n[wi] + row) : 0.f;
                            p.out[wi][(size_t)tok * p.n[wi] + row] = res + sum * __ldg(p.inv_scale + tok);
                        }
                    }
                }
            }
        }
    }
    if (!ok && lane == 0) {
        // copies still in flight land before the CTA's shared memory is given up
        int st = ws;
        uint32_t ph = wph;
        for (int k = g; k < issued; k++) {
            mbar_wait_drain(w_full + 8 * st, ph);
            if (++st == wstages) { st = 0; ph ^= 1u; }
        }
    }
}

// ---- activations: f32 rows -> f16 rows scaled by a power of two, and the inverse scale per row.
// Fused in front of the conversion, as the caller asks:
//   x2:     v = silu(x) * x2                               (crates/tl_cpu/src/ffi.rs:2097-2103, then mul)
//   norm_w: v = v / sqrt(mean(v^2) + eps) * norm_w         (crates/tl_cpu/src/ffi.rs:2444-2486)
// NC > 0: the row (k <= 4 NT NC) stays in registers, NC float4 per thread, between the pass that finds its scale and
// the pass that writes; NC = 0 reads (and recomputes) it twice.
template <int NT, int NC>
__global__ void __launch_bounds__(NT) x_to_f16_kernel(const float *__restrict__ x, const float *__restrict__ x2, const float *__restrict__ norm_w,
                                                        float eps, __half *__restrict__ xh, float *__restrict__ inv_scale, int64_t k,
                                                        uint32_t *__restrict__ sums)
{
    constexpr bool CACHED = NC > 0;
    constexpr int kActCache = NC;
    __shared__ float red[2][NT / 32];
    pdl_launch_dependents();     // a dependent launch (the few-rows kernel) may start its prologue; it waits for this grid's end before it reads
    const float *row = x + (size_t)blockIdx.x * k;
    const float *row2 = x2 ? x2 + (size_t)blockIdx.x * k : nullptr;
    __half *orow = xh + (size_t)blockIdx.x * k;
    auto value = [&](int64_t i) {
        float4 v = *reinterpret_cast<const float4 *>(row + i);
        if (row2) {
            const float4 u = *reinterpret_cast<const float4 *>(row2 + i);
            v.x = silu_f(v.x) * u.x; v.y = silu_f(v.y) * u.y; v.z = silu_f(v.z) * u.z; v.w = silu_f(v.w) * u.w;
        }
        return v;
    };
    float4 cache[CACHED ? kActCache : 1];
    float amax = 0.f, ssq = 0.f;
    auto pass1 = [&](int64_t i, int slot) {
        float4 v = value(i);
        if (CACHED) cache[slot] = v;
        if (norm_w) {
            ssq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            const float4 w = __ldg(reinterpret_cast<const float4 *>(norm_w + i));
            v.x *= w.x; v.y *= w.y; v.z *= w.z; v.w *= w.w;
        }
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    };
    if (CACHED) {
#pragma unroll
        for (int it = 0; it < kActCache; it++) {
            const int64_t i = threadIdx.x * 4 + it * (NT * 4);
            if (i < k) pass1(i, it);
        }
    } else {
        for (int64_t i = threadIdx.x * 4; i < k; i += NT * 4) pass1(i, 0);
    }
    for (int o = 16; o; o >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
    }
    if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = amax; red[1][threadIdx.x >> 5] = ssq; }
    __syncthreads();
    amax = red[0][0];
    ssq = red[1][0];
    for (int i = 1; i < NT / 32; i++) { amax = fmaxf(amax, red[0][i]); ssq += red[1][i]; }
    const float inv_rms = norm_w ? 1.0f / sqrtf(ssq / (float)k + eps) : 1.0f;
    amax *= inv_rms;
    // amax = f * 2^e with f in [0.5, 1): scale by 2^(14 - e), so the largest element lands in [2^13, 2^14)
    float scale = 1.f, inv = 1.f;
    if (amax > 0.f && amax < 3.0e38f) {
        int e;
        frexpf(amax, &e);
        scale = ldexpf(1.f, 14 - e);
        inv = ldexpf(1.f, e - 14);
    }
    auto pass2 = [&](int64_t i, int slot) {
        float4 v = CACHED ? cache[slot] : value(i);
        if (norm_w) {
            const float4 w = __ldg(reinterpret_cast<const float4 *>(norm_w + i));
            v.x = v.x * inv_rms * w.x; v.y = v.y * inv_rms * w.y; v.z = v.z * inv_rms * w.z; v.w = v.w * inv_rms * w.w;
        }
        // inside every group of four the middle two are exchanged, as store4 lays the weights out
        __half2 a = __floats2half2_rn(v.x * scale, v.z * scale), b = __floats2half2_rn(v.y * scale, v.w * scale);
        uint2 o2;
        o2.x = *reinterpret_cast<uint32_t *>(&a);
        o2.y = *reinterpret_cast<uint32_t *>(&b);
        // rows for the streaming kernel (sums given): chunk index and lane index exchanged inside every 64-group
        const int64_t dst = sums ? ((i & ~(int64_t)63) | ((i & 12) << 2) | ((i >> 2) & 12)) : i;
        *reinterpret_cast<uint2 *>(orow + dst) = o2;
        if (sums) {
            // the sum of the 32-block's rounded values (eight lanes), as a bf16 and the bf16 of what that leaves: entry
            // 2 (s & 3) + (s >> 2) of the row's eight in table [K / 256][16 rows][8]
            const float2 fa = __half22float2(a), fb = __half22float2(b);
            float sum = (fa.x + fa.y) + (fb.x + fb.y);
            for (int o = 1; o < 8; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            if ((threadIdx.x & 7) == 0) {
                const uint32_t hi = __float_as_uint(sum) & 0xFFFF0000u;
                const __nv_bfloat16 lo = __float2bfloat16_rn(sum - __uint_as_float(hi));
                const int sb = (int)(i >> 5) & 7;
                sums[((i >> 8) * 16 + blockIdx.x) * 8 + 2 * (sb & 3) + (sb >> 2)] = (hi >> 16) | ((uint32_t)__bfloat16_as_ushort(lo) << 16);
            }
        }
    };
    if (CACHED) {
#pragma unroll
        for (int it = 0; it < kActCache; it++) {
            const int64_t i = threadIdx.x * 4 + it * (NT * 4);
            if (i < k) pass2(i, it);
        }
    } else {
        for (int64_t i = threadIdx.x * 4; i < k; i += NT * 4) pass2(i, 0);
    }
    if (threadIdx.x == 0) inv_scale[blockIdx.x] = inv;
}

// Activation rows per CTA: up to 128 rows one tile; above, 256-row tiles if they give every SM work, else 128-row
// ones (more, smaller CTAs).
int pick_token_tile(int64_t m, int64_t n, int sms)
{
    const int64_t row_tiles = (n + kGemmRows - 1) / kGemmRows;
    if (m <= 128) return (int)((m + 15) / 16 * 16);
    const int64_t ctas256 = row_tiles * ((m + 255) / 256);
    if (ctas256 >= sms) return 256;
    return 128;
}

}  // namespace

bool qgemm_supported(int type) { return type == 12 || type == 14 || type == 2 || type == 8; }

namespace {
template <int FMT, int GS>
tlb_status launch_fmt_gemm_gs(dim3 grid, size_t smem, cudaStream_t stream, const CUtensorMap &map, const GemmParams &p)
{
    static bool attr_set = false;
    if (!attr_set) {
        TLB_CUDA(cudaFuncSetAttribute(qgemm_kernel<FMT, GS>, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmemMax));
        attr_set = true;
    }
    qgemm_kernel<FMT, GS><<<grid, kGemmThreads, smem, stream>>>(map, p);
    return TLB_OK;
}
template <int FMT>
tlb_status launch_fmt_gemm(dim3 grid, size_t smem, cudaStream_t stream, const CUtensorMap &map, const GemmParams &p)
{
    return p.gs == 4 ? launch_fmt_gemm_gs<FMT, 4>(grid, smem, stream, map, p) : launch_fmt_gemm_gs<FMT, 1>(grid, smem, stream, map, p);
}
}  // namespace

// K-splits for m activation rows on `tiles` 128-row tiles of `units` 256-wide K units, n_all output columns in all.
// With few token rows a tile's time is its K length (the dequantising warps set the pace), so the launch costs
// waves x units-per-split; a split count is worth its second pass over s x m x n_all partial sums when it evens out
// the last wave or fills idle SMs.  Returns the count with the least estimated time (1 = no split).
int qgemm_k_splits(int64_t m, int64_t tiles, int64_t units, int64_t n_all, int sm_count)
{
    if (m > 64 || units < 8) return 1;
    const double us_per_unit = 1.8;                                         // 4 K steps of ~0.45 us
    int best = 1;
    double best_us = 1e30;
    for (int s = 1; s <= 16 && s * 4 <= units; s++) {
        const int64_t waves = (tiles * s + sm_count - 1) / sm_count, len = (units + s - 1) / s;
        double us = (double)(waves * len) * us_per_unit + (double)waves * 2.0;   // + fill and drain of every wave
        if (s > 1) us += 4.0 + (double)(s * m * n_all) * 8.0 / 3.0e6;       // the summing launch: its latency + partials written and read
        if (us < best_us - 0.5) { best_us = us; best = s; }
    }
    return best;
}

tlb_status qgemm_prepare(GemmAct *a, const float *x, const float *x2, int64_t m, int64_t k, const float *norm_w, float eps)
{
    Context *c = ctx();
    if (!c) return TLB_ERR_DEVICE;
    a->xh = a->inv = a->sums = nullptr;
    a->m = m; a->k = k;
    if (k % 256 != 0 || m < 1 || m > INT32_MAX) return fail(TLB_ERR_SHAPE, "tensor-core GEMM: bad activation shape");
    if (((uintptr_t)x & 15) || ((uintptr_t)x2 & 15) || ((uintptr_t)norm_w & 15)) return fail(TLB_ERR_ARG, "tensor-core GEMM: activations must be 16-byte aligned");
    a->xh = storage_alloc((size_t)m * k * sizeof(__half));
    if (!a->xh) return TLB_ERR_ALLOC;
    a->inv = storage_alloc((size_t)m * sizeof(float));
    if (!a->inv) { storage_release(a->xh); a->xh = nullptr; return TLB_ERR_ALLOC; }
    __half *xh = (__half *)a->xh->ptr;
    float *inv = (float *)a->inv->ptr;
    // short rows stay in registers between the two passes; long ones are read twice (measured faster than 512
    // threads x 8 float4 at k = 14336, where the second read comes from L2)
    uint32_t *sums = nullptr;
    if (qrows_rows(m)) {     // the streaming kernel for few rows wants the 32-block sums as well (Q4_K minima)
        a->sums = storage_alloc((size_t)(k / 256) * kRowsSumBytes);
        if (!a->sums) { qgemm_release(a); return TLB_ERR_ALLOC; }
        sums = (uint32_t *)a->sums->ptr;
    }
    // few rows are few CTAs: each takes its row with 1024 threads and keeps it in registers
    if (m <= 16 && k > 4096 && k <= 32768) x_to_f16_kernel<1024, 8><<<(unsigned)m, 1024, 0, c->stream>>>(x, x2, norm_w, eps, xh, inv, k, sums);
    else if (k <= 4096) x_to_f16_kernel<256, 4><<<(unsigned)m, 256, 0, c->stream>>>(x, x2, norm_w, eps, xh, inv, k, sums);
    else x_to_f16_kernel<256, 0><<<(unsigned)m, 256, 0, c->stream>>>(x, x2, norm_w, eps, xh, inv, k, sums);
    count_launch();
    return TLB_OK;
}

void qgemm_release(GemmAct *a)
{
    if (a->xh) storage_release(a->xh);
    if (a->inv) storage_release(a->inv);
    if (a->sums) storage_release(a->sums);
    a->xh = a->inv = a->sums = nullptr;
}

namespace {
template <int FMT, int NT>
tlb_status launch_fmt_rows(int grid, size_t smem, cudaStream_t stream, const RowsParams &p)
{
    static bool attr_set = false;
    if (!attr_set) {
        TLB_CUDA(cudaFuncSetAttribute(qrows_kernel<FMT, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 216 * 1024));
        attr_set = true;
    }
    // programmatic dependent launch: the CTAs start - barriers, the first weight copies - while x_to_f16_kernel, which
    // releases its dependents at once, still converts the activations; griddepcontrol.wait stands before their first use
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kRowsThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    TLB_CUDA(cudaLaunchKernelEx(&cfg, qrows_kernel<FMT, NT>, p));
    return TLB_OK;
}
template <int FMT>
tlb_status launch_fmt_rows_nt(int grid, size_t smem, cudaStream_t stream, const RowsParams &p)
{
    return p.m <= 8 ? launch_fmt_rows<FMT, 1>(grid, smem, stream, p) : launch_fmt_rows<FMT, 2>(grid, smem, stream, p);
}
}  // namespace

// Row counts the streaming kernel takes: up to the sixteen columns of its two MMAs per chunk
bool qrows_rows(int64_t m) { return m >= 1 && m <= 16; }

// up to 16 activation rows: the streaming kernel (same operands as the GEMM)
tlb_status qrows_run(const tlb_qtensor *const *ws, int n_w, const GemmAct &a, float *const *outs, const float *resid)
{
    Context *c = ctx();
    if (!c) return TLB_ERR_DEVICE;
    const tlb_qtensor *w0 = ws[0];
    RowsParams p = {};
    int tgroups = 0, tiles_all = 0;
    for (int i = 0; i < kGemmMaxW; i++) {
        const tlb_qtensor *w = i < n_w ? ws[i] : nullptr;
        if (w && (w->type != w0->type || w->k != a.k || w->n > INT32_MAX))
            return fail(TLB_ERR_SHAPE, "quantized matmul: weight K %lld vs activation K %lld, or mixed types", (long long)w->k, (long long)a.k);
        p.w[i] = w ? w->dev() : nullptr;
        p.out[i] = w ? outs[i] : nullptr;
        p.n[i] = w ? (int)w->n : 0;
        p.n_tiles16[i] = w ? (int)w->n_tiles : 0;
        p.tile0[i] = tiles_all;
        if (w) { tgroups += (int)((w->n_tiles + kRowsWarps - 1) / kRowsWarps); tiles_all += (int)w->n_tiles; }
        p.tg_end[i] = tgroups;
    }
    if ((int64_t)tgroups * w0->upt > INT32_MAX / 256) return fail(TLB_ERR_SHAPE, "quantized matmul (few rows): weight too large");
    p.n_w = n_w;
    p.upt = (int)w0->upt;
    p.unit_bytes = qformat(w0->type)->unit_bytes;
    p.stage_w = (p.unit_bytes + 127) / 128 * 128;
    p.wstages = std::max(2, std::min(4, kRowsWBytes / kRowsWarps / p.stage_w));
    p.m = (int)a.m;
    p.tgroups = tgroups;
    p.total = tgroups * p.upt;
    // the unit steps (tile group x unit) are cut evenly over the CTAs, whatever the borders of the tile groups
    const int grid = std::min(p.total, c->sm_count);
    const int per = (p.total + grid - 1) / grid;
    p.maxp = (per + p.upt - 2) / p.upt + 1;
    bool split = false;
    for (int b = 1; b < grid && !split; b++) split = ((int64_t)p.total * b / grid) % p.upt != 0;
    p.inv_scale = (const float *)a.inv->ptr;
    p.resid = resid;
    p.sums = a.sums ? (const uint8_t *)a.sums->ptr : nullptr;
    if (!p.sums) return fail(TLB_ERR_ARG, "quantized matmul (few rows): activations prepared without their block sums");
    p.err = c->err_flag;
    p.cnt = c->mv_cnt;
    if ((size_t)tgroups * kRowsWarps > c->mv_cnt_n) return fail(TLB_ERR_SHAPE, "quantized matmul (few rows): more tiles than the context's counters");
    p.k = a.k;
    p.xh = (const __half *)a.xh->ptr;
    Storage *part = nullptr;
    if (split) {
        part = storage_alloc((size_t)grid * p.maxp * kRowsWarps * 256 * sizeof(float));
        if (!part) return TLB_ERR_ALLOC;
        p.part = (float *)part->ptr;
    }
    const size_t smem = (size_t)kRowsAStages * (kRowsABytes + kRowsSumBytes) + (size_t)kRowsWarps * p.wstages * p.stage_w + 8 * (2 * kRowsAStages + kRowsWarps * p.wstages) + 128 + 64;
    tlb_status ls;
    switch (w0->type) {
        case 12: ls = launch_fmt_rows_nt<12>(grid, smem, c->stream, p); break;
        case 14: ls = launch_fmt_rows_nt<14>(grid, smem, c->stream, p); break;
        case 2: ls = launch_fmt_rows_nt<2>(grid, smem, c->stream, p); break;
        default: ls = launch_fmt_rows_nt<8>(grid, smem, c->stream, p); break;
    }
    if (ls != TLB_OK) { if (part) storage_release(part); return ls; }
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (part) storage_release(part);
    if (e != cudaSuccess) return cuda_fail(e, "quantized matmul (few rows) launch");
    return TLB_OK;
}

tlb_status qgemm_run_multi(const tlb_qtensor *const *ws, int n_w, const GemmAct &a, float *const *outs, const float *resid)
{
    Context *c = ctx();
    if (!c) return TLB_ERR_DEVICE;
    if (n_w < 1 || n_w > kGemmMaxW || (resid && n_w != 1)) return fail(TLB_ERR_ARG, "tensor-core GEMM: %d weights in one launch", n_w);
    const tlb_qtensor *w0 = ws[0];
    if (!qgemm_supported(w0->type)) return fail(TLB_ERR_TYPE, "tensor-core GEMM: GGML type %d is not supported", w0->type);
    if (qrows_rows(a.m)) return qrows_run(ws, n_w, a, outs, resid);
    GemmParams p;
    int64_t row_tiles = 0, n_max = 0;
    for (int i = 0; i < kGemmMaxW; i++) {
        const tlb_qtensor *w = i < n_w ? ws[i] : nullptr;
        if (w && (w->type != w0->type || w->k != a.k || w->n > INT32_MAX))
            return fail(TLB_ERR_SHAPE, "tensor-core GEMM: weight K %lld vs activation K %lld, or mixed types", (long long)w->k, (long long)a.k);
        if (w) { row_tiles += (w->n + kGemmRows - 1) / kGemmRows; n_max = std::max(n_max, row_tiles * kGemmRows); }
        p.w[i] = w ? w->dev() : nullptr;
        p.out[i] = w ? outs[i] : nullptr;
        p.n[i] = w ? (int)w->n : 0;
        p.n_tiles16[i] = w ? (int)w->n_tiles : 0;
        p.rt_end[i] = (int)row_tiles;
    }
    auto encode = tensor_map_encoder();
    if (!encode) return fail(TLB_ERR_DEVICE, "cuTensorMapEncodeTiled is not available from this driver");
    const int64_t m = a.m;
    const int nt = pick_token_tile(m, n_max, c->sm_count);
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)a.k, (cuuint64_t)m};
    const cuuint64_t strides[1] = {(cuuint64_t)a.k * sizeof(__half)};
    const cuuint32_t box[2] = {(cuuint32_t)kGemmBK, (cuuint32_t)nt};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = encode(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a.xh->ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(TLB_ERR_DEVICE, "cuTensorMapEncodeTiled failed (%d)", (int)r);

    p.n_w = n_w;
    p.upt = w0->upt;
    p.m = (int)m;
    p.nt = nt;
    p.gs = nt <= 64 ? 4 : 1;
    p.nb = std::max(p.gs == 4 ? 3 : 4, std::min(kGemmMaxSlots, kGemmBBytes / (nt * 128 * p.gs)));
    p.kt_total = (int)(a.k / kGemmBK);
    p.unit_bytes = qformat(w0->type)->unit_bytes;
    p.inv_scale = (const float *)a.inv->ptr;
    p.resid = resid;
    p.err = c->err_flag;

    const size_t smem = (size_t)p.nb * nt * 128 * p.gs + (kGemmSmemMax - kGemmBBytes);
    const int64_t tok_tiles = (m + nt - 1) / nt;
    int64_t n_all = 0;
    for (int i = 0; i < kGemmMaxW; i++) { p.col0[i] = (int)n_all; n_all += p.n[i]; }
    const int splits = qgemm_k_splits(m, row_tiles * tok_tiles, p.upt, n_all, c->sm_count);
    Storage *part = nullptr;
    if (splits > 1) {
        part = storage_alloc((size_t)splits * m * n_all * sizeof(float));
        if (!part) return TLB_ERR_ALLOC;
    }
    p.splits = splits;
    p.part = part ? (float *)part->ptr : nullptr;
    p.n_all = (int)n_all;
    dim3 grid((unsigned)row_tiles, (unsigned)tok_tiles, (unsigned)splits);
    tlb_status ls;
    switch (w0->type) {
        case 12: ls = launch_fmt_gemm<12>(grid, smem, c->stream, map, p); break;
        case 14: ls = launch_fmt_gemm<14>(grid, smem, c->stream, map, p); break;
        case 2: ls = launch_fmt_gemm<2>(grid, smem, c->stream, map, p); break;
        default: ls = launch_fmt_gemm<8>(grid, smem, c->stream, map, p); break;
    }
    if (ls != TLB_OK) { if (part) storage_release(part); return ls; }
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess && splits > 1) {
        SplitSum a;
        for (int i = 0; i < kGemmMaxW; i++) { a.out[i] = p.out[i]; a.n[i] = p.n[i]; a.col0[i] = p.col0[i]; }
        a.n_w = n_w; a.n_all = (int)n_all; a.m = (int)m; a.splits = splits; a.part = p.part; a.resid = resid;
        const unsigned blocks = (unsigned)std::min<int64_t>(4 * c->sm_count, (m * n_all + 255) / 256);
        qgemm_split_sum_kernel<<<blocks, 256, 0, c->stream>>>(a);
        count_launch();
        e = cudaGetLastError();
    }
    if (part) storage_release(part);     // stream-ordered: freed after the launches above have run
    if (e != cudaSuccess) return cuda_fail(e, "qgemm launch");
    return TLB_OK;
}

tlb_status qgemm_run(const tlb_qtensor *w, const GemmAct &a, float *out, const float *resid)
{
    return qgemm_run_multi(&w, 1, a, &out, resid);
}

tlb_status launch_qgemm(const tlb_qtensor *w, const float *x, int64_t m, float *out)
{
    GemmAct a;
    TLB_TRY(qgemm_prepare(&a, x, nullptr, m, w->k, nullptr, 0.f));
    tlb_status st = qgemm_run(w, a, out, nullptr);
    qgemm_release(&a);
    return st;
}

}  // namespace tlb
