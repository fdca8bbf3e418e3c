// Shared pieces of the streaming quantized matvec: PTX wrappers, kernel parameters, and the prologue
// that turns the f32 activation into int8 MMA operands in shared memory.
#pragma once
#include "tlb_internal.h"

namespace tlb {

constexpr int kMaxCols = 8;        // columns of the MMA B operand (n = 8)

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
// The clock is first read after 64 failed polls: a wait that ends sooner (nearly all of them) never pays for it.
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *err, int code)
{
    unsigned long long t0 = 0;
    for (int it = 0;; it++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 63) == 63) {
            if (*abort_flag) return false;
            const unsigned long long now = global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > 2000000000ull) {
                *abort_flag = 1;
                atomicExch(err, code);
                return false;
            }
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *err, int code)
{
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, abort_flag, err, code);
}
__device__ __forceinline__ bool mbar_wait_drain(uint32_t bar, uint32_t parity)
{
    unsigned long long t0 = 0;
    for (int it = 0;; it++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 63) == 63) {
            const unsigned long long now = global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > 1000000000ull) return false;
        }
    }
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void named_bar(int id, int threads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
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
// (a & m) | o in one LOP3 (register operands: two immediates cannot be encoded in one instruction)
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t m, uint32_t o)
{
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(m), "r"(o));
    return d;
}
__device__ __forceinline__ float2 h2_to_f2(uint32_t h)
{
    return __half22float2(*reinterpret_cast<const __half2 *>(&h));
}
__device__ __forceinline__ uint32_t word_of(const uint4 &v, int i)
{
    return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w));
}
// D(16x8 f32) += A(16x16 f16, row) * B(16x8 f16, col)
__device__ __forceinline__ void hmma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1)
{
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// D(16x8 s32) = A(16x32 u8 or s8, row) * B(32x8 s8, col); exact integer sums
template <bool A_SIGNED>
__device__ __forceinline__ void imma16832(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    if (A_SIGNED)
        asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                     : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
    else
        asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                     : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// ---------------------------------------------------------------- kernel parameters

struct MvParams {
    const uint8_t *w[3];
    float *out[3];            // [m][n_rows] per tensor
    float *part;              // slice scratch [kb][tiles][m][16] (kb > 1): the partial result of every item
    int *tile_cnt;            // [tiles] slices of a tile finished so far; zero between launches (m > 1)
    int fold_poll;            // m == 1: `part` rests at kFoldEmpty between launches; the warp that owns slice 0 of a tile
                              // waits for the other slices' values to replace it, adds them and puts it back
    int tiles_end[3];         // cumulative tile counts
    int n_rows[3];            // valid output rows per tensor
    int n_w;
    int upt;                  // units per tile = K / 256
    int k;
    int m;                    // activation rows, 1..4
    int nl;                   // int8 levels per activation row (3 for m <= 2, else 2)
    // Work decomposition.  An ITEM is one tile (16 rows) x one K-slice of `upi` consecutive units; item
    // index = slice * tiles + tile (slice-major), so the contiguous item range of a CTA touches one or two
    // slices and needs only those blocks of the activation.  One warp owns an item from the first byte to
    // its 16 * m partial results, which it WRITES (never adds) to part[slice][tile]; the warp that
    // finishes a tile's last slice adds the slices in index order into the output.
    int upi;                  // units per item (divides upt)
    int kb;                   // K-slices = output slices = upt / upi
    int tiles;                // tiles of the launch (all tensors)
    int n_items;              // kb * tiles
    int ipc_q, ipc_r;         // n_items = grid * ipc_q + ipc_r: CTA b takes ipc_q (+1 if b < ipc_r) consecutive items
    int nb_max;               // 256-blocks of activation a CTA may need: the shared tables are sized for it
    int unit_bytes, stage_bytes;
    int spw;                  // ring stages private to each warp
    int max_seg, off_seg;     // kb == 1: slots of partial results per warp in shared memory, and where they start
    int prologue;
    const float *x;           // PLAIN: x [M,K]; ADD_NORM: residual; SILU_MUL: gate
    const float *x2;          // ADD_NORM: delta added to x (null: none); SILU_MUL: up
    const float *norm_w;
    const float *ssq_parts;   // ADD_NORM: partial sums of squares of x left by its producer (null: computed here)
    int n_parts;
    const float *att_part;    // ATTN_MERGE: per-split attention results [kv head][att_max_splits][att_rep][att_dim + 4]
    const int *att_pos;
    int att_max_splits, att_rep, att_dim, att_keys;
    int off_wtab;             // ATTN_MERGE: softmax weights of the splits per query head of this CTA
    int finish;               // FIN_*: what the warp completing a tile does with its results
    const float *resid;       // FIN_RESID: added to the result
    float *ssq_out;           // FIN_RESID: [tiles] sum of squares of each finished tile
    float eps;
    float *x_out;             // ADD_NORM: residual + delta written here by CTA 0 (may be null)
    const float *emb_table;
    const int *token;
    int *err;
    int use_pdl;
    int tp_reduce;            // the tile results are partial sums over tensor-parallel ranks: summed inside the launch (TpFuse)
    TpFuse tp;
    // shared-memory offsets (bytes from the start of dynamic shared memory)
    int off_xq, off_alam, off_xsum, off_sa, off_minv, off_bars, off_misc;
    int col_stride;           // bytes between int8 activation columns (nb_max * 256 + 64)
};

constexpr unsigned kFoldEmpty = 0xFFFFFFFFu;   // a NaN bit pattern no sum produces

// Scratch of the prologue.
struct MvShared {
    float red_sum[32];
    float red_max[32];
    int abort_flag;
};

__device__ __forceinline__ unsigned ld_acquire_sys_u32(const unsigned *p)
{
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_sys_u32(unsigned *p, unsigned v)
{
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_volatile_u32(const unsigned *p)
{
    unsigned v;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ float silu_f(float g) { return g * (1.0f / (1.0f + expf(-g))); }

// Elements 4*i4 .. 4*i4+3 of an activation written by an earlier kernel of the stream, hence the
// L2-coherent load.
__device__ __forceinline__ float4 ld_act4(const float *v, size_t i4)
{
    return __ldcg(reinterpret_cast<const float4 *>(v) + i4);
}

// Activation elements 4*k4 .. 4*k4+3 of row `mrow` as the matvec consumes them.  inv_rms == 0 selects
// the statistics pass of PRO_ADD_NORM (returns the un-normalised residual sum).  `emb` replaces p.x
// when the residual is an embedding row.
__device__ __forceinline__ float4 prologue_value(const MvParams &p, const float *emb, int mrow, int k4, float inv_rms)
{
    const size_t row4 = (size_t)mrow * (p.k / 4) + k4;
    float4 v = emb ? __ldg(reinterpret_cast<const float4 *>(emb) + row4) : ld_act4(p.x, row4);
    if (p.prologue == PRO_ADD_NORM) {
        if (p.x2) {
            const float4 d = ld_act4(p.x2, row4);
            v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
        }
        if (inv_rms != 0.f) {  // (x / rms) * weight (crates/tl_cpu/src/ffi.rs:2444-2486), the division as a multiply by 1/rms
            float4 w = __ldg(reinterpret_cast<const float4 *>(p.norm_w) + k4);
            v.x = (v.x * inv_rms) * w.x; v.y = (v.y * inv_rms) * w.y;
            v.z = (v.z * inv_rms) * w.z; v.w = (v.w * inv_rms) * w.w;
        }
    } else if (p.prologue == PRO_SILU_MUL) {
        const float4 u = ld_act4(p.x2, row4);
        v.x = silu_f(v.x) * u.x; v.y = silu_f(v.y) * u.y; v.z = silu_f(v.z) * u.z; v.w = silu_f(v.w) * u.w;
    }
    return v;
}

}  // namespace tlb

