// Kernels of prompt processing (many tokens at once) around the tensor-core GEMM: embedding rows, RoPE of
// q and k with the append of k and v to the cache, and causal GQA attention of the new tokens over the
// cache.  They compute what the fused decode chain computes for one token at a time - the op sequence of
// examples/apps/llama3/chatbot_llama3.tl:66-125 (embedding, rms_norm, apply_rope, kv update, scaled
// scores + causal mask + softmax, context) - for T tokens per launch.
//
// Attention: head_dim 128 over an f16 cache (64 tokens or more) runs on tcgen05 (prefill_attn_tc.cu); every other case -
// head_dim 64, an f32 cache, short prompts - runs here as a streaming-softmax kernel on mma.sync (f16 operands, f32
// accumulation): one CTA per (64 queries, head), each warp 16 queries; K and V tiles of 64 cache rows are staged in shared
// memory as f16 (converted on the way when the cache is f32), scores never leave registers.  The projections run in
// qgemm_tc.cu.
#include <algorithm>

#include "qmv_common.cuh"

namespace tlb {

namespace {

// ---- embedding rows: x[i, :] = table[tokens[i], :]  (crates/tl_cpu/src/tensor.rs:1094-1112)
__global__ void embed_rows_kernel(const int *__restrict__ tokens, const float *__restrict__ table, float *__restrict__ x, int dm)
{
    const float4 *src = reinterpret_cast<const float4 *>(table + (size_t)tokens[blockIdx.x] * dm);
    float4 *dst = reinterpret_cast<float4 *>(x + (size_t)blockIdx.x * dm);
    for (int i = threadIdx.x; i < dm / 4; i += blockDim.x) dst[i] = __ldg(src + i);
}

// ---- RoPE (adjacent pairs, crates/tl_cpu/src/ffi.rs:2629-2685) of q in place and of k into the cache, v into
// the cache.  Token i sits in cache row pos0 + i and is rotated by table row rope0 + i * rope_step.
// Same operation order as the decode attention kernel, so a prompt and a token-by-token run write the same bits.
template <typename T>
__global__ void rope_append_kernel(float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                                   T *__restrict__ kcache, T *__restrict__ vcache, const float *__restrict__ cos_t,
                                   const float *__restrict__ sin_t, int H, int KVH, int D, int max_seq, int pos0, int rope0, int rope_step)
{
    const int i = blockIdx.x;
    const float *cs = cos_t + (size_t)(rope0 + i * rope_step) * D, *sn = sin_t + (size_t)(rope0 + i * rope_step) * D;
    const int half = D / 2;
    for (int t = threadIdx.x; t < H * half; t += blockDim.x) {
        const int h = t / half, j = (t - h * half) * 2;
        float *p = q + ((size_t)i * H + h) * D + j;
        const float a = p[0], b = p[1], c = cs[j], s = sn[j];
        p[0] = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
        p[1] = __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c));
    }
    for (int t = threadIdx.x; t < KVH * half; t += blockDim.x) {
        const int h = t / half, j = (t - h * half) * 2;
        const float *pk = k + ((size_t)i * KVH + h) * D + j, *pv = v + ((size_t)i * KVH + h) * D + j;
        const float a = pk[0], b = pk[1], c = cs[j], s = sn[j];
        const size_t row = ((size_t)h * max_seq + pos0 + i) * D + j;
        if constexpr (sizeof(T) == 2) {
            kcache[row] = __float2half_rn(__fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s)));
            kcache[row + 1] = __float2half_rn(__fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c)));
            vcache[row] = __float2half_rn(pv[0]);
            vcache[row + 1] = __float2half_rn(pv[1]);
        } else {
            kcache[row] = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
            kcache[row + 1] = __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c));
            vcache[row] = pv[0];
            vcache[row + 1] = pv[1];
        }
    }
}

// ---- causal attention of T new tokens over the cache
constexpr int kPfQ = 64;     // queries per CTA
constexpr int kPfK = 64;     // cache rows per tile
constexpr int kPfThreads = 128;

__device__ __forceinline__ uint32_t pack_half2(float a, float b)
{
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ float exp2_approx(float x)   // 2^x, relative error 2^-22; 2^-inf = 0
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

struct PfAttnParams {
    const float *q;        // [T, H * D], rotated
    const void *kcache, *vcache;   // [KVH][max_seq][D] of this layer
    float *out;            // [T, H * D]
    int T, H, KVH, max_seq, pos0;
    float scale;
};

template <typename CT, int D>
__global__ void __launch_bounds__(kPfThreads, 3) prefill_attention_kernel(const PfAttnParams p)
{
    constexpr int RS = D + 8;                   // shared row stride in halves: 16-byte aligned rows, conflict-free fragments
    constexpr bool kAsync = sizeof(CT) == 2;    // f16 cache rows go to shared memory with cp.async, one tile ahead
    constexpr int kBuf = kAsync ? 2 : 1;
    extern __shared__ __align__(16) __half pf_smem[];   // [kBuf][K tile | V tile]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
    const int h = blockIdx.y, kvh = h / (p.H / p.KVH);
    const int qtile = (int)(gridDim.x - 1 - blockIdx.x);    // late query tiles see the most cache rows: they start first
    const int q0 = qtile * kPfQ + warp * 16;                // first query row of this warp
    const int qd = p.H * D;
    const CT *kc = reinterpret_cast<const CT *>(p.kcache) + (size_t)kvh * p.max_seq * D;
    const CT *vc = reinterpret_cast<const CT *>(p.vcache) + (size_t)kvh * p.max_seq * D;

    // Q fragments (A operand, 16 x D) of rows q0 + g and q0 + g + 8, straight from global memory
    uint32_t qa[D / 16][4];
    {
        const int r0 = min(q0 + g, p.T - 1), r1 = min(q0 + g + 8, p.T - 1);
        const float *qr0 = p.q + (size_t)r0 * qd + h * D, *qr1 = p.q + (size_t)r1 * qd + h * D;
#pragma unroll
        for (int ks = 0; ks < D / 16; ks++) {
            const float2 a = *reinterpret_cast<const float2 *>(qr0 + ks * 16 + 2 * c), b = *reinterpret_cast<const float2 *>(qr1 + ks * 16 + 2 * c);
            const float2 a8 = *reinterpret_cast<const float2 *>(qr0 + ks * 16 + 8 + 2 * c), b8 = *reinterpret_cast<const float2 *>(qr1 + ks * 16 + 8 + 2 * c);
            qa[ks][0] = pack_half2(a.x, a.y); qa[ks][1] = pack_half2(b.x, b.y);
            qa[ks][2] = pack_half2(a8.x, a8.y); qa[ks][3] = pack_half2(b8.x, b8.y);
        }
    }
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};
    const float scale2 = p.scale * 1.4426950408889634f;
    const int pq0 = p.pos0 + q0 + g, pq1 = pq0 + 8;          // cache positions of this thread's two query rows

    const int last_q = min(qtile * kPfQ + kPfQ, p.T) - 1;
    const int n_tiles = (p.pos0 + last_q) / kPfK + 1;        // tiles that hold a key <= the CTA's last query
    auto tile_async = [&](int t) {   // cache rows of tile t -> buffer t % 2, asynchronously
        __half *ks = pf_smem + (size_t)(t & 1) * 2 * kPfK * RS, *vs = ks + kPfK * RS;
        for (int i = tid; i < kPfK * (D / 8); i += kPfThreads) {
            const int key = i / (D / 8), ch = i - key * (D / 8);
            const int row = min(t * kPfK + key, p.max_seq - 1);
            cp_async16(smem_u32(ks + key * RS + ch * 8), kc + (size_t)row * D + ch * 8);
            cp_async16(smem_u32(vs + key * RS + ch * 8), vc + (size_t)row * D + ch * 8);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if constexpr (kAsync) tile_async(0);
    for (int t = 0; t < n_tiles; t++) {
        const int key0 = t * kPfK;
        const __half *Ks = pf_smem + (size_t)(kAsync ? (t & 1) : 0) * 2 * kPfK * RS, *Vs = Ks + kPfK * RS;
        if constexpr (kAsync) {
            // the buffer tile t + 1 goes to was read in iteration t - 1, which ended with a barrier
            if (t + 1 < n_tiles) {
                tile_async(t + 1);
                asm volatile("cp.async.wait_group 1;" ::: "memory");
            } else {
                asm volatile("cp.async.wait_group 0;" ::: "memory");
            }
        } else {
            __half *ks = pf_smem, *vs = pf_smem + kPfK * RS;
            for (int i = tid; i < kPfK * (D / 8); i += kPfThreads) {
                const int key = i / (D / 8), ch = i - key * (D / 8);
                const int row = min(key0 + key, p.max_seq - 1);
                const float4 a = *reinterpret_cast<const float4 *>(kc + (size_t)row * D + ch * 8), b = *reinterpret_cast<const float4 *>(kc + (size_t)row * D + ch * 8 + 4);
                const float4 e = *reinterpret_cast<const float4 *>(vc + (size_t)row * D + ch * 8), f = *reinterpret_cast<const float4 *>(vc + (size_t)row * D + ch * 8 + 4);
                *reinterpret_cast<uint4 *>(ks + key * RS + ch * 8) = make_uint4(pack_half2(a.x, a.y), pack_half2(a.z, a.w), pack_half2(b.x, b.y), pack_half2(b.z, b.w));
                *reinterpret_cast<uint4 *>(vs + key * RS + ch * 8) = make_uint4(pack_half2(e.x, e.y), pack_half2(e.z, e.w), pack_half2(f.x, f.y), pack_half2(f.z, f.w));
            }
        }
        __syncthreads();

        // scores S = Q K^T of 16 queries x 64 keys
        float s[kPfK / 8][4];
#pragma unroll
        for (int nb = 0; nb < kPfK / 8; nb++) {
            s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
            // K fragments of two 16-wide steps per ldmatrix: matrices = dims +0, +8, +16, +24 of keys nb * 8 ..
            const __half *krow = Ks + (nb * 8 + (lane & 7)) * RS + (lane >> 3) * 8;
#pragma unroll
            for (int ks = 0; ks < D / 16; ks += 2) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(smem_u32(krow + ks * 16), b0, b1, b2, b3);
                hmma16816(s[nb], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
                hmma16816(s[nb], qa[ks + 1][0], qa[ks + 1][1], qa[ks + 1][2], qa[ks + 1][3], b2, b3);
            }
        }
        // scale (times log2 e: the exponentials below are base 2), causal mask, running max
        float tmax[2] = {-INFINITY, -INFINITY};
        const bool diagonal = key0 + kPfK - 1 > p.pos0 + q0;   // some key of the tile is ahead of some query of this warp
#pragma unroll
        for (int nb = 0; nb < kPfK / 8; nb++) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int key = key0 + nb * 8 + 2 * c + (e & 1), pq = (e < 2) ? pq0 : pq1;
                const float v = (!diagonal || key <= pq) ? s[nb][e] * scale2 : -INFINITY;
                s[nb][e] = v;
                tmax[e >> 1] = fmaxf(tmax[e >> 1], v);
            }
        }
        float corr[2], mnew[2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 1));
            tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 2));
            mnew[r] = fmaxf(mrow[r], tmax[r]);               // finite from the first tile on: key 0 is visible to every query
            corr[r] = exp2_approx(mrow[r] - mnew[r]);
            mrow[r] = mnew[r];
        }
        float tsum[2] = {0.f, 0.f};
        uint32_t pa[kPfK / 16][4];
#pragma unroll
        for (int nb = 0; nb < kPfK / 8; nb++) {
            const float e0 = exp2_approx(s[nb][0] - mnew[0]), e1 = exp2_approx(s[nb][1] - mnew[0]);
            const float e2 = exp2_approx(s[nb][2] - mnew[1]), e3 = exp2_approx(s[nb][3] - mnew[1]);
            tsum[0] += e0 + e1;
            tsum[1] += e2 + e3;
            pa[nb >> 1][(nb & 1) * 2] = pack_half2(e0, e1);
            pa[nb >> 1][(nb & 1) * 2 + 1] = pack_half2(e2, e3);
        }
#pragma unroll
        for (int r = 0; r < 2; r++) lrow[r] = lrow[r] * corr[r] + tsum[r];   // per-thread partial; the quad is summed at the end
#pragma unroll
        for (int nb = 0; nb < D / 8; nb++) {
            o[nb][0] *= corr[0]; o[nb][1] *= corr[0];
            o[nb][2] *= corr[1]; o[nb][3] *= corr[1];
        }
        // O += P V: V fragments through ldmatrix.trans (rows = keys)
#pragma unroll
        for (int ks = 0; ks < kPfK / 16; ks++) {
#pragma unroll
            for (int nb = 0; nb < D / 8; nb += 2) {
                uint32_t b0, b1, b2, b3;
                const __half *vrow = Vs + (ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * RS + nb * 8 + (lane >> 4) * 8;
                ldmatrix_x4_trans(smem_u32(vrow), b0, b1, b2, b3);
                hmma16816(o[nb], pa[ks][0], pa[ks][1], pa[ks][2], pa[ks][3], b0, b1);
                hmma16816(o[nb + 1], pa[ks][0], pa[ks][1], pa[ks][2], pa[ks][3], b2, b3);
            }
        }
        __syncthreads();   // the tile has been consumed: its buffer may be refilled
    }
#pragma unroll
    for (int r = 0; r < 2; r++) {
        lrow[r] += __shfl_xor_sync(0xffffffffu, lrow[r], 1);
        lrow[r] += __shfl_xor_sync(0xffffffffu, lrow[r], 2);
    }
    const float inv0 = 1.f / lrow[0], inv1 = 1.f / lrow[1];
    const int r0 = q0 + g, r1 = q0 + g + 8;
#pragma unroll
    for (int nb = 0; nb < D / 8; nb++) {
        if (r0 < p.T) *reinterpret_cast<float2 *>(p.out + (size_t)r0 * qd + h * D + nb * 8 + 2 * c) = make_float2(o[nb][0] * inv0, o[nb][1] * inv0);
        if (r1 < p.T) *reinterpret_cast<float2 *>(p.out + (size_t)r1 * qd + h * D + nb * 8 + 2 * c) = make_float2(o[nb][2] * inv1, o[nb][3] * inv1);
    }
}

}  // namespace

tlb_status launch_embed_rows(const int *tokens, const float *table, float *x, int n_tokens, int dm)
{
    if (n_tokens <= 0) return TLB_OK;
    embed_rows_kernel<<<n_tokens, 256, 0, ctx()->stream>>>(tokens, table, x, dm);
    count_launch();
    return TLB_OK;
}

tlb_status launch_rope_append(float *q, const float *k, const float *v, void *kcache, void *vcache, int kv_f16, const float *cos_t,
                              const float *sin_t, int n_tokens, int H, int KVH, int D, int max_seq, int pos0, int rope0, int rope_step)
{
    if (n_tokens <= 0) return TLB_OK;
    if (kv_f16)
        rope_append_kernel<__half><<<n_tokens, 256, 0, ctx()->stream>>>(q, k, v, (__half *)kcache, (__half *)vcache, cos_t, sin_t, H, KVH, D, max_seq, pos0, rope0, rope_step);
    else
        rope_append_kernel<float><<<n_tokens, 256, 0, ctx()->stream>>>(q, k, v, (float *)kcache, (float *)vcache, cos_t, sin_t, H, KVH, D, max_seq, pos0, rope0, rope_step);
    count_launch();
    return TLB_OK;
}

bool prefill_attention_supported(int D) { return D == 64 || D == 128; }

tlb_status launch_prefill_attention(const float *q, const void *kcache, const void *vcache, int kv_f16, float *out, int n_tokens, int H,
                                    int KVH, int D, int max_seq, int pos0, float scale)
{
    if (n_tokens <= 0) return TLB_OK;
    if (!prefill_attention_supported(D)) return fail(TLB_ERR_SHAPE, "prompt attention: head_dim %d is not supported (64 or 128)", D);
    // head_dim 128 over an f16 cache, 64 tokens or more: both products on tcgen05 (prefill_attn_tc.cu)
    if (prefill_attention_tc_supported(D, kv_f16, n_tokens)) return launch_prefill_attention_tc(q, kcache, vcache, out, n_tokens, H, KVH, max_seq, pos0, scale);
    PfAttnParams p;
    p.q = q; p.kcache = kcache; p.vcache = vcache; p.out = out;
    p.T = n_tokens; p.H = H; p.KVH = KVH; p.max_seq = max_seq; p.pos0 = pos0; p.scale = scale;
    dim3 grid((unsigned)((n_tokens + kPfQ - 1) / kPfQ), (unsigned)H);
    const size_t tile_bytes = (size_t)2 * kPfK * (D + 8) * sizeof(__half);      // one K tile + one V tile
    const size_t smem = tile_bytes * (kv_f16 ? 2 : 1);
    static bool attr_set = false;
    if (!attr_set) {   // the double-buffered variants need more than the default 48 KB at head_dim 128
        TLB_CUDA(cudaFuncSetAttribute(prefill_attention_kernel<__half, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(4 * kPfK * 136 * sizeof(__half))));
        attr_set = true;
    }
    if (D == 128) {
        if (kv_f16) prefill_attention_kernel<__half, 128><<<grid, kPfThreads, smem, ctx()->stream>>>(p);
        else prefill_attention_kernel<float, 128><<<grid, kPfThreads, smem, ctx()->stream>>>(p);
    } else {
        if (kv_f16) prefill_attention_kernel<__half, 64><<<grid, kPfThreads, smem, ctx()->stream>>>(p);
        else prefill_attention_kernel<float, 64><<<grid, kPfThreads, smem, ctx()->stream>>>(p);
    }
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "prompt attention launch");
    return TLB_OK;
}

}  // namespace tlb
