// Causal GQA attention of T new tokens over an f16 cache on the 5th-generation tensor cores (head_dim 128): what
// prefill_attention_kernel (prefill.cu, mma.sync) computes - scaled scores, causal mask, softmax, context
// (examples/apps/llama3/chatbot_llama3.tl:66-125) - with both products on tcgen05.mma and scores, probabilities and the output
// accumulator in tensor memory.
//
// One CTA = one query head x 128 queries.  Per tile of 128 cache rows:
//   S = Q K^T   Q [128 q x 128 d] and the K tile [128 keys x 128 d] in shared memory (TMA, 128-byte swizzle), S [128 x 128] f32
//               in tensor memory, two buffers so that the scores of tile t + 1 are computed while tile t goes through softmax;
//   softmax     four warps, one thread per query row (its tensor-memory lane): the row's 128 scores with tcgen05.ld, scale,
//               causal mask, running maximum and sum in base 2; when a row's maximum moves the output accumulator's row is
//               rescaled in place (tcgen05.ld / st, skipped when no row of the warp moved); probabilities as f16 pairs
//               into tensor memory (tcgen05.st) - the A operand of the second product, never through shared memory;
//   O += P V    P from tensor memory, V^T tile [128 d x 128 keys] from shared memory (the cache keeps V as [key][d]; a
//               transposed f16 copy of the rows in use is made per launch so that the operand is K-major), O [128 x 128] f32
//               in tensor memory.
// Warp roles: 0-3 softmax / write-out, 4 TMA (lane 0), 5 MMA issue (lane 0) and tensor-memory allocation.
// Every mbarrier wait is bounded (qmv_common.cuh: mbar_wait): when one runs out the CTA sets the context's error word,
// lets its copies land, frees its tensor memory and returns.
#include <algorithm>

#include "tc05.cuh"

namespace tlb {

namespace {

constexpr int kAtQ = 128, kAtK = 128, kAtD = 128;
constexpr int kAtThreads = 192;
constexpr int kBoxBytes = 128 * 128;            // one TMA box: 128 rows x 64 f16
constexpr int kTileBytes = 2 * kBoxBytes;       // a 128 x 128 f16 operand = two boxes
// tensor memory columns
constexpr uint32_t kColS = 0, kColO = 256, kColP = 384;

struct AtParams {
    float *out;            // [T, H * 128]
    int T, H, KVH, max_seq, pos0, vt_rows;
    float scale2;          // attn_scale * log2(e)
    int *err;
};

__device__ __forceinline__ float ex2f(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b)
{
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}

__global__ void __launch_bounds__(kAtThreads, 1)
prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                            const __grid_constant__ CUtensorMap vtmap, const AtParams p)
{
    extern __shared__ uint8_t at_smem[];
    __shared__ int abort_word;
    __shared__ uint32_t tmem_slot;
    volatile int *abort_flag = &abort_word;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t base = (smem_u32(at_smem) + 1023u) & ~1023u;
    const uint32_t sQ = base, sK = base + kTileBytes, sV = sK + 2 * kTileBytes;     // K and V^T: two stages each
    const uint32_t bars = sV + 2 * kTileBytes;
    const uint32_t q_full = bars, kv_full = bars + 8, kv_empty = bars + 24, s_full = bars + 40, p_full = bars + 56, o_full = bars + 64;

    const int h = blockIdx.y, kvh = h / (p.H / p.KVH);
    const int qtile = (int)(gridDim.x - 1 - blockIdx.x);          // late query tiles see the most cache rows: they start first
    const int q0 = qtile * kAtQ;
    const int last_q = min(q0 + kAtQ, p.T) - 1;
    const int n_tiles = (p.pos0 + last_q) / kAtK + 1;             // tiles that hold a key <= the CTA's last query

    if (tid == 0) {
        abort_word = 0;
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; i++) { mbar_init(kv_full + 8 * i, 1); mbar_init(kv_empty + 8 * i, 1); mbar_init(s_full + 8 * i, 1); }
        mbar_init(p_full, 4);
        mbar_init(o_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;

    if (warp < 4) {
        // ------------------------------------------------ softmax: thread = query row
        const int row = warp * 32 + lane, q = q0 + row, qpos = p.pos0 + q;
        const uint32_t tl = tmem + ((uint32_t)(warp * 32) << 16);      // this warp's lanes
        float m_run = -INFINITY, l_run = 0.f;
        bool ok = true;
        for (int t = 0; t < n_tiles && ok; t++) {
            const int b = t & 1, key0 = t * kAtK;
            if (!mbar_wait(s_full + 8 * b, (uint32_t)(t >> 1) & 1u, abort_flag, p.err, 41)) { ok = false; break; }
            tc_fence_after();
            float s[128];
#pragma unroll
            for (int c = 0; c < 4; c++) tmem_ld32(tl + kColS + (uint32_t)(b * 128 + c * 32), reinterpret_cast<uint32_t *>(s) + c * 32);
            tmem_wait_ld();
            const bool diagonal = key0 + kAtK - 1 > p.pos0 + q0;     // some key of the tile is ahead of some query of the CTA
            float m_tile = -INFINITY;
#pragma unroll
            for (int c = 0; c < 128; c++) {
                const float v = (!diagonal || key0 + c <= qpos) ? s[c] * p.scale2 : -INFINITY;
                s[c] = v;
                m_tile = fmaxf(m_tile, v);
            }
            const float m_new = fmaxf(m_run, m_tile);                // finite from the first tile on: key 0 is visible to every query
            const float corr = ex2f(m_run - m_new);
            m_run = m_new;
            if (t > 0) {
                // the product of tile t - 1 has read P and added to O: O may be rescaled, P overwritten
                if (!mbar_wait(o_full, (uint32_t)(t - 1) & 1u, abort_flag, p.err, 42)) { ok = false; break; }
                tc_fence_after();
                if (__any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        uint32_t o[32];
                        tmem_ld32(tl + kColO + (uint32_t)(c * 32), o);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
                        tmem_st32(tl + kColO + (uint32_t)(c * 32), o);
                    }
                }
            }
            float sum = 0.f;
#pragma unroll
            for (int c = 0; c < 2; c++) {
                uint32_t pk[32];
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    const float e0 = ex2f(s[c * 64 + 2 * i] - m_new), e1 = ex2f(s[c * 64 + 2 * i + 1] - m_new);
                    sum += e0 + e1;
                    pk[i] = pack_h2(e0, e1);
                }
                tmem_st32(tl + kColP + (uint32_t)(c * 32), pk);
            }
            l_run = l_run * corr + sum;
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);
        }
        // ------------------------------------------------ write-out: O / l
        if (ok && mbar_wait(o_full, (uint32_t)(n_tiles - 1) & 1u, abort_flag, p.err, 43)) {
            tc_fence_after();
            const float inv = 1.f / l_run;
            float *dst = p.out + (size_t)q * (p.H * kAtD) + h * kAtD;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                uint32_t o[32];
                tmem_ld32(tl + kColO + (uint32_t)(c * 32), o);
                tmem_wait_ld();
                if (q < p.T) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        *reinterpret_cast<float4 *>(dst + c * 32 + i) = make_float4(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv,
                                                                                  __uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
                }
            }
        }
    } else if (warp == 4) {
        // ------------------------------------------------ TMA: Q once, then K and V^T tiles two ahead
        if (lane == 0) {
            mbar_expect_tx(q_full, kTileBytes);
            tma_load_2d(sQ, &qmap, h * kAtD, q0, q_full);
            tma_load_2d(sQ + kBoxBytes, &qmap, h * kAtD + 64, q0, q_full);
            int issued = 0;
            for (int t = 0; t < n_tiles; t++) {
                const int st = t & 1;
                if (t >= 2 && !mbar_wait(kv_empty + 8 * st, (uint32_t)((t - 2) >> 1) & 1u, abort_flag, p.err, 44)) break;
                mbar_expect_tx(kv_full + 8 * st, 2 * kTileBytes);
                const int key0 = t * kAtK;
                tma_load_2d(sK + st * kTileBytes, &kmap, 0, kvh * p.max_seq + key0, kv_full + 8 * st);
                tma_load_2d(sK + st * kTileBytes + kBoxBytes, &kmap, 64, kvh * p.max_seq + key0, kv_full + 8 * st);
                tma_load_2d(sV + st * kTileBytes, &vtmap, key0, kvh * kAtD, kv_full + 8 * st);
                tma_load_2d(sV + st * kTileBytes + kBoxBytes, &vtmap, key0 + 64, kvh * kAtD, kv_full + 8 * st);
                issued = t + 1;
            }
            if (*abort_flag) {
                mbar_wait_drain(q_full, 0);
                for (int t = max(0, issued - 2); t < issued; t++) mbar_wait_drain(kv_full + 8 * (t & 1), (uint32_t)(t >> 1) & 1u);
            }
        }
    } else {
        // ------------------------------------------------ MMA issue
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);   // f32 D, f16 A/B, K-major both, M 128, N 128
            bool ok = mbar_wait(q_full, 0, abort_flag, p.err, 45);
            auto scores = [&](int t) {   // S[t & 1] = Q K(t)^T
                const int st = t & 1;
                if (!mbar_wait(kv_full + 8 * st, (uint32_t)(t >> 1) & 1u, abort_flag, p.err, 46)) return false;
                tc_fence_after();
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const uint64_t ad = smem_desc_sw128(sQ + j * kBoxBytes), bd = smem_desc_sw128(sK + st * kTileBytes + j * kBoxBytes);
#pragma unroll
                    for (int k16 = 0; k16 < 4; k16++) umma_f16_ss(tmem + kColS + (uint32_t)(st * 128), ad + 2u * k16, bd + 2u * k16, idesc, (j | k16) != 0);
                }
                umma_commit(s_full + 8 * st);
                return true;
            };
            if (ok) ok = scores(0);
            for (int t = 0; t < n_tiles && ok; t++) {
                if (t + 1 < n_tiles) ok = scores(t + 1);      // its S buffer was read by the softmax of tile t - 1, which p_full(t - 1) confirmed
                if (!ok) break;
                if (!mbar_wait(p_full, (uint32_t)t & 1u, abort_flag, p.err, 47)) { ok = false; break; }
                tc_fence_after();
                const int st = t & 1;
#pragma unroll
                for (int j = 0; j < 2; j++) {                 // keys 64 j .. 64 j + 63: tensor-memory columns 32 j .. of P, box j of V^T
                    const uint64_t bd = smem_desc_sw128(sV + st * kTileBytes + j * kBoxBytes);
#pragma unroll
                    for (int k16 = 0; k16 < 4; k16++)
                        umma_f16_ts(tmem + kColO, tmem + kColP + (uint32_t)(j * 32 + k16 * 8), bd + 2u * k16, idesc, (t | j | k16) != 0);
                }
                umma_commit(o_full);
                umma_commit(kv_empty + 8 * st);
            }
            if (!ok) {
                // MMAs already issued finish before the tensor memory is freed: one more commit, waited for (bounded)
                umma_commit(q_full);
                mbar_wait_drain(q_full, 1);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

// q f32 [T, cols] -> f16, and V rows [kvh][key][128] of the cache -> V^T [kvh][128][keys_ld] for keys < n_keys
__global__ void q_to_f16_kernel(const float *__restrict__ q, __half *__restrict__ qh, size_t n4)
{
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        const float4 v = reinterpret_cast<const float4 *>(q)[i];
        __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
        uint2 o;
        o.x = *reinterpret_cast<uint32_t *>(&a);
        o.y = *reinterpret_cast<uint32_t *>(&b);
        reinterpret_cast<uint2 *>(qh)[i] = o;
    }
}
__global__ void __launch_bounds__(256) v_transpose_kernel(const __half *__restrict__ vcache, __half *__restrict__ vt, int max_seq, int n_keys, int keys_ld)
{
    __shared__ __half tile[32][34];
    const __half *src = vcache + (size_t)blockIdx.z * max_seq * kAtD;
    __half *dst = vt + (size_t)blockIdx.z * kAtD * keys_ld;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int d0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
    for (int j = ty; j < 32; j += 8)
        tile[j][tx] = (k0 + j < n_keys) ? src[(size_t)(k0 + j) * kAtD + d0 + tx] : __float2half(0.f);
    __syncthreads();
    for (int j = ty; j < 32; j += 8)
        if (k0 + tx < keys_ld) dst[(size_t)(d0 + j) * keys_ld + k0 + tx] = tile[tx][j];
}

}  // namespace

bool prefill_attention_tc_supported(int D, int kv_f16, int n_tokens) { return D == 128 && kv_f16 && n_tokens >= 64; }

tlb_status launch_prefill_attention_tc(const float *q, const void *kcache, const void *vcache, float *out, int n_tokens, int H, int KVH,
                                       int max_seq, int pos0, float scale)
{
    Context *c = ctx();
    if (!c) return TLB_ERR_DEVICE;
    const int T = n_tokens, n_keys = pos0 + T, keys_ld = (n_keys + 127) / 128 * 128;
    Storage *qh = storage_alloc((size_t)T * H * kAtD * sizeof(__half));
    Storage *vt = storage_alloc((size_t)KVH * kAtD * keys_ld * sizeof(__half));
    if (!qh || !vt) { if (qh) storage_release(qh); if (vt) storage_release(vt); return TLB_ERR_ALLOC; }
    auto done = [&](tlb_status st) { storage_release(qh); storage_release(vt); return st; };   // stream-ordered: freed after the launches below
    const size_t n4 = (size_t)T * H * kAtD / 4;
    q_to_f16_kernel<<<(unsigned)std::min<size_t>(148 * 8, (n4 + 255) / 256), 256, 0, c->stream>>>(q, (__half *)qh->ptr, n4);
    dim3 tg(kAtD / 32, (unsigned)(keys_ld / 32), (unsigned)KVH);
    v_transpose_kernel<<<tg, 256, 0, c->stream>>>((const __half *)vcache, (__half *)vt->ptr, max_seq, n_keys, keys_ld);
    count_launch(2);
    CUtensorMap qmap, kmap, vtmap;
    if (!encode_f16_map(&qmap, qh->ptr, (uint64_t)H * kAtD, (uint64_t)T, (uint64_t)H * kAtD * 2, 64, 128) ||
        !encode_f16_map(&kmap, kcache, kAtD, (uint64_t)KVH * max_seq, kAtD * 2, 64, 128) ||
        !encode_f16_map(&vtmap, vt->ptr, (uint64_t)keys_ld, (uint64_t)KVH * kAtD, (uint64_t)keys_ld * 2, 64, 128))
        return done(fail(TLB_ERR_DEVICE, "prompt attention: cuTensorMapEncodeTiled failed or is not available"));
    AtParams p;
    p.out = out; p.T = T; p.H = H; p.KVH = KVH; p.max_seq = max_seq; p.pos0 = pos0; p.vt_rows = keys_ld;
    p.scale2 = scale * 1.4426950408889634f;
    p.err = c->err_flag;
    const size_t smem = (size_t)5 * kTileBytes + 1024 + 128;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(prefill_attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return done(cuda_fail(e, "prompt attention attribute"));
        attr_set = true;
    }
    dim3 grid((unsigned)((T + kAtQ - 1) / kAtQ), (unsigned)H);
    prefill_attention_tc_kernel<<<grid, kAtThreads, smem, c->stream>>>(qmap, kmap, vtmap, p);
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return done(cuda_fail(e, "prompt attention launch"));
    return done(TLB_OK);
}

}  // namespace tlb
