// Attention kernels.
//
// decode_attention_kernel: one new token against the KV cache, split over the key axis
// (flash-decoding).  It replaces, for the decode step of the TL programs
// (examples/apps/llama3/chatbot_llama3.tl:66-107), the op sequence apply_rope x2, transpose,
// cat_4d (a full re-copy of the cache per step, crates/tl_cuda/src/cuda_kernels/autograd.cu:760-776),
// repeat_interleave (materialised GQA expansion, :1253-1268), matmul_4d, scale, softmax, matmul_4d,
// transpose: RoPE of q and of the new k, the in-place cache append, GQA-aware scores, softmax and
// the weighted sum of V happen in one launch, and the last CTA of each KV head merges the splits.
//
// sdpa_kernel: the generic tl_tensor_sdpa entry (flash_attention_kernel, autograd.cu:2263-2367).
#include "tlb_internal.h"

#include <algorithm>

namespace tlb {

constexpr int kAttnThreads = 512;
constexpr int kKeysPerCta = kAttnKeysPerSplit;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

template <typename T> struct KvTraits;
template <> struct KvTraits<__half> {
    static constexpr int E = 8;  // elements per 16-byte chunk
    __device__ static void load(const uint4 &v, float (&f)[8])
    {
        const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
        for (int i = 0; i < 4; i++) { float2 t = __half22float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
    }
    __device__ static float2 load2(const void *p) { return __half22float2(*reinterpret_cast<const __half2 *>(p)); }
    __device__ static __half store(float x) { return __float2half_rn(x); }
    __device__ static float round(float x) { return __half2float(__float2half_rn(x)); }
};
template <> struct KvTraits<float> {
    static constexpr int E = 4;
    __device__ static void load(const uint4 &v, float (&f)[8])
    {
        f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
    }
    __device__ static float2 load2(const void *p) { return *reinterpret_cast<const float2 *>(p); }
    __device__ static float store(float x) { return x; }
    __device__ static float round(float x) { return x; }
};

struct AttnParams {
    // new projections of sequence b: q + b * q_stride ([H * D]), k + b * kv_stride, v + b * kv_stride ([KVH * D]) floats
    const float *q, *k, *v;
    int q_stride, kv_stride;
    size_t cache_seq_bytes;   // bytes between the caches of consecutive sequences (0 for one sequence)
    int state_stride;         // ints between the pos / rope_pos entries of consecutive sequences
    void *kcache, *vcache;
    int H, KVH, D, max_seq;
    const int *pos, *rope_pos;
    const float *cos_t, *sin_t;
    float scale;
    float *partial;   // [KVH][max_splits][rep][D + 4]: D weighted sums, then the split's maximum and sum of exponentials (rows stay 16-byte aligned)
    int defer_merge;  // the consumer (o_proj prologue) merges the splits: write partial results only
    int *counters;    // [KVH]
    int max_splits;
    float *out;       // [H * D]
    int use_pdl;
    int dyn_splits;   // batch kernel: as many key ranges as the cache rows need (one per kAttnKeysPerSplit rows, what the o_proj prologue expects) instead of gridDim.x
    int row_stride;   // shared-memory row stride in bytes (16-byte chunks, count = 4 mod 8: conflict-free)
};


template <typename T, int REP>
__global__ void __launch_bounds__(kAttnThreads, 1) decode_attention_kernel(const AttnParams p)
{
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int E = KvTraits<T>::E;
    const int D = p.D, tid = threadIdx.x;
    const int kvh = blockIdx.y, split = blockIdx.x, seq = blockIdx.z;   // one grid plane per sequence of a batch
    const int RC = D / E;                // 16-byte chunks per row
    const int RS = p.row_stride;
    uint8_t *Ks = smem;
    uint8_t *Vs = Ks + (size_t)kKeysPerCta * RS;
    float *qs = reinterpret_cast<float *>(Vs + (size_t)kKeysPerCta * RS);  // [REP][D]
    float *S = qs + REP * D;                                               // [keys][REP] probabilities
    float *ml = S + kKeysPerCta * REP;                                     // [REP][2]
    float *accbuf = ml + REP * 2;                                          // [NG][REP][D]
    __shared__ int is_last;

    // Cache length and this CTA's key range.  pos was written at the end of the previous decode
    // step, which every predecessor of this launch has already waited for.
    const int pos = p.pos[(size_t)seq * p.state_stride];
    const int Tlen = pos + 1;
    const int nsplit = (Tlen + kKeysPerCta - 1) / kKeysPerCta;
    if (split >= nsplit) return;
    const int per = (Tlen + nsplit - 1) / nsplit;
    const int t0 = split * per, t1 = min(Tlen, t0 + per), nk = t1 - t0;

    // stage K and V rows [t0, t1) (rows of earlier tokens; row `pos` is patched below)
    {
        const T *kc = reinterpret_cast<const T *>(reinterpret_cast<const uint8_t *>(p.kcache) + seq * p.cache_seq_bytes) + ((size_t)kvh * p.max_seq + t0) * D;
        const T *vc = reinterpret_cast<const T *>(reinterpret_cast<const uint8_t *>(p.vcache) + seq * p.cache_seq_bytes) + ((size_t)kvh * p.max_seq + t0) * D;
        const uint32_t ks = (uint32_t)__cvta_generic_to_shared(Ks), vs = (uint32_t)__cvta_generic_to_shared(Vs);
        for (int i = tid; i < nk * RC; i += kAttnThreads) {
            int key = i / RC, ch = i - key * RC;
            if (t0 + key == pos) continue;
            cp_async16(ks + key * RS + ch * 16, reinterpret_cast<const uint8_t *>(kc) + ((size_t)key * RC + ch) * 16);
            cp_async16(vs + key * RS + ch * 16, reinterpret_cast<const uint8_t *>(vc) + ((size_t)key * RC + ch) * 16);
        }
    }
    // What does not depend on the projections is fetched before the dependency wait: the RoPE position
    // (written at the end of the previous step, like pos) and this thread's entries of the static tables.
    // Thread i < REP * D/2 rotates pair i of the REP query heads; in the CTA whose range holds row `pos`,
    // thread i < D/2 also rotates pair i of the new K and appends K and V.
    static_assert(REP * 64 <= kAttnThreads, "one query pair per thread");
    const int rp = p.rope_pos[(size_t)seq * p.state_stride];
    const float *cs = p.cos_t + (size_t)rp * D, *sn = p.sin_t + (size_t)rp * D;
    const bool rot_q = tid < REP * (D / 2);
    const bool app = pos >= t0 && pos < t1 && tid < D / 2;
    const int hq = tid / (D / 2), jq = (tid - hq * (D / 2)) * 2, jk = 2 * tid;
    float cq = 0.f, sq = 0.f, ck = 0.f, sk = 0.f;
    if (rot_q) { cq = __ldg(cs + jq); sq = __ldg(sn + jq); }
    if (app) { ck = __ldg(cs + jk); sk = __ldg(sn + jk); }
    if (p.use_pdl) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }
    // all loads of the new projections first (one round trip), then the arithmetic
    float q0 = 0.f, q1 = 0.f, k0f = 0.f, k1f = 0.f, v0f = 0.f, v1f = 0.f;
    const float *qrow = p.q + (size_t)seq * p.q_stride + (size_t)(kvh * REP + hq) * D + jq;
    const float *krow_new = p.k + (size_t)seq * p.kv_stride + (size_t)kvh * D + jk, *vrow_new = p.v + (size_t)seq * p.kv_stride + (size_t)kvh * D + jk;
    if (rot_q) { q0 = __ldcg(qrow); q1 = __ldcg(qrow + 1); }
    if (app) { k0f = __ldcg(krow_new); k1f = __ldcg(krow_new + 1); v0f = __ldcg(vrow_new); v1f = __ldcg(vrow_new + 1); }
    // RoPE (crates/tl_cpu/src/ffi.rs:2629-2685: adjacent pairs, one table row) of the REP query heads
    if (rot_q) {
        qs[hq * D + jq] = __fsub_rn(__fmul_rn(q0, cq), __fmul_rn(q1, sq));
        qs[hq * D + jq + 1] = __fadd_rn(__fmul_rn(q0, sq), __fmul_rn(q1, cq));
    }
    // the CTA whose range holds row `pos` appends the new token's K (roped) and V
    if (app) {
        T *kc = reinterpret_cast<T *>(reinterpret_cast<uint8_t *>(p.kcache) + seq * p.cache_seq_bytes) + ((size_t)kvh * p.max_seq + pos) * D;
        T *vc = reinterpret_cast<T *>(reinterpret_cast<uint8_t *>(p.vcache) + seq * p.cache_seq_bytes) + ((size_t)kvh * p.max_seq + pos) * D;
        T *krow = reinterpret_cast<T *>(Ks + (size_t)(pos - t0) * RS), *vrow = reinterpret_cast<T *>(Vs + (size_t)(pos - t0) * RS);
        T k0 = KvTraits<T>::store(__fsub_rn(__fmul_rn(k0f, ck), __fmul_rn(k1f, sk)));
        T k1 = KvTraits<T>::store(__fadd_rn(__fmul_rn(k0f, sk), __fmul_rn(k1f, ck)));
        T v0 = KvTraits<T>::store(v0f), v1 = KvTraits<T>::store(v1f);
        krow[jk] = k0; krow[jk + 1] = k1; vrow[jk] = v0; vrow[jk + 1] = v1;
        kc[jk] = k0; kc[jk + 1] = k1; vc[jk] = v0; vc[jk + 1] = v1;
    }
    cp_async_wait_all();
    __syncthreads();

    // scores: thread (key = tid/4, dq = tid%4) covers chunks dq, dq+4, ... of its key row, all REP heads
    {
        const int key = tid >> 2, dq = tid & 3;
        float dot[REP];
#pragma unroll
        for (int h = 0; h < REP; h++) dot[h] = 0.f;
        if (key < nk) {
            const uint8_t *krow = Ks + (size_t)key * RS;
            for (int ch = dq; ch < RC; ch += 4) {
                float kf[8];
                KvTraits<T>::load(*reinterpret_cast<const uint4 *>(krow + ch * 16), kf);
#pragma unroll
                for (int h = 0; h < REP; h++) {
                    const float *qv = qs + h * D + ch * E;
#pragma unroll
                    for (int e = 0; e < E; e += 4) {
                        float4 q4 = *reinterpret_cast<const float4 *>(qv + e);
                        dot[h] += q4.x * kf[e] + q4.y * kf[e + 1] + q4.z * kf[e + 2] + q4.w * kf[e + 3];
                    }
                }
            }
        }
#pragma unroll
        for (int h = 0; h < REP; h++) {
            dot[h] += __shfl_xor_sync(0xffffffffu, dot[h], 1);
            dot[h] += __shfl_xor_sync(0xffffffffu, dot[h], 2);
        }
        if (dq == 0) {
#pragma unroll
            for (int h = 0; h < REP; h++) S[key * REP + h] = key < nk ? dot[h] * p.scale : -INFINITY;
        }
    }
    __syncthreads();
    // per-head softmax statistics over this CTA's keys: warp h handles head h
    {
        const int warp = tid >> 5, lane = tid & 31;
        if (warp < REP) {
            float v[kKeysPerCta / 32], mx = -INFINITY;
#pragma unroll
            for (int i = 0; i < kKeysPerCta / 32; i++) { v[i] = S[(lane + 32 * i) * REP + warp]; mx = fmaxf(mx, v[i]); }
            for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            float sum = 0.f;
#pragma unroll
            for (int i = 0; i < kKeysPerCta / 32; i++) {
                float e = expf(v[i] - mx);   // exp(-inf) = 0 for padded keys
                S[(lane + 32 * i) * REP + warp] = e;
                sum += e;
            }
            for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            if (lane == 0) { ml[warp * 2] = mx; ml[warp * 2 + 1] = sum; }
        }
    }
    __syncthreads();
    // weighted sum of V: thread (kg, dp) covers the pair of dims (2dp, 2dp+1) for keys kg, kg+NG, ...
    const int NG = kAttnThreads / (D / 2);
    {
        const int dp = tid % (D / 2), kg = tid / (D / 2);
        float acc[REP][2];
#pragma unroll
        for (int h = 0; h < REP; h++) acc[h][0] = acc[h][1] = 0.f;
        for (int key = kg; key < nk; key += NG) {
            float2 v2 = KvTraits<T>::load2(Vs + (size_t)key * RS + dp * 2 * sizeof(T));
#pragma unroll
            for (int h = 0; h < REP; h++) {
                float pr = S[key * REP + h];
                acc[h][0] += pr * v2.x;
                acc[h][1] += pr * v2.y;
            }
        }
#pragma unroll
        for (int h = 0; h < REP; h++)
            *reinterpret_cast<float2 *>(accbuf + ((size_t)kg * REP + h) * D + 2 * dp) = make_float2(acc[h][0], acc[h][1]);
    }
    __syncthreads();
    const int kvh_all = seq * p.KVH + kvh;        // (sequence, KV head) as one index into the per-head scratch and outputs
    float *part = p.partial + ((size_t)kvh_all * p.max_splits + split) * REP * (D + 4);
    for (int i = tid; i < REP * D; i += kAttnThreads) {
        float s = 0.f;
        for (int g = 0; g < NG; g++) s += accbuf[(size_t)g * REP * D + i];
        int h = i / D, d = i - h * D;
        if (nsplit == 1 && !p.defer_merge) {
            p.out[(size_t)(kvh_all * REP + h) * D + d] = s / ml[h * 2 + 1];
        } else {
            part[h * (D + 4) + d] = s;
        }
    }
    if (nsplit == 1 && !p.defer_merge) return;
    if (tid < REP) { part[tid * (D + 4) + D] = ml[tid * 2]; part[tid * (D + 4) + D + 1] = ml[tid * 2 + 1]; }
    if (p.defer_merge) return;
    // the last CTA of this KV head to finish merges all splits
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        int old = atomicAdd(p.counters + kvh_all, 1);
        is_last = (old == nsplit - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    const float *base = p.partial + (size_t)kvh_all * p.max_splits * REP * (D + 4);
    for (int i = tid; i < REP * D; i += kAttnThreads) {
        int h = i / D, d = i - h * D;
        float M = -INFINITY;
#pragma unroll 8
        for (int s = 0; s < nsplit; s++) M = fmaxf(M, __ldcg(base + ((size_t)s * REP + h) * (D + 4) + D));
        float L = 0.f, O = 0.f;
#pragma unroll 8
        for (int s = 0; s < nsplit; s++) {
            const float *ps = base + ((size_t)s * REP + h) * (D + 4);
            float w = expf(__ldcg(ps + D) - M);
            L += __ldcg(ps + D + 1) * w;
            O += __ldcg(ps + d) * w;
        }
        p.out[(size_t)(kvh_all * REP + h) * D + d] = O / L;
    }
    if (tid == 0) p.counters[kvh_all] = 0;
}

static int attn_row_stride(int D, int esize)
{
    int rc = D * esize / 16, rs = rc;
    while (rs % 8 != 4) rs++;
    return rs * 16;
}

template <typename T, int REP>
static tlb_status launch_decode_t(const AttnParams &p, int max_splits, int KVH, int batch, bool pdl)
{
    int NG = kAttnThreads / (p.D / 2);
    size_t smem = (size_t)2 * kKeysPerCta * p.row_stride + (size_t)(REP * p.D + kKeysPerCta * REP + REP * 2 + NG * REP * p.D) * sizeof(float);
    if (smem + 1024 > ctx()->smem_optin) return fail(TLB_ERR_SHAPE, "decode attention needs %zu bytes of shared memory", smem);
    static size_t set_bytes = 0;   // the kernel also has a few bytes of static shared memory
    if (smem > set_bytes) {
        TLB_CUDA(cudaFuncSetAttribute(decode_attention_kernel<T, REP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        // same L1 / shared-memory split as the matvec kernels around it: the SMs never re-partition between launches
        TLB_CUDA(cudaFuncSetAttribute(decode_attention_kernel<T, REP>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        set_bytes = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(max_splits, KVH, batch);
    cfg.blockDim = dim3(kAttnThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx()->stream;
    cudaLaunchAttribute at[1];
    if (pdl) {
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at;
        cfg.numAttrs = 1;
    }
    TLB_CUDA(cudaLaunchKernelEx(&cfg, decode_attention_kernel<T, REP>, p));
    count_launch();
    return TLB_OK;
}

// ---------------------------------------------------------------- decode attention of a batch of sequences
// With B sequences a layer's attention reads B caches, as many bytes as its weights from a few thousand rows of context
// on, and the kernel above - one 128-key split per CTA, one CTA per SM, its phases one after the other - leaves HBM idle
// most of the time.  Here a WARP is the worker: it owns a contiguous range of 16-key blocks of one (sequence, KV head),
// streams them through a ring of its own (cp.async, three stages) and keeps the running maximum, sum and weighted V sum
// of the REP query heads in registers: Q.K^T and P.V on mma.sync.m16n8k16 (rows = the REP <= 8 query heads of the KV
// head, padded to 16; f16 operands, f32 accumulation; K rows by ldmatrix, V rows by ldmatrix.trans).  Four warps share a
// CTA (two CTAs per SM), merge their results in shared memory and write one split; the last CTA of a (sequence, KV head)
// merges the splits as above.  The warp that holds the last block rotates and appends the new token's K and V.  The
// rotated, scaled query enters as two f16 parts (value and remainder, two MMAs per K tile), so the scores carry the
// query at ~22 bits as the kernel above does; the probabilities are f16.
// One sequence on an f16 cache takes the same kernel (dyn_splits): a key range per kAttnKeysPerSplit rows in use, two
// blocks per warp, the partial results left for the o_proj launch to merge - the phases of the kernel above (stage 128
// rows, scores, softmax, weighted sum, reduction over 8 key groups) become one pass per warp.
constexpr int kBatWarps = 4, kBatThreads = kBatWarps * 32, kBatBlk = 16, kBatStages = 3;

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
// rows 0-7 of D(16x8) += A(16x16) * B(16x8) where rows 8-15 of A are zero: only the two accumulators of row lane / 4 are kept
__device__ __forceinline__ void mma_top8(float (&d)[2], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1)
{
    float j0, j1;
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%5}, {%7,%8}, {%0,%1,%9,%9};"
        : "+f"(d[0]), "+f"(d[1]), "=f"(j0), "=f"(j1) : "r"(a0), "r"(0u), "r"(a2), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b)
{
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}

template <int D, int REP>
__global__ void __launch_bounds__(kBatThreads, 2) batch_decode_attention_kernel(const AttnParams p)
{
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int RS = D * 2 + 16;                 // bytes between staged rows: consecutive rows shift by one 16-byte bank group
    constexpr int STAGE = 2 * kBatBlk * RS;        // K rows, then V rows of one block
    constexpr int KS = D / 16, DT = D / 8, RC = D / 8;
    static_assert(REP <= 8, "the query heads of a KV head are the top eight rows of the MMA");
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
    const int chunk = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
    __half *qs = reinterpret_cast<__half *>(smem);                 // [2][8][D]: rotated, scaled queries as f16 and what that leaves; rows REP.. zero
    const uint32_t ring = (uint32_t)__cvta_generic_to_shared(smem) + 2 * 8 * D * 2 + (uint32_t)warp * kBatStages * STAGE;
    __shared__ int is_last;

    const int pos = p.pos[(size_t)seq * p.state_stride];
    const int Tlen = pos + 1, nb = (Tlen + kBatBlk - 1) / kBatBlk;
    const int nchunk = p.dyn_splits ? (Tlen + kAttnKeysPerSplit - 1) / kAttnKeysPerSplit : (int)gridDim.x;
    if (chunk >= nchunk) return;
    const int workers = nchunk * kBatWarps, w = chunk * kBatWarps + warp;
    const int b0 = (int)((int64_t)nb * w / workers), b1 = (int)((int64_t)nb * (w + 1) / workers);
    const bool owner = w == workers - 1;           // its range ends with the last block: row `pos`
    const __half *kc = reinterpret_cast<const __half *>(reinterpret_cast<const uint8_t *>(p.kcache) + seq * p.cache_seq_bytes) + (size_t)kvh * p.max_seq * D;
    const __half *vc = reinterpret_cast<const __half *>(reinterpret_cast<const uint8_t *>(p.vcache) + seq * p.cache_seq_bytes) + (size_t)kvh * p.max_seq * D;

    // rows of earlier tokens; row `pos` is written by hand below, rows past it count as zero
    auto load_block = [&](int blk, int stage) {
        const uint32_t sK = ring + stage * STAGE, sV = sK + kBatBlk * RS;
        for (int i = lane; i < kBatBlk * RC; i += 32) {
            const int row = i / RC, ch = i - row * RC, key = blk * kBatBlk + row;
            if (key >= pos) {
                if (key > pos) asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(sV + row * RS + ch * 16), "r"(0u) : "memory");
                continue;
            }
            cp_async16(sK + row * RS + ch * 16, kc + (size_t)key * D + ch * 8);
            cp_async16(sV + row * RS + ch * 16, vc + (size_t)key * D + ch * 8);
        }
    };
    for (int s = 0; s < kBatStages - 1; s++) {
        if (b0 + s < b1) load_block(b0 + s, s);
        cp_async_commit();
    }

    const int rp = p.rope_pos[(size_t)seq * p.state_stride];
    const float *cs = p.cos_t + (size_t)rp * D, *sn = p.sin_t + (size_t)rp * D;
    if (p.use_pdl) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }
    // RoPE (crates/tl_cpu/src/ffi.rs:2629-2685: adjacent pairs, one table row) of the REP query heads, times the softmax scale
    for (int i = tid; i < 8 * (D / 2); i += kBatThreads) {
        const int hq = i / (D / 2), jq = (i - hq * (D / 2)) * 2;
        float r0 = 0.f, r1 = 0.f;
        if (hq < REP) {
            const float *qrow = p.q + (size_t)seq * p.q_stride + (size_t)(kvh * REP + hq) * D + jq;
            const float q0 = __ldcg(qrow), q1 = __ldcg(qrow + 1), cq = __ldg(cs + jq), sq = __ldg(sn + jq);
            r0 = __fsub_rn(__fmul_rn(q0, cq), __fmul_rn(q1, sq)) * p.scale;
            r1 = __fadd_rn(__fmul_rn(q0, sq), __fmul_rn(q1, cq)) * p.scale;
        }
        const __half2 hi = __floats2half2_rn(r0, r1);
        const float2 hf = __half22float2(hi);
        *reinterpret_cast<__half2 *>(qs + hq * D + jq) = hi;
        *reinterpret_cast<__half2 *>(qs + (8 + hq) * D + jq) = __floats2half2_rn(r0 - hf.x, r1 - hf.y);   // the query keeps ~22 bits
    }
    // the new token's K (rotated) and V: into the cache, and kept for the staged copy of the last block
    uint32_t knew[D / 64], vnew[D / 64];
    if (owner) {
#pragma unroll
        for (int i = 0; i < D / 64; i++) {
            const int jk = 2 * (lane + 32 * i);
            const float *krow = p.k + (size_t)seq * p.kv_stride + (size_t)kvh * D + jk, *vrow = p.v + (size_t)seq * p.kv_stride + (size_t)kvh * D + jk;
            const float k0f = __ldcg(krow), k1f = __ldcg(krow + 1), ck = __ldg(cs + jk), sk = __ldg(sn + jk);
            knew[i] = pack_h2(__fsub_rn(__fmul_rn(k0f, ck), __fmul_rn(k1f, sk)), __fadd_rn(__fmul_rn(k0f, sk), __fmul_rn(k1f, ck)));
            vnew[i] = pack_h2(__ldcg(vrow), __ldcg(vrow + 1));
            *reinterpret_cast<uint32_t *>(const_cast<__half *>(kc) + (size_t)pos * D + jk) = knew[i];
            *reinterpret_cast<uint32_t *>(const_cast<__half *>(vc) + (size_t)pos * D + jk) = vnew[i];
        }
    }
    __syncthreads();
    uint32_t qa[KS][2], ql[KS][2];
#pragma unroll
    for (int kk = 0; kk < KS; kk++) {
        qa[kk][0] = *reinterpret_cast<const uint32_t *>(qs + g * D + kk * 16 + 2 * c);
        qa[kk][1] = *reinterpret_cast<const uint32_t *>(qs + g * D + kk * 16 + 2 * c + 8);
        ql[kk][0] = *reinterpret_cast<const uint32_t *>(qs + (8 + g) * D + kk * 16 + 2 * c);
        ql[kk][1] = *reinterpret_cast<const uint32_t *>(qs + (8 + g) * D + kk * 16 + 2 * c + 8);
    }

    float m = -INFINITY, l = 0.f, o[DT][2];
#pragma unroll
    for (int dt = 0; dt < DT; dt++) o[dt][0] = o[dt][1] = 0.f;
    for (int blk = b0; blk < b1; blk++) {
        const int it = blk - b0, stage = it % kBatStages;
        if (blk + kBatStages - 1 < b1) load_block(blk + kBatStages - 1, (it + kBatStages - 1) % kBatStages);
        cp_async_commit();
        cp_async_wait_group<kBatStages - 1>();      // this lane's copies of block `blk` have landed
        __syncwarp();                               // ... and the other lanes'
        const uint32_t sK = ring + stage * STAGE, sV = sK + kBatBlk * RS;
        if (blk == nb - 1) {                        // only the owner gets here: the new token's row
            const int row = pos - blk * kBatBlk;
#pragma unroll
            for (int i = 0; i < D / 64; i++) {
                asm volatile("st.shared.u32 [%0], %1;" ::"r"(sK + row * RS + 4 * (lane + 32 * i)), "r"(knew[i]) : "memory");
                asm volatile("st.shared.u32 [%0], %1;" ::"r"(sV + row * RS + 4 * (lane + 32 * i)), "r"(vnew[i]) : "memory");
            }
            __syncwarp();
        }
        // scores of the block's 16 keys (two tiles of 8) for query head g: s[nt] = keys 8 nt + 2c, + 1
        float s[2][2];
#pragma unroll
        for (int nt = 0; nt < 2; nt++) {
            s[nt][0] = s[nt][1] = 0.f;
#pragma unroll
            for (int k2 = 0; k2 < KS / 2; k2++) {   // four 8 x 8 matrices: keys 8 nt .., dims 32 k2 + 8 j ..
                uint32_t kb[4];
                ldsm_x4(kb, sK + (nt * 8 + (lane & 7)) * RS + (k2 * 32 + (lane >> 3) * 8) * 2);
                mma_top8(s[nt], qa[2 * k2][0], qa[2 * k2][1], kb[0], kb[1]);
                mma_top8(s[nt], ql[2 * k2][0], ql[2 * k2][1], kb[0], kb[1]);
                mma_top8(s[nt], qa[2 * k2 + 1][0], qa[2 * k2 + 1][1], kb[2], kb[3]);
                mma_top8(s[nt], ql[2 * k2 + 1][0], ql[2 * k2 + 1][1], kb[2], kb[3]);
            }
        }
        float mx = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int e = 0; e < 2; e++) {
                if (blk * kBatBlk + nt * 8 + 2 * c + e > pos) s[nt][e] = -INFINITY;
                mx = fmaxf(mx, s[nt][e]);
            }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m, mx);           // finite: every block holds a key <= pos
        const float alpha = expf(m - m_new);
        float pr[2][2], psum = 0.f;
#pragma unroll
        for (int nt = 0; nt < 2; nt++)
#pragma unroll
            for (int e = 0; e < 2; e++) { pr[nt][e] = expf(s[nt][e] - m_new); psum += pr[nt][e]; }
        l = l * alpha + psum;
        m = m_new;
#pragma unroll
        for (int dt = 0; dt < DT; dt++) { o[dt][0] *= alpha; o[dt][1] *= alpha; }
        const uint32_t pa0 = pack_h2(pr[0][0], pr[0][1]), pa2 = pack_h2(pr[1][0], pr[1][1]);
#pragma unroll
        for (int d2 = 0; d2 < DT / 2; d2++) {       // four 8 x 8 matrices, transposed: (keys 0-7 | 8-15) x dims 16 d2 + (0-7 | 8-15)
            uint32_t vb[4];
            const int j = lane >> 3;
            ldsm_x4_t(vb, sV + ((j & 1) * 8 + (lane & 7)) * RS + (d2 * 16 + (j >> 1) * 8) * 2);
            mma_top8(o[2 * d2], pa0, pa2, vb[0], vb[1]);
            mma_top8(o[2 * d2 + 1], pa0, pa2, vb[2], vb[3]);
        }
        __syncwarp();                               // the stage is free for the copy issued at the top of the next iteration
    }
    cp_async_wait_group<0>();
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);

    // the CTA's four warps merge in shared memory (the rings are done with)
    __syncthreads();
    float *scr = reinterpret_cast<float *>(smem + 2 * 8 * D * 2);   // [warp][8][D + 2]: weighted sums, maximum, sum
    {
        float *mine = scr + ((size_t)warp * 8 + g) * (D + 2);
#pragma unroll
        for (int dt = 0; dt < DT; dt++) *reinterpret_cast<float2 *>(mine + dt * 8 + 2 * c) = make_float2(o[dt][0], o[dt][1]);
        if (c == 0) { mine[D] = m; mine[D + 1] = l; }
    }
    __syncthreads();
    const int kvh_all = seq * p.KVH + kvh;
    float *part = p.partial + ((size_t)kvh_all * p.max_splits + chunk) * REP * (D + 4);
    for (int i = tid; i < REP * D; i += kBatThreads) {
        const int h = i / D, d = i - h * D;
        float M = -INFINITY;
#pragma unroll
        for (int wq = 0; wq < kBatWarps; wq++) M = fmaxf(M, scr[((size_t)wq * 8 + h) * (D + 2) + D]);
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int wq = 0; wq < kBatWarps; wq++) {
            const float *ps = scr + ((size_t)wq * 8 + h) * (D + 2);
            const float wgt = ps[D] == -INFINITY ? 0.f : expf(ps[D] - M);    // a warp (or the whole CTA) may have had no block
            L += ps[D + 1] * wgt;
            O += ps[d] * wgt;
        }
        if (nchunk == 1 && !p.defer_merge) p.out[(size_t)(kvh_all * REP + h) * D + d] = O / L;
        else {
            part[h * (D + 4) + d] = O;
            if (d == 0) { part[h * (D + 4) + D] = M; part[h * (D + 4) + D + 1] = L; }
        }
    }
    if (nchunk == 1 || p.defer_merge) return;      // deferred: the consumer (o_proj prologue) merges the key ranges
    // the last CTA of this (sequence, KV head) to finish merges all splits
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        int old = atomicAdd(p.counters + kvh_all, 1);
        is_last = (old == nchunk - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    const float *base = p.partial + (size_t)kvh_all * p.max_splits * REP * (D + 4);
    for (int i = tid; i < REP * D; i += kBatThreads) {
        const int h = i / D, d = i - h * D;
        float M = -INFINITY;
        for (int sp = 0; sp < nchunk; sp++) M = fmaxf(M, __ldcg(base + ((size_t)sp * REP + h) * (D + 4) + D));
        float L = 0.f, O = 0.f;
        for (int sp = 0; sp < nchunk; sp++) {
            const float *ps = base + ((size_t)sp * REP + h) * (D + 4);
            const float ms = __ldcg(ps + D), wgt = ms == -INFINITY ? 0.f : expf(ms - M);
            L += __ldcg(ps + D + 1) * wgt;
            O += __ldcg(ps + d) * wgt;
        }
        p.out[(size_t)(kvh_all * REP + h) * D + d] = O / L;
    }
    if (tid == 0) p.counters[kvh_all] = 0;
}

template <int D, int REP>
static tlb_status launch_decode_batch_t(const AttnParams &p, int chunks, int KVH, int batch, bool pdl)
{
    constexpr size_t smem = (size_t)2 * 8 * D * 2 + (size_t)kBatWarps * kBatStages * (2 * kBatBlk * (D * 2 + 16));
    static bool set = false;
    if (!set) {
        TLB_CUDA(cudaFuncSetAttribute(batch_decode_attention_kernel<D, REP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        TLB_CUDA(cudaFuncSetAttribute(batch_decode_attention_kernel<D, REP>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        set = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(chunks, KVH, batch);
    cfg.blockDim = dim3(kBatThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx()->stream;
    cudaLaunchAttribute at[1];
    if (pdl) {
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at;
        cfg.numAttrs = 1;
    }
    TLB_CUDA(cudaLaunchKernelEx(&cfg, batch_decode_attention_kernel<D, REP>, p));
    count_launch();
    return TLB_OK;
}

tlb_status launch_decode_attention(const DecodeAttnJob &j)
{
    if (j.D != 64 && j.D != 128) return fail(TLB_ERR_SHAPE, "decode attention supports head_dim 64 and 128, got %d", j.D);
    if (j.H % j.KVH) return fail(TLB_ERR_SHAPE, "query heads must be a multiple of KV heads");
    int rep = j.H / j.KVH;
    AttnParams p;
    const int batch = j.batch > 1 ? j.batch : 1;
    if (j.q) { p.q = j.q; p.k = j.k; p.v = j.v; p.q_stride = j.H * j.D; p.kv_stride = j.KVH * j.D; }
    else { p.q = j.qkv; p.k = j.qkv + (size_t)j.H * j.D; p.v = j.qkv + (size_t)(j.H + j.KVH) * j.D; p.q_stride = p.kv_stride = 0; }
    p.cache_seq_bytes = j.cache_seq_bytes; p.state_stride = j.state_stride;
    p.kcache = j.kcache; p.vcache = j.vcache;
    p.H = j.H; p.KVH = j.KVH; p.D = j.D; p.max_seq = j.max_seq;
    p.pos = j.pos; p.rope_pos = j.rope_pos; p.cos_t = j.cos_t; p.sin_t = j.sin_t; p.scale = j.scale;
    p.defer_merge = j.defer_merge ? 1 : 0;
    p.partial = j.partial; p.counters = j.counters; p.max_splits = j.splits; p.out = j.out;
    p.use_pdl = j.pdl ? 1 : 0;
    p.row_stride = attn_row_stride(j.D, j.kv_f16 ? 2 : 4);
    p.dyn_splits = 0;
    if (j.kv_f16 && rep <= 8) {
        // f16 caches: warps as workers on the tensor cores.  A batch: as many key ranges per (sequence, KV head) as give
        // every SM its two CTAs.  One sequence: a key range per kAttnKeysPerSplit rows in use, the split the o_proj
        // prologue merges (grid = the most the cache can need; the CTAs beyond leave at once).
        int chunks = std::max(1, std::min(j.splits, 2 * ctx()->sm_count / (j.KVH * batch)));
        if (batch == 1) { chunks = j.splits; p.dyn_splits = 1; }
#define DISPATCH_B(DV, REPV) if (j.D == DV && rep == REPV) return launch_decode_batch_t<DV, REPV>(p, chunks, j.KVH, batch, j.pdl);
        DISPATCH_B(128, 1) DISPATCH_B(128, 2) DISPATCH_B(128, 4) DISPATCH_B(128, 8)
        DISPATCH_B(64, 1) DISPATCH_B(64, 2) DISPATCH_B(64, 4) DISPATCH_B(64, 8)
#undef DISPATCH_B
    }
#define DISPATCH(REPV)                                                                         \
    if (rep == REPV)                                                                           \
        return j.kv_f16 ? launch_decode_t<__half, REPV>(p, j.splits, j.KVH, batch, j.pdl)      \
                        : launch_decode_t<float, REPV>(p, j.splits, j.KVH, batch, j.pdl);
    DISPATCH(1) DISPATCH(2) DISPATCH(4) DISPATCH(8)
#undef DISPATCH
    return fail(TLB_ERR_SHAPE, "decode attention supports 1, 2, 4 or 8 query heads per KV head, got %d", rep);
}

// ---------------------------------------------------------------- generic SDPA
// One block per (batch*head, query row).  mask_mode 1: additive; 2: zero entries -> -1e9.
__global__ void sdpa_kernel(const float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                            const float *__restrict__ mask, int mask_mode, float *__restrict__ out, int64_t sq, int64_t sk,
                            int64_t d, int64_t mask_bh, float scale)
{
    extern __shared__ float sc[];  // [sk] scores, then 32 floats of reduction scratch
    float *red = sc + sk;
    const int64_t bh = blockIdx.y, i = blockIdx.x;
    const float *qv = q + (bh * sq + i) * d, *kb = k + bh * sk * d, *vb = v + bh * sk * d;
    const float *mrow = mask ? mask + ((mask_bh > 1 ? bh : 0) * sq + i) * sk : nullptr;
    float mx = -INFINITY;
    for (int64_t j = threadIdx.x; j < sk; j += blockDim.x) {
        float s = 0.f;
        for (int64_t e = 0; e < d; e++) s += qv[e] * kb[j * d + e];
        s *= scale;
        if (mrow) {
            if (mask_mode == 1) s += mrow[j];
            else if (mrow[j] == 0.0f) s = -1e9f;
        }
        sc[j] = s;
        mx = fmaxf(mx, s);
    }
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) red[w] = mx;
    __syncthreads();
    mx = red[0];
    for (int x = 1; x < nw; x++) mx = fmaxf(mx, red[x]);
    __syncthreads();
    float sum = 0.f;
    for (int64_t j = threadIdx.x; j < sk; j += blockDim.x) {
        float e = expf(sc[j] - mx);
        sc[j] = e;
        sum += e;
    }
    for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) red[w] = sum;
    __syncthreads();
    sum = 0.f;
    for (int x = 0; x < nw; x++) sum += red[x];
    for (int64_t e = threadIdx.x; e < d; e += blockDim.x) {
        float acc = 0.f;
        for (int64_t j = 0; j < sk; j++) acc += (sc[j] / sum) * vb[j * d + e];
        out[(bh * sq + i) * d + e] = acc;
    }
}

tlb_status launch_sdpa(const float *q, const float *k, const float *v, const float *mask, int mask_mode, float *out,
                       int64_t bh, int64_t sq, int64_t sk, int64_t d, int64_t mask_bh)
{
    if (bh * sq * d == 0) return TLB_OK;
    if (sk == 0) return fail(TLB_ERR_SHAPE, "sdpa: empty key sequence");
    size_t smem = (size_t)(sk + 32) * sizeof(float);
    if (smem > ctx()->smem_optin) return fail(TLB_ERR_SHAPE, "sdpa: key length %lld exceeds the single-pass limit", (long long)sk);
    static bool set = false;
    if (!set) {
        TLB_CUDA(cudaFuncSetAttribute(sdpa_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ctx()->smem_optin));
        set = true;
    }
    if (sq > 65535 * 32768LL || bh > 65535) return fail(TLB_ERR_SHAPE, "sdpa: grid too large");
    sdpa_kernel<<<dim3((unsigned)sq, (unsigned)bh), 128, smem, ctx()->stream>>>(q, k, v, mask, mask_mode, out, sq, sk, d, mask_bh,
                                                                               1.0f / sqrtf((float)d));
    count_launch();
    TLB_CUDA(cudaGetLastError());
    return TLB_OK;
}

}  // namespace tlb
