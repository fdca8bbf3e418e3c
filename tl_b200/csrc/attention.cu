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
