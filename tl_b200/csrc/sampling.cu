// Temperature / top-p sampling on the device, with the random number supplied by the caller.
// Restates CpuTensor::sample_impl (crates/tl_cpu/src/tensor.rs:1625-1680): probabilities = softmax(logits / temp);
// token order = probabilities descending (stable: equal probabilities keep index order); the kept prefix ends at
// the first position where the running sum exceeds top_p (or at the last token); r = u * (that running sum); the
// result is the first token of the prefix whose running sum reaches r.  The reference draws u from
// rand::thread_rng(), so its runs are not repeatable; here u is an argument and the result is a function of it.
// (The reference's CUDA back end ignores temp and top_p and returns the argmax, crates/tl_cuda/src/ffi_ops.rs:880-884:
// that behaviour is tlb_sample.)
//
// Extensions beyond the reference's CPU sampler (its CUDA samplers are all argmax, autograd.cu:2370-2446): a top-k limit on
// the kept prefix (the prefix ends at the top-p cutoff or after k tokens, whichever comes first), and a counter-based
// random number generator (Philox-4x32-10, the published algorithm of Salmon et al., SC'11) so that a decode session can
// draw its numbers on the device: u = the first output word of Philox(key = seed, counter = step) scaled to [0, 1).
//
// Three launches: probabilities (one block: maximum, sum of exponentials, division), a stable descending radix
// sort of (probability, index) pairs (CUB), and a walk over the sorted list by one warp that adds in list order
// as the reference does (lane 0 adds, the warp stages 1024 entries at a time; it stops at the cutoff).
#include <cub/device/device_radix_sort.cuh>

#include "tlb_internal.h"

namespace tlb {

namespace {

constexpr int kProbThreads = 1024;

__global__ void __launch_bounds__(kProbThreads) sample_probs_kernel(const float *__restrict__ logits, int n, float temp,
                                                                    float *__restrict__ probs, int *__restrict__ idx)
{
    __shared__ float red[kProbThreads / 32];
    __shared__ float bcast;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float mx = -INFINITY;
    for (int i = tid; i < n; i += kProbThreads) mx = fmaxf(mx, logits[i] / temp);
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    if (tid == 0) {
        float m = red[0];
        for (int i = 1; i < kProbThreads / 32; i++) m = fmaxf(m, red[i]);
        bcast = m;
    }
    __syncthreads();
    mx = bcast;
    float sum = 0.f;
    for (int i = tid; i < n; i += kProbThreads) sum += expf(logits[i] / temp - mx);
    for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    __syncthreads();
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    if (tid == 0) {
        float s = 0.f;
        for (int i = 0; i < kProbThreads / 32; i++) s += red[i];
        bcast = s;
    }
    __syncthreads();
    sum = bcast;
    for (int i = tid; i < n; i += kProbThreads) {
        probs[i] = expf(logits[i] / temp - mx) / sum;
        idx[i] = i;
    }
}

__host__ __device__ inline void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1, uint32_t (&o)[4])
{
    for (int r = 0; r < 10; r++) {
        const uint64_t p0 = (uint64_t)0xD2511F53u * c0, p1 = (uint64_t)0xCD9E8D57u * c2;
        const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0, n1 = (uint32_t)p1, n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1, n3 = (uint32_t)p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    o[0] = c0; o[1] = c1; o[2] = c2; o[3] = c3;
}
// the 24 high bits of the first output word, as a float in [0, 1)
__host__ __device__ inline float philox_uniform(uint64_t seed, uint64_t counter)
{
    uint32_t o[4];
    philox4x32_10((uint32_t)counter, (uint32_t)(counter >> 32), 0u, 0u, (uint32_t)seed, (uint32_t)(seed >> 32), o);
    return (float)(o[0] >> 8) * (1.0f / 16777216.0f);
}

// Where the walk puts its result besides out[0]: the state of a decode session (token, positions, output ring).
struct SampleSink {
    int *state;                    // [token, pos, rope_pos, out index] or null
    int *tokens_out;
    int tokens_cap;
    unsigned long long *counter;   // draw u = philox(seed, (*counter)++) on the device; null: the caller's u
    unsigned long long seed;
};

// One warp.  Pass 1: running sum in list order until it exceeds top_p or top_k tokens are in -> cutoff position and sum.
// Pass 2: r = u * sum; first position (up to the cutoff) whose running sum reaches r.
__global__ void __launch_bounds__(32) sample_walk_kernel(const float *__restrict__ sorted_p, const int *__restrict__ sorted_i, int n,
                                                         float top_p, int top_k, float u, float *__restrict__ out, const SampleSink sink)
{
    __shared__ float chunk[1024];
    const int lane = threadIdx.x;
    if (sink.counter) {
        const unsigned long long c = *sink.counter;
        u = philox_uniform(sink.seed, c);
        __syncwarp();
        if (lane == 0) *sink.counter = c + 1;
    }
    if (top_k > 0 && top_k < n) n = top_k;      // the list is sorted: the k most probable tokens are its first k entries
    float cum = 0.f;
    int cutoff = n - 1;
    bool done = false;
    for (int base = 0; base < n && !done; base += 1024) {
        const int m = min(1024, n - base);
        for (int i = lane; i < m; i += 32) chunk[i] = sorted_p[base + i];
        __syncwarp();
        if (lane == 0) {
            for (int i = 0; i < m; i++) {
                cum += chunk[i];
                if (cum > top_p) { cutoff = base + i; done = true; break; }
            }
        }
        done = __shfl_sync(0xffffffffu, (int)done, 0);
        __syncwarp();
    }
    cum = __shfl_sync(0xffffffffu, cum, 0);
    cutoff = __shfl_sync(0xffffffffu, cutoff, 0);
    const float r = u * cum;
    float acc = 0.f;
    int pick = 0;
    done = false;
    for (int base = 0; base <= cutoff && !done; base += 1024) {
        const int m = min(1024, cutoff + 1 - base);
        for (int i = lane; i < m; i += 32) chunk[i] = sorted_p[base + i];
        __syncwarp();
        if (lane == 0) {
            for (int i = 0; i < m; i++) {
                acc += chunk[i];
                if (acc >= r) { pick = base + i; done = true; break; }
            }
        }
        done = __shfl_sync(0xffffffffu, (int)done, 0);
        __syncwarp();
    }
    if (lane == 0) {
        const int tok = sorted_i[pick];              // never reached r (rounding): the first token, as the reference
        if (out) out[0] = (float)tok;
        if (sink.state) {
            const int idx = sink.state[3];
            if (sink.tokens_out && idx < sink.tokens_cap) sink.tokens_out[idx] = tok;
            sink.state[0] = tok; sink.state[1] += 1; sink.state[2] += 1; sink.state[3] = idx + 1;
        }
    }
}

}  // namespace

size_t sample_workspace_bytes(int64_t n)
{
    size_t tmp_bytes = 0;
    cub::DeviceRadixSort::SortPairsDescending(nullptr, tmp_bytes, (const float *)nullptr, (float *)nullptr, (const int *)nullptr,
                                              (int *)nullptr, (int)n, 0, 32, (cudaStream_t)0);
    return (size_t)n * 16 + tmp_bytes + 512;
}

// The sampler on a caller-owned work space (sample_workspace_bytes(n) bytes): nothing is allocated, so the launches can sit
// in a captured graph.  With `counter` the random number is drawn on the device from (seed, *counter) and the counter is
// advanced; with `state` the token also goes to a decode session's state.
tlb_status launch_sample_into(const float *logits, int64_t n, float temp, float top_p, int top_k, float u, float *out, void *workspace,
                              int *state, int *tokens_out, int tokens_cap, unsigned long long *counter, unsigned long long seed)
{
    Context *c = ctx();
    if (!c) return TLB_ERR_DEVICE;
    if (n < 1 || n > INT32_MAX) return fail(TLB_ERR_ARG, "sample: %lld logits", (long long)n);
    size_t tmp_bytes = 0;
    cub::DeviceRadixSort::SortPairsDescending(nullptr, tmp_bytes, (const float *)nullptr, (float *)nullptr, (const int *)nullptr,
                                              (int *)nullptr, (int)n, 0, 32, c->stream);
    float *probs = (float *)workspace, *sorted_p = probs + n;
    int *idx = (int *)(sorted_p + n), *sorted_i = idx + n;
    void *tmp = (void *)(((uintptr_t)(sorted_i + n) + 255) & ~(uintptr_t)255);
    sample_probs_kernel<<<1, kProbThreads, 0, c->stream>>>(logits, (int)n, temp, probs, idx);
    cudaError_t e = cub::DeviceRadixSort::SortPairsDescending(tmp, tmp_bytes, probs, sorted_p, idx, sorted_i, (int)n, 0, 32, c->stream);
    if (e == cudaSuccess) {
        const SampleSink sink{state, tokens_out, tokens_cap, counter, seed};
        sample_walk_kernel<<<1, 32, 0, c->stream>>>(sorted_p, sorted_i, (int)n, top_p, top_k, u, out, sink);
        e = cudaGetLastError();
    }
    count_launch(3);
    if (e != cudaSuccess) return cuda_fail(e, "sample launch");
    return TLB_OK;
}

tlb_status launch_sample_top_p(const float *logits, int64_t n, float temp, float top_p, float u, float *out, int top_k)
{
    Context *c = ctx();
    if (!c) return TLB_ERR_DEVICE;
    if (n < 1 || n > INT32_MAX) return fail(TLB_ERR_ARG, "sample: %lld logits", (long long)n);
    Storage *buf = storage_alloc(sample_workspace_bytes(n));
    if (!buf) return TLB_ERR_ALLOC;
    tlb_status st = launch_sample_into(logits, n, temp, top_p, top_k, u, out, buf->ptr, nullptr, nullptr, 0, nullptr, 0);
    storage_release(buf);
    return st;
}


}  // namespace tlb

using namespace tlb;

// u in [0, 1) of the session generator for (seed, counter): what a session draws on the device at that step, on the host.
extern "C" double tlb_rng_uniform(uint64_t seed, uint64_t counter) { return (double)philox_uniform(seed, counter); }

// tlb_sample_top_p with a top-k limit as well (top_k <= 0: none).
extern "C" tlb_status tlb_sample_top_k_top_p(tlb_tensor **out, const tlb_tensor *logits, float temp, int32_t top_k, float top_p, double u, tlb_tie_rule tie)
{
    if (!out) return fail(TLB_ERR_NULL, "null out");
    *out = nullptr;
    if (!logits) return fail(TLB_ERR_NULL, "sample: null tensor");
    if (logits->dt != TLB_F32) return fail(TLB_ERR_TYPE, "sample: f32 tensor expected");
    if (logits->numel() < 1) return fail(TLB_ERR_INTERNAL, "Empty tensor for sampling");
    if (temp <= 0.f || top_k == 1) return tlb_argmax(out, logits, tie);
    if (!(u >= 0.0 && u < 1.0)) return fail(TLB_ERR_ARG, "sample: the random number must lie in [0, 1)");
    int64_t one = 1;
    TLB_TRY(new_tensor(out, TLB_F32, &one, 1));
    tlb_status st = launch_sample_top_p(logits->f32(), logits->numel(), temp, top_p, (float)u, (*out)->f32(), top_k);
    if (st != TLB_OK) { tlb_tensor_release(*out); *out = nullptr; }
    return st;
}

extern "C" tlb_status tlb_sample_top_p(tlb_tensor **out, const tlb_tensor *logits, float temp, float top_p, double u, tlb_tie_rule tie)
{
    if (!out) return fail(TLB_ERR_NULL, "null out");
    *out = nullptr;
    if (!logits) return fail(TLB_ERR_NULL, "sample: null tensor");
    if (logits->dt != TLB_F32) return fail(TLB_ERR_TYPE, "sample: f32 tensor expected");
    if (logits->numel() < 1) return fail(TLB_ERR_INTERNAL, "Empty tensor for sampling");
    if (temp <= 0.f) return tlb_argmax(out, logits, tie);   // greedy, as the reference
    if (!(u >= 0.0 && u < 1.0)) return fail(TLB_ERR_ARG, "sample: the random number must lie in [0, 1)");
    int64_t one = 1;
    TLB_TRY(new_tensor(out, TLB_F32, &one, 1));
    tlb_status st = launch_sample_top_p(logits->f32(), logits->numel(), temp, top_p, (float)u, (*out)->f32(), 0);
    if (st != TLB_OK) { tlb_tensor_release(*out); *out = nullptr; }
    return st;
}
