// tlb_argmax_into: the argmax of tlb_argmax for callers that must not allocate device memory.
//
// Who needs it: a sampling loop that runs where an allocation is unwelcome or impossible - on a
// serving thread that must not take the allocator's locks or risk an out-of-memory failure in the
// middle of a request, in a process whose memory budget was handed out completely at start-up, or in
// a host callback where the CUDA runtime forbids allocation.  tlb_argmax creates its result tensor
// and, on first use, its scratch; this entry point creates nothing: the result goes into a tensor
// the caller already owns, and the per-block partial results live in a fixed array that is part of
// the library image (kScratchSlots entries, 16 KB).
//
// The fixed array bounds the input: kScratchSlots blocks of kChunk elements, 4,194,304 f32 values
// (32 times the 128,256-entry vocabulary of Llama 3).  Longer inputs are refused with TLB_ERR_ARG.
//
// Set-up: the device address of the array is looked up once per device, by the first call made
// with that device current (cudaGetSymbolAddress; this may make the runtime load the module), so
// make the first call outside any stream capture.  Later calls only launch two kernels.
//
// Sharing: every call on a device uses the same array, and a call is TWO launches (per-block
// partial results, then their fold).  Both go to the library's one stream, so calls made one after
// another never overlap on the GPU.  Calls from several host threads are safe as well: a host mutex
// is held from the first launch to the second, so the two kernels of a call are always neighbours on
// the stream and no other call's partial results can land between them.  Work that reaches the array
// from another stream (not possible through this API) would race with both.  Nothing in the array
// has to start at zero: the first kernel overwrites every slot the second kernel reads.
#include "tlb_internal.h"

#include <algorithm>

namespace tlb {

constexpr int kScratchSlots = 1024;       // partial results the fixed array can hold
constexpr int kChunk = 4096;              // input elements reduced by one block
constexpr int64_t kMaxElems = (int64_t)kScratchSlots * kChunk;
constexpr int kMaxDevices = 64;

struct __align__(16) ArgmaxPartial { float value; int pad; long long index; };

// The scratch itself: part of the loaded module, one instance per device, never freed.
static __device__ __align__(256) ArgmaxPartial g_argmax_scratch[kScratchSlots];

// Ordering of candidates: larger value wins; equal values (NaN compares equal, as in the reference)
// go to the smaller index under the first-maximum rule, else to the larger.
__device__ __forceinline__ bool wins(float v, long long i, float bv, long long bi, int tie_first)
{
    if (bi < 0) return true;
    if (v > bv) return true;
    if (v < bv) return false;
    return tie_first ? i < bi : i > bi;
}

// Block b reduces elements [b * kChunk, min(n, (b+1) * kChunk)) into scratch[b].
__global__ void __launch_bounds__(256) argmax_chunk_kernel(const float *__restrict__ x, long long n, int tie_first,
                                                            ArgmaxPartial *__restrict__ scratch)
{
    __shared__ float sv[8];
    __shared__ long long si[8];
    const long long lo = (long long)blockIdx.x * kChunk;
    const long long hi = min(n, lo + kChunk);
    float bv = 0.f;
    long long bi = -1;
    for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        float v = x[i];
        if (wins(v, i, bv, bi, tie_first)) { bv = v; bi = i; }
    }
    for (int o = 16; o; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        long long oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi >= 0 && wins(ov, oi, bv, bi, tie_first)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    if (lane == 0) { sv[w] = bv; si[w] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int j = 1; j < (int)(blockDim.x >> 5); j++)
            if (si[j] >= 0 && wins(sv[j], si[j], bv, bi, tie_first)) { bv = sv[j]; bi = si[j]; }
        ArgmaxPartial r;
        r.value = bv; r.pad = 0; r.index = bi;
        scratch[blockIdx.x] = r;
    }
}

// One warp folds the `parts` partial results and writes the index as f32 (the form tlb_argmax returns).
__global__ void __launch_bounds__(32) argmax_fold_kernel(const ArgmaxPartial *__restrict__ scratch, int parts, int tie_first,
                                                          float *__restrict__ out)
{
    float bv = 0.f;
    long long bi = -1;
    for (int j = threadIdx.x; j < parts; j += 32) {
        ArgmaxPartial r = scratch[j];
        if (r.index >= 0 && wins(r.value, r.index, bv, bi, tie_first)) { bv = r.value; bi = r.index; }
    }
    for (int o = 16; o; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        long long oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi >= 0 && wins(ov, oi, bv, bi, tie_first)) { bv = ov; bi = oi; }
    }
    if (threadIdx.x == 0) out[0] = (float)(bi < 0 ? 0 : bi);
}

// Device address of the fixed array, one entry per device ordinal; filled by the first call on that device.
static std::mutex g_setup_mu;
static std::mutex g_pair_mu;   // held across the two launches of a call: they stay adjacent on the stream
static ArgmaxPartial *g_scratch_ptr[kMaxDevices] = {nullptr};

static tlb_status scratch_for_current_device(int device, ArgmaxPartial **ptr)
{
    std::lock_guard<std::mutex> lk(g_setup_mu);
    if (!g_scratch_ptr[device]) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_argmax_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(argmax scratch)");
        if (!p) return fail(TLB_ERR_INTERNAL, "argmax_into: the fixed scratch array has no device address");
        g_scratch_ptr[device] = (ArgmaxPartial *)p;
    }
    *ptr = g_scratch_ptr[device];
    return TLB_OK;
}

}  // namespace tlb
using namespace tlb;

extern "C" tlb_status tlb_argmax_into(tlb_tensor *out, const tlb_tensor *x, tlb_tie_rule tie)
{
    if (!out || !x) return fail(TLB_ERR_NULL, "argmax_into: null tensor");
    Context *c = ctx();
    if (!c) return fail(TLB_ERR_DEVICE, "argmax_into: library not initialised; call tlb_init first (this entry point never sets up the device itself)");
    if (x->dt != TLB_F32 || out->dt != TLB_F32) return fail(TLB_ERR_TYPE, "argmax_into: f32 tensors expected");
    if (out->numel() < 1) return fail(TLB_ERR_SHAPE, "argmax_into: out must hold at least one element");
    const int64_t n = x->numel();
    if (n <= 0) return fail(TLB_ERR_INTERNAL, "Empty tensor for sampling");
    if (n > kMaxElems)
        return fail(TLB_ERR_ARG, "argmax_into: %lld elements exceed the fixed scratch (at most %lld); use tlb_argmax for larger inputs",
                    (long long)n, (long long)kMaxElems);
    if (c->device < 0 || c->device >= kMaxDevices) return fail(TLB_ERR_DEVICE, "argmax_into: device ordinal %d out of range", c->device);
    int cur = -1;
    TLB_CUDA(cudaGetDevice(&cur));
    if (cur != c->device) TLB_CUDA(cudaSetDevice(c->device));
    ArgmaxPartial *scratch = nullptr;
    TLB_TRY(scratch_for_current_device(c->device, &scratch));
    const int parts = (int)((n + kChunk - 1) / kChunk);
    const int tie_first = tie == TLB_TIE_FIRST;
    std::lock_guard<std::mutex> pair(g_pair_mu);
    argmax_chunk_kernel<<<parts, 256, 0, c->stream>>>(x->f32(), (long long)n, tie_first, scratch);
    TLB_CUDA(cudaGetLastError());
    argmax_fold_kernel<<<1, 32, 0, c->stream>>>(scratch, parts, tie_first, out->f32());
    TLB_CUDA(cudaGetLastError());
    count_launch(2);
    return TLB_OK;
}
