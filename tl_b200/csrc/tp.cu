// Tensor-parallel plumbing: one process per GPU, a communicator over the ranks of one node, and the sum of
// the row-parallel partial results (attn_output, ffn_down) across them.
//
// The reference has no multi-GPU path (crates/tl_cuda/src/device.rs:21-27 binds device 0; the collectives of
// crates/tl_cuda/src/ffi_ops.rs:726-730 are stubs), so there is nothing to mirror: this is the Megatron-style
// column / row split with one all-reduce after o_proj and one after ffn_down, and an all-gather of per-shard
// (maximum, index) pairs for the vocabulary-split output head.
//
// Two transports, same result on every rank:
//   * NCCL (ncclAllReduce / ncclAllGather on the library's stream, capturable in the decode graph).  The
//     library is found at run time (dlopen of libnccl.so.2), so libtlb200 itself does not link against it.
//   * a one-shot all-reduce over peer memory for the small, latency-bound vectors of decoding (32 KB for a
//     70B-shaped model): every rank STORES its partial into a staging slot it owns in every peer's memory
//     (NVLink through NVSwitch), raises a sequence flag on the peer, waits (bounded) for the flags of all
//     peers in its own memory, and adds the slots in rank order - all loads are local, the sum is bitwise
//     the same on every rank, and one launch replaces the multi-step NCCL kernel.  Peer mappings come from
//     CUDA IPC handles the host exchanges (tlb_tp_p2p_export / tlb_tp_p2p_attach).
// Every wait is bounded: joining (a non-blocking communicator polled against a deadline, then ncclCommAbort; the
// communicator the collectives use is created only once every rank is known to be there), and the flag wait in the kernel (~1 s, then the context's error word; the host sees
// TLB_ERR_DEVICE at the next synchronisation).
#include "tlb_internal.h"

#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <thread>

namespace tlb {

namespace {

struct NcclApi {
    void *handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRankConfig)(ncclComm_t *, int, ncclUniqueId, int, ncclConfig_t *) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t *) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Broadcast)(const void *, void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
};

std::mutex g_tp_mu;
NcclApi g_nccl;

constexpr int kMaxTp = 8;
constexpr size_t kP2pMaxFloats = 64 * 1024;   // per rank and buffer: 16 activation rows of a 70B-shaped model (8192 wide), with room

constexpr int kP2pMaxWords = 16 * 1024;       // longest vector (d_model) the matvec launches add over the ranks themselves
constexpr int kP2pCtas = 16;                  // most CTAs of one all-reduce; every CTA has flags of its own

struct P2pRegion {                 // what a rank allocates for its peers to write into (cudaMalloc, exported over IPC)
    float slots[2][kMaxTp][kP2pMaxFloats];   // [buffer][writer rank][element]
    unsigned flags[kMaxTp][kP2pCtas][8];     // flags[r][c][0]: sequence number of the last all-reduce whose CTA c of rank r wrote here (32-byte apart)
    unsigned long long words[2][kMaxTp][kP2pMaxWords];   // in-launch exchange: [buffer][writer rank][row] = {value, sequence number}
};

struct TpState {
    int rank = 0, size = 1;
    ncclComm_t comm = nullptr;
    // peer-memory all-reduce
    P2pRegion *mine = nullptr;
    P2pRegion *peer[kMaxTp] = {nullptr};
    bool p2p = false;
    bool fuse = true;               // with p2p: decode sessions exchange partial sums inside their matvec launches
    unsigned *seq = nullptr;        // device: sequence number of the next all-reduce (advanced by the kernel)
    int *arrive = nullptr;          // device: CTAs of the running all-reduce that have stored their share
    double join_timeout_s = 60.0;
} g_tp;

tlb_status nccl_fail(ncclResult_t r, const char *what)
{
    return fail(TLB_ERR_DEVICE, "NCCL error %d (%s) in %s", (int)r, g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "?", what);
}

tlb_status load_nccl()
{
    if (g_nccl.handle) return TLB_OK;
    const char *path = getenv("TLB_NCCL_LIB");   // another libnccl, or a stand-in that fails on purpose (host-side failure tests)
    void *h = dlopen(path && *path ? path : "libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h && !(path && *path)) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return fail(TLB_ERR_DEVICE, "cannot load the NCCL library (%s)", dlerror());
    NcclApi a;
    a.handle = h;
#define SYM(field, name) *(void **)(&a.field) = dlsym(h, name); if (!a.field) return fail(TLB_ERR_DEVICE, "NCCL library lacks %s", name)
    SYM(GetUniqueId, "ncclGetUniqueId");
    SYM(CommInitRankConfig, "ncclCommInitRankConfig");
    SYM(CommGetAsyncError, "ncclCommGetAsyncError");
    SYM(CommAbort, "ncclCommAbort");
    SYM(CommDestroy, "ncclCommDestroy");
    SYM(AllReduce, "ncclAllReduce");
    SYM(AllGather, "ncclAllGather");
    SYM(Broadcast, "ncclBroadcast");
    SYM(GetErrorString, "ncclGetErrorString");
#undef SYM
    g_nccl = a;
    return TLB_OK;
}

// Polls a non-blocking NCCL call to its end; past the deadline the communicator is aborted.
tlb_status wait_comm(ncclComm_t comm, double timeout_s, const char *what)
{
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        ncclResult_t st = ncclSuccess;
        ncclResult_t r = g_nccl.CommGetAsyncError(comm, &st);
        if (r != ncclSuccess) return nccl_fail(r, "ncclCommGetAsyncError");
        if (st == ncclSuccess) return TLB_OK;
        if (st != ncclInProgress) return nccl_fail(st, what);
        if (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > timeout_s) {
            g_nccl.CommAbort(comm);
            return fail(TLB_ERR_DEVICE, "%s: the other ranks did not answer within %.1f s; communicator aborted", what, timeout_s);
        }
        std::this_thread::sleep_for(std::chrono::milliseconds(2));
    }
}

// A call on a non-blocking communicator may answer "in progress" while NCCL still sets up connections; it is on the
// stream once the communicator reports success again.
tlb_status finish_call(ncclComm_t comm, ncclResult_t r, const char *what)
{
    if (r == ncclSuccess) return TLB_OK;
    if (r != ncclInProgress) return nccl_fail(r, what);
    return wait_comm(comm, g_tp.join_timeout_s, what);
}

// ---- one-shot all-reduce over peer memory ---------------------------------------------------------------------

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p)
{
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned *p, unsigned v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

struct P2pArgs {
    P2pRegion *peer[kMaxTp];
    P2pRegion *mine;
    unsigned *seq;
    int *arrive;
    int *err;
    int rank, size;
};

// x[0 .. n) := sum over ranks of their x, n a multiple of 4.  CTA c owns a contiguous range of float4s and never
// talks to the other CTAs of its grid: (1) it stores its range into slot [buf][rank] of every rank (own memory
// included); (2) behind a block barrier and a system-scope fence, one thread raises flags[rank][c] = seq on every rank;
// (3) it waits (bounded) until flags[r][c] of all ranks r in OWN memory have reached seq - CTA c of every rank covers
// the same range; (4) it adds the slots in rank order.  Buffers alternate with seq: a rank can be at most one
// all-reduce ahead of a peer that is still reading.
__global__ void __launch_bounds__(256) p2p_allreduce_kernel(float *x, int n, const P2pArgs a)
{
    __shared__ int s_ok;
    // launched as a programmatic dependent: x (and seq) are valid once the launch before has completed
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const unsigned seq = *a.seq;
    const int buf = seq & 1;
    const int n4 = n >> 2, per = (n4 + gridDim.x - 1) / gridDim.x;
    const int i0 = blockIdx.x * per, i1 = min(n4, i0 + per);
    const float4 *x4 = reinterpret_cast<const float4 *>(x);
    for (int i = i0 + threadIdx.x; i < i1; i += blockDim.x) {
        const float4 v = x4[i];
        for (int p = 0; p < a.size; p++) reinterpret_cast<float4 *>(a.peer[p]->slots[buf][a.rank])[i] = v;
    }
    __syncthreads();
    if (threadIdx.x < a.size) {
        __threadfence_system();                       // the CTA's stores are visible to every GPU before its flag is
        st_release_sys(&a.peer[threadIdx.x]->flags[a.rank][blockIdx.x][0], seq);
    }
    if (threadIdx.x < 32) {
        // lane r waits for rank r's CTA of the same index: bounded (about a second), then the error word
        bool ok = true;
        if (threadIdx.x < a.size) {
            unsigned long long t0 = 0;
            for (unsigned it = 0;; it++) {
                if ((int)(ld_acquire_sys(&a.mine->flags[threadIdx.x][blockIdx.x][0]) - seq) >= 0) break;
                if ((it & 255) == 255) {
                    unsigned long long t;
                    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
                    if (!t0) t0 = t;
                    if (t - t0 > 1000000000ull) { atomicExch(a.err, 31); ok = false; break; }
                }
            }
        }
        ok = __all_sync(0xffffffffu, ok);
        if (threadIdx.x == 0) s_ok = ok;
    }
    __syncthreads();
    if (s_ok) {
        float4 *o4 = reinterpret_cast<float4 *>(x);
        for (int i = i0 + threadIdx.x; i < i1; i += blockDim.x) {
            float4 acc = __ldcv(reinterpret_cast<const float4 *>(a.mine->slots[buf][0]) + i);
            for (int p = 1; p < a.size; p++) {
                const float4 v = __ldcv(reinterpret_cast<const float4 *>(a.mine->slots[buf][p]) + i);
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
            o4[i] = acc;
        }
    }
    // the next all-reduce uses the next sequence number: the last CTA to get here (all have read seq by then) advances it
    if (threadIdx.x == 0) {
        if (atomicAdd(a.arrive, 1) == (int)gridDim.x - 1) { *a.arrive = 0; *a.seq = seq + 1; }
    }
}

}  // namespace

bool tp_allreduce_is_kernel(int64_t n)
{
    return g_tp.size > 1 && g_tp.p2p && n % 4 == 0 && (size_t)n <= kP2pMaxFloats;
}

bool tp_fuse_args(TpFuse *out)
{
    static_assert(kTpMaxRanks == kMaxTp, "rank limits differ");
    if (!g_tp.p2p || !g_tp.fuse || g_tp.size <= 1) return false;
    for (int p = 0; p < kMaxTp; p++) out->peer_ll[p] = p < g_tp.size ? &g_tp.peer[p]->words[0][g_tp.rank][0] : nullptr;
    out->mine_ll = &g_tp.mine->words[0][0][0];
    out->seq = g_tp.seq;
    out->done = g_tp.arrive + 1;
    out->size = g_tp.size;
    out->buf_stride = kMaxTp * kP2pMaxWords;
    out->rank_stride = kP2pMaxWords;
    return true;
}

int tp_rank() { return g_tp.rank; }
int tp_size() { return g_tp.size; }

tlb_status tp_allreduce(float *x, int64_t n)
{
    Context *c = ctx();
    if (!c) return fail(TLB_ERR_DEVICE, "no device");
    if (g_tp.size <= 1) return TLB_OK;
    if (g_tp.p2p && n % 4 == 0 && (size_t)n <= kP2pMaxFloats && ((uintptr_t)x & 15) == 0) {
        P2pArgs a;
        for (int p = 0; p < kMaxTp; p++) a.peer[p] = g_tp.peer[p];
        a.mine = g_tp.mine; a.seq = g_tp.seq; a.arrive = g_tp.arrive; a.err = c->err_flag; a.rank = g_tp.rank; a.size = g_tp.size;
        const int grid = (int)std::max<int64_t>(1, std::min<int64_t>(kP2pCtas, (n / 4 + 511) / 512));
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(256);
        cfg.stream = c->stream;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at;
        cfg.numAttrs = 1;
        TLB_CUDA(cudaLaunchKernelEx(&cfg, p2p_allreduce_kernel, x, (int)n, a));
        count_launch();
        return TLB_OK;
    }
    if (!g_tp.comm) return fail(TLB_ERR_ARG, "tensor-parallel all-reduce before tlb_tp_init");
    ncclResult_t r = g_nccl.AllReduce(x, x, (size_t)n, ncclFloat32, ncclSum, g_tp.comm, c->stream);
    return finish_call(g_tp.comm, r, "ncclAllReduce");
}

tlb_status tp_allgather(const void *send, void *recv, size_t bytes_per_rank)
{
    Context *c = ctx();
    if (!c) return fail(TLB_ERR_DEVICE, "no device");
    if (g_tp.size <= 1) {
        if (send != recv) TLB_CUDA(cudaMemcpyAsync(recv, send, bytes_per_rank, cudaMemcpyDeviceToDevice, c->stream));
        return TLB_OK;
    }
    if (!g_tp.comm) return fail(TLB_ERR_ARG, "tensor-parallel all-gather before tlb_tp_init");
    ncclResult_t r = g_nccl.AllGather(send, recv, bytes_per_rank, ncclInt8, g_tp.comm, c->stream);
    return finish_call(g_tp.comm, r, "ncclAllGather");
}

}  // namespace tlb

using namespace tlb;

extern "C" {

tlb_status tlb_tp_unique_id(void *id_out, size_t id_bytes)
{
    if (!id_out) return fail(TLB_ERR_NULL, "null id buffer");
    if (id_bytes < NCCL_UNIQUE_ID_BYTES) return fail(TLB_ERR_ARG, "the id buffer must hold %d bytes", NCCL_UNIQUE_ID_BYTES);
    std::lock_guard<std::mutex> lk(g_tp_mu);
    TLB_TRY(load_nccl());
    ncclUniqueId id;
    ncclResult_t r = g_nccl.GetUniqueId(&id);
    if (r != ncclSuccess) return nccl_fail(r, "ncclGetUniqueId");
    memcpy(id_out, &id, NCCL_UNIQUE_ID_BYTES);
    return TLB_OK;
}

tlb_status tlb_tp_init(const void *id, size_t id_bytes, int rank, int size, double join_timeout_s)
{
    if (!id) return fail(TLB_ERR_NULL, "null id");
    if (id_bytes < NCCL_UNIQUE_ID_BYTES) return fail(TLB_ERR_ARG, "the id must hold %d bytes", NCCL_UNIQUE_ID_BYTES);
    if (size < 1 || size > kMaxTp || rank < 0 || rank >= size) return fail(TLB_ERR_ARG, "tensor-parallel rank %d of %d (1..%d ranks)", rank, size, kMaxTp);
    std::lock_guard<std::mutex> lk(g_tp_mu);
    if (g_tp.comm) return fail(TLB_ERR_ARG, "tlb_tp_init was already called in this process");
    TLB_TRY(load_nccl());
    // the join itself needs no device of ours (the host-side failure test runs it against a stand-in library without one);
    // with the real NCCL the device bound by tlb_init is made current first
    if (ensure_init()) TLB_CUDA(cudaSetDevice(ctx()->device));
    ncclUniqueId uid;
    memcpy(&uid, id, NCCL_UNIQUE_ID_BYTES);
    const double timeout = join_timeout_s > 0 ? join_timeout_s : 60.0;
    g_tp.join_timeout_s = timeout;
    // Step 1, the bounded join: a NON-BLOCKING communicator returns at once and is polled against the deadline; a rank
    // that never arrives ends it with ncclCommAbort and TLB_ERR_DEVICE.
    ncclConfig_t nb = NCCL_CONFIG_INITIALIZER;
    nb.blocking = 0;
    ncclComm_t probe = nullptr;
    ncclResult_t r = g_nccl.CommInitRankConfig(&probe, size, uid, rank, &nb);
    if (r != ncclSuccess && r != ncclInProgress) return nccl_fail(r, "ncclCommInitRankConfig");
    if (!probe) return fail(TLB_ERR_DEVICE, "ncclCommInitRankConfig returned no communicator");
    TLB_TRY(wait_comm(probe, timeout, "joining the tensor-parallel communicator"));
    if (!ctx()) { g_nccl.CommAbort(probe); return fail(TLB_ERR_DEVICE, "tensor parallelism needs a CUDA device (tlb_init)"); }
    // Step 2: everyone is here.  The collectives of the decode path run on an ordinary BLOCKING communicator (calls
    // return once they are on the stream, which is what stream capture into the decode graph wants); its id travels
    // from rank 0 over the first communicator, which is then closed.
    cudaStream_t s = ctx()->stream;
    ncclUniqueId uid2;
    memset(&uid2, 0, sizeof uid2);
    if (rank == 0) {
        r = g_nccl.GetUniqueId(&uid2);
        if (r != ncclSuccess) { g_nccl.CommAbort(probe); return nccl_fail(r, "ncclGetUniqueId"); }
    }
    char *idbuf = nullptr;
    tlb_status st = TLB_OK;
    cudaError_t e = cudaMalloc((void **)&idbuf, NCCL_UNIQUE_ID_BYTES);
    if (e == cudaSuccess) e = cudaMemcpyAsync(idbuf, &uid2, NCCL_UNIQUE_ID_BYTES, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) st = finish_call(probe, g_nccl.Broadcast(idbuf, idbuf, NCCL_UNIQUE_ID_BYTES, ncclInt8, 0, probe, s), "ncclBroadcast of the second id");
    if (e == cudaSuccess && st == TLB_OK) e = cudaMemcpyAsync(&uid2, idbuf, NCCL_UNIQUE_ID_BYTES, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess && st == TLB_OK) e = cudaStreamSynchronize(s);
    if (idbuf) cudaFree(idbuf);
    if (e != cudaSuccess || st != TLB_OK) { g_nccl.CommAbort(probe); return st != TLB_OK ? st : cuda_fail(e, "exchange of the second communicator id"); }
    g_nccl.CommDestroy(probe);
    ncclConfig_t bl = NCCL_CONFIG_INITIALIZER;
    bl.blocking = 1;
    ncclComm_t comm = nullptr;
    r = g_nccl.CommInitRankConfig(&comm, size, uid2, rank, &bl);
    if (r != ncclSuccess) return nccl_fail(r, "ncclCommInitRankConfig (blocking)");
    g_tp.comm = comm;
    g_tp.rank = rank;
    g_tp.size = size;
    if (size > 1) {
        // one small all-reduce and all-gather now: NCCL builds its connections on first use, which must not happen inside a
        // graph capture
        float *w = nullptr;
        TLB_CUDA(cudaMalloc(&w, 1024 * sizeof(float)));
        TLB_CUDA(cudaMemsetAsync(w, 0, 1024 * sizeof(float), s));
        st = finish_call(comm, g_nccl.AllReduce(w, w, 1024, ncclFloat32, ncclSum, comm, s), "first ncclAllReduce");
        if (st == TLB_OK) st = finish_call(comm, g_nccl.AllGather(w, w, 8, ncclInt8, comm, s), "first ncclAllGather");
        e = cudaStreamSynchronize(s);
        cudaFree(w);
        if (st != TLB_OK) return st;
        if (e != cudaSuccess) return cuda_fail(e, "first collective");
    }
    return TLB_OK;
}

tlb_status tlb_tp_poll(void)
{
    std::lock_guard<std::mutex> lk(g_tp_mu);
    if (!g_tp.comm) return TLB_OK;
    ncclResult_t st = ncclSuccess;
    ncclResult_t r = g_nccl.CommGetAsyncError(g_tp.comm, &st);
    if (r != ncclSuccess) return nccl_fail(r, "ncclCommGetAsyncError");
    if (st != ncclSuccess && st != ncclInProgress) return nccl_fail(st, "an earlier collective");
    return TLB_OK;
}

int tlb_tp_rank(void) { return g_tp.rank; }
int tlb_tp_size(void) { return g_tp.size; }

tlb_status tlb_tp_shutdown(void)
{
    // ncclCommDestroy waits for every CUDA graph that captured one of the communicator's collectives to be destroyed:
    // the decode sessions of this process hold such graphs
    if (tp_live_sessions() > 0)
        return fail(TLB_ERR_ARG, "%d tensor-parallel decode session(s) are still alive: destroy them before tlb_tp_shutdown", tp_live_sessions());
    std::lock_guard<std::mutex> lk(g_tp_mu);
    if (ctx()) cudaStreamSynchronize(ctx()->stream);
    for (int p = 0; p < kMaxTp; p++) {
        if (g_tp.peer[p] && g_tp.peer[p] != g_tp.mine) cudaIpcCloseMemHandle(g_tp.peer[p]);
        g_tp.peer[p] = nullptr;
    }
    if (g_tp.mine) cudaFree(g_tp.mine);
    if (g_tp.seq) cudaFree(g_tp.seq);
    if (g_tp.arrive) cudaFree(g_tp.arrive);
    g_tp.mine = nullptr; g_tp.seq = nullptr; g_tp.arrive = nullptr; g_tp.p2p = false;
    if (g_tp.comm) g_nccl.CommDestroy(g_tp.comm);
    g_tp.comm = nullptr;
    g_tp.rank = 0;
    g_tp.size = 1;
    return TLB_OK;
}

tlb_status tlb_allreduce(tlb_tensor *t)
{
    if (!t) return fail(TLB_ERR_NULL, "null tensor");
    if (t->dt != TLB_F32) return fail(TLB_ERR_TYPE, "all-reduce takes f32 tensors");
    return tp_allreduce(t->f32(), t->numel());
}

// Peer-memory transport, step 1: allocate this rank's region and hand out its CUDA IPC handle (64 bytes) for the
// host to pass to the other ranks of the node.
tlb_status tlb_tp_p2p_export(void *handle_out, size_t handle_bytes)
{
    if (!handle_out) return fail(TLB_ERR_NULL, "null handle buffer");
    if (handle_bytes < sizeof(cudaIpcMemHandle_t)) return fail(TLB_ERR_ARG, "the handle buffer must hold %zu bytes", sizeof(cudaIpcMemHandle_t));
    if (!ensure_init()) return TLB_ERR_DEVICE;
    std::lock_guard<std::mutex> lk(g_tp_mu);
    if (!g_tp.mine) {
        TLB_CUDA(cudaMalloc((void **)&g_tp.mine, sizeof(P2pRegion)));
        TLB_CUDA(cudaMemset(g_tp.mine, 0, sizeof(P2pRegion)));
        TLB_CUDA(cudaMalloc((void **)&g_tp.seq, sizeof(unsigned)));
        TLB_CUDA(cudaMalloc((void **)&g_tp.arrive, 4 * sizeof(int)));   // [0] all-reduce kernel, [1] tiles finished by an in-launch exchange
        const unsigned one = 1;       // flags start at 0: the first all-reduce waits for 1
        TLB_CUDA(cudaMemcpy(g_tp.seq, &one, sizeof one, cudaMemcpyHostToDevice));
        TLB_CUDA(cudaMemset(g_tp.arrive, 0, 4 * sizeof(int)));
        TLB_CUDA(cudaDeviceSynchronize());
    }
    cudaIpcMemHandle_t h;
    TLB_CUDA(cudaIpcGetMemHandle(&h, g_tp.mine));
    memcpy(handle_out, &h, sizeof h);
    return TLB_OK;
}

// Step 2: the handles of all ranks, in rank order (this rank's own entry is ignored).  After this call all-reduces
// of up to 65536 floats go over peer memory; larger ones keep using NCCL.  Every rank must have exported before any
// rank attaches, and all ranks must attach before the first all-reduce (the host's exchange orders both).
tlb_status tlb_tp_p2p_attach(const void *handles, int n_handles)
{
    if (!handles) return fail(TLB_ERR_NULL, "null handles");
    std::lock_guard<std::mutex> lk(g_tp_mu);
    if (n_handles != g_tp.size) return fail(TLB_ERR_ARG, "%d handles for %d ranks", n_handles, g_tp.size);
    if (!g_tp.mine) return fail(TLB_ERR_ARG, "tlb_tp_p2p_export must run first");
    if (g_tp.peer[g_tp.rank]) return fail(TLB_ERR_ARG, "the peers are already attached (tlb_tp_p2p_enable switches the transport back on)");
    for (int p = 0; p < g_tp.size; p++) {
        if (p == g_tp.rank) { g_tp.peer[p] = g_tp.mine; continue; }
        cudaIpcMemHandle_t h;
        memcpy(&h, (const char *)handles + (size_t)p * sizeof h, sizeof h);
        void *ptr = nullptr;
        TLB_CUDA(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
        g_tp.peer[p] = (P2pRegion *)ptr;
    }
    g_tp.p2p = true;
    return TLB_OK;
}

tlb_status tlb_tp_p2p_disable(void)
{
    std::lock_guard<std::mutex> lk(g_tp_mu);
    g_tp.p2p = false;
    return TLB_OK;
}

tlb_status tlb_tp_exchange_in_launch(int on)
{
    std::lock_guard<std::mutex> lk(g_tp_mu);
    g_tp.fuse = on != 0;
    return TLB_OK;
}

tlb_status tlb_tp_p2p_enable(void)
{
    std::lock_guard<std::mutex> lk(g_tp_mu);
    if (!g_tp.mine || !g_tp.peer[g_tp.rank]) return fail(TLB_ERR_ARG, "the peer-memory transport was never attached");
    g_tp.p2p = true;
    return TLB_OK;
}

}  // extern "C"
