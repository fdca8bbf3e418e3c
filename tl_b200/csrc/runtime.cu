// Runtime of libtlb200: device context, thread-local errors, reference-counted tensors on a
// stream-ordered memory pool, CUDA-event timing, stream capture and graphs.
#include "tlb_internal.h"

#include <cstdlib>

namespace tlb {

static thread_local std::string g_err;
static Context g_ctx;
static std::mutex g_init_mu;
static bool g_inited = false;

tlb_status fail(tlb_status code, const char *fmt, ...)
{
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_err = buf;
    return code;
}

tlb_status cuda_fail(cudaError_t e, const char *what)
{
    return fail(e == cudaErrorMemoryAllocation ? TLB_ERR_ALLOC : TLB_ERR_DEVICE, "CUDA error %d (%s) in %s",
                (int)e, cudaGetErrorString(e), what);
}

static tlb_status do_init(int device)
{
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        cudaGetLastError();
        return fail(TLB_ERR_DEVICE, "no CUDA device available (%s); libtlb200 has no CPU fallback",
                    e == cudaSuccess ? "device count 0" : cudaGetErrorString(e));
    }
    if (device < 0) {
        const char *lr = getenv("LOCAL_RANK");
        device = lr ? atoi(lr) % count : 0;
    }
    if (device >= count) return fail(TLB_ERR_ARG, "device %d out of range (%d devices)", device, count);
    TLB_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    TLB_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major < 10)
        return fail(TLB_ERR_DEVICE, "device %d is sm_%d%d; libtlb200 is built for sm_100a only", device, prop.major, prop.minor);
    g_ctx.device = device;
    g_ctx.sm_count = prop.multiProcessorCount;
    g_ctx.smem_optin = prop.sharedMemPerBlockOptin;
    TLB_CUDA(cudaStreamCreateWithFlags(&g_ctx.stream, cudaStreamNonBlocking));
    TLB_CUDA(cudaDeviceGetDefaultMemPool(&g_ctx.pool, device));
    uint64_t thresh = UINT64_MAX;  // keep freed blocks cached in the pool
    TLB_CUDA(cudaMemPoolSetAttribute(g_ctx.pool, cudaMemPoolAttrReleaseThreshold, &thresh));
    TLB_CUDA(cudaMalloc(&g_ctx.err_flag, sizeof(int)));
    TLB_CUDA(cudaMemset(g_ctx.err_flag, 0, sizeof(int)));
    g_ctx.mv_part_floats = (size_t)12 << 20;   // 48 MB: 16 slices of a 128k-row head with 3 activation rows
    TLB_CUDA(cudaMalloc(&g_ctx.mv_part, g_ctx.mv_part_floats * sizeof(float)));
    g_ctx.mv_part1_floats = (size_t)4 << 20;  // 16 MB: 16 slices of a 128k-row head with one activation row, twice over
    TLB_CUDA(cudaMalloc(&g_ctx.mv_part1, g_ctx.mv_part1_floats * sizeof(float)));
    TLB_CUDA(cudaMemset(g_ctx.mv_part1, 0xFF, g_ctx.mv_part1_floats * sizeof(float)));
    g_ctx.mv_cnt_n = (size_t)1 << 20;
    TLB_CUDA(cudaMalloc(&g_ctx.mv_cnt, g_ctx.mv_cnt_n * sizeof(int)));
    TLB_CUDA(cudaMemset(g_ctx.mv_cnt, 0, g_ctx.mv_cnt_n * sizeof(int)));
    g_inited = true;
    return TLB_OK;
}

bool ensure_init()
{
    std::lock_guard<std::mutex> lk(g_init_mu);
    if (g_inited) return true;
    return do_init(-1) == TLB_OK;
}

Context *ctx() { return g_inited ? &g_ctx : nullptr; }

size_t dtype_size(tlb_dtype dt)
{
    switch (dt) {
    case TLB_F32: case TLB_I32: case TLB_U32: return 4;
    case TLB_F64: case TLB_I64: return 8;
    case TLB_F16: case TLB_BF16: return 2;
    case TLB_U8: return 1;
    }
    return 0;
}

Storage *storage_alloc(size_t bytes)
{
    if (!ensure_init()) return nullptr;
    Storage *s = new Storage();
    s->bytes = bytes;
    size_t req = bytes ? (bytes + 255) / 256 * 256 : 256;
    cudaError_t e = cudaMallocAsync(&s->ptr, req, g_ctx.stream);
    if (e != cudaSuccess) {
        cuda_fail(e, "cudaMallocAsync");
        delete s;
        return nullptr;
    }
    g_ctx.bytes_in_use += (int64_t)req;
    return s;
}

void storage_release(Storage *s)
{
    if (!s) return;
    if (s->rc.fetch_sub(1) == 1) {
        if (s->ptr) {
            cudaFreeAsync(s->ptr, g_ctx.stream);
            g_ctx.bytes_in_use -= (int64_t)(s->bytes ? (s->bytes + 255) / 256 * 256 : 256);
        }
        delete s;
    }
}

tlb_status new_tensor(tlb_tensor **out, tlb_dtype dt, const int64_t *shape, int rank)
{
    *out = nullptr;
    if (rank < 0 || rank > kMaxRank) return fail(TLB_ERR_SHAPE, "rank %d not supported (max %d)", rank, kMaxRank);
    int64_t n = 1;
    for (int i = 0; i < rank; i++) {
        if (shape[i] < 0) return fail(TLB_ERR_SHAPE, "negative dimension %lld", (long long)shape[i]);
        n *= shape[i];
    }
    Storage *st = storage_alloc((size_t)n * dtype_size(dt));
    if (!st) return TLB_ERR_ALLOC;
    tlb_tensor *t = new tlb_tensor();
    t->st = st;
    t->dt = dt;
    t->rank = rank;
    for (int i = 0; i < rank; i++) t->shape[i] = shape[i];
    *out = t;
    return TLB_OK;
}

tlb_status new_view(tlb_tensor **out, const tlb_tensor *src, const int64_t *shape, int rank, size_t extra_off)
{
    *out = nullptr;
    if (rank < 0 || rank > kMaxRank) return fail(TLB_ERR_SHAPE, "rank %d not supported", rank);
    tlb_tensor *t = new tlb_tensor();
    t->st = src->st;
    src->st->rc.fetch_add(1);
    t->offset = src->offset + extra_off;
    t->dt = src->dt;
    t->rank = rank;
    for (int i = 0; i < rank; i++) t->shape[i] = shape[i];
    *out = t;
    return TLB_OK;
}

}  // namespace tlb

using namespace tlb;

extern "C" {

tlb_status tlb_init(int device)
{
    std::lock_guard<std::mutex> lk(g_init_mu);
    if (g_inited) {
        if (device >= 0 && device != g_ctx.device)
            return fail(TLB_ERR_ARG, "already bound to device %d", g_ctx.device);
        return TLB_OK;
    }
    return do_init(device);
}

tlb_status tlb_shutdown(void)
{
    std::lock_guard<std::mutex> lk(g_init_mu);
    if (!g_inited) return TLB_OK;
    cudaStreamSynchronize(g_ctx.stream);
    if (g_ctx.flush_buf) cudaFree(g_ctx.flush_buf);
    g_ctx.flush_buf = nullptr;
    return TLB_OK;  // stream and pool stay alive: handles may still be released after this
}

const char *tlb_last_error(void) { return g_err.c_str(); }

int tlb_device_id(void) { return g_inited ? g_ctx.device : -1; }

tlb_status tlb_sync(void)
{
    if (!ensure_init()) return TLB_ERR_DEVICE;
    // a synchronisation would invalidate a capture in progress: refuse before CUDA sees it
    if (g_ctx.capturing) return fail(TLB_ERR_ARG, "this call synchronises with the device, which a stream capture in progress does not allow");
    TLB_CUDA(cudaStreamSynchronize(g_ctx.stream));
    int flag = 0;
    TLB_CUDA(cudaMemcpy(&flag, g_ctx.err_flag, sizeof(int), cudaMemcpyDeviceToHost));
    if (flag) {
        cudaMemset(g_ctx.err_flag, 0, sizeof(int));
        cudaMemset(g_ctx.mv_cnt, 0, g_ctx.mv_cnt_n * sizeof(int));   // an abandoned launch may have left counts behind
        cudaMemset(g_ctx.mv_part1, 0xFF, g_ctx.mv_part1_floats * sizeof(float));   // ... or slices nobody collected
        return fail(TLB_ERR_DEVICE, "a kernel gave up a bounded wait (code %d)", flag);
    }
    return TLB_OK;
}

uint64_t tlb_kernel_launches(void) { return g_inited ? g_ctx.launches.load() : 0; }

tlb_status tlb_mem_stats(uint64_t *bytes_in_use, uint64_t *bytes_reserved)
{
    if (!ensure_init()) return TLB_ERR_DEVICE;
    if (bytes_in_use) *bytes_in_use = (uint64_t)g_ctx.bytes_in_use.load();
    if (bytes_reserved) {
        uint64_t r = 0;
        TLB_CUDA(cudaMemPoolGetAttribute(g_ctx.pool, cudaMemPoolAttrReservedMemCurrent, &r));
        *bytes_reserved = r;
    }
    return TLB_OK;
}

tlb_status tlb_event_create(void **ev)
{
    if (!ev) return fail(TLB_ERR_NULL, "null event pointer");
    if (!ensure_init()) return TLB_ERR_DEVICE;
    cudaEvent_t e;
    TLB_CUDA(cudaEventCreate(&e));
    *ev = (void *)e;
    return TLB_OK;
}

tlb_status tlb_event_record(void *ev)
{
    if (!ev) return fail(TLB_ERR_NULL, "null event");
    TLB_CUDA(cudaEventRecord((cudaEvent_t)ev, g_ctx.stream));
    return TLB_OK;
}

tlb_status tlb_event_elapsed_ms(void *start, void *stop, float *ms)
{
    if (!start || !stop || !ms) return fail(TLB_ERR_NULL, "null argument");
    TLB_CUDA(cudaEventSynchronize((cudaEvent_t)stop));
    TLB_CUDA(cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)stop));
    return TLB_OK;
}

tlb_status tlb_event_destroy(void *ev)
{
    if (ev) TLB_CUDA(cudaEventDestroy((cudaEvent_t)ev));
    return TLB_OK;
}

tlb_status tlb_flush_l2(void)
{
    if (!ensure_init()) return TLB_ERR_DEVICE;
    if (!g_ctx.flush_buf) {
        g_ctx.flush_bytes = (size_t)256 << 20;  // 2x the 126 MB L2
        TLB_CUDA(cudaMalloc(&g_ctx.flush_buf, g_ctx.flush_bytes));
    }
    TLB_CUDA(cudaMemsetAsync(g_ctx.flush_buf, 0, g_ctx.flush_bytes, g_ctx.stream));
    return TLB_OK;
}

/* ---- tensors ---- */

tlb_status tlb_tensor_from_host(tlb_tensor **out, const void *data, tlb_dtype dt, const int64_t *shape, int rank)
{
    if (!out) return fail(TLB_ERR_NULL, "null out");
    *out = nullptr;
    if (rank > 0 && !shape) return fail(TLB_ERR_NULL, "null shape");
    if (g_inited && g_ctx.capturing) return fail(TLB_ERR_ARG, "tensor_from_host copies from host memory and waits for it: not allowed during a stream capture");
    TLB_TRY(new_tensor(out, dt, shape, rank));
    size_t bytes = (size_t)(*out)->numel() * dtype_size(dt);
    if (bytes) {
        if (!data) { tlb_tensor_release(*out); *out = nullptr; return fail(TLB_ERR_NULL, "null data"); }
        cudaError_t e = cudaMemcpyAsync((*out)->data(), data, bytes, cudaMemcpyHostToDevice, g_ctx.stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(g_ctx.stream);  // host buffer may be pageable
        if (e != cudaSuccess) { tlb_tensor_release(*out); *out = nullptr; return cuda_fail(e, "upload"); }
    }
    return TLB_OK;
}

tlb_status tlb_tensor_zeros(tlb_tensor **out, tlb_dtype dt, const int64_t *shape, int rank)
{
    if (!out) return fail(TLB_ERR_NULL, "null out");
    TLB_TRY(new_tensor(out, dt, shape, rank));
    size_t bytes = (size_t)(*out)->numel() * dtype_size(dt);
    if (bytes) TLB_CUDA(cudaMemsetAsync((*out)->data(), 0, bytes, g_ctx.stream));
    return TLB_OK;
}

tlb_status tlb_tensor_to_host(const tlb_tensor *t, void *dst, size_t dst_bytes)
{
    if (!t || (!dst && dst_bytes)) return fail(TLB_ERR_NULL, "null argument");
    size_t bytes = (size_t)t->numel() * dtype_size(t->dt);
    if (dst_bytes < bytes) return fail(TLB_ERR_ARG, "destination holds %zu bytes, tensor has %zu", dst_bytes, bytes);
    if (bytes) TLB_CUDA(cudaMemcpyAsync(dst, t->data(), bytes, cudaMemcpyDeviceToHost, g_ctx.stream));
    return tlb_sync();
}

tlb_status tlb_tensor_retain(tlb_tensor *t)
{
    if (!t) return fail(TLB_ERR_NULL, "null tensor");
    t->rc.fetch_add(1);
    return TLB_OK;
}

tlb_status tlb_tensor_release(tlb_tensor *t)
{
    if (!t) return TLB_OK;  // release_safe semantics: null is ignored
    if (t->rc.fetch_sub(1) == 1) {
        storage_release(t->st);
        delete t;
    }
    return TLB_OK;
}

int tlb_tensor_refcount(const tlb_tensor *t) { return t ? t->rc.load() : 0; }
int tlb_tensor_rank(const tlb_tensor *t) { return t ? t->rank : -1; }
int64_t tlb_tensor_numel(const tlb_tensor *t) { return t ? t->numel() : -1; }
tlb_dtype tlb_tensor_dtype(const tlb_tensor *t) { return t ? t->dt : TLB_F32; }
void *tlb_tensor_data(const tlb_tensor *t) { return t ? t->data() : nullptr; }

tlb_status tlb_tensor_shape(const tlb_tensor *t, int64_t *shape_out, int max_rank)
{
    if (!t || !shape_out) return fail(TLB_ERR_NULL, "null argument");
    if (max_rank < t->rank) return fail(TLB_ERR_ARG, "shape buffer too small");
    for (int i = 0; i < t->rank; i++) shape_out[i] = t->shape[i];
    return TLB_OK;
}

tlb_status tlb_tensor_clone(tlb_tensor **out, const tlb_tensor *t)
{
    if (!out || !t) return fail(TLB_ERR_NULL, "null argument");
    TLB_TRY(new_tensor(out, t->dt, t->shape, t->rank));
    size_t bytes = (size_t)t->numel() * dtype_size(t->dt);
    if (bytes) TLB_CUDA(cudaMemcpyAsync((*out)->data(), t->data(), bytes, cudaMemcpyDeviceToDevice, g_ctx.stream));
    return TLB_OK;
}

tlb_status tlb_tensor_item_i64(const tlb_tensor *t, int64_t *value)
{
    if (!t || !value) return fail(TLB_ERR_NULL, "null argument");
    if (t->numel() < 1) return fail(TLB_ERR_SHAPE, "item on empty tensor");
    if (t->dt == TLB_F32) {
        float f;
        TLB_CUDA(cudaMemcpyAsync(&f, t->data(), 4, cudaMemcpyDeviceToHost, g_ctx.stream));
        TLB_TRY(tlb_sync());
        *value = (int64_t)f;
    } else if (t->dt == TLB_I64) {
        TLB_CUDA(cudaMemcpyAsync(value, t->data(), 8, cudaMemcpyDeviceToHost, g_ctx.stream));
        TLB_TRY(tlb_sync());
    } else if (t->dt == TLB_I32) {
        int32_t v;
        TLB_CUDA(cudaMemcpyAsync(&v, t->data(), 4, cudaMemcpyDeviceToHost, g_ctx.stream));
        TLB_TRY(tlb_sync());
        *value = v;
    } else {
        return fail(TLB_ERR_TYPE, "item_i64: unsupported dtype %d", (int)t->dt);
    }
    return TLB_OK;
}

/* ---- stream capture / graphs ---- */

}  // extern "C"

struct tlb_graph {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    size_t nodes = 0;
    uint64_t kernels = 0;
};

extern "C" {

tlb_status tlb_stream_begin_capture(void)
{
    if (!ensure_init()) return TLB_ERR_DEVICE;
    if (g_ctx.capturing) return fail(TLB_ERR_ARG, "capture already in progress");
    TLB_CUDA(cudaStreamBeginCapture(g_ctx.stream, cudaStreamCaptureModeThreadLocal));
    g_ctx.capturing = true;
    g_ctx.capture_launches = g_ctx.launches.load();
    return TLB_OK;
}

tlb_status tlb_stream_end_capture(tlb_graph **out)
{
    if (!out) return fail(TLB_ERR_NULL, "null out");
    *out = nullptr;
    if (!g_inited || !g_ctx.capturing) return fail(TLB_ERR_ARG, "no capture in progress");
    g_ctx.capturing = false;
    cudaGraph_t g = nullptr;
    cudaError_t ce = cudaStreamEndCapture(g_ctx.stream, &g);
    run_deferred_destroys();
    if (ce != cudaSuccess) return cuda_fail(ce, "cudaStreamEndCapture");
    tlb_graph *tg = new tlb_graph();
    tg->graph = g;
    tg->kernels = g_ctx.launches.load() - g_ctx.capture_launches;
    g_ctx.launches = g_ctx.capture_launches;  // captured launches run only when replayed
    cudaError_t e = cudaGraphGetNodes(g, nullptr, &tg->nodes);
    // Ops captured here allocate their results from the stream-ordered pool, so the graph owns allocation nodes.
    // AutoFreeOnLaunch: a replay first frees what the previous replay allocated (same addresses again), so a graph
    // can be replayed any number of times; results of a replay are valid until the next one.
    if (e == cudaSuccess) e = cudaGraphInstantiate(&tg->exec, g, cudaGraphInstantiateFlagAutoFreeOnLaunch);
    if (e != cudaSuccess) {
        cudaGraphDestroy(g);
        delete tg;
        return cuda_fail(e, "cudaGraphInstantiate");
    }
    *out = tg;
    return TLB_OK;
}

int tlb_stream_is_capturing(void) { return g_inited && g_ctx.capturing ? 1 : 0; }

tlb_status tlb_graph_replay(tlb_graph *g)
{
    if (!g) return fail(TLB_ERR_NULL, "null graph");
    TLB_CUDA(cudaGraphLaunch(g->exec, g_ctx.stream));
    g_ctx.launches += g->kernels;
    return TLB_OK;
}

int64_t tlb_graph_node_count(const tlb_graph *g) { return g ? (int64_t)g->nodes : -1; }

tlb_status tlb_graph_destroy(tlb_graph *g)
{
    if (!g) return TLB_OK;
    if (g->exec) cudaGraphExecDestroy(g->exec);
    if (g->graph) cudaGraphDestroy(g->graph);
    delete g;
    return TLB_OK;
}

}  // extern "C"
