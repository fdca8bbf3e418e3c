// Entry points with the reference's OWN raw signatures, for the places where its runtime goes around the
// backend trait, plus the few trait slots that take their arguments in a TL-specific form.
//
//   tl_cuda_mul_mv_q4_k / tl_cuda_mul_mv_q6_k (crates/tl_runtime/src/device_ffi.rs:1805-1833 declares them,
//   crates/tl_cuda/src/ffi_ops.rs:1314-1391 defines them): (x, w_raw, n, k) -> tensor, where w_raw is a U8 device tensor
//   holding the raw GGUF bytes that QTensor::gpu_raw_cache uploaded (crates/tl_runtime/src/system.rs:316-331).  The
//   reference's kernel reads those bytes as they are, one thread per output.  Here the bytes are repacked ONCE into the
//   tiled layout - a cache keyed by the raw tensor's device address, holding a reference to it - and every call after
//   the first streams the tiled copy through the fused kernels.  Exported under the reference's symbol names, so a
//   tl_runtime linked against libtlb200 instead of tl_cuda resolves them unchanged.
//   tlb_reshape_new     tl_tensor_reshape_new(T*, T* shape) (device_ffi.rs:1193): the shape arrives as a tensor of f32
//   tlb_cat_i64         tl_tensor_cat_i64 (device_ffi.rs:1250): integers travel as f32 here, so this is tlb_cat
//   tlb_map_get_1d      tl_tensor_map_get_1d (src/compiler/codegen/builtins.rs:2687): the same lookup as tlb_map_get
//   tlb_gguf_load_str   tl_gguf_load(StringStruct*) (crates/tl_runtime/src/string_ffi.rs:7-11): pointer + length
//   tlb_fused_rotary_emb GpuFusedOps::fused_rotary_emb (crates/tl_cuda/src/ops/fused.rs:129-185): rotate-half with ONE
//                       table passed as both cos and sin, as that implementation does
#include "tlb_internal.h"

#include <map>

using namespace tlb;

namespace {

struct RawKey {
    const void *ptr;
    int type;
    int64_t n, k;
    bool operator<(const RawKey &o) const
    {
        if (ptr != o.ptr) return ptr < o.ptr;
        if (type != o.type) return type < o.type;
        if (n != o.n) return n < o.n;
        return k < o.k;
    }
};
struct RawEntry {
    tlb_qtensor *q;
    tlb_tensor *raw;   // retained: the address stays this tensor's for as long as the entry lives
};
std::mutex g_raw_mu;
std::map<RawKey, RawEntry> g_raw_cache;

tlb_status qtensor_from_device_bytes(tlb_qtensor **out, int type, int64_t n, int64_t k, const uint8_t *raw_dev, size_t nbytes)
{
    const QFormat *f = qformat(type);
    if (!f || k % 256) return fail(TLB_ERR_SHAPE, "raw-bytes matvec takes Q4_K / Q6_K weights with K a multiple of 256");
    const size_t need = (size_t)n * (k / f->raw_block) * f->raw_block_bytes;
    if (nbytes < need) return fail(TLB_ERR_SHAPE, "raw weight tensor holds %zu bytes, [%lld, %lld] of type %d needs %zu", nbytes, (long long)n, (long long)k, type, need);
    tlb_qtensor *q = new tlb_qtensor();
    q->type = type; q->n = n; q->k = k;
    q->n_tiles = (n + 15) / 16;
    q->upt = k / 256;
    const size_t tiled = (size_t)q->n_tiles * q->upt * f->unit_bytes;
    q->st = storage_alloc(tiled);
    if (!q->st) { delete q; return TLB_ERR_ALLOC; }
    cudaError_t e = (n % 16) ? cudaMemsetAsync(q->st->ptr, 0, tiled, ctx()->stream) : cudaSuccess;
    tlb_status st = e == cudaSuccess ? launch_repack(type, raw_dev, q->dev(), n, k) : cuda_fail(e, "repack");
    if (st != TLB_OK) { storage_release(q->st); delete q; return st; }
    *out = q;
    return TLB_OK;
}

void *mul_mv_raw(void *x, void *w_raw, int64_t n, int64_t k, int type)
{
    tlb_tensor *xt = (tlb_tensor *)x, *wt = (tlb_tensor *)w_raw;
    if (!xt || !wt) { fail(TLB_ERR_NULL, "tl_cuda_mul_mv: null tensor"); return nullptr; }
    if (!ensure_init()) return nullptr;
    if (wt->dt != TLB_U8) { fail(TLB_ERR_TYPE, "tl_cuda_mul_mv: the raw weight must be a U8 tensor"); return nullptr; }
    tlb_qtensor *q = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_raw_mu);
        const RawKey key{wt->data(), type, n, k};
        auto it = g_raw_cache.find(key);
        if (it == g_raw_cache.end()) {
            if (qtensor_from_device_bytes(&q, type, n, k, (const uint8_t *)wt->data(), (size_t)wt->numel()) != TLB_OK) return nullptr;
            tlb_tensor_retain(wt);
            g_raw_cache[key] = RawEntry{q, wt};
        } else {
            q = it->second.q;
        }
    }
    tlb_tensor *out = nullptr;
    if (tlb_qtensor_matmul(&out, xt, q) != TLB_OK) return nullptr;
    return out;
}

}  // namespace

extern "C" {

void *tl_cuda_mul_mv_q4_k(void *x, void *w_raw, int64_t n, int64_t k) { return mul_mv_raw(x, w_raw, n, k, TLB_GGML_Q4_K); }
void *tl_cuda_mul_mv_q6_k(void *x, void *w_raw, int64_t n, int64_t k) { return mul_mv_raw(x, w_raw, n, k, TLB_GGML_Q6_K); }

// Drops the repacked copies (and the references to their raw tensors); returns how many there were.
int64_t tlb_raw_weight_cache_clear(void)
{
    std::lock_guard<std::mutex> lk(g_raw_mu);
    const int64_t n = (int64_t)g_raw_cache.size();
    for (auto &kv : g_raw_cache) {
        tlb_qtensor_release(kv.second.q);
        tlb_tensor_release(kv.second.raw);
    }
    g_raw_cache.clear();
    return n;
}

tlb_status tlb_reshape_new(tlb_tensor **out, const tlb_tensor *a, const tlb_tensor *shape)
{
    if (!out) return fail(TLB_ERR_NULL, "null out");
    *out = nullptr;
    if (!a || !shape) return fail(TLB_ERR_NULL, "reshape: null tensor");
    if (shape->dt != TLB_F32) return fail(TLB_ERR_TYPE, "reshape: the shape tensor holds f32 values");
    const int64_t rank = shape->numel();
    if (rank < 0 || rank > kMaxRank) return fail(TLB_ERR_SHAPE, "reshape: rank %lld not supported", (long long)rank);
    float dims_f[kMaxRank] = {0};
    if (rank) TLB_TRY(tlb_tensor_to_host(shape, dims_f, (size_t)rank * sizeof(float)));
    int64_t dims[kMaxRank];
    for (int64_t i = 0; i < rank; i++) dims[i] = (int64_t)dims_f[i];
    return tlb_reshape(out, a, dims, (int)rank);
}

tlb_status tlb_cat_i64(tlb_tensor **out, const tlb_tensor *a, const tlb_tensor *b, int64_t dim) { return tlb_cat(out, a, b, dim); }

tlb_status tlb_map_get_1d(tlb_tensor **out, tlb_map *m, const char *name) { return tlb_map_get(out, m, name); }

tlb_status tlb_gguf_load_str(tlb_map **out, const tlb_string *path)
{
    if (!out) return fail(TLB_ERR_NULL, "null out");
    *out = nullptr;
    if (!path || !path->ptr || path->len < 0) return fail(TLB_ERR_NULL, "null path");
    const std::string p(path->ptr, (size_t)path->len);   // TL strings carry their length; a terminator is not assumed
    return tlb_gguf_load(out, p.c_str());
}

tlb_status tlb_fused_rotary_emb(tlb_tensor **out, const tlb_tensor *x, const tlb_tensor *freqs, int64_t head_dim)
{
    if (!out) return fail(TLB_ERR_NULL, "null out");
    *out = nullptr;
    if (!x || !freqs) return fail(TLB_ERR_NULL, "fused_rotary_emb: null tensor");
    if (x->dt != TLB_F32 || freqs->dt != TLB_F32) return fail(TLB_ERR_TYPE, "fused_rotary_emb: f32 tensors expected");
    if (head_dim < 2 || head_dim % 2 || x->rank < 1 || x->shape[x->rank - 1] != head_dim)
        return fail(TLB_ERR_SHAPE, "fused_rotary_emb: the last dimension must equal head_dim (even)");
    // token / head split as crates/tl_cuda/src/ops/fused.rs:144-152
    int64_t tokens, heads;
    if (x->rank == 4) { tokens = x->shape[1]; heads = x->shape[0] * x->shape[2]; }
    else if (x->rank == 3) { tokens = x->shape[0]; heads = x->shape[1]; }
    else if (x->rank == 2) { tokens = x->shape[0]; heads = 1; }
    else { tokens = 1; heads = x->numel() / head_dim; }
    const int64_t rows = freqs->rank >= 2 ? freqs->shape[0] : 1, cols = freqs->rank >= 1 ? freqs->shape[freqs->rank - 1] : 0;
    if (rows < tokens || cols < head_dim / 2) return fail(TLB_ERR_SHAPE, "fused_rotary_emb: the table must hold [%lld, %lld] entries", (long long)tokens, (long long)(head_dim / 2));
    if (cols != head_dim / 2) return fail(TLB_ERR_SHAPE, "fused_rotary_emb: table rows of %lld entries, expected head_dim / 2 = %lld", (long long)cols, (long long)(head_dim / 2));
    TLB_TRY(new_tensor(out, TLB_F32, x->shape, x->rank));
    tlb_status st = launch_rope_half(x->f32(), freqs->f32(), freqs->f32(), (*out)->f32(), tokens, heads, head_dim);
    if (st != TLB_OK) { tlb_tensor_release(*out); *out = nullptr; }
    return st;
}

}  // extern "C"
