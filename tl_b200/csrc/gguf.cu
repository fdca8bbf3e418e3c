// GGUF loader, tensor map and the KV-cache handle table (host code).
//   tl_gguf_load        crates/tl_runtime/src/gguf.rs:34-196
//   OpaqueTensorMap     crates/tl_runtime/src/tensor_map.rs:19-22,110-150,279
//   OpaqueKVCache       crates/tl_runtime/src/system.rs:387-615
// Differences from the reference by design: quantized tensors are repacked once into the tiled
// device layout while loading (the reference copies the raw bytes into a Vec<u8> and uploads them
// on first use), and host bytes are not kept afterwards.
#include "tlb_internal.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <map>

using namespace tlb;

struct MapEntry {
    int type = 0;
    std::vector<int64_t> shape;   // row-major
    tlb_qtensor *q = nullptr;     // quantized types
    tlb_tensor *f32 = nullptr;    // F32 / F16 data, or the cached dequantisation of q
};

struct tlb_map {
    std::vector<std::string> names;
    std::map<std::string, MapEntry> entries;
    std::map<std::string, double> meta_num;        // scalar numeric / bool metadata of the GGUF file
    std::map<std::string, std::string> meta_str;   // string metadata
};

struct tlb_kvcache {
    std::vector<std::pair<tlb_tensor *, tlb_tensor *>> layers;
};

namespace tlb {

__global__ void f16_to_f32_kernel2(const __half *a, float *out, int64_t n)
{
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = __half2float(a[i]);
}

static bool ggml_known(int type)
{
    return type == TLB_GGML_F32 || type == TLB_GGML_F16 || type == TLB_GGML_Q4_0 || type == TLB_GGML_Q4_1 || type == TLB_GGML_Q5_0 ||
           type == TLB_GGML_Q5_1 || type == TLB_GGML_Q8_0 || type == TLB_GGML_Q8_1 || type == TLB_GGML_Q4_K || type == TLB_GGML_Q6_K;
}

// Product of the dimensions, or -1 when a dimension is negative or the product leaves int64.
static int64_t checked_numel(const int64_t *shape, int rank)
{
    int64_t n = 1;
    for (int i = 0; i < rank; i++) {
        if (shape[i] < 0) return -1;
        if (shape[i] && n > INT64_MAX / shape[i]) return -1;
        n *= shape[i];
    }
    return n;
}

static tlb_status map_add(tlb_map *m, const std::string &name, int type, const int64_t *shape, int rank,
                          const void *bytes, size_t nbytes)
{
    if (m->entries.count(name)) return fail(TLB_ERR_ARG, "tensor '%s' already in the map", name.c_str());
    const int64_t nelem = checked_numel(shape, rank);
    if (nelem < 0) return fail(TLB_ERR_SHAPE, "tensor '%s' has a negative or overflowing shape", name.c_str());
    const size_t need = ggml_raw_nbytes(type, nelem);
    if ((nelem && !need) || need != nbytes)
        return fail(TLB_ERR_SHAPE, "tensor '%s': %zu bytes do not match type %d x %lld elements", name.c_str(), nbytes, type, (long long)nelem);
    MapEntry e;
    e.type = type;
    e.shape.assign(shape, shape + rank);
    if (type == TLB_GGML_F32) {
        TLB_TRY(tlb_tensor_from_host(&e.f32, bytes, TLB_F32, shape, rank));
    } else if (type == TLB_GGML_F16) {  // F16 -> f32, exact widening (quantized.rs:167-180)
        tlb_tensor *h = nullptr;
        TLB_TRY(tlb_tensor_from_host(&h, bytes, TLB_F16, shape, rank));
        tlb_status st = new_tensor(&e.f32, TLB_F32, shape, rank);
        if (st == TLB_OK && nelem) {
            int blocks = (int)std::min<int64_t>((nelem + 255) / 256, 148 * 16);
            f16_to_f32_kernel2<<<blocks, 256, 0, ctx()->stream>>>((const __half *)h->data(), e.f32->f32(), nelem);
            count_launch();
        }
        tlb_tensor_release(h);
        TLB_TRY(st);
    } else {
        // block-quantized: a matrix (the reference's loader gives every tensor a QTensor, gguf.rs:129-190; 1-D
        // quantized tensors do not occur in model files and are taken as one row)
        const int64_t n = rank >= 2 ? nelem / std::max<int64_t>(1, shape[rank - 1]) : 1, k = rank >= 1 ? shape[rank - 1] : 1;
        TLB_TRY(tlb_qtensor_from_gguf_bytes(&e.q, (tlb_ggml_type)type, n, k, bytes, nbytes));
    }
    m->names.push_back(name);
    m->entries[name] = e;
    return TLB_OK;
}

struct Reader {
    const uint8_t *p;
    size_t n, off = 0;
    bool ok = true;
    template <typename T> T get()
    {
        T v{};
        if (off > n || sizeof(T) > n - off) { ok = false; return v; }
        memcpy(&v, p + off, sizeof(T));
        off += sizeof(T);
        return v;
    }
    std::string str()
    {
        uint64_t len = get<uint64_t>();
        if (!ok || len > n - off) { ok = false; return ""; }   // subtraction form: a huge length cannot wrap
        std::string s((const char *)p + off, (size_t)len);
        off += len;
        return s;
    }
    void skip(size_t b) { if (b > n - off) ok = false; else off += b; }
};

static size_t gguf_scalar_size(uint32_t t)
{
    switch (t) {
    case 0: case 1: case 7: return 1;
    case 2: case 3: return 2;
    case 4: case 5: case 6: return 4;
    case 10: case 11: case 12: return 8;
    default: return 0;
    }
}

// skips one metadata value; returns its u64 view when it is an unsigned integer (for general.alignment);
// scalar numbers and strings are also kept (num / str, when given) for tlb_map_meta_*
static bool gguf_skip_value(Reader &r, uint32_t t, uint64_t *uint_val, double *num = nullptr, bool *has_num = nullptr,
                            std::string *str = nullptr)
{
    if (t == 8) { std::string v = r.str(); if (str) *str = v; return r.ok; }
    if (num && has_num && t != 9 && r.ok) {
        const size_t sz = gguf_scalar_size(t);
        if (sz && sz <= r.n - r.off) {
            const uint8_t *q = r.p + r.off;
            *has_num = true;
            switch (t) {
            case 0: { uint8_t v; memcpy(&v, q, 1); *num = v; break; }
            case 1: { int8_t v; memcpy(&v, q, 1); *num = v; break; }
            case 2: { uint16_t v; memcpy(&v, q, 2); *num = v; break; }
            case 3: { int16_t v; memcpy(&v, q, 2); *num = v; break; }
            case 4: { uint32_t v; memcpy(&v, q, 4); *num = v; break; }
            case 5: { int32_t v; memcpy(&v, q, 4); *num = v; break; }
            case 6: { float v; memcpy(&v, q, 4); *num = v; break; }
            case 7: { uint8_t v; memcpy(&v, q, 1); *num = v ? 1.0 : 0.0; break; }
            case 10: { uint64_t v; memcpy(&v, q, 8); *num = (double)v; break; }
            case 11: { int64_t v; memcpy(&v, q, 8); *num = (double)v; break; }
            case 12: { double v; memcpy(&v, q, 8); *num = v; break; }
            default: *has_num = false;
            }
        }
    }
    if (t == 9) {
        uint32_t et = r.get<uint32_t>();
        uint64_t cnt = r.get<uint64_t>();
        if (!r.ok) return false;
        if (et == 8) {
            if (cnt > r.n - r.off) return false;      // every string takes at least its 8-byte length
            for (uint64_t i = 0; i < cnt && r.ok; i++) r.str();
            return r.ok;
        }
        size_t es = gguf_scalar_size(et);
        if (!es) return false;
        if (cnt > (r.n - r.off) / es) return false;   // the array cannot be longer than the rest of the file
        r.skip((size_t)cnt * es);
        return r.ok;
    }
    size_t s = gguf_scalar_size(t);
    if (!s) return false;
    if (uint_val && (t == 0 || t == 2 || t == 4 || t == 10)) {
        uint64_t v = 0;
        if (s <= r.n - r.off) memcpy(&v, r.p + r.off, s);
        *uint_val = v;
    }
    r.skip(s);
    return r.ok;
}

}  // namespace tlb

extern "C" {

tlb_status tlb_map_new(tlb_map **out)
{
    if (!out) return fail(TLB_ERR_NULL, "null out");
    *out = new tlb_map();
    return TLB_OK;
}

tlb_status tlb_map_meta_number(const tlb_map *m, const char *key, double *out)
{
    if (!m || !key || !out) return fail(TLB_ERR_NULL, "null argument");
    auto it = m->meta_num.find(key);
    if (it == m->meta_num.end()) return fail(TLB_ERR_INDEX, "no numeric metadata '%s'", key);
    *out = it->second;
    return TLB_OK;
}

const char *tlb_map_meta_string(const tlb_map *m, const char *key)
{
    if (!m || !key) return nullptr;
    auto it = m->meta_str.find(key);
    return it == m->meta_str.end() ? nullptr : it->second.c_str();
}

// Decoder sizes from the file instead of literals in the caller: `<arch>.block_count`, `.embedding_length`,
// `.attention.head_count`, `.attention.head_count_kv`, `.feed_forward_length`, `.attention.layer_norm_rms_epsilon`,
// `.rope.freq_base`, `.rope.dimension_count` (arch = general.architecture, "llama" if absent); vocab from the shape of
// token_embd.weight.  The reference programs hard-code these (examples/apps/llama3/chatbot_llama3.tl:67-71,95,106,196) and
// scale the scores by the literals 0.08839 (head_dim 128) / 0.125 (head_dim 64): the same literals are used here,
// 1 / sqrt(head_dim) for other sizes.  kv_f16, max_seq, tie_rule and the tp fields are left as the caller set them.
tlb_status tlb_decoder_cfg_from_map(const tlb_map *m, tlb_decoder_cfg *cfg)
{
    if (!m || !cfg) return fail(TLB_ERR_NULL, "null argument");
    const char *a = tlb_map_meta_string(m, "general.architecture");
    const std::string arch = a ? a : "llama";
    auto num = [&](const std::string &key, double *v) {
        auto it = m->meta_num.find(arch + "." + key);
        if (it == m->meta_num.end()) return false;
        *v = it->second;
        return true;
    };
    double layers, dm, heads, kvh, ffn, eps = 1e-5, base = 10000.0, rdim = 0;
    if (!num("block_count", &layers) || !num("embedding_length", &dm) || !num("attention.head_count", &heads) || !num("feed_forward_length", &ffn))
        return fail(TLB_ERR_ARG, "GGUF metadata lacks %s.block_count / embedding_length / attention.head_count / feed_forward_length", arch.c_str());
    if (!num("attention.head_count_kv", &kvh)) kvh = heads;
    num("attention.layer_norm_rms_epsilon", &eps);
    num("rope.freq_base", &base);
    if (heads < 1 || layers < 1 || dm < 1) return fail(TLB_ERR_ARG, "GGUF metadata holds a non-positive size");
    if (!num("rope.dimension_count", &rdim) || rdim < 1) rdim = dm / heads;
    auto emb = m->entries.find("token_embd.weight");
    if (emb == m->entries.end() || emb->second.shape.size() != 2) return fail(TLB_ERR_ARG, "token_embd.weight is missing or not a matrix");
    cfg->n_layers = (int32_t)layers; cfg->d_model = (int32_t)dm; cfg->n_heads = (int32_t)heads; cfg->n_kv_heads = (int32_t)kvh;
    cfg->head_dim = (int32_t)rdim; cfg->ffn = (int32_t)ffn; cfg->vocab = (int32_t)emb->second.shape[0];
    cfg->eps = (float)eps; cfg->rope_base = (float)base;
    cfg->attn_scale = cfg->head_dim == 128 ? 0.08839f : (cfg->head_dim == 64 ? 0.125f : 1.0f / sqrtf((float)cfg->head_dim));
    return TLB_OK;
}

tlb_status tlb_map_add(tlb_map *m, const char *name, tlb_ggml_type type, const int64_t *shape, int rank, const void *bytes, size_t nbytes)
{
    if (!m || !name || (rank > 0 && !shape)) return fail(TLB_ERR_NULL, "null argument");
    if (!ggml_known(type)) return fail(TLB_ERR_TYPE, "unsupported GGML type %d for '%s'", (int)type, name);
    if (!ensure_init()) return TLB_ERR_DEVICE;
    return map_add(m, name, type, shape, rank, bytes, nbytes);
}

static tlb_status gguf_load_impl(tlb_map **out, const char *path, int tp_rank, int tp_size);

tlb_status tlb_gguf_load(tlb_map **out, const char *path) { return gguf_load_impl(out, path, 0, 1); }

/* tl_gguf_load for one rank of a tensor-parallel group: only this rank's shard of every split tensor is uploaded. */
tlb_status tlb_gguf_load_tp(tlb_map **out, const char *path, int tp_rank, int tp_size)
{
    if (tp_size < 1 || tp_rank < 0 || tp_rank >= tp_size) return fail(TLB_ERR_ARG, "shard %d of %d", tp_rank, tp_size);
    return gguf_load_impl(out, path, tp_rank, tp_size);
}

static tlb_status gguf_load_impl(tlb_map **out, const char *path, int tp_rank, int tp_size)
{
    if (!out) return fail(TLB_ERR_NULL, "null out");
    *out = nullptr;
    if (!path) return fail(TLB_ERR_NULL, "null path");
    int fd = open(path, O_RDONLY);
    if (fd < 0) return fail(TLB_ERR_ARG, "Failed to open GGUF file %s", path);
    struct stat sb;
    if (fstat(fd, &sb) != 0) { close(fd); return fail(TLB_ERR_ARG, "cannot stat %s", path); }
    size_t fsize = (size_t)sb.st_size;
    if (fsize < 4) { close(fd); return fail(TLB_ERR_ARG, "File too small"); }
    void *mm = mmap(nullptr, fsize, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (mm == MAP_FAILED) return fail(TLB_ERR_ARG, "Failed to mmap GGUF file");
    tlb_status st = TLB_OK;
    tlb_map *m = new tlb_map();
    do {
        Reader r{(const uint8_t *)mm, fsize};
        if (memcmp(r.p, "GGUF", 4) != 0) {
            st = fail(TLB_ERR_ARG, memcmp(r.p, "FUGG", 4) == 0 ? "big-endian GGUF files are not supported" : "Invalid GGUF magic");
            break;
        }
        r.off = 4;
        uint32_t version = r.get<uint32_t>();
        uint64_t n_tensors = r.get<uint64_t>(), n_kv = r.get<uint64_t>();
        if (!r.ok || version < 2 || version > 3) { st = fail(TLB_ERR_ARG, "unsupported GGUF version %u", version); break; }
        uint64_t alignment = 32;  // default alignment (gguf.rs:102-110)
        for (uint64_t i = 0; i < n_kv && r.ok; i++) {
            std::string key = r.str();
            uint32_t t = r.get<uint32_t>();
            uint64_t uv = 0;
            double num = 0.0;
            bool has_num = false;
            std::string sv;
            if (!r.ok || !gguf_skip_value(r, t, &uv, &num, &has_num, &sv)) { r.ok = false; break; }
            if (key == "general.alignment" && uv) alignment = uv;
            if (has_num) m->meta_num[key] = num;
            else if (t == 8) m->meta_str[key] = sv;
        }
        if (!r.ok) { st = fail(TLB_ERR_ARG, "Failed to decode GGUF metadata"); break; }
        struct Info { std::string name; std::vector<int64_t> shape; uint32_t type; uint64_t offset; };
        std::vector<Info> infos;
        for (uint64_t i = 0; i < n_tensors && r.ok; i++) {
            Info inf;
            inf.name = r.str();
            uint32_t nd = r.get<uint32_t>();
            if (!r.ok || nd > kMaxRank) { r.ok = false; break; }
            for (uint32_t d = 0; d < nd; d++) {
                const uint64_t dim = r.get<uint64_t>();
                if (dim > (uint64_t)INT64_MAX) r.ok = false;
                inf.shape.push_back((int64_t)dim);
            }
            inf.type = r.get<uint32_t>();
            inf.offset = r.get<uint64_t>();
            // trailing 1-dims are trimmed, then GGML's fastest-first order is reversed (gguf.rs:129-136)
            while (inf.shape.size() > 1 && inf.shape.back() == 1) inf.shape.pop_back();
            std::reverse(inf.shape.begin(), inf.shape.end());
            infos.push_back(inf);
        }
        if (!r.ok) { st = fail(TLB_ERR_ARG, "Failed to decode GGUF tensor infos"); break; }
        if (alignment == 0 || alignment > (1u << 20)) { st = fail(TLB_ERR_ARG, "GGUF alignment %llu is not usable", (unsigned long long)alignment); break; }
        const uint64_t data_off = (r.off + alignment - 1) / alignment * alignment;
        for (const Info &inf : infos) {
            if (!ggml_known((int)inf.type)) continue;  // unsupported kinds are skipped (gguf.rs:157-177)
            const int64_t nelem = checked_numel(inf.shape.data(), (int)inf.shape.size());
            if (nelem < 0) continue;
            const size_t nb = ggml_raw_nbytes((int)inf.type, nelem);
            if (nelem && !nb) continue;                // not a whole number of blocks
            // "data out of bounds": skipped (gguf.rs:183-186); subtraction form, so that a huge offset cannot wrap
            if (data_off > fsize || inf.offset > fsize - data_off || nb > fsize - data_off - inf.offset) continue;
            if ((int)inf.type != TLB_GGML_F32 && (int)inf.type != TLB_GGML_F16 && !inf.shape.empty()) {
                // rows must hold whole blocks: K-quants need K % 256 == 0, the 32-blocks K % 32 == 0
                const int64_t kk = inf.shape.back();
                const bool k_quant = (int)inf.type == TLB_GGML_Q4_K || (int)inf.type == TLB_GGML_Q6_K;
                if (kk % (k_quant ? 256 : 32)) continue;
            }
            if (tp_size > 1) {
                if (!ensure_init()) { st = TLB_ERR_DEVICE; break; }
                st = tlb_map_add_tp(m, inf.name.c_str(), (tlb_ggml_type)inf.type, inf.shape.data(), (int)inf.shape.size(), r.p + data_off + inf.offset, nb, tp_rank, tp_size);
            } else {
                st = map_add(m, inf.name, (int)inf.type, inf.shape.data(), (int)inf.shape.size(), r.p + data_off + inf.offset, nb);
            }
            if (st != TLB_OK) break;
        }
    } while (0);
    munmap(mm, fsize);
    if (st != TLB_OK) { tlb_map_free(m); return st; }
    *out = m;
    return TLB_OK;
}

/* ---- tensor-parallel shards (host side) ----
 * Megatron split of a Llama block by tensor name: attn_q / attn_k / attn_v / ffn_gate / ffn_up and the output head are
 * cut along their rows (each rank keeps whole heads / hidden units / vocabulary entries: a contiguous byte range of
 * the row-major GGUF tensor); attn_output and ffn_down along their columns (per row, a contiguous range of blocks);
 * everything else (embedding, norm weights) is replicated. */
int tlb_tp_split_kind(const char *name)
{
    if (!name) return 0;
    const std::string s(name);
    auto ends = [&](const char *suffix) { const size_t n = strlen(suffix); return s.size() >= n && s.compare(s.size() - n, n, suffix) == 0; };
    if (ends("attn_q.weight") || ends("attn_k.weight") || ends("attn_v.weight") || ends("ffn_gate.weight") || ends("ffn_up.weight") || s == "output.weight") return 1;
    if (ends("attn_output.weight") || ends("ffn_down.weight")) return 2;
    return 0;
}

tlb_status tlb_tp_shard_bytes(int kind, tlb_ggml_type type, int64_t n, int64_t k, const void *bytes, size_t nbytes, int rank, int size,
                              void *out, size_t out_cap, int64_t *n_out, int64_t *k_out, size_t *out_bytes)
{
    if (!bytes || !n_out || !k_out || !out_bytes) return fail(TLB_ERR_NULL, "null argument");
    if (size < 1 || rank < 0 || rank >= size || kind < 0 || kind > 2) return fail(TLB_ERR_ARG, "shard %d of %d, kind %d", rank, size, kind);
    if (n < 0 || k < 0 || (k && n > INT64_MAX / k)) return fail(TLB_ERR_SHAPE, "bad shape");
    const size_t row_bytes = ggml_raw_nbytes(type, k);
    if ((k && !row_bytes) || row_bytes * (size_t)n != nbytes) return fail(TLB_ERR_SHAPE, "%zu bytes do not match type %d x [%lld, %lld]", nbytes, (int)type, (long long)n, (long long)k);
    int64_t sn = n, sk = k;
    if (kind == 1) {
        if (n % size) return fail(TLB_ERR_SHAPE, "%lld rows do not divide over %d ranks", (long long)n, size);
        sn = n / size;
    } else if (kind == 2) {
        if (k % size || (k && !ggml_raw_nbytes(type, k / size)))
            return fail(TLB_ERR_SHAPE, "%lld columns of GGML type %d do not divide into whole blocks over %d ranks", (long long)k, (int)type, size);
        sk = k / size;
    }
    const size_t shard_row = ggml_raw_nbytes(type, sk), total = shard_row * (size_t)sn;
    *n_out = sn; *k_out = sk; *out_bytes = total;
    if (!out) return TLB_OK;                       // size query
    if (out_cap < total) return fail(TLB_ERR_ARG, "shard needs %zu bytes, buffer holds %zu", total, out_cap);
    const uint8_t *src = (const uint8_t *)bytes;
    if (kind == 2) {
        for (int64_t r = 0; r < n; r++) memcpy((uint8_t *)out + (size_t)r * shard_row, src + (size_t)r * row_bytes + (size_t)rank * shard_row, shard_row);
    } else {
        memcpy(out, src + (kind == 1 ? (size_t)rank * total : 0), total);
    }
    return TLB_OK;
}

tlb_status tlb_map_add_tp(tlb_map *m, const char *name, tlb_ggml_type type, const int64_t *shape, int rank, const void *bytes, size_t nbytes,
                          int tp_rank, int tp_size)
{
    if (!m || !name || (rank > 0 && !shape)) return fail(TLB_ERR_NULL, "null argument");
    const int kind = rank == 2 ? tlb_tp_split_kind(name) : 0;
    if (kind == 0 || tp_size <= 1) return tlb_map_add(m, name, type, shape, rank, bytes, nbytes);
    int64_t sn = 0, sk = 0;
    size_t sb = 0;
    TLB_TRY(tlb_tp_shard_bytes(kind, type, shape[0], shape[1], bytes, nbytes, tp_rank, tp_size, nullptr, 0, &sn, &sk, &sb));
    const int64_t sshape[2] = {sn, sk};
    if (kind == 1) {   // a contiguous byte range: no copy
        return tlb_map_add(m, name, type, sshape, 2, (const uint8_t *)bytes + (size_t)tp_rank * sb, sb);
    }
    std::vector<uint8_t> tmp(sb);
    TLB_TRY(tlb_tp_shard_bytes(kind, type, shape[0], shape[1], bytes, nbytes, tp_rank, tp_size, tmp.data(), tmp.size(), &sn, &sk, &sb));
    return tlb_map_add(m, name, type, sshape, 2, tmp.data(), sb);
}

tlb_status tlb_map_free(tlb_map *m)
{
    if (!m) return TLB_OK;
    for (auto &kv : m->entries) {
        tlb_qtensor_release(kv.second.q);
        tlb_tensor_release(kv.second.f32);
    }
    delete m;
    return TLB_OK;
}

int64_t tlb_map_count(const tlb_map *m) { return m ? (int64_t)m->names.size() : -1; }

const char *tlb_map_name(const tlb_map *m, int64_t i)
{
    return (m && i >= 0 && i < (int64_t)m->names.size()) ? m->names[(size_t)i].c_str() : nullptr;
}

tlb_status tlb_map_get_quantized(tlb_qtensor **out, tlb_map *m, const char *name)
{
    if (!out) return fail(TLB_ERR_NULL, "null out");
    *out = nullptr;
    if (!m || !name) return fail(TLB_ERR_NULL, "null argument");
    auto it = m->entries.find(name);
    if (it == m->entries.end()) return fail(TLB_ERR_ARG, "Tensor '%s' not found in map", name);
    MapEntry &e = it->second;
    if (!e.q) {
        // F32 / F16 tensor: the reference wraps any type in a QTensor (tensor_map.rs:279) and multiplies it through the
        // dequantise + matmul route (system.rs:236-264).  The dense QTensor shares the f32 data the map already holds.
        if (e.shape.empty()) return fail(TLB_ERR_SHAPE, "Tensor '%s' is a scalar", name);
        tlb_qtensor *q = new tlb_qtensor();
        q->type = e.type;
        q->k = e.shape.back();
        q->n = q->k ? e.f32->numel() / q->k : 0;
        int64_t shp[2] = {q->n, q->k};
        tlb_status st = new_view(&q->dense, e.f32, shp, 2, 0);
        if (st != TLB_OK) { delete q; return st; }
        e.q = q;
    }
    tlb_qtensor_retain(e.q);
    *out = e.q;
    return TLB_OK;
}

tlb_status tlb_map_get(tlb_tensor **out, tlb_map *m, const char *name)
{
    if (!out) return fail(TLB_ERR_NULL, "null out");
    *out = nullptr;
    if (!m || !name) return fail(TLB_ERR_NULL, "null argument");
    auto it = m->entries.find(name);
    if (it == m->entries.end()) return fail(TLB_ERR_ARG, "Tensor '%s' not found in map", name);
    MapEntry &e = it->second;
    if (!e.f32) {   // cached, as QTensor::cache does
        tlb_tensor *d = nullptr;
        TLB_TRY(tlb_qtensor_dequantize(&d, e.q));
        tlb_status st = new_view(&e.f32, d, e.shape.data(), (int)e.shape.size(), 0);   // the tensor's own shape (1-D stays 1-D)
        tlb_tensor_release(d);
        TLB_TRY(st);
    }
    tlb_tensor_retain(e.f32);
    *out = e.f32;
    return TLB_OK;
}

/* ---- KV cache handle table ---- */

tlb_status tlb_kvcache_new(tlb_kvcache **out, int64_t layers)
{
    if (!out) return fail(TLB_ERR_NULL, "null out");
    *out = nullptr;
    if (layers < 0) return fail(TLB_ERR_ARG, "negative layer count");
    tlb_kvcache *c = new tlb_kvcache();
    c->layers.assign((size_t)layers, {nullptr, nullptr});
    *out = c;
    return TLB_OK;
}

tlb_status tlb_kvcache_clear(tlb_kvcache *c)
{
    if (!c) return fail(TLB_ERR_NULL, "null cache");
    for (auto &l : c->layers) {
        tlb_tensor_release(l.first);
        tlb_tensor_release(l.second);
        l = {nullptr, nullptr};
    }
    return TLB_OK;
}

tlb_status tlb_kvcache_free(tlb_kvcache *c)
{
    if (!c) return TLB_OK;
    tlb_kvcache_clear(c);
    delete c;
    return TLB_OK;
}

int64_t tlb_kvcache_len(const tlb_kvcache *c) { return c ? (int64_t)c->layers.size() : -1; }

tlb_status tlb_kvcache_resize(tlb_kvcache *c, int64_t layers)
{
    if (!c) return fail(TLB_ERR_NULL, "null cache");
    if (layers < 0) return fail(TLB_ERR_ARG, "negative layer count");
    for (size_t i = (size_t)layers; i < c->layers.size(); i++) {
        tlb_tensor_release(c->layers[i].first);
        tlb_tensor_release(c->layers[i].second);
    }
    c->layers.resize((size_t)layers, {nullptr, nullptr});
    return TLB_OK;
}

static tlb_status kv_get(tlb_tensor **out, tlb_kvcache *c, int64_t layer, bool want_v)
{
    if (!out) return fail(TLB_ERR_NULL, "null out");
    *out = nullptr;
    if (!c) return fail(TLB_ERR_NULL, "null cache");
    if (layer < 0 || layer >= (int64_t)c->layers.size()) return fail(TLB_ERR_INDEX, "KV cache layer %lld out of range", (long long)layer);
    tlb_tensor *t = want_v ? c->layers[(size_t)layer].second : c->layers[(size_t)layer].first;
    if (!t) return fail(TLB_ERR_NULL, "KV cache layer %lld is empty", (long long)layer);
    tlb_tensor_retain(t);  // the caller owns one reference (system.rs:513-553)
    *out = t;
    return TLB_OK;
}

tlb_status tlb_kvcache_get_k(tlb_tensor **out, tlb_kvcache *c, int64_t layer) { return kv_get(out, c, layer, false); }
tlb_status tlb_kvcache_get_v(tlb_tensor **out, tlb_kvcache *c, int64_t layer) { return kv_get(out, c, layer, true); }

tlb_status tlb_kvcache_update(tlb_kvcache *c, int64_t layer, tlb_tensor *k, tlb_tensor *v)
{
    if (!c || !k || !v) return fail(TLB_ERR_NULL, "null argument");
    if (layer < 0) return fail(TLB_ERR_INDEX, "negative layer");
    if (layer >= (int64_t)c->layers.size()) c->layers.resize((size_t)layer + 1, {nullptr, nullptr});  // grows on demand (system.rs:555-580)
    tlb_tensor_retain(k);
    tlb_tensor_retain(v);
    tlb_tensor_release(c->layers[(size_t)layer].first);
    tlb_tensor_release(c->layers[(size_t)layer].second);
    c->layers[(size_t)layer] = {k, v};
    return TLB_OK;
}

}  // extern "C"
