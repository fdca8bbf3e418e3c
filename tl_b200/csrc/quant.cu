// Quantized-weight storage: one-time repack of GGUF blocks into the tiled device layout,
// and the bit-exact dequantiser.
//
// Tiled layout.  A row-major [n, k] GGUF tensor is cut into UNITS of 16 rows x 256 weights,
// stored [n/16][k/256][unit]; a unit holds exactly the bytes of its 16 x 256 weights
// (Q4_K / Q4_0: 2304 B, Q8_0: 4352 B, Q6_K: 3360 B), so HBM traffic equals the GGUF byte
// count.  Inside a unit the quant bytes are arranged so that lane (r = lane/4, c = lane%4) of a
// warp - which owns rows r and r+8 of the tile in the m16n8k16 MMA fragment layout - finds
// everything it consumes in consecutive 16-byte pieces at piece*512 + lane*16: every shared
// memory read is a conflict-free 128-bit load and every unit is one contiguous bulk copy.
// Per-row headers (scales, d, dmin) follow the quant pieces, 16 bytes per row.
//
// unit_offset() is the single definition of the layout (raw byte of a row's 256-weight
// segment -> byte offset in the unit); the repack kernel scatters through it and the
// dequantiser gathers through it, so a round trip through both proves the layout lossless.
#include "qlayout.cuh"
#include "tlb_internal.h"

#include <algorithm>

namespace tlb {

static const QFormat kFormats[] = {
    {TLB_GGML_Q4_0, 2304, 32, 18},
    {TLB_GGML_Q8_0, 4352, 32, 34},
    {TLB_GGML_Q4_K, 2304, 256, 144},
    {TLB_GGML_Q6_K, 3360, 256, 210},
};

const QFormat *qformat(int t)
{
    for (const QFormat &f : kFormats)
        if (f.type == t) return &f;
    return nullptr;
}

// one thread per raw byte
__global__ void repack_kernel(int type, const uint8_t *__restrict__ raw, uint8_t *__restrict__ tiled,
                              int64_t n, int64_t k, int seg_bytes, int unit_bytes)
{
    int64_t upt = k / 256;
    int64_t total = n * upt * seg_bytes;
    for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        int raw_off = (int)(idx % seg_bytes);
        int64_t seg = idx / seg_bytes;  // row * upt + u
        int64_t row = seg / upt, u = seg % upt;
        int64_t tile = row / 16;
        int i = (int)(row % 16);
        tiled[(tile * upt + u) * unit_bytes + unit_offset(type, i, raw_off)] = raw[idx];
    }
}

tlb_status launch_repack(int type, const uint8_t *raw, uint8_t *tiled, int64_t n, int64_t k)
{
    const QFormat *f = qformat(type);
    if (!f) return fail(TLB_ERR_TYPE, "unsupported GGML type %d", type);
    int seg = 256 / f->raw_block * f->raw_block_bytes;
    int64_t total = n * (k / 256) * seg;
    if (total == 0) return TLB_OK;
    int blocks = (int)std::min<int64_t>((total + 255) / 256, 148 * 64);
    repack_kernel<<<blocks, 256, 0, ctx()->stream>>>(type, raw, tiled, n, k, seg, f->unit_bytes);
    count_launch();
    TLB_CUDA(cudaGetLastError());
    return TLB_OK;
}

// Builds, from two tiled tensors a and b of equal shape [n, k], the tiled tensor of 2n rows whose
// tile t holds rows 8t..8t+7 of a followed by rows 8t..8t+7 of b.  The decode chain uses it for
// gate | up: one MMA tile then yields gate and up of the same 8 hidden units, so SiLU(gate) * up
// can be taken where the tile is finished.  One thread per byte of a row segment.
__global__ void interleave8_kernel(int type, const uint8_t *__restrict__ a, const uint8_t *__restrict__ b,
                                   uint8_t *__restrict__ dst, int64_t n, int64_t k, int seg_bytes, int unit_bytes)
{
    const int64_t upt = k / 256;
    const int64_t total = 2 * n * upt * seg_bytes;
    for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int raw_off = (int)(idx % seg_bytes);
        const int64_t seg = idx / seg_bytes;          // drow * upt + u
        const int64_t drow = seg / upt, u = seg % upt;
        const int64_t dtile = drow / 16;
        const int di = (int)(drow % 16);
        const int64_t srow = dtile * 8 + (di & 7);     // row of a (di < 8) or b (di >= 8)
        const uint8_t *src = di < 8 ? a : b;
        dst[(dtile * upt + u) * unit_bytes + unit_offset(type, di, raw_off)] =
            src[((srow / 16) * upt + u) * unit_bytes + unit_offset(type, (int)(srow % 16), raw_off)];
    }
}

tlb_status launch_interleave8(int type, const uint8_t *a, const uint8_t *b, uint8_t *dst, int64_t n, int64_t k)
{
    const QFormat *f = qformat(type);
    if (!f) return fail(TLB_ERR_TYPE, "unsupported GGML type %d", type);
    if (n % 16) return fail(TLB_ERR_SHAPE, "interleaving needs a row count that is a multiple of 16, got %lld", (long long)n);
    int seg = 256 / f->raw_block * f->raw_block_bytes;
    int64_t total = 2 * n * (k / 256) * seg;
    if (total == 0) return TLB_OK;
    int blocks = (int)std::min<int64_t>((total + 255) / 256, 148 * 64);
    interleave8_kernel<<<blocks, 256, 0, ctx()->stream>>>(type, a, b, dst, n, k, seg, f->unit_bytes);
    count_launch();
    TLB_CUDA(cudaGetLastError());
    return TLB_OK;
}

// ---- bit-exact dequantisation ------------------------------------------------------------
// Expression shapes follow crates/tl_runtime/src/quantized.rs:182-415 exactly: separate
// f32 multiplies and subtracts (__fmul_rn / __fsub_rn are never contracted into an FMA).

__device__ __forceinline__ float f16_bits_to_f32(uint32_t lo, uint32_t hi)
{
    return __half2float(__ushort_as_half((unsigned short)(lo | (hi << 8))));
}

// one thread per 32 weights
__global__ void dequant_tiled_kernel(int type, const uint8_t *__restrict__ tiled, float *__restrict__ out,
                                     int64_t n, int64_t k, int unit_bytes)
{
    int64_t upt = k / 256;
    int64_t total = n * (k / 32);
    for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        int64_t row = idx / (k / 32);
        int64_t kb = idx % (k / 32);  // 32-weight block index within the row
        int64_t u = kb / 8;
        int sb = (int)(kb % 8);       // 32-block within the 256 segment
        const uint8_t *up = tiled + ((row / 16) * upt + u) * unit_bytes;
        int i = (int)(row % 16);
        float *o = out + row * k + kb * 32;
#define RB(off) ((uint32_t)up[unit_offset(type, i, (off))])
        if (type == TLB_GGML_Q4_0) {
            int base = sb * 18;
            float d = f16_bits_to_f32(RB(base), RB(base + 1));
            for (int j = 0; j < 16; j++) {
                uint32_t b = RB(base + 2 + j);
                o[j] = __fmul_rn(d, (float)((int)(b & 15) - 8));
                o[j + 16] = __fmul_rn(d, (float)((int)(b >> 4) - 8));
            }
        } else if (type == TLB_GGML_Q8_0) {
            int base = sb * 34;
            float d = f16_bits_to_f32(RB(base), RB(base + 1));
            for (int j = 0; j < 32; j++) o[j] = __fmul_rn(d, (float)(int8_t)RB(base + 2 + j));
        } else if (type == TLB_GGML_Q4_K) {
            float d = f16_bits_to_f32(RB(0), RB(1));
            float dmin = f16_bits_to_f32(RB(2), RB(3));
            int j = sb;  // sub-block index 0..7 (get_scale_min_k4, quantized.rs:404-415)
            uint32_t sc, mn;
            if (j < 4) {
                sc = RB(4 + j) & 63;
                mn = RB(4 + j + 4) & 63;
            } else {
                sc = (RB(4 + j + 4) & 0xF) | ((RB(4 + j - 4) >> 6) << 4);
                mn = (RB(4 + j + 4) >> 4) | ((RB(4 + j) >> 6) << 4);
            }
            float d1 = __fmul_rn(d, (float)sc), m1 = __fmul_rn(dmin, (float)mn);
            int qoff = 16 + (sb / 2) * 32;
            int hi = sb & 1;
            for (int l = 0; l < 32; l++) {
                uint32_t b = RB(qoff + l);
                uint32_t q = hi ? (b >> 4) : (b & 15);
                o[l] = __fsub_rn(__fmul_rn(d1, (float)q), m1);
            }
        } else {  // Q6_K: 32-block sb covers k = 32*sb .. 32*sb+31 -> chunk n = sb/4, quarter = sb%4
            float d = f16_bits_to_f32(RB(208), RB(209));
            int nch = sb / 4, quarter = sb % 4;
            for (int l = 0; l < 32; l++) {
                uint32_t qlb = RB(64 * nch + (quarter & 1) * 32 + l);
                uint32_t qhb = RB(128 + 32 * nch + l);
                uint32_t lo4 = (quarter >> 1) ? (qlb >> 4) : (qlb & 15);
                int q = (int)(lo4 | (((qhb >> (2 * quarter)) & 3) << 4)) - 32;
                float sc = (float)(int8_t)RB(192 + 8 * nch + l / 16 + 2 * quarter);
                o[l] = __fmul_rn(__fmul_rn(d, sc), (float)q);
            }
        }
#undef RB
    }
}

tlb_status launch_dequant_tiled(int type, const uint8_t *tiled, float *out, int64_t n, int64_t k)
{
    const QFormat *f = qformat(type);
    if (!f) return fail(TLB_ERR_TYPE, "unsupported GGML type %d", type);
    int64_t total = n * (k / 32);
    if (total == 0) return TLB_OK;
    int blocks = (int)std::min<int64_t>((total + 127) / 128, 148 * 32);
    dequant_tiled_kernel<<<blocks, 128, 0, ctx()->stream>>>(type, tiled, out, n, k, f->unit_bytes);
    count_launch();
    TLB_CUDA(cudaGetLastError());
    return TLB_OK;
}

// ---- raw GGUF blocks -> f32 (dense tensors) -------------------------------------------------
// The same expressions as above on the untiled bytes, plus the block types the tiled kernels do not take.
// Q4_1 / Q5_0 / Q5_1 / Q8_1 have no dequantiser in the reference (crates/tl_runtime/src/quantized.rs:108); they
// follow the published GGML block definitions: integer to f32, one multiply, then one add, never fused.
size_t ggml_raw_nbytes(int type, int64_t nelem)
{
    if (nelem < 0) return 0;
    auto blocks = [&](int per, int bytes) -> size_t { return nelem % per ? 0 : (size_t)(nelem / per) * bytes; };
    switch (type) {
    case TLB_GGML_F32: return (size_t)nelem * 4;
    case TLB_GGML_F16: return (size_t)nelem * 2;
    case TLB_GGML_Q4_0: return blocks(32, 18);
    case TLB_GGML_Q4_1: return blocks(32, 20);
    case TLB_GGML_Q5_0: return blocks(32, 22);
    case TLB_GGML_Q5_1: return blocks(32, 24);
    case TLB_GGML_Q8_0: return blocks(32, 34);
    case TLB_GGML_Q8_1: return blocks(32, 36);
    case TLB_GGML_Q4_K: return blocks(256, 144);
    case TLB_GGML_Q6_K: return blocks(256, 210);
    default: return 0;
    }
}

// one thread per 32 weights
__global__ void dequant_raw_kernel(int type, const uint8_t *__restrict__ raw, float *__restrict__ out, int64_t nelem)
{
    const int64_t total = nelem / 32;
    for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        float *o = out + idx * 32;
        if (type == TLB_GGML_F32) {
            for (int j = 0; j < 32; j++) o[j] = reinterpret_cast<const float *>(raw)[idx * 32 + j];
        } else if (type == TLB_GGML_F16) {
            for (int j = 0; j < 32; j++) o[j] = __half2float(reinterpret_cast<const __half *>(raw)[idx * 32 + j]);
        } else if (type == TLB_GGML_Q4_0) {
            const uint8_t *p = raw + idx * 18;
            const float d = f16_bits_to_f32(p[0], p[1]);
            for (int j = 0; j < 16; j++) {
                o[j] = __fmul_rn(d, (float)((int)(p[2 + j] & 15) - 8));
                o[j + 16] = __fmul_rn(d, (float)((int)(p[2 + j] >> 4) - 8));
            }
        } else if (type == TLB_GGML_Q8_0) {
            const uint8_t *p = raw + idx * 34;
            const float d = f16_bits_to_f32(p[0], p[1]);
            for (int j = 0; j < 32; j++) o[j] = __fmul_rn(d, (float)(int8_t)p[2 + j]);
        } else if (type == TLB_GGML_Q8_1) {
            const uint8_t *p = raw + idx * 36;
            const float d = f16_bits_to_f32(p[0], p[1]);
            for (int j = 0; j < 32; j++) o[j] = __fmul_rn(d, (float)(int8_t)p[4 + j]);
        } else if (type == TLB_GGML_Q4_1) {
            const uint8_t *p = raw + idx * 20;
            const float d = f16_bits_to_f32(p[0], p[1]), m = f16_bits_to_f32(p[2], p[3]);
            for (int j = 0; j < 16; j++) {
                o[j] = __fadd_rn(__fmul_rn(d, (float)(p[4 + j] & 15)), m);
                o[j + 16] = __fadd_rn(__fmul_rn(d, (float)(p[4 + j] >> 4)), m);
            }
        } else if (type == TLB_GGML_Q5_0 || type == TLB_GGML_Q5_1) {
            const bool with_min = type == TLB_GGML_Q5_1;
            const uint8_t *p = raw + idx * (with_min ? 24 : 22);
            const float d = f16_bits_to_f32(p[0], p[1]), m = with_min ? f16_bits_to_f32(p[2], p[3]) : 0.f;
            const uint8_t *qhp = p + (with_min ? 4 : 2), *qs = qhp + 4;
            const uint32_t qh = (uint32_t)qhp[0] | ((uint32_t)qhp[1] << 8) | ((uint32_t)qhp[2] << 16) | ((uint32_t)qhp[3] << 24);
            for (int j = 0; j < 16; j++) {
                const int x0 = (int)(qs[j] & 15) | (int)(((qh >> j) & 1u) << 4);
                const int x1 = (int)(qs[j] >> 4) | (int)(((qh >> (j + 16)) & 1u) << 4);
                if (with_min) {
                    o[j] = __fadd_rn(__fmul_rn(d, (float)x0), m);
                    o[j + 16] = __fadd_rn(__fmul_rn(d, (float)x1), m);
                } else {
                    o[j] = __fmul_rn(d, (float)(x0 - 16));
                    o[j + 16] = __fmul_rn(d, (float)(x1 - 16));
                }
            }
        }
    }
}

tlb_status launch_dequant_raw(int type, const uint8_t *raw, float *out, int64_t nelem)
{
    if (type == TLB_GGML_Q4_K || type == TLB_GGML_Q6_K) return fail(TLB_ERR_TYPE, "K-quants are dequantised from the tiled layout");
    if (nelem % 32) return fail(TLB_ERR_SHAPE, "dense dequantisation works on whole blocks of 32");
    if (nelem == 0) return TLB_OK;
    const int64_t total = nelem / 32;
    const int blocks = (int)std::min<int64_t>((total + 127) / 128, 148 * 32);
    dequant_raw_kernel<<<blocks, 128, 0, ctx()->stream>>>(type, raw, out, nelem);
    count_launch();
    TLB_CUDA(cudaGetLastError());
    return TLB_OK;
}

}  // namespace tlb

using namespace tlb;

// A dense QTensor: the bytes go up once, are dequantised to f32 [n, k] and dropped.
static tlb_status qtensor_dense(tlb_qtensor **out, int type, int64_t n, int64_t k, const void *bytes, size_t nbytes)
{
    const int64_t nelem = n * k;
    const size_t need = ggml_raw_nbytes(type, nelem);
    if (nelem && !need) return fail(TLB_ERR_SHAPE, "K = %lld does not hold whole blocks of GGML type %d", (long long)k, type);
    if (type != TLB_GGML_F32 && type != TLB_GGML_F16 && k % 32) return fail(TLB_ERR_SHAPE, "K = %lld must be a multiple of 32 for GGML type %d", (long long)k, type);
    if (nbytes != need) return fail(TLB_ERR_SHAPE, "data size mismatch: expected %zu bytes, got %zu", need, nbytes);
    if (need && !bytes) return fail(TLB_ERR_NULL, "null data");
    tlb_qtensor *q = new tlb_qtensor();
    q->type = type; q->n = n; q->k = k;
    int64_t shape[2] = {n, k};
    tlb_status st = new_tensor(&q->dense, TLB_F32, shape, 2);
    if (st == TLB_OK && need) {
        cudaStream_t s = ctx()->stream;
        if (type == TLB_GGML_F32) {
            cudaError_t e = cudaMemcpyAsync(q->dense->data(), bytes, need, cudaMemcpyHostToDevice, s);
            if (e == cudaSuccess) e = cudaStreamSynchronize(s);
            if (e != cudaSuccess) st = cuda_fail(e, "qtensor upload");
        } else if (nelem % 32) {     // F16 with a ragged element count: widened on the host (exact)
            std::vector<float> w((size_t)nelem);
            for (int64_t i = 0; i < nelem; i++) w[(size_t)i] = __half2float(reinterpret_cast<const __half *>(bytes)[i]);
            cudaError_t e = cudaMemcpyAsync(q->dense->data(), w.data(), w.size() * 4, cudaMemcpyHostToDevice, s);
            if (e == cudaSuccess) e = cudaStreamSynchronize(s);
            if (e != cudaSuccess) st = cuda_fail(e, "qtensor upload");
        } else {
            void *tmp = nullptr;
            cudaError_t e = cudaMallocAsync(&tmp, need, s);
            if (e == cudaSuccess) e = cudaMemcpyAsync(tmp, bytes, need, cudaMemcpyHostToDevice, s);
            if (e == cudaSuccess) st = launch_dequant_raw(type, (const uint8_t *)tmp, q->dense->f32(), nelem);
            if (tmp) cudaFreeAsync(tmp, s);
            if (e == cudaSuccess) e = cudaStreamSynchronize(s);
            if (e != cudaSuccess) st = cuda_fail(e, "qtensor upload");
        }
    }
    if (st != TLB_OK) { tlb_tensor_release(q->dense); delete q; return st; }
    *out = q;
    return TLB_OK;
}

extern "C" {

tlb_status tlb_qtensor_from_gguf_bytes(tlb_qtensor **out, tlb_ggml_type type, int64_t n, int64_t k,
                                       const void *bytes, size_t nbytes)
{
    if (!out) return fail(TLB_ERR_NULL, "null out");
    *out = nullptr;
    if (!ensure_init()) return TLB_ERR_DEVICE;
    const QFormat *f = qformat(type);
    if (n < 0 || k < 0) return fail(TLB_ERR_SHAPE, "negative shape");
    const bool dense_type = type == TLB_GGML_F32 || type == TLB_GGML_F16 || type == TLB_GGML_Q4_1 || type == TLB_GGML_Q5_0 ||
                            type == TLB_GGML_Q5_1 || type == TLB_GGML_Q8_1;
    if (!f && !dense_type)
        return fail(TLB_ERR_TYPE, "GGML type %d is not supported (F32, F16, Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q8_1, Q4_K, Q6_K)", (int)type);
    if (dense_type || (k % 256 != 0 && f->raw_block == 32)) return qtensor_dense(out, type, n, k, bytes, nbytes);
    if (k % 256 != 0) return fail(TLB_ERR_SHAPE, "K = %lld must be a multiple of 256 for GGML type %d", (long long)k, (int)type);
    size_t need = (size_t)n * (k / f->raw_block) * f->raw_block_bytes;
    if (nbytes != need) return fail(TLB_ERR_SHAPE, "data size mismatch: expected %zu bytes, got %zu", need, nbytes);
    if (need && !bytes) return fail(TLB_ERR_NULL, "null data");
    tlb_qtensor *q = new tlb_qtensor();
    q->type = type;
    q->n = n;
    q->k = k;
    q->n_tiles = (n + 15) / 16;
    q->upt = k / 256;
    q->st = storage_alloc((size_t)q->n_tiles * q->upt * f->unit_bytes);   // nbytes() tells tiled from dense by `st`: not yet set
    if (!q->st) { delete q; return TLB_ERR_ALLOC; }
    if (need) {
        cudaStream_t s = ctx()->stream;
        void *tmp = nullptr;
        cudaError_t e = cudaMallocAsync(&tmp, need, s);
        if (e == cudaSuccess && (n % 16)) e = cudaMemsetAsync(q->st->ptr, 0, (size_t)q->nbytes(), s);
        if (e == cudaSuccess) e = cudaMemcpyAsync(tmp, bytes, need, cudaMemcpyHostToDevice, s);
        tlb_status st = TLB_OK;
        if (e == cudaSuccess) st = launch_repack(type, (const uint8_t *)tmp, q->dev(), n, k);
        if (tmp) cudaFreeAsync(tmp, s);
        if (e == cudaSuccess) e = cudaStreamSynchronize(s);  // the host bytes may go away after return
        if (e != cudaSuccess || st != TLB_OK) {
            storage_release(q->st);
            delete q;
            return e != cudaSuccess ? cuda_fail(e, "qtensor upload") : st;
        }
    }
    *out = q;
    return TLB_OK;
}

tlb_status tlb_qtensor_retain(tlb_qtensor *q)
{
    if (!q) return fail(TLB_ERR_NULL, "null qtensor");
    q->rc.fetch_add(1);
    return TLB_OK;
}

tlb_status tlb_qtensor_release(tlb_qtensor *q)
{
    if (!q) return TLB_OK;
    if (q->rc.fetch_sub(1) == 1) {
        if (q->st) storage_release(q->st);
        tlb_tensor_release(q->dense);
        tlb_tensor_release(q->dense_t);
        delete q;
    }
    return TLB_OK;
}

tlb_status tlb_qtensor_info(const tlb_qtensor *q, int *type, int64_t *n, int64_t *k, uint64_t *device_bytes)
{
    if (!q) return fail(TLB_ERR_NULL, "null qtensor");
    if (type) *type = q->type;
    if (n) *n = q->n;
    if (k) *k = q->k;
    if (device_bytes) *device_bytes = q->nbytes();
    return TLB_OK;
}

tlb_status tlb_qtensor_dequantize(tlb_tensor **out, const tlb_qtensor *q)
{
    if (!out || !q) return fail(TLB_ERR_NULL, "null argument");
    if (!q->tiled()) return tlb_tensor_clone(out, q->dense);
    int64_t shape[2] = {q->n, q->k};
    TLB_TRY(new_tensor(out, TLB_F32, shape, 2));
    tlb_status s = launch_dequant_tiled(q->type, q->dev(), (*out)->f32(), q->n, q->k);
    if (s != TLB_OK) { tlb_tensor_release(*out); *out = nullptr; }
    return s;
}

}  // extern "C"

/* layout introspection for tests: byte offset inside a unit of raw byte `raw_off` of row `row16` */
extern "C" int tlb_layout_unit_offset(int ggml_type, int row16, int raw_off)
{
    const QFormat *f = qformat(ggml_type);
    if (!f || row16 < 0 || row16 > 15 || raw_off < 0 || raw_off >= 256 / f->raw_block * f->raw_block_bytes) return -1;
    return unit_offset(ggml_type, row16, raw_off);
}
extern "C" int tlb_layout_unit_bytes(int ggml_type)
{
    const QFormat *f = qformat(ggml_type);
    return f ? f->unit_bytes : -1;
}
