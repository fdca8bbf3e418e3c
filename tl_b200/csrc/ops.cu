// Per-op entry points behind the reference's tensor FFI: elementwise, shape, softmax, f32 matmul,
// RMSNorm, RoPE, embedding, argmax / sampling.  These keep the reference's value semantics (every
// op returns a new tensor); the decode hot path does not go through them but through the fused
// chain in decoder.cu.  Kernels replaced: crates/tl_cuda/src/cuda_kernels/autograd.cu (lines per op).
#include "tlb_internal.h"

#include <cmath>

namespace tlb {

static inline int grid_for(int64_t n, int threads, int max_blocks = 148 * 16)
{
    int64_t b = (n + threads - 1) / threads;
    return (int)std::max<int64_t>(1, std::min<int64_t>(b, max_blocks));
}

struct Strides { int64_t o[kMaxRank], a[kMaxRank], b[kMaxRank]; int rank; };

enum { OP_ADD = 0, OP_MUL = 1 };
enum { UN_SILU = 0, UN_SCALE = 1 };

// add_kernel / mul_kernel (autograd.cu:185-201) with numpy broadcasting done by index arithmetic
// instead of materialising both operands (crates/tl_cuda/src/ops/binary.rs:136-155)
__global__ void binary_kernel(int op, const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ out,
                              Strides s, int64_t n)
{
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t rem = i, ia = 0, ib = 0;
        for (int d = s.rank - 1; d >= 0; d--) {
            int64_t c = rem % s.o[d];
            rem /= s.o[d];
            ia += c * s.a[d];
            ib += c * s.b[d];
        }
        float x = a[ia], y = b[ib];
        out[i] = op == OP_ADD ? x + y : x * y;
    }
}

__global__ void same_shape_binary_kernel(int op, const float *__restrict__ a, const float *__restrict__ b,
                                         float *__restrict__ out, int64_t n)
{
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = op == OP_ADD ? a[i] + b[i] : a[i] * b[i];
}

// silu_kernel (autograd.cu:317-321) in the CPU formulation x * (1 / (1 + exp(-x))) (crates/tl_cpu/src/ffi.rs:2102);
// mul_scalar_kernel (autograd.cu:151-155)
__global__ void unary_kernel(int op, const float *__restrict__ a, float *__restrict__ out, int64_t n, float s)
{
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        float x = a[i];
        out[i] = op == UN_SILU ? x * (1.0f / (1.0f + expf(-x))) : x * s;
    }
}

__global__ void silu_mul_kernel(const float *__restrict__ g, const float *__restrict__ u, float *__restrict__ out, int64_t n)
{
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        float x = g[i];
        out[i] = (x * (1.0f / (1.0f + expf(-x)))) * u[i];
    }
}
// the same on four elements per thread (16-byte aligned operands, n a multiple of 4); out may be g
__global__ void silu_mul4_kernel(const float4 *g, const float4 *u, float4 *out, int64_t n4)
{
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
        const float4 a = g[i], b = u[i];
        float4 o;
        o.x = (a.x * (1.0f / (1.0f + expf(-a.x)))) * b.x;
        o.y = (a.y * (1.0f / (1.0f + expf(-a.y)))) * b.y;
        o.z = (a.z * (1.0f / (1.0f + expf(-a.z)))) * b.z;
        o.w = (a.w * (1.0f / (1.0f + expf(-a.w)))) * b.w;
        out[i] = o;
    }
}

__device__ __forceinline__ float warp_sum(float v)
{
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v)
{
    for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ float block_sum(float v, float *sh)
{
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) sh[w] = v;
    __syncthreads();
    float t = 0.f;
    for (int i = 0; i < nw; i++) t += sh[i];
    return t;
}
__device__ float block_max(float v, float *sh)
{
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) sh[w] = v;
    __syncthreads();
    float t = -INFINITY;
    for (int i = 0; i < nw; i++) t = fmaxf(t, sh[i]);
    return t;
}

// softmax_kernel (autograd.cu:457-486: one thread per row, three passes) -> one block per row
__global__ void softmax_kernel(const float *__restrict__ a, float *__restrict__ out, int64_t axis, int64_t inner)
{
    __shared__ float sh[32];
    int64_t row = blockIdx.x;
    int64_t o = row / inner, k = row % inner;
    const float *x = a + o * axis * inner + k;
    float *y = out + o * axis * inner + k;
    float mx = -INFINITY;
    for (int64_t j = threadIdx.x; j < axis; j += blockDim.x) mx = fmaxf(mx, x[j * inner]);
    mx = block_max(mx, sh);
    float sum = 0.f;
    for (int64_t j = threadIdx.x; j < axis; j += blockDim.x) {
        float e = expf(x[j * inner] - mx);
        y[j * inner] = e;
        sum += e;
    }
    sum = block_sum(sum, sh);
    for (int64_t j = threadIdx.x; j < axis; j += blockDim.x) y[j * inner] = y[j * inner] / sum;
}

// matmul_naive_kernel (autograd.cu:430-450: one thread per output) -> 64x64 shared-memory tiles,
// 4x4 outputs per thread, f32 FMA.  Used by the per-op attention route (matmul_4d) only.
__global__ void __launch_bounds__(256) matmul_kernel(const float *__restrict__ A, const float *__restrict__ B,
                                                     float *__restrict__ C, int64_t m, int64_t k, int64_t n, int b_batched)
{
    __shared__ float As[16][64 + 4], Bs[16][64 + 4];
    const float *a = A + (int64_t)blockIdx.z * m * k;
    const float *b = B + (b_batched ? (int64_t)blockIdx.z * k * n : 0);
    float *c = C + (int64_t)blockIdx.z * m * n;
    int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    int64_t row0 = (int64_t)blockIdx.y * 64, col0 = (int64_t)blockIdx.x * 64;
    float acc[4][4] = {};
    for (int64_t k0 = 0; k0 < k; k0 += 16) {
        for (int i = threadIdx.x; i < 64 * 16; i += 256) {
            int rr = i >> 4, kk = i & 15;
            int64_t gr = row0 + rr, gk = k0 + kk;
            As[kk][rr] = (gr < m && gk < k) ? a[gr * k + gk] : 0.f;
            int kk2 = i >> 6, cc = i & 63;
            int64_t gk2 = k0 + kk2, gc = col0 + cc;
            Bs[kk2][cc] = (gk2 < k && gc < n) ? b[gk2 * n + gc] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; kk++) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; i++) { av[i] = As[kk][ty * 4 + i]; bv[i] = Bs[kk][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] += av[i] * bv[j];
        }
        __syncthreads();
    }
    for (int i = 0; i < 4; i++)
        for (int j = 0; j < 4; j++) {
            int64_t gr = row0 + ty * 4 + i, gc = col0 + tx * 4 + j;
            if (gr < m && gc < n) c[gr * n + gc] = acc[i][j];
        }
}

// narrow_kernel / cat_kernel / transpose_nd_kernel / repeat_interleave_kernel / broadcast_to_kernel
// (autograd.cu:743-776,1253-1299,781-799): one strided gather serves them all
__global__ void copy_strided_kernel(const float *__restrict__ a, float *__restrict__ out, Strides s, int64_t n, int64_t a_off)
{
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t rem = i, ia = a_off;
        for (int d = s.rank - 1; d >= 0; d--) {
            int64_t c = rem % s.o[d];
            rem /= s.o[d];
            ia += c * s.a[d];
        }
        out[i] = a[ia];
    }
}

// The same gather when the innermost output dimension is contiguous in the source as well (narrow, cat, repeat_interleave,
// transposes of outer dimensions): rows of `inner4` float4, the row's source offset from 32-bit index arithmetic.
struct RowStrides { unsigned o[kMaxRank]; long long a[kMaxRank]; int rank; };   // outer dimensions only
__global__ void copy_rows4_kernel(const float4 *__restrict__ a, float4 *__restrict__ out, RowStrides s, unsigned rows, unsigned inner4, long long a_off4)
{
    const unsigned long long total = (unsigned long long)rows * inner4;
    for (unsigned long long i = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x; i < total; i += (unsigned long long)gridDim.x * blockDim.x) {
        const unsigned row = (unsigned)(i / inner4), col = (unsigned)(i - (unsigned long long)row * inner4);
        unsigned rem = row;
        long long ia = a_off4;
        for (int d = s.rank - 1; d >= 0; d--) {
            const unsigned c = rem % s.o[d];
            rem /= s.o[d];
            ia += (long long)c * s.a[d];
        }
        out[i] = a[ia + col];
    }
}

// out[b][j][i] = a[b][i][j]: the last two dimensions exchanged, through a 32 x 33 shared-memory tile so that both the
// reads and the writes are coalesced.
__global__ void __launch_bounds__(256) transpose_last2_kernel(const float *__restrict__ a, float *__restrict__ out, int rows, int cols)
{
    __shared__ float tile[32][33];
    const float *src = a + (size_t)blockIdx.z * rows * cols;
    float *dst = out + (size_t)blockIdx.z * rows * cols;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;       // 32 x 8
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    for (int j = ty; j < 32; j += 8)
        if (r0 + j < rows && c0 + tx < cols) tile[j][tx] = src[(size_t)(r0 + j) * cols + c0 + tx];
    __syncthreads();
    for (int j = ty; j < 32; j += 8)
        if (c0 + j < cols && r0 + tx < rows) dst[(size_t)(c0 + j) * rows + r0 + tx] = tile[tx][j];
}

// C[b][r][n] = sum_k A[b][r][k] B[b][k][n] for up to 4 rows r (the decode step's attention products: one query row per
// head against the whole cache).  COLS columns x 512 / COLS slices of k per CTA; the slices are added in index order.
// Wide results take 64 columns per CTA; narrow ones (P.V: 128 columns, thousands of k) take 16, so that there are enough
// CTAs and each thread's share of k stays short.
template <int COLS>
__global__ void __launch_bounds__(512) matmul_rows_kernel(const float *__restrict__ A, const float *__restrict__ B, float *__restrict__ C,
                                                          int m, int k, int n, int b_batched)
{
    constexpr int SL = 512 / COLS;
    __shared__ float red[SL][4][COLS];
    const float *a = A + (size_t)blockIdx.y * m * k;
    const float *b = B + (b_batched ? (size_t)blockIdx.y * k * n : 0);
    const int tx = threadIdx.x % COLS, ks = threadIdx.x / COLS, col = blockIdx.x * COLS + tx;
    const int kc = (k + SL - 1) / SL, k0 = ks * kc, k1 = min(k, k0 + kc);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    if (col < n) {
        for (int kk = k0; kk < k1; kk++) {
            const float bv = b[(size_t)kk * n + col];
#pragma unroll
            for (int r = 0; r < 4; r++)
                if (r < m) acc[r] = fmaf(__ldg(a + (size_t)r * k + kk), bv, acc[r]);
        }
    }
#pragma unroll
    for (int r = 0; r < 4; r++) red[ks][r][tx] = acc[r];
    __syncthreads();
    if (ks < m && col < n) {       // slices 0 .. m-1 each finish one row
        float v = red[0][ks][tx];
        for (int q = 1; q < SL; q++) v += red[q][ks][tx];
        C[((size_t)blockIdx.y * m + ks) * n + col] = v;
    }
}

__global__ void copy_into_kernel(const float *__restrict__ a, float *__restrict__ out, int64_t outer, int64_t a_inner,
                                 int64_t o_inner, int64_t o_off)
{
    int64_t n = outer * a_inner;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[(i / a_inner) * o_inner + o_off + i % a_inner] = a[i];
}

// rms_norm_kernel + mul_kernel (autograd.cu:612-627, two launches, one thread per row) and
// fused_add_rms_norm_kernel (autograd.cu:2508-2525) -> one block per row, weight and residual fused.
// x / sqrt(mean(x^2) + eps) then * w, in the CPU back end's operation order.
__global__ void rms_norm_kernel(const float *__restrict__ x, const float *__restrict__ res, const float *__restrict__ w,
                                float eps, float *__restrict__ out, int64_t d)
{
    __shared__ float sh[32];
    const float *xr = x + (int64_t)blockIdx.x * d;
    const float *rr = res ? res + (int64_t)blockIdx.x * d : nullptr;
    float *o = out + (int64_t)blockIdx.x * d;
    float ss = 0.f;
    for (int64_t i = threadIdx.x; i < d; i += blockDim.x) {
        float v = xr[i] + (rr ? rr[i] : 0.f);
        ss += v * v;
    }
    ss = block_sum(ss, sh);
    float rms = sqrtf(ss / (float)d + eps);
    for (int64_t i = threadIdx.x; i < d; i += blockDim.x) {
        float v = xr[i] + (rr ? rr[i] : 0.f);
        float y = __fdiv_rn(v, rms);
        o[i] = w ? y * w[i] : y;
    }
}

// crates/tl_cpu/src/ffi.rs:2629-2685: adjacent pairs, table row 0 for every vector
__global__ void rope_cpu_kernel(const float *__restrict__ x, const float *__restrict__ cos_t, const float *__restrict__ sin_t,
                                int64_t tab_len, float *__restrict__ out, int64_t npairs, int64_t d)
{
    for (int64_t p = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; p < npairs; p += (int64_t)gridDim.x * blockDim.x) {
        int64_t v = p / (d / 2), i = (p % (d / 2)) * 2;
        float c = i < tab_len ? cos_t[i] : 1.0f, s = i < tab_len ? sin_t[i] : 0.0f;
        float x0 = x[v * d + i], x1 = x[v * d + i + 1];
        out[v * d + i] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
        out[v * d + i + 1] = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
    }
}

// apply_rope_kernel (autograd.cu:1196-1227): rotate-half, one table row per token
__global__ void rope_half_kernel(const float *__restrict__ x, const float *__restrict__ cos_t, const float *__restrict__ sin_t,
                                 float *__restrict__ out, int64_t tokens, int64_t heads, int64_t d)
{
    int64_t half = d / 2, n = tokens * heads * half;
    for (int64_t p = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; p < n; p += (int64_t)gridDim.x * blockDim.x) {
        int64_t i = p % half, vh = p / half, t = vh / heads;
        float c = cos_t[t * half + i], s = sin_t[t * half + i];
        float x0 = x[vh * d + i], x1 = x[vh * d + i + half];
        out[vh * d + i] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
        out[vh * d + i + half] = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
    }
}

// embedding_f32_kernel (autograd.cu:66-81); an out-of-range id raises a flag (the CPU back end
// errors, crates/tl_cpu/src/tensor.rs:1094-1112; the CUDA one silently writes zeros)
__global__ void embedding_kernel(const float *__restrict__ table, const float *__restrict__ idx, float *__restrict__ out,
                                 int64_t n, int64_t vocab, int64_t dim, int *oob)
{
    int64_t total = n * dim;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t r = i / dim, id = (int64_t)idx[r];
        if (id < 0 || id >= vocab) {
            if (i % dim == 0) atomicExch(oob, 1);
            out[i] = 0.f;
        } else {
            out[i] = table[id * dim + i % dim];
        }
    }
}

// argmax_all_kernel (autograd.cu:1119-1132: a single thread) -> block reduction; `tie_first`
// selects the CUDA kernel's first-maximum rule, otherwise tl_cpu's last-maximum rule.
__device__ __forceinline__ bool better(float v, int64_t i, float bv, int64_t bi, int tie_first)
{
    if (bi < 0) return true;
    if (v > bv) return true;
    if (v < bv) return false;
    if (v != v || bv != bv) return tie_first ? false : i > bi;  // NaN compares Equal in the reference
    return tie_first ? i < bi : i > bi;
}

__global__ void argmax_partial_kernel(const float *__restrict__ x, int64_t n, int tie_first, float *pv, long long *pi)
{
    __shared__ float sv[32];
    __shared__ long long si[32];
    float bv = 0.f;
    int64_t bi = -1;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        float v = x[i];
        if (better(v, i, bv, bi, tie_first)) { bv = v; bi = i; }
    }
    for (int o = 16; o; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        long long oi = __shfl_xor_sync(0xffffffffu, (long long)bi, o);
        if (oi >= 0 && better(ov, oi, bv, bi, tie_first)) { bv = ov; bi = oi; }
    }
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    if (lane == 0) { sv[w] = bv; si[w] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < (int)(blockDim.x >> 5); i++)
            if (si[i] >= 0 && better(sv[i], si[i], bv, bi, tie_first)) { bv = sv[i]; bi = si[i]; }
        pv[blockIdx.x] = bv;
        pi[blockIdx.x] = bi;
    }
}

__global__ void argmax_final_kernel(const float *pv, const long long *pi, int nparts, int tie_first, float *out_f32, int *out_i32)
{
    if (threadIdx.x == 0) {
        float bv = 0.f;
        int64_t bi = -1;
        for (int i = 0; i < nparts; i++)
            if (pi[i] >= 0 && better(pv[i], pi[i], bv, bi, tie_first)) { bv = pv[i]; bi = pi[i]; }
        if (bi < 0) bi = 0;
        if (out_f32) *out_f32 = (float)bi;
        if (out_i32) *out_i32 = (int)bi;
    }
}

__global__ void causal_mask_kernel(float *out, int64_t size)
{
    int64_t n = size * size;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = (i % size > i / size) ? -INFINITY : 0.f;
}

// repetition_penalty_kernel (autograd.cu:2449-2471): each seen id penalised ONCE
// (crates/tl_cpu/src/device_impl.rs:967-1000 dedups the token list)
__global__ void rep_penalty_kernel(float *logits, const float *tokens, int64_t rows, int64_t vocab, int64_t nt, float p)
{
    for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < nt; t += (int64_t)gridDim.x * blockDim.x) {
        float tf = tokens[t];
        int64_t id = tf < 0.f ? 0 : (int64_t)tf;
        if (id >= vocab) continue;
        bool first = true;  // only the first occurrence of an id applies the penalty
        for (int64_t u = 0; u < t; u++) {
            float uf = tokens[u];
            int64_t ui = uf < 0.f ? 0 : (int64_t)uf;
            if (ui == id) { first = false; break; }
        }
        if (!first) continue;
        for (int64_t r = 0; r < rows; r++) {
            float v = logits[r * vocab + id];
            logits[r * vocab + id] = v > 0.f ? v / p : v * p;
        }
    }
}

__global__ void f32_to_f16_kernel(const float *a, __half *out, int64_t n)
{
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = __float2half_rn(a[i]);
}

#define LAUNCH_CHECK()            \
    do {                          \
        count_launch();           \
        TLB_CUDA(cudaGetLastError()); \
    } while (0)

tlb_status launch_unary(int op, const float *a, float *out, int64_t n, float s)
{
    if (n == 0) return TLB_OK;
    unary_kernel<<<grid_for(n, 256), 256, 0, ctx()->stream>>>(op, a, out, n, s);
    LAUNCH_CHECK();
    return TLB_OK;
}

tlb_status launch_silu_mul(const float *g, const float *u, float *out, int64_t n)
{
    if (n == 0) return TLB_OK;
    if (n % 4 == 0 && (((uintptr_t)g | (uintptr_t)u | (uintptr_t)out) & 15) == 0)
        silu_mul4_kernel<<<grid_for(n / 4, 256), 256, 0, ctx()->stream>>>((const float4 *)g, (const float4 *)u, (float4 *)out, n / 4);
    else
        silu_mul_kernel<<<grid_for(n, 256), 256, 0, ctx()->stream>>>(g, u, out, n);
    LAUNCH_CHECK();
    return TLB_OK;
}

tlb_status launch_softmax(const float *a, float *out, int64_t outer, int64_t axis, int64_t inner)
{
    if (outer * axis * inner == 0) return TLB_OK;
    int threads = axis >= 1024 ? 256 : (axis >= 128 ? 128 : 32);
    softmax_kernel<<<(unsigned)(outer * inner), threads, 0, ctx()->stream>>>(a, out, axis, inner);
    LAUNCH_CHECK();
    return TLB_OK;
}

tlb_status launch_matmul(const float *a, const float *b, float *out, int64_t batch, int64_t m, int64_t k, int64_t n, bool b_batched)
{
    if (batch * m * n == 0) return TLB_OK;
    if (m <= 4 && k <= INT32_MAX && n <= INT32_MAX && batch <= 65535) {
        if (n <= 256) {
            dim3 grid((unsigned)((n + 15) / 16), (unsigned)batch);
            matmul_rows_kernel<16><<<grid, 512, 0, ctx()->stream>>>(a, b, out, (int)m, (int)k, (int)n, b_batched ? 1 : 0);
        } else {
            dim3 grid((unsigned)((n + 63) / 64), (unsigned)batch);
            matmul_rows_kernel<64><<<grid, 512, 0, ctx()->stream>>>(a, b, out, (int)m, (int)k, (int)n, b_batched ? 1 : 0);
        }
        LAUNCH_CHECK();
        return TLB_OK;
    }
    dim3 grid((unsigned)((n + 63) / 64), (unsigned)((m + 63) / 64), (unsigned)batch);
    matmul_kernel<<<grid, 256, 0, ctx()->stream>>>(a, b, out, m, k, n, b_batched ? 1 : 0);
    LAUNCH_CHECK();
    return TLB_OK;
}

tlb_status launch_copy_strided(const float *a, float *out, const int64_t *oshape, const int64_t *astr, int rank, int64_t n, int64_t a_off)
{
    if (n == 0) return TLB_OK;
    // (1) the last two dimensions exchanged, everything before them in place: tiled transpose
    if (rank >= 2 && a_off == 0 && astr[rank - 1] == oshape[rank - 2] && astr[rank - 2] == 1 && oshape[rank - 1] <= INT32_MAX && oshape[rank - 2] <= INT32_MAX) {
        bool outer_plain = true;
        int64_t want = oshape[rank - 1] * oshape[rank - 2], batch = 1;
        for (int i = rank - 3; i >= 0; i--) { outer_plain = outer_plain && astr[i] == want; want *= oshape[i]; batch *= oshape[i]; }
        const int rows = (int)oshape[rank - 1], cols = (int)oshape[rank - 2];   // of the source: [rows][cols] -> [cols][rows]
        if (outer_plain && batch <= 65535 && (rows + 31) / 32 <= 65535) {
            dim3 grid((unsigned)((cols + 31) / 32), (unsigned)((rows + 31) / 32), (unsigned)batch);
            transpose_last2_kernel<<<grid, 256, 0, ctx()->stream>>>(a, out, rows, cols);
            LAUNCH_CHECK();
            return TLB_OK;
        }
    }
    // (2) rows that are contiguous on both sides, a multiple of four floats long and 16-byte aligned: float4 copies
    if (rank >= 1 && astr[rank - 1] == 1 && oshape[rank - 1] % 4 == 0 && a_off % 4 == 0 && (((uintptr_t)a | (uintptr_t)out) & 15) == 0 &&
        n / oshape[rank - 1] <= UINT32_MAX) {
        bool ok = true;
        RowStrides r;
        r.rank = rank - 1;
        for (int i = 0; i < rank - 1; i++) {
            ok = ok && astr[i] % 4 == 0 && oshape[i] <= UINT32_MAX;
            r.o[i] = (unsigned)oshape[i];
            r.a[i] = astr[i] / 4;
        }
        if (ok) {
            const unsigned rows = (unsigned)(n / oshape[rank - 1]), inner4 = (unsigned)(oshape[rank - 1] / 4);
            copy_rows4_kernel<<<grid_for(n / 4, 256), 256, 0, ctx()->stream>>>(reinterpret_cast<const float4 *>(a), reinterpret_cast<float4 *>(out), r, rows,
                                                                               inner4, a_off / 4);
            LAUNCH_CHECK();
            return TLB_OK;
        }
    }
    Strides s;
    s.rank = rank;
    for (int i = 0; i < rank; i++) { s.o[i] = oshape[i]; s.a[i] = astr[i]; s.b[i] = 0; }
    copy_strided_kernel<<<grid_for(n, 256), 256, 0, ctx()->stream>>>(a, out, s, n, a_off);
    LAUNCH_CHECK();
    return TLB_OK;
}

tlb_status launch_rms_norm(const float *x, const float *res, const float *w, float eps, float *out, int64_t rows, int64_t d)
{
    if (rows * d == 0) return TLB_OK;
    int threads = d >= 2048 ? 512 : (d >= 256 ? 128 : 32);
    rms_norm_kernel<<<(unsigned)rows, threads, 0, ctx()->stream>>>(x, res, w, eps, out, d);
    LAUNCH_CHECK();
    return TLB_OK;
}

tlb_status launch_rope_cpu(const float *x, const float *cos_t, const float *sin_t, int64_t tab_len, float *out, int64_t nvec, int64_t d)
{
    int64_t np = nvec * (d / 2);
    if (np == 0) return TLB_OK;
    rope_cpu_kernel<<<grid_for(np, 256), 256, 0, ctx()->stream>>>(x, cos_t, sin_t, tab_len, out, np, d);
    LAUNCH_CHECK();
    return TLB_OK;
}

tlb_status launch_rope_half(const float *x, const float *cos_t, const float *sin_t, float *out, int64_t tokens, int64_t heads, int64_t d)
{
    int64_t np = tokens * heads * (d / 2);
    if (np == 0) return TLB_OK;
    rope_half_kernel<<<grid_for(np, 256), 256, 0, ctx()->stream>>>(x, cos_t, sin_t, out, tokens, heads, d);
    LAUNCH_CHECK();
    return TLB_OK;
}

tlb_status launch_embedding(const float *table, const float *idx, float *out, int64_t n, int64_t vocab, int64_t dim, int *oob)
{
    if (n * dim == 0) return TLB_OK;
    embedding_kernel<<<grid_for(n * dim, 256), 256, 0, ctx()->stream>>>(table, idx, out, n, vocab, dim, oob);
    LAUNCH_CHECK();
    return TLB_OK;
}

tlb_status launch_argmax(const float *x, int64_t n, int tie_first, float *out_f32, int *out_i32)
{
    static float *pv = nullptr;
    static long long *pi = nullptr;
    const int parts = 148;
    if (!pv) {
        TLB_CUDA(cudaMalloc(&pv, parts * sizeof(float)));
        TLB_CUDA(cudaMalloc(&pi, parts * sizeof(long long)));
    }
    int blocks = (int)std::max<int64_t>(1, std::min<int64_t>(parts, (n + 1023) / 1024));
    argmax_partial_kernel<<<blocks, 256, 0, ctx()->stream>>>(x, n, tie_first, pv, pi);
    LAUNCH_CHECK();
    argmax_final_kernel<<<1, 32, 0, ctx()->stream>>>(pv, pi, blocks, tie_first, out_f32, out_i32);
    LAUNCH_CHECK();
    return TLB_OK;
}

tlb_status launch_causal_mask(float *out, int64_t size)
{
    if (size == 0) return TLB_OK;
    causal_mask_kernel<<<grid_for(size * size, 256), 256, 0, ctx()->stream>>>(out, size);
    LAUNCH_CHECK();
    return TLB_OK;
}

tlb_status launch_rep_penalty(float *logits, const float *tokens, int64_t rows, int64_t vocab, int64_t nt, float p)
{
    if (nt == 0 || rows * vocab == 0) return TLB_OK;
    rep_penalty_kernel<<<grid_for(nt, 128), 128, 0, ctx()->stream>>>(logits, tokens, rows, vocab, nt, p);
    LAUNCH_CHECK();
    return TLB_OK;
}

tlb_status launch_f32_to_f16(const float *a, __half *out, int64_t n)
{
    if (n == 0) return TLB_OK;
    f32_to_f16_kernel<<<grid_for(n, 256), 256, 0, ctx()->stream>>>(a, out, n);
    LAUNCH_CHECK();
    return TLB_OK;
}

tlb_status launch_binary_bcast(int op, const tlb_tensor *a, const tlb_tensor *b, tlb_tensor **out)
{
    // numpy broadcasting (crates/tl_cpu/src/tensor.rs:549-609)
    int rank = std::max(a->rank, b->rank);
    int64_t oshape[kMaxRank];
    Strides s;
    s.rank = rank;
    int64_t sa = 1, sb = 1;
    for (int d = rank - 1; d >= 0; d--) {
        int da = d - (rank - a->rank), db = d - (rank - b->rank);
        int64_t na = da >= 0 ? a->shape[da] : 1, nb = db >= 0 ? b->shape[db] : 1;
        if (na != nb && na != 1 && nb != 1)
            return fail(TLB_ERR_SHAPE, "shapes cannot be broadcast together (dim %d: %lld vs %lld)", d, (long long)na, (long long)nb);
        oshape[d] = std::max(na, nb);
        if (na == 0 || nb == 0) oshape[d] = 0;
        s.o[d] = oshape[d];
        s.a[d] = na == 1 ? 0 : sa;
        s.b[d] = nb == 1 ? 0 : sb;
        sa *= na;
        sb *= nb;
    }
    TLB_TRY(new_tensor(out, TLB_F32, oshape, rank));
    int64_t n = (*out)->numel();
    if (n == 0) return TLB_OK;
    if (a->numel() == n && b->numel() == n)
        same_shape_binary_kernel<<<grid_for(n, 256), 256, 0, ctx()->stream>>>(op, a->f32(), b->f32(), (*out)->f32(), n);
    else
        binary_kernel<<<grid_for(n, 256), 256, 0, ctx()->stream>>>(op, a->f32(), b->f32(), (*out)->f32(), s, n);
    LAUNCH_CHECK();
    return TLB_OK;
}

tlb_status launch_copy_into(const float *a, float *out, int64_t outer, int64_t a_inner, int64_t o_inner, int64_t o_off)
{
    int64_t n = outer * a_inner;
    if (n == 0) return TLB_OK;
    copy_into_kernel<<<grid_for(n, 256), 256, 0, ctx()->stream>>>(a, out, outer, a_inner, o_inner, o_off);
    LAUNCH_CHECK();
    return TLB_OK;
}

}  // namespace tlb
