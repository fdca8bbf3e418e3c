// extern "C" wrappers of the per-op tensor API (argument checks, shapes, error codes).
#include "tlb_internal.h"

#include <cmath>

namespace tlb {
tlb_status launch_binary_bcast(int op, const tlb_tensor *a, const tlb_tensor *b, tlb_tensor **out);
tlb_status launch_copy_into(const float *a, float *out, int64_t outer, int64_t a_inner, int64_t o_inner, int64_t o_off);
}
using namespace tlb;

#define REQ(cond, code, ...)                      \
    do {                                          \
        if (!(cond)) return fail(code, __VA_ARGS__); \
    } while (0)
#define REQ_F32(t) REQ((t)->dt == TLB_F32, TLB_ERR_TYPE, "%s: f32 tensor expected", __func__)
#define CHECK_OUT(out)                                 \
    do {                                               \
        REQ(out, TLB_ERR_NULL, "%s: null out", __func__); \
        *(out) = nullptr;                              \
        if (!ensure_init()) return TLB_ERR_DEVICE;     \
    } while (0)
// release *out when the launch failed
#define FINISH(out, st)                                        \
    do {                                                       \
        tlb_status _st = (st);                                 \
        if (_st != TLB_OK && *(out)) { tlb_tensor_release(*(out)); *(out) = nullptr; } \
        return _st;                                            \
    } while (0)

static int norm_dim(int64_t d, int rank) { return (int)(d < 0 ? d + rank : d); }

extern "C" {

tlb_status tlb_add(tlb_tensor **out, const tlb_tensor *a, const tlb_tensor *b)
{
    CHECK_OUT(out);
    REQ(a && b, TLB_ERR_NULL, "add: null tensor");
    REQ_F32(a); REQ_F32(b);
    return launch_binary_bcast(0, a, b, out);
}

tlb_status tlb_mul(tlb_tensor **out, const tlb_tensor *a, const tlb_tensor *b)
{
    CHECK_OUT(out);
    REQ(a && b, TLB_ERR_NULL, "mul: null tensor");
    REQ_F32(a); REQ_F32(b);
    return launch_binary_bcast(1, a, b, out);
}

tlb_status tlb_silu(tlb_tensor **out, const tlb_tensor *a)
{
    CHECK_OUT(out);
    REQ(a, TLB_ERR_NULL, "silu: null tensor");
    REQ_F32(a);
    TLB_TRY(new_tensor(out, TLB_F32, a->shape, a->rank));
    FINISH(out, launch_unary(0, a->f32(), (*out)->f32(), a->numel(), 0.f));
}

tlb_status tlb_scale(tlb_tensor **out, const tlb_tensor *a, float s)
{
    CHECK_OUT(out);
    REQ(a, TLB_ERR_NULL, "scale: null tensor");
    REQ_F32(a);
    TLB_TRY(new_tensor(out, TLB_F32, a->shape, a->rank));
    FINISH(out, launch_unary(1, a->f32(), (*out)->f32(), a->numel(), s));
}

tlb_status tlb_fused_silu_mul(tlb_tensor **out, const tlb_tensor *g, const tlb_tensor *u)
{
    CHECK_OUT(out);
    REQ(g && u, TLB_ERR_NULL, "fused_silu_mul: null tensor");
    REQ_F32(g); REQ_F32(u);
    REQ(g->numel() == u->numel(), TLB_ERR_SHAPE, "fused_silu_mul: shapes differ");
    TLB_TRY(new_tensor(out, TLB_F32, g->shape, g->rank));
    FINISH(out, launch_silu_mul(g->f32(), u->f32(), (*out)->f32(), g->numel()));
}

tlb_status tlb_softmax(tlb_tensor **out, const tlb_tensor *a, int64_t dim)
{
    CHECK_OUT(out);
    REQ(a, TLB_ERR_NULL, "softmax: null tensor");
    REQ_F32(a);
    int d = norm_dim(dim, a->rank);
    REQ(d >= 0 && d < a->rank, TLB_ERR_ARG, "softmax: dim %lld out of range for rank %d", (long long)dim, a->rank);
    int64_t outer = 1, inner = 1;
    for (int i = 0; i < d; i++) outer *= a->shape[i];
    for (int i = d + 1; i < a->rank; i++) inner *= a->shape[i];
    TLB_TRY(new_tensor(out, TLB_F32, a->shape, a->rank));
    FINISH(out, launch_softmax(a->f32(), (*out)->f32(), outer, a->shape[d], inner));
}

// crates/tl_cpu/src/tensor.rs:1248-1313: a [.., m, k] (1-D = [1, k]); b [k, n], batched [.., k, n], or 1-D [k]
tlb_status tlb_matmul(tlb_tensor **out, const tlb_tensor *a, const tlb_tensor *b)
{
    CHECK_OUT(out);
    REQ(a && b, TLB_ERR_NULL, "matmul: null tensor");
    REQ_F32(a); REQ_F32(b);
    REQ(a->rank >= 1 && b->rank >= 1, TLB_ERR_SHAPE, "Matmul requires at least 1D tensors");
    int64_t m = a->rank >= 2 ? a->shape[a->rank - 2] : 1, k = a->shape[a->rank - 1];
    int64_t k2 = b->rank >= 2 ? b->shape[b->rank - 2] : b->shape[0];
    int64_t n = b->rank >= 2 ? b->shape[b->rank - 1] : 1;
    REQ(k == k2, TLB_ERR_SHAPE, "Matmul shape mismatch: inner dims %lld vs %lld", (long long)k, (long long)k2);
    int64_t batch = 1;
    for (int i = 0; i < a->rank - 2; i++) batch *= a->shape[i];
    bool bb = b->rank > 2;
    if (bb) {
        int64_t b_batch = 1;
        for (int i = 0; i < b->rank - 2; i++) b_batch *= b->shape[i];
        REQ(b_batch == batch, TLB_ERR_SHAPE, "Matmul batch mismatch: %lld vs %lld", (long long)batch, (long long)b_batch);
    }
    int64_t oshape[kMaxRank];
    int r = 0;
    for (int i = 0; i < a->rank - 2; i++) oshape[r++] = a->shape[i];
    oshape[r++] = m;
    if (b->rank >= 2) oshape[r++] = n;
    TLB_TRY(new_tensor(out, TLB_F32, oshape, r));
    FINISH(out, launch_matmul(a->f32(), b->f32(), (*out)->f32(), batch, m, k, n, bb));
}

static void contiguous_strides(const tlb_tensor *a, int64_t *str)
{
    int64_t s = 1;
    for (int i = a->rank - 1; i >= 0; i--) { str[i] = s; s *= a->shape[i]; }
}

tlb_status tlb_narrow(tlb_tensor **out, const tlb_tensor *a, int64_t dim, int64_t start, int64_t len)
{
    CHECK_OUT(out);
    REQ(a, TLB_ERR_NULL, "narrow: null tensor");
    REQ_F32(a);
    int d = norm_dim(dim, a->rank);
    REQ(d >= 0 && d < a->rank, TLB_ERR_ARG, "narrow: dim out of range");
    REQ(start >= 0 && len >= 0 && start + len <= a->shape[d], TLB_ERR_INDEX, "narrow: [%lld, %lld) outside dimension of size %lld",
        (long long)start, (long long)(start + len), (long long)a->shape[d]);
    int64_t str[kMaxRank], oshape[kMaxRank];
    contiguous_strides(a, str);
    for (int i = 0; i < a->rank; i++) oshape[i] = a->shape[i];
    oshape[d] = len;
    if (d == 0) return new_view(out, a, oshape, a->rank, (size_t)(start * str[0]) * 4);  // leading-dim slice: zero-copy
    TLB_TRY(new_tensor(out, TLB_F32, oshape, a->rank));
    FINISH(out, launch_copy_strided(a->f32(), (*out)->f32(), oshape, str, a->rank, (*out)->numel(), start * str[d]));
}

tlb_status tlb_transpose(tlb_tensor **out, const tlb_tensor *a, int64_t d0, int64_t d1)
{
    CHECK_OUT(out);
    REQ(a, TLB_ERR_NULL, "transpose: null tensor");
    REQ_F32(a);
    int x = norm_dim(d0, a->rank), y = norm_dim(d1, a->rank);
    REQ(x >= 0 && x < a->rank && y >= 0 && y < a->rank, TLB_ERR_ARG, "transpose: dims (%lld, %lld) out of range for rank %d",
        (long long)d0, (long long)d1, a->rank);
    int64_t str[kMaxRank], oshape[kMaxRank];
    contiguous_strides(a, str);
    for (int i = 0; i < a->rank; i++) oshape[i] = a->shape[i];
    std::swap(oshape[x], oshape[y]);
    std::swap(str[x], str[y]);
    TLB_TRY(new_tensor(out, TLB_F32, oshape, a->rank));
    FINISH(out, launch_copy_strided(a->f32(), (*out)->f32(), oshape, str, a->rank, (*out)->numel(), 0));
}

tlb_status tlb_reshape(tlb_tensor **out, const tlb_tensor *a, const int64_t *shape, int rank)
{
    CHECK_OUT(out);
    REQ(a && (shape || rank == 0), TLB_ERR_NULL, "reshape: null argument");
    REQ(rank >= 0 && rank <= kMaxRank, TLB_ERR_SHAPE, "reshape: rank %d not supported", rank);
    int64_t n = 1, oshape[kMaxRank];
    int infer = -1;
    for (int i = 0; i < rank; i++) {
        oshape[i] = shape[i];
        if (shape[i] == -1) { REQ(infer < 0, TLB_ERR_SHAPE, "reshape: more than one -1"); infer = i; }
        else n *= shape[i];
    }
    if (infer >= 0) {
        REQ(n != 0 && a->numel() % n == 0, TLB_ERR_SHAPE, "reshape: cannot infer dimension");
        oshape[infer] = a->numel() / n;
        n *= oshape[infer];
    }
    REQ(n == a->numel(), TLB_ERR_SHAPE, "reshape: %lld elements into a shape of %lld", (long long)a->numel(), (long long)n);
    return new_view(out, a, oshape, rank, 0);  // zero-copy view (crates/tl_cuda/src/ops/shape.rs:61-74)
}

tlb_status tlb_cat(tlb_tensor **out, const tlb_tensor *a, const tlb_tensor *b, int64_t dim)
{
    CHECK_OUT(out);
    REQ(a && b, TLB_ERR_NULL, "cat: null tensor");
    REQ_F32(a); REQ_F32(b);
    REQ(a->rank == b->rank, TLB_ERR_SHAPE, "cat: ranks differ (%d vs %d)", a->rank, b->rank);
    int d = norm_dim(dim, a->rank);
    REQ(d >= 0 && d < a->rank, TLB_ERR_ARG, "cat: dim out of range");
    int64_t outer = 1, ai = 1, bi = 1, oshape[kMaxRank];
    for (int i = 0; i < a->rank; i++) {
        if (i != d) REQ(a->shape[i] == b->shape[i], TLB_ERR_SHAPE, "cat: dimension %d differs (%lld vs %lld)", i,
                        (long long)a->shape[i], (long long)b->shape[i]);
        oshape[i] = a->shape[i];
        if (i < d) outer *= a->shape[i];
        if (i >= d) { ai *= a->shape[i]; bi *= b->shape[i]; }
    }
    oshape[d] = a->shape[d] + b->shape[d];
    TLB_TRY(new_tensor(out, TLB_F32, oshape, a->rank));
    tlb_status st = launch_copy_into(a->f32(), (*out)->f32(), outer, ai, ai + bi, 0);
    if (st == TLB_OK) st = launch_copy_into(b->f32(), (*out)->f32(), outer, bi, ai + bi, ai);
    FINISH(out, st);
}

tlb_status tlb_repeat_interleave(tlb_tensor **out, const tlb_tensor *a, int64_t repeats, int64_t dim)
{
    CHECK_OUT(out);
    REQ(a, TLB_ERR_NULL, "repeat_interleave: null tensor");
    REQ_F32(a);
    int d = norm_dim(dim, a->rank);
    REQ(d >= 0 && d < a->rank, TLB_ERR_SHAPE, "Axis %lld out of bounds for repeat_interleave (rank %d)", (long long)dim, a->rank);
    REQ(repeats >= 0, TLB_ERR_ARG, "repeat_interleave: negative repeats");
    REQ(a->rank + 1 <= kMaxRank, TLB_ERR_SHAPE, "repeat_interleave: rank too large");
    // view the output as [.., axis, repeats, ..] with stride 0 along `repeats`
    int64_t str[kMaxRank], vshape[kMaxRank], vstr[kMaxRank], oshape[kMaxRank];
    contiguous_strides(a, str);
    int r = 0;
    for (int i = 0; i < a->rank; i++) {
        vshape[r] = a->shape[i]; vstr[r] = str[i]; r++;
        if (i == d) { vshape[r] = repeats; vstr[r] = 0; r++; }
        oshape[i] = a->shape[i] * (i == d ? repeats : 1);
    }
    TLB_TRY(new_tensor(out, TLB_F32, oshape, a->rank));
    FINISH(out, launch_copy_strided(a->f32(), (*out)->f32(), vshape, vstr, r, (*out)->numel(), 0));
}

tlb_status tlb_new_causal_mask(tlb_tensor **out, int64_t size)
{
    CHECK_OUT(out);
    REQ(size >= 0, TLB_ERR_ARG, "causal mask: negative size");
    int64_t shape[2] = {size, size};
    TLB_TRY(new_tensor(out, TLB_F32, shape, 2));
    FINISH(out, launch_causal_mask((*out)->f32(), size));
}

tlb_status tlb_embedding(tlb_tensor **out, const tlb_tensor *table, const tlb_tensor *idx)
{
    CHECK_OUT(out);
    REQ(table && idx, TLB_ERR_NULL, "embedding: null tensor");
    REQ_F32(table); REQ_F32(idx);
    REQ(table->rank == 2, TLB_ERR_SHAPE, "embedding: table must be [vocab, dim]");
    REQ(idx->rank + 1 <= kMaxRank, TLB_ERR_SHAPE, "embedding: index rank too large");
    int64_t oshape[kMaxRank];
    for (int i = 0; i < idx->rank; i++) oshape[i] = idx->shape[i];
    oshape[idx->rank] = table->shape[1];
    REQ(!tlb_stream_is_capturing(), TLB_ERR_ARG, "embedding reads its out-of-range flag back from the device: not allowed during a stream capture");
    TLB_TRY(new_tensor(out, TLB_F32, oshape, idx->rank + 1));
    static int *oob = nullptr;
    if (!oob) { TLB_CUDA(cudaMalloc(&oob, sizeof(int))); TLB_CUDA(cudaMemset(oob, 0, sizeof(int))); }
    tlb_status st = launch_embedding(table->f32(), idx->f32(), (*out)->f32(), idx->numel(), table->shape[0], table->shape[1], oob);
    if (st == TLB_OK) {
        int flag = 0;
        cudaError_t e = cudaMemcpyAsync(&flag, oob, sizeof(int), cudaMemcpyDeviceToHost, ctx()->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx()->stream);
        if (e != cudaSuccess) st = cuda_fail(e, "embedding check");
        else if (flag) {
            cudaMemsetAsync(oob, 0, sizeof(int), ctx()->stream);
            st = fail(TLB_ERR_INDEX, "Embedding index out of range for vocab size %lld", (long long)table->shape[0]);
        }
    }
    FINISH(out, st);
}

tlb_status tlb_rms_norm(tlb_tensor **out, const tlb_tensor *x, const tlb_tensor *w, float eps)
{
    CHECK_OUT(out);
    REQ(x, TLB_ERR_NULL, "rms_norm: null input");
    REQ_F32(x);
    int64_t d = x->rank ? x->shape[x->rank - 1] : 1;
    if (w) { REQ_F32(w); REQ(w->numel() == d, TLB_ERR_SHAPE, "rms_norm: weight has %lld elements, last dim is %lld", (long long)w->numel(), (long long)d); }
    TLB_TRY(new_tensor(out, TLB_F32, x->shape, x->rank));
    FINISH(out, launch_rms_norm(x->f32(), nullptr, w ? w->f32() : nullptr, eps, (*out)->f32(), d ? x->numel() / d : 0, d));
}

tlb_status tlb_fused_rms_norm(tlb_tensor **out, const tlb_tensor *x, const tlb_tensor *w, float eps)
{
    REQ(w, TLB_ERR_NULL, "fused_rms_norm: null weight");
    return tlb_rms_norm(out, x, w, eps);
}

tlb_status tlb_fused_add_rms_norm(tlb_tensor **out, const tlb_tensor *x, const tlb_tensor *res, const tlb_tensor *w, float eps)
{
    CHECK_OUT(out);
    REQ(x && res && w, TLB_ERR_NULL, "fused_add_rms_norm: null tensor");
    REQ_F32(x); REQ_F32(res); REQ_F32(w);
    REQ(x->numel() == res->numel(), TLB_ERR_SHAPE, "fused_add_rms_norm: residual shape differs");
    int64_t d = x->rank ? x->shape[x->rank - 1] : 1;
    REQ(w->numel() == d, TLB_ERR_SHAPE, "fused_add_rms_norm: weight size");
    TLB_TRY(new_tensor(out, TLB_F32, x->shape, x->rank));
    FINISH(out, launch_rms_norm(x->f32(), res->f32(), w->f32(), eps, (*out)->f32(), d ? x->numel() / d : 0, d));
}

// Tables are computed on the host with libm powf/cosf/sinf and uploaded, as both reference back ends
// do (crates/tl_cpu/src/ffi.rs:2589-2627, crates/tl_cuda/src/ops/llm.rs:96-117).
static tlb_status rope_table(tlb_tensor **out, int64_t dim, int64_t seq_len, float base, tlb_rope_mode mode, bool want_sin)
{
    CHECK_OUT(out);
    REQ(dim >= 0 && seq_len >= 0 && dim % 2 == 0, TLB_ERR_ARG, "rope table: dim must be even and sizes non-negative");
    int64_t half = dim / 2, cols = mode == TLB_ROPE_CPU ? dim : half;
    std::vector<float> t((size_t)(seq_len * cols));
    for (int64_t pos = 0; pos < seq_len; pos++)
        for (int64_t i = 0; i < half; i++) {
            float freq = 1.0f / powf(base, 2.0f * (float)i / (float)dim);
            float ang = (float)pos * freq;
            float v = want_sin ? sinf(ang) : cosf(ang);
            if (mode == TLB_ROPE_CPU) { t[pos * dim + 2 * i] = v; t[pos * dim + 2 * i + 1] = v; }
            else t[pos * half + i] = v;
        }
    int64_t shape[2] = {seq_len, cols};
    return tlb_tensor_from_host(out, t.data(), TLB_F32, shape, 2);
}

tlb_status tlb_rope_new_cos(tlb_tensor **out, int64_t dim, int64_t seq_len, float base, tlb_rope_mode mode)
{
    return rope_table(out, dim, seq_len, base, mode, false);
}
tlb_status tlb_rope_new_sin(tlb_tensor **out, int64_t dim, int64_t seq_len, float base, tlb_rope_mode mode)
{
    return rope_table(out, dim, seq_len, base, mode, true);
}

tlb_status tlb_apply_rope(tlb_tensor **out, const tlb_tensor *x, const tlb_tensor *cos_t, const tlb_tensor *sin_t, tlb_rope_mode mode)
{
    CHECK_OUT(out);
    REQ(x && cos_t && sin_t, TLB_ERR_NULL, "apply_rope: null tensor");
    REQ_F32(x); REQ_F32(cos_t); REQ_F32(sin_t);
    int64_t d = x->rank ? x->shape[x->rank - 1] : 0;
    TLB_TRY(new_tensor(out, TLB_F32, x->shape, x->rank));
    if (d == 0 || x->numel() == 0) return TLB_OK;
    REQ(d % 2 == 0, TLB_ERR_SHAPE, "apply_rope: head_dim %lld must be even", (long long)d);
    if (mode == TLB_ROPE_CPU) {
        int64_t tab = std::min(cos_t->numel(), sin_t->numel());
        FINISH(out, launch_rope_cpu(x->f32(), cos_t->f32(), sin_t->f32(), tab, (*out)->f32(), x->numel() / d, d));
    }
    if (x->rank < 3) { tlb_tensor_release(*out); *out = nullptr; return fail(TLB_ERR_SHAPE, "apply_rope (rotate-half): x must be [.., tokens, heads, dim]"); }
    int64_t heads = x->shape[x->rank - 2], tokens = x->numel() / (heads * d);
    int64_t per_batch = x->shape[x->rank - 3];
    if (cos_t->numel() < per_batch * (d / 2) || sin_t->numel() < per_batch * (d / 2) || tokens != per_batch) {
        tlb_tensor_release(*out); *out = nullptr;
        return fail(TLB_ERR_SHAPE, "apply_rope (rotate-half): table has fewer rows than tokens, or batch > 1");
    }
    FINISH(out, launch_rope_half(x->f32(), cos_t->f32(), sin_t->f32(), (*out)->f32(), tokens, heads, d));
}

tlb_status tlb_argmax(tlb_tensor **out, const tlb_tensor *x, tlb_tie_rule tie)
{
    CHECK_OUT(out);
    REQ(x, TLB_ERR_NULL, "argmax: null tensor");
    REQ_F32(x);
    REQ(x->numel() > 0, TLB_ERR_INTERNAL, "Empty tensor for sampling");
    int64_t one = 1;
    TLB_TRY(new_tensor(out, TLB_F32, &one, 1));
    FINISH(out, launch_argmax(x->f32(), x->numel(), tie == TLB_TIE_FIRST, (*out)->f32(), nullptr));
}

tlb_status tlb_sample(tlb_tensor **out, const tlb_tensor *logits, float temp, float top_p, tlb_tie_rule tie)
{
    (void)temp; (void)top_p;
    return tlb_argmax(out, logits, tie);
}

tlb_status tlb_repetition_penalty(tlb_tensor **out, const tlb_tensor *logits, const tlb_tensor *tokens, float penalty)
{
    CHECK_OUT(out);
    REQ(logits && tokens, TLB_ERR_NULL, "repetition_penalty: null tensor");
    REQ_F32(logits); REQ_F32(tokens);
    TLB_TRY(tlb_tensor_clone(out, logits));
    int64_t vocab = logits->rank ? logits->shape[logits->rank - 1] : 1;
    FINISH(out, launch_rep_penalty((*out)->f32(), tokens->f32(), vocab ? logits->numel() / vocab : 0, vocab, tokens->numel(), penalty));
}

tlb_status tlb_sdpa(tlb_tensor **out, const tlb_tensor *q, const tlb_tensor *k, const tlb_tensor *v, const tlb_tensor *mask, int mask_mode)
{
    CHECK_OUT(out);
    REQ(q && k && v, TLB_ERR_NULL, "sdpa: null tensor");
    REQ_F32(q); REQ_F32(k); REQ_F32(v);
    REQ(q->rank >= 2 && k->rank == q->rank && v->rank == q->rank, TLB_ERR_SHAPE, "sdpa: q, k, v must have the same rank >= 2");
    int64_t sq = q->shape[q->rank - 2], d = q->shape[q->rank - 1], sk = k->shape[k->rank - 2];
    REQ(k->shape[k->rank - 1] == d && v->shape[v->rank - 1] == d && v->shape[v->rank - 2] == sk, TLB_ERR_SHAPE, "sdpa: head dims / key length differ");
    int64_t bh = 1;
    for (int i = 0; i < q->rank - 2; i++) { REQ(q->shape[i] == k->shape[i] && q->shape[i] == v->shape[i], TLB_ERR_SHAPE, "sdpa: batch/head dims differ"); bh *= q->shape[i]; }
    int64_t mask_bh = 0;
    if (mask && mask_mode) {
        REQ_F32(mask);
        REQ(mask->numel() % (sq * sk) == 0 && mask->numel() >= sq * sk, TLB_ERR_SHAPE, "sdpa: mask must hold [.., sq, sk]");
        mask_bh = mask->numel() / (sq * sk);
        REQ(mask_bh == 1 || mask_bh == bh, TLB_ERR_SHAPE, "sdpa: mask batch must be 1 or match");
    }
    REQ(d <= 256, TLB_ERR_SHAPE, "sdpa: head_dim up to 256");
    TLB_TRY(new_tensor(out, TLB_F32, q->shape, q->rank));
    FINISH(out, launch_sdpa(q->f32(), k->f32(), v->f32(), (mask && mask_mode) ? mask->f32() : nullptr, mask_mode, (*out)->f32(), bh, sq, sk, d, mask_bh));
}

}  // extern "C"
