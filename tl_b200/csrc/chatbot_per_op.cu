// The TL chatbot's decode step, op by op, through this library's own per-op entry points - issued from native code, as
// the compiled TL program issues them (examples/apps/llama3/chatbot_llama3.tl:48-125,220-236; the tinyllama chatbot is the
// same sequence): embedding, rms_norm + mul, tl_qtensor_matmul, reshape, narrow, apply_rope, transpose, kv cache get /
// cat_4d / update, repeat_interleave, matmul_4d, scale, (causal mask,) softmax, silu, mul, add, sample, item_i64.  One
// kernel or more per op, a cache that grows by concatenation, the tensors looked up by name for every token as
// Block::from_map does: what an UNMODIFIED TL program gets behind TL_DEVICE=cuda.  It exists to measure that route
// without an interpreter's call overhead on top, and to check it against the fused session.
#include <cstdio>
#include <string>
#include <vector>

#include "tlb_internal.h"

using namespace tlb;

namespace {

// Temporaries of one step: released in one sweep, whatever the exit path.
struct Temps {
    std::vector<tlb_tensor *> t;
    std::vector<tlb_qtensor *> q;
    tlb_tensor *keep(tlb_tensor *x) { t.push_back(x); return x; }
    tlb_qtensor *keep(tlb_qtensor *x) { q.push_back(x); return x; }
    ~Temps()
    {
        for (tlb_tensor *x : t) tlb_tensor_release(x);
        for (tlb_qtensor *x : q) tlb_qtensor_release(x);
    }
};

#define OP(var, call)                         \
    tlb_tensor *var = nullptr;                \
    TLB_TRY(call);                            \
    tmp.keep(var)

}  // namespace

extern "C" tlb_status tlb_chatbot_step_per_op(tlb_map *weights, tlb_kvcache *cache, const tlb_tensor *cos_t, const tlb_tensor *sin_t,
                                              const tlb_decoder_cfg *cfg, const float *tokens, int64_t n_tokens, int64_t start_pos,
                                              int64_t *next_token, tlb_tensor **logits_out)
{
    if (!weights || !cache || !cos_t || !sin_t || !cfg || !tokens || !next_token) return fail(TLB_ERR_NULL, "null argument");
    if (n_tokens < 1) return fail(TLB_ERR_ARG, "no tokens");
    Temps tmp;
    const int64_t sl = n_tokens, H = cfg->n_heads, KVH = cfg->n_kv_heads, D = cfg->head_dim;
    auto norm = [&](tlb_tensor **out, const tlb_tensor *x, const tlb_tensor *w) -> tlb_status {   // RMSNorm::forward: rms_norm, then mul by the weight
        tlb_tensor *n = nullptr;
        TLB_TRY(tlb_rms_norm(&n, x, nullptr, cfg->eps));
        tmp.keep(n);
        TLB_TRY(tlb_mul(out, n, w));
        tmp.keep(*out);
        return TLB_OK;
    };
    auto weight1d = [&](tlb_tensor **out, const std::string &name) -> tlb_status {
        TLB_TRY(tlb_map_get_1d(out, weights, name.c_str()));
        tmp.keep(*out);
        return TLB_OK;
    };
    auto weightq = [&](tlb_qtensor **out, const std::string &name) -> tlb_status {
        TLB_TRY(tlb_map_get_quantized(out, weights, name.c_str()));
        tmp.keep(*out);
        return TLB_OK;
    };

    const int64_t tshape[1] = {sl};
    OP(idx, tlb_tensor_from_host(&idx, tokens, TLB_F32, tshape, 1));
    tlb_tensor *emb = nullptr;
    TLB_TRY(tlb_map_get(&emb, weights, "token_embd.weight"));
    tmp.keep(emb);
    OP(x0, tlb_embedding(&x0, emb, idx));
    const tlb_tensor *x = x0;
    for (int li = 0; li < cfg->n_layers; li++) {
        const std::string p = "blk." + std::to_string(li) + ".";
        tlb_tensor *an = nullptr, *fn = nullptr;
        tlb_qtensor *wq = nullptr, *wk = nullptr, *wv = nullptr, *wo = nullptr, *wg = nullptr, *wu = nullptr, *wd = nullptr;
        TLB_TRY(weight1d(&an, p + "attn_norm.weight"));
        TLB_TRY(weight1d(&fn, p + "ffn_norm.weight"));
        TLB_TRY(weightq(&wq, p + "attn_q.weight")); TLB_TRY(weightq(&wk, p + "attn_k.weight")); TLB_TRY(weightq(&wv, p + "attn_v.weight"));
        TLB_TRY(weightq(&wo, p + "attn_output.weight"));
        TLB_TRY(weightq(&wg, p + "ffn_gate.weight")); TLB_TRY(weightq(&wu, p + "ffn_up.weight")); TLB_TRY(weightq(&wd, p + "ffn_down.weight"));

        tlb_tensor *xn = nullptr;
        TLB_TRY(norm(&xn, x, an));
        // Attention::forward
        const int64_t qs[4] = {1, sl, H, D}, ks[4] = {1, sl, KVH, D};
        OP(q2, tlb_qtensor_matmul(&q2, xn, wq));
        OP(q4, tlb_reshape(&q4, q2, qs, 4));
        OP(k2, tlb_qtensor_matmul(&k2, xn, wk));
        OP(k4, tlb_reshape(&k4, k2, ks, 4));
        OP(v2, tlb_qtensor_matmul(&v2, xn, wv));
        OP(v4, tlb_reshape(&v4, v2, ks, 4));
        OP(cs, tlb_narrow(&cs, cos_t, 0, start_pos, sl));
        OP(ss, tlb_narrow(&ss, sin_t, 0, start_pos, sl));
        OP(qr, tlb_apply_rope(&qr, q4, cs, ss, TLB_ROPE_CPU));
        OP(kr, tlb_apply_rope(&kr, k4, cs, ss, TLB_ROPE_CPU));
        OP(kt, tlb_transpose(&kt, kr, 1, 2));
        OP(vt, tlb_transpose(&vt, v4, 1, 2));
        tlb_tensor *k_tot = kt, *v_tot = vt;
        if (start_pos != 0) {
            OP(ck, tlb_kvcache_get_k(&ck, cache, li));
            OP(cv, tlb_kvcache_get_v(&cv, cache, li));
            OP(kc, tlb_cat(&kc, ck, kt, 2));
            OP(vc, tlb_cat(&vc, cv, vt, 2));
            k_tot = kc; v_tot = vc;
        }
        TLB_TRY(tlb_kvcache_update(cache, li, k_tot, v_tot));
        OP(qt, tlb_transpose(&qt, qr, 1, 2));
        OP(kw, tlb_repeat_interleave(&kw, k_tot, H / KVH, 1));
        OP(vw, tlb_repeat_interleave(&vw, v_tot, H / KVH, 1));
        OP(kwt, tlb_transpose(&kwt, kw, 2, 3));
        OP(sc0, tlb_matmul(&sc0, qt, kwt));
        OP(sc1, tlb_scale(&sc1, sc0, cfg->attn_scale));
        const tlb_tensor *scores = sc1;
        if (sl > 1) {
            const int64_t ms[4] = {1, 1, sl, sl};
            OP(mask, tlb_new_causal_mask(&mask, sl));
            OP(mask4, tlb_reshape(&mask4, mask, ms, 4));
            OP(sc2, tlb_add(&sc2, sc1, mask4));
            scores = sc2;
        }
        OP(pr, tlb_softmax(&pr, scores, 3));
        OP(av, tlb_matmul(&av, pr, vw));
        OP(avt, tlb_transpose(&avt, av, 1, 2));
        const int64_t os[2] = {sl, H * D};
        OP(ao, tlb_reshape(&ao, avt, os, 2));
        OP(attn, tlb_qtensor_matmul(&attn, ao, wo));
        // Block::forward
        OP(h, tlb_add(&h, x, attn));
        tlb_tensor *y = nullptr;
        TLB_TRY(norm(&y, h, fn));
        OP(g, tlb_qtensor_matmul(&g, y, wg));
        OP(gs, tlb_silu(&gs, g));
        OP(u, tlb_qtensor_matmul(&u, y, wu));
        OP(mu, tlb_mul(&mu, gs, u));
        OP(dn, tlb_qtensor_matmul(&dn, mu, wd));
        OP(xo, tlb_add(&xo, h, dn));
        x = xo;
    }
    tlb_tensor *on = nullptr;
    tlb_qtensor *oh = nullptr;
    TLB_TRY(weight1d(&on, "output_norm.weight"));
    TLB_TRY(weightq(&oh, "output.weight"));
    tlb_tensor *xf = nullptr;
    TLB_TRY(norm(&xf, x, on));
    OP(lo, tlb_qtensor_matmul(&lo, xf, oh));
    OP(last, tlb_narrow(&last, lo, 0, sl - 1, 1));
    OP(tok, tlb_sample(&tok, last, 0.0f, 0.9f, (tlb_tie_rule)cfg->tie_rule));
    TLB_TRY(tlb_tensor_item_i64(tok, next_token));
    if (logits_out) {
        TLB_TRY(tlb_tensor_clone(logits_out, last));
    }
    return TLB_OK;
}
