/*
 * tl_oracle.h - CPU restatement of the TL reference's CPU path for GGUF-quantized
 * Llama inference.  TEST INFRASTRUCTURE ONLY: this library is the checker the GPU
 * kernels are compared against and the timed CPU baseline; the product (libtlb200)
 * never links, loads or calls it.
 *
 * Every function cites the reference file:line whose arithmetic (expression shape,
 * loop order, f32 accumulation order) it follows.  Build with -ffp-contract=off so
 * that no fused multiply-add is formed (the Rust reference never forms one).
 *
 * Parity pin: the reference's own tests hold known-answer vectors for rms_norm,
 * causal mask, RoPE row 0, matmul, softmax, embedding, argmax, repeat_interleave,
 * cat, narrow, repetition penalty and fused silu-mul / add-rms-norm; those are
 * replayed in tests/test_oracle_kat.py.  Dequantisation values, quantized matmul
 * results, logits and tokens are pinned by NO test of the reference ("parity
 * unpinned" for those): they are anchored on hand-built single-block vectors
 * derived from the format definition in crates/tl_runtime/src/quantized.rs.
 */
#ifndef TL_ORACLE_H
#define TL_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* GGML type ids as stored in a GGUF tensor-info record. */
enum {
    ORC_F32 = 0, ORC_F16 = 1, ORC_Q4_0 = 2, ORC_Q4_1 = 3, ORC_Q5_0 = 6, ORC_Q5_1 = 7, ORC_Q8_0 = 8, ORC_Q8_1 = 9,
    ORC_Q4_K = 12, ORC_Q6_K = 14
};

float    orc_f16_to_f32(uint16_t h);
uint16_t orc_f32_to_f16(float f);

/* bytes needed for nelem weights of a type, or 0 if unsupported / not divisible */
size_t orc_type_nbytes(int type, size_t nelem);

/* crates/tl_runtime/src/quantized.rs:88-109 dispatch; returns 0 on success */
int orc_dequantize(int type, const uint8_t *data, size_t nbytes, size_t nelem, float *out);

/* crates/tl_cpu/src/tensor.rs:1248-1313: naive batched matmul.
 * a: [batch, m, k]; b: [k, n] (b_batched = 0) or [batch, k, n]; out: [batch, m, n]. */
void orc_matmul(const float *a, const float *b, float *out,
                size_t batch, size_t m, size_t k, size_t n, int b_batched);

/* crates/tl_runtime/src/system.rs:193-222: y[M,N] = x[M,K] * dequant(W[N,K])^T,
 * same accumulation order as dequant -> transpose -> matmul, without materialising
 * the transposed copy (bit-identical: same multiplies and adds in the same order). */
int orc_qmatmul(int type, const uint8_t *w, size_t n, size_t k,
                const float *x, size_t m, float *out);
/* Same, with W already dequantised row-major [N,K]. */
void orc_matmul_wt(const float *w_nk, size_t n, size_t k, const float *x, size_t m, float *out);
/* Steady-state form the reference actually runs per token: B = cached transposed
 * weights [K,N], inner loop strides by N (tensor.rs:1284-1306).  Used for timing. */
void orc_matmul_cached_t(const float *w_kn, size_t n, size_t k, const float *x, size_t m, float *out);

/* columns [j0, j1) of the same loop: a bounded sample for timing */
void orc_matmul_cached_t_cols(const float *w_kn, size_t n, size_t k, const float *x, size_t m,
                              size_t j0, size_t j1, float *out);

/* crates/tl_cpu/src/ffi.rs:2444-2486 (weight may be NULL) */
void orc_rms_norm(const float *x, const float *w, float eps, size_t rows, size_t d, float *out);

/* crates/tl_cpu/src/ffi.rs:2589-2627: tables [seq_len, dim], pair-duplicated */
void orc_rope_table_cpu(size_t seq_len, size_t dim, float base, float *cos_out, float *sin_out);
/* crates/tl_cpu/src/ffi.rs:2629-2685: adjacent pairs, row 0 of the table for every vector */
void orc_apply_rope_cpu(const float *x, size_t total, size_t head_dim,
                        const float *cos_t, size_t cos_len, const float *sin_t, size_t sin_len,
                        float *out);
/* crates/tl_cuda/src/ops/llm.rs:96-117: tables [seq_len, dim/2] */
void orc_rope_table_half(size_t seq_len, size_t dim, float base, float *cos_out, float *sin_out);
/* crates/tl_cuda/src/cuda_kernels/autograd.cu:1196-1227: rotate-half, per-token row.
 * x: [tokens, heads, head_dim]; tables: [>=tokens, head_dim/2] */
void orc_apply_rope_rotate_half(const float *x, size_t tokens, size_t heads, size_t head_dim,
                                const float *cos_t, const float *sin_t, float *out);

/* crates/tl_cpu/src/tensor.rs:1065-1092 */
void orc_softmax(const float *x, size_t outer, size_t axis, size_t inner, float *out);
/* crates/tl_cpu/src/ffi.rs:2097-2103 */
void orc_silu(const float *x, size_t n, float *out);
/* crates/tl_cpu/src/tensor.rs:549-609 restricted to equal shapes / trailing broadcast */
void orc_add(const float *a, const float *b, size_t n, size_t nb, float *out);
void orc_mul(const float *a, const float *b, size_t n, size_t nb, float *out);
void orc_scale(const float *a, float s, size_t n, float *out);
/* crates/tl_cpu/src/tensor.rs:1094-1112; returns -1 on out-of-range index */
int orc_embedding(const float *table, size_t vocab, size_t dim,
                  const float *idx, size_t n, float *out);
/* crates/tl_cpu/src/tensor.rs:1178-1201 */
void orc_repeat_interleave(const float *x, size_t outer, size_t axis, size_t inner,
                           size_t repeats, float *out);
/* crates/tl_cpu/src/ffi.rs:3184-3196 */
void orc_causal_mask(size_t size, float *out);
/* crates/tl_cpu/src/tensor.rs:841-846: LAST maximal index */
size_t orc_argmax_last(const float *x, size_t n);
/* crates/tl_cuda/src/cuda_kernels/autograd.cu:1119-1132: FIRST maximal index */
size_t orc_argmax_first(const float *x, size_t n);
/* tl_cpu tensor.rs:1625-1680 sample_impl with the random number u in [0, 1) as an argument */
size_t orc_sample_top_p(const float *logits, size_t n, float temp, float top_p, double u);
/* the same with the kept prefix also limited to the top_k most probable tokens (top_k <= 0: no limit); no counterpart in the
 * reference, whose top-k sampler is an argmax (crates/tl_cuda/src/cuda_kernels/autograd.cu:2370-2415) */
size_t orc_sample_top_k_top_p(const float *logits, size_t n, float temp, long top_k, float top_p, double u);
/* Philox-4x32-10 and the uniform in [0, 1) the decode session derives from (seed, counter): first output word >> 8, / 2^24 */
void   orc_philox4x32_10(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4]);
double orc_rng_uniform(uint64_t seed, uint64_t counter);
/* crates/tl_cpu/src/device_impl.rs:967-1000 */
void orc_repetition_penalty(const float *logits, size_t n, const float *tokens, size_t nt,
                            float penalty, float *out);
/* crates/tl_cpu/src/device_impl.rs:775-870: q [bh,sq,d], k,v [bh,sk,d];
 * mask [sq,sk] or NULL; mask value 0 -> score = -1e9 */
void orc_sdpa_cpu(const float *q, const float *k, const float *v, const float *mask,
                  size_t bh, size_t sq, size_t sk, size_t d, float *out);

/* ---- Llama forward driver: replays the op order of
 * examples/apps/llama3/chatbot_llama3.tl:48-125,220-236 and
 * examples/apps/tinyllama/chatbot.tl:33-113 on GGUF-typed tensors. ---- */
typedef struct {
    int32_t n_layers, d_model, n_heads, n_kv_heads, head_dim, ffn, vocab;
    float   eps, rope_base, attn_scale; /* attn_scale is the f32 literal of the TL program */
    int32_t kv_f16;     /* 0: f32 KV cache (reference); 1: K/V rounded to f16 when cached */
    int32_t max_seq;
} orc_llama_cfg;

typedef struct orc_llama orc_llama;

orc_llama *orc_llama_new(const orc_llama_cfg *cfg);
void       orc_llama_free(orc_llama *m);
/* name: GGUF tensor name (token_embd.weight, blk.N.attn_q.weight, ...). The bytes are
 * NOT copied: caller keeps them alive. Returns 0 on success. */
int  orc_llama_set_tensor(orc_llama *m, const char *name, int type, const uint8_t *data,
                          size_t nbytes);
/* Overwrite cached K/V for one layer and position (already-roped K), kv_dim floats each. */
void orc_llama_kv_write(orc_llama *m, int layer, int pos, const float *k, const float *v);
void orc_llama_kv_clear(orc_llama *m);
/* One forward call over n tokens starting at start_pos (= current cache length).
 * logits_out: [vocab] for the LAST token.  Returns 0 on success. */
int  orc_llama_forward(orc_llama *m, const int32_t *tokens, int n, int start_pos,
                       float *logits_out);
/* hidden state after the last layer for the last token (d_model floats), for debugging */
const float *orc_llama_last_hidden(const orc_llama *m);

#ifdef __cplusplus
}
#endif
#endif
