/*
 * tl_oracle.c - CPU restatement of the TL reference CPU path (see tl_oracle.h).
 * TEST INFRASTRUCTURE ONLY.  Compile with: gcc -O3 -ffp-contract=off -fno-fast-math.
 *
 * Transcendentals go through the f32 libm entry points (powf, cosf, sinf, expf, sqrtf),
 * which is what Rust's f32::{powf,cos,sin,exp,sqrt} lower to on glibc.
 */
#include "tl_oracle.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

/* ---------------------------------------------------------------- f16 */

/* IEEE-754 binary16 -> binary32, exact (subnormals, inf, nan included); this is what
 * half::f16::to_f32 computes (call sites crates/tl_runtime/src/quantized.rs:176,208,249,290,360). */
float orc_f16_to_f32(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            /* subnormal: renormalise */
            int e = -1;
            do { man <<= 1; e++; } while ((man & 0x400u) == 0);
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* binary32 -> binary16, round to nearest even (used only for the f16 KV-cache mode and by
 * the synthetic generators; not on the reference's path). */
uint16_t orc_f32_to_f16(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t absx = x & 0x7FFFFFFFu;
    if (absx >= 0x7F800000u) { /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | ((absx > 0x7F800000u) ? 0x200u : 0));
    }
    if (absx >= 0x477FF000u) { /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7C00u);
    }
    if (absx < 0x33000001u) { /* < 2^-25 (or exactly 2^-25, ties to even 0) */
        return (uint16_t)sign;
    }
    int32_t e = (int32_t)(absx >> 23) - 127;
    uint32_t m = (absx & 0x7FFFFFu) | 0x800000u;
    uint32_t shift, half_bits;
    if (e < -14) {
        shift = (uint32_t)(13 + (-14 - e)); /* subnormal result */
        half_bits = 0;
    } else {
        shift = 13;
        half_bits = (uint32_t)(e + 15) << 10;
        m &= 0x7FFFFFu;
    }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) q++;
    return (uint16_t)(sign | (half_bits + q)); /* carry into exponent is correct by construction */
}

static inline float f16_at(const uint8_t *p)
{
    return orc_f16_to_f32((uint16_t)(p[0] | ((uint16_t)p[1] << 8)));
}

/* ---------------------------------------------------------------- dequant */

size_t orc_type_nbytes(int type, size_t nelem)
{
    switch (type) {
    case ORC_F32: return nelem * 4;
    case ORC_F16: return nelem * 2;
    case ORC_Q4_0: return (nelem % 32) ? 0 : nelem / 32 * 18;
    case ORC_Q8_0: return (nelem % 32) ? 0 : nelem / 32 * 34;
    case ORC_Q4_K: return (nelem % 256) ? 0 : nelem / 256 * 144;
    case ORC_Q6_K: return (nelem % 256) ? 0 : nelem / 256 * 210;
    case ORC_Q4_1: return (nelem % 32) ? 0 : nelem / 32 * 20;
    case ORC_Q5_0: return (nelem % 32) ? 0 : nelem / 32 * 22;
    case ORC_Q5_1: return (nelem % 32) ? 0 : nelem / 32 * 24;
    case ORC_Q8_1: return (nelem % 32) ? 0 : nelem / 32 * 36;
    default: return 0;
    }
}

/* The four block types the reference's loader accepts (crates/tl_runtime/src/gguf.rs:160-165) but its
 * dequantiser rejects (crates/tl_runtime/src/quantized.rs:108 "Unsupported quantization type"): there
 * is no reference arithmetic to follow, so these restate the published GGML block definitions in the
 * same style as the reference's Q4_0 / Q8_0 code (integer to f32, one multiply, then one add, never
 * fused).  PARITY UNPINNED for these four.
 *   Q4_1: f16 d, f16 m, 16 nibble bytes           w[j] = d*(b&15) + m, w[j+16] = d*(b>>4) + m
 *   Q5_0: f16 d, u32 qh, 16 nibble bytes          q = (nibble | bit j of qh << 4) - 16, w = d*q
 *   Q5_1: f16 d, f16 m, u32 qh, 16 nibble bytes   q = nibble | bit << 4,               w = d*q + m
 *   Q8_1: f16 d, f16 s (d * sum of quants, unused here), 32 int8                       w = d*q      */
static void dequant_q4_1(const uint8_t *data, size_t nblocks, float *out)
{
    for (size_t b = 0; b < nblocks; b++) {
        const uint8_t *p = data + b * 20;
        float d = f16_at(p), m = f16_at(p + 2);
        float *y = out + b * 32;
        for (int j = 0; j < 16; j++) {
            uint8_t byte = p[4 + j];
            y[j] = d * (float)(byte & 0x0F) + m;
            y[j + 16] = d * (float)(byte >> 4) + m;
        }
    }
}

static void dequant_q5(const uint8_t *data, size_t nblocks, float *out, int with_min)
{
    size_t bb = with_min ? 24 : 22;
    for (size_t b = 0; b < nblocks; b++) {
        const uint8_t *p = data + b * bb;
        float d = f16_at(p), m = with_min ? f16_at(p + 2) : 0.0f;
        const uint8_t *qhp = p + (with_min ? 4 : 2), *qs = qhp + 4;
        uint32_t qh = (uint32_t)qhp[0] | ((uint32_t)qhp[1] << 8) | ((uint32_t)qhp[2] << 16) | ((uint32_t)qhp[3] << 24);
        float *y = out + b * 32;
        for (int j = 0; j < 16; j++) {
            int x0 = (int)(qs[j] & 0x0F) | (int)(((qh >> j) & 1u) << 4);
            int x1 = (int)(qs[j] >> 4) | (int)(((qh >> (j + 16)) & 1u) << 4);
            if (with_min) { y[j] = d * (float)x0 + m; y[j + 16] = d * (float)x1 + m; }
            else { y[j] = d * (float)(x0 - 16); y[j + 16] = d * (float)(x1 - 16); }
        }
    }
}

static void dequant_q8_1(const uint8_t *data, size_t nblocks, float *out)
{
    for (size_t b = 0; b < nblocks; b++) {
        const uint8_t *p = data + b * 36;
        float d = f16_at(p);
        for (int j = 0; j < 32; j++) out[b * 32 + j] = d * (float)(int8_t)p[4 + j];
    }
}

/* crates/tl_runtime/src/quantized.rs:182-225 */
static void dequant_q4_0(const uint8_t *data, size_t nblocks, float *out)
{
    for (size_t b = 0; b < nblocks; b++) {
        const uint8_t *p = data + b * 18;
        float d = f16_at(p);
        float *y = out + b * 32;
        for (int j = 0; j < 16; j++) {
            uint8_t byte = p[2 + j];
            int x0 = (int)(byte & 0x0F) - 8;
            int x1 = (int)((byte >> 4) & 0x0F) - 8;
            y[j] = d * (float)x0;
            y[j + 16] = d * (float)x1;
        }
    }
}

/* crates/tl_runtime/src/quantized.rs:227-260 */
static void dequant_q8_0(const uint8_t *data, size_t nblocks, float *out)
{
    for (size_t b = 0; b < nblocks; b++) {
        const uint8_t *p = data + b * 34;
        float d = f16_at(p);
        for (int j = 0; j < 32; j++) out[b * 32 + j] = d * (float)(int8_t)p[2 + j];
    }
}

/* crates/tl_runtime/src/quantized.rs:268-329.  Note the reference's scale index:
 * is = l/16 and the four scales are scales[is+0], [is+2], [is+4], [is+6]; the product
 * is evaluated left to right: (d * sc) * q. */
static void dequant_q6_k(const uint8_t *data, size_t nblocks, float *out)
{
    for (size_t b = 0; b < nblocks; b++) {
        const uint8_t *base = data + b * 210;
        float d = f16_at(base + 208);
        const uint8_t *ql = base, *qh = base + 128, *sc = base + 192;
        float *y = out + b * 256;
        for (int chunk = 0; chunk < 2; chunk++) {
            float *yc = y + chunk * 128;
            for (int l = 0; l < 32; l++) {
                int is = l / 16;
                uint8_t ql_lo = ql[l], ql_hi = ql[l + 32], qhv = qh[l];
                int q1 = (int)((ql_lo & 0xF) | (((qhv >> 0) & 3) << 4)) - 32;
                int q2 = (int)((ql_hi & 0xF) | (((qhv >> 2) & 3) << 4)) - 32;
                int q3 = (int)((ql_lo >> 4) | (((qhv >> 4) & 3) << 4)) - 32;
                int q4 = (int)((ql_hi >> 4) | (((qhv >> 6) & 3) << 4)) - 32;
                float s1 = (float)(int8_t)sc[is + 0], s2 = (float)(int8_t)sc[is + 2];
                float s3 = (float)(int8_t)sc[is + 4], s4 = (float)(int8_t)sc[is + 6];
                yc[l + 0] = d * s1 * (float)q1;
                yc[l + 32] = d * s2 * (float)q2;
                yc[l + 64] = d * s3 * (float)q3;
                yc[l + 96] = d * s4 * (float)q4;
            }
            ql += 64; qh += 32; sc += 8;
        }
    }
}

/* crates/tl_runtime/src/quantized.rs:404-415 */
static inline void scale_min_k4(int j, const uint8_t *s, uint8_t *sc, uint8_t *m)
{
    if (j < 4) {
        *sc = s[j] & 63;
        *m = s[j + 4] & 63;
    } else {
        *sc = (uint8_t)((s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4));
        *m = (uint8_t)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
    }
}

/* crates/tl_runtime/src/quantized.rs:337-402: d1 = d*sc; min1 = dmin*m; w = d1*q - min1
 * (two multiplies and one subtract, never fused). */
static void dequant_q4_k(const uint8_t *data, size_t nblocks, float *out)
{
    for (size_t b = 0; b < nblocks; b++) {
        const uint8_t *base = data + b * 144;
        float d = f16_at(base), dmin = f16_at(base + 2);
        const uint8_t *scales = base + 4, *q = base + 16;
        float *y = out + b * 256;
        int is = 0;
        for (int j = 0; j < 256; j += 64) {
            uint8_t sc1, m1, sc2, m2;
            scale_min_k4(is, scales, &sc1, &m1);
            float d1 = d * (float)sc1, min1 = dmin * (float)m1;
            scale_min_k4(is + 1, scales, &sc2, &m2);
            float d2 = d * (float)sc2, min2 = dmin * (float)m2;
            for (int l = 0; l < 32; l++) y[j + l] = d1 * (float)(q[l] & 0xF) - min1;
            for (int l = 0; l < 32; l++) y[j + 32 + l] = d2 * (float)(q[l] >> 4) - min2;
            q += 32;
            is += 2;
        }
    }
}

int orc_dequantize(int type, const uint8_t *data, size_t nbytes, size_t nelem, float *out)
{
    size_t need = orc_type_nbytes(type, nelem);
    if (nelem != 0 && (need == 0 || need != nbytes)) return -1;
    switch (type) {
    case ORC_F32: memcpy(out, data, nelem * 4); return 0;
    case ORC_F16: /* quantized.rs:167-180 */
        for (size_t i = 0; i < nelem; i++) out[i] = f16_at(data + 2 * i);
        return 0;
    case ORC_Q4_0: dequant_q4_0(data, nelem / 32, out); return 0;
    case ORC_Q8_0: dequant_q8_0(data, nelem / 32, out); return 0;
    case ORC_Q4_K: dequant_q4_k(data, nelem / 256, out); return 0;
    case ORC_Q6_K: dequant_q6_k(data, nelem / 256, out); return 0;
    case ORC_Q4_1: dequant_q4_1(data, nelem / 32, out); return 0;
    case ORC_Q5_0: dequant_q5(data, nelem / 32, out, 0); return 0;
    case ORC_Q5_1: dequant_q5(data, nelem / 32, out, 1); return 0;
    case ORC_Q8_1: dequant_q8_1(data, nelem / 32, out); return 0;
    default: return -1;
    }
}

/* ---------------------------------------------------------------- matmul */

void orc_matmul(const float *a, const float *b, float *out,
                size_t batch, size_t m, size_t k, size_t n, int b_batched)
{
    for (size_t bi = 0; bi < batch; bi++) {
        const float *A = a + bi * m * k;
        const float *B = b + (b_batched ? bi * k * n : 0);
        float *C = out + bi * m * n;
        for (size_t i = 0; i < m; i++)
            for (size_t j = 0; j < n; j++) {
                float sum = 0.0f;
                for (size_t p = 0; p < k; p++) sum += A[i * k + p] * B[p * n + j];
                C[i * n + j] = sum;
            }
    }
}

/* Output columns are independent, so they are spread over the host threads (OpenMP); every dot product
 * still runs in the reference's sequential order, so results do not depend on the thread count.  The timed
 * CPU baseline (orc_matmul_cached_t_cols) stays single-threaded, as the reference is. */
void orc_matmul_wt(const float *w, size_t n, size_t k, const float *x, size_t m, float *out)
{
#pragma omp parallel for schedule(static)
    for (size_t j = 0; j < n; j++) {
        const float *wr = w + j * k;
        for (size_t i = 0; i < m; i++) {
            const float *xr = x + i * k;
            float sum = 0.0f;
            for (size_t p = 0; p < k; p++) sum += xr[p] * wr[p];
            out[i * n + j] = sum;
        }
    }
}

void orc_matmul_cached_t(const float *w_kn, size_t n, size_t k, const float *x, size_t m, float *out)
{
    orc_matmul(x, w_kn, out, 1, m, k, n, 0);
}

static size_t type_row_bytes(int type, size_t k) { return orc_type_nbytes(type, k); }

int orc_qmatmul(int type, const uint8_t *w, size_t n, size_t k,
                const float *x, size_t m, float *out)
{
    size_t rb = type_row_bytes(type, k);
    if (rb == 0) return -1;
    int bad = 0;
#pragma omp parallel
    {
        float *row = (float *)malloc(k * sizeof(float));
        if (!row) {
#pragma omp atomic write
            bad = 2;
        }
#pragma omp for schedule(static)
        for (size_t j = 0; j < n; j++) {
            if (!row) continue;
            if (orc_dequantize(type, w + j * rb, rb, k, row)) {
#pragma omp atomic write
                bad = 1;
                continue;
            }
            for (size_t i = 0; i < m; i++) {
                const float *xr = x + i * k;
                float sum = 0.0f;
                for (size_t p = 0; p < k; p++) sum += xr[p] * row[p];
                out[i * n + j] = sum;
            }
        }
        free(row);
    }
    return bad ? -bad : 0;
}

/* ---------------------------------------------------------------- norm / rope / misc */

void orc_rms_norm(const float *x, const float *w, float eps, size_t rows, size_t d, float *out)
{
    for (size_t g = 0; g < rows; g++) {
        const float *xr = x + g * d;
        float s = 0.0f;
        for (size_t i = 0; i < d; i++) s += xr[i] * xr[i];
        float mean_sq = s / (float)d;
        float rms = sqrtf(mean_sq + eps);
        for (size_t i = 0; i < d; i++) out[g * d + i] = xr[i] / rms;
    }
    if (w) /* second pass = mul_impl(weight) broadcast over rows */
        for (size_t g = 0; g < rows; g++)
            for (size_t i = 0; i < d; i++) out[g * d + i] = out[g * d + i] * w[i];
}

void orc_rope_table_cpu(size_t seq_len, size_t dim, float base, float *cos_out, float *sin_out)
{
    size_t half = dim / 2;
    for (size_t pos = 0; pos < seq_len; pos++)
        for (size_t i = 0; i < half; i++) {
            float freq = 1.0f / powf(base, 2.0f * (float)i / (float)dim);
            float ang = (float)pos * freq;
            float c = cosf(ang), s = sinf(ang);
            if (cos_out) { cos_out[pos * dim + 2 * i] = c; cos_out[pos * dim + 2 * i + 1] = c; }
            if (sin_out) { sin_out[pos * dim + 2 * i] = s; sin_out[pos * dim + 2 * i + 1] = s; }
        }
}

void orc_apply_rope_cpu(const float *x, size_t total, size_t head_dim,
                        const float *cos_t, size_t cos_len, const float *sin_t, size_t sin_len,
                        float *out)
{
    if (head_dim == 0 || total == 0) return;
    size_t nvec = total / head_dim;
    for (size_t v = 0; v < nvec; v++) {
        size_t off = v * head_dim;
        for (size_t i = 0; i + 1 < head_dim + 1 && i < head_dim; i += 2) {
            float c = (i < cos_len) ? cos_t[i] : 1.0f;
            float s = (i < sin_len) ? sin_t[i] : 0.0f;
            float x0 = x[off + i], x1 = x[off + i + 1];
            out[off + i] = x0 * c - x1 * s;
            out[off + i + 1] = x0 * s + x1 * c;
        }
    }
}

void orc_rope_table_half(size_t seq_len, size_t dim, float base, float *cos_out, float *sin_out)
{
    size_t half = dim / 2;
    for (size_t pos = 0; pos < seq_len; pos++)
        for (size_t i = 0; i < half; i++) {
            float freq = 1.0f / powf(base, 2.0f * (float)i / (float)dim);
            float ang = (float)pos * freq;
            if (cos_out) cos_out[pos * half + i] = cosf(ang);
            if (sin_out) sin_out[pos * half + i] = sinf(ang);
        }
}

void orc_apply_rope_rotate_half(const float *x, size_t tokens, size_t heads, size_t head_dim,
                                const float *cos_t, const float *sin_t, float *out)
{
    size_t half = head_dim / 2;
    for (size_t t = 0; t < tokens; t++)
        for (size_t h = 0; h < heads; h++) {
            const float *xv = x + (t * heads + h) * head_dim;
            float *ov = out + (t * heads + h) * head_dim;
            for (size_t i = 0; i < half; i++) {
                float c = cos_t[t * half + i], s = sin_t[t * half + i];
                float x0 = xv[i], x1 = xv[i + half];
                ov[i] = x0 * c - x1 * s;
                ov[i + half] = x0 * s + x1 * c;
            }
        }
}

void orc_softmax(const float *x, size_t outer, size_t axis, size_t inner, float *out)
{
    for (size_t i = 0; i < outer; i++)
        for (size_t k = 0; k < inner; k++) {
            float mx = -INFINITY;
            for (size_t j = 0; j < axis; j++) {
                float v = x[i * axis * inner + j * inner + k];
                if (v > mx) mx = v;
            }
            float sum = 0.0f;
            for (size_t j = 0; j < axis; j++) {
                size_t idx = i * axis * inner + j * inner + k;
                out[idx] = expf(x[idx] - mx);
                sum += out[idx];
            }
            for (size_t j = 0; j < axis; j++) out[i * axis * inner + j * inner + k] /= sum;
        }
}

void orc_silu(const float *x, size_t n, float *out)
{
    for (size_t i = 0; i < n; i++) out[i] = x[i] * (1.0f / (1.0f + expf(-x[i])));
}

void orc_add(const float *a, const float *b, size_t n, size_t nb, float *out)
{
    for (size_t i = 0; i < n; i++) out[i] = a[i] + b[i % nb];
}
void orc_mul(const float *a, const float *b, size_t n, size_t nb, float *out)
{
    for (size_t i = 0; i < n; i++) out[i] = a[i] * b[i % nb];
}
void orc_scale(const float *a, float s, size_t n, float *out)
{
    for (size_t i = 0; i < n; i++) out[i] = a[i] * s;
}

int orc_embedding(const float *table, size_t vocab, size_t dim,
                  const float *idx, size_t n, float *out)
{
    for (size_t i = 0; i < n; i++) {
        long long id = (long long)idx[i];
        if (id < 0 || (size_t)id >= vocab) return -1;
        memcpy(out + i * dim, table + (size_t)id * dim, dim * sizeof(float));
    }
    return 0;
}

void orc_repeat_interleave(const float *x, size_t outer, size_t axis, size_t inner,
                           size_t repeats, float *out)
{
    size_t o = 0;
    for (size_t i = 0; i < outer; i++)
        for (size_t j = 0; j < axis; j++)
            for (size_t r = 0; r < repeats; r++)
                for (size_t k = 0; k < inner; k++) out[o++] = x[i * axis * inner + j * inner + k];
}

void orc_causal_mask(size_t size, float *out)
{
    for (size_t i = 0; i < size; i++)
        for (size_t j = 0; j < size; j++) out[i * size + j] = (j > i) ? -INFINITY : 0.0f;
}

/* Rust's Iterator::max_by keeps the LAST of equal maxima; a NaN compares as Equal
 * (partial_cmp -> None -> unwrap_or(Equal)), i.e. the later element wins. */
size_t orc_argmax_last(const float *x, size_t n)
{
    if (n == 0) return 0;
    size_t best = 0;
    for (size_t i = 1; i < n; i++) {
        float a = x[best], b = x[i];
        int greater = (a > b); /* Ordering::Greater keeps the old one */
        if (!greater) best = i;
    }
    return best;
}

size_t orc_argmax_first(const float *x, size_t n)
{
    size_t best = 0;
    for (size_t i = 1; i < n; i++)
        if (x[i] > x[best]) best = i;
    return best;
}

/* CpuTensor::sample_impl, crates/tl_cpu/src/tensor.rs:1625-1680, with the random number u in [0, 1) passed in
 * (the reference draws it from rand::thread_rng()).  temp <= 0: the greedy branch (last maximum). */
static const float *g_sort_probs;
static int cmp_prob_desc(const void *a, const void *b)
{
    size_t ia = *(const size_t *)a, ib = *(const size_t *)b;
    float pa = g_sort_probs[ia], pb = g_sort_probs[ib];
    if (pb > pa) return 1;
    if (pb < pa) return -1;
    return ia < ib ? -1 : (ia > ib ? 1 : 0); /* slice::sort_by is stable: equal probabilities keep index order */
}
/* Philox-4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC'11): the counter-based
 * generator the library's decode session draws from on the device.  No counterpart in the reference (it draws from
 * rand::thread_rng()). */
void orc_philox4x32_10(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4])
{
    uint32_t c0 = ctr[0], c1 = ctr[1], c2 = ctr[2], c3 = ctr[3], k0 = key[0], k1 = key[1];
    for (int r = 0; r < 10; r++) {
        uint64_t p0 = (uint64_t)0xD2511F53u * c0, p1 = (uint64_t)0xCD9E8D57u * c2;
        uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0, n1 = (uint32_t)p1, n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1, n3 = (uint32_t)p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

double orc_rng_uniform(uint64_t seed, uint64_t counter)
{
    uint32_t ctr[4] = { (uint32_t)counter, (uint32_t)(counter >> 32), 0u, 0u }, key[2] = { (uint32_t)seed, (uint32_t)(seed >> 32) }, o[4];
    orc_philox4x32_10(ctr, key, o);
    return (double)((float)(o[0] >> 8) * (1.0f / 16777216.0f));
}

size_t orc_sample_top_p(const float *logits, size_t n, float temp, float top_p, double u)
{
    return orc_sample_top_k_top_p(logits, n, temp, 0, top_p, u);
}

/* sample_impl with a top-k limit on the kept prefix (top_k <= 0: none): the extension the library adds */
size_t orc_sample_top_k_top_p(const float *logits, size_t n, float temp, long top_k, float top_p, double u)
{
    if (n == 0) return 0;
    if (temp <= 0.0f) return orc_argmax_last(logits, n);
    float *probs = (float *)malloc(n * sizeof(float));
    size_t *indices = (size_t *)malloc(n * sizeof(size_t));
    float max_val = -INFINITY;
    for (size_t i = 0; i < n; i++) {
        probs[i] = logits[i] / temp;
        if (!(max_val > probs[i])) max_val = probs[i];
    }
    float sum_exp = 0.0f;
    for (size_t i = 0; i < n; i++) sum_exp += expf(probs[i] - max_val);
    for (size_t i = 0; i < n; i++) probs[i] = expf(probs[i] - max_val) / sum_exp;
    for (size_t i = 0; i < n; i++) indices[i] = i;
    g_sort_probs = probs;
    qsort(indices, n, sizeof(size_t), cmp_prob_desc);
    float cum_prob = 0.0f;
    size_t limit = (top_k > 0 && (size_t)top_k < n) ? (size_t)top_k : n;
    size_t cutoff_index = limit - 1;
    for (size_t i = 0; i < limit; i++) {
        cum_prob += probs[indices[i]];
        if (cum_prob > top_p) { cutoff_index = i; break; }
    }
    float r = (float)u * cum_prob;
    float acc = 0.0f;
    size_t selected = indices[0];
    for (size_t i = 0; i <= cutoff_index; i++) {
        acc += probs[indices[i]];
        if (acc >= r) { selected = indices[i]; break; }
    }
    free(probs);
    free(indices);
    return selected;
}

void orc_repetition_penalty(const float *logits, size_t n, const float *tokens, size_t nt,
                            float penalty, float *out)
{
    memcpy(out, logits, n * sizeof(float));
    unsigned char *seen = (unsigned char *)calloc(n ? n : 1, 1);
    for (size_t t = 0; t < nt; t++) {
        if (tokens[t] < 0) continue; /* `as usize` saturates negatives to 0 in Rust */
        size_t i = (size_t)tokens[t];
        if (i < n) seen[i] = 1;
    }
    for (size_t t = 0; t < nt; t++)
        if (tokens[t] < 0 && n > 0) seen[0] = 1;
    for (size_t i = 0; i < n; i++)
        if (seen[i]) out[i] = (out[i] > 0.0f) ? out[i] / penalty : out[i] * penalty;
    free(seen);
}

void orc_sdpa_cpu(const float *q, const float *k, const float *v, const float *mask,
                  size_t bh, size_t sq, size_t sk, size_t d, float *out)
{
    float scale = 1.0f / sqrtf((float)d);
    float *sc = (float *)malloc(sq * sk * sizeof(float));
    for (size_t h = 0; h < bh; h++) {
        const float *Q = q + h * sq * d, *K = k + h * sk * d, *V = v + h * sk * d;
        for (size_t i = 0; i < sq; i++)
            for (size_t j = 0; j < sk; j++) {
                float s = 0.0f;
                for (size_t e = 0; e < d; e++) s += Q[i * d + e] * K[j * d + e];
                sc[i * sk + j] = s * scale;
            }
        if (mask)
            for (size_t i = 0; i < sq; i++)
                for (size_t j = 0; j < sk; j++)
                    if (mask[i * sk + j] == 0.0f) sc[i * sk + j] = -1e9f;
        for (size_t i = 0; i < sq; i++) {
            float mx = -INFINITY;
            for (size_t j = 0; j < sk; j++) mx = fmaxf(mx, sc[i * sk + j]);
            float sum = 0.0f;
            for (size_t j = 0; j < sk; j++) {
                sc[i * sk + j] = expf(sc[i * sk + j] - mx);
                sum += sc[i * sk + j];
            }
            for (size_t j = 0; j < sk; j++) sc[i * sk + j] /= sum;
        }
        for (size_t i = 0; i < sq; i++)
            for (size_t j = 0; j < d; j++) {
                float s = 0.0f;
                for (size_t l = 0; l < sk; l++) s += sc[i * sk + l] * V[l * d + j];
                out[h * sq * d + i * d + j] = s;
            }
    }
    free(sc);
}

/* ---------------------------------------------------------------- Llama driver */

typedef struct { int type; const uint8_t *data; size_t nbytes; } orc_tensor;

enum { T_ATTN_NORM, T_FFN_NORM, T_Q, T_K, T_V, T_O, T_GATE, T_UP, T_DOWN, T_PER_LAYER };

struct orc_llama {
    orc_llama_cfg cfg;
    orc_tensor token_embd, output_norm, output;
    orc_tensor *layers; /* n_layers * T_PER_LAYER */
    float *kc, *vc;     /* [L][KVH][max_seq][D] */
    int cache_len;
    float *cos_t, *sin_t; /* [max_seq, D] pair-duplicated tables */
    float *hidden;
};

orc_llama *orc_llama_new(const orc_llama_cfg *cfg)
{
    orc_llama *m = (orc_llama *)calloc(1, sizeof(*m));
    if (!m) return NULL;
    m->cfg = *cfg;
    size_t L = (size_t)cfg->n_layers, kvd = (size_t)cfg->n_kv_heads * cfg->head_dim;
    m->layers = (orc_tensor *)calloc(L * T_PER_LAYER, sizeof(orc_tensor));
    m->kc = (float *)calloc(L * kvd * cfg->max_seq, sizeof(float));
    m->vc = (float *)calloc(L * kvd * cfg->max_seq, sizeof(float));
    m->cos_t = (float *)malloc((size_t)cfg->max_seq * cfg->head_dim * sizeof(float));
    m->sin_t = (float *)malloc((size_t)cfg->max_seq * cfg->head_dim * sizeof(float));
    m->hidden = (float *)calloc((size_t)cfg->d_model, sizeof(float));
    if (!m->layers || !m->kc || !m->vc || !m->cos_t || !m->sin_t || !m->hidden) {
        orc_llama_free(m);
        return NULL;
    }
    orc_rope_table_cpu((size_t)cfg->max_seq, (size_t)cfg->head_dim, cfg->rope_base, m->cos_t, m->sin_t);
    return m;
}

void orc_llama_free(orc_llama *m)
{
    if (!m) return;
    free(m->layers); free(m->kc); free(m->vc); free(m->cos_t); free(m->sin_t); free(m->hidden);
    free(m);
}

int orc_llama_set_tensor(orc_llama *m, const char *name, int type, const uint8_t *data, size_t nbytes)
{
    orc_tensor t = { type, data, nbytes };
    if (!strcmp(name, "token_embd.weight")) { m->token_embd = t; return 0; }
    if (!strcmp(name, "output_norm.weight")) { m->output_norm = t; return 0; }
    if (!strcmp(name, "output.weight")) { m->output = t; return 0; }
    int li = -1, consumed = 0;
    if (sscanf(name, "blk.%d.%n", &li, &consumed) != 1 || li < 0 || li >= m->cfg.n_layers) return -1;
    const char *rest = name + consumed;
    static const char *names[T_PER_LAYER] = {
        "attn_norm.weight", "ffn_norm.weight", "attn_q.weight", "attn_k.weight", "attn_v.weight",
        "attn_output.weight", "ffn_gate.weight", "ffn_up.weight", "ffn_down.weight" };
    for (int i = 0; i < T_PER_LAYER; i++)
        if (!strcmp(rest, names[i])) { m->layers[(size_t)li * T_PER_LAYER + i] = t; return 0; }
    return -1;
}

static size_t kv_index(const orc_llama *m, int layer, int kvh, int pos)
{
    const orc_llama_cfg *c = &m->cfg;
    return (((size_t)layer * c->n_kv_heads + kvh) * c->max_seq + pos) * c->head_dim;
}

void orc_llama_kv_write(orc_llama *m, int layer, int pos, const float *k, const float *v)
{
    const orc_llama_cfg *c = &m->cfg;
    for (int h = 0; h < c->n_kv_heads; h++) {
        memcpy(m->kc + kv_index(m, layer, h, pos), k + (size_t)h * c->head_dim, c->head_dim * sizeof(float));
        memcpy(m->vc + kv_index(m, layer, h, pos), v + (size_t)h * c->head_dim, c->head_dim * sizeof(float));
    }
    if (pos + 1 > m->cache_len) m->cache_len = pos + 1;
}

void orc_llama_kv_clear(orc_llama *m) { m->cache_len = 0; }

const float *orc_llama_last_hidden(const orc_llama *m) { return m->hidden; }

/* dequantised 1-D / f32 tensors come through tl_tensor_map_get
 * (crates/tl_runtime/src/tensor_map.rs:110-150): full dequantise to f32. */
static float *dequant_all(const orc_tensor *t, size_t nelem)
{
    float *o = (float *)malloc(nelem * sizeof(float));
    if (!o) return NULL;
    if (orc_dequantize(t->type, t->data, t->nbytes, nelem, o)) { free(o); return NULL; }
    return o;
}

static int linear(const orc_tensor *w, size_t n, size_t k, const float *x, size_t m, float *out)
{
    if (!w->data) return -1;
    if (w->type == ORC_F32) { orc_matmul_wt((const float *)w->data, n, k, x, m, out); return 0; }
    return orc_qmatmul(w->type, w->data, n, k, x, m, out);
}

int orc_llama_forward(orc_llama *m, const int32_t *tokens, int n, int start_pos, float *logits_out)
{
    const orc_llama_cfg *c = &m->cfg;
    size_t d = c->d_model, H = c->n_heads, KVH = c->n_kv_heads, D = c->head_dim, F = c->ffn;
    size_t qd = H * D, kvd = KVH * D, rep = H / KVH, sl = (size_t)n;
    if (n <= 0 || start_pos < 0 || start_pos + n > c->max_seq) return -1;
    if (n > 1 && start_pos != 0) return -2; /* the TL program's causal mask assumes sp == 0 */
    size_t T = (size_t)start_pos + sl;
    int rc = -3;

    float *x = (float *)malloc(sl * d * 4), *h = (float *)malloc(sl * d * 4);
    float *q = (float *)malloc(sl * qd * 4), *k = (float *)malloc(sl * kvd * 4), *v = (float *)malloc(sl * kvd * 4);
    float *qr = (float *)malloc(sl * qd * 4), *kr = (float *)malloc(sl * kvd * 4);
    float *sc = (float *)malloc(sl * T * 4), *ao = (float *)malloc(sl * qd * 4);
    float *t1 = (float *)malloc(sl * d * 4), *g = (float *)malloc(sl * F * 4), *u = (float *)malloc(sl * F * 4);
    float *nw = NULL;
    if (!x || !h || !q || !k || !v || !qr || !kr || !sc || !ao || !t1 || !g || !u) goto done;

    /* embedding: ids travel as f32 (crates/tl_cpu/src/tensor.rs:1094-1112) */
    for (size_t i = 0; i < sl; i++) {
        int32_t id = tokens[i];
        if (id < 0 || id >= c->vocab) { rc = -4; goto done; }
        size_t rb = orc_type_nbytes(m->token_embd.type, d);
        if (!m->token_embd.data || rb == 0) { rc = -5; goto done; }
        if (orc_dequantize(m->token_embd.type, m->token_embd.data + (size_t)id * rb, rb, d, x + i * d)) { rc = -5; goto done; }
    }

    const float *cs = m->cos_t + (size_t)start_pos * D; /* cos.narrow(0, sp, sl): row 0 = sp */
    const float *ss = m->sin_t + (size_t)start_pos * D;
    size_t tab_len = sl * D;

    for (int li = 0; li < c->n_layers; li++) {
        const orc_tensor *lt = m->layers + (size_t)li * T_PER_LAYER;
        /* attn_norm */
        free(nw); nw = dequant_all(&lt[T_ATTN_NORM], d);
        if (!nw) { rc = -6; goto done; }
        orc_rms_norm(x, nw, c->eps, sl, d, h);
        if (linear(&lt[T_Q], qd, d, h, sl, q) || linear(&lt[T_K], kvd, d, h, sl, k) ||
            linear(&lt[T_V], kvd, d, h, sl, v)) { rc = -7; goto done; }
        /* RoPE on [1,sl,H,D] and [1,sl,KVH,D] */
        orc_apply_rope_cpu(q, sl * qd, D, cs, tab_len, ss, tab_len, qr);
        orc_apply_rope_cpu(k, sl * kvd, D, cs, tab_len, ss, tab_len, kr);
        /* transpose(1,2) + cat into the cache */
        for (size_t i = 0; i < sl; i++)
            for (size_t kh = 0; kh < KVH; kh++) {
                float *kd = m->kc + kv_index(m, li, (int)kh, start_pos + (int)i);
                float *vd = m->vc + kv_index(m, li, (int)kh, start_pos + (int)i);
                for (size_t e = 0; e < D; e++) {
                    float kk = kr[i * kvd + kh * D + e], vv = v[i * kvd + kh * D + e];
                    if (c->kv_f16) { kk = orc_f16_to_f32(orc_f32_to_f16(kk)); vv = orc_f16_to_f32(orc_f32_to_f16(vv)); }
                    kd[e] = kk; vd[e] = vv;
                }
            }
        /* per head: scores = q k^T, scale, (+mask), softmax, p v */
        for (size_t hd = 0; hd < H; hd++) {
            size_t kh = hd / rep; /* repeat_interleave(rep, 1) */
            const float *K = m->kc + kv_index(m, li, (int)kh, 0);
            const float *V = m->vc + kv_index(m, li, (int)kh, 0);
            for (size_t i = 0; i < sl; i++) {
                const float *qv = qr + i * qd + hd * D;
                for (size_t t = 0; t < T; t++) {
                    float s = 0.0f;
                    for (size_t e = 0; e < D; e++) s += qv[e] * K[t * D + e];
                    s = s * c->attn_scale;
                    if (sl > 1) s = s + ((t > i) ? -INFINITY : 0.0f);
                    sc[i * T + t] = s;
                }
            }
            orc_softmax(sc, sl, T, 1, sc);
            for (size_t i = 0; i < sl; i++)
                for (size_t e = 0; e < D; e++) {
                    float s = 0.0f;
                    for (size_t t = 0; t < T; t++) s += sc[i * T + t] * V[t * D + e];
                    ao[i * qd + hd * D + e] = s; /* transpose(1,2).reshape([sl, H*D]) */
                }
        }
        if (linear(&lt[T_O], d, qd, ao, sl, t1)) { rc = -7; goto done; }
        orc_add(x, t1, sl * d, sl * d, x); /* h = x + attn_out */
        free(nw); nw = dequant_all(&lt[T_FFN_NORM], d);
        if (!nw) { rc = -6; goto done; }
        orc_rms_norm(x, nw, c->eps, sl, d, h);
        if (linear(&lt[T_GATE], F, d, h, sl, g)) { rc = -7; goto done; }
        orc_silu(g, sl * F, g);
        if (linear(&lt[T_UP], F, d, h, sl, u)) { rc = -7; goto done; }
        orc_mul(g, u, sl * F, sl * F, g);
        if (linear(&lt[T_DOWN], d, F, g, sl, t1)) { rc = -7; goto done; }
        orc_add(x, t1, sl * d, sl * d, x);
    }
    if ((int)T > m->cache_len) m->cache_len = (int)T;
    memcpy(m->hidden, x + (sl - 1) * d, d * sizeof(float));
    /* output_norm + head; the TL program runs the head on all rows and narrows to the last;
     * rows are independent, so only the last is computed here. */
    free(nw); nw = dequant_all(&m->output_norm, d);
    if (!nw) { rc = -6; goto done; }
    orc_rms_norm(x + (sl - 1) * d, nw, c->eps, 1, d, h);
    if (linear(&m->output, (size_t)c->vocab, d, h, 1, logits_out)) { rc = -7; goto done; }
    rc = 0;
done:
    free(x); free(h); free(q); free(k); free(v); free(qr); free(kr); free(sc); free(ao);
    free(t1); free(g); free(u); free(nw);
    return rc;
}

/* Columns [j0, j1) of orc_matmul_cached_t: the same inner loop (stride n through the cached
 * transposed weights, crates/tl_cpu/src/tensor.rs:1284-1306) over a subset of the outputs.
 * Used to time a bounded sample of a large matvec; out has (j1 - j0) entries per row. */
void orc_matmul_cached_t_cols(const float *w_kn, size_t n, size_t k, const float *x, size_t m,
                              size_t j0, size_t j1, float *out)
{
    for (size_t i = 0; i < m; i++)
        for (size_t j = j0; j < j1; j++) {
            float sum = 0.0f;
            for (size_t p = 0; p < k; p++) sum += x[i * k + p] * w_kn[p * n + j];
            out[i * (j1 - j0) + (j - j0)] = sum;
        }
}
