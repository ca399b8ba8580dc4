/*
 * wr_oracle.c — CPU restatement of the wayruntime GQA-attention hot path.
 *
 * TEST INFRASTRUCTURE ONLY (see wr_oracle.h).  Compile with
 *   gcc -std=c11 -O2 -ffp-contract=off -fopenmp
 * -ffp-contract=off matters: the reference objects contain no fused
 * multiply-add, and the RoPE / exp results are compared bit for bit.
 */
#include "wr_oracle.h"

#include <stdlib.h>
#include <string.h>

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float    u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* ------------------------------------------------------------------ mathx */

static const float LN2F   = 0.6931471805599453f;
static const float PIF    = 3.14159265358979f;
static const float TWOPIF = 6.28318530717958f;

/* src/core/mathx.c:37-57 — clamp, k = trunc(x/ln2 +- 0.5), degree-5 Taylor on
 * the residual, then k added into the exponent field. */
float wro_exp(float x)
{
    if (x < -88.0f) return 0.0f;
    if (x > 88.0f)  return 1e38f;
    float bias = (x >= 0) ? 0.5f : -0.5f;
    int   k    = (int)(x / LN2F + bias);
    float r    = x - (float)k * LN2F;
    float r2   = r * r;
    float t2   = r2 * 0.5f;
    float t3   = r2 * r * (1.0f / 6.0f);
    float t4   = r2 * r2 * (1.0f / 24.0f);
    float t5   = r2 * r2 * r * (1.0f / 120.0f);
    float e    = 1.0f + r + t2 + t3 + t4 + t5;
    if (k >= -126 && k <= 127)
        e = u2f(f2u(e) + ((uint32_t)k << 23));
    return e;
}

/* src/core/mathx.c:72-86 — mantissa/exponent split + 4-term atanh series. */
float wro_log(float x)
{
    if (x <= 0.0f) return -1e38f;
    uint32_t u = f2u(x);
    int      e = (int)((u >> 23) & 0xFF) - 127;
    float    m = u2f((u & 0x007FFFFFu) | 0x3F800000u);
    float    t = (m - 1.0f) / (m + 1.0f);
    float    t2 = t * t;
    float    series = 1.0f + t2 * (1.0f / 3.0f + t2 * (1.0f / 5.0f + t2 * (1.0f / 7.0f)));
    float    lnm = 2.0f * t * series;
    return lnm + (float)e * LN2F;
}

/* src/core/mathx.c:98-110 — halved-bit-pattern seed, four Newton steps. */
float wro_sqrt(float x)
{
    if (x <= 0) return 0;
    float g = u2f((f2u(x) + 0x3f800000u) >> 1);
    for (int it = 0; it < 4; it++)
        g = 0.5f * (g + x / g);
    return g;
}

/* src/core/mathx.c:124-147 — reduce by repeated +-2pi, then truncated Taylor. */
static float reduce_pi(float x)
{
    while (x >  PIF) x -= TWOPIF;
    while (x < -PIF) x += TWOPIF;
    return x;
}

float wro_sin(float x)
{
    x = reduce_pi(x);
    float x2 = x * x;
    float x3 = x2 * x;
    float x5 = x3 * x2;
    float x7 = x5 * x2;
    return x - x3 * (1.0f / 6.0f) + x5 * (1.0f / 120.0f) - x7 * (1.0f / 5040.0f);
}

float wro_cos(float x)
{
    x = reduce_pi(x);
    float x2 = x * x;
    float x4 = x2 * x2;
    float x6 = x4 * x2;
    return 1.0f - x2 * 0.5f + x4 * (1.0f / 24.0f) - x6 * (1.0f / 720.0f);
}

/* ------------------------------------------------------------------- f16 */

/* src/core/quant.c:86-114 — exact widening, subnormals renormalised. */
float wro_f16_to_f32(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t ex   = (h >> 10) & 0x1Fu;
    uint32_t man  = h & 0x3FFu;
    if (ex == 0x1Fu)
        return u2f(sign | 0x7F800000u | (man << 13));
    if (ex == 0) {
        if (man == 0)
            return u2f(sign);
        int shift = 0;
        while (!(man & 0x400u)) { man <<= 1; shift++; }
        man &= 0x3FFu;
        return u2f(sign | ((uint32_t)(113 - shift) << 23) | (man << 13));
    }
    return u2f(sign | ((ex + 112u) << 23) | (man << 13));
}

/* src/core/quant.c:121-136 — drop 13 mantissa bits; biased exponent <= 0
 * becomes signed zero, >= 31 becomes infinity (NaN included). */
uint16_t wro_f32_to_f16(float f)
{
    uint32_t b    = f2u(f);
    uint16_t sign = (uint16_t)((b >> 16) & 0x8000u);
    int32_t  ex   = (int32_t)((b >> 23) & 0xFFu) - 112;
    if (ex <= 0)  return sign;
    if (ex >= 31) return (uint16_t)(sign | 0x7C00u);
    return (uint16_t)(sign | ((uint32_t)ex << 10) | ((b >> 13) & 0x3FFu));
}

void wro_f32_to_f16_n(const float *src, uint16_t *dst, uint64_t n)
{
    for (uint64_t i = 0; i < n; i++) dst[i] = wro_f32_to_f16(src[i]);
}

void wro_f16_to_f32_n(const uint16_t *src, float *dst, uint64_t n)
{
    for (uint64_t i = 0; i < n; i++) dst[i] = wro_f16_to_f32(src[i]);
}

/* ------------------------------------------------------------------ RoPE */

/* src/core/kernels.c:1374-1405. */
void wro_rope_table(uint32_t pos, uint32_t hd, float theta_base,
                    uint32_t n_rot_pairs, float *cs, float *sn, uint8_t *rot)
{
    uint32_t half = hd / 2;
    if (theta_base < 1.0f) theta_base = 10000.0f;
    float lnb = wro_log(theta_base);
    uint32_t n_rot = half;
    if (n_rot_pairs >= 1 && n_rot_pairs < half) n_rot = n_rot_pairs;
    for (uint32_t j = 0; j < half; j++) {
        if (j >= n_rot) {
            cs[j] = 1.0f; sn[j] = 0.0f;
            if (rot) rot[j] = 0;
            continue;
        }
        float exponent = (float)(2 * j) / (float)hd;
        float powv  = wro_exp(exponent * lnb);
        float angle = (float)pos / powv;
        cs[j] = wro_cos(angle);
        sn[j] = wro_sin(angle);
        if (rot) rot[j] = 1;
    }
}

/* src/core/kernels.c:1356-1412 — element j pairs with j + hd/2. */
int wro_rope(const float *x, float *out, uint32_t seq, uint32_t heads,
             uint32_t hd, uint32_t pos, float theta_base, uint32_t n_rot_pairs)
{
    if (!x || !out) return WRO_ERR_INVAL;
    if (hd < 2 || (hd & 1) || heads == 0) return WRO_ERR_INVAL;
    uint32_t half = hd / 2;
    float   *cs  = (float *)malloc(sizeof(float) * half);
    float   *sn  = (float *)malloc(sizeof(float) * half);
    uint8_t *rot = (uint8_t *)malloc(half);
    if (!cs || !sn || !rot) { free(cs); free(sn); free(rot); return WRO_ERR_NOMEM; }
    for (uint32_t s = 0; s < seq; s++) {
        wro_rope_table(pos + s, hd, theta_base, n_rot_pairs, cs, sn, rot);
        for (uint32_t h = 0; h < heads; h++) {
            const float *src = x   + ((uint64_t)s * heads + h) * hd;
            float       *dst = out + ((uint64_t)s * heads + h) * hd;
            for (uint32_t j = 0; j < half; j++) {
                float a = src[j], b = src[j + half];
                if (!rot[j]) { dst[j] = a; dst[j + half] = b; continue; }
                dst[j]        = a * cs[j] - b * sn[j];
                dst[j + half] = a * sn[j] + b * cs[j];
            }
        }
    }
    free(cs); free(sn); free(rot);
    return WRO_OK;
}

/* ------------------------------------------------------------- KV append */

/* src/core/session.c:139-154. */
int wro_kv_append_row(uint16_t *cache, uint32_t cap_rows, uint32_t *valid_rows,
                      const float *row, uint32_t row_elems)
{
    if (!cache || !row || !valid_rows) return WRO_ERR_INTERNAL;
    uint32_t at = *valid_rows;
    if (at >= cap_rows) return WRO_ERR_CTX_FULL;
    uint16_t *dst = cache + (uint64_t)at * row_elems;
    for (uint32_t i = 0; i < row_elems; i++)
        dst[i] = wro_f32_to_f16(row[i]);
    *valid_rows = at + 1;
    return WRO_OK;
}

/* -------------------------------------------------------------- attention */

static inline float ld(const void *p, int dtype, uint64_t i)
{
    return dtype == WRO_F32 ? ((const float *)p)[i]
                            : wro_f16_to_f32(((const uint16_t *)p)[i]);
}

/* One (query row, q head) of src/core/kernels.c:1475-1523 over keys
 * [k_begin, k_end) with keys below key_lo masked.  Leaves the unnormalised
 * accumulator in o[hd] and returns the running max / denominator. */
static void attend_head(const void *q, int q_dtype, uint64_t q_off,
                        const void *k, const void *v, int kv_dtype,
                        uint32_t n_kv, uint32_t kvh, uint32_t hd,
                        uint64_t k_begin, uint64_t k_end, uint64_t key_lo,
                        float scale, float *o, float *m_io, float *l_io)
{
    float m = -1e30f, l = 0;
    for (uint32_t d = 0; d < hd; d++) o[d] = 0.0f;
    float S[WRO_FLASH_BLOCK];
    for (uint64_t t0 = k_begin; t0 < k_end; t0 += WRO_FLASH_BLOCK) {
        uint64_t bn = k_end - t0;
        if (bn > WRO_FLASH_BLOCK) bn = WRO_FLASH_BLOCK;
        float tmax = -1e30f;
        for (uint64_t b = 0; b < bn; b++) {
            uint64_t key = t0 + b;
            if (key < key_lo) { S[b] = -1e30f; continue; }
            uint64_t k_off = (key * n_kv + kvh) * hd;
            float dot = 0;
            for (uint32_t d = 0; d < hd; d++)
                dot += ld(q, q_dtype, q_off + d) * ld(k, kv_dtype, k_off + d);
            S[b] = dot * scale;
            if (S[b] > tmax) tmax = S[b];
        }
        float m_new = (m > tmax) ? m : tmax;
        float a = (m == -1e30f) ? 0.0f : wro_exp(m - m_new);
        for (uint32_t d = 0; d < hd; d++) o[d] *= a;
        l *= a;
        for (uint64_t b = 0; b < bn; b++) {
            float pw = wro_exp(S[b] - m_new);
            l += pw;
            uint64_t v_off = ((t0 + b) * n_kv + kvh) * hd;
            for (uint32_t d = 0; d < hd; d++)
                o[d] += pw * ld(v, kv_dtype, v_off + d);
        }
        m = m_new;
    }
    *m_io = m; *l_io = l;
}

static int attn_check(uint32_t seq_q, uint32_t n_q, uint32_t n_kv, uint32_t hd,
                      uint32_t seq_k, uint32_t max_seq)
{
    /* src/core/kernels.c:1429-1447 */
    if (n_q == 0 || n_kv == 0 || hd == 0 || seq_q == 0) return WRO_ERR_INVAL;
    if (n_q % n_kv != 0) return WRO_ERR_INVAL;
    if (seq_k == 0) return WRO_ERR_INVAL;
    if (seq_k > max_seq) return WRO_ERR_LIMIT;
    if (hd > WRO_FLASH_D_MAX) return WRO_ERR_LIMIT;
    return WRO_OK;
}

static float pick_scale(float scale_override, uint32_t hd)
{
    return (scale_override > 0.0f) ? scale_override : 1.0f / wro_sqrt((float)hd);
}

int wro_gqa_attention(const void *q, int q_dtype, const void *k, const void *v,
                      int kv_dtype, float *out, uint32_t seq_q, uint32_t n_q,
                      uint32_t n_kv, uint32_t hd, uint32_t seq_k,
                      float scale_override, uint32_t window, uint32_t max_seq)
{
    if (!q || !k || !v || !out) return WRO_ERR_INVAL;
    int rc = attn_check(seq_q, n_q, n_kv, hd, seq_k, max_seq);
    if (rc != WRO_OK) return rc;
    uint32_t group = n_q / n_kv;
    float scale = pick_scale(scale_override, hd);
    uint64_t key_lo = (window > 0 && seq_k > window) ? seq_k - window : 0;
    float *o = (float *)malloc(sizeof(float) * hd);
    if (!o) return WRO_ERR_NOMEM;
    for (uint32_t qs = 0; qs < seq_q; qs++) {
        for (uint32_t qh = 0; qh < n_q; qh++) {
            uint64_t row = ((uint64_t)qs * n_q + qh) * hd;
            float m, l;
            attend_head(q, q_dtype, row, k, v, kv_dtype, n_kv, qh / group, hd,
                        0, seq_k, key_lo, scale, o, &m, &l);
            float inv = (l > 0) ? 1.0f / l : 0.0f;
            for (uint32_t d = 0; d < hd; d++) out[row + d] = o[d] * inv;
        }
    }
    free(o);
    return WRO_OK;
}

int wro_decode_batch(const float *q, const uint16_t *const *k,
                     const uint16_t *const *v, const uint32_t *seq_k,
                     float *out, uint32_t n_sess, uint32_t n_q, uint32_t n_kv,
                     uint32_t hd, float scale_override, uint32_t window,
                     uint32_t max_seq, int threads)
{
    int worst = WRO_OK;
    if (threads < 1) threads = 1;
    #pragma omp parallel for schedule(dynamic, 1) num_threads(threads)
    for (uint32_t s = 0; s < n_sess; s++) {
        uint64_t off = (uint64_t)s * n_q * hd;
        int rc = wro_gqa_attention(q + off, WRO_F32, k[s], v[s], WRO_F16,
                                   out + off, 1, n_q, n_kv, hd, seq_k[s],
                                   scale_override, window, max_seq);
        if (rc != WRO_OK) {
            #pragma omp critical
            worst = rc;
        }
    }
    return worst;
}

int wro_causal_prefill_rows(const void *q, int q_dtype, const uint16_t *k,
                            const uint16_t *v, float *out, uint32_t n,
                            uint32_t p0, const uint32_t *rows, uint32_t n_rows,
                            uint32_t n_q, uint32_t n_kv, uint32_t hd,
                            float scale_override, uint32_t window,
                            uint32_t max_seq, int threads)
{
    int worst = WRO_OK;
    if (threads < 1) threads = 1;
    size_t qsz = (q_dtype == WRO_F32) ? 4 : 2;
    #pragma omp parallel for schedule(dynamic, 1) num_threads(threads)
    for (uint32_t r = 0; r < n_rows; r++) {
        uint32_t i = rows[r];
        int rc = (i < n) ? WRO_OK : WRO_ERR_INVAL;
        if (rc == WRO_OK) {
            const char *qrow = (const char *)q + (uint64_t)i * n_q * hd * qsz;
            rc = wro_gqa_attention(qrow, q_dtype, k, v, WRO_F16,
                                   out + (uint64_t)r * n_q * hd, 1, n_q, n_kv,
                                   hd, p0 + i + 1, scale_override, window, max_seq);
        }
        if (rc != WRO_OK) {
            #pragma omp critical
            worst = rc;
        }
    }
    return worst;
}

int wro_gqa_partial(const float *q, const uint16_t *k, const uint16_t *v,
                    float *m_out, float *l_out, float *o_out, uint32_t n_q,
                    uint32_t n_kv, uint32_t hd, uint32_t key_lo, uint32_t key_hi,
                    float scale_override)
{
    if (!q || !k || !v || n_q == 0 || n_kv == 0 || n_q % n_kv) return WRO_ERR_INVAL;
    uint32_t group = n_q / n_kv;
    float scale = pick_scale(scale_override, hd);
    for (uint32_t qh = 0; qh < n_q; qh++)
        attend_head(q, WRO_F32, (uint64_t)qh * hd, k, v, WRO_F16, n_kv,
                    qh / group, hd, key_lo, key_hi, 0, scale,
                    o_out + (uint64_t)qh * hd, &m_out[qh], &l_out[qh]);
    return WRO_OK;
}
