/*
 * ref_shim.c — plain-pointer entry points onto the UNMODIFIED reference.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is compiled together with the
 * reference's own sources, taken from where they lie in the reference
 * checkout, into oracle/_ref/ (see oracle/Makefile).  It adds no arithmetic:
 * each function fills the reference's tensor descriptors and calls the
 * reference op, so ctypes callers need not know the descriptor layout.
 * Built twice: with the reference's default WR_ATTN_MAX_SEQ and with
 * -DWR_ATTN_MAX_SEQ=32768 (the cap is compile-time, src/core/internal.h:186).
 */
#include <stdint.h>
#include <string.h>

#include "core/internal.h"
#include "core/mathx.h"
#include "core/quant.h"

static void describe(wr_tensor *t, int dtype, const void *data, uint32_t d0,
                     uint32_t d1, uint32_t d2, uint32_t valid_rows)
{
    memset(t, 0, sizeof(*t));
    t->data = (void *)data;
    t->dtype = (uint8_t)dtype;
    t->ndim = 3;
    t->shape[0] = d0; t->shape[1] = d1; t->shape[2] = d2;
    t->size_bytes = (uint64_t)d0 * d1 * d2 * (dtype == WR_DTYPE_F32 ? 4u : 2u);
    if (valid_rows) {
        t->flags |= WR_TENSOR_GROWABLE;
        t->valid_rows = valid_rows;
    }
}

uint32_t refshim_attn_max_seq(void) { return WR_ATTN_MAX_SEQ; }

float    refshim_exp(float x)  { return wri_exp(x); }
float    refshim_log(float x)  { return wri_log(x); }
float    refshim_sqrt(float x) { return wri_sqrt(x); }
float    refshim_sin(float x)  { return wri_sin(x); }
float    refshim_cos(float x)  { return wri_cos(x); }
float    refshim_f16_to_f32(uint16_t h) { return wri_f16_to_f32(h); }
uint16_t refshim_f32_to_f16(float f)    { return wri_f32_to_f16(f); }

void refshim_f32_to_f16_n(const float *src, uint16_t *dst, uint64_t n)
{
    for (uint64_t i = 0; i < n; i++) dst[i] = wri_f32_to_f16(src[i]);
}

void refshim_f16_to_f32_n(const uint16_t *src, float *dst, uint64_t n)
{
    for (uint64_t i = 0; i < n; i++) dst[i] = wri_f16_to_f32(src[i]);
}

int refshim_rope(const float *x, float *out, uint32_t seq, uint32_t heads,
                 uint32_t hd, uint32_t pos, float theta, uint32_t n_rot_pairs)
{
    wr_tensor X, C;
    describe(&X, WR_DTYPE_F32, x, seq, heads, hd, 0);
    describe(&C, WR_DTYPE_F32, out, seq, heads, hd, 0);
    return wri_op_rope(&X, &C, pos, theta, n_rot_pairs);
}

/* cap_rows = rows allocated for K/V; seq_k = rows visible.  When growable is
 * non-zero K/V carry WR_TENSOR_GROWABLE with valid_rows = seq_k (the KV-cache
 * read path); otherwise their shape[0] is seq_k. */
int refshim_attention(const void *q, int q_dtype, const void *k, const void *v,
                      int kv_dtype, float *out, uint32_t seq_q, uint32_t n_q,
                      uint32_t n_kv, uint32_t hd, uint32_t cap_rows,
                      uint32_t seq_k, int growable, float scale_override,
                      uint32_t window)
{
    wr_tensor Q, K, V, C;
    describe(&Q, q_dtype, q, seq_q, n_q, hd, 0);
    describe(&C, WR_DTYPE_F32, out, seq_q, n_q, hd, 0);
    if (growable) {
        describe(&K, kv_dtype, k, cap_rows, n_kv, hd, seq_k);
        describe(&V, kv_dtype, v, cap_rows, n_kv, hd, seq_k);
    } else {
        describe(&K, kv_dtype, k, seq_k, n_kv, hd, 0);
        describe(&V, kv_dtype, v, seq_k, n_kv, hd, 0);
    }
    return wri_op_gqa_attention(&Q, &K, &V, &C, scale_override, window);
}

/* n_sess independent decode calls, one session per OpenMP thread: distinct
 * sessions on distinct threads is the most the reference's thread contract
 * allows for this op (include/wayruntime/wayruntime.h:29-40). */
int refshim_decode_batch(const float *q, const uint16_t *const *k,
                         const uint16_t *const *v, const uint32_t *seq_k,
                         float *out, uint32_t n_sess, uint32_t n_q,
                         uint32_t n_kv, uint32_t hd, float scale_override,
                         uint32_t window, int threads)
{
    int worst = 0;
    if (threads < 1) threads = 1;
    #pragma omp parallel for schedule(dynamic, 1) num_threads(threads)
    for (uint32_t s = 0; s < n_sess; s++) {
        uint64_t off = (uint64_t)s * n_q * hd;
        int rc = refshim_attention(q + off, WR_DTYPE_F32, k[s], v[s],
                                   WR_DTYPE_F16, out + off, 1, n_q, n_kv, hd,
                                   seq_k[s], seq_k[s], 1, scale_override, window);
        if (rc != 0) {
            #pragma omp critical
            worst = rc;
        }
    }
    return worst;
}

/* Causal prefill the way the reference runs it (src/core/session.c:599-630):
 * one single-token attention per listed row i over keys [0, p0+i]. */
int refshim_causal_prefill_rows(const void *q, int q_dtype, const uint16_t *k,
                                const uint16_t *v, float *out, uint32_t n,
                                uint32_t p0, const uint32_t *rows,
                                uint32_t n_rows, uint32_t n_q, uint32_t n_kv,
                                uint32_t hd, float scale_override,
                                uint32_t window, int threads)
{
    int worst = 0;
    if (threads < 1) threads = 1;
    uint64_t qsz = (q_dtype == WR_DTYPE_F32) ? 4u : 2u;
    #pragma omp parallel for schedule(dynamic, 1) num_threads(threads)
    for (uint32_t r = 0; r < n_rows; r++) {
        uint32_t i = rows[r];
        int rc = (i < n) ? 0 : WR_ERR_INVAL;
        if (rc == 0) {
            const char *qrow = (const char *)q + (uint64_t)i * n_q * hd * qsz;
            rc = refshim_attention(qrow, q_dtype, k, v, WR_DTYPE_F16,
                                   out + (uint64_t)r * n_q * hd, 1, n_q, n_kv,
                                   hd, p0 + n, p0 + i + 1, 1, scale_override,
                                   window);
        }
        if (rc != 0) {
            #pragma omp critical
            worst = rc;
        }
    }
    return worst;
}

#ifdef REFSHIM_TAP
/* Whole-model capture (the `libwayruntime_ref_tap.so` variant only, linked
 * with -Wl,--wrap=wri_op_gqa_attention): every attention call the reference's
 * session code makes goes through here, runs the unmodified op, and hands the
 * result to a test callback.  Calls arrive token-major, layer-minor
 * (src/core/session.c:441-496), so the n-th call of a token is layer n. */
typedef void (*refshim_tap_fn)(void *user, uint32_t seq_k, const float *out, uint32_t n_floats);
static refshim_tap_fn g_tap;
static void          *g_tap_user;

void refshim_set_attn_tap(refshim_tap_fn fn, void *user) { g_tap = fn; g_tap_user = user; }

int __real_wri_op_gqa_attention(const wr_tensor *Q, const wr_tensor *K, const wr_tensor *V,
                                wr_tensor *C, float scale_override, uint32_t window);

int __wrap_wri_op_gqa_attention(const wr_tensor *Q, const wr_tensor *K, const wr_tensor *V,
                                wr_tensor *C, float scale_override, uint32_t window)
{
    int rc = __real_wri_op_gqa_attention(Q, K, V, C, scale_override, window);
    if (rc == 0 && g_tap && C->dtype == WR_DTYPE_F32) {
        uint32_t seq_k = (K->flags & WR_TENSOR_GROWABLE) ? K->valid_rows : K->shape[0];
        g_tap(g_tap_user, seq_k, (const float *)C->data,
              C->shape[0] * C->shape[1] * C->shape[2]);
    }
    return rc;
}
#endif
