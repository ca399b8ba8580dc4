/*
 * wr_oracle.h — CPU restatement of the wayruntime GQA-attention hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing shipped links this: it exists so the
 * CUDA kernels can be checked against the reference's arithmetic on a box
 * where the reference sources are not present.  Every function cites the
 * reference function it restates (paths are relative to the reference
 * project root).  Parity of this file with the real reference is pinned by
 * tests that compare it against the reference compiled from its own sources
 * and against committed fixtures generated from that build.
 */
#ifndef WR_ORACLE_H
#define WR_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes: same values as wr_status in include/wayruntime/wayruntime.h:82-107. */
#define WRO_OK             0
#define WRO_ERR_INVAL     (-4)
#define WRO_ERR_NOMEM     (-5)
#define WRO_ERR_CTX_FULL  (-6)
#define WRO_ERR_LIMIT     (-8)
#define WRO_ERR_INTERNAL  (-10)

/* Element types of Q/K/V buffers (values match wr_dtype, src/core/internal.h:53-55). */
#define WRO_F32 0
#define WRO_F16 1

/* Limits (src/core/internal.h:186-197). */
#define WRO_ATTN_MAX_SEQ_DEFAULT 4096
#define WRO_FLASH_BLOCK          64
#define WRO_FLASH_D_MAX          1024

/* src/core/mathx.c:37-147 (WR_MATH_APPROX=1 bodies). */
float wro_exp(float x);
float wro_log(float x);
float wro_sqrt(float x);
float wro_sin(float x);
float wro_cos(float x);

/* src/core/quant.c:86-136. */
float    wro_f16_to_f32(uint16_t h);
uint16_t wro_f32_to_f16(float f);          /* truncating */
void     wro_f32_to_f16_n(const float *src, uint16_t *dst, uint64_t n);
void     wro_f16_to_f32_n(const uint16_t *src, float *dst, uint64_t n);

/* cos/sin of the RoPE angle for every pair j < hd/2 at absolute position
 * pos: src/core/kernels.c:1374-1405.  Pairs j >= n_rot get cs=1, sn=0 and
 * rot[j]=0 (they are passed through, not multiplied). */
void wro_rope_table(uint32_t pos, uint32_t hd, float theta_base,
                    uint32_t n_rot_pairs, float *cs, float *sn, uint8_t *rot);

/* src/core/kernels.c:1356-1412 on an F32 [seq, heads, hd] buffer. */
int wro_rope(const float *x, float *out, uint32_t seq, uint32_t heads,
             uint32_t hd, uint32_t pos, float theta_base, uint32_t n_rot_pairs);

/* src/core/session.c:139-154: append one F32 row of row_elems values as
 * truncated F16 at row *valid_rows of a [cap_rows, row_elems] cache. */
int wro_kv_append_row(uint16_t *cache, uint32_t cap_rows, uint32_t *valid_rows,
                      const float *row, uint32_t row_elems);

/* src/core/kernels.c:1414-1527.  q: [seq_q, n_q, hd] of q_dtype; k, v:
 * [seq_k, n_kv, hd] of kv_dtype; out: F32 [seq_q, n_q, hd].  max_seq is the
 * compiled cap the reference was built with (WR_ATTN_MAX_SEQ). */
int wro_gqa_attention(const void *q, int q_dtype, const void *k, const void *v,
                      int kv_dtype, float *out, uint32_t seq_q, uint32_t n_q,
                      uint32_t n_kv, uint32_t hd, uint32_t seq_k,
                      float scale_override, uint32_t window, uint32_t max_seq);

/* n_sess independent decode calls (src/core/batch.c:152-164 runs them one
 * after another; they share nothing), spread over `threads` host threads.
 * q: F32 [n_sess, n_q, hd]; k[i], v[i]: F16 [seq_k[i], n_kv, hd]. */
int wro_decode_batch(const float *q, const uint16_t *const *k,
                     const uint16_t *const *v, const uint32_t *seq_k,
                     float *out, uint32_t n_sess, uint32_t n_q, uint32_t n_kv,
                     uint32_t hd, float scale_override, uint32_t window,
                     uint32_t max_seq, int threads);

/* The reference's prefill is a loop of single-token bodies
 * (src/core/session.c:599-630): row i attends keys [0, p0+i].  Rows listed in
 * rows[] (n_rows of them, each < n) are computed; out is F32 [n_rows, n_q, hd].
 * q: [n, n_q, hd] of q_dtype; k, v: F16 [p0+n, n_kv, hd]. */
int wro_causal_prefill_rows(const void *q, int q_dtype, const uint16_t *k,
                            const uint16_t *v, float *out, uint32_t n,
                            uint32_t p0, const uint32_t *rows, uint32_t n_rows,
                            uint32_t n_q, uint32_t n_kv, uint32_t hd,
                            float scale_override, uint32_t window,
                            uint32_t max_seq, int threads);

/* Split-KV algebra (same online-softmax merge as src/core/kernels.c:1503-1506
 * applied across shards): one (m, l, o[hd]) triple per (row, head) from keys
 * [key_lo, key_hi).  o is unnormalised. */
int wro_gqa_partial(const float *q, const uint16_t *k, const uint16_t *v,
                    float *m_out, float *l_out, float *o_out, uint32_t n_q,
                    uint32_t n_kv, uint32_t hd, uint32_t key_lo, uint32_t key_hi,
                    float scale_override);

#ifdef __cplusplus
}
#endif
#endif
