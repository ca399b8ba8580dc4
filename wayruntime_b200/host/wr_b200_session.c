/*
 * wr_b200_session.c — the session / batch objects of wayruntime with the
 * attention hot path on a B200.
 *
 * Drop-in for the reference's src/core/session.c and src/core/batch.c: it
 * defines the same 15 external symbols (wr_session_create, wr_session_destroy,
 * wr_session_pos, wr_session_max_context, wr_session_status, wr_prefill,
 * wr_step, wr_batch_step, wri_session_decode_body, wri_session_kv_rollback,
 * wri_session_prefill, wri_session_step, wri_batch_decode_step,
 * wri_self_test_llm_step, wri_self_test_batch_step), so that linking these
 * objects before the reference archive leaves session.o and batch.o unused.
 * It is compiled against the reference's own headers (include/, src/) at
 * integration time.  The public entry points restate the reference's argument
 * checks, locking order and cursor rules (they are the contract a drop-in has
 * to reproduce); everything behind them is new.
 *
 * Two ways to run the layers around attention, chosen per model at session
 * create:
 *   device glue (default when every weight the stack needs is F32 in GGML
 *     layout, which is what the reference's loader produces from F32 / F16 /
 *     BF16 files): the weights are mirrored on the device once per model
 *     (wr_cuda_model) and the whole stack — embedding, RMSNorm, projections,
 *     QK-norm, RoPE + KV append + attention, FFN, final norm, LM head — runs
 *     there; a step moves token ids in and logits out.  F32 arithmetic in a
 *     different summation order than the host's: agrees with the reference to
 *     F32 rounding, not bit for bit.
 *   host glue (WR_B200_GLUE=host, quantised weights, or any model the device
 *     stack does not cover): embedding, RMSNorm, matmuls, QK-norm, residual
 *     adds and the LM head run through the reference's own ops, with the
 *     reference's own numerics; only RoPE on Q and K, the F16 KV append and
 *     the attention itself (src/core/session.c:471-496) go to the GPU.
 * Both go through libwr_cuda.so; neither has a CPU attention path.
 *
 * Execution order is layer-lockstep over a set of rows: the n sessions of a
 * batched step, or the n tokens of a prefill.  Rows interact only through
 * attention, and every host op runs per row with M = 1 exactly as the
 * reference's decode body does, so per-row host arithmetic is unchanged.
 *
 * Gemma-class models (src/core/session.c:251-437: sandwich norms, per-layer
 * head_dim, sliding-window layers with their own RoPE base, shared-KV layers,
 * per-layer-input embeddings, GeGLU, embedding scale, logit soft-cap) run
 * with host glue: every layer that owns a cache has its own device cache of
 * that layer's head_dim, a shared layer attends over its source layer's, and
 * the prompt is taken token by token through the decode kernels (the
 * tensor-core prefill kernel is head_dim 128, no window).
 *
 * All row scratch (Q / K / V / attention / residual rows for a whole batch or
 * a prefill chunk) is page-locked host memory taken once at wr_session_create
 * and freed at destroy — "no reallocation during decode"
 * (include/wayruntime/wayruntime.h:388-392) holds for it as for the KV pages —
 * so the device calls read and write the rows in place instead of staging
 * them.  A prompt longer than WR_B200_ROWS_MAX tokens is prefilled in chunks of
 * that many rows; rows are independent and key tiles sit at absolute
 * positions, so chunking does not change any row's result.
 *
 * Environment: WR_CUDA_DEVICE selects the device (default 0);
 * WR_B200_GLUE=host keeps the layer glue on the host; WR_B200_PREFILL=decode makes wr_prefill run token by token through the
 * decode kernel (F32-exact queries) instead of the tensor-core prefill kernel
 * (F16 queries and probabilities).
 */
#include <inttypes.h>
#include <stdlib.h>
#include <string.h>

#include "core/internal.h"
#include "core/quant.h"
#include "core/tensor.h"
#include "wr_cuda.h"

/* ------------------------------------------------------------- device side */

#include "wr_b200_host.h"

static wr_cuda_ctx *cuda_ctx(int *rc_out)
{
    int rc = 0;
    wr_cuda_ctx *c = wr_b200_cuda_ctx(&rc);
    if (!c)
        wri_log_msg(0, "b200 session: no usable sm_100 device (rc=%d); there is no CPU "
                       "fallback for attention", rc);
    if (rc_out) *rc_out = rc;
    return c;
}

/* Optional observer of every attention result (tests compare these rows with
 * the reference's per layer): called once per row after the device call. */
typedef void (*wr_b200_attn_tap_fn)(void *user, uint32_t layer, uint32_t pos, const float *attn,
                                    uint32_t n_floats);
static wr_b200_attn_tap_fn g_attn_tap;
static void               *g_attn_tap_user;

void wr_b200_set_attn_tap(wr_b200_attn_tap_fn fn, void *user)
{
    g_attn_tap_user = user;
    g_attn_tap = fn;
}

/* ------------------------------------------------------------------ session */

/* Rows a session's scratch holds: a whole batch (WR_BATCH_MAX) or one prefill chunk. */
#define WR_B200_ROWS_MAX 256u

typedef struct row_buffers {
    uint32_t rows;             /* capacity */
    float *resid;   /* [rows][hidden]  */
    float *q;       /* [rows][n_q*hd]  */
    float *k, *v;   /* [rows][n_kv*hd] */
    float *attn;    /* [rows][n_q*hd]  */
    float *normed, *proj, *gate, *up;   /* one row each */
    float *hid_out, *norm_out;          /* [WR_BATCH_MAX][hidden], dense: results of a device pass */
    void  *block;              /* page-locked (wr_cuda_host_alloc) */
} row_buffers;

typedef struct b200_session {
    struct wr_session pub;     /* first member: generate.c reads s->model through it */
    wr_cuda_kv *kv;            /* all layers (uniform head_dim); NULL for a Gemma-class model */
    wr_cuda_kv *kv_layer[WR_MAX_LAYERS];   /* Gemma: one cache per layer; a shared layer aliases its source's */
    float      *ple;           /* Gemma per-layer-input scratch: proj, table [n_layers*ple]; g, pli [ple]; delta [hidden] */
    wr_cuda_ctx *cuda;
    wr_cuda_model *dm;         /* the model's device mirror (shared by its sessions), or NULL: host glue */
    float      *host;          /* one page-locked block holding the scratch tensors */
    row_buffers rb;            /* taken once at create */
} b200_session;

static b200_session *priv(wr_session *s) { return (b200_session *)s; }

static void f32_tensor(wr_tensor *t, float *data, uint32_t ndim, uint32_t d0, uint32_t d1, uint32_t d2)
{
    memset(t, 0, sizeof(*t));
    uint64_t n = d0;
    if (ndim >= 2) n *= d1;
    if (ndim >= 3) n *= d2;
    t->data = data;
    t->size_bytes = n * 4u;
    t->ndim = (uint8_t)ndim;
    t->dtype = WR_DTYPE_F32;
    t->flags = WR_TENSOR_ARENA;
    t->shape[0] = d0;
    if (ndim >= 2) t->shape[1] = d1;
    if (ndim >= 3) t->shape[2] = d2;
}

static uint32_t max_ffn(const wr_model *m)
{
    uint32_t f = m->ffn_dim;
    for (uint32_t L = 0; L < m->n_layers; L++)
        if (m->ffn_dim_per_layer[L] > f) f = m->ffn_dim_per_layer[L];
    return f;
}

static size_t pad16(size_t n) { return (n + 15u) & ~(size_t)15u; }

/* Per-layer head dim (src/core/session.c:108-113). */
static uint32_t layer_head_dim(const wr_model *m, uint32_t L)
{
    if (m->is_gemma && m->has_swa && m->swa_pattern[L] && m->head_dim_swa) return m->head_dim_swa;
    return m->head_dim;
}

static uint32_t max_head_dim(const wr_model *m)
{
    uint32_t hd = m->head_dim;
    for (uint32_t L = 0; L < m->n_layers; L++)
        if (layer_head_dim(m, L) > hd) hd = layer_head_dim(m, L);
    return hd;
}

/* The layer whose cache layer L reads: itself, or for the trailing shared layers the last
 * non-shared layer of the same kind, sliding-window or global (src/core/session.c:122-134). */
static uint32_t kv_source_layer(const wr_model *m, uint32_t L, int local)
{
    if (!m->is_gemma || m->kv_shared_layers == 0 || m->kv_shared_layers >= m->n_layers) return L;
    const uint32_t first_shared = m->n_layers - m->kv_shared_layers;
    if (L < first_shared) return L;
    for (int cand = (int)first_shared - 1; cand >= 0; cand--) {
        const int cand_local = (m->has_swa && m->swa_pattern[cand]) ? 1 : 0;
        if (cand_local == local) return (uint32_t)cand;
    }
    return L;
}

/* The reference's own square root for the per-layer-input scale (src/core/session.c:98-104):
 * 24 Newton steps, kept as they are so that the arithmetic stays bit-identical. */
static float newton_sqrtf(float x)
{
    if (x <= 0.0f) return 0.0f;
    float g = x > 1.0f ? x : 1.0f;
    for (int i = 0; i < 24; i++) g = 0.5f * (g + x / g);
    return g;
}

static int rows_alloc(row_buffers *rb, wr_cuda_ctx *cuda, const wr_model *m, uint32_t rows)
{
    const size_t hid = m->hidden_dim, nq = (size_t)m->n_q_heads * max_head_dim(m),
                 nkv = (size_t)m->n_kv_heads * max_head_dim(m), ffn = max_ffn(m);
    const size_t total = rows * (pad16(hid) + 2 * pad16(nq) + 2 * pad16(nkv)) + 2 * pad16(hid) +
                         2 * pad16(ffn) + 2 * WR_BATCH_MAX * pad16(hid);
    memset(rb, 0, sizeof(*rb));
    int rc = wr_cuda_host_alloc(cuda, total * sizeof(float), &rb->block);
    if (rc != 0) return rc;
    float *p = rb->block;
    rb->rows = rows;
    rb->resid = p;  p += rows * pad16(hid);
    rb->q = p;      p += rows * pad16(nq);
    rb->attn = p;   p += rows * pad16(nq);
    rb->k = p;      p += rows * pad16(nkv);
    rb->v = p;      p += rows * pad16(nkv);
    rb->normed = p; p += pad16(hid);
    rb->proj = p;   p += pad16(hid);
    rb->gate = p;   p += pad16(ffn);
    rb->up = p;     p += pad16(ffn);
    rb->hid_out = p;  p += WR_BATCH_MAX * pad16(hid);
    rb->norm_out = p;
    return WR_OK;
}

/* ------------------------------------------------------ device model mirrors
 *
 * One wr_cuda_model per wr_model, shared by the model's sessions and dropped
 * with the last of them.  The table is tiny (models per process) and touched
 * only at session create / destroy. */

typedef struct dev_model_slot {
    const wr_model *m;
    wr_cuda_model  *dm;
    uint32_t        refs;
} dev_model_slot;

#define DEV_MODEL_SLOTS 16
static dev_model_slot g_dev_models[DEV_MODEL_SLOTS];
static volatile int   g_dev_guard;

static void dev_lock(void)   { while (__atomic_exchange_n(&g_dev_guard, 1, __ATOMIC_ACQUIRE)) { } }
static void dev_unlock(void) { __atomic_store_n(&g_dev_guard, 0, __ATOMIC_RELEASE); }

static int f32_vec(const wr_tensor *t, uint32_t n)
{
    return t->data && t->dtype == WR_DTYPE_F32 && t->size_bytes >= (uint64_t)n * 4u;
}

/* a [in -> out] projection kept as F32 in GGML layout (out rows of in floats) */
static int f32_ggml(const wr_tensor *t, uint32_t in, uint32_t out)
{
    return t->data && t->dtype == WR_DTYPE_F32 && (t->flags & WR_TENSOR_GGML_WEIGHT) && t->ndim == 2 &&
           t->shape[0] == in && t->shape[1] == out && t->size_bytes >= (uint64_t)in * out * 4u;
}

/* Can the device stack run this model as it sits in memory? */
static int device_glue_covers(const wr_model *m)
{
    const char *mode = getenv("WR_B200_GLUE");
    if (mode && strcmp(mode, "host") == 0) return 0;
    if (m->is_gemma) return 0;                       /* sandwich norms, PLE, per-layer head_dim: host glue */
    const uint32_t hid = m->hidden_dim, hd = m->head_dim, nq = m->n_q_heads * hd, nkv = m->n_kv_heads * hd;
    if ((hid & 3u) || (hd & 3u) || m->n_layers > WR_CUDA_MAX_LAYERS) return 0;
    if (!(m->embed_table.data && m->embed_table.dtype == WR_DTYPE_F32 && m->embed_table.ndim == 2 &&
          m->embed_table.shape[0] == m->vocab_size && m->embed_table.shape[1] == hid))
        return 0;
    if (!(m->lm_head.data && m->lm_head.dtype == WR_DTYPE_F32 && m->lm_head.ndim == 2 &&
          m->lm_head.shape[0] == m->vocab_size && m->lm_head.shape[1] == hid))
        return 0;
    if (!f32_vec(&m->final_norm, hid)) return 0;
    for (uint32_t L = 0; L < m->n_layers; L++) {
        const uint32_t ffn = m->ffn_dim_per_layer[L] ? m->ffn_dim_per_layer[L] : m->ffn_dim;
        if (ffn == 0 || (ffn & 3u)) return 0;
        if (!f32_vec(&m->attn_norm[L], hid) || !f32_vec(&m->ffn_norm[L], hid)) return 0;
        if (!f32_ggml(&m->wq[L], hid, nq) || !f32_ggml(&m->wk[L], hid, nkv) ||
            !f32_ggml(&m->wv[L], hid, nkv) || !f32_ggml(&m->wo[L], nq, hid) ||
            !f32_ggml(&m->w_gate[L], hid, ffn) || !f32_ggml(&m->w_up[L], hid, ffn) ||
            !f32_ggml(&m->w_down[L], ffn, hid))
            return 0;
        const int qk = m->has_qk_norm && m->q_norm[L].data && m->k_norm[L].data;
        if (qk && (!f32_vec(&m->q_norm[L], hd) || !f32_vec(&m->k_norm[L], hd))) return 0;
    }
    return 1;
}

static wr_cuda_model *dev_model_acquire(const wr_model *m, wr_cuda_ctx *cuda)
{
    if (!device_glue_covers(m)) return NULL;
    wr_cuda_model *dm = NULL;
    dev_lock();
    dev_model_slot *free_slot = NULL;
    for (int i = 0; i < DEV_MODEL_SLOTS; i++) {
        if (g_dev_models[i].m == m && g_dev_models[i].dm) {
            g_dev_models[i].refs++;
            dm = g_dev_models[i].dm;
            break;
        }
        if (!g_dev_models[i].dm && !free_slot) free_slot = &g_dev_models[i];
    }
    if (!dm && free_slot) {
        wr_cuda_layer_desc *layers = calloc(m->n_layers, sizeof(*layers));
        if (layers) {
            wr_cuda_model_desc d;
            memset(&d, 0, sizeof(d));
            d.n_layers = m->n_layers; d.hidden = m->hidden_dim; d.n_q_heads = m->n_q_heads;
            d.n_kv_heads = m->n_kv_heads; d.head_dim = m->head_dim; d.vocab = m->vocab_size;
            d.n_rot_pairs = m->n_rot_pairs; d.max_rows = WR_B200_ROWS_MAX;
            d.rms_eps = m->rms_eps;
            d.rope_theta = (m->rope_freq_base > 0.0f) ? m->rope_freq_base : 10000.0f;
            d.attn_scale = (m->attn_scale > 0.0f) ? m->attn_scale : 0.0f;
            d.embed = m->embed_table.data; d.lm_head = m->lm_head.data; d.final_norm = m->final_norm.data;
            d.layers = layers;
            for (uint32_t L = 0; L < m->n_layers; L++) {
                wr_cuda_layer_desc *l = &layers[L];
                const int qk = m->has_qk_norm && m->q_norm[L].data && m->k_norm[L].data;
                l->attn_norm = m->attn_norm[L].data; l->wq = m->wq[L].data; l->wk = m->wk[L].data;
                l->wv = m->wv[L].data; l->wo = m->wo[L].data; l->ffn_norm = m->ffn_norm[L].data;
                l->w_gate = m->w_gate[L].data; l->w_up = m->w_up[L].data; l->w_down = m->w_down[L].data;
                l->q_norm = qk ? m->q_norm[L].data : NULL;
                l->k_norm = qk ? m->k_norm[L].data : NULL;
                l->ffn_dim = m->ffn_dim_per_layer[L] ? m->ffn_dim_per_layer[L] : m->ffn_dim;
            }
            int rc = wr_cuda_model_create(cuda, &d, &dm);
            free(layers);
            if (rc == 0) {
                free_slot->m = m; free_slot->dm = dm; free_slot->refs = 1;
                wri_log_msg(2, "b200 session: layer glue on the device (%" PRIu64 " MiB of weights and scratch)",
                            wr_cuda_model_bytes(dm) >> 20);
            } else {
                dm = NULL;
                wri_log_msg(1, "b200 session: device mirror of the weights failed (rc=%d); the layer glue "
                               "stays on the host, attention on the device", rc);
            }
        }
    }
    dev_unlock();
    return dm;
}

static void dev_model_release(wr_cuda_model *dm)
{
    if (!dm) return;
    wr_cuda_model *drop = NULL;
    dev_lock();
    for (int i = 0; i < DEV_MODEL_SLOTS; i++)
        if (g_dev_models[i].dm == dm) {
            if (--g_dev_models[i].refs == 0) {
                drop = dm;
                memset(&g_dev_models[i], 0, sizeof(g_dev_models[i]));
            }
            break;
        }
    dev_unlock();
    if (drop) wr_cuda_model_destroy(drop);
}

static void session_caches_free(b200_session *bs)
{
    const wr_model *m = bs->pub.model;
    if (bs->kv) wr_cuda_kv_destroy(bs->kv);
    bs->kv = NULL;
    for (uint32_t L = 0; m && L < m->n_layers; L++) {
        if (!bs->kv_layer[L]) continue;
        const int local = (m->has_swa && m->swa_pattern[L]) ? 1 : 0;
        if (kv_source_layer(m, L, local) == L) wr_cuda_kv_destroy(bs->kv_layer[L]);   /* owners only */
        bs->kv_layer[L] = NULL;
    }
    free(bs->ple);
    bs->ple = NULL;
}

wr_status wr_session_create(wr_model *m, const wr_session_params *params, wr_session **out)
{
    if (!out) return WR_ERR_INVAL;
    *out = NULL;
    if (!m) return WR_ERR_INVAL;
    if (!m->weights_committed || !m->lock) return WR_ERR_STATE;
    if (m->n_layers == 0) return WR_ERR_INVAL;
    if (m->n_layers > WR_MAX_LAYERS) return WR_ERR_LIMIT;
    if (m->n_kv_heads == 0 || m->n_q_heads == 0 || m->head_dim == 0 || m->hidden_dim == 0 ||
        m->vocab_size == 0 || m->max_context == 0)
        return WR_ERR_INVAL;
    if (!m->is_gemma && (m->kv_shared_layers || m->has_swa || m->pl_emb_dim)) return WR_ERR_UNSUPPORTED;

    uint32_t max_ctx = m->max_context;
    if (params && params->max_context) {
        if (params->max_context > m->max_context) return WR_ERR_INVAL;
        max_ctx = params->max_context;
    }
    if (max_ctx > WR_ATTN_MAX_SEQ) return WR_ERR_LIMIT;

    int crc = 0;
    wr_cuda_ctx *cuda = cuda_ctx(&crc);
    if (!cuda) return (crc < 0) ? (wr_status)crc : WR_ERR_UNSUPPORTED;

    b200_session *bs = calloc(1, sizeof(*bs));
    if (!bs) return WR_ERR_NOMEM;
    wr_session *s = &bs->pub;
    s->model = m;
    s->max_context = max_ctx;
    s->last_status = WR_OK;
    s->lock = wr_mutex_create();
    if (!s->lock) { free(bs); return WR_ERR_NOMEM; }

    const uint32_t hid = m->hidden_dim, hd = max_head_dim(m), ffn = max_ffn(m);
    const size_t nq = (size_t)m->n_q_heads * hd, nkv = (size_t)m->n_kv_heads * hd;
    const size_t total = pad16(hid) * 3 + pad16(nq) * 2 + pad16(nkv) * 2 + pad16(ffn) * 2 +
                         pad16(m->vocab_size);
    /* page-locked: the device pass writes logits / hidden rows straight into these tensors */
    void *host_block = NULL;
    if (wr_cuda_host_alloc(cuda, total * sizeof(float), &host_block) != 0 || !host_block) {
        wr_mutex_destroy(s->lock); free(bs); return WR_ERR_NOMEM;
    }
    bs->host = host_block;
    memset(bs->host, 0, total * sizeof(float));
    float *p = bs->host;
    f32_tensor(&s->residual, p, 1, hid, 0, 0);                 p += pad16(hid);
    f32_tensor(&s->normed, p, 1, hid, 0, 0);                   p += pad16(hid);
    f32_tensor(&s->ffn_proj, p, 1, hid, 0, 0);                 p += pad16(hid);
    f32_tensor(&s->q, p, 3, 1, m->n_q_heads, hd);              p += pad16(nq);
    f32_tensor(&s->attn, p, 3, 1, m->n_q_heads, hd);           p += pad16(nq);
    f32_tensor(&s->k_row, p, 3, 1, m->n_kv_heads, hd);         p += pad16(nkv);
    f32_tensor(&s->v_row, p, 3, 1, m->n_kv_heads, hd);         p += pad16(nkv);
    f32_tensor(&s->ffn_gate, p, 1, ffn, 0, 0);                 p += pad16(ffn);
    f32_tensor(&s->ffn_up, p, 1, ffn, 0, 0);                   p += pad16(ffn);
    f32_tensor(&s->logits, p, 1, m->vocab_size, 0, 0);

    bs->cuda = cuda;
    int rc = 0;
    if (!m->is_gemma) {
        rc = wr_cuda_kv_create(cuda, m->n_layers, m->n_kv_heads, hd, max_ctx, &bs->kv);
    } else {
        /* one cache per owning layer, of that layer's head_dim (src/core/session.c:647-674) */
        for (uint32_t L = 0; L < m->n_layers && rc == 0; L++) {
            const int local = (m->has_swa && m->swa_pattern[L]) ? 1 : 0;
            const uint32_t src = kv_source_layer(m, L, local);
            if (src != L) bs->kv_layer[L] = bs->kv_layer[src];          /* src < L: already made */
            else rc = wr_cuda_kv_create(cuda, 1, m->n_kv_heads, layer_head_dim(m, L), max_ctx, &bs->kv_layer[L]);
        }
        if (rc == 0 && m->pl_emb_dim) {
            const size_t pl = (size_t)m->n_layers * m->pl_emb_dim;
            bs->ple = calloc(2 * pl + 2 * (size_t)m->pl_emb_dim + hid, sizeof(float));
            if (!bs->ple) rc = WR_ERR_NOMEM;
        }
    }
    if (rc == 0) {
        uint32_t rows = max_ctx < WR_B200_ROWS_MAX ? max_ctx : WR_B200_ROWS_MAX;
        if (rows < WR_BATCH_MAX) rows = WR_BATCH_MAX;
        rc = rows_alloc(&bs->rb, cuda, m, rows);
    }
    if (rc != 0) {
        wri_log_msg(0, "b200 session: device KV / row scratch allocation failed (rc=%d)", rc);
        session_caches_free(bs);
        wr_cuda_host_free(cuda, bs->host);
        wr_mutex_destroy(s->lock);
        free(bs);
        return (wr_status)rc;
    }
    bs->dm = dev_model_acquire(m, cuda);
    wr_mutex_lock(m->lock);
    m->session_refs++;
    wr_mutex_unlock(m->lock);
    *out = s;
    return WR_OK;
}

void wr_session_destroy(wr_session *s)
{
    if (!s) return;
    b200_session *bs = priv(s);
    wr_model *m = s->model;
    if (m && m->lock) {
        wr_mutex_lock(m->lock);
        if (m->session_refs > 0) m->session_refs--;
        wr_mutex_unlock(m->lock);
    }
    dev_model_release(bs->dm);
    session_caches_free(bs);
    if (bs->rb.block) wr_cuda_host_free(bs->cuda, bs->rb.block);
    if (bs->host) wr_cuda_host_free(bs->cuda, bs->host);
    if (s->lock) wr_mutex_destroy(s->lock);
    free(bs);
}

/* The committed KV length is s->pos, passed to every device call; a failed
 * step never advanced it, so there is nothing to undo (the reference resets
 * per-layer cursors here, src/core/session.c:160-168). */
void wri_session_kv_rollback(wr_session *s) { (void)s; }

uint32_t wr_session_pos(const wr_session *s)
{
    return s ? __atomic_load_n(&s->pos, __ATOMIC_ACQUIRE) : 0;
}
uint32_t wr_session_max_context(const wr_session *s) { return s ? s->max_context : 0; }
wr_status wr_session_status(const wr_session *s)
{
    return s ? __atomic_load_n(&s->last_status, __ATOMIC_ACQUIRE) : WR_ERR_INVAL;
}

/* --------------------------------------------------------- forward over rows */

static wr_status fail(const char *what, uint32_t layer, int rc)
{
    wri_log_msg(0, "b200 session: %s failed at layer %u (rc=%d)", what, layer, rc);
    return (rc < 0) ? (wr_status)rc : WR_ERR_INTERNAL;
}

enum { ATTN_DECODE = 0, ATTN_PREFILL = 1 };

/* Layer stack (minus the LM head) for `rows` rows.
 *   ATTN_DECODE : row r is the new token of session kvs[r] at position pos[r];
 *   ATTN_PREFILL: rows are consecutive tokens of session kvs[0] from pos[0].
 * On success rb->resid holds the pre-final-norm hidden rows. */
static wr_status forward_rows(const wr_model *m, row_buffers *rb, uint32_t R, const uint32_t *tokens,
                              wr_cuda_kv *const *kvs, const uint32_t *pos, int mode)
{
    if (R == 0 || R > rb->rows) return WR_ERR_INTERNAL;
    const uint32_t hid = m->hidden_dim, hd = m->head_dim;
    const uint32_t nq = m->n_q_heads * hd, nkv = m->n_kv_heads * hd;
    const size_t s_hid = pad16(hid), s_q = pad16(nq), s_kv = pad16(nkv);
    const float eps = m->rms_eps;
    const float theta = (m->rope_freq_base > 0.0f) ? m->rope_freq_base : 10000.0f;
    int crc = 0;
    wr_cuda_ctx *cuda = cuda_ctx(&crc);
    if (!cuda) return (crc < 0) ? (wr_status)crc : WR_ERR_UNSUPPORTED;
    /* the device calls want dense [rows, heads, hd] blocks */
    if (s_q != nq || s_kv != nkv) return WR_ERR_UNSUPPORTED;
    wr_tensor t_res, t_norm, t_q, t_k, t_v, t_a, t_proj, t_gate, t_up;
    int rc;

    for (uint32_t r = 0; r < R; r++) {
        f32_tensor(&t_res, rb->resid + r * s_hid, 1, hid, 0, 0);
        rc = wri_op_embed(&m->embed_table, tokens[r], &t_res);
        if (rc != WR_OK) return fail("embed", 0, rc);
    }
    for (uint32_t L = 0; L < m->n_layers; L++) {
        const uint32_t ffn = m->ffn_dim_per_layer[L] ? m->ffn_dim_per_layer[L] : m->ffn_dim;
        for (uint32_t r = 0; r < R; r++) {           /* norm, projections, QK-norm: per row, M = 1 */
            f32_tensor(&t_res, rb->resid + r * s_hid, 1, hid, 0, 0);
            f32_tensor(&t_norm, rb->normed, 1, hid, 0, 0);
            rc = wri_op_rmsnorm(&t_res, &m->attn_norm[L], &t_norm, eps);
            if (rc != WR_OK) return fail("attn norm", L, rc);
            f32_tensor(&t_norm, rb->normed, 2, 1, hid, 0);
            f32_tensor(&t_q, rb->q + r * s_q, 2, 1, nq, 0);
            f32_tensor(&t_k, rb->k + r * s_kv, 2, 1, nkv, 0);
            f32_tensor(&t_v, rb->v + r * s_kv, 2, 1, nkv, 0);
            rc = wri_op_matmul(&t_norm, &m->wq[L], &t_q);
            if (rc != WR_OK) return fail("wq matmul", L, rc);
            rc = wri_op_matmul(&t_norm, &m->wk[L], &t_k);
            if (rc != WR_OK) return fail("wk matmul", L, rc);
            rc = wri_op_matmul(&t_norm, &m->wv[L], &t_v);
            if (rc != WR_OK) return fail("wv matmul", L, rc);
            if (m->has_qk_norm && m->q_norm[L].data && m->k_norm[L].data) {
                f32_tensor(&t_q, rb->q + r * s_q, 2, m->n_q_heads, hd, 0);
                rc = wri_op_rmsnorm(&t_q, &m->q_norm[L], &t_q, eps);
                if (rc != WR_OK) return fail("q norm", L, rc);
                f32_tensor(&t_k, rb->k + r * s_kv, 2, m->n_kv_heads, hd, 0);
                rc = wri_op_rmsnorm(&t_k, &m->k_norm[L], &t_k, eps);
                if (rc != WR_OK) return fail("k norm", L, rc);
            }
        }
        /* RoPE(Q, K) + KV append + attention: one device call for all rows */
        const float scale = (m->attn_scale > 0.0f) ? m->attn_scale : 0.0f;
        if (mode == ATTN_DECODE) {
            rc = wr_cuda_decode_step(cuda, R, kvs, L, pos, rb->q, rb->k, rb->v, rb->attn, m->n_q_heads,
                                     theta, m->n_rot_pairs, WR_CUDA_APPEND_ROPE, scale, 0,
                                     WR_CUDA_MEM_HOST);
            if (rc != 0) return fail("cuda decode step", L, rc);
        } else {
            rc = wr_cuda_kv_append(cuda, 1, kvs, L, pos, R, rb->k, rb->v, rb->q, m->n_q_heads, theta,
                                   m->n_rot_pairs, WR_CUDA_APPEND_ROPE, WR_CUDA_MEM_HOST);
            if (rc != 0) return fail("cuda kv append", L, rc);
            rc = wr_cuda_attn_prefill(cuda, kvs[0], L, pos[0], R, rb->q, WR_CUDA_F32, rb->attn,
                                      m->n_q_heads, scale, 0, WR_CUDA_MEM_HOST);
            if (rc != 0) return fail("cuda prefill attention", L, rc);
        }
        WRI_CTR_ADD(WR_CTR_ATTENTION_CALLS, R);   /* one launch, R attention calls (kernels.c:1423) */
        if (g_attn_tap)
            for (uint32_t r = 0; r < R; r++)
                g_attn_tap(g_attn_tap_user, L, mode == ATTN_DECODE ? pos[r] : pos[0] + r,
                           rb->attn + r * s_q, nq);

        for (uint32_t r = 0; r < R; r++) {           /* output projection, FFN: per row */
            f32_tensor(&t_res, rb->resid + r * s_hid, 1, hid, 0, 0);
            f32_tensor(&t_a, rb->attn + r * s_q, 2, 1, nq, 0);
            f32_tensor(&t_proj, rb->proj, 2, 1, hid, 0);
            rc = wri_op_matmul(&t_a, &m->wo[L], &t_proj);
            if (rc != WR_OK) return fail("wo matmul", L, rc);
            f32_tensor(&t_proj, rb->proj, 1, hid, 0, 0);
            rc = wri_op_add(&t_res, &t_proj, &t_res);
            if (rc != WR_OK) return fail("attn residual", L, rc);

            f32_tensor(&t_norm, rb->normed, 1, hid, 0, 0);
            rc = wri_op_rmsnorm(&t_res, &m->ffn_norm[L], &t_norm, eps);
            if (rc != WR_OK) return fail("ffn norm", L, rc);
            f32_tensor(&t_norm, rb->normed, 2, 1, hid, 0);
            f32_tensor(&t_gate, rb->gate, 2, 1, ffn, 0);
            f32_tensor(&t_up, rb->up, 2, 1, ffn, 0);
            rc = wri_op_matmul(&t_norm, &m->w_gate[L], &t_gate);
            if (rc != WR_OK) return fail("gate matmul", L, rc);
            rc = wri_op_matmul(&t_norm, &m->w_up[L], &t_up);
            if (rc != WR_OK) return fail("up matmul", L, rc);
            f32_tensor(&t_gate, rb->gate, 1, ffn, 0, 0);
            f32_tensor(&t_up, rb->up, 1, ffn, 0, 0);
            rc = wri_op_fused_silu_mul(&t_gate, &t_up, &t_gate);
            if (rc != WR_OK) return fail("swiglu", L, rc);
            f32_tensor(&t_gate, rb->gate, 2, 1, ffn, 0);
            f32_tensor(&t_proj, rb->proj, 2, 1, hid, 0);
            rc = wri_op_matmul(&t_gate, &m->w_down[L], &t_proj);
            if (rc != WR_OK) return fail("down matmul", L, rc);
            f32_tensor(&t_proj, rb->proj, 1, hid, 0, 0);
            rc = wri_op_add(&t_res, &t_proj, &t_res);
            if (rc != WR_OK) return fail("ffn residual", L, rc);
        }
    }
    return WR_OK;
}

/* Gemma-class layer stack (src/core/session.c:202-437) for R rows, row r = the new token of session
 * sess[r] at position pos[r].  Host ops exactly as the reference runs them, per row with M = 1; per
 * layer one device call for all rows: wr_cuda_decode_step on the layer's own cache (RoPE with the
 * layer's base and rotary share, append, attention with the model's explicit scale and the layer's
 * window), or — a shared layer — RoPE of Q on the host and wr_cuda_attn_decode over the source
 * layer's cache.  Rows of a layer are dense [R][heads][hd_L].  Scratch for the per-layer-input
 * arithmetic is one row's; those steps run row by row.  On success rb->resid holds the hidden rows. */
static wr_status forward_rows_gemma(const wr_model *m, b200_session *const *sess, row_buffers *rb, uint32_t R,
                                    const uint32_t *tokens, const uint32_t *pos)
{
    if (R == 0 || R > rb->rows || R > WR_BATCH_MAX) return WR_ERR_INTERNAL;
    const uint32_t hid = m->hidden_dim, qheads = m->n_q_heads, kheads = m->n_kv_heads;
    const size_t s_hid = pad16(hid);
    const float eps = m->rms_eps;
    const float theta_default = (m->rope_freq_base > 0.0f) ? m->rope_freq_base : 10000.0f;
    const uint32_t ple = m->pl_emb_dim, pl = m->n_layers * ple;
    const int want_ple = m->per_layer_token_embd.data && m->per_layer_model_proj.data &&
                         m->per_layer_proj_norm.data && ple;
    int crc = 0;
    wr_cuda_ctx *cuda = cuda_ctx(&crc);
    if (!cuda) return (crc < 0) ? (wr_status)crc : WR_ERR_UNSUPPORTED;
    wr_tensor t_res, t_norm, t_q, t_k, t_v, t_a, t_proj, t_gate, t_up, t_x, t_y;
    int rc;

    for (uint32_t r = 0; r < R; r++) {
        float *res = rb->resid + r * s_hid;
        f32_tensor(&t_res, res, 1, hid, 0, 0);
        rc = wri_op_embed(&m->embed_table, tokens[r], &t_res);
        if (rc != WR_OK) return fail("embed", 0, rc);
        if (m->embed_scale != 0.0f)
            for (uint32_t j = 0; j < hid; j++) res[j] *= m->embed_scale;
        if (want_ple) {                              /* per-layer-input table of this token (session.c:221-245) */
            float *proj = sess[r]->ple, *table = proj + pl;
            if (!proj) return WR_ERR_INTERNAL;
            f32_tensor(&t_x, res, 2, 1, hid, 0);
            f32_tensor(&t_y, proj, 2, 1, pl, 0);
            rc = wri_op_matmul(&t_x, &m->per_layer_model_proj, &t_y);
            if (rc != WR_OK) return fail("ple proj matmul", 0, rc);
            f32_tensor(&t_y, proj, 2, m->n_layers, ple, 0);
            rc = wri_op_rmsnorm(&t_y, &m->per_layer_proj_norm, &t_y, eps);
            if (rc != WR_OK) return fail("ple proj norm", 0, rc);
            f32_tensor(&t_y, table, 1, pl, 0, 0);
            rc = wri_op_embed(&m->per_layer_token_embd, tokens[r], &t_y);
            if (rc != WR_OK) return fail("ple table embed", 0, rc);
            const float tscale = newton_sqrtf((float)ple), comb = 0.70710678f;
            for (uint32_t j = 0; j < pl; j++) table[j] = (proj[j] + table[j] * tscale) * comb;
        }
    }

    for (uint32_t L = 0; L < m->n_layers; L++) {
        const uint32_t ffn = m->ffn_dim_per_layer[L] ? m->ffn_dim_per_layer[L] : m->ffn_dim;
        const int local = (m->has_swa && m->swa_pattern[L]) ? 1 : 0;
        const uint32_t hd = layer_head_dim(m, L), nq = qheads * hd, nkv = kheads * hd;
        const float theta = (local && m->rope_freq_base_swa > 0.0f) ? m->rope_freq_base_swa : theta_default;
        const uint32_t n_rot = local ? 0u : m->n_rot_pairs;       /* partial rotary on global layers only */
        const uint32_t ksrc = kv_source_layer(m, L, local);
        const int shared = (ksrc != L);
        const uint32_t window = (local && m->swa_mode != WR_SWA_DISABLED) ? m->sliding_window : 0u;
        const int qk_norm = m->has_qk_norm && m->q_norm[L].data && m->k_norm[L].data;
        if ((nq & 3u) || (nkv & 3u)) return WR_ERR_UNSUPPORTED;    /* rows move as 16-byte vectors */

        for (uint32_t r = 0; r < R; r++) {           /* A1-A4: norm, projections, head norms (V: weightless) */
            f32_tensor(&t_res, rb->resid + r * s_hid, 1, hid, 0, 0);
            f32_tensor(&t_norm, rb->normed, 1, hid, 0, 0);
            rc = wri_op_rmsnorm(&t_res, &m->attn_norm[L], &t_norm, eps);
            if (rc != WR_OK) return fail("attn norm", L, rc);
            f32_tensor(&t_norm, rb->normed, 2, 1, hid, 0);
            f32_tensor(&t_q, rb->q + (size_t)r * nq, 2, 1, nq, 0);
            rc = wri_op_matmul(&t_norm, &m->wq[L], &t_q);
            if (rc != WR_OK) return fail("wq matmul", L, rc);
            if (!shared) {
                f32_tensor(&t_k, rb->k + (size_t)r * nkv, 2, 1, nkv, 0);
                f32_tensor(&t_v, rb->v + (size_t)r * nkv, 2, 1, nkv, 0);
                rc = wri_op_matmul(&t_norm, &m->wk[L], &t_k);
                if (rc != WR_OK) return fail("wk matmul", L, rc);
                rc = wri_op_matmul(&t_norm, &m->wv[L], &t_v);
                if (rc != WR_OK) return fail("wv matmul", L, rc);
            }
            if (qk_norm) {
                f32_tensor(&t_q, rb->q + (size_t)r * nq, 2, qheads, hd, 0);
                rc = wri_op_rmsnorm(&t_q, &m->q_norm[L], &t_q, eps);
                if (rc != WR_OK) return fail("q norm", L, rc);
                if (!shared) {
                    f32_tensor(&t_k, rb->k + (size_t)r * nkv, 2, kheads, hd, 0);
                    rc = wri_op_rmsnorm(&t_k, &m->k_norm[L], &t_k, eps);
                    if (rc != WR_OK) return fail("k norm", L, rc);
                }
            }
            if (!shared) {                           /* weightless RMS of V before the append (session.c:331-336) */
                f32_tensor(&t_v, rb->v + (size_t)r * nkv, 2, kheads, hd, 0);
                rc = wri_op_rmsnorm(&t_v, NULL, &t_v, eps);
                if (rc != WR_OK) return fail("v norm", L, rc);
            } else {                                 /* shared layer: only Q is rotated; its K is already in the cache */
                f32_tensor(&t_q, rb->q + (size_t)r * nq, 3, 1, qheads, hd);
                rc = wri_op_rope(&t_q, &t_q, pos[r], theta, n_rot);
                if (rc != WR_OK) return fail("q rope", L, rc);
            }
        }
        /* A5-A6: one device call for all rows */
        wr_cuda_kv *kvs[WR_BATCH_MAX];
        uint32_t lens[WR_BATCH_MAX];
        for (uint32_t r = 0; r < R; r++) {
            kvs[r] = sess[r]->kv_layer[ksrc];
            lens[r] = pos[r] + 1;
            if (!kvs[r]) return WR_ERR_INTERNAL;
        }
        if (!shared)
            rc = wr_cuda_decode_step(cuda, R, kvs, 0, pos, rb->q, rb->k, rb->v, rb->attn, qheads, theta, n_rot,
                                     WR_CUDA_APPEND_ROPE, m->attn_scale, window, WR_CUDA_MEM_HOST);
        else
            rc = wr_cuda_attn_decode(cuda, R, kvs, 0, lens, rb->q, rb->attn, qheads, m->attn_scale, window,
                                     WR_CUDA_MEM_HOST);
        if (rc != 0) return fail("cuda attention", L, rc);
        WRI_CTR_ADD(WR_CTR_ATTENTION_CALLS, R);
        if (g_attn_tap)
            for (uint32_t r = 0; r < R; r++) g_attn_tap(g_attn_tap_user, L, pos[r], rb->attn + (size_t)r * nq, nq);

        for (uint32_t r = 0; r < R; r++) {           /* A7-A9, F1-F6, per-layer input, output scale */
            float *res = rb->resid + r * s_hid;
            f32_tensor(&t_res, res, 1, hid, 0, 0);
            f32_tensor(&t_a, rb->attn + (size_t)r * nq, 2, 1, nq, 0);
            f32_tensor(&t_proj, rb->proj, 2, 1, hid, 0);
            rc = wri_op_matmul(&t_a, &m->wo[L], &t_proj);
            if (rc != WR_OK) return fail("wo matmul", L, rc);
            f32_tensor(&t_proj, rb->proj, 1, hid, 0, 0);
            rc = wri_op_rmsnorm(&t_proj, &m->post_attn_norm[L], &t_proj, eps);
            if (rc != WR_OK) return fail("post-attn norm", L, rc);
            rc = wri_op_add(&t_res, &t_proj, &t_res);
            if (rc != WR_OK) return fail("attn residual", L, rc);

            f32_tensor(&t_norm, rb->normed, 1, hid, 0, 0);
            rc = wri_op_rmsnorm(&t_res, &m->ffn_norm[L], &t_norm, eps);
            if (rc != WR_OK) return fail("ffn norm", L, rc);
            f32_tensor(&t_norm, rb->normed, 2, 1, hid, 0);
            f32_tensor(&t_gate, rb->gate, 2, 1, ffn, 0);
            f32_tensor(&t_up, rb->up, 2, 1, ffn, 0);
            rc = wri_op_matmul(&t_norm, &m->w_gate[L], &t_gate);
            if (rc != WR_OK) return fail("gate matmul", L, rc);
            rc = wri_op_matmul(&t_norm, &m->w_up[L], &t_up);
            if (rc != WR_OK) return fail("up matmul", L, rc);
            f32_tensor(&t_gate, rb->gate, 1, ffn, 0, 0);
            f32_tensor(&t_up, rb->up, 1, ffn, 0, 0);
            rc = wri_op_fused_gelu_mul(&t_gate, &t_up, &t_gate);
            if (rc != WR_OK) return fail("geglu", L, rc);
            f32_tensor(&t_gate, rb->gate, 2, 1, ffn, 0);
            f32_tensor(&t_proj, rb->proj, 2, 1, hid, 0);
            rc = wri_op_matmul(&t_gate, &m->w_down[L], &t_proj);
            if (rc != WR_OK) return fail("down matmul", L, rc);
            f32_tensor(&t_proj, rb->proj, 1, hid, 0, 0);
            rc = wri_op_rmsnorm(&t_proj, &m->post_ffw_norm[L], &t_proj, eps);
            if (rc != WR_OK) return fail("post-ffw norm", L, rc);
            rc = wri_op_add(&t_res, &t_proj, &t_res);
            if (rc != WR_OK) return fail("ffn residual", L, rc);

            if (want_ple && m->inp_gate[L].data && m->pl_proj[L].data && m->post_norm[L].data) {
                float *table = sess[r]->ple + pl, *g = table + pl, *pli = g + ple, *delta = pli + ple;
                f32_tensor(&t_x, res, 2, 1, hid, 0);
                f32_tensor(&t_y, g, 2, 1, ple, 0);
                rc = wri_op_matmul(&t_x, &m->inp_gate[L], &t_y);
                if (rc != WR_OK) return fail("ple gate matmul", L, rc);
                memcpy(pli, table + (size_t)L * ple, (size_t)ple * sizeof(float));
                f32_tensor(&t_x, g, 1, ple, 0, 0);
                f32_tensor(&t_y, pli, 1, ple, 0, 0);
                rc = wri_op_fused_gelu_mul(&t_x, &t_y, &t_x);
                if (rc != WR_OK) return fail("ple geglu", L, rc);
                f32_tensor(&t_x, g, 2, 1, ple, 0);
                f32_tensor(&t_y, delta, 2, 1, hid, 0);
                rc = wri_op_matmul(&t_x, &m->pl_proj[L], &t_y);
                if (rc != WR_OK) return fail("ple proj matmul", L, rc);
                f32_tensor(&t_y, delta, 1, hid, 0, 0);
                rc = wri_op_rmsnorm(&t_y, &m->post_norm[L], &t_y, eps);
                if (rc != WR_OK) return fail("ple post norm", L, rc);
                rc = wri_op_add(&t_res, &t_y, &t_res);
                if (rc != WR_OK) return fail("ple residual", L, rc);
            }
            if (m->layer_output_scale[L].data) {     /* applied directly, no (1+w) (session.c:430-436) */
                const float sc = wri_read_elem_f32(&m->layer_output_scale[L], 0);
                if (sc != 1.0f)
                    for (uint32_t j = 0; j < hid; j++) res[j] *= sc;
            }
        }
    }
    return WR_OK;
}

/* Final RMSNorm into s->normed, then logits <- normed x lm_head (src/core/session.c:554). */
static wr_status finish_row(wr_session *s, const float *resid_row, int compute_logits)
{
    const wr_model *m = s->model;
    wr_tensor t_res;
    f32_tensor(&t_res, (float *)resid_row, 1, m->hidden_dim, 0, 0);
    int rc = wri_op_rmsnorm(&t_res, &m->final_norm, &s->normed, m->rms_eps);
    if (rc != WR_OK) return fail("final norm", m->n_layers, rc);
    memcpy(s->residual.data, resid_row, (size_t)m->hidden_dim * 4u);
    if (!compute_logits) return WR_OK;
    wr_tensor lmv, nv, lv;
    rc = wri_tensor_view_2d(&m->lm_head, m->hidden_dim, m->vocab_size, &lmv);
    if (rc != WR_OK) return fail("lm-head view", m->n_layers, rc);
    f32_tensor(&nv, (float *)s->normed.data, 2, 1, m->hidden_dim, 0);
    f32_tensor(&lv, (float *)s->logits.data, 2, 1, m->vocab_size, 0);
    rc = wri_op_matmul(&nv, &lmv, &lv);
    if (rc != WR_OK) return fail("lm-head matmul", m->n_layers, rc);
    if (m->is_gemma && m->logit_softcap > 0.0f)      /* x = cap * tanh(x / cap) (session.c:562-566) */
        wri_softcap((float *)s->logits.data, m->vocab_size, m->logit_softcap);
    return WR_OK;
}

/* The same pass with the layer glue on the device: one call, token ids in,
 * results for rows [out_from, R) out.  outs[i] is the session that receives row
 * out_from+i: its residual / normed tensors, and its logits when want_logits. */
static wr_status forward_device(const wr_model *m, wr_cuda_model *dm, row_buffers *rb, uint32_t R,
                                const uint32_t *tokens, wr_cuda_kv *const *kvs, const uint32_t *pos,
                                int mode, uint32_t out_from, wr_session *const *outs, int want_logits)
{
    if (R == 0 || R > rb->rows || out_from > R || R - out_from > WR_BATCH_MAX) return WR_ERR_INTERNAL;
    int crc = 0;
    wr_cuda_ctx *cuda = cuda_ctx(&crc);
    if (!cuda) return (crc < 0) ? (wr_status)crc : WR_ERR_UNSUPPORTED;
    const uint32_t hid = m->hidden_dim, nq = m->n_q_heads * m->head_dim, n_out = R - out_from;
    float *logit_ptrs[WR_BATCH_MAX];
    for (uint32_t i = 0; i < n_out; i++) logit_ptrs[i] = want_logits ? (float *)outs[i]->logits.data : NULL;
    float *tap = NULL;
    if (g_attn_tap) {
        tap = malloc((size_t)m->n_layers * R * nq * sizeof(float));
        if (!tap) return WR_ERR_NOMEM;
    }
    int rc = wr_cuda_model_forward(cuda, dm, mode == ATTN_DECODE ? WR_CUDA_FWD_DECODE : WR_CUDA_FWD_PREFILL,
                                   R, kvs, pos, tokens, out_from, n_out ? rb->hid_out : NULL,
                                   n_out ? rb->norm_out : NULL, (want_logits && n_out) ? logit_ptrs : NULL,
                                   NULL, tap);
    if (rc != 0) {
        free(tap);
        return fail("device forward pass", 0, rc);
    }
    /* what the host ops would have counted (kernels.c:990-991, :1423) */
    WRI_CTR_ADD(WR_CTR_ATTENTION_CALLS, (uint64_t)R * m->n_layers);
    WRI_CTR_ADD(WR_CTR_MATMUL_CALLS, (uint64_t)R * m->n_layers * 7u + (want_logits ? n_out : 0u));
    if (tap) {
        for (uint32_t L = 0; L < m->n_layers; L++)
            for (uint32_t r = 0; r < R; r++)
                g_attn_tap(g_attn_tap_user, L, mode == ATTN_DECODE ? pos[r] : pos[0] + r,
                           tap + ((size_t)L * R + r) * nq, nq);
        free(tap);
    }
    for (uint32_t i = 0; i < n_out; i++) {
        memcpy(outs[i]->residual.data, rb->hid_out + (size_t)i * hid, (size_t)hid * 4u);
        memcpy(outs[i]->normed.data, rb->norm_out + (size_t)i * hid, (size_t)hid * 4u);
    }
    return WR_OK;
}

/* One token of one session (the row's results land in the session's tensors). */
static wr_status step_one(wr_session *s, uint32_t token, int compute_logits)
{
    row_buffers *rb = &priv(s)->rb;
    wr_cuda_kv *kv = priv(s)->kv;
    uint32_t pos = s->pos;
    if (priv(s)->dm) {
        if (token >= s->model->vocab_size) return WR_ERR_INVAL;
        return forward_device(s->model, priv(s)->dm, rb, 1, &token, &kv, &pos, ATTN_DECODE, 0, &s,
                              compute_logits);
    }
    wr_status st;
    if (s->model->is_gemma) {
        b200_session *me = priv(s);
        st = forward_rows_gemma(s->model, &me, rb, 1, &token, &pos);
    } else {
        st = forward_rows(s->model, rb, 1, &token, &kv, &pos, ATTN_DECODE);
    }
    if (st == WR_OK) st = finish_row(s, rb->resid, compute_logits);
    return st;
}

/* One token of one session, without the LM head; pos is not advanced.
 * Kept as an external symbol because the reference exports it. */
wr_status wri_session_decode_body(wr_session *s, uint32_t token)
{
    return step_one(s, token, 0);
}

wr_status wri_session_step(wr_session *s, uint32_t token, int compute_logits)
{
    if (!s) return WR_ERR_INVAL;
    wr_mutex_lock(s->lock);
    wr_status st;
    if (s->pos >= s->max_context) {
        st = WR_ERR_CTX_FULL;                       /* consumed nothing */
    } else {
        st = step_one(s, token, compute_logits);
        if (st == WR_OK) __atomic_store_n(&s->pos, s->pos + 1, __ATOMIC_RELEASE);
    }
    __atomic_store_n(&s->last_status, st, __ATOMIC_RELEASE);
    wr_mutex_unlock(s->lock);
    return st;
}

int wri_session_prefill(wr_session *s, const uint32_t *ids, uint32_t n)
{
    if (!s) return WR_ERR_INVAL;
    if (n == 0) return 0;
    if (!ids) return WR_ERR_INVAL;
    wr_mutex_lock(s->lock);
    wr_status st = WR_OK;
    /* All-or-nothing (src/core/session.c:608-626): position and cache are
     * untouched unless every token goes through. */
    if ((uint64_t)s->pos + n > s->max_context) {
        st = WR_ERR_CTX_FULL;
    } else {
        const char *mode = getenv("WR_B200_PREFILL");
        const int by_token = (mode && strcmp(mode, "decode") == 0) || s->model->head_dim != 128 ||
                             s->model->is_gemma;
        wr_cuda_kv *kv = priv(s)->kv;
        row_buffers *rb = &priv(s)->rb;
        wr_cuda_model *dm = priv(s)->dm;
        if (dm) {
            for (uint32_t i = 0; i < n && st == WR_OK; i++)
                if (ids[i] >= s->model->vocab_size) st = WR_ERR_INVAL;   /* before anything is appended */
        }
        if (st != WR_OK) {
            /* refused */
        } else if (by_token) {
            uint32_t pos = s->pos;
            for (uint32_t i = 0; st == WR_OK && i < n; i++, pos++) {
                if (dm) {
                    st = forward_device(s->model, dm, rb, 1, &ids[i], &kv, &pos, ATTN_DECODE,
                                        (i + 1 == n) ? 0u : 1u, &s, 0);
                } else if (s->model->is_gemma) {
                    b200_session *me = priv(s);
                    st = forward_rows_gemma(s->model, &me, rb, 1, &ids[i], &pos);
                } else {
                    st = forward_rows(s->model, rb, 1, &ids[i], &kv, &pos, ATTN_DECODE);
                }
            }
            if (st == WR_OK && !dm) st = finish_row(s, rb->resid, 0);
        } else if (dm) {
            uint32_t done = 0;
            while (st == WR_OK && done < n) {
                const uint32_t cnt = (n - done < rb->rows) ? n - done : rb->rows;
                uint32_t pos = s->pos + done;
                const int last_chunk = (done + cnt == n);
                st = forward_device(s->model, dm, rb, cnt, ids + done, &kv, &pos, ATTN_PREFILL,
                                    last_chunk ? cnt - 1 : cnt, &s, 0);
                done += cnt;
            }
        } else {
            /* chunks of at most rb->rows tokens: rows are independent, key tiles absolute */
            uint32_t done = 0, last = 0;
            while (st == WR_OK && done < n) {
                last = (n - done < rb->rows) ? n - done : rb->rows;
                uint32_t pos = s->pos + done;
                st = forward_rows(s->model, rb, last, ids + done, &kv, &pos, ATTN_PREFILL);
                done += last;
            }
            if (st == WR_OK)
                st = finish_row(s, rb->resid + (size_t)(last - 1) * pad16(s->model->hidden_dim), 0);
        }
        if (st == WR_OK) __atomic_store_n(&s->pos, s->pos + n, __ATOMIC_RELEASE);
    }
    __atomic_store_n(&s->last_status, st, __ATOMIC_RELEASE);
    wr_mutex_unlock(s->lock);
    return (st == WR_OK) ? (int)n : (int)st;
}

int wr_prefill(wr_session *s, const uint32_t *ids, uint32_t n) { return wri_session_prefill(s, ids, n); }

const float *wr_step(wr_session *s, uint32_t token)
{
    if (!s) return NULL;
    if (wri_session_step(s, token, 1) != WR_OK) return NULL;
    return (const float *)s->logits.data;
}

/* -------------------------------------------------------------------- batch */

int wri_batch_decode_step(wr_session *const *sessions, const uint32_t *tokens, uint32_t n)
{
    if (!sessions || !tokens) return WR_ERR_INVAL;
    if (n == 0 || n > WR_BATCH_MAX) return WR_ERR_LIMIT;
    wr_model *m = sessions[0] ? sessions[0]->model : NULL;
    if (!m || !m->weights_committed) return WR_ERR_STATE;
    for (uint32_t i = 0; i < n; i++) {
        if (!sessions[i] || sessions[i]->model != m) return WR_ERR_INVAL;
        for (uint32_t j = 0; j < i; j++)
            if (sessions[i] == sessions[j]) return WR_ERR_INVAL;
    }
    /* lock in ascending address order (src/core/batch.c:106-120) */
    wr_session *order[WR_BATCH_MAX];
    for (uint32_t i = 0; i < n; i++) order[i] = sessions[i];
    for (uint32_t i = 1; i < n; i++)
        for (uint32_t j = i; j > 0 && (uintptr_t)order[j - 1] > (uintptr_t)order[j]; j--) {
            wr_session *t = order[j]; order[j] = order[j - 1]; order[j - 1] = t;
        }
    for (uint32_t i = 0; i < n; i++) wr_mutex_lock(order[i]->lock);

    wr_status st = WR_OK;
    for (uint32_t i = 0; i < n && st == WR_OK; i++)
        if (sessions[i]->pos >= sessions[i]->max_context) st = WR_ERR_CTX_FULL;
    if (st == WR_OK) {
        /* the rows of the whole batch live in the scratch of one of its (locked) sessions */
        row_buffers *rb = &priv(order[0])->rb;
        wr_cuda_kv *kvs[WR_BATCH_MAX];
        uint32_t pos[WR_BATCH_MAX];
        for (uint32_t i = 0; i < n; i++) { kvs[i] = priv(sessions[i])->kv; pos[i] = sessions[i]->pos; }
        wr_cuda_model *dm = priv(order[0])->dm;
        for (uint32_t i = 0; i < n && dm; i++)
            if (priv(sessions[i])->dm != dm) dm = NULL;
        if (dm) {
            for (uint32_t i = 0; i < n && st == WR_OK; i++)
                if (tokens[i] >= m->vocab_size) st = WR_ERR_INVAL;
            if (st == WR_OK)
                st = forward_device(m, dm, rb, n, tokens, kvs, pos, ATTN_DECODE, 0, sessions, 1);
        } else {
            if (m->is_gemma) {
                b200_session *bss[WR_BATCH_MAX];
                for (uint32_t i = 0; i < n; i++) bss[i] = priv(sessions[i]);
                st = forward_rows_gemma(m, bss, rb, n, tokens, pos);
            } else {
                st = forward_rows(m, rb, n, tokens, kvs, pos, ATTN_DECODE);    /* all sessions, one grid per layer */
            }
            for (uint32_t i = 0; i < n && st == WR_OK; i++)
                st = finish_row(sessions[i], rb->resid + (size_t)i * pad16(m->hidden_dim), 1);
        }
    }
    if (st == WR_OK)
        for (uint32_t i = 0; i < n; i++)
            __atomic_store_n(&sessions[i]->pos, sessions[i]->pos + 1, __ATOMIC_RELEASE);
    for (uint32_t i = 0; i < n; i++) __atomic_store_n(&sessions[i]->last_status, st, __ATOMIC_RELEASE);
    for (uint32_t i = n; i > 0; i--) wr_mutex_unlock(order[i - 1]->lock);
    return (st == WR_OK) ? (int)n : (int)st;
}

int wr_batch_step(wr_session *const *sessions, const uint32_t *tokens, uint32_t n, const float **logits_out)
{
    int rc = wri_batch_decode_step(sessions, tokens, n);
    if (rc < 0) return rc;
    if (logits_out)
        for (uint32_t i = 0; i < n; i++) logits_out[i] = (const float *)sessions[i]->logits.data;
    return rc;
}

/* --------------------------------------------------------------- self-tests
 *
 * Same contracts as the reference's fixtures (src/core/session.c:888-999,
 * src/core/batch.c:257-390) on a small synthetic model with patterned weights:
 * cursor accounting, refusal without consumption, CTX_FULL, and batched
 * logits byte-equal to serial ones.  They need a B200 (return -2 without). */

static int fx_alloc(wr_tensor *t, uint32_t ndim, uint32_t d0, uint32_t d1, uint16_t flags, uint32_t salt,
                    float constant)
{
    uint32_t shape[2] = { d0, d1 };
    if (wri_tensor_init(t, WR_DTYPE_F32, ndim, shape, flags, NULL) != WR_OK) return -1;
    uint64_t n = (uint64_t)d0 * (ndim > 1 ? d1 : 1);
    float *p = t->data;
    for (uint64_t i = 0; i < n; i++)
        p[i] = salt ? (float)((int32_t)((i * 37u + salt * 11u) % 41u) - 20) * 0.01f : constant;
    return 0;
}

static int fx_model(wr_model *m, uint32_t layers)
{
    memset(m, 0, sizeof(*m));
    m->n_layers = layers; m->n_q_heads = 4; m->n_kv_heads = 2; m->head_dim = 8;
    m->hidden_dim = 32; m->ffn_dim = 64; m->vocab_size = 64; m->max_context = 16;
    m->train_context = 16; m->rms_eps = 1e-5f; m->rope_freq_base = 10000.0f;
    m->weights_committed = 1;
    m->lock = wr_mutex_create();
    if (!m->lock) return -1;
    int bad = 0;
    bad |= fx_alloc(&m->embed_table, 2, 64, 32, 0, 3, 0);
    bad |= fx_alloc(&m->final_norm, 1, 32, 0, 0, 0, 1.0f);
    bad |= fx_alloc(&m->lm_head, 2, 64, 32, WR_TENSOR_GGML_WEIGHT, 5, 0);
    for (uint32_t L = 0; L < layers; L++) {
        bad |= fx_alloc(&m->attn_norm[L], 1, 32, 0, 0, 0, 1.0f);
        bad |= fx_alloc(&m->ffn_norm[L], 1, 32, 0, 0, 0, 1.0f);
        /* GGML matmul weights carry the logical [in, out] shape (src/core/session.c:909-911) */
        bad |= fx_alloc(&m->wq[L], 2, 32, 32, WR_TENSOR_GGML_WEIGHT, 7 + L, 0);
        bad |= fx_alloc(&m->wk[L], 2, 32, 16, WR_TENSOR_GGML_WEIGHT, 9 + L, 0);
        bad |= fx_alloc(&m->wv[L], 2, 32, 16, WR_TENSOR_GGML_WEIGHT, 11 + L, 0);
        bad |= fx_alloc(&m->wo[L], 2, 32, 32, WR_TENSOR_GGML_WEIGHT, 13 + L, 0);
        bad |= fx_alloc(&m->w_gate[L], 2, 32, 64, WR_TENSOR_GGML_WEIGHT, 15 + L, 0);
        bad |= fx_alloc(&m->w_up[L], 2, 32, 64, WR_TENSOR_GGML_WEIGHT, 17 + L, 0);
        bad |= fx_alloc(&m->w_down[L], 2, 64, 32, WR_TENSOR_GGML_WEIGHT, 19 + L, 0);
    }
    return bad;
}

static void fx_model_free(wr_model *m)
{
    wri_tensor_free(&m->embed_table);
    wri_tensor_free(&m->final_norm);
    wri_tensor_free(&m->lm_head);
    for (uint32_t L = 0; L < m->n_layers; L++) {
        wri_tensor_free(&m->attn_norm[L]); wri_tensor_free(&m->ffn_norm[L]);
        wri_tensor_free(&m->wq[L]); wri_tensor_free(&m->wk[L]); wri_tensor_free(&m->wv[L]);
        wri_tensor_free(&m->wo[L]); wri_tensor_free(&m->w_gate[L]); wri_tensor_free(&m->w_up[L]);
        wri_tensor_free(&m->w_down[L]);
    }
    if (m->lock) wr_mutex_destroy(m->lock);
}

int wri_self_test_llm_step(void)
{
    int crc = 0;
    if (!cuda_ctx(&crc)) return -2;
    wr_model *m = calloc(1, sizeof(*m));
    if (!m) return -1;
    int ret = -1;
    wr_session *s = NULL;
    if (fx_model(m, 2) != 0) goto out;
    if (wr_session_create(m, NULL, &s) != WR_OK) goto out;
    if (wr_session_pos(s) != 0 || wr_session_max_context(s) != 16) goto out;
    if (!wr_step(s, 3) || wr_session_pos(s) != 1) goto out;                 /* cursor 0 -> 1 */
    if (wr_step(s, 64) != NULL || wr_session_pos(s) != 1) goto out;         /* out-of-vocab: nothing consumed */
    if (wr_session_status(s) != WR_ERR_INVAL) goto out;
    uint32_t ids[14];
    for (uint32_t i = 0; i < 14; i++) ids[i] = (i * 5u + 1u) % 64u;
    if (wr_prefill(s, ids, 14) != 14 || wr_session_pos(s) != 15) goto out;
    if (wr_prefill(s, ids, 2) != WR_ERR_CTX_FULL || wr_session_pos(s) != 15) goto out;  /* all-or-nothing */
    if (!wr_step(s, 7) || wr_session_pos(s) != 16) goto out;                /* now full */
    if (wr_step(s, 7) != NULL || wr_session_status(s) != WR_ERR_CTX_FULL) goto out;
    if (wr_session_pos(s) != 16) goto out;                                   /* CTX_FULL consumed nothing */
    ret = 0;
out:
    if (s) wr_session_destroy(s);
    fx_model_free(m);
    free(m);
    return ret;
}

int wri_self_test_batch_step(void)
{
    enum { N = 3, STEPS = 4 };
    int crc = 0;
    if (!cuda_ctx(&crc)) return -2;
    wr_model *m = calloc(1, sizeof(*m));
    if (!m) return -1;
    int ret = -1;
    wr_session *ser[N] = { 0 }, *bat[N] = { 0 };
    float *keep = NULL;
    if (fx_model(m, 1) != 0) goto out;
    keep = malloc(sizeof(float) * N * STEPS * 64);
    if (!keep) goto out;
    for (int i = 0; i < N; i++)
        if (wr_session_create(m, NULL, &ser[i]) != WR_OK || wr_session_create(m, NULL, &bat[i]) != WR_OK)
            goto out;
    for (int t = 0; t < STEPS; t++)
        for (int i = 0; i < N; i++) {
            const float *lg = wr_step(ser[i], (uint32_t)((i * 7 + t * 3 + 1) % 64));
            if (!lg) goto out;
            memcpy(keep + ((size_t)t * N + i) * 64, lg, 64 * sizeof(float));
        }
    for (int t = 0; t < STEPS; t++) {
        uint32_t toks[N];
        const float *lg[N];
        for (int i = 0; i < N; i++) toks[i] = (uint32_t)((i * 7 + t * 3 + 1) % 64);
        if (wr_batch_step((wr_session *const *)bat, toks, N, lg) != N) goto out;
        for (int i = 0; i < N; i++)
            if (memcmp(lg[i], keep + ((size_t)t * N + i) * 64, 64 * sizeof(float)) != 0) goto out;   /* byte-equal */
    }
    ret = 0;
out:
    for (int i = 0; i < N; i++) { if (ser[i]) wr_session_destroy(ser[i]); if (bat[i]) wr_session_destroy(bat[i]); }
    free(keep);
    fx_model_free(m);
    free(m);
    return ret;
}
