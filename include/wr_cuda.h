/*
 * wr_cuda.h — C-ABI of the B200 (sm_100a) attention hot path for wayruntime.
 *
 * This is the seam the reference's C11 host code (src/core/session.c,
 * src/core/batch.c) calls in place of its CPU ops:
 *
 *   wr_cuda_kv_append     <- wri_op_rope on Q and K + kv_append_row on K and V
 *                            (src/core/session.c:471-487, kernels.c:1356,
 *                             session.c:139)
 *   wr_cuda_attn_decode   <- wri_op_gqa_attention with seq_q = 1, once per
 *                            session (src/core/session.c:490-496,
 *                             kernels.c:1414; batched: batch.c:152-164)
 *   wr_cuda_attn_prefill  <- the wri_session_prefill loop of single-token
 *                            attention calls (src/core/session.c:599-630)
 *
 * Plain pointers and sizes only.  Every function returns a wr_status value
 * (include/wayruntime/wayruntime.h:82-107): 0 or a negative code; nothing
 * aborts, prints or falls back to the CPU.  There is no CPU path: without an
 * sm_100 device every entry point fails with WR_CUDA_ERR_UNSUPPORTED.
 *
 * Threading: a context serialises its own calls with a mutex, so distinct
 * sessions may be driven from distinct threads (wayruntime.h:29-40).
 */
#ifndef WR_CUDA_H
#define WR_CUDA_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* wr_status values used here (wayruntime.h:82-107). */
#define WR_CUDA_OK               0
#define WR_CUDA_ERR_UNSUPPORTED (-3)
#define WR_CUDA_ERR_INVAL       (-4)
#define WR_CUDA_ERR_NOMEM       (-5)
#define WR_CUDA_ERR_CTX_FULL    (-6)
#define WR_CUDA_ERR_STATE       (-7)
#define WR_CUDA_ERR_LIMIT       (-8)
#define WR_CUDA_ERR_INTERNAL    (-10)

/* Where the caller's Q / K / V / output buffers live. */
#define WR_CUDA_MEM_HOST   0   /* host memory; the call copies and synchronises */
#define WR_CUDA_MEM_DEVICE 1   /* device memory; the call only enqueues */

/* Element types (values of wr_dtype, src/core/internal.h:53-55). */
#define WR_CUDA_F32 0
#define WR_CUDA_F16 1

/* wr_cuda_kv_append flags. */
#define WR_CUDA_APPEND_ROPE 1u  /* rotate K (and Q when given) before storing */

#define WR_CUDA_BATCH_MAX        16    /* WR_BATCH_MAX, wayruntime.h:423 */
#define WR_CUDA_ATTN_MAX_SEQ     4096  /* default cap, WR_ATTN_MAX_SEQ (internal.h:186) */
#define WR_CUDA_ATTN_MAX_SEQ_TOP 1048576
#define WR_CUDA_HEAD_DIM_MAX     1024  /* WR_FLASH_D_MAX (internal.h:197) */
#define WR_CUDA_PAGE_TOKENS      64    /* tokens per KV page = WR_FLASH_BLOCK */
#define WR_CUDA_TRIPLE_PAD       4     /* floats before o[] in a split-KV triple */

typedef struct wr_cuda_ctx wr_cuda_ctx;  /* one device, one stream, one page pool */
typedef struct wr_cuda_kv  wr_cuda_kv;   /* one session's paged F16 K/V cache   */

/* ---- device / context -------------------------------------------------- */

/* WR_CUDA_OK when `device` exists and is compute capability 10.x.  This is
 * the check wr_engine_create makes beside its endian probe
 * (src/core/engine.c:130): no B200 bound -> WR_ERR_UNSUPPORTED. */
int wr_cuda_device_check(int device);

int  wr_cuda_ctx_create(int device, wr_cuda_ctx **out);
void wr_cuda_ctx_destroy(wr_cuda_ctx *ctx);

/* Wait for everything enqueued on the context's stream.  Also reports (and
 * clears) a device-side error flag: a bounded wait that gave up inside a
 * kernel surfaces here — and at the end of every call that takes
 * WR_CUDA_MEM_HOST buffers — as WR_CUDA_ERR_INTERNAL. */
int  wr_cuda_ctx_sync(wr_cuda_ctx *ctx);

/* The context's cudaStream_t, for callers that time or order against it. */
void *wr_cuda_ctx_stream(wr_cuda_ctx *ctx);

/* Sequence cap for sessions and attention calls on this context; the
 * reference's WR_ATTN_MAX_SEQ is a compile-time constant (internal.h:186),
 * here it is a setting so long-context shards need no rebuild. */
int  wr_cuda_ctx_set_attn_max_seq(wr_cuda_ctx *ctx, uint32_t max_seq);

/* Every device-side wait in this library (an mbarrier phase, an arrival
 * counter, a peer's flag) gives up after this many cycles of SM clock: the
 * kernel records an error word, unwinds and returns, and the next call that
 * synchronises (wr_cuda_ctx_sync, or any call with WR_CUDA_MEM_HOST buffers)
 * returns WR_CUDA_ERR_INTERNAL once and clears the word; the context stays
 * usable.  The reference has no counterpart (its ops cannot stall); the
 * contract kept is its "a failed step consumes nothing" (session.c:160-168,
 * :589-592).  Default WR_CUDA_WAIT_LIMIT_DEFAULT, about two seconds. */
#define WR_CUDA_WAIT_LIMIT_DEFAULT 4000000000LL
int  wr_cuda_ctx_set_wait_limit(wr_cuda_ctx *ctx, int64_t cycles);
/* The error word of the last give-up reported (0: none yet): a small number
 * naming the wait that ran out, for a log line next to WR_CUDA_ERR_INTERNAL. */
int  wr_cuda_ctx_last_device_error(wr_cuda_ctx *ctx);

/* Page-locked host memory for a caller's row buffers (Q / K / V / attention
 * rows): with such buffers the WR_CUDA_MEM_HOST calls need no staging copy —
 * the decode kernels read and write them in place.  The reference's session
 * scratch comes from one arena sized at create (session.c:699-708); a host
 * layer allocates these once per session in the same place and frees them at
 * destroy.  64-byte aligned.  WR_CUDA_ERR_NOMEM when the host cannot pin. */
int  wr_cuda_host_alloc(wr_cuda_ctx *ctx, uint64_t bytes, void **out);
void wr_cuda_host_free(wr_cuda_ctx *ctx, void *p);

/* Number of kernels this library has launched on the context so far. */
uint64_t wr_cuda_ctx_launch_count(wr_cuda_ctx *ctx);

/* ---- KV cache (session_build / wr_session_create, session.c:640-814) ---- */

/* All pages of the session are taken from the context's pool here, once:
 * no allocation happens during decode.  max_ctx above the context's cap is
 * WR_CUDA_ERR_LIMIT (session.c:755). */
int  wr_cuda_kv_create(wr_cuda_ctx *ctx, uint32_t n_layers, uint32_t n_kv_heads,
                       uint32_t head_dim, uint32_t max_ctx, wr_cuda_kv **out);
void wr_cuda_kv_destroy(wr_cuda_kv *kv);
uint32_t wr_cuda_kv_max_ctx(const wr_cuda_kv *kv);

/* Copy rows [row0, row0+n) of one layer's K (which=0) or V (which=1) between
 * the paged cache and a [n, n_kv_heads, head_dim] F16 buffer in the
 * reference's row layout (session.c:647-674).  Used to load a prepared cache
 * and to compare cache bytes with the reference's. */
int wr_cuda_kv_write_rows(wr_cuda_ctx *ctx, wr_cuda_kv *kv, uint32_t layer,
                          int which, uint32_t row0, uint32_t n,
                          const uint16_t *src, int mem);
int wr_cuda_kv_read_rows(wr_cuda_ctx *ctx, wr_cuda_kv *kv, uint32_t layer,
                         int which, uint32_t row0, uint32_t n, uint16_t *dst,
                         int mem);

/* ---- the hot path -------------------------------------------------------- */

/* Fused RoPE + KV append for one layer.  Session s contributes n_tokens
 * consecutive rows at cache rows positions[s] .. positions[s]+n_tokens-1
 * (its absolute positions).  k_rows, v_rows: F32 [n_sess*n_tokens,
 * n_kv_heads, head_dim].  With WR_CUDA_APPEND_ROPE, K is rotated with the
 * reference's RoPE (kernels.c:1356-1412: its polynomial sin/cos, pairing j
 * with j+head_dim/2, n_rot_pairs as there) and q_rows — F32
 * [n_sess*n_tokens, n_q_heads, head_dim], may be NULL — is rotated in place.
 * K and V are stored with the reference's truncating F32->F16
 * (quant.c:121-136), so cache bytes equal the reference's.
 * The call does not move any committed length: the host passes seq_lens to
 * the attention calls and simply does not advance them when a step fails
 * (wri_session_kv_rollback, session.c:160).  A row past max_ctx is
 * WR_CUDA_ERR_CTX_FULL before anything is launched (session.c:144). */
int wr_cuda_kv_append(wr_cuda_ctx *ctx, uint32_t n_sess, wr_cuda_kv *const *kv,
                      uint32_t layer, const uint32_t *positions,
                      uint32_t n_tokens, const float *k_rows,
                      const float *v_rows, float *q_rows, uint32_t n_q_heads,
                      float theta_base, uint32_t n_rot_pairs, uint32_t flags,
                      int mem);

/* Decode attention, all sessions in one grid.  q, out: F32 [n_sess,
 * n_q_heads, head_dim] (q already rotated, e.g. by wr_cuda_kv_append).
 * seq_lens[s] = rows of session s to attend (the row just appended
 * included).  scale_override <= 0 selects 1/sqrt(head_dim); window > 0
 * keeps the last `window` keys (kernels.c:1456-1464).  Validation follows
 * kernels.c:1418-1454.  A session's result does not depend on which other
 * sessions share the call. */
int wr_cuda_attn_decode(wr_cuda_ctx *ctx, uint32_t n_sess,
                        wr_cuda_kv *const *kv, uint32_t layer,
                        const uint32_t *seq_lens, const float *q, float *out,
                        uint32_t n_q_heads, float scale_override,
                        uint32_t window, int mem);

/* The batched decode layer-step in one call: wr_cuda_kv_append with
 * n_tokens = 1 followed by wr_cuda_attn_decode over seq_lens[s] =
 * positions[s] + 1 — the per-layer body of wri_batch_decode_step
 * (src/core/batch.c:152-164 -> session.c:471-496) for all sessions at once.
 * q: F32 [n_sess, n_q_heads, head_dim], un-rotated on entry (rotated in
 * place when it is device memory); out: F32 of the same shape.  With host
 * buffers q, k_rows and v_rows cross the bus once and only out comes back;
 * page-locked host buffers are read and written by the kernels themselves (no
 * copy operations), pageable ones are staged.  Host q rows are left as given. */
int wr_cuda_decode_step(wr_cuda_ctx *ctx, uint32_t n_sess, wr_cuda_kv *const *kv,
                        uint32_t layer, const uint32_t *positions, float *q,
                        const float *k_rows, const float *v_rows, float *out,
                        uint32_t n_q_heads, float theta_base, uint32_t n_rot_pairs,
                        uint32_t flags, float scale_override, uint32_t window,
                        int mem);

/* Decode attention that never allocates.  (No counterpart in the reference:
 * its attention op mallocs a scratch row on every call, kernels.c:1471.)
 * Same arguments, checks and result as wr_cuda_attn_decode with device
 * buffers, but the split-KV scratch lives in a fixed array inside the library
 * image instead of buffers the context grows on demand.  It is meant for
 * callers that may not allocate at step time — a serving loop whose device
 * memory is fully committed to the KV pool, a thread that must not enter the
 * CUDA allocator.  head_dim 128 only; q and out are device memory; a call
 * needing more than WR_CUDA_STATIC_MAX_ITEMS work items (sessions x kv heads
 * x key chunks) or WR_CUDA_STATIC_MAX_GROUPS groups is WR_CUDA_ERR_LIMIT.
 * The first call on a device resolves the array's address: make it before
 * opening a stream capture.  All calls share the one array per device, so
 * calls that overlap on the GPU race; issue them one after another. */
#define WR_CUDA_STATIC_MAX_ITEMS  4096
#define WR_CUDA_STATIC_MAX_GROUPS 1024
int wr_cuda_attn_decode_static(wr_cuda_ctx *ctx, uint32_t n_sess,
                               wr_cuda_kv *const *kv, uint32_t layer,
                               const uint32_t *seq_lens, const float *q,
                               float *out, uint32_t n_q_heads,
                               float scale_override, uint32_t window);

/* Causal prefill attention for n new tokens of one session whose rows
 * [0, p0+n) are already in the cache: query i attends rows [0, p0+i]
 * (row i of the reference's prefill loop, session.c:599-630).
 * q: [n, n_q_heads, head_dim] of q_dtype; out: F32 of the same shape. */
int wr_cuda_attn_prefill(wr_cuda_ctx *ctx, wr_cuda_kv *kv, uint32_t layer,
                         uint32_t p0, uint32_t n, const void *q, int q_dtype,
                         float *out, uint32_t n_q_heads, float scale_override,
                         uint32_t window, int mem);

/* ---- split-KV across devices --------------------------------------------- */

/* Like wr_cuda_attn_decode over this device's shard of each session's keys,
 * but emits one triple per (session, q head) instead of the normalised row:
 * triples is F32 [n_sess, n_q_heads, WR_CUDA_TRIPLE_PAD + head_dim] holding
 * (m, l, 0, 0, o[head_dim]) with m the running max (natural-log domain,
 * -1e30 for an empty shard), l the denominator and o the unnormalised
 * accumulator — the state of kernels.c:1480-1516 after the shard's keys.
 * seq_lens[s] may be 0 (empty shard). */
int wr_cuda_attn_decode_partial(wr_cuda_ctx *ctx, uint32_t n_sess,
                                wr_cuda_kv *const *kv, uint32_t layer,
                                const uint32_t *seq_lens, const float *q,
                                float *triples, uint32_t n_q_heads,
                                float scale_override, int mem);

/* Merge n_shards triples per row with the online-softmax rule
 * (kernels.c:1503-1506 applied across shards): triples is F32 [n_shards,
 * n_rows, WR_CUDA_TRIPLE_PAD + head_dim], out F32 [n_rows, head_dim]. */
int wr_cuda_attn_combine(wr_cuda_ctx *ctx, uint32_t n_shards, uint32_t n_rows,
                         uint32_t head_dim, const float *triples, float *out,
                         int mem);

/* ---- Peer exchange for key-sharded decode (no reference counterpart: the
 * reference is single-device; this is the multi-GPU form of the merge above).
 *
 * One process per GPU.  Every rank creates an exchange object (a device
 * buffer for world x max_rows triples, twice, plus flags), publishes its
 * handle (WR_CUDA_XCHG_HANDLE_BYTES opaque bytes, valid in other processes of
 * this machine), receives everybody's handles in rank order by whatever
 * transport the host has, and connects: the peers' buffers are then mapped
 * over NVLink.  WR_CUDA_ERR_UNSUPPORTED when two of the devices cannot reach
 * each other's memory. */
typedef struct wr_cuda_xchg wr_cuda_xchg;
#define WR_CUDA_XCHG_MAX_WORLD    8
#define WR_CUDA_XCHG_HANDLE_BYTES 64

int  wr_cuda_xchg_create(wr_cuda_ctx *ctx, uint32_t world, uint32_t rank,
                         uint32_t max_rows, uint32_t head_dim, wr_cuda_xchg **out);
int  wr_cuda_xchg_handle(wr_cuda_xchg *x, void *handle_out);
int  wr_cuda_xchg_connect(wr_cuda_xchg *x, const void *handles /* world x 64 bytes */);
/* The same connection for exchange objects that live in ONE process (one
 * thread per GPU, or several contexts of a test): all[r] is rank r's object;
 * devices other than the caller's need peer access enabled by the host. */
int  wr_cuda_xchg_connect_local(wr_cuda_xchg *x, wr_cuda_xchg *const *all);
/* Destroy is collective: a peer's kernel may still be storing into this
 * rank's buffer, so every rank first synchronises its context
 * (wr_cuda_ctx_sync, also after a step that timed out) and the ranks agree
 * (a barrier of the host's transport) before any of them destroys. */
void wr_cuda_xchg_destroy(wr_cuda_xchg *x);

/* All-gather + merge in one kernel: stores this rank's triples (device, F32
 * [n_rows, WR_CUDA_TRIPLE_PAD + head_dim], as written by
 * wr_cuda_attn_decode_partial) into every rank's buffer, waits (bounded; an
 * expired wait surfaces at wr_cuda_ctx_sync as WR_CUDA_ERR_INTERNAL) for every
 * rank's triples of the same step, and merges them in rank order into out
 * (device, F32 [n_rows, head_dim]).  Every rank must make the same sequence of
 * calls with the same n_rows.  Enqueues on the context's stream and returns. */
int wr_cuda_attn_exchange_combine(wr_cuda_ctx *ctx, wr_cuda_xchg *x, uint32_t n_rows,
                                  const float *triples, float *out);

/* Key-sharded decode with the exchange fused into the decode kernel (no
 * reference counterpart, as above): wr_cuda_attn_decode_partial and
 * wr_cuda_attn_exchange_combine in one call.  The decode kernel's own warps
 * store every finished (session, q head) triple into all ranks' buffers,
 * flag each row there, wait (bounded) for the same rows from every rank and
 * merge them in rank order into out (device, F32 [n_sess, n_q_heads,
 * head_dim]) — one kernel.  Where a session of this rank has fewer than two
 * key chunks (a short or empty shard) the rows are published per step instead
 * and a small second kernel does the waiting and merging.  q is device
 * memory; head_dim 128.  Identical bits to the two-call sequence.  Every rank
 * makes the same sequence of calls. */
int wr_cuda_attn_decode_exchange(wr_cuda_ctx *ctx, wr_cuda_xchg *x, uint32_t n_sess,
                                 wr_cuda_kv *const *kv, uint32_t layer,
                                 const uint32_t *seq_lens, const float *q, float *out,
                                 uint32_t n_q_heads, float scale_override);

/* ---- the layer stack around attention, device-resident ------------------- */

/* A device copy of one model's F32 weights plus the row scratch of a forward
 * pass.  Replaces, for the callers of attention, the host loop of the
 * reference's decode body (src/core/session.c:405-568: RMSNorm, Q/K/V
 * projections, per-head QK-norm, attention, output projection, residual,
 * RMSNorm, SwiGLU FFN, residual; then final RMSNorm and LM head,
 * session.c:540-560) so that a row enters the device as a token id and leaves
 * as logits instead of crossing the bus twice per layer.  Llama / Qwen3-class
 * layers only (no sandwich norms, no per-layer embeddings).
 *
 * Weights are host pointers to F32 data in the GGML layout the reference keeps
 * them in: a [in -> out] projection is out rows of in floats
 * (src/core/kernels.c:978-1000).  embed and lm_head are [vocab][hidden]; they
 * may be the same pointer (tied), and are then uploaded once. */
#define WR_CUDA_MAX_LAYERS  64   /* WR_MAX_LAYERS, src/core/internal.h:184 */
#define WR_CUDA_FWD_DECODE  0    /* row r = next token of session kv[r] at positions[r] */
#define WR_CUDA_FWD_PREFILL 1    /* rows = consecutive tokens of kv[0] from positions[0] */

typedef struct wr_cuda_model wr_cuda_model;

typedef struct wr_cuda_layer_desc {
    const float *attn_norm;           /* [hidden] */
    const float *wq, *wk, *wv;        /* [n_q*hd][hidden], [n_kv*hd][hidden] x2 */
    const float *q_norm, *k_norm;     /* [head_dim] each, or both NULL */
    const float *wo;                  /* [hidden][n_q*hd] */
    const float *ffn_norm;            /* [hidden] */
    const float *w_gate, *w_up;       /* [ffn_dim][hidden] */
    const float *w_down;              /* [hidden][ffn_dim] */
    uint32_t ffn_dim, reserved;
} wr_cuda_layer_desc;

typedef struct wr_cuda_model_desc {
    uint32_t n_layers, hidden, n_q_heads, n_kv_heads, head_dim, vocab;
    uint32_t n_rot_pairs;             /* as wr_cuda_kv_append */
    uint32_t max_rows;                /* rows one forward pass may carry (prefill chunk) */
    float rms_eps, rope_theta, attn_scale /* <= 0: 1/sqrt(head_dim) */, reserved;
    const float *embed, *lm_head, *final_norm;
    const wr_cuda_layer_desc *layers; /* n_layers entries */
} wr_cuda_model_desc;

/* Uploads every weight (one device allocation) and takes the row scratch; the
 * host copies are not referenced after the call returns. */
int  wr_cuda_model_create(wr_cuda_ctx *ctx, const wr_cuda_model_desc *desc, wr_cuda_model **out);
void wr_cuda_model_destroy(wr_cuda_model *m);
uint64_t wr_cuda_model_bytes(const wr_cuda_model *m);      /* device bytes held */
uint64_t wr_cuda_model_launches(const wr_cuda_model *m);   /* glue kernels launched so far */
/* host time, in ns, that the last forward pass spent enqueueing before it began to wait for the device */
uint64_t wr_cuda_model_last_enqueue_ns(const wr_cuda_model *m);

/* One forward pass over n_rows rows (decode: n_rows <= WR_CUDA_BATCH_MAX
 * sessions, one new token each; prefill: n_rows <= max_rows tokens of one
 * session), KV appended at `positions` as wr_cuda_decode_step /
 * wr_cuda_kv_append do — the caller commits the new length only when the call
 * returns 0.  A token id >= vocab is WR_CUDA_ERR_INVAL before anything runs
 * (session.c:413).  Results are written for rows [out_from, n_rows), all to
 * host memory, each pointer optional: hidden_out [n][hidden] (the residual
 * stream before the final norm), normed_out [n][hidden], logits_out[i] ->
 * [vocab] for row out_from+i (an entry may be NULL), argmax_out[i] = the first
 * maximum of that row's logits (the lowest id wins a tie, src/cli/wayrt.c:805).
 * Logits / arg-max for at most WR_CUDA_BATCH_MAX rows per call.  attn_tap_out,
 * when given, receives every layer's attention rows, [n_layers][n_rows][n_q*hd].
 * The call synchronises and reports a device-side give-up like every
 * host-buffer call.  One forward pass per model at a time (serialised inside). */
int wr_cuda_model_forward(wr_cuda_ctx *ctx, wr_cuda_model *m, int mode, uint32_t n_rows,
                          wr_cuda_kv *const *kv, const uint32_t *positions,
                          const uint32_t *tokens, uint32_t out_from, float *hidden_out,
                          float *normed_out, float *const *logits_out, uint32_t *argmax_out,
                          float *attn_tap_out);

#ifdef __cplusplus
}
#endif
#endif
