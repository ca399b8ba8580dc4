// attn_decode.cu — host side of decode attention, the any-head_dim kernel and
// the cross-shard combine.
//
// Reference behaviour restated here (paths inside the reference project):
//   wri_op_gqa_attention, seq_q = 1      src/core/kernels.c:1414-1527
//   per-session loop of a batched step   src/core/batch.c:152-164
//   per-layer decode body                src/core/session.c:471-496
#include <algorithm>

#include "attn_decode_hd128.cuh"
#include "wr_internal.cuh"

namespace {

// ---------------------------------------------------------------- generic
//
// Any head_dim (the reference accepts every even head_dim up to 1024; its own
// known-answer tests use 2, 4 and 8).  One CTA per (session, q head); each
// warp owns an interleaved subset of the keys with its own online-softmax
// state; lanes stride the head dimension.  Correctness path, not tuned.
struct generic_params {
    wr_batch_desc b;
    uint32_t key_lo[WR_CUDA_BATCH_MAX];
    const float *q;
    float *out;
    uint32_t n_sess, n_q, n_kv, group, hd, emit_triples;
    float scale;
};

constexpr int kGenWarps = 4;
constexpr int kGenDPerLane = WR_CUDA_HEAD_DIM_MAX / 32;

__global__ void __launch_bounds__(kGenWarps * 32) attn_decode_generic_kernel(const generic_params p)
{
    extern __shared__ float gsm[];   // [warps][hd] + m[warps] + l[warps]
    const uint32_t s = blockIdx.x / p.n_q, qh = blockIdx.x % p.n_q;
    const uint32_t kvh = qh / p.group;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t hd = p.hd, seq_len = p.b.seq_len[s], key_lo = p.key_lo[s];
    const float *qrow = p.q + ((size_t)s * p.n_q + qh) * hd;
    const uint64_t *pages = p.b.pages[s];

    float qv[kGenDPerLane], o[kGenDPerLane];
#pragma unroll
    for (int i = 0; i < kGenDPerLane; ++i) {
        uint32_t d = lane + i * 32;
        qv[i] = d < hd ? qrow[d] : 0.f;
        o[i] = 0.f;
    }
    float m = WR_NEG_SENTINEL, l = 0.f;
    for (uint32_t key = key_lo + warp; key < seq_len; key += kGenWarps) {
        const char *page = (const char *)pages[key / kPageTokens];
        const uint32_t tok = key % kPageTokens;
        const char *kb = page + wr_block_off(kvh, 0, hd);
        const char *vb = page + wr_block_off(kvh, 1, hd);
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < kGenDPerLane; ++i) {
            uint32_t d = lane + i * 32;
            if (d < hd) dot += qv[i] * __half2float(*(const __half *)(kb + wr_elem_off(tok, d, hd)));
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
        const float sc = dot * p.scale;
        const float m_new = fmaxf(m, sc);
        const float a = (m == WR_NEG_SENTINEL) ? 0.f : __expf(m - m_new);
        const float pw = __expf(sc - m_new);
        l = l * a + pw;
#pragma unroll
        for (int i = 0; i < kGenDPerLane; ++i) {
            uint32_t d = lane + i * 32;
            if (d < hd)
                o[i] = o[i] * a + pw * __half2float(*(const __half *)(vb + wr_elem_off(tok, d, hd)));
        }
        m = m_new;
    }
    float *so = gsm;
    float *smm = gsm + kGenWarps * hd;
    float *sl = smm + kGenWarps;
#pragma unroll
    for (int i = 0; i < kGenDPerLane; ++i) {
        uint32_t d = lane + i * 32;
        if (d < hd) so[warp * hd + d] = o[i];
    }
    if (lane == 0) { smm[warp] = m; sl[warp] = l; }
    __syncthreads();
    float mstar = WR_NEG_SENTINEL;
    for (int wv = 0; wv < kGenWarps; ++wv) mstar = fmaxf(mstar, smm[wv]);
    float L = 0.f;
    float wg[kGenWarps];
    for (int wv = 0; wv < kGenWarps; ++wv) {
        wg[wv] = (smm[wv] == WR_NEG_SENTINEL) ? 0.f : __expf(smm[wv] - mstar);
        L += wg[wv] * sl[wv];
    }
    const size_t row = (size_t)s * p.n_q + qh;
    for (uint32_t d = threadIdx.x; d < hd; d += blockDim.x) {
        float acc = 0.f;
        for (int wv = 0; wv < kGenWarps; ++wv) acc += wg[wv] * so[wv * hd + d];
        if (p.emit_triples) p.out[row * (WR_CUDA_TRIPLE_PAD + hd) + WR_CUDA_TRIPLE_PAD + d] = acc;
        else p.out[row * hd + d] = (L > 0.f) ? acc / L : 0.f;
    }
    if (p.emit_triples && threadIdx.x == 0) {
        float *tr = p.out + row * (WR_CUDA_TRIPLE_PAD + hd);
        tr[0] = mstar; tr[1] = L; tr[2] = 0.f; tr[3] = 0.f;
    }
}

// Cross-shard merge of (m, l, o) triples: one thread per output element.
__global__ void attn_combine_kernel(const float *__restrict__ triples, float *__restrict__ out,
                                    uint32_t n_shards, uint32_t n_rows, uint32_t hd)
{
    const uint32_t stride = WR_CUDA_TRIPLE_PAD + hd;
    const uint64_t total = (uint64_t)n_rows * hd;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total;
         i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t row = (uint32_t)(i / hd), d = (uint32_t)(i % hd);
        float mstar = WR_NEG_SENTINEL;
        for (uint32_t g = 0; g < n_shards; ++g)
            mstar = fmaxf(mstar, triples[((size_t)g * n_rows + row) * stride]);
        float L = 0.f, acc = 0.f;
        for (uint32_t g = 0; g < n_shards; ++g) {
            const float *tr = triples + ((size_t)g * n_rows + row) * stride;
            const float wgt = (tr[0] == WR_NEG_SENTINEL) ? 0.f : __expf(tr[0] - mstar);
            L += wgt * tr[1];
            acc += wgt * tr[WR_CUDA_TRIPLE_PAD + d];
        }
        out[i] = (L > 0.f) ? acc / L : 0.f;
    }
}

float scale_for(uint32_t hd, float scale_override)
{
    if (scale_override > 0.0f) return scale_override;   // kernels.c:1457-1459
    // wri_sqrt (mathx.c:98-110) returns the correctly rounded root for the
    // head dims in use; 1/sqrtf in float is the same value.
    return 1.0f / sqrtf((float)hd);
}

}  // namespace

// Argument checks of wri_op_gqa_attention (kernels.c:1418-1454) and of the
// batch entry (batch.c:128-137).  Caller holds ctx->lock.
int wr_decode_validate(wr_cuda_ctx *ctx, uint32_t n_sess, wr_cuda_kv *const *kv, uint32_t layer,
                       const uint32_t *seq_lens, const void *q, const void *out, uint32_t n_q,
                       int mem, int emit_triples)
{
    int rc = wr_kv_batch_check(ctx, n_sess, kv, layer);
    if (rc != WR_CUDA_OK) return rc;
    if (!seq_lens || !q || !out) return WR_CUDA_ERR_INVAL;
    if (mem != WR_CUDA_MEM_HOST && mem != WR_CUDA_MEM_DEVICE) return WR_CUDA_ERR_INVAL;
    if (mem == WR_CUDA_MEM_DEVICE && (((uintptr_t)q | (uintptr_t)out) & 15u))
        return WR_CUDA_ERR_INVAL;                                         // rows move as 16-byte vectors
    if (n_q == 0 || n_q % kv[0]->n_kv != 0) return WR_CUDA_ERR_INVAL;     // kernels.c:1429-1432
    for (uint32_t s = 0; s < n_sess; ++s) {
        if (seq_lens[s] == 0 && !emit_triples) return WR_CUDA_ERR_INVAL;  // kernels.c:1439
        if (seq_lens[s] > ctx->attn_max_seq) return WR_CUDA_ERR_LIMIT;    // kernels.c:1444
        if (seq_lens[s] > kv[s]->max_ctx) return WR_CUDA_ERR_INVAL;       // capacity, kernels.c:1449-1454
    }
    return WR_CUDA_OK;
}

// Work decomposition of one head_dim-128 decode launch: sessions sorted by
// descending length (their larger chunks are drawn from the work queue first,
// which evens out the finish), per-session chunking (a function of that
// session alone), item numbering.  Shared by every entry point that launches
// the kernel, so that they all give the same bits.  Fills everything of `p`
// that depends on the batch; the caller adds buffers, scale and flags.
void wr_decode_plan(uint32_t n_sess, wr_cuda_kv *const *kv, uint32_t layer, const uint32_t *seq_lens,
                    uint32_t n_q, uint32_t window, wr_decode::params &p, uint32_t &nt, uint32_t &items)
{
    using namespace wr_decode;
    const uint32_t n_kv = kv[0]->n_kv, hd = kv[0]->hd;
    const uint32_t group = n_q / n_kv;
    nt = group <= 4 ? 1u : 2u;
    const uint32_t qsubs = (group + 4 * nt - 1) / (4 * nt);
    uint32_t order[WR_CUDA_BATCH_MAX];
    for (uint32_t s = 0; s < n_sess; ++s) order[s] = s;
    std::stable_sort(order, order + n_sess,
                     [&](uint32_t a, uint32_t b) { return seq_lens[a] > seq_lens[b]; });
    items = 0;
    for (uint32_t i = 0; i < n_sess; ++i) {
        const uint32_t s = order[i];
        const uint32_t len = seq_lens[s];
        const uint32_t key_lo = (window > 0 && len > window) ? len - window : 0;  // kernels.c:1463
        const uint32_t n_tiles = (len + kTile - 1) / kTile;
        const uint32_t tile_lo = key_lo / kTile;
        const uint32_t span = n_tiles - tile_lo;
        const uint32_t ct = chunk_tiles_for(span, n_kv, qsubs); // chunk length: this session and the cache geometry alone
        const uint32_t nc = (span + ct - 1) / ct;              // 0 for an empty shard
        p.b.pages[i] = kv[s]->d_pages + (size_t)layer * kv[s]->n_pages;
        p.b.seq_len[i] = len;
        p.page_base[i] = kv[s]->contig[layer]
                             ? (const char *)kv[s]->pages[(size_t)layer * kv[s]->n_pages]
                             : nullptr;
        p.row[i] = s;
        p.key_lo[i] = key_lo;
        p.tile_lo[i] = tile_lo;
        p.n_tiles[i] = n_tiles;
        p.chunk_tiles[i] = ct;
        p.n_chunks[i] = nc;
        p.item_base[i] = items;
        items += n_kv * qsubs * nc;
    }
    for (uint32_t s = n_sess; s <= WR_CUDA_BATCH_MAX; ++s) p.item_base[s] = items;
    for (uint32_t i = n_sess; i < WR_CUDA_BATCH_MAX; ++i) p.page_base[i] = nullptr;
    p.page_bytes = wr_page_bytes(n_kv, hd);
    p.n_groups = n_sess * n_kv * qsubs;
    p.n_sess = n_sess;
    p.n_q = n_q;
    p.n_kv = n_kv;
    p.group = group;
    p.qsubs = qsubs;
}

// Enqueue the decode kernel on device-resident q / out.  Caller holds
// ctx->lock and has validated the arguments.
int wr_decode_launch(wr_cuda_ctx *ctx, uint32_t n_sess, wr_cuda_kv *const *kv, uint32_t layer,
                     const uint32_t *seq_lens, const float *dq, float *dout, uint32_t n_q,
                     float scale_override, uint32_t window, int emit_triples, wr_decode_xchg *xchg,
                     bool early_tiles)
{
    const uint32_t n_kv = kv[0]->n_kv, hd = kv[0]->hd;
    const uint32_t group = n_q / n_kv;
    const float scale = scale_for(hd, scale_override);

    if (hd == wr_decode::kHd) {
        using namespace wr_decode;
        params p;
        uint32_t nt = 1, items = 0;
        wr_decode_plan(n_sess, kv, layer, seq_lens, n_q, window, p, nt, items);
        int rc = wr_ctx_reserve_ws(ctx, (size_t)std::max(items, 1u) * 8 * kTripleStride * sizeof(float),
                                   (size_t)p.n_groups * kTicketsPerGroup + kTicketExtra);
        if (rc != WR_CUDA_OK) return rc;
        p.q = dq;
        p.out = dout;
        p.ws = ctx->ws;
        p.tickets = ctx->tickets;
        p.err = ctx->dev_err;
        p.wait_limit = ctx->wait_limit;
        p.emit_triples = (uint32_t)emit_triples;
        p.scale = scale;
        p.x_world = 0;
        p.x_step = 0;
        p.x_done = nullptr;
        p.x_recv = 0;
        p.x_max_rows = 0;
        p.x_rows_in = nullptr;
        p.x_row_flag_in = nullptr;
        if (xchg) {
            for (uint32_t w = 0; w < xchg->world; ++w) {
                p.x_rows[w] = xchg->rows[w];
                p.x_flag[w] = xchg->flag[w];
                p.x_row_flag[w] = xchg->row_flag[w];
            }
            p.x_done = xchg->done;
            p.x_world = xchg->world;
            p.x_step = xchg->step;
            p.x_max_rows = xchg->max_rows;
            p.x_rows_in = xchg->rows_in;
            p.x_row_flag_in = xchg->row_flag_in;
            // The merge warps can take the other ranks' rows and finish the output themselves when
            // every row of this rank goes through them, i.e. every session has at least two chunks.
            bool all_merged = xchg->want_recv;
            for (uint32_t s = 0; s < n_sess; ++s)
                if (p.n_chunks[s] < 2) all_merged = false;
            p.x_recv = all_merged ? 1u : 0u;
            xchg->did_recv = all_merged;
        }
        if (!(ctx->attr_flags & 1u)) {
            WR_CUDA_TRY(cudaFuncSetAttribute(attn_decode_hd128_kernel<1>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)sizeof(smem_layout)));
            WR_CUDA_TRY(cudaFuncSetAttribute(attn_decode_hd128_kernel<2>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)sizeof(smem_layout)));
            ctx->attr_flags |= 1u;
        }
        const uint32_t grid = std::max(1u, std::min<uint32_t>(items, (uint32_t)ctx->sm_count));
        // A grid that covers every SM (one CTA each: the kernel takes the whole register file) can
        // only start on an SM when the CTA before it there has exited, i.e. has passed its own wait;
        // that is what makes the early first-tile loads safe, so they need the full grid.
        const bool full = grid == (uint32_t)ctx->sm_count;
        p.early_tiles = (early_tiles && full) ? 1u : 0u;
        ctx->pdl_kind = full ? WR_PDL_DECODE_FULL : WR_PDL_DECODE_PART;
        ctx->pdl_index = ctx->launches + 1;
        if (nt == 1)
            WR_CUDA_TRY(wr_launch_pdl(attn_decode_hd128_kernel<1>, dim3(grid), dim3(kThreads), sizeof(smem_layout),
                                      ctx->stream, p));
        else
            WR_CUDA_TRY(wr_launch_pdl(attn_decode_hd128_kernel<2>, dim3(grid), dim3(kThreads), sizeof(smem_layout),
                                      ctx->stream, p));
    } else {
        generic_params p;
        for (uint32_t s = 0; s < n_sess; ++s) {
            const uint32_t len = seq_lens[s];
            p.b.pages[s] = kv[s]->d_pages + (size_t)layer * kv[s]->n_pages;
            p.b.seq_len[s] = len;
            p.key_lo[s] = (window > 0 && len > window) ? len - window : 0;
        }
        p.q = dq;
        p.out = dout;
        p.n_sess = n_sess;
        p.n_q = n_q;
        p.n_kv = n_kv;
        p.group = group;
        p.hd = hd;
        p.emit_triples = (uint32_t)emit_triples;
        p.scale = scale;
        const size_t smem = (size_t)(kGenWarps * hd + 2 * kGenWarps) * sizeof(float);
        attn_decode_generic_kernel<<<n_sess * n_q, kGenWarps * 32, smem, ctx->stream>>>(p);
    }
    ctx->launches++;
    WR_CUDA_TRY(cudaGetLastError());
    return WR_CUDA_OK;
}

static int decode_common(wr_cuda_ctx *ctx, uint32_t n_sess, wr_cuda_kv *const *kv, uint32_t layer,
                         const uint32_t *seq_lens, const float *q, float *out, uint32_t n_q,
                         float scale_override, uint32_t window, int mem, int emit_triples)
{
    if (!ctx) return WR_CUDA_ERR_INVAL;
    std::lock_guard<std::mutex> g(ctx->lock);
    int rc = wr_decode_validate(ctx, n_sess, kv, layer, seq_lens, q, out, n_q, mem, emit_triples);
    if (rc != WR_CUDA_OK) return rc;
    WR_CUDA_TRY(cudaSetDevice(ctx->device));
    const uint32_t hd = kv[0]->hd;
    const size_t q_bytes = (size_t)n_sess * n_q * hd * sizeof(float);
    const size_t out_row = emit_triples ? (WR_CUDA_TRIPLE_PAD + hd) : hd;
    const size_t out_bytes = (size_t)n_sess * n_q * out_row * sizeof(float);
    const float *dq = q;
    float *dout = out;
    if (mem == WR_CUDA_MEM_HOST) {
        rc = wr_ctx_reserve_stage(ctx, q_bytes + out_bytes, 0);
        if (rc != WR_CUDA_OK) return rc;
        dq = (const float *)ctx->stage_dev;
        dout = (float *)((char *)ctx->stage_dev + q_bytes);
        WR_CUDA_TRY(cudaMemcpyAsync((void *)dq, q, q_bytes, cudaMemcpyHostToDevice, ctx->stream));
    }
    // Back-to-back decode launches (nothing of this library's in between, so no page is being
    // written): the second one may request its first tiles while the first one drains.
    const bool early = mem == WR_CUDA_MEM_DEVICE && ctx->pdl_index == ctx->launches &&
                       ctx->pdl_kind == WR_PDL_DECODE_FULL;
    rc = wr_decode_launch(ctx, n_sess, kv, layer, seq_lens, dq, dout, n_q, scale_override, window,
                          emit_triples, nullptr, early);
    if (rc != WR_CUDA_OK) return rc;
    if (mem == WR_CUDA_MEM_HOST) {
        WR_CUDA_TRY(cudaMemcpyAsync(out, dout, out_bytes, cudaMemcpyDeviceToHost, ctx->stream));
        return wr_ctx_sync_checked(ctx);
    }
    return WR_CUDA_OK;
}

// One whole decode layer-step for a batch: append the new K/V rows (RoPE on
// K and Q), then attend over rows [0, positions[s]] of every session.  With
// host buffers the inputs cross the bus once and only the attention rows come
// back.
extern "C" int wr_cuda_decode_step(wr_cuda_ctx *ctx, uint32_t n_sess, wr_cuda_kv *const *kv,
                                   uint32_t layer, const uint32_t *positions, float *q,
                                   const float *k_rows, const float *v_rows, float *out,
                                   uint32_t n_q_heads, float theta_base, uint32_t n_rot_pairs,
                                   uint32_t flags, float scale_override, uint32_t window, int mem)
{
    if (!ctx) return WR_CUDA_ERR_INVAL;
    int rc = wr_append_validate(ctx, n_sess, kv, layer, positions, 1, k_rows, v_rows, q, n_q_heads,
                                mem);
    if (rc != WR_CUDA_OK) return rc;
    uint32_t seq_lens[WR_CUDA_BATCH_MAX];
    for (uint32_t s = 0; s < n_sess; ++s) seq_lens[s] = positions[s] + 1;
    std::lock_guard<std::mutex> g(ctx->lock);
    rc = wr_decode_validate(ctx, n_sess, kv, layer, seq_lens, q, out, n_q_heads, mem, 0);
    if (rc != WR_CUDA_OK) return rc;
    WR_CUDA_TRY(cudaSetDevice(ctx->device));
    const uint32_t hd = kv[0]->hd, n_kv = kv[0]->n_kv;
    const size_t kv_bytes = (size_t)n_sess * n_kv * hd * sizeof(float);
    const size_t q_bytes = (size_t)n_sess * n_q_heads * hd * sizeof(float);
    const float *dk = k_rows, *dv = v_rows, *dq_in = nullptr;
    float *dq = q, *dout = out;
    bool staged_out = false;
    if (mem == WR_CUDA_MEM_HOST) {
        // Page-locked host buffers (cudaHostAlloc / cudaHostRegister) are read and
        // written by the kernels themselves: the K/V/Q rows cross the bus as the
        // append kernel's loads and the attention rows as the decode kernel's
        // stores, with no copy operations in the stream.  Q is rotated into a
        // device buffer (the decode kernel reads it many times); the host's Q
        // rows stay as they are.  Pageable buffers take the staged path.
        const void *dev_k = wr_host_device_alias(k_rows), *dev_v = wr_host_device_alias(v_rows);
        const void *dev_q = wr_host_device_alias(q), *dev_o = wr_host_device_alias(out);
        // (rows move as 16-byte vectors: a page-locked buffer at an odd offset is staged instead)
        const bool aligned = ((((uintptr_t)dev_k | (uintptr_t)dev_v | (uintptr_t)dev_q | (uintptr_t)dev_o) & 15u) == 0);
        const bool zero_copy = dev_k && dev_v && dev_q && dev_o && aligned && (flags & WR_CUDA_APPEND_ROPE);
        rc = wr_ctx_reserve_stage(ctx, 2 * kv_bytes + 2 * q_bytes, 0);
        if (rc != WR_CUDA_OK) return rc;
        char *d = (char *)ctx->stage_dev;
        dq = (float *)(d + 2 * kv_bytes);
        if (zero_copy) {
            dk = (const float *)dev_k;
            dv = (const float *)dev_v;
            dq_in = (const float *)dev_q;
            dout = (float *)dev_o;
        } else {
            dk = (const float *)d;
            dv = (const float *)(d + kv_bytes);
            dout = (float *)(d + 2 * kv_bytes + q_bytes);
            staged_out = true;
            WR_CUDA_TRY(cudaMemcpyAsync((void *)dk, k_rows, kv_bytes, cudaMemcpyHostToDevice, ctx->stream));
            WR_CUDA_TRY(cudaMemcpyAsync((void *)dv, v_rows, kv_bytes, cudaMemcpyHostToDevice, ctx->stream));
            WR_CUDA_TRY(cudaMemcpyAsync(dq, q, q_bytes, cudaMemcpyHostToDevice, ctx->stream));
        }
    }
    // Early first-tile loads in the decode kernel: the append below writes one row per session, into
    // the session's last page, which those loads skip.  Every other page must be settled when the
    // decode kernel's CTAs can start: true when the kernel before the append is not one of this
    // library's early-starting kernels, or is a decode launch that covered every SM.
    const int prev = (ctx->pdl_index == ctx->launches) ? ctx->pdl_kind : WR_PDL_NONE;
    const bool early = prev == WR_PDL_NONE || prev == WR_PDL_DECODE_FULL;
    rc = wr_append_launch(ctx, n_sess, kv, layer, positions, 1, dk, dv, dq, n_q_heads, theta_base,
                          n_rot_pairs, flags, dq_in);
    if (rc != WR_CUDA_OK) return rc;
    rc = wr_decode_launch(ctx, n_sess, kv, layer, seq_lens, dq, dout, n_q_heads, scale_override,
                          window, 0, nullptr, early);
    if (rc != WR_CUDA_OK) return rc;
    if (mem == WR_CUDA_MEM_HOST) {
        if (staged_out)
            WR_CUDA_TRY(cudaMemcpyAsync(out, dout, q_bytes, cudaMemcpyDeviceToHost, ctx->stream));
        return wr_ctx_sync_checked(ctx);
    }
    return WR_CUDA_OK;
}

extern "C" int wr_cuda_attn_decode(wr_cuda_ctx *ctx, uint32_t n_sess, wr_cuda_kv *const *kv,
                                   uint32_t layer, const uint32_t *seq_lens, const float *q,
                                   float *out, uint32_t n_q_heads, float scale_override,
                                   uint32_t window, int mem)
{
    return decode_common(ctx, n_sess, kv, layer, seq_lens, q, out, n_q_heads, scale_override,
                         window, mem, 0);
}

extern "C" int wr_cuda_attn_decode_partial(wr_cuda_ctx *ctx, uint32_t n_sess,
                                           wr_cuda_kv *const *kv, uint32_t layer,
                                           const uint32_t *seq_lens, const float *q,
                                           float *triples, uint32_t n_q_heads,
                                           float scale_override, int mem)
{
    return decode_common(ctx, n_sess, kv, layer, seq_lens, q, triples, n_q_heads, scale_override,
                         0, mem, 1);
}

extern "C" int wr_cuda_attn_combine(wr_cuda_ctx *ctx, uint32_t n_shards, uint32_t n_rows,
                                    uint32_t head_dim, const float *triples, float *out, int mem)
{
    if (!ctx || !triples || !out || n_shards == 0 || n_rows == 0 || head_dim == 0)
        return WR_CUDA_ERR_INVAL;
    if (head_dim > WR_CUDA_HEAD_DIM_MAX) return WR_CUDA_ERR_LIMIT;
    if (mem != WR_CUDA_MEM_HOST && mem != WR_CUDA_MEM_DEVICE) return WR_CUDA_ERR_INVAL;
    std::lock_guard<std::mutex> g(ctx->lock);
    WR_CUDA_TRY(cudaSetDevice(ctx->device));
    const size_t in_bytes = (size_t)n_shards * n_rows * (WR_CUDA_TRIPLE_PAD + head_dim) * sizeof(float);
    const size_t out_bytes = (size_t)n_rows * head_dim * sizeof(float);
    const float *din = triples;
    float *dout = out;
    if (mem == WR_CUDA_MEM_HOST) {
        int rc = wr_ctx_reserve_stage(ctx, in_bytes + out_bytes, 0);
        if (rc != WR_CUDA_OK) return rc;
        din = (const float *)ctx->stage_dev;
        dout = (float *)((char *)ctx->stage_dev + in_bytes);
        WR_CUDA_TRY(cudaMemcpyAsync((void *)din, triples, in_bytes, cudaMemcpyHostToDevice, ctx->stream));
    }
    const uint64_t total = (uint64_t)n_rows * head_dim;
    const uint32_t blocks = (uint32_t)std::min<uint64_t>((total + 255) / 256, (uint64_t)ctx->sm_count * 8);
    attn_combine_kernel<<<blocks, 256, 0, ctx->stream>>>(din, dout, n_shards, n_rows, head_dim);
    ctx->launches++;
    WR_CUDA_TRY(cudaGetLastError());
    if (mem == WR_CUDA_MEM_HOST) {
        WR_CUDA_TRY(cudaMemcpyAsync(out, dout, out_bytes, cudaMemcpyDeviceToHost, ctx->stream));
        return wr_ctx_sync_checked(ctx);
    }
    return WR_CUDA_OK;
}
