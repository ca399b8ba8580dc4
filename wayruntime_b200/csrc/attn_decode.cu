// attn_decode.cu — batched split-KV decode attention over the paged F16 cache.
//
// Restates wri_op_gqa_attention for seq_q = 1 (src/core/kernels.c:1414-1527)
// as called once per session by the decode body (src/core/session.c:490-496)
// and, for a batch, once per session by src/core/batch.c:152-164 — here all
// sessions run in ONE grid.
//
// Shape of the kernel (head_dim 128):
//   * work item = (session, kv head, q-head subgroup of <= 8, chunk of keys);
//     the chunk length depends only on that session's length, never on the
//     rest of the batch, so a session's bits do not depend on its batch mates;
//   * persistent CTAs (2 per SM) walk items round-robin.  One producer thread
//     streams 32 KB K|V tiles (64 keys of one kv head, contiguous in the page)
//     into a 3-stage shared-memory ring with TMA bulk copies completing on
//     mbarriers; the ring keeps filling across item boundaries;
//   * four consumer warps each take 16 keys of every tile.  All q heads of the
//     GQA group share the tile: they are the rows of a 16-row tensor-core
//     tile, each head twice — rows 0..7 carry the F16 high part of the F32
//     query (pre-multiplied by the scale), rows 8..15 the F16 low part — so
//     scores keep F32-level query precision.  Probabilities are split the
//     same way for P*V.  Accumulation is F32;
//   * each warp keeps its own online-softmax state (m, l, O); warps merge
//     through shared memory per item; chunks merge through a global scratch
//     buffer, the last CTA of a group (arrival ticket) doing the merge in
//     chunk order, so the result is deterministic.
//   Memory-bound by design: K and V are read once from HBM per decode step.
#include <algorithm>

#include "wr_internal.cuh"

namespace {

constexpr int kHd = 128;
constexpr int kTile = 64;
constexpr int kStages = 3;
constexpr int kConsWarps = 4;
constexpr int kConsThreads = kConsWarps * 32;
constexpr int kThreads = kConsThreads + 32;
constexpr uint32_t kBlockBytes = kTile * kHd * 2;      // one K or V tile of one head
constexpr uint32_t kStageBytes = 2 * kBlockBytes;      // K then V, adjacent in the page
constexpr int kTripleStride = WR_CUDA_TRIPLE_PAD + kHd;  // m, l, 0, 0, o[128]
constexpr int kMrgStride = kHd + 8;                    // padded row of the warp-merge buffer
constexpr int kMaxChunks = 16;

struct decode_params {
    wr_batch_desc b;
    uint32_t key_lo[WR_CUDA_BATCH_MAX];
    uint32_t tile_lo[WR_CUDA_BATCH_MAX];
    uint32_t n_tiles[WR_CUDA_BATCH_MAX];
    uint32_t chunk_tiles[WR_CUDA_BATCH_MAX];
    uint32_t n_chunks[WR_CUDA_BATCH_MAX];
    uint32_t item_base[WR_CUDA_BATCH_MAX + 1];
    const float *q;
    float *out;        // [n_sess, n_q, hd] rows, or triples when emit_triples
    float *ws;         // per-item partial triples
    int *tickets;
    int *err;
    uint32_t n_sess, n_q, n_kv, group, qsubs, emit_triples;
    float scale;
};

struct item_t {
    uint32_t s, h, qs, c, t_begin, t_end;
};

__device__ __forceinline__ item_t decode_item(const decode_params &p, uint32_t it)
{
    item_t r;
    uint32_t s = 0;
    while (s + 1 < p.n_sess && it >= p.item_base[s + 1]) ++s;
    uint32_t local = it - p.item_base[s];
    uint32_t nc = p.n_chunks[s];
    r.s = s;
    r.c = local % nc;
    uint32_t gq = local / nc;
    r.qs = gq % p.qsubs;
    r.h = gq / p.qsubs;
    r.t_begin = p.tile_lo[s] + r.c * p.chunk_tiles[s];
    r.t_end = min(r.t_begin + p.chunk_tiles[s], p.n_tiles[s]);
    return r;
}

struct smem_layout {
    alignas(1024) uint8_t stage[kStages][kStageBytes];
    float mrg_o[kConsWarps][8][kMrgStride];
    float mrg_m[kConsWarps][8];
    float mrg_l[kConsWarps][8];
    alignas(8) uint64_t full[kStages];
    uint64_t empty[kStages];
    int last_flag;
    int abort_flag;
};

__device__ __forceinline__ void cons_bar()
{
    asm volatile("bar.sync 1, %0;" ::"n"(kConsThreads) : "memory");
}

__global__ void __launch_bounds__(kThreads, 2) attn_decode_hd128_kernel(const decode_params p)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    smem_layout &sm = *reinterpret_cast<smem_layout *>(smem_raw);
    const uint32_t tid = threadIdx.x;
    const uint32_t warp = tid >> 5, lane = tid & 31;
    const uint32_t n_items = p.item_base[p.n_sess];

    if (tid == 0) {
        for (int i = 0; i < kStages; ++i) {
            mbar_init(&sm.full[i], 1);
            mbar_init(&sm.empty[i], kConsWarps);
        }
        sm.abort_flag = 0;
        sm.last_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();

    if (warp == kConsWarps) {
        // ------------------------------------------------------- producer
        if (lane == 0) {
            uint32_t fill = 0;
            bool ok = true;
            for (uint32_t it = blockIdx.x; it < n_items && ok; it += gridDim.x) {
                const item_t w = decode_item(p, it);
                const uint64_t *pages = p.b.pages[w.s];
                for (uint32_t t = w.t_begin; t < w.t_end; ++t, ++fill) {
                    const uint32_t st = fill % kStages;
                    if (fill >= kStages && !mbar_wait(&sm.empty[st], ((fill / kStages) - 1) & 1)) {
                        ok = false;
                        break;
                    }
                    const char *src = (const char *)pages[t] + wr_block_off(w.h, 0, kHd);
                    mbar_expect_tx(&sm.full[st], kStageBytes);
                    bulk_g2s(sm.stage[st], src, kStageBytes, &sm.full[st]);
                }
            }
            if (!ok) {
                atomicExch(p.err, 1);
                // Copies already issued still land in this CTA's shared
                // memory: wait (bounded) for them before leaving.
                const uint32_t first = fill > kStages ? fill - kStages : 0;
                for (uint32_t f = first; f < fill; ++f)
                    (void)mbar_wait(&sm.full[f % kStages], (f / kStages) & 1);
            }
        }
        return;
    }

    // ----------------------------------------------------------- consumers
    const uint32_t r = lane >> 2;    // row of the 16x8 accumulator tile = q head slot
    const uint32_t tq = lane & 3;
    uint32_t cons = 0;

    for (uint32_t it = blockIdx.x; it < n_items; it += gridDim.x) {
        const item_t w = decode_item(p, it);
        const uint32_t seq_len = p.b.seq_len[w.s];
        const uint32_t key_lo = p.key_lo[w.s];
        const uint32_t heads_here = min(8u, p.group - w.qs * 8u);
        const uint32_t qh = w.h * p.group + w.qs * 8u + r;   // valid when r < heads_here

        // Query fragments: A operand rows r (high part) and r+8 (low part).
        uint32_t qa[kHd / 16][4];
        {
            const float *qrow = p.q + ((size_t)w.s * p.n_q + qh) * kHd;
            const bool live = r < heads_here;
#pragma unroll
            for (int ks = 0; ks < kHd / 16; ++ks) {
                float2 x = make_float2(0.f, 0.f), y = make_float2(0.f, 0.f);
                if (live) {
                    x = *reinterpret_cast<const float2 *>(qrow + ks * 16 + 2 * tq);
                    y = *reinterpret_cast<const float2 *>(qrow + ks * 16 + 8 + 2 * tq);
                }
                split_half2(x.x * p.scale, x.y * p.scale, qa[ks][0], qa[ks][1]);
                split_half2(y.x * p.scale, y.y * p.scale, qa[ks][2], qa[ks][3]);
            }
        }

        float m = WR_NEG_SENTINEL, l = 0.f;
        float oacc[kHd / 8][4];
#pragma unroll
        for (int i = 0; i < kHd / 8; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;

        for (uint32_t t = w.t_begin; t < w.t_end; ++t, ++cons) {
            const uint32_t st = cons % kStages;
            if (!mbar_wait(&sm.full[st], (cons / kStages) & 1)) {
                atomicExch(p.err, 2);
                return;
            }
            const uint32_t kbase = smem_u32(sm.stage[st]);
            const uint32_t vbase = kbase + kBlockBytes;
            const uint32_t key0 = t * kTile + warp * 16;     // first key of this warp's slice
            const bool need_mask = (key0 + 16 > seq_len) || (key0 < key_lo);

            if (key0 + 16 > seq_len) {
                // Rows past the session's length were never written for this
                // position (or belong to a rolled-back step): clear this
                // warp's V rows so that 0 * garbage cannot make a NaN.
                for (uint32_t i = lane; i < 16 * 16; i += 32) {
                    uint32_t krow = warp * 16 + (i >> 4), ch = i & 15;
                    if (t * kTile + krow >= seq_len)
                        *reinterpret_cast<uint4 *>(sm.stage[st] + kBlockBytes + (ch >> 3) * 8192 +
                                                   krow * 128 + (ch & 7) * 16) = make_uint4(0, 0, 0, 0);
                }
                fence_proxy_async();
                __syncwarp();
            }

            // ---- S = (Q*scale) K^T for 16 keys: two 16x8 tiles
            float sacc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            {
                const uint32_t mi = lane >> 3;
                const uint32_t krow = warp * 16 + (mi >> 1) * 8 + (lane & 7);
                const uint32_t rowaddr = kbase + krow * 128;
                const uint32_t sw = krow & 7;
#pragma unroll
                for (int ks = 0; ks < kHd / 16; ++ks) {
                    const uint32_t chunk = ((ks & 3) * 2 + (mi & 1)) ^ sw;
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4(b0, b1, b2, b3, rowaddr + (ks >> 2) * 8192 + chunk * 16);
                    mma_16816(sacc[0], qa[ks], b0, b1);
                    mma_16816(sacc[1], qa[ks], b2, b3);
                }
            }
            float sc[2][2];
            sc[0][0] = sacc[0][0] + sacc[0][2];
            sc[0][1] = sacc[0][1] + sacc[0][3];
            sc[1][0] = sacc[1][0] + sacc[1][2];
            sc[1][1] = sacc[1][1] + sacc[1][3];

            bool live[2][2] = {{true, true}, {true, true}};
            if (need_mask) {
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        uint32_t key = key0 + nt * 8 + 2 * tq + c;
                        live[nt][c] = key < seq_len && key >= key_lo;
                    }
            }
            float tmax = WR_NEG_SENTINEL;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int c = 0; c < 2; ++c)
                    if (live[nt][c]) tmax = fmaxf(tmax, sc[nt][c]);
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
            const float m_new = fmaxf(m, tmax);
            const float a = (m == WR_NEG_SENTINEL) ? 0.f : __expf(m - m_new);
            float pr[2][2];
            float psum = 0.f;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    pr[nt][c] = live[nt][c] ? __expf(sc[nt][c] - m_new) : 0.f;
                    psum += pr[nt][c];
                }
            l = l * a + psum;
            m = m_new;
#pragma unroll
            for (int i = 0; i < kHd / 8; ++i) {
                oacc[i][0] *= a; oacc[i][1] *= a; oacc[i][2] *= a; oacc[i][3] *= a;
            }

            // ---- O += P V : P rows r (high) / r+8 (low), k = this warp's 16 keys
            uint32_t pa[4];
            split_half2(pr[0][0], pr[0][1], pa[0], pa[1]);
            split_half2(pr[1][0], pr[1][1], pa[2], pa[3]);
            {
                const uint32_t mi = lane >> 3;
                const uint32_t krow = warp * 16 + (mi & 1) * 8 + (lane & 7);
                const uint32_t rowaddr = vbase + krow * 128;
                const uint32_t sw = krow & 7;
#pragma unroll
                for (int nd = 0; nd < kHd / 8; nd += 2) {
                    const uint32_t c16 = nd + (mi >> 1);
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(b0, b1, b2, b3,
                                      rowaddr + (c16 >> 3) * 8192 + (((c16 & 7) ^ sw) * 16));
                    mma_16816(oacc[nd], pa, b0, b1);
                    mma_16816(oacc[nd + 1], pa, b2, b3);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.empty[st]);
        }

        // ---- merge the four warps' states for this item
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        if (tq == 0) {
            sm.mrg_m[warp][r] = m;
            sm.mrg_l[warp][r] = l;
        }
#pragma unroll
        for (int nd = 0; nd < kHd / 8; ++nd)
            *reinterpret_cast<float2 *>(&sm.mrg_o[warp][r][nd * 8 + 2 * tq]) =
                make_float2(oacc[nd][0] + oacc[nd][2], oacc[nd][1] + oacc[nd][3]);
        cons_bar();

        const uint32_t nc = p.n_chunks[w.s];
        const bool direct = (nc == 1);
        const uint32_t d = tid;   // 0..127
        for (uint32_t rr = 0; rr < heads_here; ++rr) {
            float mstar = WR_NEG_SENTINEL;
#pragma unroll
            for (int wv = 0; wv < kConsWarps; ++wv) mstar = fmaxf(mstar, sm.mrg_m[wv][rr]);
            float L = 0.f, acc = 0.f;
#pragma unroll
            for (int wv = 0; wv < kConsWarps; ++wv) {
                const float mw = sm.mrg_m[wv][rr];
                const float wgt = (mw == WR_NEG_SENTINEL) ? 0.f : __expf(mw - mstar);
                L += wgt * sm.mrg_l[wv][rr];
                acc += wgt * sm.mrg_o[wv][rr][d];
            }
            const uint32_t head = w.h * p.group + w.qs * 8u + rr;
            const size_t row = (size_t)w.s * p.n_q + head;
            if (direct && !p.emit_triples) {
                p.out[row * kHd + d] = (L > 0.f) ? acc / L : 0.f;
            } else {
                float *tr = direct ? p.out + row * kTripleStride
                                   : p.ws + ((size_t)it * 8 + rr) * kTripleStride;
                tr[WR_CUDA_TRIPLE_PAD + d] = acc;
                if (d == 0) {
                    tr[0] = mstar; tr[1] = L; tr[2] = 0.f; tr[3] = 0.f;
                }
            }
        }

        if (!direct) {
            // Arrival ticket: the CTA that completes the group merges it.
            __threadfence();
            cons_bar();
            const uint32_t gidx = (w.s * p.n_kv + w.h) * p.qsubs + w.qs;
            if (tid == 0) {
                int prev = atomicAdd(&p.tickets[gidx], 1);
                sm.last_flag = (prev == (int)nc - 1);
            }
            cons_bar();
            if (sm.last_flag) {
                __threadfence();
                const size_t first_item = (size_t)it - w.c;
                for (uint32_t rr = 0; rr < heads_here; ++rr) {
                    float mstar = WR_NEG_SENTINEL;
                    for (uint32_t c = 0; c < nc; ++c)
                        mstar = fmaxf(mstar, __ldcg(p.ws + ((first_item + c) * 8 + rr) * kTripleStride));
                    float L = 0.f, acc = 0.f;
                    for (uint32_t c = 0; c < nc; ++c) {
                        const float *tr = p.ws + ((first_item + c) * 8 + rr) * kTripleStride;
                        const float mc = __ldcg(tr);
                        const float wgt = (mc == WR_NEG_SENTINEL) ? 0.f : __expf(mc - mstar);
                        L += wgt * __ldcg(tr + 1);
                        acc += wgt * __ldcg(tr + WR_CUDA_TRIPLE_PAD + d);
                    }
                    const uint32_t head = w.h * p.group + w.qs * 8u + rr;
                    const size_t row = (size_t)w.s * p.n_q + head;
                    if (p.emit_triples) {
                        float *tr = p.out + row * kTripleStride;
                        tr[WR_CUDA_TRIPLE_PAD + d] = acc;
                        if (d == 0) {
                            tr[0] = mstar; tr[1] = L; tr[2] = 0.f; tr[3] = 0.f;
                        }
                    } else {
                        p.out[row * kHd + d] = (L > 0.f) ? acc / L : 0.f;
                    }
                }
                if (tid == 0) p.tickets[gidx] = 0;   // ready for the next launch
            }
        }
        cons_bar();   // merge buffers are free again
    }
}

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
    if (n_q == 0 || n_q % kv[0]->n_kv != 0) return WR_CUDA_ERR_INVAL;     // kernels.c:1429-1432
    for (uint32_t s = 0; s < n_sess; ++s) {
        if (seq_lens[s] == 0 && !emit_triples) return WR_CUDA_ERR_INVAL;  // kernels.c:1439
        if (seq_lens[s] > ctx->attn_max_seq) return WR_CUDA_ERR_LIMIT;    // kernels.c:1444
        if (seq_lens[s] > kv[s]->max_ctx) return WR_CUDA_ERR_INVAL;       // capacity, kernels.c:1449-1454
    }
    return WR_CUDA_OK;
}

// Enqueue the decode kernel on device-resident q / out.  Caller holds
// ctx->lock and has validated the arguments.
int wr_decode_launch(wr_cuda_ctx *ctx, uint32_t n_sess, wr_cuda_kv *const *kv, uint32_t layer,
                     const uint32_t *seq_lens, const float *dq, float *dout, uint32_t n_q,
                     float scale_override, uint32_t window, int emit_triples)
{
    int rc;
    const uint32_t n_kv = kv[0]->n_kv, hd = kv[0]->hd;
    const uint32_t group = n_q / n_kv;
    const float scale = scale_for(hd, scale_override);

    if (hd == kHd) {
        decode_params p;
        const uint32_t qsubs = (group + 7u) / 8u;
        uint32_t items = 0;
        for (uint32_t s = 0; s < n_sess; ++s) {
            const uint32_t len = seq_lens[s];
            const uint32_t key_lo = (window > 0 && len > window) ? len - window : 0;  // kernels.c:1463
            const uint32_t n_tiles = (len + kTile - 1) / kTile;
            const uint32_t tile_lo = key_lo / kTile;
            const uint32_t span = n_tiles - tile_lo;
            // Chunk length is a function of this session alone.
            uint32_t ct = (span + kMaxChunks - 1) / kMaxChunks;
            ct = std::max(4u, (ct + 3u) & ~3u);
            const uint32_t nc = std::max(1u, (span + ct - 1) / ct);
            p.b.pages[s] = kv[s]->d_pages + (size_t)layer * kv[s]->n_pages;
            p.b.seq_len[s] = len;
            p.key_lo[s] = key_lo;
            p.tile_lo[s] = tile_lo;
            p.n_tiles[s] = n_tiles;
            p.chunk_tiles[s] = ct;
            p.n_chunks[s] = nc;
            p.item_base[s] = items;
            items += n_kv * qsubs * nc;
        }
        p.item_base[n_sess] = items;
        for (uint32_t s = n_sess + 1; s <= WR_CUDA_BATCH_MAX; ++s) p.item_base[s] = items;
        rc = wr_ctx_reserve_ws(ctx, (size_t)items * 8 * kTripleStride * sizeof(float),
                               (size_t)n_sess * n_kv * qsubs);
        if (rc != WR_CUDA_OK) return rc;
        p.q = dq;
        p.out = dout;
        p.ws = ctx->ws;
        p.tickets = ctx->tickets;
        p.err = ctx->dev_err;
        p.n_sess = n_sess;
        p.n_q = n_q;
        p.n_kv = n_kv;
        p.group = group;
        p.qsubs = qsubs;
        p.emit_triples = (uint32_t)emit_triples;
        p.scale = scale;
        if (!(ctx->attr_flags & 1u)) {
            WR_CUDA_TRY(cudaFuncSetAttribute(attn_decode_hd128_kernel,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)sizeof(smem_layout)));
            ctx->attr_flags |= 1u;
        }
        const uint32_t grid = std::min<uint32_t>(items, (uint32_t)ctx->sm_count * 2u);
        attn_decode_hd128_kernel<<<grid, kThreads, sizeof(smem_layout), ctx->stream>>>(p);
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
    rc = wr_decode_launch(ctx, n_sess, kv, layer, seq_lens, dq, dout, n_q, scale_override, window,
                          emit_triples);
    if (rc != WR_CUDA_OK) return rc;
    if (mem == WR_CUDA_MEM_HOST) {
        WR_CUDA_TRY(cudaMemcpyAsync(out, dout, out_bytes, cudaMemcpyDeviceToHost, ctx->stream));
        WR_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
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
    const float *dk = k_rows, *dv = v_rows;
    float *dq = q, *dout = out;
    if (mem == WR_CUDA_MEM_HOST) {
        rc = wr_ctx_reserve_stage(ctx, 2 * kv_bytes + 2 * q_bytes, 0);
        if (rc != WR_CUDA_OK) return rc;
        char *d = (char *)ctx->stage_dev;
        dk = (const float *)d;
        dv = (const float *)(d + kv_bytes);
        dq = (float *)(d + 2 * kv_bytes);
        dout = (float *)(d + 2 * kv_bytes + q_bytes);
        WR_CUDA_TRY(cudaMemcpyAsync((void *)dk, k_rows, kv_bytes, cudaMemcpyHostToDevice, ctx->stream));
        WR_CUDA_TRY(cudaMemcpyAsync((void *)dv, v_rows, kv_bytes, cudaMemcpyHostToDevice, ctx->stream));
        WR_CUDA_TRY(cudaMemcpyAsync(dq, q, q_bytes, cudaMemcpyHostToDevice, ctx->stream));
    }
    rc = wr_append_launch(ctx, n_sess, kv, layer, positions, 1, dk, dv, dq, n_q_heads, theta_base,
                          n_rot_pairs, flags);
    if (rc != WR_CUDA_OK) return rc;
    rc = wr_decode_launch(ctx, n_sess, kv, layer, seq_lens, dq, dout, n_q_heads, scale_override,
                          window, 0);
    if (rc != WR_CUDA_OK) return rc;
    if (mem == WR_CUDA_MEM_HOST) {
        WR_CUDA_TRY(cudaMemcpyAsync(out, dout, q_bytes, cudaMemcpyDeviceToHost, ctx->stream));
        WR_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
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
        WR_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    }
    return WR_CUDA_OK;
}
