// attn_decode_hd128.cuh — the decode attention kernel for head_dim 128.
//
// Restates wri_op_gqa_attention for seq_q = 1 (src/core/kernels.c:1414-1527):
// scores = q.k * scale, online softmax with the -1e30 sentinel, o += p * v,
// out = o / l — for every session of a batch in ONE grid.
//
// Organisation
//   * work item = (session, kv head, q-head subgroup of <= 4*NT heads, chunk
//     of keys).  The chunk length is a function of that session's length
//     only, so a session's result does not depend on its batch mates.
//   * six warps of a CTA are self-contained engines: each owns a 16 KB K slot, a 16 KB
//     V slot and a Q slot in shared memory and refills them itself with TMA
//     bulk copies (one 16 KB copy per K or V tile: 64 keys of one kv head are
//     contiguous in the page and already in the swizzled order ldmatrix
//     wants).  While an engine computes Q.K on tile t the V of tile t is in
//     flight; while it computes P.V the K of tile t+1 is in flight — across
//     item boundaries too.  No CTA-wide barrier exists.
//   * items come from a global queue (the first one is static); an engine
//     draws the index of a future item one item ahead and loads the page
//     pointer of a future tile one tile ahead, so neither latency is exposed.
//     Which engine runs an item has no effect on the item's result.
//   * tensor-core tiles are transposed so that nothing is wasted on the tiny
//     head count: S^T[key, slot] = K[key, :] . Q^T[:, slot] puts 16 keys on the
//     M side and the q heads on the 8-wide N side, each head twice — slot 2h
//     carries the F16 high part of the (scaled) F32 query, slot 2h+1 the F16
//     low part, so scores keep F32-level query precision.  Probabilities are
//     split the same way (movmatrix transposes them into the B operand) and
//     O^T[dim, slot] += V^T[dim, key] . P^T[key, slot].  Accumulation is F32.
//   * chunks of one (session, kv head, subgroup) are merged in chunk order
//     (deterministic) once the last of them has arrived.  The engines only
//     count arrivals (a fire-and-forget release increment); the merging — L2
//     round trips during which a stream would stand still — is done by two
//     more warps per CTA: merge warp w of the grid owns the (group, head
//     pair) jobs w, w + W, ...; it waits for the job's arrival count and
//     fetches all its rows in one round trip.  While they wait they keep
//     running the merge code on nothing, so that its instructions are still
//     cached when the last groups — the end of the kernel's critical path —
//     arrive.
//   The kernel is HBM-bound by design: K and V are read exactly once.
#pragma once

#include "wr_internal.cuh"

namespace wr_decode {

constexpr int kHd = 128;
constexpr int kTile = 64;                              // keys per tile = tokens per page
constexpr int kWarps = 6;                              // engines per CTA
constexpr int kMergeWarps = 2;                         // per CTA, after the engines
constexpr int kThreads = (kWarps + kMergeWarps) * 32;
constexpr int kTicketsPerGroup = 4;                    // arrival counters reserved per group: one per head pair (<= 8 heads)
constexpr int kTicketExtra = 2;                        // after the tickets: work queue, engine exits
constexpr uint32_t kBlockBytes = kTile * kHd * 2;      // one K or V tile of one head
constexpr int kTripleStride = WR_CUDA_TRIPLE_PAD + kHd;  // m, l, 0, 0, o[128]
constexpr int kMaxChunks = 128;                        // per session (lane c of a merge warp holds chunks c, c+32, c+64, c+96)
constexpr int kChunkSlots = kMaxChunks / 32;
constexpr int kChunkBatch = 16;                        // chunk rows a merge keeps in flight per head
#ifndef WR_DECODE_MIN_CHUNK_TILES
#define WR_DECODE_MIN_CHUNK_TILES 2
#endif
#ifndef WR_DECODE_ITEMS_TARGET
#define WR_DECODE_ITEMS_TARGET 128
#endif
constexpr int kMinChunkTiles = WR_DECODE_MIN_CHUNK_TILES;
constexpr int kItemsPerSessionTarget = WR_DECODE_ITEMS_TARGET;   // work items one session should offer the engines

// Tiles per chunk: a function of the session's own span and of the cache
// geometry only — never of its batch mates (batch invariance).  A session
// is cut so that it offers about kItemsPerSessionTarget items (kv heads x
// q subgroups x chunks): with eight kv heads that is 16 chunks, with one kv
// head (a KV-head-sharded cache) up to 128, so that a small batch still
// reaches every engine of the machine.  Sessions longer than 64 tiles use at
// least 32 chunks, which keeps items short enough to balance a few long
// sessions.  A chunk is never shorter than kMinChunkTiles.
__host__ __device__ inline uint32_t chunk_tiles_for(uint32_t span_tiles, uint32_t n_kv, uint32_t qsubs)
{
    const uint32_t per_chunk = n_kv * qsubs;
    uint32_t max_chunks = ((uint32_t)kItemsPerSessionTarget + per_chunk - 1) / per_chunk;
    if (max_chunks < 16u) max_chunks = 16u;
    if (span_tiles > 64u && max_chunks < 32u) max_chunks = 32u;
    if (max_chunks > (uint32_t)kMaxChunks) max_chunks = (uint32_t)kMaxChunks;
    const uint32_t ct = (span_tiles + max_chunks - 1) / max_chunks;
    return ct < (uint32_t)kMinChunkTiles ? (uint32_t)kMinChunkTiles : ct;
}

// Sessions appear here sorted by descending length (longest chunks are drawn
// first); row[i] is the caller's index of entry i.
struct params {
    wr_batch_desc b;
    uint32_t row[WR_CUDA_BATCH_MAX];
    uint32_t key_lo[WR_CUDA_BATCH_MAX];
    uint32_t tile_lo[WR_CUDA_BATCH_MAX];
    uint32_t n_tiles[WR_CUDA_BATCH_MAX];
    uint32_t chunk_tiles[WR_CUDA_BATCH_MAX];
    uint32_t n_chunks[WR_CUDA_BATCH_MAX];      // 0 for a session with no keys (empty shard)
    uint32_t item_base[WR_CUDA_BATCH_MAX + 1];
    const char *page_base[WR_CUDA_BATCH_MAX];  // non-null: page t = page_base + t * page_bytes
    uint64_t page_bytes;
    const float *q;
    float *out;        // [n_sess, n_q, hd] rows, or triples when emit_triples
    float *ws;         // per-item partial triples, 8 rows each
    int *tickets;      // arrival counters [n_groups][kTicketsPerGroup], then the work queue and the engine exits
    int *err;
    uint32_t n_sess, n_q, n_kv, group, qsubs, emit_triples, n_groups;
    float scale;
    long long wait_limit;   // SM clock cycles a device-side wait may last
    // Key-sharded decode with the exchange fused in (x_world > 0): finished triples go
    // straight into every rank's exchange buffer, slot of this rank, instead of `out`.
    float *x_rows[WR_CUDA_XCHG_MAX_WORLD];       // per rank: this rank's row slot in that rank's buffer
    uint32_t *x_flag[WR_CUDA_XCHG_MAX_WORLD];    // per rank: this rank's step flag in that rank's buffer
    int *x_done;                                 // rows of this launch that have been stored everywhere
    uint32_t x_world, x_step;
    uint32_t *x_row_flag[WR_CUDA_XCHG_MAX_WORLD];// per rank: this rank's per-row flags in that rank's buffer
    const float *x_rows_in;                      // this rank's buffer: every rank's rows of this step, [world][max_rows][132]
    const uint32_t *x_row_flag_in;               // ... and their per-row flags, [world][max_rows]
    uint32_t x_max_rows;
    uint32_t x_recv;                             // merge warps also receive, merge across ranks and write `out` (final rows)
    // An engine may request its first K/V tile before the earlier kernels have completed, unless
    // that tile is the session's last page (where the row appended just before this launch lands).
    // Set by the host only where it knows that every other page is settled (wr_cuda_decode_step).
    uint32_t early_tiles;
};

// Stores of one finished warp's rows (row_first .. row_first + rows - 1) are done: flag each row on
// every rank, count them, and when every row of the launch has been stored on every rank, publish the
// step number to all ranks as well.
__device__ __forceinline__ void xchg_rows_done(const params &p, uint32_t row_first, uint32_t rows, uint32_t lane)
{
    __threadfence_system();                      // this lane's peer stores are ordered before the flags and the count
    __syncwarp();
    // per-row flags, for receivers that take rows one by one (relaxed stores after the fence above)
    for (uint32_t i = lane; i < rows * p.x_world; i += 32) {
        const uint32_t w = i % p.x_world, r = row_first + i / p.x_world;
        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p.x_row_flag[w] + r), "r"(p.x_step) : "memory");
    }
    if (lane == 0) {
        const uint32_t total = p.n_sess * p.n_q;
        if ((uint32_t)atomicAdd(p.x_done, (int)rows) + rows == total) {
            // One system-scope fence orders every counted row before the flags; the flag stores
            // themselves are relaxed and go out together (a release per flag would wait for the
            // round trip of the one before it: eight ranks, eight NVLink round trips in a row).
            __threadfence_system();
            for (uint32_t w = 0; w < p.x_world; ++w)
                asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p.x_flag[w]), "r"(p.x_step) : "memory");
            *p.x_done = 0;                       // ready for the next launch
        }
    }
}

}  // namespace wr_decode

// Host side (attn_decode.cu): the batch-dependent part of `params`.
void wr_decode_plan(uint32_t n_sess, wr_cuda_kv *const *kv, uint32_t layer, const uint32_t *seq_lens,
                    uint32_t n_q, uint32_t window, wr_decode::params &p, uint32_t &nt, uint32_t &items);

namespace wr_decode {

struct warp_smem {
    alignas(128) uint8_t k[kBlockBytes];
    alignas(128) uint8_t v[kBlockBytes];
    alignas(128) float q[8][kHd];
};

struct smem_layout {
    warp_smem w[kWarps];
    alignas(8) uint64_t full_k[kWarps];
    uint64_t full_v[kWarps];
};

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a)
{
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ int atom_add_acq_rel(int *addr, int v)
{
    int old;
    asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], %2;" : "=r"(old) : "l"(addr), "r"(v) : "memory");
    return old;
}
__device__ __forceinline__ void red_add_release(int *addr, int v)
{
    asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_relaxed(const int *addr)
{
    int v;
    asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void fence_acq_rel_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }
__device__ __forceinline__ int atom_add_relaxed(int *addr, int v)
{
    int old;
    asm volatile("atom.add.relaxed.gpu.global.s32 %0, [%1], %2;" : "=r"(old) : "l"(addr), "r"(v) : "memory");
    return old;
}

// Merge the nc partial triples of two heads (hs0, hs0 + 1) of one (session, kv
// head, subgroup), in chunk order, into their output rows.  Called by a whole
// warp.  This is the end of the kernel's critical path and pure L2 latency, so
// every load is issued before the first result is used: lane c holds (m, l) of
// chunk c, and all chunk rows of both heads are in flight at once.
__device__ __forceinline__ void merge_head_pair(const params &p, size_t row0, size_t first_item, uint32_t nc,
                                             uint32_t hs0, uint32_t heads_here, uint32_t lane, bool dry_run)
{
    // lane c holds (m, l) of chunks c, c + 32, c + 64, c + 96
    float mc[2][kChunkSlots], lc[2][kChunkSlots];
#pragma unroll
    for (uint32_t e = 0; e < 2; ++e) {
        const uint32_t hs = hs0 + e;
#pragma unroll
        for (int q = 0; q < kChunkSlots; ++q) {
            mc[e][q] = WR_NEG_SENTINEL;
            lc[e][q] = 0.f;
            const uint32_t c = q * 32 + lane;
            if (c < nc && hs < heads_here) {
                const float *tr = p.ws + ((first_item + c) * 8 + hs) * kTripleStride;
                mc[e][q] = __ldcg(tr);
                lc[e][q] = __ldcg(tr + 1);
            }
        }
    }
    float4 acc[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
    float mstar[2], wgt[2][kChunkSlots], L[2] = {0.f, 0.f};
    // chunk rows in batches of kChunkBatch (one batch unless the session is long)
#pragma unroll 1
    for (uint32_t c0 = 0; c0 == 0 || c0 < nc; c0 += kChunkBatch) {
        float4 ov[2][kChunkBatch];
#pragma unroll
        for (uint32_t e = 0; e < 2; ++e) {
            const uint32_t hs = hs0 + e;
#pragma unroll
            for (int j = 0; j < kChunkBatch; ++j)
                ov[e][j] = (c0 + j < nc && hs < heads_here)
                               ? __ldcg(reinterpret_cast<const float4 *>(
                                     p.ws + ((first_item + c0 + j) * 8 + hs) * kTripleStride + WR_CUDA_TRIPLE_PAD) + lane)
                               : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (c0 == 0) {
#pragma unroll
            for (uint32_t e = 0; e < 2; ++e) {
                float mx = mc[e][0];
#pragma unroll
                for (int q = 1; q < kChunkSlots; ++q) mx = fmaxf(mx, mc[e][q]);
#pragma unroll
                for (int off = 16; off > 0; off >>= 1)
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
                mstar[e] = mx;
#pragma unroll
                for (int q = 0; q < kChunkSlots; ++q)
                    wgt[e][q] = (mc[e][q] == WR_NEG_SENTINEL) ? 0.f : __expf(mc[e][q] - mx);
            }
        }
        const uint32_t slot = c0 >> 5;             // the whole batch lies in one group of 32 chunks
#pragma unroll
        for (uint32_t e = 0; e < 2; ++e) {
            float wsel = wgt[e][0], lsel = lc[e][0];
#pragma unroll
            for (int q = 1; q < kChunkSlots; ++q)
                if (slot == (uint32_t)q) { wsel = wgt[e][q]; lsel = lc[e][q]; }
            const float wl = wsel * lsel;
#pragma unroll
            for (int j = 0; j < kChunkBatch; ++j) {
                const float wj = __shfl_sync(0xffffffffu, wsel, (c0 + j) & 31);
                L[e] += __shfl_sync(0xffffffffu, wl, (c0 + j) & 31);
                acc[e].x += wj * ov[e][j].x; acc[e].y += wj * ov[e][j].y;
                acc[e].z += wj * ov[e][j].z; acc[e].w += wj * ov[e][j].w;
            }
        }
    }
#pragma unroll
    for (uint32_t e = 0; e < 2; ++e) {
        const uint32_t hs = hs0 + e;
        if (hs >= heads_here) break;
        float4 &a4 = acc[e];
        if (dry_run) continue;
        if (p.x_world > 0) {
            // the row goes to every rank at once (plain 16-byte stores over NVLink, this rank included)
            for (uint32_t w = 0; w < p.x_world; ++w) {
                float *tr = p.x_rows[w] + (row0 + hs) * kTripleStride;
                reinterpret_cast<float4 *>(tr + WR_CUDA_TRIPLE_PAD)[lane] = a4;
                if (lane == 0) *reinterpret_cast<float4 *>(tr) = make_float4(mstar[e], L[e], 0.f, 0.f);
            }
        } else if (p.emit_triples) {
            float *tr = p.out + (row0 + hs) * kTripleStride;
            reinterpret_cast<float4 *>(tr + WR_CUDA_TRIPLE_PAD)[lane] = a4;
            if (lane == 0) {
                tr[0] = mstar[e]; tr[1] = L[e]; tr[2] = 0.f; tr[3] = 0.f;
            }
        } else {
            const float inv = (L[e] > 0.f) ? 1.0f / L[e] : 0.f;
            a4.x *= inv; a4.y *= inv; a4.z *= inv; a4.w *= inv;
            reinterpret_cast<float4 *>(p.out + (row0 + hs) * kHd)[lane] = a4;
        }
    }
    if (p.x_world > 0 && !dry_run) {
        const uint32_t nrow = min(2u, heads_here - hs0), first = (uint32_t)row0 + hs0;
        xchg_rows_done(p, first, nrow, lane);
        if (p.x_recv) {
            // Take the same rows from every rank (bounded wait on their per-row flags in this rank's
            // buffer), merge in rank order and write the final rows: no second kernel.
            const long long t0 = clock64();
            for (;;) {
                bool mine = true;
                for (uint32_t i = lane; i < nrow * p.x_world; i += 32) {
                    const uint32_t g = i % p.x_world, r = first + i / p.x_world;
                    uint32_t seen;
                    asm volatile("ld.acquire.sys.global.u32 %0, [%1];"
                                 : "=r"(seen)
                                 : "l"(p.x_row_flag_in + (size_t)g * p.x_max_rows + r)
                                 : "memory");
                    mine = mine && (seen == p.x_step);
                }
                if (__all_sync(0xffffffffu, mine)) break;
                const bool late = clock64() - t0 > p.wait_limit;
                if (__any_sync(0xffffffffu, late)) {
                    if (lane == 0) atomicCAS(p.err, 0, 22);
                    return;
                }
            }
            __syncwarp();
            for (uint32_t e = 0; e < nrow; ++e) {
                const float4 r4 = wr_merge_ranks(p.x_rows_in, p.x_world, p.x_max_rows, kTripleStride, first + e, lane);
                reinterpret_cast<float4 *>(p.out + (size_t)(first + e) * kHd)[lane] = r4;
            }
        }
    }
}

// One tile of work, with everything the compute loop needs to know about it.
struct tile_desc {
    uint32_t it;          // item index (addresses the partial-triple scratch)
    uint32_t s, h, qs;    // sorted session slot, kv head, q-head subgroup
    uint32_t t;           // tile index = page index
    uint32_t flags;       // bit0 valid, bit1 first tile of item, bit2 last tile of item
    const char *page;
};

// Walks this engine's tiles in order, across items.
struct tile_stream {
    uint32_t it, s, h, qs, t, t_end;
    int pending;          // lane 0: the next item's index, drawn from the queue one item ago
    bool have;
};

template <int NT>
__global__ void __launch_bounds__(kThreads, 1) attn_decode_hd128_kernel(const params p)
{
    extern __shared__ __align__(128) uint8_t smem_raw[];
    smem_layout &sm = *reinterpret_cast<smem_layout *>(smem_raw);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t n_items = p.item_base[p.n_sess];
    const uint32_t n_engines = gridDim.x * kWarps;
    const uint32_t engine = warp * gridDim.x + blockIdx.x;   // neighbours in item order sit on different SMs
    warp_smem &ws = sm.w[warp];
    uint64_t *bar_k = &sm.full_k[warp], *bar_v = &sm.full_v[warp];
    int *queue = p.tickets + (size_t)p.n_groups * kTicketsPerGroup, *exits = queue + 1;
    constexpr uint32_t kHeadsMax = 4 * NT;
    const uint32_t g = lane >> 2, t4 = lane & 3;
    const uint64_t stream_policy = l2_policy_evict_first();
    // Let the next kernel in the stream be scheduled while this one runs (it waits for this one's
    // completion before it touches shared state); everything up to pdl_wait() below is this
    // kernel's own prologue, overlapped with the tail of the kernel before it.
    pdl_trigger();

    if (warp >= kWarps) {
        pdl_wait();                      // counters, scratch rows and `out` belong to earlier launches until now
        // ----------------------------------------------------------- merge warps
        // Jobs are (group, head pair) in group order, which is also roughly the
        // order in which groups complete; merge warp w of the grid takes jobs
        // w, w + W, ...  Each job has its own arrival counter.
        // While its group is incomplete the warp keeps running the merge code on
        // nothing (no memory access): the engines' loop would otherwise push that
        // code out of the instruction caches, and fetching it back costs several
        // microseconds exactly when the last groups arrive.
        constexpr uint32_t kPairs = kHeadsMax / 2;
        const uint32_t n_mergers = gridDim.x * kMergeWarps;
        const long long t_start = clock64();
        for (uint32_t job = (warp - kWarps) * gridDim.x + blockIdx.x; job < p.n_groups * kPairs; job += n_mergers) {
            const uint32_t gidx = job / kPairs, pair = job % kPairs;
            const uint32_t qs = gidx % p.qsubs, sh = gidx / p.qsubs;
            const uint32_t h = sh % p.n_kv, s = sh / p.n_kv;
            const uint32_t nc = p.n_chunks[s];
            const uint32_t heads = min(kHeadsMax, p.group - qs * kHeadsMax);
            if (nc <= 1 || 2 * pair >= heads) continue;          // written directly by its engine / no such heads
            const size_t row0 = (size_t)p.row[s] * p.n_q + h * p.group + qs * kHeadsMax;
            const size_t first_item = (size_t)p.item_base[s] + (size_t)(h * p.qsubs + qs) * nc;
            int *ticket = p.tickets + (size_t)gidx * kTicketsPerGroup + pair;
            for (;;) {
                int ready = 0;
                if (lane == 0) {
                    ready = ((uint32_t)ld_relaxed(ticket) == nc);
                    if (ready) fence_acq_rel_gpu();
                    else if (clock64() - t_start > 2 * p.wait_limit) {
                        atomicExch(p.err, 4);
                        ready = -1;
                    }
                }
                ready = __shfl_sync(0xffffffffu, ready, 0);
                if (ready < 0) return;
                merge_head_pair(p, row0, first_item, ready ? nc : 0u, 2 * pair, heads, lane, !ready);
                if (ready) break;
            }
            if (lane == 0) *ticket = 0;                          // ready for the next launch
        }
        return;
    }

    if (lane == 0) {
        mbar_init(bar_k, 1);
        mbar_init(bar_v, 1);
        fence_barrier_init();
    }
    __syncwarp();

    // A session with no keys (an empty split-KV shard) has no items: its
    // triples are the neutral element of the merge.
    if (p.emit_triples && blockIdx.x == 0) {
        pdl_wait();                      // `out` / the peers' buffers are written here
        for (uint32_t s = 0; s < p.n_sess; ++s) {
            if (p.n_chunks[s] != 0) continue;
            if (p.x_world > 0) {
                // engine warp w writes rows w, w + kWarps, ... of the session to every rank
                for (uint32_t r = warp; r < p.n_q; r += kWarps) {
                    for (uint32_t w = 0; w < p.x_world; ++w) {
                        float *tr = p.x_rows[w] + ((size_t)p.row[s] * p.n_q + r) * kTripleStride;
                        for (uint32_t i = lane; i < (uint32_t)kTripleStride; i += 32) tr[i] = (i == 0) ? WR_NEG_SENTINEL : 0.f;
                    }
                    xchg_rows_done(p, p.row[s] * p.n_q + r, 1, lane);
                }
                continue;
            }
            float *base = p.out + (size_t)p.row[s] * p.n_q * kTripleStride;
            for (uint32_t i = threadIdx.x; i < p.n_q * kTripleStride; i += kWarps * 32)   // (engine threads only)
                base[i] = (i % kTripleStride == 0) ? WR_NEG_SENTINEL : 0.f;
        }
    }

    // The first item of an engine is fixed (its own number); later ones come
    // from the queue, drawn one item before they are needed.  Items are ordered
    // longest chunks first, so the queue hands the short ones to whoever is
    // free near the end.
    auto draw = [&]() -> int {       // lane 0: take the next item index from the queue
        return (int)n_engines + atom_add_relaxed(queue, 1);
    };
    tile_stream ts;
    ts.have = false;
    ts.it = engine;
    ts.t = ts.t_end = 0;
    ts.s = ts.h = ts.qs = 0;
    ts.pending = 0;
    bool started = false;
    auto next_tile = [&]() -> tile_desc {
        tile_desc d;
        d.flags = 0;
        d.it = d.s = d.h = d.qs = d.t = 0;
        d.page = nullptr;
        if (!ts.have || ts.t >= ts.t_end) {
            if (started) {
                ts.it = (uint32_t)__shfl_sync(0xffffffffu, ts.pending, 0);
                if (lane == 0) ts.pending = draw();
            }
            started = true;
            if (ts.it >= n_items) {
                ts.have = false;
                ts.it = 0xffffffffu;     // stay exhausted
                return d;
            }
            uint32_t s = 0;
            while (s + 1 < p.n_sess && ts.it >= p.item_base[s + 1]) ++s;
            const uint32_t local = ts.it - p.item_base[s];
            const uint32_t nc = p.n_chunks[s];
            const uint32_t c = local % nc, gq = local / nc;
            ts.s = s;
            ts.qs = gq % p.qsubs;
            ts.h = gq / p.qsubs;
            ts.t = p.tile_lo[s] + c * p.chunk_tiles[s];
            ts.t_end = min(ts.t + p.chunk_tiles[s], p.n_tiles[s]);
            ts.have = true;
            d.flags |= 2u;
        }
        d.it = ts.it;
        d.s = ts.s;
        d.h = ts.h;
        d.qs = ts.qs;
        d.t = ts.t;
        d.flags |= 1u;
        if (ts.t + 1 >= ts.t_end) d.flags |= 4u;
        // consumed one tile later, so a table lookup is off the critical path
        d.page = p.page_base[ts.s] ? p.page_base[ts.s] + (uint64_t)ts.t * p.page_bytes
                                   : (const char *)p.b.pages[ts.s][ts.t];
        ++ts.t;
        return d;
    };
    // k_already: the K copy of this (first) tile was issued earlier with mbar_expect_tx_only
    auto issue_k = [&](const tile_desc &d, bool k_already = false) {   // lane 0 only
        const char *src = d.page + wr_block_off(d.h, 0, kHd);
        uint32_t bytes = k_already ? 0u : kBlockBytes;
        const bool first = (d.flags & 2u) != 0;
        const uint32_t heads = min(kHeadsMax, p.group - d.qs * kHeadsMax);
        if (first) bytes += heads * kHd * 4u;
        mbar_expect_tx(bar_k, bytes);
        if (!k_already) bulk_g2s_hint(ws.k, src, kBlockBytes, bar_k, stream_policy);
        if (first) {
            const float *qsrc =
                p.q + ((size_t)p.row[d.s] * p.n_q + d.h * p.group + d.qs * kHeadsMax) * kHd;
            bulk_g2s(ws.q, qsrc, heads * kHd * 4u, bar_k);
        }
    };
    auto issue_v = [&](const tile_desc &d) {   // lane 0 only
        mbar_expect_tx(bar_v, kBlockBytes);
        bulk_g2s_hint(ws.v, d.page + wr_block_off(d.h, 1, kHd), kBlockBytes, bar_v, stream_policy);
    };

    // The engine's first tile is known without the queue.  If it is a page no kernel in flight can
    // be writing, its K and V are requested now, while the kernels before this one finish.
    tile_desc d0 = next_tile();
    const bool early = p.early_tiles && (d0.flags & 1u) && d0.t + 1 < p.n_tiles[d0.s];
    if (early && lane == 0) {
        mbar_expect_tx_only(bar_k, kBlockBytes);
        bulk_g2s_hint(ws.k, d0.page + wr_block_off(d0.h, 0, kHd), kBlockBytes, bar_k, stream_policy);
        issue_v(d0);
    }
    pdl_wait();                          // Q, the new K/V rows, the queue and the scratch: after the earlier kernels
    if (lane == 0) ts.pending = draw();
    if (lane == 0 && (d0.flags & 1u)) {
        issue_k(d0, early);
        if (!early) issue_v(d0);
    }
    tile_desc d1 = next_tile();
    uint32_t uses = 0;
    const uint32_t kaddr = smem_u32(ws.k), vaddr = smem_u32(ws.v);

    uint32_t qb[NT][kHd / 16][2];       // B operand: Q^T, slot column g
    float m[NT], l[NT];
    float oacc[NT][kHd / 16][4];        // O^T: dims on M, slots on N
    // Arrival of a finished item is signalled with a release, which has to wait
    // for the item's partial stores to be acknowledged (about a microsecond).
    // Mid-stream that wait is avoided by signalling one item late, just before
    // the next item's stores are issued: by then the old ones completed long ago.
    int *pend_ticket = nullptr;         // lane 0: counters of the item not yet signalled
    uint32_t pend_pairs = 0;
    auto signal_pending = [&]() {       // lane 0 only
        for (uint32_t pr = 0; pr < pend_pairs; ++pr) red_add_release(pend_ticket + pr, 1);
        pend_ticket = nullptr;
        pend_pairs = 0;
    };

    while (d0.flags & 1u) {
        const uint32_t seq_len = p.b.seq_len[d0.s];
        const uint32_t key_lo = p.key_lo[d0.s];
        const uint32_t heads_here = min(kHeadsMax, p.group - d0.qs * kHeadsMax);

        // ---------------- K tile (and, on the item's first tile, its Q rows)
        if (!mbar_wait(bar_k, uses & 1, p.wait_limit)) {
            if (lane == 0) atomicExch(p.err, 2);
            (void)mbar_wait(bar_v, uses & 1, p.wait_limit);    // this tile's V copy may still be landing
            return;
        }
        if (d0.flags & 2u) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                m[nt] = WR_NEG_SENTINEL;
                l[nt] = 0.f;
#pragma unroll
                for (int i = 0; i < kHd / 16; ++i)
                    oacc[nt][i][0] = oacc[nt][i][1] = oacc[nt][i][2] = oacc[nt][i][3] = 0.f;
                const uint32_t hs = nt * 4 + (g >> 1);
                const bool live = hs < heads_here;
                const float *qrow = ws.q[hs];
#pragma unroll
                for (int ks = 0; ks < kHd / 16; ++ks) {
                    float2 x = make_float2(0.f, 0.f), y = make_float2(0.f, 0.f);
                    if (live) {
                        x = *reinterpret_cast<const float2 *>(qrow + ks * 16 + 2 * t4);
                        y = *reinterpret_cast<const float2 *>(qrow + ks * 16 + 8 + 2 * t4);
                    }
                    uint32_t xh, xl, yh, yl;
                    split_half2(x.x * p.scale, x.y * p.scale, xh, xl);
                    split_half2(y.x * p.scale, y.y * p.scale, yh, yl);
                    qb[nt][ks][0] = (g & 1) ? xl : xh;
                    qb[nt][ks][1] = (g & 1) ? yl : yh;
                }
            }
        }

        // S^T = K . Q^T : four 16-key M tiles, eight 16-dim K steps
        float sacc[NT][4][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int mt = 0; mt < 4; ++mt)
                sacc[nt][mt][0] = sacc[nt][mt][1] = sacc[nt][mt][2] = sacc[nt][mt][3] = 0.f;
        {
            const uint32_t mi = lane >> 3;
            const uint32_t krow0 = (mi & 1) * 8 + (lane & 7);
#pragma unroll
            for (int mt = 0; mt < 4; ++mt) {
                const uint32_t krow = mt * 16 + krow0;
                const uint32_t rowaddr = kaddr + krow * 128;
                const uint32_t sw = krow & 7;
#pragma unroll
                for (int ks = 0; ks < kHd / 16; ++ks) {
                    const uint32_t c16 = ks * 2 + (mi >> 1);
                    uint32_t a[4];
                    ldmatrix_x4(a[0], a[1], a[2], a[3],
                                rowaddr + (c16 >> 3) * 8192 + (((c16 & 7) ^ sw) * 16));
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
                        mma_16816(sacc[nt][mt], a, qb[nt][ks][0], qb[nt][ks][1]);
                }
            }
        }
        __syncwarp();
        if (lane == 0 && (d1.flags & 1u)) issue_k(d1);    // K slot is free: fetch the next K tile

        // ---------------- online softmax for this thread's head slot(s)
        const uint32_t key0 = d0.t * kTile;
        const bool tail = key0 + kTile > seq_len;
        const bool need_mask = tail || key0 < key_lo;
        uint32_t pb[NT][4][2];              // B operand: P^T per 16-key step
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            float sc[4][2];
            float tmax = WR_NEG_SENTINEL;
#pragma unroll
            for (int mt = 0; mt < 4; ++mt) {
                sc[mt][0] = sacc[nt][mt][0] + sacc[nt][mt][1];    // key mt*16+g   (high + low part)
                sc[mt][1] = sacc[nt][mt][2] + sacc[nt][mt][3];    // key mt*16+g+8
                if (need_mask) {
                    const uint32_t ka = key0 + mt * 16 + g, kb2 = ka + 8;
                    if (!(ka < seq_len && ka >= key_lo)) sc[mt][0] = WR_NEG_SENTINEL;
                    if (!(kb2 < seq_len && kb2 >= key_lo)) sc[mt][1] = WR_NEG_SENTINEL;
                }
                tmax = fmaxf(tmax, fmaxf(sc[mt][0], sc[mt][1]));
            }
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 4));
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 8));
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 16));
            const float m_new = fmaxf(m[nt], tmax);
            const float a = (m[nt] == WR_NEG_SENTINEL) ? 0.f : __expf(m[nt] - m_new);
            float psum = 0.f;
#pragma unroll
            for (int mt = 0; mt < 4; ++mt) {
                const float p0 = (sc[mt][0] == WR_NEG_SENTINEL) ? 0.f : __expf(sc[mt][0] - m_new);
                const float p1 = (sc[mt][1] == WR_NEG_SENTINEL) ? 0.f : __expf(sc[mt][1] - m_new);
                psum += p0 + p1;
                // (high, low) pair of p sits where S^T had (slot 2h, slot 2h+1);
                // the 8x8 transpose turns it into the B fragment of P^T.
                const __half p0h = __float2half_rn(p0), p1h = __float2half_rn(p1);
                __half2 h0 = __halves2half2(p0h, __float2half_rn(p0 - __half2float(p0h)));
                __half2 h1 = __halves2half2(p1h, __float2half_rn(p1 - __half2float(p1h)));
                pb[nt][mt][0] = movmatrix_trans(*reinterpret_cast<uint32_t *>(&h0));
                pb[nt][mt][1] = movmatrix_trans(*reinterpret_cast<uint32_t *>(&h1));
            }
            l[nt] = l[nt] * a + psum;
            m[nt] = m_new;
#pragma unroll
            for (int i = 0; i < kHd / 16; ++i) {
                oacc[nt][i][0] *= a; oacc[nt][i][1] *= a; oacc[nt][i][2] *= a; oacc[nt][i][3] *= a;
            }
        }

        // ---------------- V tile
        if (!mbar_wait(bar_v, uses & 1, p.wait_limit)) {
            if (lane == 0) atomicExch(p.err, 3);
            if (d1.flags & 1u) (void)mbar_wait(bar_k, (uses + 1) & 1, p.wait_limit);   // the next K copy is in flight
            return;
        }
        ++uses;
        if (tail) {
            // Rows past the session's length were never written for this
            // position (or belong to a rolled-back step): clear them so that
            // 0 * garbage cannot make a NaN.
            const uint32_t first_bad = seq_len - key0;
            for (uint32_t i = first_bad * 16 + lane; i < kTile * 16; i += 32) {
                const uint32_t krow = i >> 4, ch = i & 15;
                *reinterpret_cast<uint4 *>(ws.v + (ch >> 3) * 8192 + krow * 128 + (ch & 7) * 16) =
                    make_uint4(0, 0, 0, 0);
            }
            fence_proxy_async();   // these generic writes precede the next bulk copy into the slot
            __syncwarp();
        }
        // O^T += V^T . P^T : eight 16-dim M tiles, four 16-key K steps
        {
            const uint32_t mi = lane >> 3;
            const uint32_t krow0 = (mi >> 1) * 8 + (lane & 7);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                const uint32_t krow = kk * 16 + krow0;
                const uint32_t rowaddr = vaddr + krow * 128;
                const uint32_t sw = krow & 7;
#pragma unroll
                for (int md = 0; md < kHd / 16; ++md) {
                    const uint32_t c16 = md * 2 + (mi & 1);
                    uint32_t a[4];
                    ldmatrix_x4_trans(a[0], a[1], a[2], a[3],
                                      rowaddr + (c16 >> 3) * 8192 + (((c16 & 7) ^ sw) * 16));
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
                        mma_16816(oacc[nt][md], a, pb[nt][kk][0], pb[nt][kk][1]);
                }
            }
        }
        __syncwarp();
        if (lane == 0 && (d1.flags & 1u)) issue_v(d1);    // V slot is free: fetch the next V tile

        if (d0.flags & 4u) {
            // ---------------- item done: emit its row(s) or its partial triple
            const uint32_t nc = p.n_chunks[d0.s];
            const bool direct = (nc == 1);
            const size_t row0 = (size_t)p.row[d0.s] * p.n_q + d0.h * p.group + d0.qs * kHeadsMax;
            if (lane == 0 && pend_ticket) signal_pending();      // the previous item (before new stores are in flight)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                float lt = l[nt];
                lt += __shfl_xor_sync(0xffffffffu, lt, 4);
                lt += __shfl_xor_sync(0xffffffffu, lt, 8);
                lt += __shfl_xor_sync(0xffffffffu, lt, 16);
                const uint32_t hs = nt * 4 + t4;            // this thread's head slot
                if (hs < heads_here) {
                    if (direct && !p.emit_triples) {
                        const float inv = (lt > 0.f) ? 1.0f / lt : 0.f;
                        float *o = p.out + (row0 + hs) * kHd;
#pragma unroll
                        for (int md = 0; md < kHd / 16; ++md) {
                            o[md * 16 + g] = (oacc[nt][md][0] + oacc[nt][md][1]) * inv;
                            o[md * 16 + g + 8] = (oacc[nt][md][2] + oacc[nt][md][3]) * inv;
                        }
                    } else {
                        // a one-chunk session's triple is final: with the exchange fused in it goes to every rank
                        const uint32_t n_dst = (direct && p.x_world > 0) ? p.x_world : 1u;
                        for (uint32_t w = 0; w < n_dst; ++w) {
                            float *tr = direct ? (p.x_world > 0 ? p.x_rows[w] : p.out) + (row0 + hs) * kTripleStride
                                               : p.ws + ((size_t)d0.it * 8 + hs) * kTripleStride;
#pragma unroll
                            for (int md = 0; md < kHd / 16; ++md) {
                                tr[WR_CUDA_TRIPLE_PAD + md * 16 + g] = oacc[nt][md][0] + oacc[nt][md][1];
                                tr[WR_CUDA_TRIPLE_PAD + md * 16 + g + 8] = oacc[nt][md][2] + oacc[nt][md][3];
                            }
                            if (g == 0) {
                                tr[0] = m[nt]; tr[1] = lt; tr[2] = 0.f; tr[3] = 0.f;
                            }
                        }
                    }
                }
            }

            if (direct && p.x_world > 0) xchg_rows_done(p, (uint32_t)row0, heads_here, lane);
            if (!direct) {
                // Note the arrival (signalled as described above).  __syncwarp
                // orders every lane's partial stores before lane 0's release; the
                // merge warp that sees the full count acquires it and re-reads
                // the partials through L2.
                __syncwarp();
                const uint32_t gidx = (d0.s * p.n_kv + d0.h) * p.qsubs + d0.qs;
                if (lane == 0) {
                    pend_ticket = p.tickets + (size_t)gidx * kTicketsPerGroup;
                    pend_pairs = (heads_here + 1) / 2;
                    if (!(d1.flags & 1u)) signal_pending();      // the engine's last item: nothing to wait for
                }
            }
        }
        d0 = d1;
        d1 = next_tile();
    }
    if (lane == 0 && pend_ticket) signal_pending();

    // The last engine to leave rewinds the queue for the next launch.
    if (lane == 0) {
        if (atom_add_acq_rel(exits, 1) == (int)n_engines - 1) {
            *queue = 0;
            *exits = 0;
        }
    }
}

}  // namespace wr_decode
