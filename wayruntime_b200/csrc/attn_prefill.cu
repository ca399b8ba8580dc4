// attn_prefill.cu — causal prefill attention on the 5th-generation tensor cores.
//
// The reference has no batched causal op: its prefill runs one single-token
// attention per new token (src/core/session.c:599-630), token i seeing cache
// rows [0, p0+i] through wri_op_gqa_attention (src/core/kernels.c:1414-1527).
// This kernel computes the same rows all at once as a dense contraction.
//
// One CTA = one 128-token query tile of TWO q heads of the same GQA group (a
// lone head when the group size is odd), so every K|V tile staged in shared
// memory feeds both.  Data flow:
//   * TMA warp: the two Q tiles through a 2-D tensor map (cp.async.bulk.tensor,
//     128-byte swizzle, out-of-range rows zero-filled), then K|V tiles of 64
//     keys straight from the paged cache with linear bulk copies — the page
//     layout already is the swizzled operand image the tensor core reads;
//   * two MMA warps (one issuing thread per head): S = Q.K^T as tcgen05.mma
//     M128 N64 K16 x8 into TMEM (S is double-buffered; the scores of tile
//     i+2 are issued as soon as the softmax has read tile i out of TMEM), and
//     O += P.V as M128 N128 K16 x4 (V is the MN-major operand); completion is
//     signalled with tcgen05.commit on mbarriers;
//   * two softmax warpgroups (one per head), one thread per query row: the 64
//     scores of the next tile are fetched from TMEM while the current tile is
//     exponentiated; mask (causal / window), exponentiate against a running
//     reference max, write P as F16 into shared memory in operand order.  The
//     two heads' warps on one scheduler take turns on the special-function
//     unit.  O stays in TMEM; it is rescaled only when the row max has grown
//     by more than 2^8 (exact: the final division by l uses the same
//     reference max), and read once at the end, normalised, transposed
//     through shared memory and stored as whole F32 rows.
// Every wait has a time limit; on expiry the kernel records an error, still
// frees its TMEM and returns.
#include <cuda.h>

#include <algorithm>

#include "wr_internal.cuh"

namespace {

constexpr int kHd = 128;
constexpr int kBM = 128;                 // query rows per head per CTA
constexpr int kBN = 64;                  // keys per tile = page tokens
constexpr int kStages = 3;               // per ring (K and V tiles are staged separately)
constexpr int kGroupThreads = 128;       // one softmax warpgroup
constexpr int kThreads = 2 * kGroupThreads + 96;     // + TMA warp + one MMA warp per head
constexpr uint32_t kQHalfBytes = kBM * 128;      // 64 dims of 128 rows
constexpr uint32_t kQBytes = 2 * kQHalfBytes;    // 32 KB per head
constexpr uint32_t kKVBlock = kBN * kHd * 2;     // 16 KB: one K or V tile
constexpr uint32_t kPBytes = kBM * kBN * 2;      // 16 KB
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTmemS = 0;                   // S of (head h, tile parity b) at columns 64*(2h+b)
constexpr uint32_t kTmemO = 256;                 // O of head h at columns 256 + 128*h
constexpr float kRescaleLog2 = 8.0f;             // move the reference max when it is 2^8 behind
constexpr float kLog2e = 1.4426950408889634f;

struct prefill_params {
    const uint64_t *pages;      // page table of (session, layer)
    float *out;                 // [n, n_q, hd] F32
    int *err;
    uint32_t n, p0, n_q, n_kv, group, n_pairs, window, n_qtiles;
    float scale_log2;           // score scale * log2(e)
    long long wait_limit;       // SM clock cycles a device-side wait may last
};

struct smem_layout {
    alignas(1024) uint8_t q[2][kQBytes];                 // per head
    alignas(1024) uint8_t k[kStages][kKVBlock];          // K ring (freed after the scores)
    alignas(1024) uint8_t v[kStages][kKVBlock];          // V ring (freed after P.V)
    alignas(1024) uint8_t p[2][2][kPBytes];              // [head][tile parity]
    alignas(8) uint64_t bar_q;
    uint64_t full_k[kStages];
    uint64_t empty_k[kStages];
    uint64_t full_v[kStages];
    uint64_t empty_v[kStages];
    uint64_t s_full[2][2];                               // [head][tile parity]
    uint64_t s_free[2][2];                               // softmax has read S out of TMEM
    uint64_t p_ready[2][2];
    uint64_t pv_done[2][2];                              // P.V of the tile using P[parity] has completed
    uint64_t xu_turn[4][2];                              // [scheduler][head]: that head's warp may exponentiate
    uint32_t tmem_base;
};

// ---- tcgen05 / TMA wrappers ------------------------------------------------

__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes)
{
    // start address [0,14) (>>4), leading byte offset [16,30) (>>4), stride byte
    // offset [32,46) (>>4), descriptor version 1 at [46,48), 128-byte swizzle (2) at [61,64)
    const uint64_t lo = (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16);
    const uint64_t hi = (uint64_t)(sbo_bytes >> 4) | (1ull << 14) | (2ull << 29);
    return lo | (hi << 32);
}
// F16 x F16 -> F32 instruction descriptor: c_format F32 (bit 4), N>>3 at [17,23), M>>4 at [24,29),
// bit 16 = B operand is MN-major.
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t m, uint32_t n, bool b_mn_major)
{
    return (1u << 4) | ((b_mn_major ? 1u : 0u) << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// 32 consecutive F32 columns of this thread's TMEM lane (no wait).
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, float *v)
{
    uint32_t *r = reinterpret_cast<uint32_t *>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
          "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
          "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
          "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float *v)
{
    const uint32_t *r = reinterpret_cast<const uint32_t *>(v);
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ float ex2_approx(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Tiled 2-D tensor copy global -> shared (no multicast).  The inner coordinate
// x is in elements; x * 2 bytes is a multiple of 16 for every caller.
__device__ __forceinline__ void tma_load_2d(void *dst_smem, const CUtensorMap *map, int x, int y,
                                            uint64_t *bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst_smem)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

// Tiled 2-D tensor store shared -> global; rows and columns beyond the tensor's
// extent are dropped by the hardware.  x * 4 bytes is a multiple of 16 for the caller.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, int x, int y, const void *src_smem)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(map), "r"(x), "r"(y), "r"(smem_u32(src_smem))
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit_and_wait_read()
{
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

// ---- the kernel ------------------------------------------------------------

__global__ void __launch_bounds__(kThreads, 1)
attn_prefill_hd128_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap out_map,
                          const prefill_params p)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    smem_layout &sm = *reinterpret_cast<smem_layout *>(smem_raw);
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // Heaviest tiles first: the last query tile of the prompt has the most keys.
    const uint32_t per_tile = p.n_kv * p.n_pairs;
    const uint32_t qt = p.n_qtiles - 1 - blockIdx.x / per_tile;
    const uint32_t kvh = (blockIdx.x % per_tile) / p.n_pairs;
    const uint32_t pair = blockIdx.x % p.n_pairs;
    const uint32_t head0 = kvh * p.group + 2 * pair;
    const uint32_t n_heads = min(2u, p.group - 2 * pair);          // 1 for the odd head of a group
    const uint32_t tok0 = qt * kBM;
    const uint32_t rows_here = min((uint32_t)kBM, p.n - tok0);
    // keys visible to this tile: [key_first, key_end)
    const uint32_t key_end = p.p0 + tok0 + rows_here;
    uint32_t key_first = 0;
    if (p.window > 0 && p.p0 + tok0 + 1 > p.window) key_first = p.p0 + tok0 + 1 - p.window;
    const uint32_t t_first = key_first / kBN;
    const uint32_t n_kt = (key_end + kBN - 1) / kBN - t_first;     // >= 1

    // The TMA warp sets the barriers up and starts the first copies (Q, and the first
    // ring's worth of K and V tiles) at once: they fly while TMEM is being allocated
    // and the other warps arrive at the barrier below.
    if (warp == 8 && lane == 0) {
        mbar_init(&sm.bar_q, 1);
        for (int i = 0; i < kStages; ++i) {
            mbar_init(&sm.full_k[i], 1);
            mbar_init(&sm.empty_k[i], n_heads);      // one tcgen05.commit per head
            mbar_init(&sm.full_v[i], 1);
            mbar_init(&sm.empty_v[i], n_heads);
        }
        for (int h = 0; h < 2; ++h) {
            mbar_init(&sm.s_full[h][0], 1);
            mbar_init(&sm.s_full[h][1], 1);
            mbar_init(&sm.s_free[h][0], kGroupThreads);
            mbar_init(&sm.s_free[h][1], kGroupThreads);
            mbar_init(&sm.p_ready[h][0], kGroupThreads);
            mbar_init(&sm.p_ready[h][1], kGroupThreads);
            mbar_init(&sm.pv_done[h][0], 1);
            mbar_init(&sm.pv_done[h][1], 1);
            for (int q = 0; q < 4; ++q) mbar_init(&sm.xu_turn[q][h], 1);
        }
        fence_barrier_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&sm.tmem_base)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // lane 0 of the TMA warp streams the K tiles, lane 1 the V tiles: separate rings,
    // because a K tile is free again long before its V tile is.
    auto issue_kv_tile = [&](uint32_t i) {
        uint8_t (*ring)[kKVBlock] = lane == 0 ? sm.k : sm.v;
        uint64_t *full = lane == 0 ? sm.full_k : sm.full_v;
        const uint32_t st = i % kStages;
        const char *src = (const char *)p.pages[t_first + i] + wr_block_off(kvh, lane, kHd);
        mbar_expect_tx(&full[st], kKVBlock);
        bulk_g2s(ring[st], src, kKVBlock, &full[st]);
    };
    if (warp == 8) {
        __syncwarp();                                   // lane 1 uses barriers that lane 0 has just set up
        if (lane == 0) {
            mbar_expect_tx(&sm.bar_q, n_heads * kQBytes);
            for (uint32_t h = 0; h < n_heads; ++h) {
                tma_load_2d(sm.q[h], &q_map, (int)((head0 + h) * kHd), (int)tok0, &sm.bar_q);
                tma_load_2d(sm.q[h] + kQHalfBytes, &q_map, (int)((head0 + h) * kHd + 64), (int)tok0,
                            &sm.bar_q);
            }
        }
        if (lane < 2)
            for (uint32_t i = 0; i < min((uint32_t)kStages, n_kt); ++i) issue_kv_tile(i);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;

    if (warp == 8) {
        // ------------------------------------------------------------ TMA warp
        if (lane < 2) {
            uint64_t *empty = lane == 0 ? sm.empty_k : sm.empty_v;
            for (uint32_t i = kStages; i < n_kt; ++i) {
                const uint32_t st = i % kStages;
                if (!mbar_wait(&empty[st], ((i / kStages) - 1) & 1, p.wait_limit)) {
                    atomicExch(p.err, 11);
                    break;
                }
                issue_kv_tile(i);
            }
        }
    } else if (warp >= 9) {
        // ------------------------------------- MMA warps: one issuing thread per head
        // (while one of them waits on a barrier the other keeps the tensor core fed)
        const uint32_t h = warp - 9;
        if (lane == 0 && h < n_heads) {
            const uint32_t idesc_s = umma_idesc(kBM, kBN, false);
            const uint32_t idesc_o = umma_idesc(kBM, kHd, true);
            bool ok = mbar_wait(&sm.bar_q, 0, p.wait_limit);
            // This one thread feeds the tensor core, so its instruction count
            // per tile matters: descriptors are built once and an operand is
            // selected by adding its byte offset (>>4) to the address field.
            const uint64_t qd = umma_desc(smem_u32(sm.q[h]), 16, 1024);
            const uint64_t k_desc0 = umma_desc(smem_u32(sm.k[0]), 16, 1024);
            const uint64_t v_desc0 = umma_desc(smem_u32(sm.v[0]), 8192, 1024);
            const uint64_t p_desc0 = umma_desc(smem_u32(sm.p[0][0]), 16, 1024);
            auto issue_s = [&](uint32_t h, uint32_t i) {

                const uint64_t kd = k_desc0 + (uint64_t)((i % kStages) * (kKVBlock >> 4));
                const uint32_t d = tmem + kTmemS + 64 * (2 * h + (i & 1));
#pragma unroll
                for (int kk = 0; kk < kHd / 16; ++kk) {
                    const uint32_t half = kk >> 2, off = (kk & 3) * 32;
                    umma_f16(d, qd + ((half * kQHalfBytes + off) >> 4),
                             kd + ((half * (kBN * 128) + off) >> 4), idesc_s, kk > 0);
                }
                umma_commit(&sm.s_full[h][i & 1]);
            };
            // Scores run two tiles ahead of the softmax that consumes them (S is
            // double-buffered in TMEM), so a softmax does not wait for its S.
            for (uint32_t i = 0; ok && i < min(2u, n_kt); ++i) {
                ok = mbar_wait(&sm.full_k[i], 0, p.wait_limit);
                if (!ok) break;
                tc_fence_after();
                issue_s(h, i);
                umma_commit(&sm.empty_k[i]);                     // this head is done with K tile i
            }
            for (uint32_t i = 0; ok && i < n_kt; ++i) {
                if (i + 2 < n_kt) {
                    // the softmax of tile i has its scores in registers: S[i&1] can take
                    // tile i+2 while that softmax is still exponentiating
                    ok = mbar_wait(&sm.s_free[h][i & 1], (i >> 1) & 1, p.wait_limit);
                    if (ok) ok = mbar_wait(&sm.full_k[(i + 2) % kStages], ((i + 2) / kStages) & 1, p.wait_limit);
                    if (!ok) break;
                    tc_fence_after();
                    issue_s(h, i + 2);
                    umma_commit(&sm.empty_k[(i + 2) % kStages]);
                }
                // softmax of (head h, tile i) has written P[i&1]
                ok = mbar_wait(&sm.p_ready[h][i & 1], (i >> 1) & 1, p.wait_limit);
                if (ok) ok = mbar_wait(&sm.full_v[i % kStages], (i / kStages) & 1, p.wait_limit);
                if (!ok) break;
                tc_fence_after();
                const uint64_t vd = v_desc0 + (uint64_t)((i % kStages) * (kKVBlock >> 4));
                const uint64_t pd = p_desc0 + (uint64_t)((2 * h + (i & 1)) * (kPBytes >> 4));
                const uint32_t d = tmem + kTmemO + 128 * h;
#pragma unroll
                for (int kk = 0; kk < kBN / 16; ++kk)
                    umma_f16(d, pd + ((kk * 32) >> 4), vd + ((kk * 2048) >> 4), idesc_o, (i > 0) || (kk > 0));
                umma_commit(&sm.pv_done[h][i & 1]);              // O_h holds tiles 0..i, P[i&1] is free
                umma_commit(&sm.empty_v[i % kStages]);           // this head is done with V tile i
            }
            if (!ok) atomicExch(p.err, 12);
        }
    } else if (warp < 4 * n_heads) {
        // ----------------------------- softmax warpgroup h: one thread per query row
        const uint32_t h = warp >> 2;
        const uint32_t row = tid & (kGroupThreads - 1);     // TMEM lane
        const uint32_t lane_base = ((warp & 3u) * 32u) << 16;
        const uint32_t s_base = tmem + lane_base + kTmemS + 128 * h;
        const uint32_t o_addr = tmem + lane_base + kTmemO + 128 * h;
        const uint32_t qpos = p.p0 + tok0 + row;            // absolute position of this query
        uint32_t lo_key = 0;
        if (p.window > 0 && qpos + 1 > p.window) lo_key = qpos + 1 - p.window;
        const float c2 = p.scale_log2;
        float m_ref = WR_NEG_SENTINEL;                      // reference max, log2 domain
        float l = 0.f;
        const uint32_t quad = warp & 3u;                    // scheduler this warp and its twin of the other head share
        const bool two = (n_heads == 2);
        // The scores of the current tile live in s[]; the next tile's are fetched
        // from TMEM while this tile is still being exponentiated.
        float s[kBN];
        bool ok = mbar_wait(&sm.s_full[h][0], 0, p.wait_limit);
        if (ok) {
            tc_fence_after();
            tmem_ld32_nowait(s_base, s);
            tmem_ld32_nowait(s_base + 32, s + 32);
            tmem_wait_ld();
            tc_fence_before();
            mbar_arrive(&sm.s_free[h][0]);                      // S[0] may take tile 2
        }
        for (uint32_t i = 0; ok && i < n_kt; ++i) {
            const uint32_t key0 = (t_first + i) * kBN;
            // tiles that no row's causal or window limit cuts through need no masking
            const bool edge = (key0 + kBN - 1 > p.p0 + tok0) || (p.window > 0);
            if (edge) {
#pragma unroll
                for (int j = 0; j < kBN; ++j) {
                    const uint32_t key = key0 + j;
                    if (key > qpos || key < lo_key) s[j] = WR_NEG_SENTINEL;
                }
            }
            // four independent max chains instead of one 64-deep dependency
            float mx[4] = {s[0], s[1], s[2], s[3]};
#pragma unroll
            for (int j = 4; j < kBN; j += 4) {
                mx[0] = fmaxf(mx[0], s[j]);
                mx[1] = fmaxf(mx[1], s[j + 1]);
                mx[2] = fmaxf(mx[2], s[j + 2]);
                mx[3] = fmaxf(mx[3], s[j + 3]);
            }
            const float tmax = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
            // Move the reference max (and rescale O) only when it is far behind.
            // The rescale uses warp-wide TMEM instructions, so the warp decides
            // together; rows that do not need it multiply by one.
            const float tm2 = tmax * c2;
            const bool grow = (tmax > WR_NEG_SENTINEL) && (m_ref != WR_NEG_SENTINEL) && (tm2 > m_ref + kRescaleLog2);
            if (tmax > WR_NEG_SENTINEL && m_ref == WR_NEG_SENTINEL) m_ref = tm2;
            if (__any_sync(0xffffffffu, grow)) {
                const float a = grow ? ex2_approx(m_ref - tm2) : 1.0f;
                // O must hold every earlier tile (tile i-1 was the last one issued)
                ok = mbar_wait(&sm.pv_done[h][(i - 1) & 1], ((i - 1) >> 1) & 1, p.wait_limit);
                if (!ok) break;
                tc_fence_after();
#pragma unroll 1
                for (int c = 0; c < kHd; c += 32) {
                    float o[32];
                    tmem_ld32_nowait(o_addr + c, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int e = 0; e < 32; ++e) o[e] *= a;
                    tmem_st32(o_addr + c, o);
                }
                tmem_wait_st();
                if (grow) {
                    l *= a;
                    m_ref = tm2;
                }
            }
            // P = 2^(s*c2 - m_ref) as F16 in operand order: row `row`, 8 chunks of 8 keys;
            // P[i&1] is free once the P.V of tile i-2 has read it
            if (i >= 2) {
                ok = mbar_wait(&sm.pv_done[h][i & 1], ((i >> 1) - 1) & 1, p.wait_limit);
                if (!ok) break;
            }
            // The exponentials saturate the special-function unit, which this warp
            // shares with the same-numbered warp of the other head: the two take
            // turns, so that one's loads, max and hand-offs run under the other's
            // exponentials instead of both queueing for the unit at once.
            if (two && (h == 1 || i > 0)) {
                ok = mbar_wait(&sm.xu_turn[quad][h], (h == 1 ? i : i - 1) & 1, p.wait_limit);
                if (!ok) break;
            }
            uint8_t *prow = sm.p[h][i & 1] + row * 128;
            // (no visible key yet for this row: every score is the sentinel and must give 0)
            const float neg_m = (m_ref == WR_NEG_SENTINEL) ? 0.f : -m_ref;
            float psum[4] = {0.f, 0.f, 0.f, 0.f};
            auto exp_chunk = [&](int c) {
                uint32_t w[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    // a masked score is -1e30: the fused multiply-add stays hugely negative, 2^x gives 0
                    const float p0 = ex2_approx(fmaf(s[c * 8 + 2 * e], c2, neg_m));
                    const float p1 = ex2_approx(fmaf(s[c * 8 + 2 * e + 1], c2, neg_m));
                    psum[e] += p0 + p1;
                    const __half2 hh = __floats2half2_rn(p0, p1);
                    w[e] = *reinterpret_cast<const uint32_t *>(&hh);
                }
                *reinterpret_cast<uint4 *>(prow + ((c ^ (row & 7)) * 16)) = make_uint4(w[0], w[1], w[2], w[3]);
            };
            const bool more = i + 1 < n_kt;
            const uint32_t s_next = s_base + 64 * ((i + 1) & 1);
#pragma unroll
            for (int c = 0; c < 4; ++c) exp_chunk(c);
            if (more) {
                // columns 0..31 are spent: refill them with the next tile's (its scores
                // were issued two tiles ahead, so this wait normally falls through)
                ok = mbar_wait(&sm.s_full[h][(i + 1) & 1], ((i + 1) >> 1) & 1, p.wait_limit);
                if (!ok) break;
                tc_fence_after();
                tmem_ld32_nowait(s_next, s);
            }
#pragma unroll
            for (int c = 4; c < 7; ++c) exp_chunk(c);
            if (two && lane == 0) mbar_arrive(&sm.xu_turn[quad][h ^ 1]);   // a little early: hides the hand-off
            exp_chunk(7);
            if (more) tmem_ld32_nowait(s_next + 32, s + 32);
            l += (psum[0] + psum[1]) + (psum[2] + psum[3]);
            if (i == n_kt - 1 && (key_end % kBN) != 0) {
                // Cache rows past the last key were never written for this
                // prompt (or belong to a rolled-back step): clear them in the
                // staged V tile so that 0 * garbage cannot make a NaN (each head's
                // group does it before releasing its own P.V; the writes are equal).
                ok = mbar_wait(&sm.full_v[i % kStages], (i / kStages) & 1, p.wait_limit);
                if (!ok) break;
                if (row < kBN && key0 + row >= key_end) {
                    uint8_t *vrow = sm.v[i % kStages] + row * 128;
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        *reinterpret_cast<uint4 *>(vrow + c * 16) = make_uint4(0, 0, 0, 0);
                        *reinterpret_cast<uint4 *>(vrow + 8192 + c * 16) = make_uint4(0, 0, 0, 0);
                    }
                }
            }
            fence_proxy_async();          // P (generic writes) is read by the tensor core
            tc_fence_before();
            mbar_arrive(&sm.p_ready[h][i & 1]);
            if (more) {
                tmem_wait_ld();
                tc_fence_before();
                mbar_arrive(&sm.s_free[h][(i + 1) & 1]);        // S[(i+1)&1] may take tile i+3
            }
        }
        tmem_wait_ld();                   // (an early exit may leave a fetch in flight)
        if (ok) {
            // The last P.V completes after every earlier one (one issuing thread,
            // in order); this group has already observed the previous phase of that
            // barrier (tile n_kt-3), so the parity wait is one completion behind at most.
            ok = mbar_wait(&sm.pv_done[h][(n_kt - 1) & 1], ((n_kt - 1) >> 1) & 1, p.wait_limit);
            if (ok) {
                tc_fence_after();
                const float inv = (l > 0.f) ? 1.0f / l : 0.f;
                // O leaves TMEM one row per thread.  Each warp lays its 32 rows out in
                // shared memory as four tiles of 32 rows x 32 columns (128-byte rows, the
                // eight 16-byte chunks of a row XOR-swizzled with the row number, which is
                // both conflict free for these row-wise writes and the layout a 128-byte
                // swizzled tensor map expects) and hands them to the TMA engine, which
                // writes them out and drops the rows beyond the prompt.  This head's Q and
                // P tiles serve as the staging area: every MMA that read them has completed.
                const uint32_t wq = warp & 3u;
                uint8_t *stage = (wq < 2) ? sm.q[h] + wq * (kQBytes / 2) : sm.p[h][wq - 2];
                float o[kHd];                                      // the whole row: one wait for four loads
#pragma unroll
                for (int c = 0; c < kHd; c += 32) tmem_ld32_nowait(o_addr + c, o + c);
                tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < kHd; c += 32) {
                    float4 *trow = reinterpret_cast<float4 *>(stage + (c / 32) * 4096 + lane * 128);
#pragma unroll
                    for (int e = 0; e < 8; ++e)
                        trow[e ^ (lane & 7)] = make_float4(o[c + 4 * e] * inv, o[c + 4 * e + 1] * inv,
                                                            o[c + 4 * e + 2] * inv, o[c + 4 * e + 3] * inv);
                }
                fence_proxy_async();                               // generic writes -> TMA reads
                __syncwarp();
                if (lane == 0 && wq * 32u < rows_here) {
                    const int y = (int)(tok0 + wq * 32u);
                    const int x = (int)((head0 + h) * kHd);
#pragma unroll
                    for (int c = 0; c < 4; ++c) tma_store_2d(&out_map, x + 32 * c, y, stage + c * 4096);
                    tma_store_commit_and_wait_read();              // the staging area is read before the CTA ends
                }
            }
        }
        if (!ok) atomicExch(p.err, 13);
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols)
                     : "memory");
    }
}

// F32 -> F16 (round to nearest) copy of Q for callers that hold F32 queries.
__global__ void q_to_f16_kernel(const float *__restrict__ src, __half *__restrict__ dst, size_t n)
{
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        dst[i] = __float2half_rn(src[i]);
}

typedef CUresult (*encode_tiled_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                    const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                    CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                    CUtensorMapFloatOOBfill);

encode_tiled_fn get_encode_tiled()
{
    static encode_tiled_fn fn = nullptr;
    if (!fn) {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (encode_tiled_fn)sym;
        else
            (void)cudaGetLastError();
    }
    return fn;
}

}  // namespace

extern "C" int wr_cuda_attn_prefill(wr_cuda_ctx *ctx, wr_cuda_kv *kv, uint32_t layer, uint32_t p0,
                                    uint32_t n, const void *q, int q_dtype, float *out,
                                    uint32_t n_q_heads, float scale_override, uint32_t window, int mem)
{
    if (!ctx || !kv || kv->ctx != ctx || !q || !out) return WR_CUDA_ERR_INVAL;
    if (layer >= kv->n_layers) return WR_CUDA_ERR_INVAL;
    if (q_dtype != WR_CUDA_F32 && q_dtype != WR_CUDA_F16) return WR_CUDA_ERR_INVAL;
    if (mem != WR_CUDA_MEM_HOST && mem != WR_CUDA_MEM_DEVICE) return WR_CUDA_ERR_INVAL;
    if (n == 0) return WR_CUDA_OK;
    if (n_q_heads == 0 || n_q_heads % kv->n_kv != 0) return WR_CUDA_ERR_INVAL;   // kernels.c:1429-1432
    if (kv->hd != kHd) return WR_CUDA_ERR_UNSUPPORTED;       // tensor-core tiles are built for head_dim 128
    std::lock_guard<std::mutex> g(ctx->lock);
    if ((uint64_t)p0 + n > ctx->attn_max_seq) return WR_CUDA_ERR_LIMIT;           // kernels.c:1444
    if ((uint64_t)p0 + n > kv->max_ctx) return WR_CUDA_ERR_INVAL;                 // capacity, kernels.c:1449-1454
    encode_tiled_fn encode = get_encode_tiled();
    if (!encode) return WR_CUDA_ERR_INTERNAL;
    WR_CUDA_TRY(cudaSetDevice(ctx->device));

    const size_t elems = (size_t)n * n_q_heads * kHd;
    const size_t q_in_bytes = elems * (q_dtype == WR_CUDA_F32 ? 4 : 2);
    const size_t q16_bytes = (elems * 2 + 255) & ~(size_t)255;
    const size_t out_bytes = elems * 4;
    // staging layout: [q as F16][q as given (host callers)][out (host callers)]
    size_t need = 0;
    const bool convert = (q_dtype == WR_CUDA_F32);
    const bool host = (mem == WR_CUDA_MEM_HOST);
    if (convert) need += q16_bytes;
    if (host) need += ((q_in_bytes + 255) & ~(size_t)255) + out_bytes;
    if (need) {
        int rc = wr_ctx_reserve_stage(ctx, need, 0);
        if (rc != WR_CUDA_OK) return rc;
    }
    char *stage = (char *)ctx->stage_dev;
    size_t off = 0;
    __half *q16 = nullptr;
    if (convert) {
        q16 = (__half *)(stage + off);
        off += q16_bytes;
    }
    const void *dq = q;
    float *dout = out;
    if (host) {
        dq = stage + off;
        off += (q_in_bytes + 255) & ~(size_t)255;
        dout = (float *)(stage + off);
        WR_CUDA_TRY(cudaMemcpyAsync((void *)dq, q, q_in_bytes, cudaMemcpyHostToDevice, ctx->stream));
    }
    if (convert) {
        const uint32_t blocks = (uint32_t)std::min<size_t>((elems + 255) / 256, (size_t)ctx->sm_count * 16);
        q_to_f16_kernel<<<blocks, 256, 0, ctx->stream>>>((const float *)dq, q16, elems);
        ctx->launches++;
        WR_CUDA_TRY(cudaGetLastError());
    } else {
        q16 = (__half *)dq;
    }
    if (((uintptr_t)q16 & 15u) || ((uintptr_t)dout & 15u)) return WR_CUDA_ERR_INVAL;

    CUtensorMap q_map;
    const cuuint64_t dims[2] = {(cuuint64_t)n_q_heads * kHd, (cuuint64_t)n};
    const cuuint64_t strides[1] = {(cuuint64_t)n_q_heads * kHd * 2};
    const cuuint32_t box[2] = {64, kBM};
    const cuuint32_t estr[2] = {1, 1};
    if (encode(&q_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void *)q16, dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return WR_CUDA_ERR_INTERNAL;

    CUtensorMap out_map;                                          // F32 [n, n_q_heads * hd], boxes of 32 x 32
    const cuuint64_t odims[2] = {(cuuint64_t)n_q_heads * kHd, (cuuint64_t)n};
    const cuuint64_t ostrides[1] = {(cuuint64_t)n_q_heads * kHd * 4};
    const cuuint32_t obox[2] = {32, 32};
    if (encode(&out_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void *)dout, odims, ostrides, obox, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return WR_CUDA_ERR_INTERNAL;

    prefill_params p;
    p.pages = kv->d_pages + (size_t)layer * kv->n_pages;
    p.out = dout;
    p.err = ctx->dev_err;
    p.wait_limit = ctx->wait_limit;
    p.n = n;
    p.p0 = p0;
    p.n_q = n_q_heads;
    p.n_kv = kv->n_kv;
    p.group = n_q_heads / kv->n_kv;
    p.n_pairs = (p.group + 1) / 2;
    p.window = window;
    p.n_qtiles = (n + kBM - 1) / kBM;
    const float scale = (scale_override > 0.0f) ? scale_override : 1.0f / sqrtf((float)kHd);   // kernels.c:1457-1459
    p.scale_log2 = scale * kLog2e;
    if (!(ctx->attr_flags & 2u)) {
        WR_CUDA_TRY(cudaFuncSetAttribute(attn_prefill_hd128_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)sizeof(smem_layout)));
        ctx->attr_flags |= 2u;
    }
    const uint32_t grid = p.n_qtiles * p.n_kv * p.n_pairs;
    attn_prefill_hd128_kernel<<<grid, kThreads, sizeof(smem_layout), ctx->stream>>>(q_map, out_map, p);
    ctx->launches++;
    WR_CUDA_TRY(cudaGetLastError());
    if (host) {
        WR_CUDA_TRY(cudaMemcpyAsync(out, dout, out_bytes, cudaMemcpyDeviceToHost, ctx->stream));
        return wr_ctx_sync_checked(ctx);
    }
    return WR_CUDA_OK;
}
