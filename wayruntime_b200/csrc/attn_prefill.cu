// attn_prefill.cu — causal prefill attention on the 5th-generation tensor cores.
//
// The reference has no batched causal op: its prefill runs one single-token
// attention per new token (src/core/session.c:599-630), token i seeing cache
// rows [0, p0+i] through wri_op_gqa_attention (src/core/kernels.c:1414-1527).
// This kernel computes the same rows all at once as a dense contraction.
//
// Work is cut into BLOCKS of 128 query rows of one q head.  A CTA always holds
// two blocks that read the same K/V tiles: two q heads of one GQA group over
// the same 128 tokens, or — for the odd head of a group — the same head over
// two consecutive 128-token ranges.  CTAs are persistent (one per SM): they
// draw work tiles, longest first, from a counter in global memory, and the
// next tile's queries and first scores are in flight while the previous
// tile's output leaves.
//
// Per CTA, per step of 128 keys (two cache pages):
//   * producer warp: K and V tiles come straight from the paged cache with
//     linear bulk copies — the page layout already is the swizzled operand image
//     the tensor core reads; Q tiles come through a 2-D tensor map
//     (cp.async.bulk.tensor, 128-byte swizzle, rows past the prompt zero-filled);
//   * MMA warp (the whole warp runs the control flow and works the operands
//     out, one elected lane issues): S_b = Q_b.K^T as eight tcgen05.mma M128 N128
//     K16 into the block's 128 score columns of TMEM, and O_b += P_b.V as eight
//     more with P read from TMEM (the A operand) and V as the MN-major B operand.
//     The two blocks alternate — the tensor core works on one block's tiles
//     while the other block's scores are being exponentiated — so neither S nor
//     P needs a second buffer: P overwrites the first 64 columns of its own S,
//     and the next scores are issued right behind the P.V that consumed it (the
//     tensor core executes in issue order);
//   * two softmax warpgroups (one per block, one thread per query row): fetch
//     the 128 scores from TMEM, mask (causal / window), row maximum,
//     exponentiate against a running reference maximum — packed two-element
//     FMA-pipe instructions and three-input maxima keep the instruction count
//     down, and a share of the exponentials runs as a polynomial on the FMA
//     pipe, because the special-function unit is as loaded as the tensor core
//     here — and write P as F16 back into TMEM.  O stays in TMEM; it is rescaled
//     only when the row maximum has grown by more than 2^8 (exact: the final
//     division by l uses the same reference maximum), read once at the end,
//     normalised, and sent out in pieces of 32 rows x 16 values through two swizzled
//     shared-memory buffers as TMA tensor stores (a store instruction whose lanes each write a
//     row of their own touches 32 cache lines for 512 bytes).
// Every wait has a time limit; on expiry the kernel records an error, still
// frees its TMEM and returns.
#include <cuda.h>

#include <algorithm>

#include "wr_internal.cuh"

namespace {

constexpr int kHd = 128;
constexpr int kBM = 128;                 // query rows per block
constexpr int kBN = 128;                 // keys per step = two cache pages
constexpr int kStages = 2;               // per ring (K and V tiles are staged separately)
constexpr int kGroupThreads = 128;       // one softmax warpgroup
constexpr int kThreads = 2 * kGroupThreads + 64;     // + producer warp + MMA warp
constexpr uint32_t kQHalfBytes = kBM * 128;      // 64 dims of 128 rows
constexpr uint32_t kQBytes = 2 * kQHalfBytes;    // 32 KB per block
constexpr uint32_t kPageBlock = 64 * kHd * 2;    // 16 KB: K or V of one head in one page
constexpr uint32_t kKVTile = 2 * kPageBlock;     // 32 KB: 128 keys
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTmemS = 0;                   // S (then P) of block b at columns 128*b
constexpr uint32_t kTmemO = 256;                 // O of block b at columns 256 + 128*b
constexpr float kRescaleLog2 = 8.0f;             // move the reference max when it is 2^8 behind
constexpr float kLog2e = 1.4426950408889634f;
constexpr int kTileSlots = 4;                    // ring of published work tiles
// Of every kPolyPeriod pairs of exponentials one pair is evaluated on the FMA pipe (0: none).
#ifndef WR_PREFILL_POLY_PERIOD
#define WR_PREFILL_POLY_PERIOD 4
#endif
constexpr int kPolyPeriod = WR_PREFILL_POLY_PERIOD;

// Development aid, off by default: built with -DWR_PREFILL_TIMELINE the kernel's CTA 0
// writes clock64() stamps of its hand-offs into a device buffer (kTlRoles rows of
// kTlEvents stamps: row 0/1 = softmax group of block 0/1, row 2 = MMA thread), which
// wr_cuda_debug_prefill_timeline copies out.
#ifdef WR_PREFILL_TIMELINE
// Rows 3 (softmax group of block 0) and 4 (MMA warp) hold tile-level stamps as clock * 16 + tag.
constexpr int kTlRoles = 5, kTlEvents = 512, kTlCtas = 160;     // + per CTA: start ns, end ns, tiles, steps
__device__ __forceinline__ long long tl_ns()
{
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#ifndef WR_PREFILL_TL_CTA
#define WR_PREFILL_TL_CTA 0
#endif
#define TL_DECL uint32_t tl_n = 0, tl_m = 0; const bool tl_on = (blockIdx.x == WR_PREFILL_TL_CTA) && p.tl != nullptr
#define TL(role) do { if (tl_on && tl_n < kTlEvents) p.tl[(role) * kTlEvents + tl_n++] = clock64(); } while (0)
#define TLT(role, tag) do { if (tl_on && tl_m < kTlEvents) p.tl[(role) * kTlEvents + tl_m++] = clock64() * 16 + (tag); } while (0)
// where a role was when one of its waits ran out: four values at the end of its row
#define TLFAIL(role, a, b, c, d) do { if (p.tl) { long long *r = p.tl + (role) * kTlEvents + kTlEvents - 4; r[0] = (a); r[1] = (b); r[2] = (c); r[3] = (d); } } while (0)
#else
#define TL_DECL
#define TL(role)
#define TLT(role, tag)
#define TLFAIL(role, a, b, c, d)
#endif

struct prefill_params {
#ifdef WR_PREFILL_TIMELINE
    long long *tl;
#endif
    const uint64_t *pages;      // page table of (session, layer)
    const char *page_base;      // non-null: page t = page_base + t * page_bytes
    uint64_t page_bytes;
    int *err;
    int *sched;                 // [0] next work tile, [1] CTAs that have left
    uint32_t n, p0, n_q, n_kv, group, window, n_qtiles, n_tiles;
    float scale_log2;           // score scale * log2(e)
    long long wait_limit;       // SM clock cycles a device-side wait may last
    uint32_t early;             // the kernel before this one only reads what this one reads
};

// A published work tile: up to two blocks over the same KV head.
struct tile_info {
    uint32_t valid, nblk, kvh, pad;
    uint32_t head[2], qt[2];
};

struct smem_layout {
    alignas(1024) uint8_t q[2][kQBytes];                 // per block: [64-dim half][128 rows][128 B]
    alignas(1024) uint8_t k[kStages][kKVTile];           // [64-dim half][128 keys][128 B]
    alignas(1024) uint8_t v[kStages][kKVTile];           // [page][64-dim half][64 keys][128 B]
    alignas(8) uint64_t q_full[2];                       // per block
    uint64_t q_free[2];                                  // per block: its last scores of the tile have completed
    uint64_t k_full[kStages], k_free[kStages];
    uint64_t v_full[kStages], v_free[kStages];
    uint64_t s_full[2];                                  // per block: scores are in TMEM
    uint64_t p_full[2];                                  // per block: P is in TMEM (one arrival per warp)
    uint64_t o_done[2];                                  // per block: the tile's last P.V has completed
    uint64_t o_free[2];                                  // per block: O has been read out (one arrival per warp)
    uint64_t tile_ready[kTileSlots];
    tile_info tile[kTileSlots];
    uint32_t tmem_base;
    // per softmax warp: two buffers of 32 rows x 16 output values on their way out (16-byte pieces
    // swizzled by row pair: the 64-byte swizzle of the output tensor map)
    alignas(1024) uint8_t out_stage[8][2][32 * 64];
};
static_assert(sizeof(smem_layout) <= 232448, "the CTA's shared memory is 227 KB at most");

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
// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one()
{
    uint32_t pred;
    asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(pred));
    return pred != 0;
}
// D[tmem] (+)= A[smem] . B[smem]; descriptors as (low, high) words
__device__ __forceinline__ void umma_ss(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                        uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\t"
        "mov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
        ::"r"(tmem_d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] . B[smem]
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                        uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
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
// 16 consecutive 32-bit columns of this thread's TMEM lane: 32 F16 probabilities, two per column.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t *r)
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ float ex2_approx(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Two F32 values in one 64-bit register, for the packed FMA-pipe instructions
// (one issue slot for two elements: the softmax warps are issue-bound).
__device__ __forceinline__ uint64_t pack2(float a, float b)
{
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float &a, float &b)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c)
{
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b)
{
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t sub2(uint64_t a, uint64_t b)
{
    uint64_t d;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float max3(float a, float b, float c)
{
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// 2^x on the FMA pipe for a packed pair: x = r + f with r the nearest integer, a degree-3
// polynomial for 2^f on [-0.5, 0.5] (relative error 7.6e-5, well inside the
// F16 rounding of P), r added to the exponent field.  x <= -126 gives ~1e-38.
__device__ __forceinline__ void ex2_poly2(uint64_t x2, float &p0, float &p1)
{
    float x0, x1;
    unpack2(x2, x0, x1);
    x2 = pack2(fmaxf(x0, -126.0f), fmaxf(x1, -126.0f));
    const uint64_t magic = pack2(12582912.0f, 12582912.0f);
    const uint64_t t2 = add2(x2, magic);
    const uint64_t f2 = sub2(x2, sub2(t2, magic));
    uint64_t q2 = fma2(pack2(0.05516839f, 0.05516839f), f2, pack2(0.24260326f, 0.24260326f));
    q2 = fma2(q2, f2, pack2(0.69326085f, 0.69326085f));
    q2 = fma2(q2, f2, pack2(0.99992865f, 0.99992865f));
    float q0, q1, t0, t1;
    unpack2(q2, q0, q1);
    unpack2(t2, t0, t1);
    p0 = __int_as_float(__float_as_int(q0) + (__float_as_int(t0) << 23));
    p1 = __int_as_float(__float_as_int(q1) + (__float_as_int(t1) << 23));
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
// Tiled 2-D tensor copy shared -> global (rows past the tensor's extent are dropped), tracked by
// the issuing thread's bulk group.  x in elements; x * 4 bytes is a multiple of 16 for the caller.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, const void *src_smem, int x, int y)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(smem_u32(src_smem)), "r"(x), "r"(y)
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// The issuing thread's bulk stores, except the N latest, have finished reading shared memory.
template <int N>
__device__ __forceinline__ void tma_store_wait_read()
{
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// ---- work tiles -------------------------------------------------------------
//
// Tiles are numbered longest first.  Query tiles are taken from the end of the
// prompt in pairs (r1, r0 = r1 - 1); pair k contributes, in this order,
//   n_kv tiles of the odd head of each group over (r0, r1)      [only if group is odd]
//   n_kv * (group / 2) head-pair tiles over r1
//   n_kv * (group / 2) head-pair tiles over r0                  [only if r0 >= 0]
__host__ __device__ inline uint32_t tiles_per_qpair(uint32_t n_kv, uint32_t group)
{
    return n_kv * ((group & 1u) + 2u * (group / 2u));
}
__host__ __device__ inline uint32_t prefill_tile_count(uint32_t n_qtiles, uint32_t n_kv, uint32_t group)
{
    uint32_t n = (n_qtiles / 2u) * tiles_per_qpair(n_kv, group);
    if (n_qtiles & 1u) n += n_kv * ((group & 1u) + group / 2u);      // the first query tile on its own
    return n;
}
__device__ inline tile_info decode_tile(const prefill_params &p, uint32_t idx)
{
    tile_info t;
    t.valid = 0; t.nblk = 0; t.kvh = 0; t.pad = 0;
    t.head[0] = t.head[1] = 0; t.qt[0] = t.qt[1] = 0;
    if (idx >= p.n_tiles) return t;
    t.valid = 1;
    const uint32_t per = tiles_per_qpair(p.n_kv, p.group), pairs = p.group / 2u, odd = p.group & 1u;
    const uint32_t k = idx / per;                    // query-tile pair, counted from the end of the prompt
    uint32_t r = idx % per;
    const int r1 = (int)p.n_qtiles - 1 - 2 * (int)k, r0 = r1 - 1;
    if (odd && r < p.n_kv) {                         // the odd head of group r over both query tiles
        t.kvh = r;
        t.head[0] = t.head[1] = r * p.group + p.group - 1;
        if (r0 >= 0) { t.nblk = 2; t.qt[0] = (uint32_t)r0; t.qt[1] = (uint32_t)r1; }
        else { t.nblk = 1; t.qt[0] = (uint32_t)r1; }
        return t;
    }
    r -= odd * p.n_kv;
    // (a lone first query tile has only the "r1" half of the list)
    const uint32_t qt = (r < p.n_kv * pairs || r0 < 0) ? (uint32_t)r1 : (uint32_t)r0;
    r %= p.n_kv * pairs;
    t.kvh = r / pairs;
    t.nblk = 2;
    t.head[0] = t.kvh * p.group + 2u * (r % pairs);
    t.head[1] = t.head[0] + 1;
    t.qt[0] = t.qt[1] = qt;
    return t;
}

// Key-step range [lo, hi) of a block, in steps of kBN keys.
struct block_range {
    uint32_t tok0, rows, key_end, lo, hi;
};
__device__ __forceinline__ block_range range_of(const prefill_params &p, uint32_t qt)
{
    block_range b;
    b.tok0 = qt * kBM;
    b.rows = min((uint32_t)kBM, p.n - b.tok0);
    b.key_end = p.p0 + b.tok0 + b.rows;
    uint32_t key_first = 0;
    if (p.window > 0 && p.p0 + b.tok0 + 1 > p.window) key_first = p.p0 + b.tok0 + 1 - p.window;
    b.lo = key_first / kBN;
    b.hi = (b.key_end + kBN - 1) / kBN;
    return b;
}

// ---- the kernel ------------------------------------------------------------

__global__ void __launch_bounds__(kThreads, 1)
attn_prefill_hd128_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap o_map,
                          const prefill_params p)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    smem_layout &sm = *reinterpret_cast<smem_layout *>(smem_raw);
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#ifdef WR_PREFILL_TIMELINE
    if (tid == 0 && p.tl && blockIdx.x < kTlCtas) p.tl[kTlRoles * kTlEvents + blockIdx.x * 4] = tl_ns();
#endif
    // The next kernel in the stream may be scheduled now; this kernel's own set-up (barriers, TMEM)
    // overlaps the kernel before it.  What that kernel may still be writing — Q, the cache rows
    // appended for this prompt, the work counter, the output rows — is touched after pdl_wait();
    // with p.early (the kernel before is a prefill launch too: a reader) the first tile's loads
    // and arithmetic do not wait, only the counter and the output stores do.
    pdl_trigger();

    if (warp == 8 && lane == 0) {
        mbar_init(&sm.q_full[0], 1);
        mbar_init(&sm.q_full[1], 1);
        mbar_init(&sm.q_free[0], 1);
        mbar_init(&sm.q_free[1], 1);
        for (int i = 0; i < kStages; ++i) {
            mbar_init(&sm.k_full[i], 1);
            mbar_init(&sm.k_free[i], 1);
            mbar_init(&sm.v_full[i], 1);
            mbar_init(&sm.v_free[i], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&sm.s_full[b], 1);
            mbar_init(&sm.p_full[b], 4);
            mbar_init(&sm.o_done[b], 1);
            mbar_init(&sm.o_free[b], 4);
        }
        for (int i = 0; i < kTileSlots; ++i) mbar_init(&sm.tile_ready[i], 1);
        fence_barrier_init();
        if (!p.early) pdl_wait();
        // The first tile's first loads (Q of block 0, the first K tile, Q of block 1) start
        // at once: they fly while TMEM is allocated and the other warps reach the barrier.
        const tile_info ti = decode_tile(p, blockIdx.x);
        const block_range r0 = range_of(p, ti.qt[0]), r1 = range_of(p, ti.qt[ti.nblk - 1]);
        const uint32_t lo = min(r0.lo, r1.lo);
        const uint32_t n_pages_all = (p.p0 + p.n + 63u) / 64u;
        for (uint32_t b = 0; b < ti.nblk; ++b) {
            mbar_expect_tx(&sm.q_full[b], kQBytes);
            tma_load_2d(sm.q[b], &q_map, (int)(ti.head[b] * kHd), (int)(ti.qt[b] * kBM), &sm.q_full[b]);
            tma_load_2d(sm.q[b] + kQHalfBytes, &q_map, (int)(ti.head[b] * kHd + 64), (int)(ti.qt[b] * kBM), &sm.q_full[b]);
            if (b == 0) {
                const uint32_t n_pg = (2 * lo + 1 < n_pages_all) ? 2u : 1u;
                mbar_expect_tx(&sm.k_full[0], n_pg * kPageBlock);
                for (uint32_t pg = 0; pg < n_pg; ++pg) {
                    const char *src = (p.page_base ? p.page_base + (uint64_t)(2 * lo + pg) * p.page_bytes
                                                   : (const char *)p.pages[2 * lo + pg]) + wr_block_off(ti.kvh, 0, kHd);
                    bulk_g2s(sm.k[0] + pg * 8192, src, 8192, &sm.k_full[0]);
                    bulk_g2s(sm.k[0] + kQHalfBytes + pg * 8192, src + 8192, 8192, &sm.k_full[0]);
                }
            }
        }
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&sm.tmem_base)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;
    const long long limit = p.wait_limit;
    const uint32_t n_pages_total = (p.p0 + p.n + 63u) / 64u;     // pages that hold rows of this prompt

    auto page_ptr = [&](uint32_t t) -> const char * {
        return p.page_base ? p.page_base + (uint64_t)t * p.page_bytes : (const char *)p.pages[t];
    };
    // Work tile number `it` of this CTA: the first one is the CTA's own number (every
    // role works it out for itself, nobody waits), later ones are published by the producer.
    auto tile_of = [&](uint32_t it, bool &ok) -> tile_info {
        if (it == 0) return decode_tile(p, blockIdx.x);
        const uint32_t slot = it % kTileSlots;
        ok = mbar_wait(&sm.tile_ready[slot], ((it - 1) / kTileSlots) & 1, limit);
        if (!ok) return decode_tile(p, p.n_tiles);                   // (invalid)
        return sm.tile[slot];
    };

    if (warp == 8) {
        // ---------------------------------------------------------- producer warp
        // lane 0: work tiles, Q and K tiles; lane 1: V tiles (a K tile is free
        // again long before its V tile is, so the two rings run independently).
        if (lane == 0) {
            uint32_t kcount = 0;
            uint32_t q_loads[2] = {0, 0};                        // Q blocks requested per buffer
            tile_info ti = decode_tile(p, blockIdx.x);
            bool ok = true;
            for (uint32_t it = 0; ok && ti.valid; ++it) {
                const block_range r0 = range_of(p, ti.qt[0]), r1 = range_of(p, ti.qt[ti.nblk - 1]);
                const uint32_t lo = min(r0.lo, r1.lo), hi = max(r0.hi, r1.hi);
                // (a block's buffer is free again when the block's last scores of the tile before have
                // completed — block 0's come half a step before block 1's)
                auto load_q = [&](uint32_t b, uint32_t head, uint32_t qt) -> bool {
                    if (q_loads[b] > 0 && !mbar_wait(&sm.q_free[b], (q_loads[b] - 1) & 1, limit)) return false;
                    ++q_loads[b];
                    mbar_expect_tx(&sm.q_full[b], kQBytes);
                    tma_load_2d(sm.q[b], &q_map, (int)(head * kHd), (int)(qt * kBM), &sm.q_full[b]);
                    tma_load_2d(sm.q[b] + kQHalfBytes, &q_map, (int)(head * kHd + 64), (int)(qt * kBM), &sm.q_full[b]);
                    return true;
                };
                auto load_k = [&](uint32_t j) -> bool {
                    const uint32_t st = kcount % kStages;
                    if (kcount >= kStages && !mbar_wait(&sm.k_free[st], ((kcount / kStages) - 1) & 1, limit)) return false;
                    // [64-dim half][128 keys][128 B]: each page contributes 64 keys to each half
                    const uint32_t n_pg = (2 * j + 1 < n_pages_total) ? 2u : 1u;
                    mbar_expect_tx(&sm.k_full[st], n_pg * kPageBlock);
                    for (uint32_t pg = 0; pg < n_pg; ++pg) {
                        const char *src = page_ptr(2 * j + pg) + wr_block_off(ti.kvh, 0, kHd);
                        bulk_g2s(sm.k[st] + pg * 8192, src, 8192, &sm.k_full[st]);
                        bulk_g2s(sm.k[st] + kQHalfBytes + pg * 8192, src + 8192, 8192, &sm.k_full[st]);
                    }
                    ++kcount;
                    return true;
                };
                // what the first scores need goes first: Q of block 0, the first K tile, Q of block 1
                // (the CTA's first tile had these issued before the CTA-wide barrier)
                if (it > 0) {
                    ok = load_q(0, ti.head[0], ti.qt[0]);
                    ok = ok && load_k(lo);
                    if (ti.nblk > 1) ok = ok && load_q(1, ti.head[1], ti.qt[1]);
                } else {
                    kcount = 1;
                    q_loads[0] = 1;
                    q_loads[1] = ti.nblk > 1 ? 1u : 0u;
                }
                // The next tile is claimed late — when this tile's last K tile is being
                // requested, a step or two before its end — so that the tiles still unclaimed
                // go to the CTAs that really finish first; claimed at the start, every CTA
                // would hold its second tile before it had done any work.
                uint32_t next_tile = 0;
                bool claimed = false;
                for (uint32_t j = lo + 1; j < hi && ok; ++j) {
                    if (!claimed && j + 1 >= hi) {
                        pdl_wait();                              // the counter is the earlier launch's until it has ended
                        next_tile = gridDim.x + (uint32_t)atomicAdd(p.sched, 1);
                        claimed = true;
                    }
                    ok = load_k(j);
                }
                if (!ok) break;
                if (!claimed) {
                    pdl_wait();
                    next_tile = gridDim.x + (uint32_t)atomicAdd(p.sched, 1);
                }
                ti = decode_tile(p, next_tile);
                const uint32_t slot = (it + 1) % kTileSlots;
                sm.tile[slot] = ti;
                mbar_arrive(&sm.tile_ready[slot]);               // (release: the tile is visible to the waiters)
            }
            if (!ok) atomicCAS(p.err, 0, 11);
#ifdef WR_PREFILL_TIMELINE
            if (p.tl && blockIdx.x < kTlCtas) p.tl[kTlRoles * kTlEvents + blockIdx.x * 4 + 3] = kcount;
#endif
        } else if (lane == 1) {
            if (!p.early) pdl_wait();
            uint32_t vcount = 0;
            bool ok = true;
            for (uint32_t it = 0; ok; ++it) {
                const tile_info ti = tile_of(it, ok);
                if (!ok || !ti.valid) break;
                const block_range r0 = range_of(p, ti.qt[0]), r1 = range_of(p, ti.qt[ti.nblk - 1]);
                const uint32_t lo = min(r0.lo, r1.lo), hi = max(r0.hi, r1.hi);
                for (uint32_t j = lo; j < hi && ok; ++j, ++vcount) {
                    const uint32_t st = vcount % kStages;
                    if (vcount >= kStages) {
                        ok = mbar_wait(&sm.v_free[st], ((vcount / kStages) - 1) & 1, limit);
                        if (!ok) break;
                    }
                    const uint32_t n_pg = (2 * j + 1 < n_pages_total) ? 2u : 1u;
                    mbar_expect_tx(&sm.v_full[st], n_pg * kPageBlock);
                    for (uint32_t pg = 0; pg < n_pg; ++pg)
                        bulk_g2s(sm.v[st] + pg * kPageBlock, page_ptr(2 * j + pg) + wr_block_off(ti.kvh, 1, kHd),
                                 kPageBlock, &sm.v_full[st]);
                }
            }
            if (!ok) atomicCAS(p.err, 0, 14);
        }
    } else if (warp == 9) {
        // ------------------------------------------------ MMA warp
        // The whole warp runs this control flow and works the operands out; one
        // elected lane issues the tensor-core instructions, and only the
        // instruction itself is predicated.  (Issued from a branch that only one
        // lane takes, operand arithmetic included, every value has to be moved out
        // of that lane's registers one instruction at a time, in competition with
        // the softmax warps for issue slots: measured 100-220 clk per instruction
        // against 64 this way.)
        const bool lead = elect_one();
        const uint32_t idesc_s = umma_idesc(kBM, kBN, false);
        const uint32_t idesc_o = umma_idesc(kBM, kHd, true);
        // descriptor words: the high word is fixed per operand kind, an operand is
        // selected by adding its byte offset (>>4) to the address field of the low word
        const uint64_t kmaj0 = umma_desc(0, 16, 1024), mnmaj0 = umma_desc(0, 8192, 1024);
        const uint32_t kmaj_hi = (uint32_t)(kmaj0 >> 32), kmaj_lo = (uint32_t)kmaj0;
        const uint32_t mnmaj_hi = (uint32_t)(mnmaj0 >> 32), mnmaj_lo = (uint32_t)mnmaj0;
        const uint32_t q_lo0 = kmaj_lo | ((smem_u32(sm.q[0]) & 0x3FFFFu) >> 4);
        const uint32_t k_lo0 = kmaj_lo | ((smem_u32(sm.k[0]) & 0x3FFFFu) >> 4);
        const uint32_t v_lo0 = mnmaj_lo | ((smem_u32(sm.v[0]) & 0x3FFFFu) >> 4);
        // ring positions advance by one per step; parity flips when a ring wraps
        uint32_t k_st = 0, k_par = 0;            // K stage / parity of the next step to score
        uint32_t v_st = 0, v_par = 0;            // V stage / parity of the next step to multiply
        uint32_t p_uses0 = 0, p_uses1 = 0;       // P hand-offs seen per block
        uint32_t o_uses0 = 0, o_uses1 = 0;       // work tiles finished per block
        uint32_t q_uses0 = 0, q_uses1 = 0;       // Q tiles seen per block
        bool ok = true;
        TL_DECL;
        // S_b = Q_b . K^T for the K tile in stage st
        auto issue_s = [&](uint32_t b, uint32_t st) {
            const uint32_t q_lo = q_lo0 + b * (kQBytes >> 4), k_lo = k_lo0 + st * (kKVTile >> 4);
            const uint32_t d = tmem + kTmemS + 128 * b;
#pragma unroll
            for (int kk = 0; kk < kHd / 16; ++kk) {
                const uint32_t off = ((kk >> 2) * kQHalfBytes + (kk & 3) * 32) >> 4;
                if (lead) umma_ss(d, q_lo + off, kmaj_hi, k_lo + off, kmaj_hi, idesc_s, kk > 0);
            }
            if (lead) umma_commit(&sm.s_full[b]);
        };
        // O_b (+)= P_b . V for the V tile in stage st, n_kk steps of 16 keys
        auto issue_pv = [&](uint32_t b, uint32_t st, uint32_t n_kk, bool accumulate) {
            const uint32_t v_lo = v_lo0 + st * (kKVTile >> 4);
            const uint32_t d = tmem + kTmemO + 128 * b, a = tmem + kTmemS + 128 * b;
            if (n_kk == kBN / 16) {
#pragma unroll
                for (int kk = 0; kk < kBN / 16; ++kk)
                    if (lead)
                        umma_ts(d, a + 8 * kk, v_lo + (((kk >> 2) * kPageBlock + (kk & 3) * 2048) >> 4), mnmaj_hi, idesc_o,
                                accumulate || kk > 0);
            } else {
                for (uint32_t kk = 0; kk < n_kk; ++kk)
                    if (lead)
                        umma_ts(d, a + 8 * kk, v_lo + (((kk >> 2) * kPageBlock + (kk & 3) * 2048) >> 4), mnmaj_hi, idesc_o,
                                accumulate || kk > 0);
            }
        };
        for (uint32_t it = 0; ok; ++it) {
            const tile_info ti = tile_of(it, ok);
            if (!ok || !ti.valid) break;
            const block_range rg0 = range_of(p, ti.qt[0]), rg1 = range_of(p, ti.qt[ti.nblk - 1]);
            const uint32_t lo = min(rg0.lo, rg1.lo), hi = max(rg0.hi, rg1.hi);
            const bool two = ti.nblk > 1;
            const uint32_t lo1 = two ? rg1.lo : hi, hi1 = two ? rg1.hi : hi;     // block 1's steps (none when absent)
            if (lane == 0) TLT(4, 1);                            // tile known

            // first scores of the tile
            ok = mbar_wait(&sm.k_full[k_st], k_par, limit);
            if (ok && lo >= rg0.lo && lo < rg0.hi) ok = mbar_wait(&sm.q_full[0], (q_uses0++) & 1, limit);
            if (!ok) break;
            tc_fence_after();
            if (lo >= rg0.lo && lo < rg0.hi) issue_s(0, k_st);
            if (lead && rg0.hi == lo + 1) umma_commit(&sm.q_free[0]);        // block 0's Q is no longer read
            if (two) {
                ok = mbar_wait(&sm.q_full[1], (q_uses1++) & 1, limit);
                if (!ok) break;
                tc_fence_after();
                if (lo >= lo1 && lo < hi1) issue_s(1, k_st);
                if (lead && hi1 == lo + 1) umma_commit(&sm.q_free[1]);
            }
            if (lead) umma_commit(&sm.k_free[k_st]);
            if (++k_st == kStages) { k_st = 0; k_par ^= 1; }
            if (lane == 0) TLT(4, 2);                            // first scores issued
            for (uint32_t j = lo; j < hi && ok; ++j) {
                const bool more = j + 1 < hi;
                // this step's V tile and the next step's K tile landed long ago
                ok = mbar_wait(&sm.v_full[v_st], v_par, limit);
                if (ok && more) ok = mbar_wait(&sm.k_full[k_st], k_par, limit);
                if (!ok) break;
                // one block: wait for its P, issue its P.V, then its next scores
                auto step_block = [&](uint32_t b, uint32_t blo, uint32_t bhi, uint32_t key_end, uint32_t &p_uses,
                                      uint32_t &o_uses) -> bool {
                    if (j >= blo && j < bhi) {
                        bool good = true;
                        // the first P.V of a tile overwrites O: the previous tile's rows must have left TMEM
                        if (j == blo && o_uses > 0) good = mbar_wait(&sm.o_free[b], (o_uses - 1) & 1, limit);
                        const bool last = (j + 1 == bhi);
                        // steps of 16 keys; the last tile stops at the block's last key
                        const uint32_t n_kk = last ? (key_end - j * kBN + 15u) / 16u : (uint32_t)(kBN / 16);
                        if (good) good = mbar_wait(&sm.p_full[b], p_uses & 1, limit);
                        ++p_uses;
                        if (!good) return false;
                        if (lane == 0) TL(2);                    // P seen
                        tc_fence_after();
                        issue_pv(b, v_st, n_kk, j > blo);
                        if (last) {
                            if (lead) umma_commit(&sm.o_done[b]);
                            ++o_uses;
                        }
                    }
                    if (more && j + 1 >= blo && j + 1 < bhi) {
                        issue_s(b, k_st);                        // (P_b of step j was consumed just above)
                        if (lead && j + 2 == bhi) umma_commit(&sm.q_free[b]);       // the block's last scores
                    }
                    if (lane == 0) TL(2);                        // P.V and next scores issued
                    return true;
                };
                ok = step_block(0, rg0.lo, rg0.hi, rg0.key_end, p_uses0, o_uses0);
                if (ok && two) ok = step_block(1, lo1, hi1, rg1.key_end, p_uses1, o_uses1);
                if (!ok) break;
                if (lead) {
                    umma_commit(&sm.v_free[v_st]);
                    if (more) umma_commit(&sm.k_free[k_st]);
                }
                if (++v_st == kStages) { v_st = 0; v_par ^= 1; }
                if (more && ++k_st == kStages) { k_st = 0; k_par ^= 1; }
            }
            if (lane == 0) TLT(4, 3);                            // last P.V issued
        }
        if (!ok && lane == 0) atomicCAS(p.err, 0, 12);
    } else {
        // ----------------------------- softmax warpgroup b: one thread per query row
        const uint32_t b = warp >> 2;
        const uint32_t row = tid & (kGroupThreads - 1);     // TMEM lane
        const uint32_t wq = warp & 3u;
        const uint32_t lane_base = (wq * 32u) << 16;
        const uint32_t s_addr = tmem + lane_base + kTmemS + 128 * b;
        const uint32_t o_addr = tmem + lane_base + kTmemO + 128 * b;
        const float c2 = p.scale_log2;
        uint32_t s_uses = 0, o_uses = 0, vc = 0;
        bool ok = true;
        TL_DECL;
#ifdef WR_PREFILL_TIMELINE
        const bool tl_me = (lane == 0 && wq == 0);
#define TLS() do { if (tl_me) TL(b); } while (0)
#define TLST(tag) do { if (tl_me && b == 0) TLT(3, tag); } while (0)
#else
#define TLS()
#define TLST(tag)
#endif
        for (uint32_t it = 0; ok; ++it) {
            const tile_info ti = tile_of(it, ok);
            if (!ok || !ti.valid) break;
            const block_range rg0 = range_of(p, ti.qt[0]), rg1 = range_of(p, ti.qt[ti.nblk - 1]);
            const uint32_t lo = min(rg0.lo, rg1.lo), hi = max(rg0.hi, rg1.hi);
            if (b >= ti.nblk) {                              // a lone block: this group sits the tile out
                vc += hi - lo;
                continue;
            }
            const block_range me = (b == 0) ? rg0 : rg1;
            const uint32_t head = (b == 0) ? ti.head[0] : ti.head[1];
            TLST(1);                                             // tile known
            const uint32_t qpos = p.p0 + me.tok0 + row;      // absolute position of this query
            uint32_t lo_key = 0;
            if (p.window > 0 && qpos + 1 > p.window) lo_key = qpos + 1 - p.window;
            float m_ref = WR_NEG_SENTINEL;                   // reference max, log2 domain
            float l = 0.f;
            for (uint32_t j = me.lo; j < me.hi && ok; ++j) {
                ok = mbar_wait(&sm.s_full[b], s_uses & 1, limit);
                ++s_uses;
                if (!ok) break;
                TLS();                                           // 0: scores ready
                if (j == me.lo) TLST(2);                         // the tile's first scores
                tc_fence_after();
                float s[kBN];
#pragma unroll
                for (int c = 0; c < kBN; c += 32) tmem_ld32_nowait(s_addr + c, s + c);
                tmem_wait_ld();
                const uint32_t key0 = j * kBN;
                // steps that no row's causal or window limit cuts through need no masking
                const bool edge = (key0 + kBN - 1 > p.p0 + me.tok0) || (p.window > 0);
                if (edge) {
                    if (p.window == 0) {
                        // causal limit only: key i of this step is visible iff i <= qpos - key0
                        // (negative for a row that lies before the whole step: nothing visible)
                        const int last_visible = (int)(qpos - key0);
#pragma unroll
                        for (int i = 0; i < kBN; ++i)
                            if (i > last_visible) s[i] = WR_NEG_SENTINEL;
                    } else {
#pragma unroll
                        for (int i = 0; i < kBN; ++i) {
                            const uint32_t key = key0 + i;
                            if (key > qpos || key < lo_key) s[i] = WR_NEG_SENTINEL;
                        }
                    }
                }
                // eight independent chains of three-input maxima
                float mx[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) mx[e] = fmaxf(s[2 * e], s[2 * e + 1]);
#pragma unroll
                for (int i = 16; i < kBN; i += 16)
#pragma unroll
                    for (int e = 0; e < 8; ++e) mx[e] = max3(mx[e], s[i + 2 * e], s[i + 2 * e + 1]);
                const float tmax = fmaxf(max3(mx[0], mx[1], mx[2]), max3(max3(mx[3], mx[4], mx[5]), mx[6], mx[7]));
                // Move the reference max (and rescale O) only when it is far behind.
                // The rescale uses warp-wide TMEM instructions, so the warp decides
                // together; rows that do not need it multiply by one.  O is quiet here:
                // this step's scores were issued behind the previous step's P.V, so that
                // P.V has completed, and the next one waits for the P written below.
                const float tm2 = tmax * c2;
                const bool grow = (tmax > WR_NEG_SENTINEL) && (m_ref != WR_NEG_SENTINEL) && (tm2 > m_ref + kRescaleLog2);
                if (tmax > WR_NEG_SENTINEL && m_ref == WR_NEG_SENTINEL) m_ref = tm2;
                if (__any_sync(0xffffffffu, grow)) {
                    const float a = grow ? ex2_approx(m_ref - tm2) : 1.0f;
#pragma unroll 1
                    for (int c = 0; c < kHd; c += 32) {
                        float o[32];
                        tmem_ld32_nowait(o_addr + c, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int e = 0; e < 32; ++e) o[e] *= a;
                        tmem_st32(o_addr + c, o);
                    }
                    if (grow) {
                        l *= a;
                        m_ref = tm2;
                    }
                }
                TLS();                                           // 1: maximum known
                // P = 2^(s*c2 - m_ref) as F16, two keys per TMEM column, over the first 64 columns of S
                // (no visible key yet for this row: every score is the sentinel and must give 0)
                const float neg_m = (m_ref == WR_NEG_SENTINEL) ? 0.f : -m_ref;
                const uint64_t c2_2 = pack2(c2, c2), neg_m2 = pack2(neg_m, neg_m);
                uint64_t psum2[2] = {pack2(0.f, 0.f), pack2(0.f, 0.f)};
#pragma unroll
                for (int c = 0; c < kBN / 32; ++c) {
                    uint32_t w[16];
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        // a masked score is -1e30: the fused multiply-add stays hugely negative, 2^x gives 0
                        const uint64_t x2 = fma2(pack2(s[c * 32 + 2 * e], s[c * 32 + 2 * e + 1]), c2_2, neg_m2);
                        float p0, p1;
                        // one pair in kPolyPeriod goes to the FMA pipe, the others to the special-function unit
                        if (kPolyPeriod > 0 && (e % (kPolyPeriod > 0 ? kPolyPeriod : 1)) == kPolyPeriod - 1) {
                            ex2_poly2(x2, p0, p1);
                        } else {
                            float x0, x1;
                            unpack2(x2, x0, x1);
                            p0 = ex2_approx(x0);
                            p1 = ex2_approx(x1);
                        }
                        psum2[e & 1] = add2(psum2[e & 1], pack2(p0, p1));
                        const __half2 hh = __floats2half2_rn(p0, p1);
                        w[e] = *reinterpret_cast<const uint32_t *>(&hh);
                    }
                    tmem_st16(s_addr + 16 * c, w);
                }
                {
                    float pa, pb, pc, pd;
                    unpack2(psum2[0], pa, pb);
                    unpack2(psum2[1], pc, pd);
                    l += (pa + pb) + (pc + pd);
                }
                TLS();                                           // 2: P stores issued
                if (key0 + kBN > p.p0 + p.n) {
                    // Cache rows past the prompt's last key were never written for it
                    // (or belong to a rolled-back step): clear them in the staged V
                    // tile so that 0 * garbage cannot make a NaN (both groups do it
                    // before releasing their own P.V; the writes are equal).
                    const uint32_t vn = vc + (j - lo), vst = vn % kStages;
                    ok = mbar_wait(&sm.v_full[vst], (vn / kStages) & 1, limit);
                    if (!ok) break;
                    const uint32_t first_bad = p.p0 + p.n - key0;
                    if (row >= first_bad) {
                        uint8_t *vrow = sm.v[vst] + (row >> 6) * kPageBlock + (row & 63u) * 128;
#pragma unroll
                        for (int c = 0; c < 8; ++c) {
                            *reinterpret_cast<uint4 *>(vrow + c * 16) = make_uint4(0, 0, 0, 0);
                            *reinterpret_cast<uint4 *>(vrow + 8192 + c * 16) = make_uint4(0, 0, 0, 0);
                        }
                    }
                    fence_proxy_async();          // generic writes -> tensor-core reads
                }
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                // (a warp cannot arrive twice in one phase: its next scores are issued
                // behind the P.V that waits for all four arrivals of this one)
                if (lane == 0) mbar_arrive(&sm.p_full[b]);
                TLS();                                           // 3: P handed over
                if (j + 1 == me.hi) TLST(3);                     // the tile's last P
            }
            vc += hi - lo;
            if (!ok) break;
            // ---- the tile's last P.V has completed: O leaves TMEM, normalised
            ok = mbar_wait(&sm.o_done[b], o_uses & 1, limit);
            ++o_uses;
            if (!ok) break;
            tc_fence_after();
            TLST(4);                                             // last P.V complete
            float o[kHd];
#pragma unroll
            for (int c = 0; c < kHd; c += 32) tmem_ld32_nowait(o_addr + c, o + c);
            tmem_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.o_free[b]);       // the next tile may overwrite O
            // A thread holds one row, and a store instruction in which every lane writes to a row of
            // its own touches 32 cache lines for 512 bytes (measured: 6500 clk to get a tile's 128 KB
            // out, with every shared-memory access of the CTA queued behind it).  So the warp puts
            // pieces of 32 rows x 16 values into shared memory, swizzled, and the TMA unit writes them
            // out as whole sectors (rows past the prompt are outside the tensor and dropped).  Two
            // buffers take turns: a piece is waited for only when its buffer is needed again.
            pdl_wait();                                      // output rows: after the earlier kernels have ended
            {
                const float inv = (l > 0.f) ? 1.0f / l : 0.f;
                const bool send = (lane == 0) && (wq * 32u < me.rows);   // (a piece wholly past the prompt is not sent)
#pragma unroll
                for (int c = 0; c < kHd / 16; ++c) {
                    uint8_t *stage = sm.out_stage[warp][c & 1];
                    if (lane == 0) tma_store_wait_read<1>();     // the piece before the last has left this buffer
                    __syncwarp();
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        *reinterpret_cast<float4 *>(stage + lane * 64 + ((k ^ ((lane >> 1) & 3u)) << 4)) =
                            make_float4(o[16 * c + 4 * k] * inv, o[16 * c + 4 * k + 1] * inv, o[16 * c + 4 * k + 2] * inv,
                                        o[16 * c + 4 * k + 3] * inv);
                    fence_proxy_async();                         // generic writes -> the TMA unit's reads
                    __syncwarp();
                    if (send) tma_store_2d(&o_map, stage, (int)(head * kHd + 16 * c), (int)(me.tok0 + wq * 32u));
                }
            }
            TLST(5);                                             // output rows issued
        }
        if (!ok) atomicCAS(p.err, 0, 13);
        if (lane == 0) tma_store_wait_read<0>();                 // shared memory stays valid until the last piece is read
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols)
                     : "memory");
    }
#ifdef WR_PREFILL_TIMELINE
    if (tid == 0 && p.tl && blockIdx.x < kTlCtas) p.tl[kTlRoles * kTlEvents + blockIdx.x * 4 + 1] = tl_ns();
#endif
    // The last CTA to leave rewinds the work counter for the next launch.
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(p.sched + 1, 1) == (int)gridDim.x - 1) {
            p.sched[0] = 0;
            p.sched[1] = 0;
            __threadfence();
        }
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
    if (!ctx->prefill_sched) {
        WR_CUDA_TRY(cudaMalloc((void **)&ctx->prefill_sched, 2 * sizeof(int)));
        WR_CUDA_TRY(cudaMemsetAsync(ctx->prefill_sched, 0, 2 * sizeof(int), ctx->stream));
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

    // output rows [n][n_q * 128] F32, written in pieces of 32 rows x 16 values
    CUtensorMap o_map;
    const cuuint64_t o_strides[1] = {(cuuint64_t)n_q_heads * kHd * 4};
    const cuuint32_t o_box[2] = {16, 32};
    if (encode(&o_map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void *)dout, dims, o_strides, o_box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return WR_CUDA_ERR_INTERNAL;

    prefill_params p;
    p.pages = kv->d_pages + (size_t)layer * kv->n_pages;
    p.page_base = kv->contig[layer] ? (const char *)kv->pages[(size_t)layer * kv->n_pages] : nullptr;
    p.page_bytes = wr_page_bytes(kv->n_kv, kHd);
#ifdef WR_PREFILL_TIMELINE
    if (!ctx->debug_buf) {
        WR_CUDA_TRY(cudaMalloc(&ctx->debug_buf, (kTlRoles * kTlEvents + 4 * kTlCtas) * sizeof(long long)));
    }
    WR_CUDA_TRY(cudaMemsetAsync(ctx->debug_buf, 0, (kTlRoles * kTlEvents + 4 * kTlCtas) * sizeof(long long), ctx->stream));
    p.tl = (long long *)ctx->debug_buf;
#endif
    p.err = ctx->dev_err;
    p.sched = ctx->prefill_sched;
    p.wait_limit = ctx->wait_limit;
    p.n = n;
    p.p0 = p0;
    p.n_q = n_q_heads;
    p.n_kv = kv->n_kv;
    p.group = n_q_heads / kv->n_kv;
    p.window = window;
    p.n_qtiles = (n + kBM - 1) / kBM;
    p.n_tiles = prefill_tile_count(p.n_qtiles, p.n_kv, p.group);
    const float scale = (scale_override > 0.0f) ? scale_override : 1.0f / sqrtf((float)kHd);   // kernels.c:1457-1459
    p.scale_log2 = scale * kLog2e;
    if (!(ctx->attr_flags & 2u)) {
        WR_CUDA_TRY(cudaFuncSetAttribute(attn_prefill_hd128_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)sizeof(smem_layout)));
        ctx->attr_flags |= 2u;
    }
    const uint32_t grid = std::min<uint32_t>(p.n_tiles, (uint32_t)ctx->sm_count);
    // Back-to-back prefill launches (nothing of this library's in between, Q taken as given): the
    // earlier one only reads, and with one CTA per SM a CTA of this launch starts where one of the
    // earlier launch has left, so its first tile need not wait for the stragglers.
    const bool full = grid == (uint32_t)ctx->sm_count;
    p.early = (!convert && !host && full && ctx->pdl_index == ctx->launches &&
               ctx->pdl_kind == WR_PDL_PREFILL_FULL) ? 1u : 0u;
    WR_CUDA_TRY(wr_launch_pdl(attn_prefill_hd128_kernel, dim3(grid), dim3(kThreads), sizeof(smem_layout), ctx->stream,
                              q_map, o_map, p));
    ctx->launches++;
    ctx->pdl_kind = full ? WR_PDL_PREFILL_FULL : WR_PDL_NONE;
    ctx->pdl_index = ctx->launches;
    WR_CUDA_TRY(cudaGetLastError());
    if (host) {
        WR_CUDA_TRY(cudaMemcpyAsync(out, dout, out_bytes, cudaMemcpyDeviceToHost, ctx->stream));
        return wr_ctx_sync_checked(ctx);
    }
    return WR_CUDA_OK;
}

#ifdef WR_PREFILL_TIMELINE
// Copies the last launch's stamps out: kTlRoles x kTlEvents int64 values (0 = unused).
extern "C" int wr_cuda_debug_prefill_timeline(wr_cuda_ctx *ctx, long long *host_out, uint32_t n)
{
    if (!ctx || !host_out || !ctx->debug_buf) return WR_CUDA_ERR_INVAL;
    std::lock_guard<std::mutex> g(ctx->lock);
    WR_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    const size_t want = std::min<size_t>(n, (size_t)kTlRoles * kTlEvents + 4 * kTlCtas) * sizeof(long long);
    WR_CUDA_TRY(cudaMemcpy(host_out, ctx->debug_buf, want, cudaMemcpyDeviceToHost));
    return WR_CUDA_OK;
}
#endif
