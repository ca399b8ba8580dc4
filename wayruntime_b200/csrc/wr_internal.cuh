// wr_internal.cuh — host-side objects and device helpers shared by the
// translation units of libwr_cuda.so.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <vector>

#include "wr_cuda.h"

// ----------------------------------------------------------------- layout
//
// KV page = WR_CUDA_PAGE_TOKENS (64) consecutive tokens of one layer, all KV
// heads.  Inside a page: [kv_head][K|V] blocks of 64*head_dim F16.
//
// head_dim % 64 == 0 ("tiled" blocks): the block is [head_dim/64][64 tok][64
// dims] with the eight 16-byte chunks of each 128-byte row permuted by
// chunk ^ (tok & 7).  That is the 128-byte-swizzled K-major operand image the
// 5th-gen tensor cores read from shared memory, and it also makes ldmatrix
// rows conflict-free, so one linear bulk copy of a block into shared memory
// serves both the decode and the prefill kernel with no re-layout.
//
// other head_dim ("linear" blocks): [64 tok][pad8(head_dim)] row-major.

constexpr uint32_t kPageTokens = WR_CUDA_PAGE_TOKENS;

__host__ __device__ inline bool wr_tiled(uint32_t hd) { return (hd & 63u) == 0; }
__host__ __device__ inline uint32_t wr_hd_pad(uint32_t hd) { return (hd + 7u) & ~7u; }
__host__ __device__ inline uint32_t wr_block_bytes(uint32_t hd)
{
    return kPageTokens * wr_hd_pad(hd) * 2u;
}
__host__ __device__ inline uint64_t wr_page_bytes(uint32_t n_kv, uint32_t hd)
{
    return (uint64_t)n_kv * 2u * wr_block_bytes(hd);
}
// Byte offset of element (tok, d) inside one (head, K|V) block.
__host__ __device__ inline uint32_t wr_elem_off(uint32_t tok, uint32_t d, uint32_t hd)
{
    if (wr_tiled(hd)) {
        uint32_t half = d >> 6, dd = d & 63u;
        uint32_t chunk = (dd >> 3) ^ (tok & 7u);
        return half * (kPageTokens * 128u) + tok * 128u + chunk * 16u + (dd & 7u) * 2u;
    }
    return (tok * wr_hd_pad(hd) + d) * 2u;
}
// Byte offset of the (head, which) block inside a page; which: 0 = K, 1 = V.
__host__ __device__ inline uint64_t wr_block_off(uint32_t head, uint32_t which, uint32_t hd)
{
    return ((uint64_t)head * 2u + which) * wr_block_bytes(hd);
}

// ------------------------------------------------------------ host objects

struct wr_page_pool {
    uint64_t page_bytes = 0;
    std::vector<void *> slabs;       // cudaMalloc'd regions
    std::vector<void *> free_pages;  // page base pointers
};

struct wr_cuda_ctx {
    int device = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    std::mutex lock;
    uint32_t attn_max_seq = WR_CUDA_ATTN_MAX_SEQ;
    uint64_t launches = 0;
    std::vector<wr_page_pool> pools;
    // split-KV scratch: per-chunk partial triples and per-group arrival tickets
    float *ws = nullptr;
    size_t ws_bytes = 0;
    int *tickets = nullptr;
    size_t ticket_count = 0;
    int *prefill_sched = nullptr;    // prefill kernel: next work tile, CTAs that have left
    void *debug_buf = nullptr;       // development builds only (kernel timelines)
    int *host_err = nullptr;         // error word: page-locked host memory, mapped into the device
    int *dev_err = nullptr;          // its device-side address (what kernels get)
    int last_err = 0;                // the last non-zero error word read back (which wait gave up)
    // staging for WR_CUDA_MEM_HOST calls
    void *stage_dev = nullptr;
    size_t stage_dev_bytes = 0;
    void *stage_host = nullptr;      // pinned
    size_t stage_host_bytes = 0;
    int live_kv = 0;
    uint32_t attr_flags = 0;         // per-device kernel attributes already set
    // SM clock cycles a device-side wait may last before the kernel gives up
    // (wr_cuda_ctx_set_wait_limit); every kernel of the context gets this value.
    long long wait_limit = WR_CUDA_WAIT_LIMIT_DEFAULT;
    // The last kernel this context launched with programmatic dependent launch (pdl_kind), valid
    // while pdl_index == launches (nothing of ours was launched since).
    uint64_t pdl_index = ~0ull;
    int pdl_kind = 0;                // WR_PDL_*
};
enum { WR_PDL_NONE = 0, WR_PDL_APPEND = 1, WR_PDL_DECODE_FULL = 2, WR_PDL_DECODE_PART = 3, WR_PDL_PREFILL_FULL = 4 };

struct wr_cuda_kv {
    wr_cuda_ctx *ctx = nullptr;
    uint32_t n_layers = 0, n_kv = 0, hd = 0, max_ctx = 0, n_pages = 0;
    std::vector<void *> pages;       // n_layers * n_pages page pointers (host copy)
    uint64_t *d_pages = nullptr;     // same table on the device
    std::vector<uint8_t> contig;     // per layer: pages are consecutive in memory
    size_t pool_index = 0;
};

// Kernel-parameter block describing the sessions of one batched launch.
struct wr_batch_desc {
    const uint64_t *pages[WR_CUDA_BATCH_MAX];   // device page table of (session, layer)
    uint32_t seq_len[WR_CUDA_BATCH_MAX];
};

// ------------------------------------------------------------ host helpers

#define WR_CUDA_TRY(expr)                                                   \
    do {                                                                    \
        cudaError_t e__ = (expr);                                           \
        if (e__ != cudaSuccess) {                                           \
            (void)cudaGetLastError();                                       \
            return e__ == cudaErrorMemoryAllocation ? WR_CUDA_ERR_NOMEM     \
                                                    : WR_CUDA_ERR_INTERNAL; \
        }                                                                   \
    } while (0)

// Where a key-sharded decode launch delivers its triples when the exchange is fused into it.
struct wr_decode_xchg {
    float *rows[WR_CUDA_XCHG_MAX_WORLD];       // per rank: this rank's row slot in that rank's buffer
    uint32_t *flag[WR_CUDA_XCHG_MAX_WORLD];    // per rank: this rank's step flag in that rank's buffer
    uint32_t *row_flag[WR_CUDA_XCHG_MAX_WORLD];// per rank: this rank's per-row flags in that rank's buffer
    const float *rows_in;                      // this rank's own buffer: every rank's rows of this step ...
    const uint32_t *row_flag_in;               // ... and their per-row flags, [world][max_rows]
    int *done;
    uint32_t world, step, max_rows;
    bool want_recv;                            // merge in the decode kernel itself where the plan allows it
    bool did_recv;                             // out: it did (no second kernel needed)
};
int wr_decode_validate(wr_cuda_ctx *ctx, uint32_t n_sess, wr_cuda_kv *const *kv, uint32_t layer,
                       const uint32_t *seq_lens, const void *q, const void *out, uint32_t n_q, int mem,
                       int emit_triples);
int wr_decode_launch(wr_cuda_ctx *ctx, uint32_t n_sess, wr_cuda_kv *const *kv, uint32_t layer,
                     const uint32_t *seq_lens, const float *dq, float *dout, uint32_t n_q,
                     float scale_override, uint32_t window, int emit_triples, wr_decode_xchg *xchg,
                     bool early_tiles = false);

int wr_ctx_reserve_stage(wr_cuda_ctx *ctx, size_t dev_bytes, size_t host_bytes);
// Wait for the context's stream and report (and clear) the device-side error
// word: WR_CUDA_ERR_INTERNAL when a kernel gave up on a bounded wait.  Every
// call that synchronises ends with this.  Caller holds ctx->lock.
int wr_ctx_sync_checked(wr_cuda_ctx *ctx);
int wr_ctx_reserve_ws(wr_cuda_ctx *ctx, size_t ws_bytes, size_t tickets);
int wr_kv_batch_check(wr_cuda_ctx *ctx, uint32_t n_sess, wr_cuda_kv *const *kv, uint32_t layer);
int wr_append_validate(wr_cuda_ctx *ctx, uint32_t n_sess, wr_cuda_kv *const *kv, uint32_t layer,
                       const uint32_t *positions, uint32_t n_tokens, const float *k_rows,
                       const float *v_rows, const float *q_rows, uint32_t n_q_heads, int mem);
int wr_append_launch(wr_cuda_ctx *ctx, uint32_t n_sess, wr_cuda_kv *const *kv, uint32_t layer,
                     const uint32_t *positions, uint32_t n_tokens, const float *dk,
                     const float *dv, float *dq, uint32_t n_q_heads, float theta_base,
                     uint32_t n_rot_pairs, uint32_t flags,
                     const float *dq_in /* null: rotate dq in place */);

// One-kernel layer-step for short contexts (attn_step_small.cu): QK-norm, RoPE, append and the
// new token's attention, for sessions of head_dim 128 with at most WR_STEP_SMALL_MAX_KEYS keys.
#define WR_STEP_SMALL_MAX_KEYS 1024u
bool wr_step_small_covers(const wr_cuda_kv *kv, uint32_t n_q_heads, uint32_t position);
int wr_step_small_launch(wr_cuda_ctx *ctx, uint32_t n_sess, wr_cuda_kv *const *kv, uint32_t layer,
                         const uint32_t *positions, float *dq, const float *dk, const float *dv, float *dout,
                         uint32_t n_q_heads, float theta_base, uint32_t n_rot_pairs, const float *q_norm,
                         const float *k_norm, float eps, float scale_override);

// Resolve the device addresses of the allocation-free decode path's scratch
// arrays and set its kernels' attributes, once per device (that device current).
int wr_static_setup(int device);

// Device-side address of a page-locked host buffer (the same pointer under
// unified addressing), or null when `p` is pageable host memory.
const void *wr_host_device_alias(const void *p);

// ---------------------------------------------------------- device helpers

#ifdef __CUDACC__

// Programmatic dependent launch.  A kernel launched with wr_launch_pdl may begin (be scheduled, run
// its prologue) as soon as every CTA of the kernel before it in the stream has executed
// pdl_trigger() or exited; it must execute pdl_wait() before it touches anything an earlier kernel
// may still be reading or writing — the wait returns once the earlier kernels have completed and
// their memory is visible.  Under an ordinary launch both are no-ops.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... Params>
inline cudaError_t wr_launch_pdl(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 const Params &...p)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, p...);
}

// Reference sentinel for "no score yet" / masked keys (src/core/kernels.c:1480).
#define WR_NEG_SENTINEL (-1e30f)

__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
// Adds to the phase's pending byte count without arriving (the arrival comes with a later call).
__device__ __forceinline__ void mbar_expect_tx_only(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait: returns false when the phase did not complete within `limit`
// cycles of SM clock (the context's wait limit; the caller records an error
// and unwinds; nothing in this library spins without a limit).
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, long long limit)
{
    const uint32_t addr = smem_u32(bar);
    long long t0 = 0;                       // the clock is read only once a poll has failed
    for (bool first = true;; first = false) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
        if (first) t0 = clock64();
        else if (clock64() - t0 > limit) return false;
    }
}
// One non-blocking look at a barrier phase.
__device__ __forceinline__ bool mbar_test(uint64_t *bar, uint32_t parity)
{
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}
__device__ __forceinline__ void fence_barrier_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// Linear bulk copy global -> shared through the TMA unit; completion is
// signalled on `bar` as transaction bytes.  Addresses and size are multiples
// of 16 bytes.
__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src, uint32_t bytes,
                                         uint64_t *bar)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst_smem)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// Same copy with an L2 eviction policy: streamed-once data (K/V tiles of a
// decode step) is marked evict-first so that it does not push the small
// re-used data (partials, page tables, queries) out of L2.
__device__ __forceinline__ uint64_t l2_policy_evict_first()
{
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_g2s_hint(void *dst_smem, const void *src, uint32_t bytes,
                                              uint64_t *bar, uint64_t policy)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1], %2, [%3], %4;"
        ::"r"(smem_u32(dst_smem)), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t &r0, uint32_t &r1, uint32_t &r2,
                                            uint32_t &r3, uint32_t addr)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t &r0, uint32_t &r1, uint32_t &r2,
                                                  uint32_t &r3, uint32_t addr)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
// D(16x8,f32) += A(16x16,f16,row) * B(16x8,f16,col)
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                          uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Split an F32 pair into F16 (hi, lo) pairs with hi + lo ~= x to ~2^-22.
__device__ __forceinline__ void split_half2(float x, float y, uint32_t &hi, uint32_t &lo)
{
    __half2 h = __floats2half2_rn(x, y);
    float2 hf = __half22float2(h);
    __half2 l = __floats2half2_rn(x - hf.x, y - hf.y);
    hi = *reinterpret_cast<uint32_t *>(&h);
    lo = *reinterpret_cast<uint32_t *>(&l);
}

// Cross-rank merge of one row's (m, l, o) triples, rank order, for output elements 4c .. 4c+3: the
// reference's online-softmax update (src/core/kernels.c:1503-1506) across shards.  One function for
// every kernel that merges, so that they all give the same bits.  rows: [world][max_rows][4 + hd].
__device__ __forceinline__ float4 wr_merge_ranks(const float *rows, uint32_t world, uint32_t max_rows,
                                                 uint32_t stride, uint32_t row, uint32_t c)
{
    float mstar = WR_NEG_SENTINEL;
    for (uint32_t g = 0; g < world; ++g)
        mstar = fmaxf(mstar, __ldcg(rows + ((size_t)g * max_rows + row) * stride));
    float L = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t g = 0; g < world; ++g) {
        const float *tr = rows + ((size_t)g * max_rows + row) * stride;
        const float m = __ldcg(tr);
        const float wgt = (m == WR_NEG_SENTINEL) ? 0.f : __expf(m - mstar);
        L += wgt * __ldcg(tr + 1);
        const float4 o = __ldcg(reinterpret_cast<const float4 *>(tr + WR_CUDA_TRIPLE_PAD) + c);
        acc.x += wgt * o.x; acc.y += wgt * o.y; acc.z += wgt * o.z; acc.w += wgt * o.w;
    }
    float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
    if (L > 0.f) r = make_float4(acc.x / L, acc.y / L, acc.z / L, acc.w / L);
    return r;
}

// The reference's truncating F32 -> F16 (src/core/quant.c:121-136).
__device__ __forceinline__ uint16_t wr_f32_to_f16_trunc(float f)
{
    uint32_t b = __float_as_uint(f);
    uint32_t sign = (b >> 16) & 0x8000u;
    int32_t ex = (int32_t)((b >> 23) & 0xFFu) - 112;
    if (ex <= 0) return (uint16_t)sign;
    if (ex >= 31) return (uint16_t)(sign | 0x7C00u);
    return (uint16_t)(sign | ((uint32_t)ex << 10) | ((b >> 13) & 0x3FFu));
}

#endif  // __CUDACC__
