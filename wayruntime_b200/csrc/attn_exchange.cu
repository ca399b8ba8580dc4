// attn_exchange.cu — all-gather of split-KV partial triples and their merge in
// ONE kernel, over NVLink peer memory.
//
// Key-sharded long-context decode leaves every rank with one (m, l, o) triple
// per (session, q head) for its range of keys (wr_cuda_attn_decode_partial);
// the result is the online-softmax merge of the ranks' triples in rank order
// (the reference's update, src/core/kernels.c:1503-1506, across shards).  The
// library path is an NCCL all-gather followed by wr_cuda_attn_combine: two more
// launches and a collective's latency for 270 KB.  Here each rank's kernel
//   1. stores its own triples into every rank's exchange buffer (plain 16-byte
//      stores to peer memory mapped through CUDA IPC; its own buffer included),
//   2. publishes them: the last CTA to finish sets this rank's flag in every
//      peer's buffer to the step number (one system-scope fence, then relaxed
//      stores that go out together),
//   3. waits — with a time limit — until its own buffer carries every rank's
//      flag for this step (system-scope acquire),
//   4. merges the world's triples from its own buffer into the output rows.
// Buffers and flags are double-buffered by step parity: a rank can be at most
// one step ahead of a peer that still reads the previous step's triples.
// No multicast, no TMA: ordinary loads and stores only.
#include <algorithm>

#include "wr_internal.cuh"

struct wr_cuda_xchg {
    wr_cuda_ctx *ctx = nullptr;
    uint32_t world = 0, rank = 0, max_rows = 0, hd = 0;
    size_t bytes = 0;
    char *local = nullptr;                       // this rank's buffer (cudaMalloc, IPC-exported)
    char *peer[WR_CUDA_XCHG_MAX_WORLD] = {};     // every rank's buffer as mapped here (peer[rank] == local)
    bool opened[WR_CUDA_XCHG_MAX_WORLD] = {};
    int *done = nullptr;                         // CTAs of the current launch that finished storing
    uint32_t step = 0;
    bool connected = false;
};

namespace {

// Buffer of one rank: step flags [2][world] (kFlagBytes), per-row flags [2][world][max_rows], then the
// rows [2][world][max_rows][4 + hd]; the first index is the step's parity.
constexpr size_t kFlagBytes = 1024;
__host__ __device__ inline size_t row_flag_bytes(uint32_t world, uint32_t max_rows)
{
    return (((size_t)2 * world * max_rows * sizeof(uint32_t)) + 255u) & ~(size_t)255u;
}

struct xchg_params {
    char *peer[WR_CUDA_XCHG_MAX_WORLD];
    const float *local_triples;
    float *out;
    int *done;
    int *err;
    uint32_t world, rank, max_rows, hd, n_rows, step, parity;
    uint32_t skip_store;     // the rows were delivered by the decode kernel itself
    long long wait_limit;
};

__device__ __forceinline__ void st_relaxed_sys(uint32_t *addr, uint32_t v)
{
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *addr)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
    return v;
}
__device__ __forceinline__ float *slot_rows(char *buf, uint32_t parity, uint32_t src, const xchg_params &p)
{
    const size_t stride = WR_CUDA_TRIPLE_PAD + p.hd;
    return reinterpret_cast<float *>(buf + kFlagBytes + row_flag_bytes(p.world, p.max_rows)) +
           ((size_t)parity * p.world + src) * p.max_rows * stride;
}
__device__ __forceinline__ uint32_t *slot_flag(char *buf, uint32_t parity, uint32_t src, const xchg_params &p)
{
    return reinterpret_cast<uint32_t *>(buf) + parity * p.world + src;
}

__global__ void __launch_bounds__(256) attn_exchange_combine_kernel(const xchg_params p)
{
    const uint32_t stride = WR_CUDA_TRIPLE_PAD + p.hd;
    const uint32_t row_f4 = stride / 4;
    const uint32_t total_f4 = p.n_rows * row_f4;
    const uint32_t gtid = blockIdx.x * blockDim.x + threadIdx.x, gsize = gridDim.x * blockDim.x;

    __shared__ int s_ok;
    if (!p.skip_store) {
        // 1. this rank's triples into every rank's buffer
        const float4 *src = reinterpret_cast<const float4 *>(p.local_triples);
        for (uint32_t peer = 0; peer < p.world; ++peer) {
            float4 *dst = reinterpret_cast<float4 *>(slot_rows(p.peer[peer], p.parity, p.rank, p));
            for (uint32_t i = gtid; i < total_f4; i += gsize) dst[i] = src[i];
        }
        __threadfence_system();
    }
    __syncthreads();

    // 2. the last CTA to get here publishes the step number to every rank
    if (threadIdx.x == 0) {
        s_ok = 1;
        if (!p.skip_store && atomicAdd(p.done, 1) == (int)gridDim.x - 1) {
            // one fence, then the flags as relaxed stores that travel together (a release per flag
            // would serialise one NVLink round trip per rank)
            __threadfence_system();
            for (uint32_t peer = 0; peer < p.world; ++peer)
                st_relaxed_sys(slot_flag(p.peer[peer], p.parity, p.rank, p), p.step);
            *p.done = 0;                                  // ready for the next launch
        }
    }
    __syncthreads();

    // 3. wait for every rank's triples of this step (bounded)
    if (threadIdx.x < p.world) {
        const uint32_t *flag = slot_flag(p.peer[p.rank], p.parity, threadIdx.x, p);
        const long long t0 = clock64();
        while (ld_acquire_sys(flag) != p.step) {
            if (clock64() - t0 > p.wait_limit) {          // the context's wait limit
                atomicExch(p.err, 21);
                s_ok = 0;
                break;
            }
            __nanosleep(200);
        }
    }
    __syncthreads();
    if (!s_ok) return;

    // 4. merge in rank order: one thread per four output elements
    const uint32_t out_f4 = p.hd / 4;
    const uint32_t total_out = p.n_rows * out_f4;
    const float *rows_in = slot_rows(p.peer[p.rank], p.parity, 0, p);
    for (uint32_t i = gtid; i < total_out; i += gsize) {
        const uint32_t row = i / out_f4, c = i % out_f4;
        reinterpret_cast<float4 *>(p.out)[i] = wr_merge_ranks(rows_in, p.world, p.max_rows, stride, row, c);
    }
}

}  // namespace

extern "C" int wr_cuda_xchg_create(wr_cuda_ctx *ctx, uint32_t world, uint32_t rank, uint32_t max_rows,
                                   uint32_t head_dim, wr_cuda_xchg **out)
{
    if (!ctx || !out) return WR_CUDA_ERR_INVAL;
    *out = nullptr;
    if (world == 0 || world > WR_CUDA_XCHG_MAX_WORLD || rank >= world || max_rows == 0) return WR_CUDA_ERR_INVAL;
    if (head_dim == 0 || head_dim % 4 != 0 || head_dim > 1024) return WR_CUDA_ERR_INVAL;
    std::lock_guard<std::mutex> g(ctx->lock);
    WR_CUDA_TRY(cudaSetDevice(ctx->device));
    wr_cuda_xchg *x = new (std::nothrow) wr_cuda_xchg();
    if (!x) return WR_CUDA_ERR_NOMEM;
    x->ctx = ctx;
    x->world = world;
    x->rank = rank;
    x->max_rows = max_rows;
    x->hd = head_dim;
    x->bytes = kFlagBytes + row_flag_bytes(world, max_rows) +
               (size_t)2 * world * max_rows * (WR_CUDA_TRIPLE_PAD + head_dim) * sizeof(float);
    if (cudaMalloc((void **)&x->local, x->bytes) != cudaSuccess ||
        cudaMalloc((void **)&x->done, sizeof(int)) != cudaSuccess) {
        (void)cudaGetLastError();
        if (x->local) (void)cudaFree(x->local);
        delete x;
        return WR_CUDA_ERR_NOMEM;
    }
    if (cudaMemset(x->local, 0, x->bytes) != cudaSuccess || cudaMemset(x->done, 0, sizeof(int)) != cudaSuccess ||
        cudaDeviceSynchronize() != cudaSuccess) {
        (void)cudaGetLastError();
        (void)cudaFree(x->local);
        (void)cudaFree(x->done);
        delete x;
        return WR_CUDA_ERR_INTERNAL;
    }
    x->peer[rank] = x->local;
    x->connected = (world == 1);
    *out = x;
    return WR_CUDA_OK;
}

extern "C" int wr_cuda_xchg_handle(wr_cuda_xchg *x, void *handle_out)
{
    if (!x || !handle_out) return WR_CUDA_ERR_INVAL;
    static_assert(sizeof(cudaIpcMemHandle_t) <= WR_CUDA_XCHG_HANDLE_BYTES, "handle size");
    std::lock_guard<std::mutex> g(x->ctx->lock);
    WR_CUDA_TRY(cudaSetDevice(x->ctx->device));
    cudaIpcMemHandle_t h;
    WR_CUDA_TRY(cudaIpcGetMemHandle(&h, x->local));
    memset(handle_out, 0, WR_CUDA_XCHG_HANDLE_BYTES);
    memcpy(handle_out, &h, sizeof(h));
    return WR_CUDA_OK;
}

extern "C" int wr_cuda_xchg_connect(wr_cuda_xchg *x, const void *handles)
{
    if (!x || !handles) return WR_CUDA_ERR_INVAL;
    std::lock_guard<std::mutex> g(x->ctx->lock);
    if (x->connected) return WR_CUDA_ERR_STATE;
    WR_CUDA_TRY(cudaSetDevice(x->ctx->device));
    for (uint32_t r = 0; r < x->world; ++r) {
        if (r == x->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, (const char *)handles + (size_t)r * WR_CUDA_XCHG_HANDLE_BYTES, sizeof(h));
        void *ptr = nullptr;
        if (cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            (void)cudaGetLastError();
            return WR_CUDA_ERR_UNSUPPORTED;               // no peer access between these two devices
        }
        x->peer[r] = (char *)ptr;
        x->opened[r] = true;
    }
    x->connected = true;
    return WR_CUDA_OK;
}

extern "C" int wr_cuda_xchg_connect_local(wr_cuda_xchg *x, wr_cuda_xchg *const *all)
{
    if (!x || !all) return WR_CUDA_ERR_INVAL;
    std::lock_guard<std::mutex> g(x->ctx->lock);
    if (x->connected) return WR_CUDA_ERR_STATE;
    for (uint32_t r = 0; r < x->world; ++r) {
        const wr_cuda_xchg *o = all[r];
        if (!o || o->world != x->world || o->rank != r || o->max_rows != x->max_rows || o->hd != x->hd)
            return WR_CUDA_ERR_INVAL;
        if (r == x->rank && o != x) return WR_CUDA_ERR_INVAL;
    }
    for (uint32_t r = 0; r < x->world; ++r) x->peer[r] = all[r]->local;   // same address space: no IPC mapping
    x->connected = true;
    return WR_CUDA_OK;
}

extern "C" void wr_cuda_xchg_destroy(wr_cuda_xchg *x)
{
    if (!x) return;
    {
        std::lock_guard<std::mutex> g(x->ctx->lock);
        (void)cudaSetDevice(x->ctx->device);
        (void)cudaStreamSynchronize(x->ctx->stream);
        for (uint32_t r = 0; r < x->world; ++r)
            if (x->opened[r]) (void)cudaIpcCloseMemHandle(x->peer[r]);
        if (x->local) (void)cudaFree(x->local);
        if (x->done) (void)cudaFree(x->done);
        (void)cudaGetLastError();
    }
    delete x;
}

extern "C" int wr_cuda_attn_exchange_combine(wr_cuda_ctx *ctx, wr_cuda_xchg *x, uint32_t n_rows,
                                             const float *triples, float *out)
{
    if (!ctx || !x || x->ctx != ctx || !triples || !out) return WR_CUDA_ERR_INVAL;
    if (!x->connected) return WR_CUDA_ERR_STATE;
    if (n_rows == 0 || n_rows > x->max_rows) return WR_CUDA_ERR_INVAL;
    if (((uintptr_t)triples | (uintptr_t)out) & 15u) return WR_CUDA_ERR_INVAL;   // rows move as 16-byte vectors
    std::lock_guard<std::mutex> g(ctx->lock);
    WR_CUDA_TRY(cudaSetDevice(ctx->device));
    xchg_params p;
    for (uint32_t r = 0; r < WR_CUDA_XCHG_MAX_WORLD; ++r) p.peer[r] = x->peer[r];
    p.local_triples = triples;
    p.out = out;
    p.done = x->done;
    p.err = ctx->dev_err;
    p.world = x->world;
    p.rank = x->rank;
    p.max_rows = x->max_rows;
    p.hd = x->hd;
    p.n_rows = n_rows;
    p.wait_limit = ctx->wait_limit;
    p.skip_store = 0;
    p.step = ++x->step;
    p.parity = x->step & 1u;
    // few CTAs: every one of them has to be resident while it waits for the peers
    const uint32_t work = n_rows * ((WR_CUDA_TRIPLE_PAD + x->hd) / 4);
    const uint32_t blocks = std::max(1u, std::min((work + 255u) / 256u, (uint32_t)ctx->sm_count / 2u));
    attn_exchange_combine_kernel<<<blocks, 256, 0, ctx->stream>>>(p);
    ctx->launches++;
    WR_CUDA_TRY(cudaGetLastError());
    return WR_CUDA_OK;
}

// Key-sharded decode with the exchange fused into the decode kernel: the warps that finish
// a (session, q head) triple store it straight into every rank's exchange buffer, flag the row
// there, then wait for the same row from every rank and merge — all inside the decode kernel
// when every session of this rank has at least two key chunks.  Otherwise the last warp
// publishes this rank's step flag and a small second kernel waits for every rank's flag and
// merges.  Same result bits as wr_cuda_attn_decode_partial + wr_cuda_attn_exchange_combine.
extern "C" int wr_cuda_attn_decode_exchange(wr_cuda_ctx *ctx, wr_cuda_xchg *x, uint32_t n_sess,
                                            wr_cuda_kv *const *kv, uint32_t layer, const uint32_t *seq_lens,
                                            const float *q, float *out, uint32_t n_q_heads, float scale_override)
{
    if (!ctx || !x || x->ctx != ctx) return WR_CUDA_ERR_INVAL;
    if (!x->connected) return WR_CUDA_ERR_STATE;
    std::lock_guard<std::mutex> g(ctx->lock);
    int rc = wr_decode_validate(ctx, n_sess, kv, layer, seq_lens, q, out, n_q_heads, WR_CUDA_MEM_DEVICE, 1);
    if (rc != WR_CUDA_OK) return rc;
    if (kv[0]->hd != 128 || x->hd != 128) return WR_CUDA_ERR_UNSUPPORTED;      // the fused path is the head_dim-128 kernel's
    const uint32_t n_rows = n_sess * n_q_heads;
    if (n_rows == 0 || n_rows > x->max_rows) return WR_CUDA_ERR_INVAL;
    WR_CUDA_TRY(cudaSetDevice(ctx->device));
    xchg_params p;
    for (uint32_t r = 0; r < WR_CUDA_XCHG_MAX_WORLD; ++r) p.peer[r] = x->peer[r];
    p.local_triples = nullptr;
    p.out = out;
    p.done = x->done;
    p.err = ctx->dev_err;
    p.world = x->world;
    p.rank = x->rank;
    p.max_rows = x->max_rows;
    p.hd = x->hd;
    p.n_rows = n_rows;
    p.wait_limit = ctx->wait_limit;
    p.skip_store = 1;
    p.step = ++x->step;
    p.parity = x->step & 1u;
    wr_decode_xchg dx;
    const size_t stride = WR_CUDA_TRIPLE_PAD + x->hd;
    const size_t rows_off = kFlagBytes + row_flag_bytes(x->world, x->max_rows);
    for (uint32_t w = 0; w < x->world; ++w) {
        dx.rows[w] = reinterpret_cast<float *>(x->peer[w] + rows_off) +
                     ((size_t)p.parity * x->world + x->rank) * x->max_rows * stride;
        dx.flag[w] = reinterpret_cast<uint32_t *>(x->peer[w]) + p.parity * x->world + x->rank;
        dx.row_flag[w] = reinterpret_cast<uint32_t *>(x->peer[w] + kFlagBytes) +
                         ((size_t)p.parity * x->world + x->rank) * x->max_rows;
    }
    dx.rows_in = reinterpret_cast<const float *>(x->local + rows_off) + (size_t)p.parity * x->world * x->max_rows * stride;
    dx.row_flag_in = reinterpret_cast<const uint32_t *>(x->local + kFlagBytes) + (size_t)p.parity * x->world * x->max_rows;
    dx.done = x->done;
    dx.world = x->world;
    dx.step = p.step;
    dx.max_rows = x->max_rows;
    dx.want_recv = true;
    dx.did_recv = false;
    rc = wr_decode_launch(ctx, n_sess, kv, layer, seq_lens, q, out, n_q_heads, scale_override, 0, 1, &dx);
    if (rc != WR_CUDA_OK) return rc;
    // Every session of this rank had at least two chunks: the decode kernel's merge warps have also
    // received the other ranks' rows and written the result; nothing is left for a second kernel.
    if (dx.did_recv) return WR_CUDA_OK;
    const uint32_t work = n_rows * (x->hd / 4);
    const uint32_t blocks = std::max(1u, std::min((work + 255u) / 256u, (uint32_t)ctx->sm_count));
    attn_exchange_combine_kernel<<<blocks, 256, 0, ctx->stream>>>(p);
    ctx->launches++;
    WR_CUDA_TRY(cudaGetLastError());
    return WR_CUDA_OK;
}
