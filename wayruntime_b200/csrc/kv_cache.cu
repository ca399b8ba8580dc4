// kv_cache.cu — context, page pool, the paged F16 KV cache and the fused
// RoPE + KV-append kernel.
//
// Reference behaviour restated here (paths inside the reference project):
//   session_build / wr_session_create   src/core/session.c:640-814
//   kv_append_row                       src/core/session.c:139-154
//   wri_op_rope                         src/core/kernels.c:1356-1412
//   wri_f32_to_f16 (truncating)         src/core/quant.c:121-136
#include <algorithm>
#include <new>

#include "mathx_dev.cuh"
#include "wr_internal.cuh"

// ------------------------------------------------------------------ device

extern "C" int wr_cuda_device_check(int device)
{
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        (void)cudaGetLastError();
        return WR_CUDA_ERR_UNSUPPORTED;
    }
    if (device < 0 || device >= n) return WR_CUDA_ERR_UNSUPPORTED;
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess) {
        (void)cudaGetLastError();
        return WR_CUDA_ERR_UNSUPPORTED;
    }
    return major == 10 ? WR_CUDA_OK : WR_CUDA_ERR_UNSUPPORTED;
}

extern "C" int wr_cuda_ctx_create(int device, wr_cuda_ctx **out)
{
    if (!out) return WR_CUDA_ERR_INVAL;
    *out = nullptr;
    int rc = wr_cuda_device_check(device);
    if (rc != WR_CUDA_OK) return rc;
    WR_CUDA_TRY(cudaSetDevice(device));
    wr_cuda_ctx *ctx = new (std::nothrow) wr_cuda_ctx();
    if (!ctx) return WR_CUDA_ERR_NOMEM;
    ctx->device = device;
    cudaError_t e = cudaDeviceGetAttribute(&ctx->sm_count, cudaDevAttrMultiProcessorCount, device);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
    // The error word lives in page-locked host memory that the device sees too: a kernel that gives
    // up writes it across the bus (rare, and slow is fine), and the host reads it after a
    // synchronisation without a copy operation in the stream.
    if (e == cudaSuccess) e = cudaHostAlloc((void **)&ctx->host_err, sizeof(int), cudaHostAllocPortable | cudaHostAllocMapped);
    if (e == cudaSuccess) {
        *ctx->host_err = 0;
        e = cudaHostGetDevicePointer((void **)&ctx->dev_err, ctx->host_err, 0);
    }
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        wr_cuda_ctx_destroy(ctx);
        return e == cudaErrorMemoryAllocation ? WR_CUDA_ERR_NOMEM : WR_CUDA_ERR_INTERNAL;
    }
    *ctx->host_err = 0;
    // The allocation-free decode entry point keeps its scratch in a __device__
    // array of this library: instantiate it (and its kernels) now, so that its
    // memory is taken at start-up, before the caller sizes the KV pool.
    rc = wr_static_setup(device);
    if (rc != WR_CUDA_OK) {
        wr_cuda_ctx_destroy(ctx);
        return rc;
    }
    *out = ctx;
    return WR_CUDA_OK;
}

extern "C" void wr_cuda_ctx_destroy(wr_cuda_ctx *ctx)
{
    if (!ctx) return;
    (void)cudaSetDevice(ctx->device);
    if (ctx->stream) (void)cudaStreamSynchronize(ctx->stream);
    for (auto &pool : ctx->pools)
        for (void *slab : pool.slabs) (void)cudaFree(slab);
    if (ctx->ws) (void)cudaFree(ctx->ws);
    if (ctx->tickets) (void)cudaFree(ctx->tickets);
    if (ctx->prefill_sched) (void)cudaFree(ctx->prefill_sched);
    if (ctx->debug_buf) (void)cudaFree(ctx->debug_buf);
    if (ctx->host_err) (void)cudaFreeHost(ctx->host_err);       // (dev_err is its device-side alias)
    if (ctx->stage_dev) (void)cudaFree(ctx->stage_dev);
    if (ctx->stage_host) (void)cudaFreeHost(ctx->stage_host);
    if (ctx->stream) (void)cudaStreamDestroy(ctx->stream);
    (void)cudaGetLastError();
    delete ctx;
}

int wr_ctx_sync_checked(wr_cuda_ctx *ctx)
{
    WR_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    const int word = *(volatile int *)ctx->host_err;
    if (word != 0) {
        ctx->last_err = word;
        *(volatile int *)ctx->host_err = 0;
        // A kernel that gave up left its arrival tickets and work queue mid-count.
        if (ctx->tickets)
            WR_CUDA_TRY(cudaMemsetAsync(ctx->tickets, 0, ctx->ticket_count * sizeof(int), ctx->stream));
        if (ctx->prefill_sched)
            WR_CUDA_TRY(cudaMemsetAsync(ctx->prefill_sched, 0, 2 * sizeof(int), ctx->stream));
        WR_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
        return WR_CUDA_ERR_INTERNAL;
    }
    return WR_CUDA_OK;
}

extern "C" int wr_cuda_ctx_sync(wr_cuda_ctx *ctx)
{
    if (!ctx) return WR_CUDA_ERR_INVAL;
    std::lock_guard<std::mutex> g(ctx->lock);
    WR_CUDA_TRY(cudaSetDevice(ctx->device));
    return wr_ctx_sync_checked(ctx);
}

extern "C" int wr_cuda_ctx_last_device_error(wr_cuda_ctx *ctx)
{
    if (!ctx) return 0;
    std::lock_guard<std::mutex> g(ctx->lock);
    return ctx->last_err;
}

extern "C" int wr_cuda_ctx_set_wait_limit(wr_cuda_ctx *ctx, int64_t cycles)
{
    if (!ctx || cycles <= 0) return WR_CUDA_ERR_INVAL;
    std::lock_guard<std::mutex> g(ctx->lock);
    ctx->wait_limit = (long long)cycles;
    return WR_CUDA_OK;
}

extern "C" void *wr_cuda_ctx_stream(wr_cuda_ctx *ctx) { return ctx ? (void *)ctx->stream : nullptr; }

extern "C" int wr_cuda_ctx_set_attn_max_seq(wr_cuda_ctx *ctx, uint32_t max_seq)
{
    if (!ctx || max_seq == 0) return WR_CUDA_ERR_INVAL;
    if (max_seq > WR_CUDA_ATTN_MAX_SEQ_TOP) return WR_CUDA_ERR_LIMIT;
    std::lock_guard<std::mutex> g(ctx->lock);
    ctx->attn_max_seq = max_seq;
    return WR_CUDA_OK;
}

extern "C" int wr_cuda_host_alloc(wr_cuda_ctx *ctx, uint64_t bytes, void **out)
{
    if (!ctx || !out || bytes == 0) return WR_CUDA_ERR_INVAL;
    *out = nullptr;
    std::lock_guard<std::mutex> g(ctx->lock);
    WR_CUDA_TRY(cudaSetDevice(ctx->device));
    void *p = nullptr;
    if (cudaHostAlloc(&p, (size_t)bytes, cudaHostAllocPortable | cudaHostAllocMapped) != cudaSuccess) {
        (void)cudaGetLastError();
        return WR_CUDA_ERR_NOMEM;
    }
    *out = p;
    return WR_CUDA_OK;
}

extern "C" void wr_cuda_host_free(wr_cuda_ctx *ctx, void *p)
{
    if (!ctx || !p) return;
    std::lock_guard<std::mutex> g(ctx->lock);
    (void)cudaSetDevice(ctx->device);
    (void)cudaStreamSynchronize(ctx->stream);      // a kernel may still be reading the rows in place
    (void)cudaFreeHost(p);
    (void)cudaGetLastError();
}

extern "C" uint64_t wr_cuda_ctx_launch_count(wr_cuda_ctx *ctx)
{
    if (!ctx) return 0;
    std::lock_guard<std::mutex> g(ctx->lock);
    return ctx->launches;
}

int wr_ctx_reserve_stage(wr_cuda_ctx *ctx, size_t dev_bytes, size_t host_bytes)
{
    if (dev_bytes > ctx->stage_dev_bytes) {
        WR_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
        if (ctx->stage_dev) (void)cudaFree(ctx->stage_dev);
        ctx->stage_dev = nullptr;
        ctx->stage_dev_bytes = 0;
        size_t want = std::max(dev_bytes, (size_t)1 << 20);
        WR_CUDA_TRY(cudaMalloc(&ctx->stage_dev, want));
        ctx->stage_dev_bytes = want;
    }
    if (host_bytes > ctx->stage_host_bytes) {
        WR_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
        if (ctx->stage_host) (void)cudaFreeHost(ctx->stage_host);
        ctx->stage_host = nullptr;
        ctx->stage_host_bytes = 0;
        size_t want = std::max(host_bytes, (size_t)1 << 20);
        WR_CUDA_TRY(cudaMallocHost(&ctx->stage_host, want));
        ctx->stage_host_bytes = want;
    }
    return WR_CUDA_OK;
}

int wr_ctx_reserve_ws(wr_cuda_ctx *ctx, size_t ws_bytes, size_t tickets)
{
    if (ws_bytes > ctx->ws_bytes) {
        WR_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
        if (ctx->ws) (void)cudaFree(ctx->ws);
        ctx->ws = nullptr;
        ctx->ws_bytes = 0;
        size_t want = std::max(ws_bytes, (size_t)8 << 20);
        WR_CUDA_TRY(cudaMalloc((void **)&ctx->ws, want));
        ctx->ws_bytes = want;
    }
    if (tickets > ctx->ticket_count) {
        WR_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
        if (ctx->tickets) (void)cudaFree(ctx->tickets);
        ctx->tickets = nullptr;
        ctx->ticket_count = 0;
        size_t want = std::max(tickets, (size_t)4096);
        WR_CUDA_TRY(cudaMalloc((void **)&ctx->tickets, want * sizeof(int)));
        // Tickets start at zero; the kernel that consumes a ticket group
        // resets it, so no per-launch clearing is needed.
        WR_CUDA_TRY(cudaMemset(ctx->tickets, 0, want * sizeof(int)));
        ctx->ticket_count = want;
    }
    return WR_CUDA_OK;
}

// -------------------------------------------------------------- page pool

static int pool_take(wr_cuda_ctx *ctx, uint64_t page_bytes, size_t n, size_t *pool_index,
                     std::vector<void *> &out)
{
    size_t pi = 0;
    for (; pi < ctx->pools.size(); ++pi)
        if (ctx->pools[pi].page_bytes == page_bytes) break;
    if (pi == ctx->pools.size()) {
        ctx->pools.emplace_back();
        ctx->pools.back().page_bytes = page_bytes;
    }
    wr_page_pool &pool = ctx->pools[pi];
    if (pool.free_pages.size() < n) {
        size_t need = n - pool.free_pages.size();
        void *slab = nullptr;
        WR_CUDA_TRY(cudaMalloc(&slab, need * page_bytes));
        // Pages start zeroed so that the unwritten tail of a partly filled
        // page holds finite values.
        cudaError_t e = cudaMemsetAsync(slab, 0, need * page_bytes, ctx->stream);
        if (e != cudaSuccess) {
            (void)cudaGetLastError();
            (void)cudaFree(slab);
            return WR_CUDA_ERR_INTERNAL;
        }
        pool.slabs.push_back(slab);
        for (size_t i = need; i-- > 0;)
            pool.free_pages.push_back((char *)slab + i * page_bytes);
    }
    out.assign(pool.free_pages.end() - n, pool.free_pages.end());
    std::reverse(out.begin(), out.end());
    pool.free_pages.resize(pool.free_pages.size() - n);
    *pool_index = pi;
    return WR_CUDA_OK;
}

extern "C" int wr_cuda_kv_create(wr_cuda_ctx *ctx, uint32_t n_layers, uint32_t n_kv_heads,
                                 uint32_t head_dim, uint32_t max_ctx, wr_cuda_kv **out)
{
    if (!ctx || !out) return WR_CUDA_ERR_INVAL;
    *out = nullptr;
    if (n_layers == 0 || n_kv_heads == 0 || head_dim == 0 || max_ctx == 0) return WR_CUDA_ERR_INVAL;
    if (head_dim & 1u) return WR_CUDA_ERR_INVAL;                // RoPE pairs (kernels.c:1366)
    if (head_dim > WR_CUDA_HEAD_DIM_MAX) return WR_CUDA_ERR_LIMIT;
    if (n_layers > 64) return WR_CUDA_ERR_LIMIT;                // WR_MAX_LAYERS (internal.h:184)
    std::lock_guard<std::mutex> g(ctx->lock);
    if (max_ctx > ctx->attn_max_seq) return WR_CUDA_ERR_LIMIT;  // session.c:755
    WR_CUDA_TRY(cudaSetDevice(ctx->device));
    wr_cuda_kv *kv = new (std::nothrow) wr_cuda_kv();
    if (!kv) return WR_CUDA_ERR_NOMEM;
    kv->ctx = ctx;
    kv->n_layers = n_layers;
    kv->n_kv = n_kv_heads;
    kv->hd = head_dim;
    kv->max_ctx = max_ctx;
    kv->n_pages = (max_ctx + kPageTokens - 1) / kPageTokens;
    size_t total = (size_t)n_layers * kv->n_pages;
    int rc = pool_take(ctx, wr_page_bytes(n_kv_heads, head_dim), total, &kv->pool_index, kv->pages);
    if (rc != WR_CUDA_OK) {
        delete kv;
        return rc;
    }
    cudaError_t e = cudaMalloc((void **)&kv->d_pages, total * sizeof(uint64_t));
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(kv->d_pages, kv->pages.data(), total * sizeof(uint64_t),
                            cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        auto &fp = ctx->pools[kv->pool_index].free_pages;
        fp.insert(fp.end(), kv->pages.begin(), kv->pages.end());
        if (kv->d_pages) (void)cudaFree(kv->d_pages);
        delete kv;
        return e == cudaErrorMemoryAllocation ? WR_CUDA_ERR_NOMEM : WR_CUDA_ERR_INTERNAL;
    }
    // A layer whose pages came out of the pool back to back needs no table
    // lookup on the device: page i sits at base + i * page_bytes.
    kv->contig.assign(n_layers, 1);
    const uint64_t pb = wr_page_bytes(n_kv_heads, head_dim);
    for (uint32_t L = 0; L < n_layers; ++L)
        for (uint32_t i = 1; i < kv->n_pages; ++i)
            if ((char *)kv->pages[(size_t)L * kv->n_pages + i] !=
                (char *)kv->pages[(size_t)L * kv->n_pages + i - 1] + pb)
                kv->contig[L] = 0;
    ctx->live_kv++;
    *out = kv;
    return WR_CUDA_OK;
}

extern "C" void wr_cuda_kv_destroy(wr_cuda_kv *kv)
{
    if (!kv) return;
    wr_cuda_ctx *ctx = kv->ctx;
    std::lock_guard<std::mutex> g(ctx->lock);
    (void)cudaSetDevice(ctx->device);
    (void)cudaStreamSynchronize(ctx->stream);
    // Returned pages are cleared again so the next owner starts from zeros.
    for (void *p : kv->pages)
        (void)cudaMemsetAsync(p, 0, ctx->pools[kv->pool_index].page_bytes, ctx->stream);
    auto &fp = ctx->pools[kv->pool_index].free_pages;
    fp.insert(fp.end(), kv->pages.rbegin(), kv->pages.rend());
    (void)cudaStreamSynchronize(ctx->stream);
    if (kv->d_pages) (void)cudaFree(kv->d_pages);
    (void)cudaGetLastError();
    ctx->live_kv--;
    delete kv;
}

extern "C" uint32_t wr_cuda_kv_max_ctx(const wr_cuda_kv *kv) { return kv ? kv->max_ctx : 0; }

int wr_kv_batch_check(wr_cuda_ctx *ctx, uint32_t n_sess, wr_cuda_kv *const *kv, uint32_t layer)
{
    if (!ctx || !kv || n_sess == 0) return WR_CUDA_ERR_INVAL;
    if (n_sess > WR_CUDA_BATCH_MAX) return WR_CUDA_ERR_LIMIT;      // batch.c:128-131
    for (uint32_t s = 0; s < n_sess; ++s) {
        if (!kv[s] || kv[s]->ctx != ctx) return WR_CUDA_ERR_INVAL;
        if (layer >= kv[s]->n_layers) return WR_CUDA_ERR_INVAL;
        if (kv[s]->n_kv != kv[0]->n_kv || kv[s]->hd != kv[0]->hd) return WR_CUDA_ERR_INVAL;
        for (uint32_t t = 0; t < s; ++t)
            if (kv[t] == kv[s]) return WR_CUDA_ERR_INVAL;          // distinct sessions (batch.c:133-137)
    }
    return WR_CUDA_OK;
}

// ------------------------------------------------------- row copy kernels

// One thread per 16-byte chunk (8 dims) of the row-layout buffer.
__global__ void kv_rows_copy_kernel(const uint64_t *__restrict__ pages, uint16_t *rows,
                                    uint32_t row0, uint32_t n, uint32_t n_kv, uint32_t hd,
                                    uint32_t which, int to_cache)
{
    const uint32_t chunks_per_head = wr_hd_pad(hd) / 8u;
    const uint64_t total = (uint64_t)n * n_kv * chunks_per_head;
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < total;
         i += (uint64_t)gridDim.x * blockDim.x) {
        uint32_t c = (uint32_t)(i % chunks_per_head);
        uint64_t rest = i / chunks_per_head;
        uint32_t head = (uint32_t)(rest % n_kv);
        uint32_t r = (uint32_t)(rest / n_kv);
        uint32_t row = row0 + r;
        char *page = (char *)pages[row / kPageTokens];
        char *blk = page + wr_block_off(head, which, hd);
        uint32_t tok = row % kPageTokens;
        uint16_t *rp = rows + ((uint64_t)r * n_kv + head) * hd + c * 8u;
        uint32_t lim = min(8u, hd - c * 8u);
        if (lim == 8u && (hd & 7u) == 0) {
            uint4 *cp = (uint4 *)(blk + wr_elem_off(tok, c * 8u, hd));
            if (to_cache) *cp = *(const uint4 *)rp;
            else *(uint4 *)rp = *cp;
        } else {
            for (uint32_t e = 0; e < lim; ++e) {
                uint16_t *cp = (uint16_t *)(blk + wr_elem_off(tok, c * 8u + e, hd));
                if (to_cache) *cp = rp[e];
                else rp[e] = *cp;
            }
        }
    }
}

static int kv_rows_xfer(wr_cuda_ctx *ctx, wr_cuda_kv *kv, uint32_t layer, int which, uint32_t row0,
                        uint32_t n, uint16_t *buf, int mem, int to_cache)
{
    if (!ctx || !kv || kv->ctx != ctx || !buf) return WR_CUDA_ERR_INVAL;
    if (layer >= kv->n_layers || (which != 0 && which != 1)) return WR_CUDA_ERR_INVAL;
    if (n == 0) return WR_CUDA_OK;
    if ((uint64_t)row0 + n > kv->max_ctx) return WR_CUDA_ERR_CTX_FULL;
    if (mem != WR_CUDA_MEM_HOST && mem != WR_CUDA_MEM_DEVICE) return WR_CUDA_ERR_INVAL;
    // device rows move as 16-byte vectors when head_dim allows it
    if (mem == WR_CUDA_MEM_DEVICE && (kv->hd & 7u) == 0 && ((uintptr_t)buf & 15u)) return WR_CUDA_ERR_INVAL;
    std::lock_guard<std::mutex> g(ctx->lock);
    WR_CUDA_TRY(cudaSetDevice(ctx->device));
    size_t bytes = (size_t)n * kv->n_kv * kv->hd * 2u;
    uint16_t *dbuf = buf;
    if (mem == WR_CUDA_MEM_HOST) {
        int rc = wr_ctx_reserve_stage(ctx, bytes, 0);
        if (rc != WR_CUDA_OK) return rc;
        dbuf = (uint16_t *)ctx->stage_dev;
        if (to_cache)
            WR_CUDA_TRY(cudaMemcpyAsync(dbuf, buf, bytes, cudaMemcpyHostToDevice, ctx->stream));
    }
    uint64_t work = (uint64_t)n * kv->n_kv * (wr_hd_pad(kv->hd) / 8u);
    uint32_t blocks = (uint32_t)std::min<uint64_t>((work + 255) / 256, (uint64_t)ctx->sm_count * 16);
    kv_rows_copy_kernel<<<blocks, 256, 0, ctx->stream>>>(
        kv->d_pages + (size_t)layer * kv->n_pages, dbuf, row0, n, kv->n_kv, kv->hd, (uint32_t)which,
        to_cache);
    ctx->launches++;
    WR_CUDA_TRY(cudaGetLastError());
    if (mem == WR_CUDA_MEM_HOST) {
        if (!to_cache)
            WR_CUDA_TRY(cudaMemcpyAsync(buf, dbuf, bytes, cudaMemcpyDeviceToHost, ctx->stream));
        return wr_ctx_sync_checked(ctx);
    }
    return WR_CUDA_OK;
}

extern "C" int wr_cuda_kv_write_rows(wr_cuda_ctx *ctx, wr_cuda_kv *kv, uint32_t layer, int which,
                                     uint32_t row0, uint32_t n, const uint16_t *src, int mem)
{
    return kv_rows_xfer(ctx, kv, layer, which, row0, n, const_cast<uint16_t *>(src), mem, 1);
}

extern "C" int wr_cuda_kv_read_rows(wr_cuda_ctx *ctx, wr_cuda_kv *kv, uint32_t layer, int which,
                                    uint32_t row0, uint32_t n, uint16_t *dst, int mem)
{
    return kv_rows_xfer(ctx, kv, layer, which, row0, n, dst, mem, 0);
}

const void *wr_host_device_alias(const void *p)
{
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return nullptr;
    }
    if (attr.type != cudaMemoryTypeHost || !attr.devicePointer) return nullptr;
    return attr.devicePointer;
}

// ------------------------------------------------- fused RoPE + KV append

struct append_params {
    wr_batch_desc b;                 // b.seq_len[s] = first row (position) of session s
    const float *k_rows;
    const float *v_rows;
    float *q_rows;                   // rotated Q rows are written here ...
    const float *q_in;               // ... from these rows (the same buffer when rotating in place)
    uint32_t n_sess, n_tokens, n_kv, n_q, hd, n_rot;
    float theta;
    uint32_t rope;
};

// A pair's cos/sin depend only on (position, j): each CTA computes the table
// of its token once and applies it to its share of the heads.
//
// A token's work is split over 1 + ceil(n_q / 8) CTAs: CTA y = 0 of a token
// takes K and V of every KV head, CTA y >= 1 takes eight Q heads.  The kernel
// is latency bound (a few hundred KB per step), so every thread first issues
// the loads of its first (head, pair) items, then the pair angles are
// evaluated (by the first hd/2 threads) while those loads are in flight, and
// only then are the rows rotated and stored.
constexpr int kAppendThreads = 256;
constexpr int kAppendQHeads = 8;          // Q heads per CTA
constexpr int kAppendBatch = 2;           // (head, pair) items per thread whose loads are issued together

__global__ void __launch_bounds__(kAppendThreads) rope_kv_append_kernel(const append_params p)
{
    extern __shared__ float trig[];                              // cs[half], sn[half]
    const uint32_t half = p.hd / 2u;
    const uint32_t tok_idx = blockIdx.x;                         // s * n_tokens + t
    const uint32_t s = tok_idx / p.n_tokens, t = tok_idx % p.n_tokens;
    const uint32_t row = p.b.seq_len[s] + t;                     // absolute position = cache row
    float *cs_tab = trig, *sn_tab = trig + half;
    pdl_trigger();                       // the decode kernel behind this one may be scheduled now
    auto build_table = [&]() {
        if (p.rope) {
            const float ln_theta = wrmath::log_ref(p.theta);
            for (uint32_t j = threadIdx.x; j < p.n_rot; j += blockDim.x) {
                float sn, cs;
                wrmath::rope_angle(row, j, p.hd, ln_theta, sn, cs);
                cs_tab[j] = cs;
                sn_tab[j] = sn;
            }
        }
        __syncthreads();
    };
    constexpr uint32_t kStep = kAppendThreads * kAppendBatch;

    if (blockIdx.y == 0) {
        // ---- K and V rows of this token into the page
        char *page = (char *)p.b.pages[s][row / kPageTokens];
        const uint32_t tk = row % kPageTokens;
        const float *__restrict__ krow = p.k_rows + (size_t)tok_idx * p.n_kv * p.hd;
        const float *__restrict__ vrow = p.v_rows + (size_t)tok_idx * p.n_kv * p.hd;
        const uint32_t work = p.n_kv * half;
        // the pair angles need nothing from earlier kernels: they are evaluated while the kernel
        // before this one is still finishing; the rows are read after it has completed
        build_table();
        bool table_ready = true;
        pdl_wait();
        for (uint32_t base = 0; base < work; base += kStep) {
            float x0[kAppendBatch], x1[kAppendBatch], v0[kAppendBatch], v1[kAppendBatch];
#pragma unroll
            for (int u = 0; u < kAppendBatch; ++u) {
                const uint32_t i = base + u * kAppendThreads + threadIdx.x;
                if (i < work) {
                    const uint32_t h = i / half, j = i % half;
                    x0[u] = krow[h * p.hd + j];
                    x1[u] = krow[h * p.hd + j + half];
                    v0[u] = vrow[h * p.hd + j];
                    v1[u] = vrow[h * p.hd + j + half];
                }
            }
            if (!table_ready) {
                build_table();
                table_ready = true;
            }
#pragma unroll
            for (int u = 0; u < kAppendBatch; ++u) {
                const uint32_t i = base + u * kAppendThreads + threadIdx.x;
                if (i >= work) continue;
                const uint32_t h = i / half, j = i % half;
                float y0 = x0[u], y1 = x1[u];
                if (p.rope && j < p.n_rot) {   // kernels.c:1406-1407, products rounded separately
                    const float cs = cs_tab[j], sn = sn_tab[j];
                    y0 = wrmath::sub(wrmath::mul(x0[u], cs), wrmath::mul(x1[u], sn));
                    y1 = wrmath::add(wrmath::mul(x0[u], sn), wrmath::mul(x1[u], cs));
                }
                const uint32_t off0 = wr_elem_off(tk, j, p.hd), off1 = wr_elem_off(tk, j + half, p.hd);
                char *kb = page + wr_block_off(h, 0, p.hd);
                char *vb = page + wr_block_off(h, 1, p.hd);
                *(uint16_t *)(kb + off0) = wr_f32_to_f16_trunc(y0);
                *(uint16_t *)(kb + off1) = wr_f32_to_f16_trunc(y1);
                *(uint16_t *)(vb + off0) = wr_f32_to_f16_trunc(v0[u]);
                *(uint16_t *)(vb + off1) = wr_f32_to_f16_trunc(v1[u]);
            }
        }
        return;
    }

    // ---- eight Q heads of this token: rotated in place, or from q_in into q_rows
    // (then the pairs beyond n_rot are copied through as well)
    if (!(p.q_rows && p.rope)) return;
    build_table();
    pdl_wait();
    const uint32_t head0 = (blockIdx.y - 1) * kAppendQHeads;
    const uint32_t n_heads = min((uint32_t)kAppendQHeads, p.n_q - head0);
    const size_t qoff = ((size_t)tok_idx * p.n_q + head0) * p.hd;
    float *qrow = p.q_rows + qoff;
    const float *__restrict__ qsrc = p.q_in + qoff;
    const bool in_place = (p.q_in == p.q_rows);
    const uint32_t pairs = in_place ? p.n_rot : half;             // per head
    const uint32_t work = n_heads * pairs;
    bool table_ready = true;
    for (uint32_t base = 0; base < work; base += kStep) {
        float x0[kAppendBatch], x1[kAppendBatch];
#pragma unroll
        for (int u = 0; u < kAppendBatch; ++u) {
            const uint32_t i = base + u * kAppendThreads + threadIdx.x;
            if (i < work) {
                const uint32_t h = i / pairs, j = i % pairs;
                x0[u] = qsrc[h * p.hd + j];
                x1[u] = qsrc[h * p.hd + j + half];
            }
        }
        if (!table_ready) {
            build_table();
            table_ready = true;
        }
#pragma unroll
        for (int u = 0; u < kAppendBatch; ++u) {
            const uint32_t i = base + u * kAppendThreads + threadIdx.x;
            if (i >= work) continue;
            const uint32_t h = i / pairs, j = i % pairs;
            float y0 = x0[u], y1 = x1[u];
            if (j < p.n_rot) {
                const float cs = cs_tab[j], sn = sn_tab[j];
                y0 = wrmath::sub(wrmath::mul(x0[u], cs), wrmath::mul(x1[u], sn));
                y1 = wrmath::add(wrmath::mul(x0[u], sn), wrmath::mul(x1[u], cs));
            }
            qrow[h * p.hd + j] = y0;
            qrow[h * p.hd + j + half] = y1;
        }
    }
}

int wr_append_validate(wr_cuda_ctx *ctx, uint32_t n_sess, wr_cuda_kv *const *kv, uint32_t layer,
                       const uint32_t *positions, uint32_t n_tokens, const float *k_rows,
                       const float *v_rows, const float *q_rows, uint32_t n_q_heads, int mem)
{
    int rc = wr_kv_batch_check(ctx, n_sess, kv, layer);
    if (rc != WR_CUDA_OK) return rc;
    if (!positions || !k_rows || !v_rows) return WR_CUDA_ERR_INVAL;
    if (q_rows && n_q_heads == 0) return WR_CUDA_ERR_INVAL;
    if (mem != WR_CUDA_MEM_HOST && mem != WR_CUDA_MEM_DEVICE) return WR_CUDA_ERR_INVAL;
    for (uint32_t s = 0; s < n_sess; ++s)
        if ((uint64_t)positions[s] + n_tokens > kv[s]->max_ctx) return WR_CUDA_ERR_CTX_FULL;
    return WR_CUDA_OK;
}

// Enqueue the kernel on device-resident rows.  Caller holds ctx->lock and has
// validated the arguments.
int wr_append_launch(wr_cuda_ctx *ctx, uint32_t n_sess, wr_cuda_kv *const *kv, uint32_t layer,
                     const uint32_t *positions, uint32_t n_tokens, const float *dk,
                     const float *dv, float *dq, uint32_t n_q_heads, float theta_base,
                     uint32_t n_rot_pairs, uint32_t flags, const float *dq_in)
{
    append_params p;
    for (uint32_t s = 0; s < n_sess; ++s) {
        p.b.pages[s] = kv[s]->d_pages + (size_t)layer * kv[s]->n_pages;
        p.b.seq_len[s] = positions[s];
    }
    const uint32_t hd = kv[0]->hd, half = hd / 2u;
    p.k_rows = dk;
    p.v_rows = dv;
    p.q_rows = dq;
    p.q_in = dq_in ? dq_in : dq;
    p.n_sess = n_sess;
    p.n_tokens = n_tokens;
    p.n_kv = kv[0]->n_kv;
    p.n_q = n_q_heads;
    p.hd = hd;
    p.n_rot = (n_rot_pairs >= 1 && n_rot_pairs < half) ? n_rot_pairs : half;  // kernels.c:1381-1383
    p.theta = (theta_base < 1.0f) ? 10000.0f : theta_base;                    // kernels.c:1374
    p.rope = (flags & WR_CUDA_APPEND_ROPE) ? 1u : 0u;
    const uint32_t q_ctas = (dq && p.rope) ? (n_q_heads + kAppendQHeads - 1) / kAppendQHeads : 0u;
    const dim3 grid(n_sess * n_tokens, 1 + q_ctas);
    WR_CUDA_TRY(wr_launch_pdl(rope_kv_append_kernel, grid, dim3(kAppendThreads), hd * sizeof(float), ctx->stream, p));
    ctx->launches++;
    ctx->pdl_kind = WR_PDL_APPEND;
    ctx->pdl_index = ctx->launches;
    WR_CUDA_TRY(cudaGetLastError());
    return WR_CUDA_OK;
}

extern "C" int wr_cuda_kv_append(wr_cuda_ctx *ctx, uint32_t n_sess, wr_cuda_kv *const *kv,
                                 uint32_t layer, const uint32_t *positions, uint32_t n_tokens,
                                 const float *k_rows, const float *v_rows, float *q_rows,
                                 uint32_t n_q_heads, float theta_base, uint32_t n_rot_pairs,
                                 uint32_t flags, int mem)
{
    int rc = wr_append_validate(ctx, n_sess, kv, layer, positions, n_tokens, k_rows, v_rows,
                                q_rows, n_q_heads, mem);
    if (rc != WR_CUDA_OK) return rc;
    if (n_tokens == 0) return WR_CUDA_OK;
    std::lock_guard<std::mutex> g(ctx->lock);
    WR_CUDA_TRY(cudaSetDevice(ctx->device));
    const size_t rows = (size_t)n_sess * n_tokens;
    const size_t kv_bytes = rows * kv[0]->n_kv * kv[0]->hd * sizeof(float);
    const size_t q_bytes = q_rows ? rows * n_q_heads * kv[0]->hd * sizeof(float) : 0;
    const float *dk = k_rows, *dv = v_rows;
    float *dq = q_rows;
    if (mem == WR_CUDA_MEM_HOST) {
        rc = wr_ctx_reserve_stage(ctx, 2 * kv_bytes + q_bytes, 0);
        if (rc != WR_CUDA_OK) return rc;
        char *d = (char *)ctx->stage_dev;
        WR_CUDA_TRY(cudaMemcpyAsync(d, k_rows, kv_bytes, cudaMemcpyHostToDevice, ctx->stream));
        WR_CUDA_TRY(cudaMemcpyAsync(d + kv_bytes, v_rows, kv_bytes, cudaMemcpyHostToDevice,
                                    ctx->stream));
        dk = (const float *)d;
        dv = (const float *)(d + kv_bytes);
        if (q_rows) {
            WR_CUDA_TRY(cudaMemcpyAsync(d + 2 * kv_bytes, q_rows, q_bytes, cudaMemcpyHostToDevice,
                                        ctx->stream));
            dq = (float *)(d + 2 * kv_bytes);
        }
    }
    rc = wr_append_launch(ctx, n_sess, kv, layer, positions, n_tokens, dk, dv, dq, n_q_heads,
                          theta_base, n_rot_pairs, flags, nullptr);
    if (rc != WR_CUDA_OK) return rc;
    if (mem == WR_CUDA_MEM_HOST) {
        if (q_rows && (flags & WR_CUDA_APPEND_ROPE))
            WR_CUDA_TRY(cudaMemcpyAsync(q_rows, dq, q_bytes, cudaMemcpyDeviceToHost, ctx->stream));
        return wr_ctx_sync_checked(ctx);
    }
    return WR_CUDA_OK;
}
