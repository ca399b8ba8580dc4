// attn_decode_static.cu — decode attention for callers that must not allocate.
//
// wr_cuda_attn_decode keeps its split-KV scratch (per-chunk partial results,
// arrival tickets, work queue) in buffers that the context grows with
// cudaMalloc when a larger batch shows up.  Some callers cannot tolerate that:
// a serving loop that has handed every spare byte of the device to its KV
// pool and must never see an allocation fail mid-step, a step function that
// runs on a thread which is not allowed to enter the CUDA allocator (it
// synchronises the whole device), or a host that has frozen its memory map
// after start-up.  For them this file offers the same kernel over a scratch
// area that is part of the library image itself: a file-scope __device__
// array.  The CUDA runtime instantiates a module's device arrays when the
// module is first used on a device, so wr_cuda_ctx_create touches this one
// (wr_static_setup): from context creation to process exit the array occupies
// its 17 MB on that device, and its cost lands at start-up, before the caller
// sizes a KV pool, not at the first step.
//
// Limits and rules
//   * head_dim 128 only (the other head dims use a kernel with no scratch);
//   * at most WR_CUDA_STATIC_MAX_ITEMS work items per call — sessions x kv
//     heads x chunks, 16 sessions of 32768 keys with 8 kv heads are 4096 — and
//     WR_CUDA_STATIC_MAX_GROUPS (session, kv head, q subgroup) triples; a
//     larger call is refused with WR_CUDA_ERR_LIMIT before anything runs;
//   * q and out must be device memory (the host-buffer convenience path
//     needs staging, which is an allocation); anything else is refused with
//     WR_CUDA_ERR_INVAL after a pointer-attribute query, which allocates
//     nothing;
//   * the array's device address is looked up (cudaGetSymbolAddress) once per
//     device, when the first context on that device is created; a call on a
//     device that somehow skipped that does it itself, so make the first call
//     on a device before opening any stream capture;
//   * every call uses the same array: the tickets and the queue are cleared
//     on the stream before each launch, the partial results are always
//     written before they are read; two calls that overlap on the GPU (two
//     contexts, two streams) would race on it — serialise them.
#include <algorithm>

#include "attn_decode_hd128.cuh"
#include "wr_internal.cuh"

namespace {

using namespace wr_decode;

constexpr size_t kScratchFloats = (size_t)WR_CUDA_STATIC_MAX_ITEMS * 8 * kTripleStride;
constexpr size_t kTicketInts = (size_t)WR_CUDA_STATIC_MAX_GROUPS * kTicketsPerGroup + kTicketExtra;     // + queue, exits

// In host code these names are host-side stand-ins, not device addresses: the
// kernel gets the pointers that cudaGetSymbolAddress returns.
static __device__ __align__(256) float g_static_ws[kScratchFloats];
static __device__ __align__(256) int g_static_tickets[kTicketInts];

struct static_ptrs {
    float *ws = nullptr;
    int *tickets = nullptr;
    bool attr_set = false;
};
constexpr int kMaxDevices = 64;
static_ptrs g_ptrs[kMaxDevices];
std::mutex g_ptrs_lock;

// Once per device, with that device current.
int static_setup(int device, static_ptrs **out)
{
    if (device < 0 || device >= kMaxDevices) return WR_CUDA_ERR_LIMIT;
    std::lock_guard<std::mutex> g(g_ptrs_lock);
    static_ptrs &sp = g_ptrs[device];
    if (!sp.ws) {
        float *ws = nullptr;
        int *tk = nullptr;
        WR_CUDA_TRY(cudaGetSymbolAddress((void **)&ws, g_static_ws));
        WR_CUDA_TRY(cudaGetSymbolAddress((void **)&tk, g_static_tickets));
        sp.tickets = tk;
        sp.ws = ws;
    }
    if (!sp.attr_set) {
        WR_CUDA_TRY(cudaFuncSetAttribute(attn_decode_hd128_kernel<1>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)sizeof(smem_layout)));
        WR_CUDA_TRY(cudaFuncSetAttribute(attn_decode_hd128_kernel<2>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)sizeof(smem_layout)));
        sp.attr_set = true;
    }
    *out = &sp;
    return WR_CUDA_OK;
}

// true when `p` is memory the device can address as its own or a peer's allocation
bool is_device_pointer(const void *p)
{
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    return attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
}

}  // namespace

int wr_static_setup(int device)
{
    static_ptrs *sp = nullptr;
    return static_setup(device, &sp);
}

extern "C" int wr_cuda_attn_decode_static(wr_cuda_ctx *ctx, uint32_t n_sess, wr_cuda_kv *const *kv,
                                          uint32_t layer, const uint32_t *seq_lens, const float *q,
                                          float *out, uint32_t n_q_heads, float scale_override,
                                          uint32_t window)
{
    if (!ctx) return WR_CUDA_ERR_INVAL;
    std::lock_guard<std::mutex> g(ctx->lock);
    int rc = wr_kv_batch_check(ctx, n_sess, kv, layer);
    if (rc != WR_CUDA_OK) return rc;
    if (!seq_lens || !q || !out) return WR_CUDA_ERR_INVAL;
    if ((((uintptr_t)q | (uintptr_t)out) & 15u)) return WR_CUDA_ERR_INVAL;
    const uint32_t n_kv = kv[0]->n_kv, hd = kv[0]->hd;
    if (hd != (uint32_t)kHd) return WR_CUDA_ERR_UNSUPPORTED;
    if (n_q_heads == 0 || n_q_heads % n_kv != 0) return WR_CUDA_ERR_INVAL;
    for (uint32_t s = 0; s < n_sess; ++s) {
        if (seq_lens[s] == 0) return WR_CUDA_ERR_INVAL;
        if (seq_lens[s] > ctx->attn_max_seq) return WR_CUDA_ERR_LIMIT;
        if (seq_lens[s] > kv[s]->max_ctx) return WR_CUDA_ERR_INVAL;
    }
    WR_CUDA_TRY(cudaSetDevice(ctx->device));
    static_ptrs *sp = nullptr;
    rc = static_setup(ctx->device, &sp);
    if (rc != WR_CUDA_OK) return rc;

    if (!is_device_pointer(q) || !is_device_pointer(out)) return WR_CUDA_ERR_INVAL;

    // The work decomposition is wr_cuda_attn_decode's own, so the result is the same.
    params p;
    uint32_t nt = 1, items = 0;
    wr_decode_plan(n_sess, kv, layer, seq_lens, n_q_heads, window, p, nt, items);
    if (items > WR_CUDA_STATIC_MAX_ITEMS || p.n_groups > WR_CUDA_STATIC_MAX_GROUPS)
        return WR_CUDA_ERR_LIMIT;           // the fixed scratch area cannot hold this call
    p.q = q;
    p.out = out;
    p.ws = sp->ws;
    p.tickets = sp->tickets;
    p.err = ctx->dev_err;
    p.wait_limit = ctx->wait_limit;
    p.emit_triples = 0;
    p.x_world = 0;
    p.x_step = 0;
    p.early_tiles = 0;
    p.x_recv = 0;
    p.x_max_rows = 0;
    p.x_rows_in = nullptr;
    p.x_row_flag_in = nullptr;
    p.x_done = nullptr;
    p.scale = (scale_override > 0.0f) ? scale_override : 1.0f / sqrtf((float)hd);
    // The array keeps whatever the previous call (or an aborted one) left:
    // the counters must start at zero.
    WR_CUDA_TRY(cudaMemsetAsync(sp->tickets, 0, ((size_t)p.n_groups * kTicketsPerGroup + kTicketExtra) * sizeof(int), ctx->stream));
    const uint32_t grid = std::max(1u, std::min<uint32_t>(items, (uint32_t)ctx->sm_count));
    if (nt == 1)
        attn_decode_hd128_kernel<1><<<grid, kThreads, sizeof(smem_layout), ctx->stream>>>(p);
    else
        attn_decode_hd128_kernel<2><<<grid, kThreads, sizeof(smem_layout), ctx->stream>>>(p);
    ctx->launches++;
    WR_CUDA_TRY(cudaGetLastError());
    return WR_CUDA_OK;
}
