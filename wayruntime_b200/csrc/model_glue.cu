// model_glue.cu — the layer stack around attention, device-resident.
//
// The reference's decode body (src/core/session.c:405-568) runs, per layer:
// RMSNorm, the Q/K/V projections, per-head QK-norm, RoPE + KV append +
// attention, the output projection, a residual add, RMSNorm, the gate / up
// projections, SiLU(gate)*up, the down projection, a residual add; then the
// final RMSNorm and the LM head.  With attention on the GPU, leaving the rest
// on the host makes every layer cross the bus twice.  This file keeps a copy of
// the F32 weights on the device (wr_cuda_model) and runs the whole stack there:
// the rows of a forward pass enter as token ids and leave as logits.
//
// All arithmetic is F32, as the reference's F32 paths are (kernels.c:978-1090
// matmul with GGML-layout weights W[out][in]; :1276-1313 RMSNorm
// x * (1/sqrt(mean(x^2)+eps)) * w; :1318-1350 SiLU(a)*b).  Sums run in a
// different order than the host's SIMD loops, so results agree to F32 rounding,
// not bit for bit.  A row's result does not depend on how many other rows
// share the call (same lanes, same order), which keeps batched logits
// byte-equal to serial ones as the reference promises (src/core/batch.c:1-40).
//
// Kernels: a row-block GEMV (each warp owns 1-4 weight rows, the activation
// rows sit in shared memory, the weights stream from HBM exactly once per group
// of up to 16 activation rows) with optional fused RMSNorm on the input, fused
// residual add or SiLU*up on the output; per-head RMSNorm; embedding gather;
// row RMSNorm; a two-step arg-max with the reference's tie rule (first maximum wins,
// src/cli/wayrt.c:805-812).
#include <math.h>
#include <stdlib.h>

#include <chrono>

#include "wr_internal.cuh"

namespace {

constexpr int kGemvThreads = 128;      // 4 warps per CTA
constexpr int kGemvWarps = kGemvThreads / 32;
constexpr int kChunk = 512;            // activation floats staged per row and pass
constexpr uint32_t kLogitRowsMax = WR_CUDA_BATCH_MAX;

struct GemvSeg {
    const float *w;        // [n][k] row-major (GGML layout of a [k -> n] weight)
    float *out;            // [rows][out_stride]
    uint32_t n, out_stride;
};

struct GemvParams {
    GemvSeg seg[3];
    uint32_t cta_end[3];   // running CTA count after each segment
    uint32_t n_seg;
    const float *x;        // [rows][x_stride]
    uint32_t x_stride, k, rows;
    const float *norm_w;   // fused RMSNorm weight over k, or null
    float eps;
    const float *add;      // residual rows added to the result, or null (may alias out)
    uint32_t add_stride;
    uint32_t swiglu;       // seg[0] = gate, seg[1] = up: seg[0].out <- SiLU(gate) * up
};

__device__ __forceinline__ float4 ldg_stream(const float *p)
{
    float4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(p));
    return v;
}

// Sum M per-lane partials across the warp.  Afterwards every lane holds, in
// v[0], the warp total of the value whose index the function returns; lanes
// whose index bits agree hold the same total.  Each step that still has more
// than one live value halves them by exchanging the half the partner keeps,
// so the whole reduction costs about M shuffles instead of 5*M.
template <int M>
__device__ __forceinline__ int warp_reduce_many(float (&v)[M], int lane)
{
    static_assert(M >= 1 && M <= 32 && (M & (M - 1)) == 0, "power of two up to 32");
    int width = M, idx = 0;
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) {
        if (width > 1) {
            const int half = width / 2;
            const bool upper = (lane & o) != 0;
#pragma unroll
            for (int i = 0; i < M / 2; ++i) {
                if (i < half) {
                    const float send = upper ? v[i] : v[i + half];
                    const float keep = upper ? v[i + half] : v[i];
                    v[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
                }
            }
            if (upper) idx += half;
            width = half;
        } else {
            v[0] += __shfl_xor_sync(0xffffffffu, v[0], o);
        }
    }
    return idx;
}

// lanes that write: those whose non-index bits are zero
template <int M>
__device__ __forceinline__ bool reduce_writer(int lane)
{
    // index bits are the top log2(M) of the five lane bits
    int used = 0;
    for (int m = M, o = 16; m > 1; m >>= 1, o >>= 1) used |= o;
    return (lane & ~used & 31) == 0;
}

// ---- the GEMV pair ---------------------------------------------------------
//
// y[r][n] = sum_k W[n][k] * x[r][k], optionally with RMSNorm fused on x, and a
// residual add or SiLU(gate)*up on the way out.  Two kernels, one arithmetic:
// K is cut into four quarters; inside a quarter lane l takes the 16-byte
// vectors l, l+32, ... in ascending order with fused multiply-adds, starting
// from zero; lane l then adds its four quarter sums in order; the 32 lane sums
// are added by the xor butterfly (offsets 16, 8, 4, 2, 1).  The fused norm
// multiplies x by the norm weight first and the finished sum by
// 1/sqrt(mean(x^2)+eps) last, the sum of squares following the same quarter /
// lane / butterfly order.  Because both kernels compute every output by exactly
// this recipe, a row's bits do not depend on how many rows share the call or on
// which kernel served it.
//
//   gemv_splitk_kernel (<= 4 activation rows): a CTA owns C weight rows and
//     its four warps take one quarter each, so every lane has all its loads in
//     flight at once and nothing is staged; x comes straight from L2.  With few
//     rows the weights are all the traffic, and one warp per weight row would
//     leave most of the device idle on a narrow output (1024 rows = 7 warps/SM).
//   gemv_rows_kernel (up to 16 rows per CTA): each warp owns NW weight rows
//     and walks the four quarters itself; the activation rows of the current
//     piece of a quarter sit in shared memory for all four warps, so x costs
//     RG/(4*NW) of the weight bytes instead of RG/C.

struct KQuarters {
    uint32_t vec, per;     // 16-byte vectors in K; vectors per quarter
    __device__ __forceinline__ explicit KQuarters(uint32_t k) : vec(k / 4), per((k / 4 + 3) / 4) {}
    __device__ __forceinline__ uint32_t lo(uint32_t q) const { return q * per < vec ? q * per : vec; }
    __device__ __forceinline__ uint32_t hi(uint32_t q) const { return (q + 1) * per < vec ? (q + 1) * per : vec; }
};

__device__ __forceinline__ float sumsq4(float ss, const float4 v)
{
    return fmaf(v.w, v.w, fmaf(v.z, v.z, fmaf(v.y, v.y, fmaf(v.x, v.x, ss))));
}
__device__ __forceinline__ float4 mul4(const float4 a, const float4 b)
{
    return make_float4(__fmul_rn(a.x, b.x), __fmul_rn(a.y, b.y), __fmul_rn(a.z, b.z), __fmul_rn(a.w, b.w));
}
__device__ __forceinline__ float dot4(const float4 w, const float4 x, float acc)
{
    acc = fmaf(w.x, x.x, acc);
    acc = fmaf(w.y, x.y, acc);
    acc = fmaf(w.z, x.z, acc);
    return fmaf(w.w, x.w, acc);
}
__device__ __forceinline__ float inv_rms_of(float sumsq, uint32_t k, float eps)
{
    return 1.0f / sqrtf(__fadd_rn(__fdiv_rn(sumsq, (float)k), eps));
}
__device__ __forceinline__ float silu_mul(float g, float u)
{
    return __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), u);
}

// weight rows of a CTA / warp: plain, or swiglu (first half gate rows, second half the same rows of up)
template <int NR>
__device__ __forceinline__ void weight_rows(const GemvParams &p, const GemvSeg &seg, uint32_t n0,
                                            const float *(&wrow)[NR])
{
    constexpr int H = (NR >= 2) ? NR / 2 : 1;
#pragma unroll
    for (int c = 0; c < NR; ++c) {
        uint32_t n = p.swiglu ? n0 + (c % H) : n0 + c;
        const float *base = p.swiglu ? ((c < H) ? p.seg[0].w : p.seg[1].w) : seg.w;
        if (n >= seg.n) n = seg.n - 1;               // clamped rows are computed and dropped
        wrow[c] = base + (size_t)n * p.k;
    }
}

constexpr int kPrefetchRegs = 16;        // 16-byte weight vectors a lane holds before the dependency wait

template <int RG, int C>
__global__ void __launch_bounds__(kGemvThreads) gemv_splitk_kernel(const GemvParams p)
{
    __shared__ float part[kGemvWarps][C * RG + RG][32];      // per quarter (= warp): every lane's partial sums
    __shared__ float red[C * RG + RG];
    pdl_trigger();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t r0 = blockIdx.y * RG;
    uint32_t cta = blockIdx.x, s = 0;
    if (!p.swiglu) {
        while (s + 1 < p.n_seg && cta >= p.cta_end[s]) ++s;
        if (s > 0) cta -= p.cta_end[s - 1];
    }
    const GemvSeg seg = p.seg[s];
    constexpr int H = (C >= 2) ? C / 2 : 1;
    const uint32_t n0 = cta * (p.swiglu ? H : C);
    const float *wrow[C];
    weight_rows<C>(p, seg, n0, wrow);
    const float *xrow[RG];
#pragma unroll
    for (int r = 0; r < RG; ++r) {
        const uint32_t row = (r0 + r < p.rows) ? r0 + r : p.rows - 1;    // clamped rows are dropped at the end
        xrow[r] = p.x + (size_t)row * p.x_stride;
    }
    const KQuarters kq(p.k);
    const uint32_t v_lo = kq.lo(warp), v_hi = kq.hi(warp);

    float acc[C][RG], ss[RG];
#pragma unroll
    for (int r = 0; r < RG; ++r) {
        ss[r] = 0.f;
#pragma unroll
        for (int c = 0; c < C; ++c) acc[c][r] = 0.f;
    }
    // Weights do not depend on the kernel before this one: the first PV vectors of the lane's walk
    // (all of it for K up to 512 * PV) are requested before the dependency wait, so their trip from
    // HBM overlaps that kernel's tail; the activations are read after it.
    constexpr int PV = kPrefetchRegs / C;
    float4 wbuf[PV][C];
#pragma unroll
    for (int i = 0; i < PV; ++i) {
        const uint32_t v = v_lo + lane + 32u * i;
        if (v < v_hi) {
#pragma unroll
            for (int c = 0; c < C; ++c) wbuf[i][c] = ldg_stream(wrow[c] + 4 * v);
        }
    }
    pdl_wait();
    auto step = [&](uint32_t v, const float4 (&w)[C]) {
        float4 nw = make_float4(1.f, 1.f, 1.f, 1.f);
        if (p.norm_w) nw = *reinterpret_cast<const float4 *>(p.norm_w + 4 * v);
#pragma unroll
        for (int r = 0; r < RG; ++r) {
            float4 xv = *reinterpret_cast<const float4 *>(xrow[r] + 4 * v);
            if (p.norm_w) {
                ss[r] = sumsq4(ss[r], xv);
                xv = mul4(xv, nw);
            }
#pragma unroll
            for (int c = 0; c < C; ++c) acc[c][r] = dot4(w[c], xv, acc[c][r]);
        }
    };
#pragma unroll
    for (int i = 0; i < PV; ++i) {
        const uint32_t v = v_lo + lane + 32u * i;
        if (v < v_hi) step(v, wbuf[i]);
    }
#pragma unroll 2
    for (uint32_t v = v_lo + lane + 32u * PV; v < v_hi; v += 32) {
        float4 w[C];
#pragma unroll
        for (int c = 0; c < C; ++c) w[c] = ldg_stream(wrow[c] + 4 * v);
        step(v, w);
    }
    constexpr int M = C * RG;
#pragma unroll
    for (int i = 0; i < M; ++i) part[warp][i][lane] = acc[i / RG][i % RG];
    if (p.norm_w) {
#pragma unroll
        for (int r = 0; r < RG; ++r) part[warp][M + r][lane] = ss[r];
    }
    __syncthreads();
    // every lane adds its four quarter sums in order, then the butterfly over the lanes
    for (int idx = warp; idx < M + (p.norm_w ? RG : 0); idx += kGemvWarps) {
        float t = part[0][idx][lane];
#pragma unroll
        for (int q = 1; q < kGemvWarps; ++q) t = __fadd_rn(t, part[q][idx][lane]);
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) t = __fadd_rn(t, __shfl_xor_sync(0xffffffffu, t, o));
        if (lane == 0) red[idx] = t;
    }
    __syncthreads();
    const int n_out = p.swiglu ? H * RG : C * RG;
    if (tid < n_out) {
        const int c = tid / RG, r = tid % RG;
        const uint32_t n = n0 + c, row = r0 + r;
        if (n < seg.n && row < p.rows) {
            const float inv = p.norm_w ? inv_rms_of(red[M + r], p.k, p.eps) : 1.0f;
            float y = __fmul_rn(red[c * RG + r], inv);
            if (p.swiglu) {
                const float u = __fmul_rn(red[(c + H) * RG + r], inv);
                seg.out[(size_t)row * seg.out_stride + n] = silu_mul(y, u);
            } else {
                if (p.add) y = __fadd_rn(p.add[(size_t)row * p.add_stride + n], y);
                seg.out[(size_t)row * seg.out_stride + n] = y;
            }
        }
    }
}

// RG: activation rows per CTA (row group); NW: weight rows per warp.
template <int RG, int NW>
__global__ void __launch_bounds__(kGemvThreads) gemv_rows_kernel(const GemvParams p)
{
    constexpr int kPieceVec = kChunk / 4;            // 16-byte vectors of x staged per row and pass
    __shared__ __align__(16) float xs[RG][kChunk];
    __shared__ float inv_rms[RG];
    pdl_trigger();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t r0 = blockIdx.y * RG;
    uint32_t cta = blockIdx.x, s = 0;
    if (!p.swiglu) {
        while (s + 1 < p.n_seg && cta >= p.cta_end[s]) ++s;
        if (s > 0) cta -= p.cta_end[s - 1];
    }
    const GemvSeg seg = p.seg[s];
    constexpr int H = (NW >= 2) ? NW / 2 : 1;
    const uint32_t n0 = (cta * kGemvWarps + warp) * (p.swiglu ? H : NW);
    const float *wrow[NW];
    weight_rows<NW>(p, seg, n0, wrow);
    const KQuarters kq(p.k);
    pdl_wait();

    if (p.norm_w) {                                  // sum of squares in the shared order
        for (int r = warp; r < RG; r += kGemvWarps) {
            float t = 0.f;
            if (r0 + r < p.rows) {
                const float *xr = p.x + (size_t)(r0 + r) * p.x_stride;
#pragma unroll 1
                for (uint32_t q = 0; q < 4; ++q) {
                    float ss = 0.f;
                    for (uint32_t v = kq.lo(q) + lane; v < kq.hi(q); v += 32)
                        ss = sumsq4(ss, *reinterpret_cast<const float4 *>(xr + 4 * v));
                    t = (q == 0) ? ss : __fadd_rn(t, ss);
                }
            }
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) t = __fadd_rn(t, __shfl_xor_sync(0xffffffffu, t, o));
            if (lane == 0) inv_rms[r] = inv_rms_of(t, p.k, p.eps);
        }
    }

    constexpr int M = NW * RG;
    constexpr int G = (M > 32) ? 32 : M;
    constexpr int NG = M / G;
    float lane_tot[NW][RG];                          // this lane's quarter sums, added in quarter order

#pragma unroll 1
    for (uint32_t q = 0; q < 4; ++q) {
        const uint32_t v_lo = kq.lo(q), v_hi = kq.hi(q);
        float acc[NW][RG];
#pragma unroll
        for (int c = 0; c < NW; ++c)
#pragma unroll
            for (int r = 0; r < RG; ++r) acc[c][r] = 0.f;
        for (uint32_t c0 = v_lo; c0 < v_hi; c0 += kPieceVec) {
            const uint32_t nvec = (v_hi - c0 < (uint32_t)kPieceVec) ? v_hi - c0 : (uint32_t)kPieceVec;
            __syncthreads();                         // the previous piece has been consumed
            for (uint32_t i = tid; i < RG * nvec; i += kGemvThreads) {
                const uint32_t r = i / nvec, vv = i % nvec;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (r0 + r < p.rows) {
                    v = *reinterpret_cast<const float4 *>(p.x + (size_t)(r0 + r) * p.x_stride + 4 * (c0 + vv));
                    if (p.norm_w) v = mul4(v, *reinterpret_cast<const float4 *>(p.norm_w + 4 * (c0 + vv)));
                }
                *reinterpret_cast<float4 *>(&xs[r][4 * vv]) = v;
            }
            __syncthreads();
#pragma unroll 2
            for (uint32_t vv = lane; vv < nvec; vv += 32) {
                float4 w[NW];
#pragma unroll
                for (int c = 0; c < NW; ++c) w[c] = ldg_stream(wrow[c] + 4 * (c0 + vv));
#pragma unroll
                for (int r = 0; r < RG; ++r) {
                    const float4 xv = *reinterpret_cast<const float4 *>(&xs[r][4 * vv]);
#pragma unroll
                    for (int c = 0; c < NW; ++c) acc[c][r] = dot4(w[c], xv, acc[c][r]);
                }
            }
        }
#pragma unroll
        for (int c = 0; c < NW; ++c)
#pragma unroll
            for (int r = 0; r < RG; ++r) lane_tot[c][r] = (q == 0) ? acc[c][r] : __fadd_rn(lane_tot[c][r], acc[c][r]);
    }
    // the butterfly over the lanes, once, for all NW * RG sums
    float tot[NG];
    int tot_idx[NG];
#pragma unroll
    for (int g = 0; g < NG; ++g) {
        float v[G];
#pragma unroll
        for (int i = 0; i < G; ++i) v[i] = lane_tot[(g * G + i) / RG][(g * G + i) % RG];
        tot_idx[g] = warp_reduce_many<G>(v, lane) + g * G;
        tot[g] = v[0];
    }
    __syncthreads();                                 // inv_rms is complete (and visible) for every warp

    if (!p.swiglu) {
#pragma unroll
        for (int g = 0; g < NG; ++g) {
            const uint32_t c = tot_idx[g] / RG, r = tot_idx[g] % RG, n = n0 + c, row = r0 + r;
            if (reduce_writer<G>(lane) && n < seg.n && row < p.rows) {
                float y = __fmul_rn(tot[g], p.norm_w ? inv_rms[r] : 1.0f);
                if (p.add) y = __fadd_rn(p.add[(size_t)row * p.add_stride + n], y);
                seg.out[(size_t)row * seg.out_stride + n] = y;
            }
        }
    } else if constexpr (NW >= 2) {
        // flat index = c * RG + r over all NW rows: gate rows are c < H, up rows c >= H.  A lane that
        // holds gate (c, r) needs up (c + H, r): with M <= 32 it sits in the same group at index
        // + H*RG, whose owner differs in one lane bit; with two groups it is this lane's other total.
        if constexpr (NG == 2) {
            const uint32_t c = tot_idx[0] / RG, r = tot_idx[0] % RG, n = n0 + c, row = r0 + r;
            // group 0 holds rows [0, 32/RG) = gate, group 1 the same positions of up
            if (n < seg.n && row < p.rows) {
                const float inv = p.norm_w ? inv_rms[r] : 1.0f;
                seg.out[(size_t)row * seg.out_stride + n] =
                    silu_mul(__fmul_rn(tot[0], inv), __fmul_rn(tot[1], inv));
            }
        } else {
            // index bits are the top log2(M) lane bits; + H*RG = + M/2 flips the highest one (lane bit 4)
            const float other = __shfl_xor_sync(0xffffffffu, tot[0], 16);
            const uint32_t c = tot_idx[0] / RG, r = tot_idx[0] % RG, n = n0 + c, row = r0 + r;
            if (reduce_writer<G>(lane) && c < (uint32_t)H && n < seg.n && row < p.rows) {
                const float inv = p.norm_w ? inv_rms[r] : 1.0f;
                seg.out[(size_t)row * seg.out_stride + n] =
                    silu_mul(__fmul_rn(tot[0], inv), __fmul_rn(other, inv));
            }
        }
    }
}

// resid[r][:] = table[token[r]][:]
__global__ void embed_rows_kernel(const uint32_t *tokens, const float *table, float *out, uint32_t hidden)
{
    const float4 *src = reinterpret_cast<const float4 *>(table + (size_t)tokens[blockIdx.x] * hidden);
    float4 *dst = reinterpret_cast<float4 *>(out + (size_t)blockIdx.x * hidden);
    for (uint32_t i = threadIdx.x; i < hidden / 4; i += blockDim.x) dst[i] = src[i];
}

// In-place RMSNorm of every head vector: vectors [0, n_a) of `a`, then [0, n_b) of `b`; one warp each.
__global__ void head_rmsnorm_kernel(float *a, const float *wa, uint32_t n_a, float *b, const float *wb,
                                    uint32_t n_b, uint32_t dim, float eps)
{
    const uint32_t v = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (v >= n_a + n_b) return;
    float *x = (v < n_a) ? a + (size_t)v * dim : b + (size_t)(v - n_a) * dim;
    const float *w = (v < n_a) ? wa : wb;
    float ss = 0.f;
    for (uint32_t i = lane; i < dim; i += 32) ss += x[i] * x[i];
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
    for (uint32_t i = lane; i < dim; i += 32) x[i] = x[i] * inv * w[i];
}

// out[r][:] = RMSNorm(x[r][:]) * w; one block per row
__global__ void rmsnorm_rows_kernel(const float *x, uint32_t x_stride, const float *w, float *out,
                                    uint32_t out_stride, uint32_t dim, float eps)
{
    __shared__ float part[32];
    const float *xr = x + (size_t)blockIdx.x * x_stride;
    float ss = 0.f;
    for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) ss += xr[i] * xr[i];
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = (threadIdx.x < (blockDim.x >> 5)) ? part[threadIdx.x] : 0.f;
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (threadIdx.x == 0) part[0] = 1.0f / sqrtf(t / (float)dim + eps);
    }
    __syncthreads();
    const float inv = part[0];
    float *o_ = out + (size_t)blockIdx.x * out_stride;
    for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) o_[i] = xr[i] * inv * w[i];
}

// First maximum of each row (strict >, so the lowest id wins a tie), in two steps: kArgmaxParts
// blocks per row each reduce a slice of the vocabulary to (value, index); one warp per row then
// reduces the slices' results.  (value, index) pairs are compared as "greater value, or equal
// value and lower index", so the order of the reduction does not matter.
constexpr int kArgmaxParts = 64;

__device__ __forceinline__ bool argmax_better(float v, uint32_t i, float bv, uint32_t bi)
{
    return bi == 0xffffffffu || (i != 0xffffffffu && (v > bv || (v == bv && i < bi)));
}

__device__ __forceinline__ void argmax_warp(float &best, uint32_t &at)
{
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, at, o);
        if (argmax_better(ov, oi, best, at)) { best = ov; at = oi; }
    }
}

__global__ void __launch_bounds__(256) argmax_parts_kernel(const float *logits, uint32_t vocab, float *part_v,
                                                           uint32_t *part_i)
{
    __shared__ float bv[8];
    __shared__ uint32_t bi[8];
    const uint32_t row = blockIdx.y, part = blockIdx.x;
    const uint32_t per = (vocab + kArgmaxParts - 1) / kArgmaxParts;
    const uint32_t lo = part * per, hi = min(lo + per, vocab);
    const float *r = logits + (size_t)row * vocab;
    float best = -INFINITY;
    uint32_t at = 0xffffffffu;
    for (uint32_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float v = r[i];
        if (argmax_better(v, i, best, at)) { best = v; at = i; }
    }
    argmax_warp(best, at);
    if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = best; bi[threadIdx.x >> 5] = at; }
    __syncthreads();
    if (threadIdx.x < 32) {
        best = threadIdx.x < 8 ? bv[threadIdx.x] : -INFINITY;
        at = threadIdx.x < 8 ? bi[threadIdx.x] : 0xffffffffu;
        argmax_warp(best, at);
        if (threadIdx.x == 0) {
            part_v[row * kArgmaxParts + part] = best;
            part_i[row * kArgmaxParts + part] = at;
        }
    }
}

__global__ void argmax_final_kernel(const float *part_v, const uint32_t *part_i, uint32_t *out)
{
    const uint32_t row = blockIdx.x, lane = threadIdx.x;
    float best = -INFINITY;
    uint32_t at = 0xffffffffu;
    for (uint32_t i = lane; i < (uint32_t)kArgmaxParts; i += 32) {
        const float v = part_v[row * kArgmaxParts + i];
        const uint32_t idx = part_i[row * kArgmaxParts + i];
        if (argmax_better(v, idx, best, at)) { best = v; at = idx; }
    }
    argmax_warp(best, at);
    if (lane == 0) out[row] = at;
}

template <int RG, int NW>
void launch_gemv_t(const GemvParams &p, uint32_t ctas, cudaStream_t st)
{
    dim3 grid(ctas, (p.rows + RG - 1) / RG);
    (void)wr_launch_pdl(gemv_rows_kernel<RG, NW>, grid, dim3(kGemvThreads), 0, st, p);
}

template <int RG, int C>
void launch_splitk_t(const GemvParams &p, uint32_t ctas, cudaStream_t st)
{
    dim3 grid(ctas, (p.rows + RG - 1) / RG);
    (void)wr_launch_pdl(gemv_splitk_kernel<RG, C>, grid, dim3(kGemvThreads), 0, st, p);
}

template <int C>
void launch_splitk(const GemvParams &p, uint32_t ctas, cudaStream_t st)
{
    if (p.rows == 1) launch_splitk_t<1, C>(p, ctas, st);
    else if (p.rows == 2) launch_splitk_t<2, C>(p, ctas, st);
    else launch_splitk_t<4, C>(p, ctas, st);
}

template <int NW>
void launch_gemv_rg(const GemvParams &p, uint32_t ctas, cudaStream_t st)
{
    const uint32_t r = p.rows;
    if (r == 1) launch_gemv_t<1, NW>(p, ctas, st);
    else if (r == 2) launch_gemv_t<2, NW>(p, ctas, st);
    else if (r <= 4) launch_gemv_t<4, NW>(p, ctas, st);
    else if (r <= 8) launch_gemv_t<8, NW>(p, ctas, st);
    else launch_gemv_t<16, NW>(p, ctas, st);
}

// Weight rows per warp from the total output width: narrow outputs take one row
// per warp so that the grid still covers the device.
int weight_rows_per_warp(uint32_t n_total)
{
    if (n_total >= 32768) return 4;
    if (n_total >= 2048) return 2;
    return 1;
}

}  // namespace

// ------------------------------------------------------------------ the model

struct wr_cuda_layer_dev {
    const float *attn_norm, *wq, *wk, *wv, *q_norm, *k_norm, *wo, *ffn_norm, *w_gate, *w_up, *w_down;
    uint32_t ffn;
};

struct wr_cuda_model {
    wr_cuda_ctx *ctx = nullptr;
    uint32_t n_layers = 0, hidden = 0, n_q = 0, n_kv = 0, hd = 0, vocab = 0, n_rot = 0, max_rows = 0;
    float eps = 0.f, theta = 0.f, scale = 0.f;
    char *slab = nullptr;                // every weight, one allocation
    size_t slab_bytes = 0;
    const float *embed = nullptr, *lm_head = nullptr, *final_norm = nullptr;
    std::vector<wr_cuda_layer_dev> layers;
    // row scratch (device)
    float *resid = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *attn = nullptr, *gate = nullptr;
    float *normed = nullptr, *logits = nullptr;
    uint32_t *tokens = nullptr, *best = nullptr, *part_i = nullptr;
    float *part_v = nullptr;             // arg-max partials [16][kArgmaxParts]
    uint32_t *h_tokens = nullptr;        // pinned: token ids in, arg-max ids out
    uint32_t ffn_max = 0;
    uint64_t launches = 0;
    uint64_t last_enqueue_ns = 0;        // host time the last forward pass spent before it began to wait
    std::mutex fwd;                      // one forward pass at a time (the scratch rows are shared)
};

namespace {

constexpr uint32_t kSplitKRowsMax = 4;

int gemv(wr_cuda_model *m, GemvParams &p, uint32_t n_total_for_width)
{
    if (p.rows <= kSplitKRowsMax) {
        // weight rows per CTA: 2 for narrow outputs (more CTAs), 4 otherwise
        const int c = (p.swiglu || n_total_for_width >= 4096) ? 4 : 2;
        const uint32_t cols_per_cta = p.swiglu ? (uint32_t)c / 2 : (uint32_t)c;
        uint32_t ctas = 0;
        if (p.swiglu) {
            ctas = (p.seg[0].n + cols_per_cta - 1) / cols_per_cta;
        } else {
            for (uint32_t s = 0; s < p.n_seg; ++s) {
                ctas += (p.seg[s].n + cols_per_cta - 1) / cols_per_cta;
                p.cta_end[s] = ctas;
            }
        }
        if (c == 4) launch_splitk<4>(p, ctas, m->ctx->stream);
        else launch_splitk<2>(p, ctas, m->ctx->stream);
        ++m->launches;
        WR_CUDA_TRY(cudaGetLastError());
        return WR_CUDA_OK;
    }
    const int nw = p.swiglu ? 2 : weight_rows_per_warp(n_total_for_width);
    const uint32_t cols_per_cta = (p.swiglu ? 1u : (uint32_t)nw) * kGemvWarps;
    uint32_t ctas = 0;
    if (p.swiglu) {
        ctas = (p.seg[0].n + cols_per_cta - 1) / cols_per_cta;
    } else {
        for (uint32_t s = 0; s < p.n_seg; ++s) {
            ctas += (p.seg[s].n + cols_per_cta - 1) / cols_per_cta;
            p.cta_end[s] = ctas;
        }
    }
    cudaStream_t st = m->ctx->stream;
    if (nw == 4) launch_gemv_rg<4>(p, ctas, st);
    else if (nw == 2) launch_gemv_rg<2>(p, ctas, st);
    else launch_gemv_rg<1>(p, ctas, st);
    ++m->launches;
    WR_CUDA_TRY(cudaGetLastError());
    return WR_CUDA_OK;
}

size_t up256(size_t n) { return (n + 255u) & ~(size_t)255u; }

}  // namespace

extern "C" int wr_cuda_model_create(wr_cuda_ctx *ctx, const wr_cuda_model_desc *d, wr_cuda_model **out)
{
    if (!ctx || !d || !out) return WR_CUDA_ERR_INVAL;
    *out = nullptr;
    if (d->n_layers == 0 || d->n_layers > WR_CUDA_MAX_LAYERS || !d->layers || !d->embed || !d->lm_head ||
        !d->final_norm || d->hidden == 0 || d->n_q_heads == 0 || d->n_kv_heads == 0 || d->head_dim == 0 ||
        d->vocab == 0 || d->max_rows == 0)
        return WR_CUDA_ERR_INVAL;
    // rows move as 16-byte vectors
    if ((d->hidden & 3u) || (d->head_dim & 3u)) return WR_CUDA_ERR_UNSUPPORTED;
    for (uint32_t L = 0; L < d->n_layers; ++L) {
        const wr_cuda_layer_desc &l = d->layers[L];
        if (!l.attn_norm || !l.wq || !l.wk || !l.wv || !l.wo || !l.ffn_norm || !l.w_gate || !l.w_up ||
            !l.w_down || l.ffn_dim == 0)
            return WR_CUDA_ERR_INVAL;
        if ((l.q_norm == nullptr) != (l.k_norm == nullptr)) return WR_CUDA_ERR_INVAL;
        if (l.ffn_dim & 3u) return WR_CUDA_ERR_UNSUPPORTED;
    }
    std::lock_guard<std::mutex> g(ctx->lock);
    WR_CUDA_TRY(cudaSetDevice(ctx->device));
    wr_cuda_model *m = new (std::nothrow) wr_cuda_model();
    if (!m) return WR_CUDA_ERR_NOMEM;
    m->ctx = ctx;
    m->n_layers = d->n_layers; m->hidden = d->hidden; m->n_q = d->n_q_heads; m->n_kv = d->n_kv_heads;
    m->hd = d->head_dim; m->vocab = d->vocab; m->n_rot = d->n_rot_pairs; m->max_rows = d->max_rows;
    m->eps = d->rms_eps; m->theta = d->rope_theta; m->scale = d->attn_scale;
    const size_t hid = d->hidden, nq = (size_t)d->n_q_heads * d->head_dim, nkv = (size_t)d->n_kv_heads * d->head_dim;
    const bool tied = (d->embed == d->lm_head);

    size_t total = up256((size_t)d->vocab * hid * 4) * (tied ? 1 : 2) + up256(hid * 4);
    for (uint32_t L = 0; L < d->n_layers; ++L) {
        const size_t ffn = d->layers[L].ffn_dim;
        if (ffn > m->ffn_max) m->ffn_max = (uint32_t)ffn;
        total += 2 * up256(hid * 4) + 2 * up256((size_t)d->head_dim * 4) + 2 * up256(nq * hid * 4) +
                 2 * up256(nkv * hid * 4) + 3 * up256(ffn * hid * 4);
    }
    const size_t R = d->max_rows, LR = kLogitRowsMax;
    const size_t scratch = up256(R * hid * 4) + 2 * up256(R * nq * 4) + 2 * up256(R * nkv * 4) +
                           up256(R * (size_t)m->ffn_max * 4) + up256(LR * hid * 4) +
                           up256(LR * (size_t)d->vocab * 4) + 2 * up256(R * 4) + 2 * up256(LR * kArgmaxParts * 4);
    m->slab_bytes = total + scratch;
    cudaError_t e = cudaMalloc(&m->slab, m->slab_bytes);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        delete m;
        return WR_CUDA_ERR_NOMEM;
    }
    e = cudaHostAlloc((void **)&m->h_tokens, 2 * R * sizeof(uint32_t), cudaHostAllocPortable);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        cudaFree(m->slab);
        delete m;
        return WR_CUDA_ERR_NOMEM;
    }
    char *cur = m->slab;
    bool ok = true;
    auto put = [&](const float *src, size_t n_floats) -> const float * {
        char *dst = cur;
        cur += up256(n_floats * 4);
        if (ok && cudaMemcpyAsync(dst, src, n_floats * 4, cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess)
            ok = false;
        return reinterpret_cast<const float *>(dst);
    };
    auto take = [&](size_t n_floats) -> float * {
        char *dst = cur;
        cur += up256(n_floats * 4);
        return reinterpret_cast<float *>(dst);
    };
    m->lm_head = put(d->lm_head, (size_t)d->vocab * hid);
    m->embed = tied ? m->lm_head : put(d->embed, (size_t)d->vocab * hid);
    m->final_norm = put(d->final_norm, hid);
    m->layers.resize(d->n_layers);
    for (uint32_t L = 0; L < d->n_layers; ++L) {
        const wr_cuda_layer_desc &l = d->layers[L];
        wr_cuda_layer_dev &o = m->layers[L];
        const size_t ffn = l.ffn_dim;
        o.ffn = l.ffn_dim;
        o.attn_norm = put(l.attn_norm, hid);
        o.ffn_norm = put(l.ffn_norm, hid);
        o.q_norm = l.q_norm ? put(l.q_norm, d->head_dim) : nullptr;
        o.k_norm = l.k_norm ? put(l.k_norm, d->head_dim) : nullptr;
        if (!l.q_norm) cur += 2 * up256((size_t)d->head_dim * 4);
        o.wq = put(l.wq, nq * hid);
        o.wo = put(l.wo, nq * hid);
        o.wk = put(l.wk, nkv * hid);
        o.wv = put(l.wv, nkv * hid);
        o.w_gate = put(l.w_gate, ffn * hid);
        o.w_up = put(l.w_up, ffn * hid);
        o.w_down = put(l.w_down, ffn * hid);
    }
    m->resid = take(R * hid);
    m->q = take(R * nq);
    m->attn = take(R * nq);
    m->k = take(R * nkv);
    m->v = take(R * nkv);
    m->gate = take(R * (size_t)m->ffn_max);
    m->normed = take(LR * hid);
    m->logits = take(LR * (size_t)d->vocab);
    m->tokens = reinterpret_cast<uint32_t *>(take(R));
    m->best = reinterpret_cast<uint32_t *>(take(R));
    m->part_v = take(LR * kArgmaxParts);
    m->part_i = reinterpret_cast<uint32_t *>(take(LR * kArgmaxParts));
    if (ok && cudaStreamSynchronize(ctx->stream) != cudaSuccess) ok = false;
    if (!ok || (size_t)(cur - m->slab) > m->slab_bytes) {
        (void)cudaGetLastError();
        cudaFreeHost(m->h_tokens);
        cudaFree(m->slab);
        delete m;
        return WR_CUDA_ERR_INTERNAL;
    }
    *out = m;
    return WR_CUDA_OK;
}

extern "C" void wr_cuda_model_destroy(wr_cuda_model *m)
{
    if (!m) return;
    {
        std::lock_guard<std::mutex> g(m->ctx->lock);
        cudaSetDevice(m->ctx->device);
        cudaStreamSynchronize(m->ctx->stream);
        cudaFree(m->slab);
        cudaFreeHost(m->h_tokens);
    }
    delete m;
}

extern "C" uint64_t wr_cuda_model_bytes(const wr_cuda_model *m) { return m ? m->slab_bytes : 0; }
extern "C" uint64_t wr_cuda_model_launches(const wr_cuda_model *m) { return m ? m->launches : 0; }
extern "C" uint64_t wr_cuda_model_last_enqueue_ns(const wr_cuda_model *m) { return m ? m->last_enqueue_ns : 0; }

extern "C" int wr_cuda_model_forward(wr_cuda_ctx *ctx, wr_cuda_model *m, int mode, uint32_t n_rows,
                                     wr_cuda_kv *const *kv, const uint32_t *positions,
                                     const uint32_t *tokens, uint32_t out_from, float *hidden_out,
                                     float *normed_out, float *const *logits_out, uint32_t *argmax_out,
                                     float *attn_tap_out)
{
    if (!ctx || !m || m->ctx != ctx || !kv || !positions || !tokens) return WR_CUDA_ERR_INVAL;
    if (mode != WR_CUDA_FWD_DECODE && mode != WR_CUDA_FWD_PREFILL) return WR_CUDA_ERR_INVAL;
    if (n_rows == 0 || n_rows > m->max_rows || out_from > n_rows) return WR_CUDA_ERR_LIMIT;
    if (mode == WR_CUDA_FWD_DECODE && n_rows > WR_CUDA_BATCH_MAX) return WR_CUDA_ERR_LIMIT;
    const uint32_t n_out = n_rows - out_from;
    if ((logits_out || argmax_out) && n_out > kLogitRowsMax) return WR_CUDA_ERR_LIMIT;
    if ((normed_out || logits_out || argmax_out) && n_out == 0) return WR_CUDA_ERR_INVAL;
    for (uint32_t r = 0; r < n_rows; ++r)
        if (tokens[r] >= m->vocab) return WR_CUDA_ERR_INVAL;      // refused before anything runs
    const uint32_t n_sess = (mode == WR_CUDA_FWD_DECODE) ? n_rows : 1;
    for (uint32_t s = 0; s < n_sess; ++s)
        if (!kv[s] || kv[s]->n_layers != m->n_layers || kv[s]->n_kv != m->n_kv || kv[s]->hd != m->hd)
            return WR_CUDA_ERR_INVAL;

    std::lock_guard<std::mutex> fg(m->fwd);
    const auto t_begin = std::chrono::steady_clock::now();
    cudaStream_t st = ctx->stream;
    const uint32_t hid = m->hidden, nq = m->n_q * m->hd, nkv = m->n_kv * m->hd;

    // Decode rows are processed in an order of their own: the sessions that the one-kernel
    // short-context step covers first, the others after them, so that each kind is a contiguous
    // block of rows.  Which kind a session is depends on that session alone.  perm[i] = caller's row.
    uint32_t perm[WR_CUDA_BATCH_MAX], pos_p[WR_CUDA_BATCH_MAX], n_short = 0;
    wr_cuda_kv *kv_p[WR_CUDA_BATCH_MAX];
    bool permuted = false;
    if (mode == WR_CUDA_FWD_DECODE) {
        const bool use_small = (getenv("WR_CUDA_STEP_SMALL_OFF") == nullptr);
        uint32_t n = 0;
        for (int pass = 0; pass < 2; ++pass)
            for (uint32_t r = 0; r < n_rows; ++r) {
                const bool small = use_small && wr_step_small_covers(kv[r], m->n_q, positions[r]);
                if (small == (pass == 0)) perm[n++] = r;
            }
        for (uint32_t i = 0; i < n_rows; ++i) {
            if (perm[i] != i) permuted = true;
            kv_p[i] = kv[perm[i]];
            pos_p[i] = positions[perm[i]];
            if (use_small && wr_step_small_covers(kv_p[i], m->n_q, pos_p[i])) n_short = i + 1;
            if (pos_p[i] >= kv_p[i]->max_ctx) return WR_CUDA_ERR_CTX_FULL;
        }
    }
    {
        std::lock_guard<std::mutex> g(ctx->lock);
        WR_CUDA_TRY(cudaSetDevice(ctx->device));
        for (uint32_t r = 0; r < n_rows; ++r)
            m->h_tokens[r] = tokens[mode == WR_CUDA_FWD_DECODE ? perm[r] : r];
        WR_CUDA_TRY(cudaMemcpyAsync(m->tokens, m->h_tokens, n_rows * sizeof(uint32_t),
                                    cudaMemcpyHostToDevice, st));
        embed_rows_kernel<<<n_rows, 128, 0, st>>>(m->tokens, m->embed, m->resid, hid);
        ++m->launches;
        WR_CUDA_TRY(cudaGetLastError());
    }
    for (uint32_t L = 0; L < m->n_layers; ++L) {
        const wr_cuda_layer_dev &l = m->layers[L];
        int rc;
        {
            std::lock_guard<std::mutex> g(ctx->lock);
            GemvParams p{};
            p.seg[0] = {l.wq, m->q, nq, nq};
            p.seg[1] = {l.wk, m->k, nkv, nkv};
            p.seg[2] = {l.wv, m->v, nkv, nkv};
            p.n_seg = 3;
            p.x = m->resid; p.x_stride = hid; p.k = hid; p.rows = n_rows;
            p.norm_w = l.attn_norm; p.eps = m->eps;
            rc = gemv(m, p, nq + 2 * nkv);
            if (rc != WR_CUDA_OK) return rc;
            const uint32_t r_lo = (mode == WR_CUDA_FWD_DECODE) ? n_short : 0;    // rows of the three-kernel path
            if (l.q_norm && r_lo < n_rows) {
                const uint32_t n_a = (n_rows - r_lo) * m->n_q, n_b = (n_rows - r_lo) * m->n_kv;
                head_rmsnorm_kernel<<<(n_a + n_b + 3) / 4, 128, 0, st>>>(m->q + (size_t)r_lo * nq, l.q_norm, n_a,
                                                                       m->k + (size_t)r_lo * nkv, l.k_norm, n_b,
                                                                       m->hd, m->eps);
                ++m->launches;
                WR_CUDA_TRY(cudaGetLastError());
            }
            if (mode == WR_CUDA_FWD_DECODE && n_short) {
                rc = wr_step_small_launch(ctx, n_short, kv_p, L, pos_p, m->q, m->k, m->v, m->attn, m->n_q,
                                          m->theta, m->n_rot, l.q_norm, l.k_norm, m->eps, m->scale);
                if (rc != WR_CUDA_OK) return rc;
            }
        }
        if (mode == WR_CUDA_FWD_DECODE) {
            if (n_short < n_rows) {
                rc = wr_cuda_decode_step(ctx, n_rows - n_short, kv_p + n_short, L, pos_p + n_short,
                                         m->q + (size_t)n_short * nq, m->k + (size_t)n_short * nkv,
                                         m->v + (size_t)n_short * nkv, m->attn + (size_t)n_short * nq, m->n_q,
                                         m->theta, m->n_rot, WR_CUDA_APPEND_ROPE, m->scale, 0, WR_CUDA_MEM_DEVICE);
                if (rc != WR_CUDA_OK) return rc;
            }
        } else {
            rc = wr_cuda_kv_append(ctx, 1, kv, L, positions, n_rows, m->k, m->v, m->q, m->n_q, m->theta,
                                   m->n_rot, WR_CUDA_APPEND_ROPE, WR_CUDA_MEM_DEVICE);
            if (rc != WR_CUDA_OK) return rc;
            rc = wr_cuda_attn_prefill(ctx, kv[0], L, positions[0], n_rows, m->q, WR_CUDA_F32, m->attn,
                                      m->n_q, m->scale, 0, WR_CUDA_MEM_DEVICE);
            if (rc != WR_CUDA_OK) return rc;
        }
        {
            std::lock_guard<std::mutex> g(ctx->lock);
            if (attn_tap_out) {
                float *dst = attn_tap_out + (size_t)L * n_rows * nq;
                if (!permuted) {
                    WR_CUDA_TRY(cudaMemcpyAsync(dst, m->attn, (size_t)n_rows * nq * 4, cudaMemcpyDeviceToHost, st));
                } else {
                    for (uint32_t i = 0; i < n_rows; ++i)
                        WR_CUDA_TRY(cudaMemcpyAsync(dst + (size_t)perm[i] * nq, m->attn + (size_t)i * nq,
                                                    (size_t)nq * 4, cudaMemcpyDeviceToHost, st));
                }
            }
            GemvParams p{};
            p.seg[0] = {l.wo, m->resid, hid, hid};
            p.n_seg = 1;
            p.x = m->attn; p.x_stride = nq; p.k = nq; p.rows = n_rows;
            p.add = m->resid; p.add_stride = hid;
            rc = gemv(m, p, hid);
            if (rc != WR_CUDA_OK) return rc;

            GemvParams f{};
            f.seg[0] = {l.w_gate, m->gate, l.ffn, m->ffn_max};
            f.seg[1] = {l.w_up, nullptr, l.ffn, 0};
            f.n_seg = 2;
            f.swiglu = 1;
            f.x = m->resid; f.x_stride = hid; f.k = hid; f.rows = n_rows;
            f.norm_w = l.ffn_norm; f.eps = m->eps;
            rc = gemv(m, f, l.ffn);
            if (rc != WR_CUDA_OK) return rc;

            GemvParams dn{};
            dn.seg[0] = {l.w_down, m->resid, hid, hid};
            dn.n_seg = 1;
            dn.x = m->gate; dn.x_stride = m->ffn_max; dn.k = l.ffn; dn.rows = n_rows;
            dn.add = m->resid; dn.add_stride = hid;
            rc = gemv(m, dn, hid);
            if (rc != WR_CUDA_OK) return rc;
        }
    }
    std::lock_guard<std::mutex> g(ctx->lock);
    // Device rows [o_lo, n_rows) are finished (final norm, LM head); device row i is the caller's row
    // perm[i] when the decode rows were reordered, and then every row is finished and only the asked
    // ones are copied out.
    const uint32_t o_lo = permuted ? 0u : out_from, n_fin = n_rows - o_lo;
    auto caller_row = [&](uint32_t i) { return permuted ? perm[i] : i; };
    if ((logits_out || argmax_out) && n_fin > kLogitRowsMax) return WR_CUDA_ERR_LIMIT;
    const float *res_out = m->resid + (size_t)o_lo * hid;
    if (hidden_out && n_out) {
        if (!permuted) {
            WR_CUDA_TRY(cudaMemcpyAsync(hidden_out, res_out, (size_t)n_out * hid * 4, cudaMemcpyDeviceToHost, st));
        } else {
            for (uint32_t i = 0; i < n_rows; ++i)
                if (perm[i] >= out_from)
                    WR_CUDA_TRY(cudaMemcpyAsync(hidden_out + (size_t)(perm[i] - out_from) * hid,
                                                m->resid + (size_t)i * hid, (size_t)hid * 4,
                                                cudaMemcpyDeviceToHost, st));
        }
    }
    if ((normed_out || logits_out || argmax_out) && n_out) {
        // the final norm of at most 16 rows is kept for the LM head; more rows (normed_out only) go in passes
        for (uint32_t done = 0; done < n_fin; done += kLogitRowsMax) {
            const uint32_t nr = (n_fin - done < kLogitRowsMax) ? n_fin - done : kLogitRowsMax;
            rmsnorm_rows_kernel<<<nr, 256, 0, st>>>(res_out + (size_t)done * hid, hid, m->final_norm, m->normed,
                                                    hid, hid, m->eps);
            ++m->launches;
            WR_CUDA_TRY(cudaGetLastError());
            if (normed_out) {
                if (!permuted) {
                    WR_CUDA_TRY(cudaMemcpyAsync(normed_out + (size_t)done * hid, m->normed, (size_t)nr * hid * 4,
                                                cudaMemcpyDeviceToHost, st));
                } else {
                    for (uint32_t i = 0; i < nr; ++i)
                        if (perm[done + i] >= out_from)
                            WR_CUDA_TRY(cudaMemcpyAsync(normed_out + (size_t)(perm[done + i] - out_from) * hid,
                                                        m->normed + (size_t)i * hid, (size_t)hid * 4,
                                                        cudaMemcpyDeviceToHost, st));
                }
            }
        }
    }
    if ((logits_out || argmax_out) && n_out) {
        GemvParams p{};
        p.seg[0] = {m->lm_head, m->logits, m->vocab, m->vocab};
        p.n_seg = 1;
        p.x = m->normed; p.x_stride = hid; p.k = hid; p.rows = n_fin;
        int rc = gemv(m, p, m->vocab);
        if (rc != WR_CUDA_OK) return rc;
        if (argmax_out) {
            argmax_parts_kernel<<<dim3(kArgmaxParts, n_fin), 256, 0, st>>>(m->logits, m->vocab, m->part_v, m->part_i);
            argmax_final_kernel<<<n_fin, 32, 0, st>>>(m->part_v, m->part_i, m->best);
            m->launches += 2;
            WR_CUDA_TRY(cudaGetLastError());
            WR_CUDA_TRY(cudaMemcpyAsync(m->h_tokens + m->max_rows, m->best, n_fin * sizeof(uint32_t),
                                        cudaMemcpyDeviceToHost, st));
        }
        if (logits_out)
            for (uint32_t i = 0; i < n_fin; ++i) {
                const uint32_t c = caller_row(o_lo + i);
                if (c >= out_from && logits_out[c - out_from])
                    WR_CUDA_TRY(cudaMemcpyAsync(logits_out[c - out_from], m->logits + (size_t)i * m->vocab,
                                                (size_t)m->vocab * 4, cudaMemcpyDeviceToHost, st));
            }
    }
    m->last_enqueue_ns = (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(
                             std::chrono::steady_clock::now() - t_begin).count();
    int rc = wr_ctx_sync_checked(ctx);
    if (rc != WR_CUDA_OK) return rc;
    if (argmax_out)
        for (uint32_t i = 0; i < n_fin; ++i) {
            const uint32_t c = caller_row(o_lo + i);
            if (c >= out_from) argmax_out[c - out_from] = m->h_tokens[m->max_rows + i];
        }
    return WR_CUDA_OK;
}
