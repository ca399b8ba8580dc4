// attn_step_small.cu — one layer-step of attention for short contexts, in ONE
// kernel: per-head QK-norm, RoPE on Q and K, the truncating F16 append of K / V
// and the attention of the new token over its session's keys.
//
// This is the reference's per-layer body between the projections and the
// output projection (src/core/session.c:458-496: wri_op_rmsnorm on the [heads,
// hd] views, wri_op_rope x2, kv_append_row x2, wri_op_gqa_attention) for the
// case the big kernels serve badly: one new token per session and at most
// kSmallMaxKeys keys, where three launches (norm, append, the split-KV decode
// kernel with its queue, arrival counters and merge warps) cost 20 us to move
// a few hundred KB.  One CTA per (session, kv head) does all of it out of shared
// memory.  Used by the device-resident layer stack (model_glue.cu) for every
// session whose own length allows it — the choice depends on that session
// alone, so a session's bits do not depend on its batch mates.
//
// Bit-level contracts kept: the cache bytes (norm as head_rmsnorm_kernel does
// it, RoPE with the reference's polynomials and separately rounded products,
// truncating F16 convert) are the ones the three-kernel path stores.  The
// softmax is the materialised form (all scores, one maximum, one sum) in F32
// with exp from the hardware; the reference's online form differs from it by
// float associativity only (kernels.c:1466-1470).
#include "mathx_dev.cuh"
#include "wr_internal.cuh"

namespace {

constexpr int kSmallThreads = 256;
constexpr int kSmallWarps = kSmallThreads / 32;
constexpr uint32_t kSmallMaxKeys = WR_STEP_SMALL_MAX_KEYS;
constexpr uint32_t kSmallMaxGroup = 8;     // q heads per kv head
constexpr uint32_t kHd = 128;

struct step_small_params {
    wr_batch_desc b;                 // b.seq_len[s] = position of the new token of session s
    float *q;                        // [n_sess][n_q][128]: raw projections in, (normed, rotated) rows out
    const float *k, *v;              // [n_sess][n_kv][128] raw projections
    float *out;                      // [n_sess][n_q][128]
    const float *q_norm, *k_norm;    // [128] each, or both null
    uint32_t n_kv, n_q, n_rot;
    float eps, theta, scale;
};

__device__ __forceinline__ const char *row_chunk(const char *block, uint32_t tok, uint32_t c)
{
    // 16-byte chunk c (dims 8c .. 8c+7) of token `tok` inside a tiled (head, K|V) block
    return block + (c >> 3) * (kPageTokens * 128u) + tok * 128u + (((c & 7u) ^ (tok & 7u)) << 4);
}

// GM: upper bound of q heads per kv head this instantiation is unrolled for (the kernel runs its code
// once, on a handful of warps, so code size is time: a cold instruction line costs as much as a load).
template <int GM>
__global__ void __launch_bounds__(kSmallThreads) attn_step_small_kernel(const step_small_params p)
{
    __shared__ __align__(16) float sq[GM][kHd];                  // this kv head's q rows
    __shared__ __align__(16) float sk[kHd], sv[kHd];
    __shared__ __align__(16) __half nk[kHd], nv[kHd];            // the new row as the cache holds it
    __shared__ float cs_tab[kHd / 2], sn_tab[kHd / 2];
    __shared__ float sc[GM][kSmallMaxKeys];                      // scores, then probabilities
    __shared__ float s_inv_l[GM];
    __shared__ float s_qnw[kHd], s_knw[kHd];                     // QK-norm weights
    __shared__ const char *s_page[kSmallMaxKeys / kPageTokens];  // this session's pages of this layer

    const uint32_t s = blockIdx.x / p.n_kv, kvh = blockIdx.x % p.n_kv;
    const uint32_t G = p.n_q / p.n_kv;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t pos = p.b.seq_len[s], n_keys = pos + 1;
    constexpr uint32_t half = kHd / 2;

    // ---- what does not depend on the kernel before this one (the projections): norm weights, the
    //      session's page pointers, the pair angles of this position (kernels.c:1400-1405).  The kernel
    //      behind this one may be scheduled meanwhile, and this part overlaps the one before.
    pdl_trigger();
    const uint64_t *pages = p.b.pages[s];
    if (p.q_norm) {
        if (tid < kHd) s_qnw[tid] = p.q_norm[tid];
        else if (tid < 2 * kHd) s_knw[tid - kHd] = p.k_norm[tid - kHd];
    }
    if (tid < (n_keys + kPageTokens - 1) / kPageTokens) s_page[tid] = (const char *)pages[tid];
    if (tid < p.n_rot) {
        float sn, cs;
        wrmath::rope_angle(pos, tid, kHd, wrmath::log_ref(p.theta), sn, cs);
        cs_tab[tid] = cs;
        sn_tab[tid] = sn;
    }
    pdl_wait();
    // ---- rows in
    float *qrows = p.q + ((size_t)s * p.n_q + (size_t)kvh * G) * kHd;
    for (uint32_t i = tid; i < G * kHd; i += kSmallThreads) sq[i / kHd][i % kHd] = qrows[i];
    if (tid < kHd) sk[tid] = p.k[((size_t)s * p.n_kv + kvh) * kHd + tid];
    else if (tid < 2 * kHd) sv[tid - kHd] = p.v[((size_t)s * p.n_kv + kvh) * kHd + tid - kHd];
    __syncthreads();

    // ---- per-head RMSNorm of K and of the G q heads (one warp per vector), as head_rmsnorm_kernel
    if (p.q_norm) {
        for (uint32_t vct = warp; vct < G + 1; vct += kSmallWarps) {
            float *x = (vct == 0) ? sk : sq[vct - 1];
            const float *w = (vct == 0) ? s_knw : s_qnw;
            float ss = 0.f;
            for (uint32_t i = lane; i < kHd; i += 32) ss += x[i] * x[i];
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const float inv = 1.0f / sqrtf(ss / (float)kHd + p.eps);
            for (uint32_t i = lane; i < kHd; i += 32) x[i] = x[i] * inv * w[i];
        }
        __syncthreads();
    }

    // ---- RoPE (pairs j, j + 64; products rounded separately, kernels.c:1406-1407)
    for (uint32_t i = tid; i < (G + 1) * half; i += kSmallThreads) {
        const uint32_t vct = i / half, j = i % half;
        if (j < p.n_rot) {
            float *x = (vct == 0) ? sk : sq[vct - 1];
            const float cs = cs_tab[j], sn = sn_tab[j];
            const float x0 = x[j], x1 = x[j + half];
            x[j] = wrmath::sub(wrmath::mul(x0, cs), wrmath::mul(x1, sn));
            x[j + half] = wrmath::add(wrmath::mul(x0, sn), wrmath::mul(x1, cs));
        }
    }
    __syncthreads();

    // ---- append: the new K / V row into its page (truncating convert), and kept for this CTA's own use;
    //      the rotated q rows go back to the caller's buffer
    if (tid < kHd) {
        char *page = const_cast<char *>(s_page[pos / kPageTokens]);
        const uint32_t tk = pos % kPageTokens, off = wr_elem_off(tk, tid, kHd);
        const uint16_t kb = wr_f32_to_f16_trunc(sk[tid]), vb = wr_f32_to_f16_trunc(sv[tid]);
        *(uint16_t *)(page + wr_block_off(kvh, 0, kHd) + off) = kb;
        *(uint16_t *)(page + wr_block_off(kvh, 1, kHd) + off) = vb;
        nk[tid] = __ushort_as_half(kb);
        nv[tid] = __ushort_as_half(vb);
    }
    for (uint32_t i = tid; i < G * kHd; i += kSmallThreads) qrows[i] = sq[i / kHd][i % kHd];
    __syncthreads();

    // ---- scores: one thread per key, all G heads at once.  The sixteen 16-byte loads of a key row are
    //      issued together (the kernel is latency bound: what matters is the number of round trips).
    for (uint32_t key = tid; key < n_keys; key += kSmallThreads) {
        float dot[(uint32_t)GM];
#pragma unroll
        for (uint32_t g = 0; g < (uint32_t)GM; ++g) dot[g] = 0.f;
        const char *kb = s_page[key / kPageTokens] + wr_block_off(kvh, 0, kHd);
        const uint32_t tok = key % kPageTokens;
        uint4 raw[kHd / 8];
#pragma unroll
        for (uint32_t c = 0; c < kHd / 8; ++c) {
            if (key == pos) raw[c] = *reinterpret_cast<const uint4 *>(&nk[8 * c]);
            else raw[c] = __ldg(reinterpret_cast<const uint4 *>(row_chunk(kb, tok, c)));
        }
#pragma unroll
        for (uint32_t c = 0; c < kHd / 8; ++c) {
            const __half2 *h2 = reinterpret_cast<const __half2 *>(&raw[c]);
            float kf[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __half22float2(h2[i]);
                kf[2 * i] = f.x;
                kf[2 * i + 1] = f.y;
            }
#pragma unroll
            for (uint32_t g = 0; g < (uint32_t)GM; ++g) {
                if (g < G) {
                    const float4 qa = *reinterpret_cast<const float4 *>(&sq[g][8 * c]);
                    const float4 qb = *reinterpret_cast<const float4 *>(&sq[g][8 * c + 4]);
                    float d = dot[g];
                    d = fmaf(qa.x, kf[0], d); d = fmaf(qa.y, kf[1], d); d = fmaf(qa.z, kf[2], d); d = fmaf(qa.w, kf[3], d);
                    d = fmaf(qb.x, kf[4], d); d = fmaf(qb.y, kf[5], d); d = fmaf(qb.z, kf[6], d); d = fmaf(qb.w, kf[7], d);
                    dot[g] = d;
                }
            }
        }
#pragma unroll
        for (uint32_t g = 0; g < (uint32_t)GM; ++g)
            if (g < G) sc[g][key] = dot[g] * p.scale;
    }
    __syncthreads();

    // ---- softmax: warp g owns head g
    for (uint32_t g = warp; g < G; g += kSmallWarps) {
        float m = WR_NEG_SENTINEL;
        for (uint32_t key = lane; key < n_keys; key += 32) m = fmaxf(m, sc[g][key]);
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        float l = 0.f;
        for (uint32_t key = lane; key < n_keys; key += 32) {
            const float pw = __expf(sc[g][key] - m);
            sc[g][key] = pw;
            l += pw;
        }
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
        if (lane == 0) s_inv_l[g] = (l > 0.f) ? 1.0f / l : 0.f;
    }
    __syncthreads();

    // ---- P.V: thread = (16-byte chunk c of the row, key group kg of 16); all G heads at once
    {
        const uint32_t kg = lane & 15u, c = warp * 2u + (lane >> 4);
        float acc[(uint32_t)GM][8];
#pragma unroll
        for (uint32_t g = 0; g < (uint32_t)GM; ++g)
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[g][i] = 0.f;
        constexpr uint32_t kBatch = 8;               // V rows whose loads are in flight together
        for (uint32_t key0 = kg; key0 < n_keys; key0 += 16 * kBatch) {
            uint4 raw[kBatch];
#pragma unroll
            for (uint32_t u = 0; u < kBatch; ++u) {
                const uint32_t key = key0 + 16 * u;
                raw[u] = make_uint4(0u, 0u, 0u, 0u);
                if (key < n_keys) {
                    if (key == pos) {
                        raw[u] = *reinterpret_cast<const uint4 *>(&nv[8 * c]);
                    } else {
                        const char *vb = s_page[key / kPageTokens] + wr_block_off(kvh, 1, kHd);
                        raw[u] = __ldg(reinterpret_cast<const uint4 *>(row_chunk(vb, key % kPageTokens, c)));
                    }
                }
            }
#pragma unroll
            for (uint32_t u = 0; u < kBatch; ++u) {
                const uint32_t key = key0 + 16 * u;
                if (key >= n_keys) break;
                const __half2 *h2 = reinterpret_cast<const __half2 *>(&raw[u]);
                float vf[8];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __half22float2(h2[i]);
                    vf[2 * i] = f.x;
                    vf[2 * i + 1] = f.y;
                }
#pragma unroll
                for (uint32_t g = 0; g < (uint32_t)GM; ++g) {
                    if (g < G) {
                        const float pw = sc[g][key];
#pragma unroll
                        for (int i = 0; i < 8; ++i) acc[g][i] = fmaf(pw, vf[i], acc[g][i]);
                    }
                }
            }
        }
        // add the 16 key groups (lane bits 0-3)
#pragma unroll
        for (uint32_t g = 0; g < (uint32_t)GM; ++g) {
            if (g < G) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float a = acc[g][i];
                    a += __shfl_xor_sync(0xffffffffu, a, 8);
                    a += __shfl_xor_sync(0xffffffffu, a, 4);
                    a += __shfl_xor_sync(0xffffffffu, a, 2);
                    a += __shfl_xor_sync(0xffffffffu, a, 1);
                    acc[g][i] = a;
                }
                if (kg == 0) {
                    const float inv = s_inv_l[g];
                    float *o = p.out + ((size_t)s * p.n_q + (size_t)kvh * G + g) * kHd + 8 * c;
                    *reinterpret_cast<float4 *>(o) =
                        make_float4(acc[g][0] * inv, acc[g][1] * inv, acc[g][2] * inv, acc[g][3] * inv);
                    *reinterpret_cast<float4 *>(o + 4) =
                        make_float4(acc[g][4] * inv, acc[g][5] * inv, acc[g][6] * inv, acc[g][7] * inv);
                }
            }
        }
    }
}

}  // namespace

bool wr_step_small_covers(const wr_cuda_kv *kv, uint32_t n_q_heads, uint32_t position)
{
    return kv->hd == kHd && kv->n_kv > 0 && n_q_heads % kv->n_kv == 0 && n_q_heads / kv->n_kv <= kSmallMaxGroup &&
           position + 1 <= kSmallMaxKeys;
}

// Enqueue on device-resident rows.  Caller holds ctx->lock; every session must pass
// wr_step_small_covers and wr_kv_batch_check, and positions[s] < max_ctx.
int wr_step_small_launch(wr_cuda_ctx *ctx, uint32_t n_sess, wr_cuda_kv *const *kv, uint32_t layer,
                         const uint32_t *positions, float *dq, const float *dk, const float *dv, float *dout,
                         uint32_t n_q_heads, float theta_base, uint32_t n_rot_pairs, const float *q_norm,
                         const float *k_norm, float eps, float scale_override)
{
    if (n_sess == 0 || n_sess > WR_CUDA_BATCH_MAX) return WR_CUDA_ERR_LIMIT;
    step_small_params p;
    for (uint32_t s = 0; s < n_sess; ++s) {
        if (!wr_step_small_covers(kv[s], n_q_heads, positions[s])) return WR_CUDA_ERR_UNSUPPORTED;
        if (positions[s] >= kv[s]->max_ctx) return WR_CUDA_ERR_CTX_FULL;
        p.b.pages[s] = kv[s]->d_pages + (size_t)layer * kv[s]->n_pages;
        p.b.seq_len[s] = positions[s];
    }
    constexpr uint32_t half = kHd / 2u;
    p.q = dq;
    p.k = dk;
    p.v = dv;
    p.out = dout;
    p.q_norm = q_norm;
    p.k_norm = k_norm;
    p.n_kv = kv[0]->n_kv;
    p.n_q = n_q_heads;
    p.n_rot = (n_rot_pairs >= 1 && n_rot_pairs < half) ? n_rot_pairs : half;     // kernels.c:1381-1383
    p.eps = eps;
    p.theta = (theta_base < 1.0f) ? 10000.0f : theta_base;                       // kernels.c:1374
    p.scale = (scale_override > 0.0f) ? scale_override : 1.0f / sqrtf((float)kHd);
    const uint32_t group = n_q_heads / p.n_kv, grid = n_sess * p.n_kv;
    const dim3 g3(grid), b3(kSmallThreads);
    if (group == 1) WR_CUDA_TRY(wr_launch_pdl(attn_step_small_kernel<1>, g3, b3, 0, ctx->stream, p));
    else if (group == 2) WR_CUDA_TRY(wr_launch_pdl(attn_step_small_kernel<2>, g3, b3, 0, ctx->stream, p));
    else if (group <= 4) WR_CUDA_TRY(wr_launch_pdl(attn_step_small_kernel<4>, g3, b3, 0, ctx->stream, p));
    else WR_CUDA_TRY(wr_launch_pdl(attn_step_small_kernel<8>, g3, b3, 0, ctx->stream, p));
    ctx->launches++;
    WR_CUDA_TRY(cudaGetLastError());
    return WR_CUDA_OK;
}
