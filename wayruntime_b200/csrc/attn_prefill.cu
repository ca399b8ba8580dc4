// attn_prefill.cu — causal prefill attention (placeholder until the kernel lands).
#include "wr_internal.cuh"

extern "C" int wr_cuda_attn_prefill(wr_cuda_ctx *, wr_cuda_kv *, uint32_t, uint32_t, uint32_t,
                                    const void *, int, float *, uint32_t, float, uint32_t, int)
{
    return WR_CUDA_ERR_UNSUPPORTED;
}
