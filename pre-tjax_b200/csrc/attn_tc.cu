// tcgen05 flash-attention kernels (placeholder translation unit until the kernels land: reports "not supported"
// so that every call is served by the exact-fp32 CUDA-core kernels).
#include "attn_common.cuh"

namespace ptj {
bool attn_tc_supported(const ptj_attn_shape&, const void* const*, int) { return false; }
int attn_fwd_tc(const void*, const void*, const void*, void*, float*, float*, const ptj_attn_shape&, const AttnDropout&,
                cudaStream_t) { return PTJ_ERR_UNSUPPORTED; }
int attn_bwd_tc(const void*, const void*, const void*, const void*, const void*, const float*, const float*, void*,
                void*, void*, const ptj_attn_shape&, const ptj_attn_shape&, const AttnDropout&, cudaStream_t) {
  return PTJ_ERR_UNSUPPORTED;
}
}  // namespace ptj
