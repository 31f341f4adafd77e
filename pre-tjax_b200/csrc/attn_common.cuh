// Declarations shared by the attention translation units.
#pragma once
#include "common.cuh"

namespace ptj {

// Dropout on attention probabilities: element (b*H+h, i, j) of the [B*H, S, S] probability tensor, flat index idx.
// This site spends 16 random bits per element: one Philox4x32-10 call (counter idx / 8) serves 8 consecutive keys,
// element e = idx % 8 takes the low (e even) or high (e odd) half of word e / 2 and is dropped when that half is
// below floor(p * 65536). The softmax stage of the tensor-core kernels is ALU-bound, hence the cheaper stream.
struct AttnDropout {
  uint32_t thr16;    // floor(p * 65536), clamped to 65535
  float eval_scale;  // 1 - p
  int train;
  uint64_t seed;
  uint32_t stream_id;
  __device__ __forceinline__ float factor(int64_t bh, int64_t S, int64_t i, int64_t j) const {
    if (!train) return eval_scale;
    if (thr16 == 0u) return 1.f;
    const uint64_t idx = (static_cast<uint64_t>(bh) * S + i) * S + j;
    const Philox4 r = philox4x32_10(seed, idx >> 3, stream_id);
    const uint32_t e = static_cast<uint32_t>(idx & 7);
    const uint32_t w = (e >> 1) == 0 ? r.x : (e >> 1) == 1 ? r.y : (e >> 1) == 2 ? r.z : r.w;
    const uint32_t h = (e & 1) ? (w >> 16) : (w & 0xffffu);
    return h >= thr16 ? 1.f : 0.f;
  }
};
inline uint32_t attn_dropout_threshold16(float p) {
  double t = static_cast<double>(p) * 65536.0;
  if (t <= 0.0) return 0u;
  if (t >= 65535.0) return 65535u;
  return static_cast<uint32_t>(t);
}

int attn_fwd_simt(const void* q, const void* k, const void* v, void* o, float* row_max, float* row_sum,
                  const ptj_attn_shape& sh, const AttnDropout& dr, int dtype, cudaStream_t st);
int attn_bwd_simt(const void* d_o, const void* q, const void* k, const void* v, const void* o, const float* row_max,
                  const float* row_sum, void* dq, void* dk, void* dv, const ptj_attn_shape& sh,
                  const ptj_attn_shape& dsh, const AttnDropout& dr, int dtype, cudaStream_t st);

// tcgen05 kernels: bf16, d_head == 64, seq % 128 == 0, 16-byte aligned strides.
bool attn_tc_supported(const ptj_attn_shape& sh, const void* const* ptrs, int nptrs);
int attn_fwd_tc(const void* q, const void* k, const void* v, void* o, float* row_max, float* row_sum,
                const ptj_attn_shape& sh, const AttnDropout& dr, cudaStream_t st);
int attn_bwd_tc(const void* d_o, const void* q, const void* k, const void* v, const void* o, const float* row_max,
                const float* row_sum, void* dq, void* dk, void* dv, const ptj_attn_shape& sh,
                const ptj_attn_shape& dsh, const AttnDropout& dr, cudaStream_t st);

}  // namespace ptj
