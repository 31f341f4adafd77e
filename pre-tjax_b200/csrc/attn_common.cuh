// Declarations shared by the attention translation units.
#pragma once
#include "common.cuh"

namespace ptj {

// Dropout on attention probabilities: element (b*H+h, i, j) of the [B*H, S, S] probability tensor is element
// ((b*H+h)*S + i)*S + j of the site's mask stream.
struct AttnDropout {
  uint32_t thr16;    // floor(p * 65536)
  float eval_scale;  // 1 - p
  int train;
  uint64_t seed;
  uint32_t stream_id;
  __device__ __forceinline__ float factor(int64_t bh, int64_t S, int64_t i, int64_t j) const {
    if (!train) return eval_scale;
    if (thr16 == 0u) return 1.f;
    const uint64_t idx = (static_cast<uint64_t>(bh) * S + i) * S + j;
    return dropout_keep(seed, stream_id, idx, thr16) ? 1.f : 0.f;
  }
};

// row_kstart (all four paths, optional): int32[batch, seq], the first key each query row may attend to; row i then
// attends keys [row_kstart[b, i], i] (empty when row_kstart > i: zero output row, statistics (0, 1)). NULL = 0.
int attn_fwd_simt(const void* q, const void* k, const void* v, void* o, float* row_max, float* row_sum,
                  const int32_t* row_kstart, const ptj_attn_shape& sh, const AttnDropout& dr, int dtype, cudaStream_t st);
int attn_bwd_simt(const void* d_o, const void* q, const void* k, const void* v, const void* o, const float* row_max,
                  const float* row_sum, void* dq, void* dk, void* dv, const int32_t* row_kstart,
                  const ptj_attn_shape& sh, const ptj_attn_shape& dsh, const AttnDropout& dr, int dtype, cudaStream_t st);

// tcgen05 kernels: bf16, d_head == 64, seq % 128 == 0, 16-byte aligned strides.
bool attn_tc_supported(const ptj_attn_shape& sh, const void* const* ptrs, int nptrs);
// keep_bits (optional, both directions): the call's dropout keep flags from attn_keep_bits_tc; NULL = the kernels draw
// the same flags themselves.
size_t attn_keep_bits_bytes(const ptj_attn_shape& sh);
int attn_keep_bits_tc(uint32_t* bits, const ptj_attn_shape& sh, const AttnDropout& dr, cudaStream_t st);
int attn_fwd_tc(const void* q, const void* k, const void* v, void* o, float* row_max, float* row_sum,
                const uint32_t* keep_bits, const int32_t* row_kstart, const ptj_attn_shape& sh, const AttnDropout& dr,
                cudaStream_t st);
// workspace: attn_bwd_tc_workspace_bytes(sh) bytes, 16-byte aligned (per-KV-tile dQ shares and per-row constants)
size_t attn_bwd_tc_workspace_bytes(const ptj_attn_shape& sh);
int attn_bwd_tc(const void* d_o, const void* q, const void* k, const void* v, const void* o, const float* row_max,
                const float* row_sum, void* dq, void* dk, void* dv, const ptj_attn_shape& sh,
                const ptj_attn_shape& dsh, const AttnDropout& dr, const uint32_t* keep_bits,
                const int32_t* row_kstart, void* workspace, size_t workspace_bytes, cudaStream_t st);

}  // namespace ptj
