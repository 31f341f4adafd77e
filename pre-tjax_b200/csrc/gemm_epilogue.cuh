// Elementwise epilogue shared by the tensor-core and the SIMT GEMM kernels: bias, GELU (saving the pre-activation),
// GELU backward, dropout + residual, accumulate. Works on one row segment held in registers by one thread. The
// epilogue warps of the tensor-core kernel run this while the next tile is being multiplied, so it is written to
// stay well under the instruction budget of one tile's MMAs: 16-byte loads/stores, one Philox call per 8 elements.
#pragma once
#include "common.cuh"

namespace ptj {

struct EpilogueParams {
  void* c;               // [M, ldc] output, float or bf16
  const float* bias;     // [N] or nullptr
  const void* aux;       // [M, ldc] same type as c (GELU_BWD: pre-activation, DROPOUT_RESID: residual)
  void* aux_out;         // [M, ldc] same type as c (GELU: pre-activation) or nullptr
  int64_t M, N, ldc;
  int mode;              // PTJ_EPI_*
  int vec_ok;            // rows of c / aux / aux_out start on 16-byte boundaries
  int bias_vec_ok;       // bias is 16-byte aligned
  uint32_t drop_thr;     // dropout_threshold16(p)
  float eval_scale;
  int train;
  uint64_t seed;
  uint32_t stream_id;
};

template <typename TOut, int CNT>
__device__ __forceinline__ void load_row(const TOut* src, int64_t n0, int64_t N, bool full, float (&a)[CNT]) {
  constexpr int V = Elem<TOut>::kVec;
  if (full) {
#pragma unroll
    for (int j = 0; j < CNT; j += V) {
      float t[V];
      Elem<TOut>::load_vec(src + n0 + j, t);
#pragma unroll
      for (int q = 0; q < V; ++q) a[j + q] = t[q];
    }
  } else {
#pragma unroll
    for (int j = 0; j < CNT; ++j) a[j] = n0 + j < N ? Elem<TOut>::load(src + n0 + j) : 0.f;
  }
}

template <typename TOut, int CNT>
__device__ __forceinline__ void store_row(TOut* dst, int64_t n0, int64_t N, bool full, const float (&v)[CNT]) {
  constexpr int V = Elem<TOut>::kVec;
  if (full) {
#pragma unroll
    for (int j = 0; j < CNT; j += V) {
      float t[V];
#pragma unroll
      for (int q = 0; q < V; ++q) t[q] = v[j + q];
      Elem<TOut>::store_vec(dst + n0 + j, t);
    }
  } else {
#pragma unroll
    for (int j = 0; j < CNT; ++j)
      if (n0 + j < N) Elem<TOut>::store(dst + n0 + j, v[j]);
  }
}

// acc[0..CNT) are columns n0 .. n0+CNT-1 of row m. CNT and n0 are multiples of 8.
template <typename TOut, int CNT>
__device__ __forceinline__ void epilogue_row_segment(const EpilogueParams& ep, int64_t m, int64_t n0, float (&acc)[CNT]) {
  constexpr bool kFast = sizeof(TOut) == 2;  // bf16 output: hardware tanh is exact enough after rounding
  if (m >= ep.M || n0 >= ep.N) return;
  TOut* crow = static_cast<TOut*>(ep.c) + m * ep.ldc;
  const TOut* arow = ep.aux ? static_cast<const TOut*>(ep.aux) + m * ep.ldc : nullptr;
  TOut* orow = ep.aux_out ? static_cast<TOut*>(ep.aux_out) + m * ep.ldc : nullptr;
  const bool full = ep.vec_ok && n0 + CNT <= ep.N;

  if (ep.bias != nullptr) {
    if (ep.bias_vec_ok && n0 + CNT <= ep.N) {
#pragma unroll
      for (int j = 0; j < CNT; j += 4) {
        const float4 b4 = __ldg(reinterpret_cast<const float4*>(ep.bias + n0 + j));
        acc[j] += b4.x; acc[j + 1] += b4.y; acc[j + 2] += b4.z; acc[j + 3] += b4.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < CNT; ++j)
        if (n0 + j < ep.N) acc[j] += ep.bias[n0 + j];
    }
  }
  if (ep.mode == PTJ_EPI_GELU) {
    // the activation sees the pre-activation as stored (rounded to the output type), like a separate GELU kernel would
    if (sizeof(TOut) == 2) {
#pragma unroll
      for (int j = 0; j < CNT; ++j) acc[j] = __bfloat162float(__float2bfloat16_rn(acc[j]));
    }
    if (orow != nullptr) store_row<TOut, CNT>(orow, n0, ep.N, full, acc);
#pragma unroll
    for (int j = 0; j < CNT; ++j) acc[j] = gelu_tanh<kFast>(acc[j]);
  } else if (ep.mode == PTJ_EPI_GELU_BWD) {
    float a[CNT];
    load_row<TOut, CNT>(arow, n0, ep.N, full, a);
#pragma unroll
    for (int j = 0; j < CNT; ++j) acc[j] *= gelu_tanh_grad<kFast>(a[j]);
  } else if (ep.mode == PTJ_EPI_ACCUM) {
    float a[CNT];
    load_row<TOut, CNT>(crow, n0, ep.N, full, a);
#pragma unroll
    for (int j = 0; j < CNT; ++j) acc[j] += a[j];
  } else if (ep.mode == PTJ_EPI_DROPOUT_RESID) {
    float a[CNT];
    load_row<TOut, CNT>(arow, n0, ep.N, full, a);
    // mask indexed by the logical element position m * N + n (the stream ptj_dropout uses on a contiguous [M, N])
    const uint64_t base = static_cast<uint64_t>(m) * static_cast<uint64_t>(ep.N) + static_cast<uint64_t>(n0);
    if (!ep.train) {
#pragma unroll
      for (int j = 0; j < CNT; ++j) acc[j] = fmaf(acc[j], ep.eval_scale, a[j]);
    } else if (ep.drop_thr == 0u) {
#pragma unroll
      for (int j = 0; j < CNT; ++j) acc[j] += a[j];
    } else if ((base & 7) == 0) {
#pragma unroll
      for (int j = 0; j < CNT; j += 8) {
        const uint32_t keep = dropout_keep_bits8(ep.seed, ep.stream_id, (base + j) >> 3, ep.drop_thr);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[j + e] = a[j + e] + (((keep >> e) & 1u) ? acc[j + e] : 0.f);
      }
    } else {
#pragma unroll
      for (int j = 0; j < CNT; ++j)
        acc[j] = a[j] + (dropout_keep(ep.seed, ep.stream_id, base + j, ep.drop_thr) ? acc[j] : 0.f);
    }
  }
  store_row<TOut, CNT>(crow, n0, ep.N, full, acc);
}

}  // namespace ptj
