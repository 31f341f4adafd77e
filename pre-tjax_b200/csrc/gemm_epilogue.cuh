// Elementwise epilogue shared by the tensor-core and the SIMT GEMM kernels: bias, GELU (saving the pre-activation),
// GELU backward, dropout + residual, accumulate. Works on one row segment held in registers by one thread.
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
  uint32_t drop_thr;
  float eval_scale;
  int train;
  uint64_t seed;
  uint32_t stream_id;
};

// acc[0..CNT) are columns n0 .. n0+CNT-1 of row m. CNT is a multiple of 8.
template <typename TOut, int CNT>
__device__ __forceinline__ void epilogue_row_segment(const EpilogueParams& ep, int64_t m, int64_t n0, float (&acc)[CNT]) {
  constexpr int V = Elem<TOut>::kVec;
  if (m >= ep.M || n0 >= ep.N) return;
  TOut* crow = static_cast<TOut*>(ep.c) + m * ep.ldc;
  const TOut* arow = ep.aux ? static_cast<const TOut*>(ep.aux) + m * ep.ldc : nullptr;
  TOut* orow = ep.aux_out ? static_cast<TOut*>(ep.aux_out) + m * ep.ldc : nullptr;
  const bool full = ep.vec_ok && n0 + CNT <= ep.N;

  if (ep.bias != nullptr) {
#pragma unroll
    for (int j = 0; j < CNT; ++j)
      if (n0 + j < ep.N) acc[j] += ep.bias[n0 + j];
  }
  if (ep.mode == PTJ_EPI_GELU) {
    if (orow != nullptr) {
      if (full) {
#pragma unroll
        for (int j = 0; j < CNT; j += V) {
          float t[V];
#pragma unroll
          for (int q = 0; q < V; ++q) t[q] = acc[j + q];
          Elem<TOut>::store_vec(orow + n0 + j, t);
        }
      } else {
#pragma unroll
        for (int j = 0; j < CNT; ++j)
          if (n0 + j < ep.N) Elem<TOut>::store(orow + n0 + j, acc[j]);
      }
    }
    // the activation sees the value as stored (rounded to the output type), like a separate GELU kernel would
#pragma unroll
    for (int j = 0; j < CNT; ++j) {
      float x = acc[j];
      if (sizeof(TOut) == 2) x = __bfloat162float(__float2bfloat16_rn(x));
      acc[j] = gelu_tanh<sizeof(TOut) == 2>(x);
    }
  } else if (ep.mode == PTJ_EPI_GELU_BWD || ep.mode == PTJ_EPI_DROPOUT_RESID || ep.mode == PTJ_EPI_ACCUM) {
    float a[CNT];
    const TOut* src = ep.mode == PTJ_EPI_ACCUM ? crow : arow;
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
      for (int j = 0; j < CNT; ++j) a[j] = n0 + j < ep.N ? Elem<TOut>::load(src + n0 + j) : 0.f;
    }
    if (ep.mode == PTJ_EPI_GELU_BWD) {
#pragma unroll
      for (int j = 0; j < CNT; ++j) acc[j] *= gelu_tanh_grad<sizeof(TOut) == 2>(a[j]);
    } else if (ep.mode == PTJ_EPI_ACCUM) {
#pragma unroll
      for (int j = 0; j < CNT; ++j) acc[j] += a[j];
    } else {
      // dropout mask indexed by the logical element position m * N + n (same stream as ptj_dropout on [M, N])
      const uint64_t base = static_cast<uint64_t>(m) * static_cast<uint64_t>(ep.N) + static_cast<uint64_t>(n0);
      if (!ep.train) {
#pragma unroll
        for (int j = 0; j < CNT; ++j) acc[j] = a[j] + acc[j] * ep.eval_scale;
      } else if ((base & 3) == 0) {
#pragma unroll
        for (int j = 0; j < CNT; j += 4) {
          const Philox4 r = philox4x32_10(ep.seed, (base + j) >> 2, ep.stream_id);
          acc[j] = a[j] + (r.x >= ep.drop_thr ? acc[j] : 0.f);
          acc[j + 1] = a[j + 1] + (r.y >= ep.drop_thr ? acc[j + 1] : 0.f);
          acc[j + 2] = a[j + 2] + (r.z >= ep.drop_thr ? acc[j + 2] : 0.f);
          acc[j + 3] = a[j + 3] + (r.w >= ep.drop_thr ? acc[j + 3] : 0.f);
        }
      } else {
#pragma unroll
        for (int j = 0; j < CNT; ++j)
          acc[j] = a[j] + (dropout_keep(ep.seed, ep.stream_id, base + j, ep.drop_thr) ? acc[j] : 0.f);
      }
    }
  }
  if (full) {
#pragma unroll
    for (int j = 0; j < CNT; j += V) {
      float t[V];
#pragma unroll
      for (int q = 0; q < V; ++q) t[q] = acc[j + q];
      Elem<TOut>::store_vec(crow + n0 + j, t);
    }
  } else {
#pragma unroll
    for (int j = 0; j < CNT; ++j)
      if (n0 + j < ep.N) Elem<TOut>::store(crow + n0 + j, acc[j]);
  }
}

}  // namespace ptj
