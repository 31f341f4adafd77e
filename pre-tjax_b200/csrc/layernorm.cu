// LayerNorm forward / backward. Semantics of the reference: unbiased standard deviation (divide by n-1) and no
// epsilon (model_torch_func.py:104-108). Backward formula: model_triton.py:1773-1783 (dx) and :1652-1660 (dgamma,
// dbeta). HBM-bound: one warp owns one row, the row lives in registers between the statistics and the output pass,
// all global accesses are 16-byte vectors.
#include "common.cuh"

namespace ptj {
namespace {

constexpr int kLnThreads = 256;
constexpr int kLnWarps = kLnThreads / 32;

inline int ln_grid(int64_t rows) {
  int64_t blocks = ceil_div(rows, kLnWarps);
  int64_t cap = static_cast<int64_t>(kNumSMs) * 8;  // 8 resident 256-thread blocks per SM
  return static_cast<int>(blocks < cap ? blocks : cap);
}
inline int ln_bwd_grid(int64_t rows) {
  int64_t blocks = ceil_div(rows, kLnWarps);
  int64_t cap = static_cast<int64_t>(kNumSMs) * 2;
  return static_cast<int>(blocks < cap ? blocks : cap);
}

template <typename T, int NV>
__global__ void __launch_bounds__(kLnThreads)
ln_fwd_kernel(const T* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
              T* __restrict__ y, int64_t rows, int dim) {
  constexpr int V = Elem<T>::kVec;
  const int lane = threadIdx.x & 31;
  const int nvec = dim / V;
  float g[NV][V], b[NV][V];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = lane + 32 * i;
#pragma unroll
    for (int j = 0; j < V; ++j) {
      g[i][j] = vi < nvec ? gamma[vi * V + j] : 0.f;
      b[i][j] = vi < nvec ? beta[vi * V + j] : 0.f;
    }
  }
  const float inv_n = 1.f / static_cast<float>(dim), inv_nm1 = 1.f / static_cast<float>(dim - 1);
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * kLnWarps + (threadIdx.x >> 5); row < rows;
       row += static_cast<int64_t>(gridDim.x) * kLnWarps) {
    const T* xr = x + row * dim;
    float v[NV][V];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = lane + 32 * i;
      if (vi < nvec) {
        Elem<T>::load_vec(xr + vi * V, v[i]);
#pragma unroll
        for (int j = 0; j < V; ++j) s += v[i][j];
      } else {
#pragma unroll
        for (int j = 0; j < V; ++j) v[i][j] = 0.f;
      }
    }
    const float mean = warp_sum(s) * inv_n;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      if (lane + 32 * i < nvec) {
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float d = v[i][j] - mean;
          ss += d * d;
        }
      }
    }
    const float rstd = 1.f / sqrtf(warp_sum(ss) * inv_nm1);
    T* yr = y + row * dim;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = lane + 32 * i;
      if (vi < nvec) {
        float o[V];
#pragma unroll
        for (int j = 0; j < V; ++j) o[j] = g[i][j] * ((v[i][j] - mean) * rstd) + b[i][j];
        Elem<T>::store_vec(yr + vi * V, o);
      }
    }
  }
}

// Any dim / alignment: one block per row, scalar accesses.
template <typename T>
__global__ void __launch_bounds__(kLnThreads)
ln_fwd_generic_kernel(const T* __restrict__ x, const float* __restrict__ gamma,
                      const float* __restrict__ beta, T* __restrict__ y, int64_t rows, int dim) {
  __shared__ float red[33];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * dim;
    float s = 0.f;
    for (int c = threadIdx.x; c < dim; c += blockDim.x) s += Elem<T>::load(xr + c);
    const float mean = block_sum(s, red) / static_cast<float>(dim);
    float ss = 0.f;
    for (int c = threadIdx.x; c < dim; c += blockDim.x) {
      const float d = Elem<T>::load(xr + c) - mean;
      ss += d * d;
    }
    const float rstd = 1.f / sqrtf(block_sum(ss, red) / static_cast<float>(dim - 1));
    for (int c = threadIdx.x; c < dim; c += blockDim.x)
      Elem<T>::store(y + row * dim + c, gamma[c] * ((Elem<T>::load(xr + c) - mean) * rstd) + beta[c]);
  }
}

// dx and the per-block partial sums of dgamma / dbeta in one pass over (dy, x).
template <typename T, int NV>
__global__ void __launch_bounds__(kLnThreads)
ln_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ gamma,
              const T* dx_add, T* dx, float* __restrict__ partial, int64_t rows, int dim) {
  constexpr int V = Elem<T>::kVec;
  extern __shared__ float sm_acc[];  // [2][dim]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nvec = dim / V;
  float g[NV][V], dg[NV][V], db[NV][V];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = lane + 32 * i;
#pragma unroll
    for (int j = 0; j < V; ++j) {
      g[i][j] = vi < nvec ? gamma[vi * V + j] : 0.f;
      dg[i][j] = 0.f;
      db[i][j] = 0.f;
    }
  }
  const float inv_n = 1.f / static_cast<float>(dim), inv_nm1 = 1.f / static_cast<float>(dim - 1);
  const float n_adj = static_cast<float>(dim) * inv_nm1;
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * kLnWarps + warp; row < rows;
       row += static_cast<int64_t>(gridDim.x) * kLnWarps) {
    const T* xr = x + row * dim;
    const T* gr = dy + row * dim;
    float v[NV][V], u[NV][V];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = lane + 32 * i;
      if (vi < nvec) {
        Elem<T>::load_vec(xr + vi * V, v[i]);
        Elem<T>::load_vec(gr + vi * V, u[i]);
#pragma unroll
        for (int j = 0; j < V; ++j) s += v[i][j];
      } else {
#pragma unroll
        for (int j = 0; j < V; ++j) { v[i][j] = 0.f; u[i][j] = 0.f; }
      }
    }
    const float mean = warp_sum(s) * inv_n;
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      if (lane + 32 * i < nvec) {
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float d = v[i][j] - mean;
          ss += d * d;
        }
      }
    }
    const float rstd = 1.f / sqrtf(warp_sum(ss) * inv_nm1);
    // xhat, parameter-gradient partials, and the two row means of the dx formula
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      if (lane + 32 * i < nvec) {
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float xh = (v[i][j] - mean) * rstd;
          v[i][j] = xh;
          dg[i][j] += u[i][j] * xh;
          db[i][j] += u[i][j];
          const float gh = u[i][j] * g[i][j];
          u[i][j] = gh;
          s1 += gh;
          s2 += gh * xh;
        }
      }
    }
    if (dx != nullptr) {
      const float m1 = warp_sum(s1) * inv_n;
      const float m2 = warp_sum(s2) * inv_n * n_adj;
      T* dr = dx + row * dim;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int vi = lane + 32 * i;
        if (vi < nvec) {
          float o[V];
#pragma unroll
          for (int j = 0; j < V; ++j) o[j] = (u[i][j] - m1 - v[i][j] * m2) * rstd;
          if (dx_add != nullptr) {  // gradient arriving over the residual connection
            float r[V];
            Elem<T>::load_vec(dx_add + row * dim + vi * V, r);
#pragma unroll
            for (int j = 0; j < V; ++j) o[j] += r[j];
          }
          Elem<T>::store_vec(dr + vi * V, o);
        }
      }
    }
  }
  if (partial == nullptr) return;
  // warps fold their register partials into shared memory one after another: fixed order => reproducible
  for (int w = 0; w < kLnWarps; ++w) {
    if (warp == w) {
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int vi = lane + 32 * i;
        if (vi < nvec) {
#pragma unroll
          for (int j = 0; j < V; ++j) {
            const int c = vi * V + j;
            if (w == 0) {
              sm_acc[c] = dg[i][j];
              sm_acc[dim + c] = db[i][j];
            } else {
              sm_acc[c] += dg[i][j];
              sm_acc[dim + c] += db[i][j];
            }
          }
        }
      }
    }
    __syncthreads();
  }
  float* out = partial + static_cast<size_t>(blockIdx.x) * 2 * dim;
  for (int c = threadIdx.x; c < 2 * dim; c += blockDim.x) out[c] = sm_acc[c];
}

template <typename T>
__global__ void __launch_bounds__(kLnThreads)
ln_bwd_generic_kernel(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ gamma,
                      const T* dx_add, T* dx, float* __restrict__ partial, int64_t rows, int dim) {
  __shared__ float red[33];
  float* out = partial ? partial + static_cast<size_t>(blockIdx.x) * 2 * dim : nullptr;
  if (out)
    for (int c = threadIdx.x; c < 2 * dim; c += blockDim.x) out[c] = 0.f;
  const float n_adj = static_cast<float>(dim) / static_cast<float>(dim - 1);
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * dim;
    const T* gr = dy + row * dim;
    float s = 0.f;
    for (int c = threadIdx.x; c < dim; c += blockDim.x) s += Elem<T>::load(xr + c);
    const float mean = block_sum(s, red) / static_cast<float>(dim);
    float ss = 0.f;
    for (int c = threadIdx.x; c < dim; c += blockDim.x) {
      const float d = Elem<T>::load(xr + c) - mean;
      ss += d * d;
    }
    const float rstd = 1.f / sqrtf(block_sum(ss, red) / static_cast<float>(dim - 1));
    float s1 = 0.f, s2 = 0.f;
    for (int c = threadIdx.x; c < dim; c += blockDim.x) {
      const float xh = (Elem<T>::load(xr + c) - mean) * rstd;
      const float u = Elem<T>::load(gr + c);
      if (out) {  // column c is only ever touched by this thread of this block
        out[c] += u * xh;
        out[dim + c] += u;
      }
      s1 += u * gamma[c];
      s2 += u * gamma[c] * xh;
    }
    if (dx != nullptr) {
      const float m1 = block_sum(s1, red) / static_cast<float>(dim);
      const float m2 = block_sum(s2, red) / static_cast<float>(dim) * n_adj;
      for (int c = threadIdx.x; c < dim; c += blockDim.x) {
        const float xh = (Elem<T>::load(xr + c) - mean) * rstd;
        const float gh = Elem<T>::load(gr + c) * gamma[c];
        const float r = dx_add != nullptr ? Elem<T>::load(dx_add + row * dim + c) : 0.f;
        Elem<T>::store(dx + row * dim + c, (gh - m1 - xh * m2) * rstd + r);
      }
    }
  }
}

// dgamma[c] = sum over blocks of partial[b][0][c], dbeta likewise; blocks summed in index order.
__global__ void ln_bwd_finalize_kernel(const float* __restrict__ partial, float* __restrict__ dgamma,
                                       float* __restrict__ dbeta, int nblocks, int dim) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= 2 * dim) return;
  float s = 0.f;
  for (int b = 0; b < nblocks; ++b) s += partial[static_cast<size_t>(b) * 2 * dim + c];
  if (c < dim) dgamma[c] = s; else dbeta[c - dim] = s;
}

template <typename T>
int launch_fwd(const T* x, const float* gamma, const float* beta, T* y, int64_t rows, int dim, cudaStream_t st) {
  constexpr int V = Elem<T>::kVec;
  const bool vec_ok = dim % V == 0 && aligned16(x) && aligned16(y);
  const int nv = vec_ok ? static_cast<int>(ceil_div(dim / V, 32)) : 99;
  const int grid = ln_grid(rows);
#define PTJ_LN_FWD(NV) case NV: ln_fwd_kernel<T, NV><<<grid, kLnThreads, 0, st>>>(x, gamma, beta, y, rows, dim); break;
  switch (nv) {
    PTJ_LN_FWD(1) PTJ_LN_FWD(2) PTJ_LN_FWD(3) PTJ_LN_FWD(4) PTJ_LN_FWD(5) PTJ_LN_FWD(6) PTJ_LN_FWD(7) PTJ_LN_FWD(8)
    default: {
      const int g = static_cast<int>(rows < kNumSMs * 8 ? rows : kNumSMs * 8);
      ln_fwd_generic_kernel<T><<<g, kLnThreads, 0, st>>>(x, gamma, beta, y, rows, dim);
    }
  }
#undef PTJ_LN_FWD
  PTJ_CHECK_LAUNCH();
  return PTJ_OK;
}

template <typename T>
int launch_bwd(const T* dy, const T* x, const float* gamma, const T* dx_add, T* dx, float* dgamma, float* dbeta,
               float* scratch, int64_t rows, int dim, cudaStream_t st) {
  constexpr int V = Elem<T>::kVec;
  const bool vec_ok = dim % V == 0 && aligned16(x) && aligned16(dy) && (dx == nullptr || aligned16(dx)) &&
                      (dx_add == nullptr || aligned16(dx_add)) &&
                      static_cast<size_t>(dim) * 2 * sizeof(float) <= 96 * 1024;
  const int nv = vec_ok ? static_cast<int>(ceil_div(dim / V, 32)) : 99;
  const int grid = ln_bwd_grid(rows);
  float* partial = dgamma != nullptr ? scratch : nullptr;
  const size_t smem = static_cast<size_t>(dim) * 2 * sizeof(float);
#define PTJ_LN_BWD(NV)                                                                                   \
  case NV:                                                                                               \
    if (smem > 48 * 1024)                                                                                \
      cudaFuncSetAttribute(ln_bwd_kernel<T, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    ln_bwd_kernel<T, NV><<<grid, kLnThreads, smem, st>>>(dy, x, gamma, dx_add, dx, partial, rows, dim);           \
    break;
  switch (nv) {
    PTJ_LN_BWD(1) PTJ_LN_BWD(2) PTJ_LN_BWD(3) PTJ_LN_BWD(4) PTJ_LN_BWD(5) PTJ_LN_BWD(6) PTJ_LN_BWD(7) PTJ_LN_BWD(8)
    default:
      ln_bwd_generic_kernel<T><<<grid, kLnThreads, 0, st>>>(dy, x, gamma, dx_add, dx, partial, rows, dim);
  }
#undef PTJ_LN_BWD
  PTJ_CHECK_LAUNCH();
  if (partial != nullptr) {
    ln_bwd_finalize_kernel<<<static_cast<int>(ceil_div(2 * dim, 256)), 256, 0, st>>>(partial, dgamma, dbeta, grid, dim);
    PTJ_CHECK_LAUNCH();
  }
  return PTJ_OK;
}

}  // namespace
}  // namespace ptj

using namespace ptj;

extern "C" int ptj_layernorm_fwd(const void* x, const float* gamma, const float* beta, void* y, int64_t rows,
                                 int64_t dim, int dtype, void* stream) {
  if (rows < 0 || dim < 1 || dim > (1 << 20)) return PTJ_ERR_BAD_SHAPE;
  if (rows == 0) return PTJ_OK;
  if (!x || !gamma || !beta || !y) return PTJ_ERR_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == PTJ_F32)
    return launch_fwd(static_cast<const float*>(x), gamma, beta, static_cast<float*>(y), rows, (int)dim, st);
  if (dtype == PTJ_BF16)
    return launch_fwd(static_cast<const __nv_bfloat16*>(x), gamma, beta, static_cast<__nv_bfloat16*>(y), rows,
                      (int)dim, st);
  return PTJ_ERR_DTYPE;
}

extern "C" size_t ptj_layernorm_bwd_scratch_floats(int64_t rows, int64_t dim) {
  if (rows <= 0 || dim <= 0) return 0;
  return static_cast<size_t>(ln_bwd_grid(rows)) * 2 * static_cast<size_t>(dim);
}

extern "C" int ptj_layernorm_bwd(const void* dy, const void* x, const float* gamma, const void* dx_add, void* dx,
                                 float* dgamma, float* dbeta, float* scratch, size_t scratch_floats, int64_t rows,
                                 int64_t dim, int dtype, void* stream) {
  if (rows < 0 || dim < 1 || dim > (1 << 20)) return PTJ_ERR_BAD_SHAPE;
  if ((dgamma == nullptr) != (dbeta == nullptr)) return PTJ_ERR_BAD_SHAPE;
  if (!dy || !x || !gamma) return PTJ_ERR_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (rows == 0) {
    if (dgamma) {
      cudaMemsetAsync(dgamma, 0, sizeof(float) * dim, st);
      cudaMemsetAsync(dbeta, 0, sizeof(float) * dim, st);
    }
    return PTJ_OK;
  }
  if (dgamma && (scratch == nullptr || scratch_floats < ptj_layernorm_bwd_scratch_floats(rows, dim)))
    return PTJ_ERR_WORKSPACE;
  if (dtype == PTJ_F32)
    return launch_bwd(static_cast<const float*>(dy), static_cast<const float*>(x), gamma,
                      static_cast<const float*>(dx_add), static_cast<float*>(dx), dgamma, dbeta, scratch, rows, (int)dim,
                      st);
  if (dtype == PTJ_BF16)
    return launch_bwd(static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x), gamma,
                      static_cast<const __nv_bfloat16*>(dx_add), static_cast<__nv_bfloat16*>(dx), dgamma, dbeta, scratch,
                      rows, (int)dim, st);
  return PTJ_ERR_DTYPE;
}
