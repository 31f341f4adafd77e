// Row-wise log-softmax forward/backward and the fused cross-entropy forward+backward over a large vocabulary.
// One thread block owns one row at a time. Pass 1 is an online max / sum-of-exponentials over 16-byte vectors
// (Milakov & Gimelshein, "Online normalizer calculation for softmax"); pass 2 re-reads the row (it is still in
// L2: a row of 50257 bf16 is 100 KB) and writes the result with plain vector stores. No atomics, no helper tensors.
#include "common.cuh"

namespace ptj {
namespace {

constexpr int kRowThreads = 256;

inline int row_grid(int64_t rows) {
  int64_t cap = static_cast<int64_t>(kNumSMs) * 8;
  return static_cast<int>(rows < cap ? rows : cap);
}

template <typename T> __device__ __forceinline__ float fast_exp(float x);
template <> __device__ __forceinline__ float fast_exp<float>(float x) { return expf(x); }
template <> __device__ __forceinline__ float fast_exp<__nv_bfloat16>(float x) { return __expf(x); }

// Number of leading scalar elements before `p` reaches a 16-byte boundary (0 when vectors are not usable).
template <typename T>
__device__ __forceinline__ int head_elems(const T* p, int64_t cols, bool vec) {
  if (!vec) return static_cast<int>(cols < 0x7fffffff ? cols : 0x7fffffff);
  const uintptr_t mis = (reinterpret_cast<uintptr_t>(p) & 15u) / sizeof(T);
  const int h = static_cast<int>((Elem<T>::kVec - mis) % Elem<T>::kVec);
  return h < cols ? h : static_cast<int>(cols);
}

// Visit every column of a row: f1(col) for scalar positions, fv(col) for aligned vectors starting at col.
template <typename T, typename F1, typename FV>
__device__ __forceinline__ void row_visit(int64_t cols, int head, bool vec, F1 f1, FV fv) {
  constexpr int V = Elem<T>::kVec;
  for (int64_t c = threadIdx.x; c < head; c += blockDim.x) f1(c);
  if (!vec) return;  // head == cols in scalar mode
  const int64_t nvec = (cols - head) / V;
  for (int64_t i = threadIdx.x; i < nvec; i += blockDim.x) fv(head + i * V);
  for (int64_t c = head + nvec * V + threadIdx.x; c < cols; c += blockDim.x) f1(c);
}

struct MaxSum {
  float m, s;
  int64_t arg;
};

// Online (max, sum exp(x - max), argmax) of one row; every thread returns the block-wide result.
template <typename T, bool WANT_ARG>
__device__ __forceinline__ MaxSum row_max_sum(const T* xr, int64_t cols, int head, bool vec, float* red,
                                              int64_t* red_arg) {
  constexpr int V = Elem<T>::kVec;
  float m = -INFINITY, s = 0.f;
  int64_t arg = 0;
  row_visit<T>(
      cols, head, vec,
      [&](int64_t c) {
        const float x = Elem<T>::load(xr + c);
        if (x > m) {
          s = s * fast_exp<T>(m - x) + 1.f;
          m = x;
          arg = c;
        } else {
          s += fast_exp<T>(x - m);
        }
      },
      [&](int64_t c) {
        float v[V];
        Elem<T>::load_vec(xr + c, v);
        float vm = v[0];
        int am = 0;
#pragma unroll
        for (int j = 1; j < V; ++j)
          if (v[j] > vm) { vm = v[j]; am = j; }
        if (vm > m) {
          s *= fast_exp<T>(m - vm);
          m = vm;
          arg = c + am;
        }
#pragma unroll
        for (int j = 0; j < V; ++j) s += fast_exp<T>(v[j] - m);
      });
  const float bm = block_max(m, red);
  // first index attaining the maximum (the convention of torch.argmax on CPU)
  int64_t best = 0;
  if (WANT_ARG) {
    int64_t cand = (m == bm && s > 0.f) ? arg : INT64_MAX;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const int64_t other = __shfl_xor_sync(0xffffffffu, cand, o);
      cand = other < cand ? other : cand;
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red_arg[threadIdx.x >> 5] = cand;
    __syncthreads();
    best = INT64_MAX;
    for (int w = 0; w < (blockDim.x >> 5); ++w) best = red_arg[w] < best ? red_arg[w] : best;
  }
  const float bs = block_sum(s > 0.f ? s * fast_exp<T>(m - bm) : 0.f, red);
  return MaxSum{bm, bs, best};
}

template <typename T>
__global__ void __launch_bounds__(kRowThreads)
log_softmax_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int64_t cols, int64_t ld_x,
                       int64_t ld_y, bool vec) {
  grid_dep_sync();
  constexpr int V = Elem<T>::kVec;
  __shared__ float red[33];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * ld_x;
    T* yr = y + row * ld_y;
    const int head = head_elems(xr, cols, vec);
    const MaxSum ms = row_max_sum<T, false>(xr, cols, head, vec, red, nullptr);
    const float shift = ms.m + logf(ms.s);
    row_visit<T>(
        cols, head, vec, [&](int64_t c) { Elem<T>::store(yr + c, Elem<T>::load(xr + c) - shift); },
        [&](int64_t c) {
          float v[V];
          Elem<T>::load_vec(xr + c, v);
#pragma unroll
          for (int j = 0; j < V; ++j) v[j] -= shift;
          Elem<T>::store_vec(yr + c, v);
        });
  }
}

// dx = dy - softmax(x) * sum(dy)    (model_triton.py:91-102)
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
log_softmax_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, T* __restrict__ dx, int64_t rows,
                       int64_t cols, int64_t ld, bool vec) {
  grid_dep_sync();
  constexpr int V = Elem<T>::kVec;
  __shared__ float red[33];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * ld;
    const T* gr = dy + row * ld;
    T* dr = dx + row * ld;
    const int head = head_elems(xr, cols, vec);
    const MaxSum ms = row_max_sum<T, false>(xr, cols, head, vec, red, nullptr);
    float gs = 0.f;
    row_visit<T>(
        cols, head, vec, [&](int64_t c) { gs += Elem<T>::load(gr + c); },
        [&](int64_t c) {
          float v[V];
          Elem<T>::load_vec(gr + c, v);
#pragma unroll
          for (int j = 0; j < V; ++j) gs += v[j];
        });
    const float gsum = block_sum(gs, red);
    const float k = gsum / ms.s;
    row_visit<T>(
        cols, head, vec,
        [&](int64_t c) {
          Elem<T>::store(dr + c, Elem<T>::load(gr + c) - fast_exp<T>(Elem<T>::load(xr + c) - ms.m) * k);
        },
        [&](int64_t c) {
          float v[V], g[V];
          Elem<T>::load_vec(xr + c, v);
          Elem<T>::load_vec(gr + c, g);
#pragma unroll
          for (int j = 0; j < V; ++j) g[j] -= fast_exp<T>(v[j] - ms.m) * k;
          Elem<T>::store_vec(dr + c, g);
        });
  }
}

// Rows that contribute: the same predicate the cross-entropy kernel applies (a label that is not padding and lies
// inside the vocabulary), so that the divisor always matches the rows that were summed.
__global__ void count_valid_kernel(const int32_t* __restrict__ labels, int64_t rows, int64_t cols,
                                   float* __restrict__ n_valid) {
  grid_dep_sync();
  __shared__ float red[33];
  float c = 0.f;
  for (int64_t i = threadIdx.x; i < rows; i += blockDim.x) c += (labels[i] > 0 && labels[i] < cols) ? 1.f : 0.f;
  const float t = block_sum(c, red);  // exact: counts stay far below 2^24 per thread and in total
  if (threadIdx.x == 0) *n_valid = t;
}

// Fused forward + backward of the mean cross entropy over non-padding rows
// (loss_and_optimizer_triton.py:83-106): dlogits = (softmax - onehot) / n_valid, zero rows where label == 0.
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
cross_entropy_kernel(const int32_t* __restrict__ labels, const T* logits, T* dlogits,
                     float* __restrict__ row_stats, const float* __restrict__ n_valid, int64_t rows, int64_t cols,
                     int64_t ld, bool vec) {
  grid_dep_sync();
  constexpr int V = Elem<T>::kVec;
  __shared__ float red[33];
  __shared__ int64_t red_arg[kRowThreads / 32];
  const float inv_n = 1.f / *n_valid;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = logits + row * ld;
    T* dr = dlogits != nullptr ? dlogits + row * ld : nullptr;
    const int head = head_elems(xr, cols, vec);
    const int64_t label = labels[row];
    if (label == 0 || label < 0 || label >= cols) {  // padding (or an id outside the vocabulary): no contribution
      if (threadIdx.x == 0) {
        row_stats[row] = 0.f;
        row_stats[rows + row] = 0.f;
      }
      if (dr != nullptr) {
        row_visit<T>(
            cols, head, vec, [&](int64_t c) { Elem<T>::store(dr + c, 0.f); },
            [&](int64_t c) {
              float z[V];
#pragma unroll
              for (int j = 0; j < V; ++j) z[j] = 0.f;
              Elem<T>::store_vec(dr + c, z);
            });
      }
      continue;
    }
    const float x_label = Elem<T>::load(xr + label);  // read before the row is overwritten in place
    const MaxSum ms = row_max_sum<T, true>(xr, cols, head, vec, red, red_arg);
    if (threadIdx.x == 0) {
      row_stats[row] = -(x_label - ms.m - logf(ms.s));
      row_stats[rows + row] = ms.arg == label ? 1.f : 0.f;
    }
    if (dr != nullptr) {
      const float k = inv_n / ms.s;
      row_visit<T>(
          cols, head, vec,
          [&](int64_t c) {
            const float g = fast_exp<T>(Elem<T>::load(xr + c) - ms.m) * k - (c == label ? inv_n : 0.f);
            Elem<T>::store(dr + c, g);
          },
          [&](int64_t c) {
            float v[V];
            Elem<T>::load_vec(xr + c, v);
#pragma unroll
            for (int j = 0; j < V; ++j) v[j] = fast_exp<T>(v[j] - ms.m) * k - (c + j == label ? inv_n : 0.f);
            Elem<T>::store_vec(dr + c, v);
          });
    }
  }
}

__global__ void ce_finalize_kernel(const float* __restrict__ row_stats, const float* __restrict__ n_valid,
                                   int64_t rows, float* __restrict__ out3) {
  grid_dep_sync();
  __shared__ float red[33];
  float l = 0.f, h = 0.f;
  for (int64_t i = threadIdx.x; i < rows; i += blockDim.x) {
    l += row_stats[i];
    h += row_stats[rows + i];
  }
  const float lt = block_sum(l, red);
  const float ht = block_sum(h, red);
  if (threadIdx.x == 0) {
    const float n = *n_valid;
    out3[0] = lt / n;  // 0/0 = NaN when every row is padding, like torch.nanmean of all-NaN
    out3[1] = ht / n;
    out3[2] = n / static_cast<float>(rows);
  }
}

// Index of the largest element of every row (first index on ties): the greedy-decoding step of `predict`
// (loss_and_optimizer_triton.py:203-212), which the reference takes with torch.argmax over a logits slice.
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
argmax_rows_kernel(const T* __restrict__ x, int32_t* __restrict__ out, int64_t rows, int64_t cols, int64_t ld) {
  grid_dep_sync();
  __shared__ float red[33];
  __shared__ int64_t red_arg[kRowThreads / 32];
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * ld;
    const MaxSum ms = row_max_sum<T, true>(xr, cols, head_elems(xr, cols, true), true, red, red_arg);
    if (threadIdx.x == 0) out[row] = static_cast<int32_t>(ms.arg);
    __syncthreads();
  }
}

// Vector mode needs every tensor of a row to share the same distance to a 16-byte boundary.
template <typename T>
bool same_phase(const void* a, int64_t lda, const void* b, int64_t ldb) {
  if (b == nullptr) return true;
  const bool base = (reinterpret_cast<uintptr_t>(a) & 15u) == (reinterpret_cast<uintptr_t>(b) & 15u);
  const bool step = (static_cast<uint64_t>(lda) * sizeof(T)) % 16 == (static_cast<uint64_t>(ldb) * sizeof(T)) % 16;
  return base && step;
}

}  // namespace
}  // namespace ptj

using namespace ptj;

extern "C" int ptj_log_softmax_fwd(const void* x, void* y, int64_t rows, int64_t cols, int64_t ld_x, int64_t ld_y,
                                   int dtype, void* stream) {
  if (rows < 0 || cols < 1 || ld_x < cols || ld_y < cols) return PTJ_ERR_BAD_SHAPE;
  if (rows == 0) return PTJ_OK;
  if (!x || !y) return PTJ_ERR_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == PTJ_F32) {
    launch_k(log_softmax_fwd_kernel<float>, row_grid(rows), kRowThreads, 0, st, 
        static_cast<const float*>(x), static_cast<float*>(y), rows, cols, ld_x, ld_y, same_phase<float>(x, ld_x, y, ld_y));
  } else if (dtype == PTJ_BF16) {
    launch_k(log_softmax_fwd_kernel<__nv_bfloat16>, row_grid(rows), kRowThreads, 0, st, 
        static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), rows, cols, ld_x, ld_y,
        same_phase<__nv_bfloat16>(x, ld_x, y, ld_y));
  } else {
    return PTJ_ERR_DTYPE;
  }
  PTJ_CHECK_LAUNCH();
  return PTJ_OK;
}

extern "C" int ptj_log_softmax_bwd(const void* dy, const void* x, void* dx, int64_t rows, int64_t cols, int64_t ld,
                                   int dtype, void* stream) {
  if (rows < 0 || cols < 1 || ld < cols) return PTJ_ERR_BAD_SHAPE;
  if (rows == 0) return PTJ_OK;
  if (!dy || !x || !dx) return PTJ_ERR_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == PTJ_F32) {
    const bool vec = same_phase<float>(x, ld, dy, ld) && same_phase<float>(x, ld, dx, ld);
    launch_k(log_softmax_bwd_kernel<float>, row_grid(rows), kRowThreads, 0, st, 
        static_cast<const float*>(dy), static_cast<const float*>(x), static_cast<float*>(dx), rows, cols, ld, vec);
  } else if (dtype == PTJ_BF16) {
    const bool vec = same_phase<__nv_bfloat16>(x, ld, dy, ld) && same_phase<__nv_bfloat16>(x, ld, dx, ld);
    launch_k(log_softmax_bwd_kernel<__nv_bfloat16>, row_grid(rows), kRowThreads, 0, st, 
        static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(dx),
        rows, cols, ld, vec);
  } else {
    return PTJ_ERR_DTYPE;
  }
  PTJ_CHECK_LAUNCH();
  return PTJ_OK;
}

extern "C" int ptj_cross_entropy(const int32_t* labels, const void* logits, void* dlogits, float* row_stats,
                                 float* n_valid, int count_in_kernel, float* out3, int64_t rows, int64_t cols,
                                 int64_t ld, int dtype, void* stream) {
  if (rows < 1 || cols < 1 || ld < cols) return PTJ_ERR_BAD_SHAPE;
  if (!labels || !logits || !row_stats || !n_valid || !out3) return PTJ_ERR_BAD_SHAPE;
  if (dtype != PTJ_F32 && dtype != PTJ_BF16) return PTJ_ERR_DTYPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (count_in_kernel) {
    launch_k(count_valid_kernel, 1, 1024, 0, st, labels, rows, cols, n_valid);
    PTJ_CHECK_LAUNCH();
  }
  if (dtype == PTJ_F32) {
    launch_k(cross_entropy_kernel<float>, row_grid(rows), kRowThreads, 0, st, 
        labels, static_cast<const float*>(logits), static_cast<float*>(dlogits), row_stats, n_valid, rows, cols, ld,
        same_phase<float>(logits, ld, dlogits, ld));
  } else {
    launch_k(cross_entropy_kernel<__nv_bfloat16>, row_grid(rows), kRowThreads, 0, st, 
        labels, static_cast<const __nv_bfloat16*>(logits), static_cast<__nv_bfloat16*>(dlogits), row_stats, n_valid,
        rows, cols, ld, same_phase<__nv_bfloat16>(logits, ld, dlogits, ld));
  }
  PTJ_CHECK_LAUNCH();
  launch_k(ce_finalize_kernel, 1, 1024, 0, st, row_stats, n_valid, rows, out3);
  PTJ_CHECK_LAUNCH();
  return PTJ_OK;
}

extern "C" int ptj_argmax_rows(const void* x, int32_t* out, int64_t rows, int64_t cols, int64_t ld, int dtype,
                               void* stream) {
  if (rows < 0 || cols < 1 || cols > 0x7fffffffLL || ld < cols) return PTJ_ERR_BAD_SHAPE;
  if (rows == 0) return PTJ_OK;
  if (!x || !out) return PTJ_ERR_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == PTJ_F32) {
    launch_k(argmax_rows_kernel<float>, row_grid(rows), kRowThreads, 0, st, static_cast<const float*>(x), out, rows,
             cols, ld);
  } else if (dtype == PTJ_BF16) {
    launch_k(argmax_rows_kernel<__nv_bfloat16>, row_grid(rows), kRowThreads, 0, st,
             static_cast<const __nv_bfloat16*>(x), out, rows, cols, ld);
  } else {
    return PTJ_ERR_DTYPE;
  }
  PTJ_CHECK_LAUNCH();
  return PTJ_OK;
}
