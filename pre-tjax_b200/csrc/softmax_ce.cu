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

// ---- bf16 cross entropy, rows that start on a 16-byte boundary ---------------------------------------------------
// The kernel above spends about 25 instructions per logit (64-bit column arithmetic, arg-max bookkeeping and the
// online rescale inside the inner loop, a compare per element for the label) and is issue-bound at half of the memory
// roofline. This one walks the row three times with 16-byte vectors and does the least possible per element:
//   1. maximum only, on packed bf16 pairs (half an instruction per element);
//   2. sum of 2^((x - max) log2 e), two floats wide;
//   3. dlogits = 2^(x log2 e + c), with c = -max log2 e + log2(1 / (n_valid * sum)) folding both scale factors into
//      the exponent; the label's element is patched by one thread afterwards.
// Passes 2 and 3 read the row from L2 (512-thread blocks, three per SM: the 444 rows in flight, 100 KB each at
// GPT-2's vocabulary, stay well inside the L2). Accuracy: the label is the arg-max iff x[label] equals the maximum and no earlier column does (ties go to
// the first index, as in torch.argmax); the second condition is only walked for rows where the first holds.
constexpr int kCeThreads = 512;

__device__ __forceinline__ uint32_t bf2_max(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("max.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ float ex2_approx(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ uint64_t bf2_as_f2(uint32_t w) {
  return f2_pack(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
__device__ __forceinline__ uint64_t f2_add2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

constexpr float kLog2e = 1.4426950408889634f;

// maximum of a row (every thread gets it): packed bf16 pairs over the 16-byte vectors, the last cols & 7 elements one by one
__device__ __forceinline__ float row_max_bf16(const __nv_bfloat16* xr, int cols, float* red) {
  const uint4* xv = reinterpret_cast<const uint4*>(xr);
  const int nvec = cols >> 3;
  uint32_t pm = 0xff80ff80u;  // two packed -inf
  int i = threadIdx.x;
  for (; i + 3 * kCeThreads < nvec; i += 4 * kCeThreads) {
    const uint4 a = xv[i], b = xv[i + kCeThreads], c = xv[i + 2 * kCeThreads], d = xv[i + 3 * kCeThreads];
    pm = bf2_max(pm, bf2_max(bf2_max(bf2_max(a.x, a.y), bf2_max(a.z, a.w)), bf2_max(bf2_max(b.x, b.y), bf2_max(b.z, b.w))));
    pm = bf2_max(pm, bf2_max(bf2_max(bf2_max(c.x, c.y), bf2_max(c.z, c.w)), bf2_max(bf2_max(d.x, d.y), bf2_max(d.z, d.w))));
  }
  for (; i < nvec; i += kCeThreads) {
    const uint4 a = xv[i];
    pm = bf2_max(pm, bf2_max(bf2_max(a.x, a.y), bf2_max(a.z, a.w)));
  }
  float m = fmaxf(__uint_as_float(pm << 16), __uint_as_float(pm & 0xffff0000u));
  for (int c = (nvec << 3) + threadIdx.x; c < cols; c += kCeThreads) m = fmaxf(m, __bfloat162float(xr[c]));
  return block_max(m, red);
}

// sum over the row of 2^(x log2 e + nml), nml = -max log2 e (every thread gets it)
__device__ __forceinline__ float row_expsum_bf16(const __nv_bfloat16* xr, int cols, float nml, float* red) {
  const uint4* xv = reinterpret_cast<const uint4*>(xr);
  const int nvec = cols >> 3;
  const uint64_t l2e2 = f2_pack(kLog2e, kLog2e), nml2 = f2_pack(nml, nml);
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  auto add8 = [&](const uint4& a) {
    float e0, e1, e2, e3, e4, e5, e6, e7;
    f2_unpack(f2_fma(bf2_as_f2(a.x), l2e2, nml2), e0, e1);
    f2_unpack(f2_fma(bf2_as_f2(a.y), l2e2, nml2), e2, e3);
    f2_unpack(f2_fma(bf2_as_f2(a.z), l2e2, nml2), e4, e5);
    f2_unpack(f2_fma(bf2_as_f2(a.w), l2e2, nml2), e6, e7);
    s0 += ex2_approx(e0) + ex2_approx(e1);
    s1 += ex2_approx(e2) + ex2_approx(e3);
    s2 += ex2_approx(e4) + ex2_approx(e5);
    s3 += ex2_approx(e6) + ex2_approx(e7);
  };
  // (four loads in flight per thread, as in the maximum pass, measured no faster here: 344 against 340 us)
  for (int i = threadIdx.x; i < nvec; i += kCeThreads) add8(xv[i]);
  for (int c = (nvec << 3) + threadIdx.x; c < cols; c += kCeThreads) s0 += ex2_approx(fmaf(__bfloat162float(xr[c]), kLog2e, nml));
  return block_sum((s0 + s1) + (s2 + s3), red);
}

__global__ void __launch_bounds__(kCeThreads, 3)
cross_entropy_bf16_kernel(const int32_t* __restrict__ labels, const __nv_bfloat16* logits, __nv_bfloat16* dlogits,
                          float* __restrict__ row_stats, const float* __restrict__ n_valid, int64_t rows, int cols,
                          int64_t ld) {
  grid_dep_sync();
  __shared__ float red[33];
  const float inv_n = 1.f / *n_valid;
  const int nvec = cols >> 3;        // whole 16-byte vectors; the last cols & 7 elements are walked one by one
  const int tail0 = nvec << 3;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const __nv_bfloat16* xr = logits + row * ld;
    const uint4* xv = reinterpret_cast<const uint4*>(xr);
    __nv_bfloat16* dr = dlogits != nullptr ? dlogits + row * ld : nullptr;
    const int label = labels[row];
    if (label <= 0 || label >= cols) {  // padding (or an id outside the vocabulary): no contribution
      if (threadIdx.x == 0) {
        row_stats[row] = 0.f;
        row_stats[rows + row] = 0.f;
      }
      if (dr != nullptr) {
        for (int i = threadIdx.x; i < nvec; i += kCeThreads) reinterpret_cast<uint4*>(dr)[i] = make_uint4(0u, 0u, 0u, 0u);
        for (int c = tail0 + threadIdx.x; c < cols; c += kCeThreads) dr[c] = __float2bfloat16_rn(0.f);
      }
      continue;
    }
    const float x_label = __bfloat162float(xr[label]);  // read before the row is overwritten in place
    // pass 1: maximum
    const float m = row_max_bf16(xr, cols, red);
    // is the label the first column that attains the maximum?
    float hit = 0.f;
    if (x_label == m) {  // (uniform over the block)
      int earlier = 0;
      for (int c = threadIdx.x; c < label; c += kCeThreads) earlier |= (__bfloat162float(xr[c]) == m) ? 1 : 0;
      hit = __syncthreads_or(earlier) ? 0.f : 1.f;
    }
    // pass 2: sum of exponentials
    const float nml = -m * kLog2e;
    const uint64_t l2e2 = f2_pack(kLog2e, kLog2e);
    const float s = row_expsum_bf16(xr, cols, nml, red);
    if (threadIdx.x == 0) {
      row_stats[row] = -(x_label - m - logf(s));
      row_stats[rows + row] = hit;
    }
    if (dr == nullptr) continue;
    // pass 3: dlogits = softmax / n_valid, the label's column minus 1 / n_valid
    const float c3 = nml + log2f(inv_n / s);
    const uint64_t c32 = f2_pack(c3, c3);
    uint4* dv = reinterpret_cast<uint4*>(dr);
    auto grad8 = [&](const uint4& a) {
      const uint32_t w[4] = {a.x, a.y, a.z, a.w};
      uint32_t o[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float y0, y1;
        f2_unpack(f2_fma(bf2_as_f2(w[q]), l2e2, c32), y0, y1);
        __nv_bfloat162 h = __floats2bfloat162_rn(ex2_approx(y0), ex2_approx(y1));
        o[q] = *reinterpret_cast<uint32_t*>(&h);
      }
      return make_uint4(o[0], o[1], o[2], o[3]);
    };
    for (int i = threadIdx.x; i < nvec; i += kCeThreads) dv[i] = grad8(xv[i]);
    for (int c = tail0 + threadIdx.x; c < cols; c += kCeThreads)
      dr[c] = __float2bfloat16_rn(ex2_approx(fmaf(__bfloat162float(xr[c]), kLog2e, c3)));
    __syncthreads();  // the label's column has been written (by whichever thread owns it) before it is patched
    if (threadIdx.x == 0) dr[label] = __float2bfloat16_rn(ex2_approx(fmaf(x_label, kLog2e, c3)) - inv_n);
  }
}

// log-softmax forward / backward on the same three-pass scheme (bf16, every row on a 16-byte boundary)
__global__ void __launch_bounds__(kCeThreads, 3)
log_softmax_fwd_bf16_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, int64_t rows, int cols,
                            int64_t ld_x, int64_t ld_y) {
  grid_dep_sync();
  __shared__ float red[33];
  const int nvec = cols >> 3;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const __nv_bfloat16* xr = x + row * ld_x;
    __nv_bfloat16* yr = y + row * ld_y;
    const float m = row_max_bf16(xr, cols, red);
    const float s = row_expsum_bf16(xr, cols, -m * kLog2e, red);
    const float nshift = -(m + logf(s));
    const uint64_t ns2 = f2_pack(nshift, nshift);
    const uint4* xv = reinterpret_cast<const uint4*>(xr);
    uint4* yv = reinterpret_cast<uint4*>(yr);
    for (int i = threadIdx.x; i < nvec; i += kCeThreads) {
      const uint4 a = xv[i];
      const uint32_t w[4] = {a.x, a.y, a.z, a.w};
      uint32_t o[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float y0, y1;
        f2_unpack(f2_add2(bf2_as_f2(w[q]), ns2), y0, y1);
        __nv_bfloat162 h = __floats2bfloat162_rn(y0, y1);
        o[q] = *reinterpret_cast<uint32_t*>(&h);
      }
      yv[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
    for (int c = (nvec << 3) + threadIdx.x; c < cols; c += kCeThreads) yr[c] = __float2bfloat16_rn(__bfloat162float(xr[c]) + nshift);
  }
}

// dx = dy - softmax(x) * sum(dy)    (model_triton.py:91-102)
__global__ void __launch_bounds__(kCeThreads, 3)
log_softmax_bwd_bf16_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                            __nv_bfloat16* __restrict__ dx, int64_t rows, int cols, int64_t ld) {
  grid_dep_sync();
  __shared__ float red[33];
  const int nvec = cols >> 3;
  const int tail0 = nvec << 3;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const __nv_bfloat16* xr = x + row * ld;
    const __nv_bfloat16* gr = dy + row * ld;
    __nv_bfloat16* dr = dx + row * ld;
    const uint4* xv = reinterpret_cast<const uint4*>(xr);
    const uint4* gv = reinterpret_cast<const uint4*>(gr);
    const float m = row_max_bf16(xr, cols, red);
    const float nml = -m * kLog2e;
    const float s = row_expsum_bf16(xr, cols, nml, red);
    uint64_t g0 = 0ull, g1 = 0ull;  // two packed +0.0f each
    for (int i = threadIdx.x; i < nvec; i += kCeThreads) {
      const uint4 a = gv[i];
      g0 = f2_add2(g0, f2_add2(bf2_as_f2(a.x), bf2_as_f2(a.y)));
      g1 = f2_add2(g1, f2_add2(bf2_as_f2(a.z), bf2_as_f2(a.w)));
    }
    float ga, gb;
    f2_unpack(f2_add2(g0, g1), ga, gb);
    float gs = ga + gb;
    for (int c = tail0 + threadIdx.x; c < cols; c += kCeThreads) gs += __bfloat162float(gr[c]);
    const float nk = -block_sum(gs, red) / s;
    const uint64_t l2e2 = f2_pack(kLog2e, kLog2e), nml2 = f2_pack(nml, nml), nk2 = f2_pack(nk, nk);
    uint4* dv = reinterpret_cast<uint4*>(dr);
    for (int i = threadIdx.x; i < nvec; i += kCeThreads) {
      const uint4 a = xv[i], g = gv[i];
      const uint32_t w[4] = {a.x, a.y, a.z, a.w}, u[4] = {g.x, g.y, g.z, g.w};
      uint32_t o[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float y0, y1;
        f2_unpack(f2_fma(bf2_as_f2(w[q]), l2e2, nml2), y0, y1);
        f2_unpack(f2_fma(f2_pack(ex2_approx(y0), ex2_approx(y1)), nk2, bf2_as_f2(u[q])), y0, y1);
        __nv_bfloat162 h = __floats2bfloat162_rn(y0, y1);
        o[q] = *reinterpret_cast<uint32_t*>(&h);
      }
      dv[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
    for (int c = tail0 + threadIdx.x; c < cols; c += kCeThreads)
      dr[c] = __float2bfloat16_rn(fmaf(ex2_approx(fmaf(__bfloat162float(xr[c]), kLog2e, nml)), nk, __bfloat162float(gr[c])));
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
  } else if (dtype == PTJ_BF16 && aligned16(x) && aligned16(y) && ld_x % 8 == 0 && ld_y % 8 == 0 && cols <= 0x7fffffffLL) {
    const int64_t cap = static_cast<int64_t>(kNumSMs) * 3;
    launch_k(log_softmax_fwd_bf16_kernel, static_cast<int>(rows < cap ? rows : cap), kCeThreads, 0, st,
             static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), rows, static_cast<int>(cols), ld_x, ld_y);
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
  } else if (dtype == PTJ_BF16 && aligned16(x) && aligned16(dy) && aligned16(dx) && ld % 8 == 0 && cols <= 0x7fffffffLL) {
    const int64_t cap = static_cast<int64_t>(kNumSMs) * 3;
    launch_k(log_softmax_bwd_bf16_kernel, static_cast<int>(rows < cap ? rows : cap), kCeThreads, 0, st,
             static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(dx),
             rows, static_cast<int>(cols), ld);
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
  } else if (aligned16(logits) && (dlogits == nullptr || aligned16(dlogits)) && ld % 8 == 0 && cols <= 0x7fffffffLL) {
    const int64_t cap = static_cast<int64_t>(kNumSMs) * 3;  // three resident 512-thread blocks per SM
    launch_k(cross_entropy_bf16_kernel, static_cast<int>(rows < cap ? rows : cap), kCeThreads, 0, st, labels,
             static_cast<const __nv_bfloat16*>(logits), static_cast<__nv_bfloat16*>(dlogits), row_stats, n_valid, rows,
             static_cast<int>(cols), ld);
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
