// Elementwise HBM-bound operators: tanh-GELU forward/backward, dropout (+ residual add), fp32 -> bf16 cast.
// One 16-byte vector per thread per iteration, grid-stride, grid = multiple of the SM count.
#include "common.cuh"

namespace ptj {
namespace {

constexpr int kEwThreads = 256;

inline int ew_grid(int64_t nvec) {
  int64_t blocks = ceil_div(nvec, kEwThreads);
  int64_t cap = static_cast<int64_t>(kNumSMs) * 16;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks < cap ? blocks : cap);
}

// OP: 0 = gelu forward (a = x), 1 = gelu backward (a = dy, b = x_preact)
template <typename T, int OP>
__global__ void __launch_bounds__(kEwThreads)
gelu_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, int64_t n, bool vec) {
  grid_dep_sync();
  constexpr int V = Elem<T>::kVec;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t nvec = vec ? n / V : 0;
  for (int64_t i = tid; i < nvec; i += stride) {
    float va[V], vb[V], o[V];
    Elem<T>::load_vec(a + i * V, va);
    if (OP == 1) Elem<T>::load_vec(b + i * V, vb);
#pragma unroll
    for (int j = 0; j < V; ++j)
      o[j] = OP == 0 ? gelu_tanh<sizeof(T) == 2>(va[j]) : va[j] * gelu_tanh_grad<sizeof(T) == 2>(vb[j]);
    Elem<T>::store_vec(out + i * V, o);
  }
  for (int64_t i = nvec * V + tid; i < n; i += stride) {
    const float x = Elem<T>::load(a + i);
    Elem<T>::store(out + i, OP == 0 ? gelu_tanh<sizeof(T) == 2>(x) : x * gelu_tanh_grad<sizeof(T) == 2>(Elem<T>::load(b + i)));
  }
}

// y = (resid ? resid : 0) + x * mask   (train)   or   + x * (1 - p)   (eval)
template <typename T>
__global__ void __launch_bounds__(kEwThreads)
dropout_kernel(const T* __restrict__ x, const T* __restrict__ resid, T* __restrict__ y, int64_t n, bool vec,
               uint32_t thr, float eval_scale, int train, uint64_t seed, uint32_t stream_id) {
  grid_dep_sync();
  seed = resolve_seed(seed);
  constexpr int V = Elem<T>::kVec;
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t nvec = vec ? n / V : 0;
  for (int64_t i = tid; i < nvec; i += stride) {
    float vx[V], vr[V], o[V];
    Elem<T>::load_vec(x + i * V, vx);
    if (resid != nullptr) Elem<T>::load_vec(resid + i * V, vr);
    uint32_t keep = 0xffu;
    if (train && thr != 0u) {
      // V = 8: the vector is exactly one Philox call; V = 4: the even / odd vector takes the low / high four lanes
      keep = dropout_keep_bits8(seed, stream_id, static_cast<uint64_t>(i * V) >> 3, thr);
      if (V == 4) keep >>= (i & 1) * 4;
    }
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float d = train ? (((keep >> j) & 1u) ? vx[j] : 0.f) : vx[j] * eval_scale;
      o[j] = resid != nullptr ? vr[j] + d : d;
    }
    Elem<T>::store_vec(y + i * V, o);
  }
  for (int64_t i = nvec * V + tid; i < n; i += stride) {
    const float k = train ? (dropout_keep(seed, stream_id, static_cast<uint64_t>(i), thr) ? 1.f : 0.f) : eval_scale;
    const float d = Elem<T>::load(x + i) * k;
    Elem<T>::store(y + i, resid != nullptr ? Elem<T>::load(resid + i) + d : d);
  }
}

__global__ void __launch_bounds__(kEwThreads)
cast_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int64_t n, bool vec) {
  grid_dep_sync();
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t nvec = vec ? n / 8 : 0;
  for (int64_t i = tid; i < nvec; i += stride) {
    float v[8];
    const float4 a = *reinterpret_cast<const float4*>(src + i * 8);
    const float4 b = *reinterpret_cast<const float4*>(src + i * 8 + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    Elem<__nv_bfloat16>::store_vec(dst + i * 8, v);
  }
  for (int64_t i = nvec * 8 + tid; i < n; i += stride) dst[i] = __float2bfloat16_rn(src[i]);
}

template <typename T, int OP>
int launch_gelu(const void* a, const void* b, void* out, int64_t n, cudaStream_t st) {
  const bool vec = aligned16(a) && aligned16(out) && (OP == 0 || aligned16(b));
  launch_k(gelu_kernel<T, OP>, ew_grid(n / Elem<T>::kVec), kEwThreads, 0, st, 
      static_cast<const T*>(a), static_cast<const T*>(b), static_cast<T*>(out), n, vec);
  PTJ_CHECK_LAUNCH();
  return PTJ_OK;
}

}  // namespace
}  // namespace ptj

using namespace ptj;

extern "C" int ptj_gelu_fwd(const void* x, void* y, int64_t n, int dtype, void* stream) {
  if (n < 0) return PTJ_ERR_BAD_SHAPE;
  if (n == 0) return PTJ_OK;
  if (!x || !y) return PTJ_ERR_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == PTJ_F32) return launch_gelu<float, 0>(x, nullptr, y, n, st);
  if (dtype == PTJ_BF16) return launch_gelu<__nv_bfloat16, 0>(x, nullptr, y, n, st);
  return PTJ_ERR_DTYPE;
}

extern "C" int ptj_gelu_bwd(const void* dy, const void* x_preact, void* dx, int64_t n, int dtype, void* stream) {
  if (n < 0) return PTJ_ERR_BAD_SHAPE;
  if (n == 0) return PTJ_OK;
  if (!dy || !x_preact || !dx) return PTJ_ERR_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == PTJ_F32) return launch_gelu<float, 1>(dy, x_preact, dx, n, st);
  if (dtype == PTJ_BF16) return launch_gelu<__nv_bfloat16, 1>(dy, x_preact, dx, n, st);
  return PTJ_ERR_DTYPE;
}

extern "C" int ptj_dropout(const void* x, const void* residual, void* y, int64_t n, float p, int train,
                           uint64_t seed, uint32_t stream_id, int dtype, void* stream) {
  if (n < 0 || !(p >= 0.f && p <= 1.f)) return PTJ_ERR_BAD_SHAPE;
  if (n == 0) return PTJ_OK;
  if (!x || !y) return PTJ_ERR_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool vec = aligned16(x) && aligned16(y) && (residual == nullptr || aligned16(residual));
  const uint32_t thr = dropout_threshold16(p);
  if (dtype == PTJ_F32) {
    launch_k(dropout_kernel<float>, ew_grid(n / 4), kEwThreads, 0, st, 
        static_cast<const float*>(x), static_cast<const float*>(residual), static_cast<float*>(y), n, vec, thr,
        1.f - p, train, seed, stream_id);
  } else if (dtype == PTJ_BF16) {
    launch_k(dropout_kernel<__nv_bfloat16>, ew_grid(n / 8), kEwThreads, 0, st, 
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(residual),
        static_cast<__nv_bfloat16*>(y), n, vec, thr, 1.f - p, train, seed, stream_id);
  } else {
    return PTJ_ERR_DTYPE;
  }
  PTJ_CHECK_LAUNCH();
  return PTJ_OK;
}

extern "C" int ptj_cast_f32_to_bf16(const float* src, void* dst_bf16, int64_t n, void* stream) {
  if (n < 0) return PTJ_ERR_BAD_SHAPE;
  if (n == 0) return PTJ_OK;
  if (!src || !dst_bf16) return PTJ_ERR_BAD_SHAPE;
  const bool vec = aligned16(src) && aligned16(dst_bf16);
  launch_k(cast_kernel, ew_grid(n / 8), kEwThreads, 0, static_cast<cudaStream_t>(stream), 
      src, static_cast<__nv_bfloat16*>(dst_bf16), n, vec);
  PTJ_CHECK_LAUNCH();
  return PTJ_OK;
}
