// Fused AdamW over flat parameter / gradient / moment buffers, global gradient norm, gradient clipping.
// Formula of the reference optimizer (loss_and_optimizer_triton.py:376-401):
//   m <- b1 m + (1-b1) g ; v <- b2 v + (1-b2) g^2 ; p <- p - lr * ( m/(1-b1^t) / (sqrt(v/(1-b2^t)) + eps) + wd p )
// HBM-bound: 16 B read (p, g, m, v) and 12 B written per parameter, plus 2 B for the optional bf16 shadow.
#include "common.cuh"

namespace ptj {
namespace {

constexpr int kOptThreads = 256;
constexpr int kMaxSegments = 1024;

inline int opt_grid(int64_t nvec) {
  int64_t blocks = ceil_div(nvec, kOptThreads);
  const int64_t cap = static_cast<int64_t>(kNumSMs) * 8;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks < cap ? blocks : cap);
}

__global__ void __launch_bounds__(kOptThreads)
sumsq_stage1_kernel(const float* __restrict__ x, float* __restrict__ partial, int64_t n) {
  grid_dep_sync();
  __shared__ float red[33];
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const bool vec = (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
  const int64_t nvec = vec ? n / 4 : 0;
  float s = 0.f;
  for (int64_t i = tid; i < nvec; i += stride) {
    const float4 v = reinterpret_cast<const float4*>(x)[i];
    s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  for (int64_t i = nvec * 4 + tid; i < n; i += stride) s += x[i] * x[i];
  const float t = block_sum(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = t;
}
__global__ void __launch_bounds__(1024)
sumsq_stage2_kernel(const float* __restrict__ partial, float* __restrict__ out, int nblocks) {
  grid_dep_sync();
  __shared__ float red[33];
  float s = 0.f;
  for (int i = threadIdx.x; i < nblocks; i += blockDim.x) s += partial[i];
  const float t = block_sum(s, red);
  if (threadIdx.x == 0) *out = t;
}

__global__ void __launch_bounds__(kOptThreads)
adamw_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
             __nv_bfloat16* __restrict__ shadow, int64_t n, const int64_t* __restrict__ seg_start,
             const uint8_t* __restrict__ seg_decay, int nseg, float lr, float beta1, float beta2, float eps, float wd,
             float inv_bc1, float inv_bc2, float grad_scale, const float* __restrict__ sumsq, float max_norm) {
  grid_dep_sync();
  __shared__ int64_t s_start[kMaxSegments + 1];
  __shared__ uint8_t s_decay[kMaxSegments];
  if (nseg > 0) {  // the segment tables may be null when there are no segments
    for (int i = threadIdx.x; i <= nseg; i += blockDim.x) s_start[i] = seg_start[i];
    for (int i = threadIdx.x; i < nseg; i += blockDim.x) s_decay[i] = seg_decay[i];
  }
  __syncthreads();
  float gs = grad_scale;
  if (sumsq != nullptr) {
    const float norm = sqrtf(*sumsq) * grad_scale;
    gs *= fminf(1.f, max_norm / (norm + 1e-6f));
  }
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t nvec = n / 4;  // n % 4 == 0 and 16-byte alignment are checked on the host
  for (int64_t i = tid; i < nvec; i += stride) {
    const int64_t e = i * 4;
    float w = wd;
    if (nseg > 0) {  // last segment whose start is <= e
      int lo = 0, hi = nseg - 1;
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (s_start[mid] <= e) lo = mid; else hi = mid - 1;
      }
      w = s_decay[lo] ? wd : 0.f;
    }
    float4 pp = reinterpret_cast<float4*>(p)[i];
    const float4 gg = reinterpret_cast<const float4*>(g)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float* pa = &pp.x; const float* ga = &gg.x; float* ma = &mm.x; float* va = &vv.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gj = ga[j] * gs;
      ma[j] = ma[j] * beta1 + (1.f - beta1) * gj;
      va[j] = va[j] * beta2 + (1.f - beta2) * gj * gj;
      const float mh = ma[j] * inv_bc1, vh = va[j] * inv_bc2;
      pa[j] = pa[j] + (-lr * (mh / (sqrtf(vh) + eps) + w * pa[j]));
    }
    reinterpret_cast<float4*>(p)[i] = pp;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    if (shadow != nullptr) {
      const __nv_bfloat162 lo2 = __floats2bfloat162_rn(pp.x, pp.y), hi2 = __floats2bfloat162_rn(pp.z, pp.w);
      uint2 o;
      o.x = *reinterpret_cast<const uint32_t*>(&lo2);
      o.y = *reinterpret_cast<const uint32_t*>(&hi2);
      reinterpret_cast<uint2*>(shadow)[i] = o;
    }
  }
}

}  // namespace
}  // namespace ptj

using namespace ptj;

extern "C" size_t ptj_sumsq_scratch_floats(int64_t n) {
  if (n <= 0) return 1;
  return static_cast<size_t>(opt_grid(n / 4));
}

extern "C" int ptj_sumsq(const float* x, float* out, float* scratch, size_t scratch_floats, int64_t n, void* stream) {
  if (n < 0) return PTJ_ERR_BAD_SHAPE;
  if (!out || (n > 0 && !x)) return PTJ_ERR_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (n == 0) {
    cudaMemsetAsync(out, 0, sizeof(float), st);
    return PTJ_OK;
  }
  if (!scratch || scratch_floats < ptj_sumsq_scratch_floats(n)) return PTJ_ERR_WORKSPACE;
  const int grid = opt_grid(n / 4);
  launch_k(sumsq_stage1_kernel, grid, kOptThreads, 0, st, x, scratch, n);
  PTJ_CHECK_LAUNCH();
  launch_k(sumsq_stage2_kernel, 1, 1024, 0, st, scratch, out, grid);
  PTJ_CHECK_LAUNCH();
  return PTJ_OK;
}

extern "C" int ptj_adamw(float* p, const float* g, float* m, float* v, void* shadow_bf16, int64_t n,
                         const int64_t* seg_start, const uint8_t* seg_decay, int nseg, float lr, float beta1,
                         float beta2, float eps, float weight_decay, int64_t t, float grad_scale, const float* sumsq,
                         float max_norm, void* stream) {
  if (n < 0 || n % 4 != 0 || t < 1 || nseg < 0 || nseg > kMaxSegments) return PTJ_ERR_BAD_SHAPE;
  if (n == 0) return PTJ_OK;
  if (!p || !g || !m || !v) return PTJ_ERR_BAD_SHAPE;
  if (nseg > 0 && (!seg_start || !seg_decay)) return PTJ_ERR_BAD_SHAPE;
  if (!aligned16(p) || !aligned16(g) || !aligned16(m) || !aligned16(v) ||
      (shadow_bf16 && (reinterpret_cast<uintptr_t>(shadow_bf16) & 7u)))
    return PTJ_ERR_MISALIGNED;
  // bias corrections in double on the host: 1 - b^t loses all precision in float for t beyond a few thousand
  const float inv_bc1 = static_cast<float>(1.0 / (1.0 - pow(static_cast<double>(beta1), static_cast<double>(t))));
  const float inv_bc2 = static_cast<float>(1.0 / (1.0 - pow(static_cast<double>(beta2), static_cast<double>(t))));
  launch_k(adamw_kernel, opt_grid(n / 4), kOptThreads, 0, static_cast<cudaStream_t>(stream), 
      p, g, m, v, static_cast<__nv_bfloat16*>(shadow_bf16), n, seg_start, seg_decay, nseg, lr, beta1, beta2, eps,
      weight_decay, inv_bc1, inv_bc2, grad_scale, sumsq, max_norm);
  PTJ_CHECK_LAUNCH();
  return PTJ_OK;
}
