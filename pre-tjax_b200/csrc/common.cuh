// Shared device/host helpers for the sm_100a kernels: vector loads, reductions, Philox, launch bookkeeping.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include "../../include/ptj_b200.h"

namespace ptj {

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs; grids are sized in multiples of this

extern void count_launch(int n);

#define PTJ_CHECK_LAUNCH()                                   \
  do {                                                       \
    ::ptj::count_launch(1);                                  \
    if (cudaPeekAtLastError() != cudaSuccess) {              \
      (void)cudaGetLastError();                              \
      return PTJ_ERR_LAUNCH;                                 \
    }                                                        \
  } while (0)

// Programmatic dependent launch: every kernel of this library is launched so that its blocks may become resident while
// the previous kernel of the stream is still draining, and calls grid_dep_sync() before its first access to global
// memory. The call (1) lets the NEXT kernel's blocks start their own set-up once all blocks of this one have reached
// this point, and (2) waits until every earlier kernel of the stream has completed and its writes are visible.
// Kernels that allocate tensor memory call it only after their allocation, so a dependent block can never hold
// tensor memory that a block of an earlier, still running kernel is waiting for.
constexpr bool pdl_enabled() { return true; }

__device__ __forceinline__ void grid_dep_sync() {
  asm volatile("griddepcontrol.launch_dependents;\n\tgriddepcontrol.wait;" ::: "memory");
}

template <typename... KArgs, typename... Args>
inline void launch_k(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  (void)cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);  // errors surface through cudaPeekAtLastError
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline size_t dtype_size(int dtype) { return dtype == PTJ_BF16 ? 2 : 4; }
inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---- element access, fp32 math on either storage type ------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<float> {
  static constexpr int kVec = 4;  // elements per 16-byte vector
  static __device__ __forceinline__ float load(const float* p) { return *p; }
  static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
  static __device__ __forceinline__ float round(float v) { return v; }  // value as it will be stored
  static __device__ __forceinline__ void load_vec(const float* p, float (&v)[4]) {
    float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
  static __device__ __forceinline__ void store_vec(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <> struct Elem<__nv_bfloat16> {
  static constexpr int kVec = 8;
  static __device__ __forceinline__ float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
  static __device__ __forceinline__ float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
  static __device__ __forceinline__ void load_vec(const __nv_bfloat16* p, float (&v)[8]) {
    uint4 t = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ void store_vec(__nv_bfloat16* p, const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};

// ---- reductions ------------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide sum; every thread gets the result. `smem` needs 33 floats. Result is order-deterministic.
__device__ __forceinline__ float block_sum(float v, float* smem) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? smem[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) smem[32] = t;
  }
  __syncthreads();
  return smem[32];
}
__device__ __forceinline__ float block_max(float v, float* smem) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? smem[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) smem[32] = t;
  }
  __syncthreads();
  return smem[32];
}

// ---- Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11) -----------------
struct Philox4 { uint32_t x, y, z, w; };
__host__ __device__ __forceinline__ Philox4 philox4x32_10(uint64_t seed, uint64_t ctr, uint32_t stream_id) {
  uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
  uint32_t c0 = static_cast<uint32_t>(ctr), c1 = static_cast<uint32_t>(ctr >> 32), c2 = stream_id, c3 = 0x5054'4a31u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = static_cast<uint64_t>(0xD2511F53u) * c0;
    const uint64_t p1 = static_cast<uint64_t>(0xCD9E8D57u) * c2;
    const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c1 ^ k0;
    const uint32_t n1 = static_cast<uint32_t>(p1);
    const uint32_t n2 = static_cast<uint32_t>(p0 >> 32) ^ c3 ^ k1;
    const uint32_t n3 = static_cast<uint32_t>(p0);
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  return Philox4{c0, c1, c2, c3};
}
// ---- the dropout mask stream (one definition for every site) ---------------------------------------------------
// Element idx of a site's index space takes 16 random bits: Philox call number idx / 8 (counter low/high words),
// keyed by the site's seed and stream id, yields four 32-bit words = eight 16-bit lanes; element e = idx % 8 uses the
// low half of word e / 2 when e is even and the high half when odd. The element is DROPPED when its lane is below
// floor(p * 65536). Forward and backward regenerate the same bits; nothing is stored.
// A `seed` argument of any entry point is either the 63-bit seed itself or, with bit 63 set, the DEVICE ADDRESS (low 63
// bits) of a uint64 that holds it. The second form lets a caller replay the same recorded launches (a CUDA graph of a
// whole training step) with fresh masks: it rewrites the words in device memory between replays. Kernels resolve the
// argument once, before their first use of it.
constexpr uint64_t kSeedIsPointer = 1ull << 63;
__device__ __forceinline__ uint64_t resolve_seed(uint64_t s) {
  return (s & kSeedIsPointer) ? __ldg(reinterpret_cast<const uint64_t*>(s & ~kSeedIsPointer)) : s;
}
__host__ __device__ __forceinline__ uint32_t dropout_threshold16(float p) {
  double t = static_cast<double>(p) * 65536.0;
  if (t <= 0.0) return 0u;
  if (t >= 65535.0) return 65535u;
  return static_cast<uint32_t>(t);
}
// keep flags (bit e = element 8*call + e) of one Philox call
__host__ __device__ __forceinline__ uint32_t dropout_keep_bits8(uint64_t seed, uint32_t stream_id, uint64_t call,
                                                                uint32_t thr16) {
  const Philox4 r = philox4x32_10(seed, call, stream_id);
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
  uint32_t bits = 0;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    bits |= ((w[e] & 0xffffu) >= thr16 ? 1u : 0u) << (2 * e);
    bits |= ((w[e] >> 16) >= thr16 ? 1u : 0u) << (2 * e + 1);
  }
  return bits;
}
// keep flag of a single element (any idx)
__host__ __device__ __forceinline__ bool dropout_keep(uint64_t seed, uint32_t stream_id, uint64_t idx, uint32_t thr16) {
  return (dropout_keep_bits8(seed, stream_id, idx >> 3, thr16) >> (idx & 7)) & 1u;
}

// ---- tanh-GELU (model_torch_func.py:60-62) -------------------------------------------------------------------
// FAST = true uses the hardware tanh approximation (relative error about 2^-11): invisible once the result is rounded
// to bf16 (2^-8), and it keeps GEMM epilogues off the critical path. The float32 path always uses tanhf.
template <bool FAST>
__device__ __forceinline__ float tanh_sel(float x) {
  if (FAST) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
  }
  return tanhf(x);
}
// gelu(x) = 0.5 x (1 + tanh(u)), u = sqrt(2/pi) (x + 0.044715 x^3) = x (k + k c x^2)
template <bool FAST = false>
__device__ __forceinline__ float gelu_tanh(float x) {
  const float k = 0.7978845608028654f, kc = 0.7978845608028654f * 0.044715f;
  const float t = tanh_sel<FAST>(x * fmaf(x * x, kc, k));
  const float hx = 0.5f * x;
  return fmaf(hx, t, hx);
}
// d gelu / dx = 0.5 (1 + t) + 0.5 x (1 - t^2) (k + 3 k c x^2)   (model_triton.py:262-267)
template <bool FAST = false>
__device__ __forceinline__ float gelu_tanh_grad(float x) {
  const float k = 0.7978845608028654f, kc = 0.7978845608028654f * 0.044715f;
  const float x2 = x * x;
  const float t = tanh_sel<FAST>(x * fmaf(x2, kc, k));
  const float dt = fmaf(-t, t, 1.f) * fmaf(x2, 3.f * kc, k);
  return fmaf(0.5f * x, dt, fmaf(0.5f, t, 0.5f));
}

// Two-wide forms for the bf16 GEMM epilogues (hardware tanh, packed fp32 arithmetic: half the issue slots).
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ void gelu_tanh_x2(float& x0, float& x1) {
  const float k = 0.7978845608028654f, kc = 0.7978845608028654f * 0.044715f;
  const uint64_t x = f2_pack(x0, x1);
  const uint64_t u = f2_mul(x, f2_fma(f2_mul(x, x), f2_pack(kc, kc), f2_pack(k, k)));
  float u0, u1;
  f2_unpack(u, u0, u1);
  const uint64_t t = f2_pack(tanh_sel<true>(u0), tanh_sel<true>(u1));
  const uint64_t hx = f2_mul(x, f2_pack(0.5f, 0.5f));
  f2_unpack(f2_fma(hx, t, hx), x0, x1);
}
// g *= gelu'(x) for two elements
__device__ __forceinline__ void gelu_tanh_grad_mul_x2(float& g0, float& g1, float xa, float xb) {
  const float k = 0.7978845608028654f, kc = 0.7978845608028654f * 0.044715f;
  const uint64_t x = f2_pack(xa, xb);
  const uint64_t x2 = f2_mul(x, x);
  const uint64_t u = f2_mul(x, f2_fma(x2, f2_pack(kc, kc), f2_pack(k, k)));
  float u0, u1;
  f2_unpack(u, u0, u1);
  const uint64_t t = f2_pack(tanh_sel<true>(u0), tanh_sel<true>(u1));
  const uint64_t one = f2_pack(1.f, 1.f), half = f2_pack(0.5f, 0.5f);
  const uint64_t nt = f2_mul(t, f2_pack(-1.f, -1.f));
  const uint64_t dt = f2_mul(f2_fma(nt, t, one), f2_fma(x2, f2_pack(3.f * kc, 3.f * kc), f2_pack(k, k)));
  const uint64_t d = f2_fma(f2_mul(x, half), dt, f2_fma(half, t, half));
  f2_unpack(f2_mul(f2_pack(g0, g1), d), g0, g1);
}

}  // namespace ptj
