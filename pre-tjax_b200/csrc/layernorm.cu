// LayerNorm forward / backward. Semantics of the reference: unbiased standard deviation (divide by n-1) and no
// epsilon (model_torch_func.py:104-108). Backward formula: model_triton.py:1773-1783 (dx) and :1652-1660 (dgamma,
// dbeta). HBM-bound: one warp owns one row, the row lives in registers between the statistics and the output pass,
// all global accesses are 16-byte vectors.
#include <mutex>
#include <type_traits>

#include "common.cuh"

namespace ptj {
namespace {

constexpr int kLnThreads = 256;

// V consecutive floats (V = 4 or 8, 16-byte aligned) with 16-byte loads. Scalar loads here would make every lane
// touch its own 32-byte sector per instruction and swamp L1 with 30x the traffic of the activations themselves.
template <int V>
__device__ __forceinline__ void load_params(const float* __restrict__ p, float (&out)[V]) {
#pragma unroll
  for (int q = 0; q < V / 4; ++q) {
    const float4 t = __ldg(reinterpret_cast<const float4*>(p) + q);
    out[4 * q] = t.x; out[4 * q + 1] = t.y; out[4 * q + 2] = t.z; out[4 * q + 3] = t.w;
  }
}
constexpr int kLnWarps = kLnThreads / 32;

inline int ln_grid(int64_t rows) {
  int64_t blocks = ceil_div(rows, kLnWarps);
  int64_t cap = static_cast<int64_t>(kNumSMs) * 8;  // 8 resident 256-thread blocks per SM
  return static_cast<int>(blocks < cap ? blocks : cap);
}
inline int ln_bwd_grid(int64_t rows) {
  int64_t blocks = ceil_div(rows, kLnWarps);
  int64_t cap = static_cast<int64_t>(kNumSMs) * 2;  // two resident blocks per SM; each block leaves one partial row
  return static_cast<int>(blocks < cap ? blocks : cap);
}

template <typename T, int NV>
__global__ void __launch_bounds__(kLnThreads, NV <= 4 ? 4 : 2)
ln_fwd_kernel(const T* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
              T* __restrict__ y, int64_t rows, int dim) {
  grid_dep_sync();
  constexpr int V = Elem<T>::kVec;
  const int lane = threadIdx.x & 31;
  const int nvec = dim / V;
  // gamma / beta are re-read from L1 for every row: keeping them in registers would halve the resident warps
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
        float o[V], gm[V], bt[V];
        load_params<V>(gamma + vi * V, gm);
        load_params<V>(beta + vi * V, bt);
#pragma unroll
        for (int j = 0; j < V; ++j) o[j] = gm[j] * ((v[i][j] - mean) * rstd) + bt[j];
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
  grid_dep_sync();
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

// Optional second output of the backward kernel: dropout (mask stream of site (seed, stream_id), element index =
// row * dim + column, i.e. the stream ptj_dropout uses on the contiguous [rows, dim] tensor) applied to dx, so that the
// consumer of "dropout backward of dx" needs no separate pass over dx.
struct LnMask {
  void* out;
  float* colsum;  // optional: column sums of `out` (the bias gradient of the linear layer that produced the branch)
  uint32_t thr;
  float eval_scale;
  int train;
  uint64_t seed;
  uint32_t stream_id;
};

// dx and the per-block partial sums of dgamma / dbeta in one pass over (dy, x). The running column sums live in
// shared memory (one private strip per warp, laid out [slot][lane] so accesses are conflict-free) rather than in
// registers: the kernel is latency-bound, and the lower register count doubles the number of resident warps.
template <typename T, int NV>
__global__ void __launch_bounds__(kLnThreads, (NV * Elem<T>::kVec <= 32) ? 2 : 1)
ln_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ gamma,
              const T* dx_add, T* dx, float* __restrict__ partial, int64_t rows, int dim, const LnMask mk) {
  grid_dep_sync();
  constexpr int V = Elem<T>::kVec;
  constexpr int kSlots = NV * V * 32;   // per-warp accumulator slots per quantity
  extern __shared__ float sm_acc[];     // [kLnWarps][nq][kSlots], nq = 2 (dgamma, dbeta) or 3 (+ column sums of mk.out)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nvec = dim / V;
  const bool want_cs = partial != nullptr && mk.colsum != nullptr;
  const uint64_t mask_seed = (mk.out != nullptr && mk.train && mk.thr != 0u) ? resolve_seed(mk.seed) : 0ull;
  const int nq = want_cs ? 3 : 2;
  float* acc_g = sm_acc + warp * nq * kSlots;
  float* acc_b = acc_g + kSlots;
  float* acc_d = acc_b + kSlots;
  if (partial != nullptr) {
#pragma unroll
    for (int s = 0; s < NV * V; ++s) {
      acc_g[s * 32 + lane] = 0.f;
      acc_b[s * 32 + lane] = 0.f;
      if (want_cs) acc_d[s * 32 + lane] = 0.f;
    }
  }
  const float inv_n = 1.f / static_cast<float>(dim), inv_nm1 = 1.f / static_cast<float>(dim - 1);
  const float n_adj = static_cast<float>(dim) * inv_nm1;
  // every lane always owns the same columns: its slice of gamma stays in registers for all rows
  float gmr[NV][V];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int vi = lane + 32 * i;
    if (vi < nvec) {
      load_params<V>(gamma + vi * V, gmr[i]);
    } else {
#pragma unroll
      for (int j = 0; j < V; ++j) gmr[i][j] = 0.f;
    }
  }
  const int64_t row_step = static_cast<int64_t>(gridDim.x) * kLnWarps;
  for (int64_t row = static_cast<int64_t>(blockIdx.x) * kLnWarps + warp; row < rows; row += row_step) {
    const T* xr = x + row * dim;
    const T* gr = dy + row * dim;
    float v[NV][V], u[NV][V], r[NV][V];
    float s = 0.f;
    // all of the row's loads go out together (the residual-path gradient included), and the next row of this warp is
    // pulled into L2 while this one is being processed
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int vi = lane + 32 * i;
      if (vi < nvec) {
        Elem<T>::load_vec(xr + vi * V, v[i]);
        Elem<T>::load_vec(gr + vi * V, u[i]);
        if (dx_add != nullptr) Elem<T>::load_vec(dx_add + row * dim + vi * V, r[i]);
        if (row + row_step < rows) {
          const int64_t nxt = (row + row_step) * dim + vi * V;
          asm volatile("prefetch.global.L2 [%0];" ::"l"(x + nxt));
          asm volatile("prefetch.global.L2 [%0];" ::"l"(dy + nxt));
          if (dx_add != nullptr) asm volatile("prefetch.global.L2 [%0];" ::"l"(dx_add + nxt));
        }
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
      const int vi = lane + 32 * i;
      if (vi < nvec) {
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float xh = (v[i][j] - mean) * rstd;
          v[i][j] = xh;
          if (partial != nullptr) {
            const int slot = (i * V + j) * 32 + lane;
            acc_g[slot] += u[i][j] * xh;
            acc_b[slot] += u[i][j];
          }
          const float gh = u[i][j] * gmr[i][j];
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
#pragma unroll
            for (int j = 0; j < V; ++j) o[j] += r[i][j];
          }
          Elem<T>::store_vec(dr + vi * V, o);
          if (mk.out != nullptr) {  // second output: dropout applied to dx as stored (rounded to T), see LnMask
            T* mr = static_cast<T*>(mk.out) + row * dim;
            const uint64_t idx = static_cast<uint64_t>(row) * dim + static_cast<uint64_t>(vi) * V;
            uint32_t keep = 0xffu;
            if (mk.train && mk.thr != 0u)
              keep = dropout_keep_bits8(mask_seed, mk.stream_id, idx >> 3, mk.thr) >> (idx & 7);
#pragma unroll
            for (int j = 0; j < V; ++j) {
              const float r = Elem<T>::round(o[j]);
              o[j] = mk.train ? (((keep >> j) & 1u) ? r : 0.f) : Elem<T>::round(r * mk.eval_scale);
              if (want_cs) acc_d[(i * V + j) * 32 + lane] += o[j];  // the value as stored
            }
            Elem<T>::store_vec(mr + vi * V, o);
          }
        }
      }
    }
  }
  if (partial == nullptr) return;
  __syncthreads();
  // fold the warps' strips in warp order (fixed order => reproducible) and scatter slots back to columns
  float* out = partial + static_cast<size_t>(blockIdx.x) * nq * dim;
  for (int t = threadIdx.x; t < nq * kSlots; t += blockDim.x) {
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < kLnWarps; ++w) sum += sm_acc[w * nq * kSlots + t];
    const int which = t / kSlots, rem = t - which * kSlots;
    const int ij = rem >> 5, ln = rem & 31;
    const int vi = ln + 32 * (ij / V);
    if (vi < nvec) out[which * dim + vi * V + (ij % V)] = sum;
  }
}

// ---- bf16 backward, rows of up to 2048 columns: several warps per row, rows staged through shared memory ---------
// The warp-per-row kernel above spends 1 600 instructions per row and keeps one row per warp in flight; it runs at a
// third of the memory roofline, issue- and latency-bound at once. Here a row is spread over W = ceil(dim / 256) warps
// (one 16-byte vector per lane), so a thread's running column sums are 24 registers instead of shared-memory strips,
// the arithmetic runs two floats wide (fma.rn.f32x2), and the loads are decoupled from the registers: every thread
// copies its own vectors of the next kRing - 1 rows into a private shared-memory ring with cp.async (each thread reads
// back only what it copied itself, so the ring needs no barrier), which keeps ~24 rows per SM in flight. Row sums
// cross the W warps of a row group through shared memory and a named barrier. RG row groups per block take
// alternate rows of the block's contiguous row range; their column sums are folded in group order at the end.
constexpr int kRing = 4;
__host__ __device__ constexpr int ln_rows_groups(int W) { return W >= 7 ? 1 : 12 / W; }

__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t bf2_to_f2(uint32_t w) {  // two packed bf16 -> two floats
  return f2_pack(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
__device__ __forceinline__ float f2_hsum(uint64_t v) {
  float a, b;
  f2_unpack(v, a, b);
  return a + b;
}
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))),
               "l"(gsrc)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Sum of one value per warp over the W warps of a row group (every thread gets the total; fixed order). `slot` is this
// exchange's own W floats; a slot is reused one row later, with two other exchanges' barriers in between.
template <int W>
__device__ __forceinline__ float group_sum(float v, float* slot, int wr, int lane, int bar_id) {
  v = warp_sum(v);
  if constexpr (W == 1) return v;
  if (lane == 0) slot[wr] = v;
  asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "n"(32 * W) : "memory");
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < W; ++w) t += slot[w];
  return t;
}

// two values at once, one barrier
template <int W>
__device__ __forceinline__ void group_sum2(float& a, float& b, float* slot, int wr, int lane, int bar_id) {
  a = warp_sum(a);
  b = warp_sum(b);
  if constexpr (W == 1) return;
  if (lane == 0) {
    slot[wr] = a;
    slot[W + wr] = b;
  }
  asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "n"(32 * W) : "memory");
  a = 0.f;
  b = 0.f;
#pragma unroll
  for (int w = 0; w < W; ++w) {
    a += slot[w];
    b += slot[W + w];
  }
}

template <int W>
__global__ void __launch_bounds__(32 * W * ln_rows_groups(W), 2)
ln_bwd_rows_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const float* __restrict__ gamma, const __nv_bfloat16* dx_add, __nv_bfloat16* dx,
                   float* __restrict__ partial, int64_t rows, int dim, const LnMask mk) {
  grid_dep_sync();
  constexpr int RG = ln_rows_groups(W);
  constexpr int kThreads = 32 * W * RG;
  extern __shared__ __align__(16) unsigned char sm_raw[];
  uint4* ring = reinterpret_cast<uint4*>(sm_raw);                                   // [kRing][3][kThreads]
  float* red = reinterpret_cast<float*>(sm_raw + sizeof(uint4) * kRing * 3 * kThreads);  // [RG][4][W]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int grp = warp / W, wr = warp - grp * W;
  const int nvec = dim >> 3;
  const int vi = wr * 32 + lane;
  const bool live = vi < nvec;
  const bool want_sums = partial != nullptr;
  const bool want_cs = want_sums && mk.colsum != nullptr;
  const bool masked = mk.out != nullptr;
  const bool draw = masked && mk.train && mk.thr != 0u;
  const uint64_t mask_seed = draw ? resolve_seed(mk.seed) : 0ull;
  float* my_red = red + grp * 4 * W;
  const int bar_id = 1 + grp;
  const float inv_n = 1.f / static_cast<float>(dim), inv_nm1 = 1.f / static_cast<float>(dim - 1);
  const float n_adj = static_cast<float>(dim) * inv_nm1;

  uint64_t gm[4];
  {
    float g8[8];
    if (live) {
      load_params<8>(gamma + vi * 8, g8);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) g8[j] = 0.f;
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) gm[q] = f2_pack(g8[2 * q], g8[2 * q + 1]);
  }
  uint64_t acc_g[4], acc_b[4], acc_d[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) acc_g[q] = acc_b[q] = acc_d[q] = 0ull;  // two packed +0.0f

  // this block's rows [r0, r1); group g takes r0 + g, r0 + g + RG, ...
  const int64_t r0 = rows * blockIdx.x / gridDim.x, r1 = rows * (blockIdx.x + 1) / gridDim.x;
  const int n_my = r0 + grp < r1 ? static_cast<int>((r1 - r0 - grp + RG - 1) / RG) : 0;
  auto row_of = [&](int it) { return r0 + grp + static_cast<int64_t>(it) * RG; };
  auto fetch = [&](int it) {
    if (it < n_my && live) {
      const int64_t off = row_of(it) * dim + vi * 8;
      uint4* dst = ring + (it % kRing) * 3 * kThreads + tid;
      cp_async16(dst, x + off);
      cp_async16(dst + kThreads, dy + off);
      if (dx_add != nullptr) cp_async16(dst + 2 * kThreads, dx_add + off);
    }
    cp_async_commit();  // (an empty group when there is nothing to fetch keeps the wait count uniform)
  };
#pragma unroll
  for (int it = 0; it < kRing - 1; ++it) fetch(it);

  for (int it = 0; it < n_my; ++it) {
    fetch(it + kRing - 1);
    cp_async_wait<kRing - 1>();
    const int64_t row = row_of(it);
    uint64_t xv[4], dv[4];
    uint4 rres = make_uint4(0u, 0u, 0u, 0u);
    {
      const uint4* src = ring + (it % kRing) * 3 * kThreads + tid;
      uint4 tx = make_uint4(0u, 0u, 0u, 0u), td = tx;
      if (live) {
        tx = src[0];
        td = src[kThreads];
        if (dx_add != nullptr) rres = src[2 * kThreads];
      }
      xv[0] = bf2_to_f2(tx.x); xv[1] = bf2_to_f2(tx.y); xv[2] = bf2_to_f2(tx.z); xv[3] = bf2_to_f2(tx.w);
      dv[0] = bf2_to_f2(td.x); dv[1] = bf2_to_f2(td.y); dv[2] = bf2_to_f2(td.z); dv[3] = bf2_to_f2(td.w);
    }
    // mean, then the centred sum of squares (two passes over registers, as in the forward kernel)
    const float mean = group_sum<W>(f2_hsum(f2_add(f2_add(xv[0], xv[1]), f2_add(xv[2], xv[3]))), my_red, wr, lane, bar_id) * inv_n;
    const uint64_t nmean = f2_pack(-mean, -mean);
    uint64_t ssq = 0ull;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      xv[q] = f2_add(xv[q], nmean);
      ssq = f2_fma(xv[q], xv[q], ssq);
    }
    // (lanes beyond the row hold x = 0 and would add mean^2: they contribute nothing instead)
    const float rstd = 1.f / sqrtf(group_sum<W>(live ? f2_hsum(ssq) : 0.f, my_red + W, wr, lane, bar_id) * inv_nm1);
    const uint64_t rstd2 = f2_pack(rstd, rstd);
    uint64_t s1 = 0ull, s2 = 0ull;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      xv[q] = f2_mul(xv[q], rstd2);                 // xhat
      acc_g[q] = f2_fma(dv[q], xv[q], acc_g[q]);    // dgamma += dy * xhat
      acc_b[q] = f2_add(acc_b[q], dv[q]);           // dbeta  += dy
      dv[q] = f2_mul(dv[q], gm[q]);                 // dy * gamma
      s1 = f2_add(s1, dv[q]);
      s2 = f2_fma(dv[q], xv[q], s2);
    }
    if (dx == nullptr) continue;  // parameter gradients only (uniform over the block)
    float m1 = f2_hsum(s1), m2 = f2_hsum(s2);
    group_sum2<W>(m1, m2, my_red + 2 * W, wr, lane, bar_id);
    m1 *= inv_n;
    m2 *= inv_n * n_adj;
    // dx = (dy*gamma - m1 - xhat * m2) * rstd (+ the gradient arriving over the residual connection)
    const uint64_t c1 = f2_pack(-m1 * rstd, -m1 * rstd), c2 = f2_pack(-m2 * rstd, -m2 * rstd);
    const uint32_t rw[4] = {rres.x, rres.y, rres.z, rres.w};
    uint32_t ow[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint64_t o = f2_fma(xv[q], c2, f2_fma(dv[q], rstd2, c1));
      if (dx_add != nullptr) o = f2_add(o, bf2_to_f2(rw[q]));
      float a, b;
      f2_unpack(o, a, b);
      __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
      ow[q] = *reinterpret_cast<uint32_t*>(&h);
    }
    if (live) *reinterpret_cast<uint4*>(dx + row * dim + vi * 8) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    if (masked) {  // second output: dropout applied to dx as stored (rounded to bf16), see LnMask
      if (mk.train) {
        if (draw) {
          const Philox4 r = philox4x32_10(mask_seed, static_cast<uint64_t>(row) * nvec + vi, mk.stream_id);
          const uint32_t rnd[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint32_t keep = ((rnd[q] & 0xffffu) >= mk.thr ? 0x0000ffffu : 0u) |
                                  ((rnd[q] >> 16) >= mk.thr ? 0xffff0000u : 0u);
            ow[q] &= keep;
          }
        }
      } else {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float a, b;
          f2_unpack(bf2_to_f2(ow[q]), a, b);
          __nv_bfloat162 h = __floats2bfloat162_rn(a * mk.eval_scale, b * mk.eval_scale);
          ow[q] = *reinterpret_cast<uint32_t*>(&h);
        }
      }
      if (live)
        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(mk.out) + row * dim + vi * 8) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
      if (want_cs) {
#pragma unroll
        for (int q = 0; q < 4; ++q) acc_d[q] = f2_add(acc_d[q], bf2_to_f2(ow[q]));  // the values as stored
      }
    }
  }
  if (!want_sums) return;
  // fold the row groups' column sums in group order (fixed order => reproducible); the ring is free by now
  cp_async_wait<0>();
  __syncthreads();
  const int nq = want_cs ? 3 : 2;
  float* fold = reinterpret_cast<float*>(sm_raw);  // [RG][nq][W * 256]
  constexpr int kCols = W * 256;
  {
    float* mine = fold + static_cast<size_t>(grp) * nq * kCols + vi * 8;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      f2_unpack(acc_g[q], mine[2 * q], mine[2 * q + 1]);
      f2_unpack(acc_b[q], mine[kCols + 2 * q], mine[kCols + 2 * q + 1]);
      if (want_cs) f2_unpack(acc_d[q], mine[2 * kCols + 2 * q], mine[2 * kCols + 2 * q + 1]);
    }
  }
  __syncthreads();
  float* out = partial + static_cast<size_t>(blockIdx.x) * nq * dim;
  for (int t = tid; t < nq * dim; t += kThreads) {
    const int which = t / dim, c = t - which * dim;
    float sum = 0.f;
#pragma unroll
    for (int g = 0; g < RG; ++g) sum += fold[(static_cast<size_t>(g) * nq + which) * kCols + c];
    out[t] = sum;
  }
}

template <typename T>
__global__ void __launch_bounds__(kLnThreads)
ln_bwd_generic_kernel(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ gamma,
                      const T* dx_add, T* dx, float* __restrict__ partial, int64_t rows, int dim) {
  grid_dep_sync();
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

// dgamma[c] = sum over blocks of partial[b][0][c], dbeta likewise. A block owns 32 columns; its 8 warps each sum a
// strided subset of the partial rows and the 8 results are added in warp order (fixed order => reproducible).
__global__ void __launch_bounds__(256)
ln_bwd_finalize_kernel(const float* __restrict__ partial, float* __restrict__ dgamma, float* __restrict__ dbeta,
                       float* __restrict__ dsum, int nq, int nblocks, int dim) {
  grid_dep_sync();
  // 8 columns x 32 row groups per block: many small blocks, each row group sums every 32nd partial row in order
  __shared__ float red[32][9];
  const int col = threadIdx.x & 7, grp = threadIdx.x >> 3;
  const int c = blockIdx.x * 8 + col;
  float s = 0.f;
  if (c < nq * dim)
    for (int b = grp; b < nblocks; b += 32) s += partial[static_cast<size_t>(b) * nq * dim + c];
  red[grp][col] = s;
  __syncthreads();
  if (grp == 0 && c < nq * dim) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 32; ++w) t += red[w][col];
    if (c < dim) dgamma[c] = t;
    else if (c < 2 * dim) dbeta[c - dim] = t;
    else dsum[c - 2 * dim] = t;
  }
}

template <typename T>
int launch_fwd(const T* x, const float* gamma, const float* beta, T* y, int64_t rows, int dim, cudaStream_t st) {
  constexpr int V = Elem<T>::kVec;
  const bool vec_ok = dim % V == 0 && aligned16(x) && aligned16(y) && aligned16(gamma) && aligned16(beta);
  const int nv = vec_ok ? static_cast<int>(ceil_div(dim / V, 32)) : 99;
  const int grid = ln_grid(rows);
#define PTJ_LN_FWD(NV) case NV: launch_k(ln_fwd_kernel<T, NV>, grid, kLnThreads, 0, st, x, gamma, beta, y, rows, dim); break;
  switch (nv) {
    PTJ_LN_FWD(1) PTJ_LN_FWD(2) PTJ_LN_FWD(3) PTJ_LN_FWD(4) PTJ_LN_FWD(5) PTJ_LN_FWD(6) PTJ_LN_FWD(7) PTJ_LN_FWD(8)
    default: {
      const int g = static_cast<int>(rows < kNumSMs * 8 ? rows : kNumSMs * 8);
      launch_k(ln_fwd_generic_kernel<T>, g, kLnThreads, 0, st, x, gamma, beta, y, rows, dim);
    }
  }
#undef PTJ_LN_FWD
  PTJ_CHECK_LAUNCH();
  return PTJ_OK;
}

template <typename T>
int launch_bwd(const T* dy, const T* x, const float* gamma, const T* dx_add, T* dx, float* dgamma, float* dbeta,
               float* scratch, int64_t rows, int dim, const LnMask& mk, cudaStream_t st) {
  constexpr int V = Elem<T>::kVec;
  const bool vec_ok = dim % V == 0 && aligned16(x) && aligned16(dy) && (dx == nullptr || aligned16(dx)) &&
                      (dx_add == nullptr || aligned16(dx_add)) && aligned16(gamma) && (mk.out == nullptr || aligned16(mk.out));
  const int nv = vec_ok ? static_cast<int>(ceil_div(dim / V, 32)) : 99;
  const int grid = ln_bwd_grid(rows);
  float* partial = dgamma != nullptr ? scratch : nullptr;
  const int nq = (partial != nullptr && mk.colsum != nullptr) ? 3 : 2;
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    if (vec_ok && dim >= 8 && dim <= 2048) {  // several warps per row, rows staged through shared memory
      const int w = static_cast<int>(ceil_div(dim, 256));
#define PTJ_LN_ROWS(W)                                                                                              \
  case W: {                                                                                                         \
    constexpr int kT = 32 * W * ln_rows_groups(W);                                                                  \
    constexpr size_t kRingBytes = sizeof(uint4) * kRing * 3 * kT;                                                   \
    constexpr size_t kFoldBytes = sizeof(float) * ln_rows_groups(W) * 3 * W * 256;                                  \
    constexpr size_t kSm = (kRingBytes > kFoldBytes ? kRingBytes : kFoldBytes) + sizeof(float) * ln_rows_groups(W) * 4 * W; \
    static_assert(kSm <= 227 * 1024, "shared memory of the LayerNorm backward");                                    \
    cudaFuncSetAttribute(ln_bwd_rows_kernel<W>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSm);             \
    launch_k(ln_bwd_rows_kernel<W>, grid, kT, kSm, st, dy, x, gamma, dx_add, dx, partial, rows, dim, mk);            \
  } break;
      switch (w) {
        PTJ_LN_ROWS(1) PTJ_LN_ROWS(2) PTJ_LN_ROWS(3) PTJ_LN_ROWS(4) PTJ_LN_ROWS(5) PTJ_LN_ROWS(6) PTJ_LN_ROWS(7) PTJ_LN_ROWS(8)
      }
#undef PTJ_LN_ROWS
      PTJ_CHECK_LAUNCH();
      if (partial != nullptr) {
        launch_k(ln_bwd_finalize_kernel, static_cast<int>(ceil_div(nq * dim, 8)), 256, 0, st, partial, dgamma, dbeta,
                 mk.colsum, nq, grid, dim);
        PTJ_CHECK_LAUNCH();
      }
      return PTJ_OK;
    }
  }
  const size_t smem = static_cast<size_t>(kLnWarps) * nq * (nv <= 8 ? nv : 0) * V * 32 * sizeof(float);
#define PTJ_LN_BWD(NV)                                                                                   \
  case NV:                                                                                               \
    if (smem > 48 * 1024)                                                                                \
      cudaFuncSetAttribute(ln_bwd_kernel<T, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    launch_k(ln_bwd_kernel<T, NV>, grid, kLnThreads, smem, st, dy, x, gamma, dx_add, dx, partial, rows, dim, mk);       \
    break;
  switch (nv) {
    PTJ_LN_BWD(1) PTJ_LN_BWD(2) PTJ_LN_BWD(3) PTJ_LN_BWD(4) PTJ_LN_BWD(5) PTJ_LN_BWD(6) PTJ_LN_BWD(7) PTJ_LN_BWD(8)
    default:
      if (mk.out != nullptr) return PTJ_ERR_UNSUPPORTED;  // the masked output needs vector-aligned rows of <= 8 x 32 vectors
      launch_k(ln_bwd_generic_kernel<T>, grid, kLnThreads, 0, st, dy, x, gamma, dx_add, dx, partial, rows, dim);
  }
#undef PTJ_LN_BWD
  PTJ_CHECK_LAUNCH();
  if (partial != nullptr) {
    launch_k(ln_bwd_finalize_kernel, static_cast<int>(ceil_div(nq * dim, 8)), 256, 0, st, partial, dgamma, dbeta,
             mk.colsum, nq, grid, dim);
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

// floats of partial sums the backward kernel writes: one row of nq * dim per thread block
static size_t ln_bwd_partial_floats(int64_t rows, int64_t dim, int nq) {
  if (rows <= 0 || dim <= 0) return 0;
  return static_cast<size_t>(ln_bwd_grid(rows)) * nq * static_cast<size_t>(dim);
}

extern "C" size_t ptj_layernorm_bwd_scratch_floats(int64_t rows, int64_t dim) {
  return ln_bwd_partial_floats(rows, dim, 3);  // dgamma, dbeta and the optional column sums of the dropped output
}

static int layernorm_bwd_impl(const void* dy, const void* x, const float* gamma, const void* dx_add, void* dx,
                              float* dgamma, float* dbeta, float* scratch, size_t scratch_floats, int64_t rows,
                              int64_t dim, const LnMask& mk, int dtype, void* stream) {
  if (rows < 0 || dim < 1 || dim > (1 << 20)) return PTJ_ERR_BAD_SHAPE;
  if ((dgamma == nullptr) != (dbeta == nullptr)) return PTJ_ERR_BAD_SHAPE;
  if (!dy || !x || !gamma) return PTJ_ERR_BAD_SHAPE;
  if (mk.out != nullptr && dx == nullptr) return PTJ_ERR_BAD_SHAPE;
  if (mk.colsum != nullptr && (mk.out == nullptr || dgamma == nullptr)) return PTJ_ERR_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (rows == 0) {
    if (dgamma) {
      cudaMemsetAsync(dgamma, 0, sizeof(float) * dim, st);
      cudaMemsetAsync(dbeta, 0, sizeof(float) * dim, st);
    }
    return PTJ_OK;
  }
  if (dgamma && (scratch == nullptr || scratch_floats < ln_bwd_partial_floats(rows, dim, mk.colsum != nullptr ? 3 : 2)))
    return PTJ_ERR_WORKSPACE;
  if (dtype == PTJ_F32)
    return launch_bwd(static_cast<const float*>(dy), static_cast<const float*>(x), gamma,
                      static_cast<const float*>(dx_add), static_cast<float*>(dx), dgamma, dbeta, scratch, rows, (int)dim,
                      mk, st);
  if (dtype == PTJ_BF16)
    return launch_bwd(static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x), gamma,
                      static_cast<const __nv_bfloat16*>(dx_add), static_cast<__nv_bfloat16*>(dx), dgamma, dbeta, scratch,
                      rows, (int)dim, mk, st);
  return PTJ_ERR_DTYPE;
}

extern "C" int ptj_layernorm_bwd(const void* dy, const void* x, const float* gamma, const void* dx_add, void* dx,
                                 float* dgamma, float* dbeta, float* scratch, size_t scratch_floats, int64_t rows,
                                 int64_t dim, int dtype, void* stream) {
  const LnMask none{nullptr, nullptr, 0u, 1.f, 0, 0ull, 0u};
  return layernorm_bwd_impl(dy, x, gamma, dx_add, dx, dgamma, dbeta, scratch, scratch_floats, rows, dim, none, dtype,
                            stream);
}

extern "C" int ptj_layernorm_bwd_dropout(const void* dy, const void* x, const float* gamma, const void* dx_add, void* dx,
                                         void* dx_dropped, float* dropped_colsum, float* dgamma, float* dbeta, float* scratch,
                                         size_t scratch_floats, int64_t rows, int64_t dim, float p, int train,
                                         uint64_t seed, uint32_t stream_id, int dtype, void* stream) {
  if (!dx_dropped || !(p >= 0.f && p <= 1.f)) return PTJ_ERR_BAD_SHAPE;
  const LnMask mk{dx_dropped, dropped_colsum, dropout_threshold16(p), 1.f - p, train, seed, stream_id};
  return layernorm_bwd_impl(dy, x, gamma, dx_add, dx, dgamma, dbeta, scratch, scratch_floats, rows, dim, mk, dtype,
                            stream);
}
// ---- LayerNorm backward for callers that must not allocate ------------------------------------------------------
// The partial column sums of ptj_layernorm_bwd normally live in a scratch buffer the caller allocates. Some callers
// cannot do that: code that runs inside a process whose device memory was handed out up front to another allocator
// (a framework-owned pool sized to the whole GPU, where cudaMalloc would fail, fragment the pool or stall the device),
// or a step that must stay off the driver's allocation path for latency reasons. For them the scratch is this
// fixed array in the library's own image: 148 * 2 thread blocks x (dgamma, dbeta) x kStaticMaxDim floats = 4.6 MiB,
// held by every GPU that loads the library until the process exits.
constexpr int kStaticMaxDim = 2048;
constexpr size_t kStaticScratchFloats = static_cast<size_t>(kNumSMs) * 2 * 2 * kStaticMaxDim;
static __device__ __align__(256) float g_ln_bwd_static_scratch[kStaticScratchFloats];

namespace ptj {
namespace {
// The array's name is only a host-side handle; kernels need its DEVICE address, which differs per GPU. It is looked
// up once per device, with that device current, and cached.
float* static_scratch_for_current_device() {
  constexpr int kMaxDev = 64;
  static float* cache[kMaxDev] = {};
  static std::mutex mu;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) {
    (void)cudaGetLastError();
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (cache[dev] == nullptr) {
    float* ptr = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_ln_bwd_static_scratch) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    cache[dev] = ptr;
  }
  return cache[dev];
}
}  // namespace
}  // namespace ptj

extern "C" size_t ptj_layernorm_bwd_noalloc_max_dim(void) { return kStaticMaxDim; }

extern "C" int ptj_layernorm_bwd_noalloc(const void* dy, const void* x, const float* gamma, const void* dx_add, void* dx,
                                         float* dgamma, float* dbeta, int64_t rows, int64_t dim, int dtype,
                                         void* stream) {
  if (rows < 0 || dim < 1) return PTJ_ERR_BAD_SHAPE;
  if (dim > kStaticMaxDim || ln_bwd_partial_floats(rows, dim, 2) > kStaticScratchFloats) return PTJ_ERR_TOO_LARGE;
  float* scratch = static_scratch_for_current_device();  // first call on a device resolves the address
  if (scratch == nullptr) return PTJ_ERR_DEVICE;
  return ptj_layernorm_bwd(dy, x, gamma, dx_add, dx, dgamma, dbeta, scratch, kStaticScratchFloats, rows, dim, dtype,
                           stream);
}
