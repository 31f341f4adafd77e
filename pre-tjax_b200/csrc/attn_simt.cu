// Causal attention forward / backward in exact fp32 arithmetic on CUDA cores, for any head size up to 128 and any
// sequence length. One warp owns one query row (forward, dQ) or one key row (dK, dV); lanes sweep 32 keys (queries) at
// a time. Semantics: model_triton.py:510-517, 608-611 (forward), :550-577, 801-811 (backward); dropout acts on the
// probabilities and is not rescaled. No atomics: the backward is split into a dQ pass and a dK/dV pass that both
// recompute the probabilities from the saved row maximum and row sum.
#include "attn_common.cuh"

namespace ptj {
namespace {

constexpr int kWarpsPerBlock = 4;
constexpr int kMaxD = 128;

template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
attn_fwd_simt_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, T* __restrict__ o,
                     float* __restrict__ row_max, float* __restrict__ row_sum, const int32_t* __restrict__ kstart,
                     const ptj_attn_shape sh, float scale, AttnDropout dr) {
  grid_dep_sync();
  dr.seed = resolve_seed(dr.seed);
  __shared__ float qs[kWarpsPerBlock][kMaxD];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int64_t S = sh.seq, D = sh.d_head;
  const int64_t total = sh.batch * sh.heads * S;
  for (int64_t rid = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + w; rid < total;
       rid += static_cast<int64_t>(gridDim.x) * kWarpsPerBlock) {
    const int64_t i = rid % S, bh = rid / S, h = bh % sh.heads, b = bh / sh.heads;
    const T* qr = q + b * sh.q_strides[0] + h * sh.q_strides[1] + i * sh.q_strides[2];
    const T* kb = k + b * sh.k_strides[0] + h * sh.k_strides[1];
    const T* vb = v + b * sh.v_strides[0] + h * sh.v_strides[1];
    __syncwarp();
    for (int d = lane; d < D; d += 32) qs[w][d] = Elem<T>::load(qr + d);
    __syncwarp();
    float m = -INFINITY, l = 0.f, acc[kMaxD / 32] = {0.f, 0.f, 0.f, 0.f};
    // the row attends keys [ks, i]: the whole causal prefix, or from its document's first token when kstart is given
    const int64_t ks = kstart != nullptr ? kstart[b * S + i] : 0;
    const bool empty = ks > i;  // the row attends nothing: zero output, neutral statistics
    for (int64_t j0 = (ks > 0 ? ks : 0) / 32 * 32; j0 <= i && !empty; j0 += 32) {
      const int64_t j = j0 + lane;
      float s = -INFINITY;
      if (j <= i && j >= ks) {
        const T* kr = kb + j * sh.k_strides[2];
        float t = 0.f;
        for (int d = 0; d < D; ++d) t = fmaf(qs[w][d], Elem<T>::load(kr + d), t);
        s = t * scale;
      }
      const float mnew = fmaxf(m, warp_max(s));  // finite: the first 32 keys visited include key ks <= i
      const float p = (j <= i && j >= ks) ? expf(s - mnew) : 0.f;
      const float corr = expf(m - mnew);
      l = l * corr + warp_sum(p);
      const float pd = p * dr.factor(bh, S, i, j);
#pragma unroll
      for (int t = 0; t < kMaxD / 32; ++t) acc[t] *= corr;
      const int cnt = static_cast<int>(i - j0 + 1 < 32 ? i - j0 + 1 : 32);
      for (int jj = 0; jj < cnt; ++jj) {
        const float pj = __shfl_sync(0xffffffffu, pd, jj);
        const T* vr = vb + (j0 + jj) * sh.v_strides[2];
#pragma unroll
        for (int t = 0; t < kMaxD / 32; ++t) {
          const int d = lane + 32 * t;
          if (d < D) acc[t] = fmaf(pj, Elem<T>::load(vr + d), acc[t]);
        }
      }
      m = mnew;
    }
    T* orow = o + b * sh.o_strides[0] + h * sh.o_strides[1] + i * sh.o_strides[2];
    if (empty) { m = 0.f; l = 1.f; }
    const float inv = empty ? 0.f : 1.f / l;
#pragma unroll
    for (int t = 0; t < kMaxD / 32; ++t) {
      const int d = lane + 32 * t;
      if (d < D) Elem<T>::store(orow + d, acc[t] * inv);
    }
    if (lane == 0) {
      row_max[rid] = m;
      row_sum[rid] = l;
    }
  }
}

// MODE 0: dQ (warp per query row, lanes over keys). MODE 1: dK and dV (warp per key row, lanes over queries).
template <typename T, int MODE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
attn_bwd_simt_kernel(const T* __restrict__ d_o, const T* __restrict__ q, const T* __restrict__ k,
                     const T* __restrict__ v, const T* __restrict__ o, const float* __restrict__ row_max,
                     const float* __restrict__ row_sum, T* __restrict__ dq, T* __restrict__ dk, T* __restrict__ dv,
                     const int32_t* __restrict__ kstart, const ptj_attn_shape sh, const ptj_attn_shape dsh, float scale,
                     AttnDropout dr) {
  grid_dep_sync();
  dr.seed = resolve_seed(dr.seed);
  __shared__ float xs[kWarpsPerBlock][kMaxD];  // MODE 0: q row;  MODE 1: k row
  __shared__ float ys[kWarpsPerBlock][kMaxD];  // MODE 0: dO row; MODE 1: v row
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int64_t S = sh.seq, D = sh.d_head;
  const int64_t total = sh.batch * sh.heads * S;
  for (int64_t rid = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + w; rid < total;
       rid += static_cast<int64_t>(gridDim.x) * kWarpsPerBlock) {
    const int64_t r = rid % S, bh = rid / S, h = bh % sh.heads, b = bh / sh.heads;
    const T* qb = q + b * sh.q_strides[0] + h * sh.q_strides[1];
    const T* kb = k + b * sh.k_strides[0] + h * sh.k_strides[1];
    const T* vb = v + b * sh.v_strides[0] + h * sh.v_strides[1];
    const T* ob = o + b * sh.o_strides[0] + h * sh.o_strides[1];
    const T* gb = d_o + b * sh.o_strides[0] + h * sh.o_strides[1];
    __syncwarp();
    for (int d = lane; d < D; d += 32) {
      xs[w][d] = Elem<T>::load((MODE == 0 ? qb + r * sh.q_strides[2] : kb + r * sh.k_strides[2]) + d);
      ys[w][d] = Elem<T>::load((MODE == 0 ? gb + r * sh.o_strides[2] : vb + r * sh.v_strides[2]) + d);
    }
    __syncwarp();
    float acc0[kMaxD / 32] = {0.f, 0.f, 0.f, 0.f}, acc1[kMaxD / 32] = {0.f, 0.f, 0.f, 0.f};
    if (MODE == 0) {
      const int64_t i = r;
      float dl = 0.f;  // delta_i = sum_d dO[i,d] * O[i,d]
      for (int d = lane; d < D; d += 32) dl += ys[w][d] * Elem<T>::load(ob + i * sh.o_strides[2] + d);
      const float delta = warp_sum(dl);
      const float m = row_max[rid], inv_l = 1.f / row_sum[rid];
      const int64_t ks = kstart != nullptr ? kstart[b * S + i] : 0;
      for (int64_t j0 = (ks > 0 ? ks : 0) / 32 * 32; j0 <= i; j0 += 32) {
        const int64_t j = j0 + lane;
        float ds = 0.f;
        if (j <= i && j >= ks) {
          const T* kr = kb + j * sh.k_strides[2];
          const T* vr = vb + j * sh.v_strides[2];
          float s = 0.f, dpd = 0.f;
          for (int d = 0; d < D; ++d) {
            s = fmaf(xs[w][d], Elem<T>::load(kr + d), s);
            dpd = fmaf(ys[w][d], Elem<T>::load(vr + d), dpd);
          }
          const float p = expf(s * scale - m) * inv_l;
          ds = p * (dpd * dr.factor(bh, S, i, j) - delta) * scale;
        }
        const int cnt = static_cast<int>(i - j0 + 1 < 32 ? i - j0 + 1 : 32);
        for (int jj = 0; jj < cnt; ++jj) {
          const float dsj = __shfl_sync(0xffffffffu, ds, jj);
          const T* kr = kb + (j0 + jj) * sh.k_strides[2];
#pragma unroll
          for (int t = 0; t < kMaxD / 32; ++t) {
            const int d = lane + 32 * t;
            if (d < D) acc0[t] = fmaf(dsj, Elem<T>::load(kr + d), acc0[t]);
          }
        }
      }
      T* out = dq + b * dsh.q_strides[0] + h * dsh.q_strides[1] + i * dsh.q_strides[2];
#pragma unroll
      for (int t = 0; t < kMaxD / 32; ++t) {
        const int d = lane + 32 * t;
        if (d < D) Elem<T>::store(out + d, acc0[t]);
      }
    } else {
      const int64_t j = r;
      for (int64_t i0 = j; i0 < S; i0 += 32) {
        const int64_t i = i0 + lane;
        float pd = 0.f, ds = 0.f;
        if (i < S && (kstart == nullptr || kstart[b * S + i] <= j)) {  // query i attends key j
          const T* qr = qb + i * sh.q_strides[2];
          const T* gr = gb + i * sh.o_strides[2];
          const T* orow = ob + i * sh.o_strides[2];
          float s = 0.f, dpd = 0.f, delta = 0.f;
          for (int d = 0; d < D; ++d) {
            const float g = Elem<T>::load(gr + d);
            s = fmaf(xs[w][d], Elem<T>::load(qr + d), s);
            dpd = fmaf(ys[w][d], g, dpd);
            delta = fmaf(g, Elem<T>::load(orow + d), delta);
          }
          const int64_t ri = bh * S + i;
          const float p = expf(s * scale - row_max[ri]) / row_sum[ri];
          const float f = dr.factor(bh, S, i, j);
          pd = p * f;
          ds = p * (dpd * f - delta) * scale;
        }
        const int cnt = static_cast<int>(S - i0 < 32 ? S - i0 : 32);
        for (int ii = 0; ii < cnt; ++ii) {
          const float pdi = __shfl_sync(0xffffffffu, pd, ii);
          const float dsi = __shfl_sync(0xffffffffu, ds, ii);
          const T* gr = gb + (i0 + ii) * sh.o_strides[2];
          const T* qr = qb + (i0 + ii) * sh.q_strides[2];
#pragma unroll
          for (int t = 0; t < kMaxD / 32; ++t) {
            const int d = lane + 32 * t;
            if (d < D) {
              acc0[t] = fmaf(pdi, Elem<T>::load(gr + d), acc0[t]);  // dV
              acc1[t] = fmaf(dsi, Elem<T>::load(qr + d), acc1[t]);  // dK
            }
          }
        }
      }
      T* outv = dv + b * dsh.v_strides[0] + h * dsh.v_strides[1] + j * dsh.v_strides[2];
      T* outk = dk + b * dsh.k_strides[0] + h * dsh.k_strides[1] + j * dsh.k_strides[2];
#pragma unroll
      for (int t = 0; t < kMaxD / 32; ++t) {
        const int d = lane + 32 * t;
        if (d < D) {
          Elem<T>::store(outv + d, acc0[t]);
          Elem<T>::store(outk + d, acc1[t]);
        }
      }
    }
  }
}

inline int simt_grid(int64_t rows) {
  int64_t b = ceil_div(rows, kWarpsPerBlock);
  const int64_t cap = static_cast<int64_t>(kNumSMs) * 16;
  return static_cast<int>(b < cap ? b : cap);
}

}  // namespace

int attn_fwd_simt(const void* q, const void* k, const void* v, void* o, float* row_max, float* row_sum,
                  const int32_t* row_kstart, const ptj_attn_shape& sh, const AttnDropout& dr, int dtype, cudaStream_t st) {
  if (sh.d_head > kMaxD) return PTJ_ERR_UNSUPPORTED;
  const float scale = 1.f / sqrtf(static_cast<float>(sh.d_head));
  const int grid = simt_grid(sh.batch * sh.heads * sh.seq);
  if (dtype == PTJ_F32)
    launch_k(attn_fwd_simt_kernel<float>, grid, kWarpsPerBlock * 32, 0, st, 
        static_cast<const float*>(q), static_cast<const float*>(k), static_cast<const float*>(v), static_cast<float*>(o),
        row_max, row_sum, row_kstart, sh, scale, dr);
  else
    launch_k(attn_fwd_simt_kernel<__nv_bfloat16>, grid, kWarpsPerBlock * 32, 0, st, 
        static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v),
        static_cast<__nv_bfloat16*>(o), row_max, row_sum, row_kstart, sh, scale, dr);
  PTJ_CHECK_LAUNCH();
  return PTJ_OK;
}

template <typename T>
static int bwd_simt_typed(const void* d_o, const void* q, const void* k, const void* v, const void* o,
                          const float* row_max, const float* row_sum, void* dq, void* dk, void* dv,
                          const int32_t* row_kstart, const ptj_attn_shape& sh, const ptj_attn_shape& dsh,
                          const AttnDropout& dr, cudaStream_t st) {
  const float scale = 1.f / sqrtf(static_cast<float>(sh.d_head));
  const int grid = simt_grid(sh.batch * sh.heads * sh.seq);
  launch_k(attn_bwd_simt_kernel<T, 0>, grid, kWarpsPerBlock * 32, 0, st, 
      static_cast<const T*>(d_o), static_cast<const T*>(q), static_cast<const T*>(k), static_cast<const T*>(v),
      static_cast<const T*>(o), row_max, row_sum, static_cast<T*>(dq), static_cast<T*>(dk), static_cast<T*>(dv),
      row_kstart, sh, dsh, scale, dr);
  PTJ_CHECK_LAUNCH();
  launch_k(attn_bwd_simt_kernel<T, 1>, grid, kWarpsPerBlock * 32, 0, st, 
      static_cast<const T*>(d_o), static_cast<const T*>(q), static_cast<const T*>(k), static_cast<const T*>(v),
      static_cast<const T*>(o), row_max, row_sum, static_cast<T*>(dq), static_cast<T*>(dk), static_cast<T*>(dv),
      row_kstart, sh, dsh, scale, dr);
  PTJ_CHECK_LAUNCH();
  return PTJ_OK;
}

int attn_bwd_simt(const void* d_o, const void* q, const void* k, const void* v, const void* o, const float* row_max,
                  const float* row_sum, void* dq, void* dk, void* dv, const int32_t* row_kstart,
                  const ptj_attn_shape& sh, const ptj_attn_shape& dsh, const AttnDropout& dr, int dtype, cudaStream_t st) {
  if (sh.d_head > kMaxD) return PTJ_ERR_UNSUPPORTED;
  if (dtype == PTJ_F32)
    return bwd_simt_typed<float>(d_o, q, k, v, o, row_max, row_sum, dq, dk, dv, row_kstart, sh, dsh, dr, st);
  return bwd_simt_typed<__nv_bfloat16>(d_o, q, k, v, o, row_max, row_sum, dq, dk, dv, row_kstart, sh, dsh, dr, st);
}

}  // namespace ptj
