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
  int64_t mask_row0;     // row of the logical [M, N] matrix that row 0 of c is (non-zero when c is a row range of it)
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

// The arithmetic of the epilogue for one row segment, in two phases: acc[0..CNT) are columns n0 .. n0+CNT-1 of row m
// (CNT and n0 multiples of 8). epilogue_pre adds the bias; in GELU mode acc then holds the pre-activation (already
// rounded to the output type) which the caller may store into aux_out. epilogue_post turns acc into the values to
// store into C. epilogue_pre returns false when the segment lies outside the matrix (nothing to compute or store).
template <typename TOut, int CNT>
__device__ __forceinline__ bool epilogue_pre(const EpilogueParams& ep, int64_t m, int64_t n0, float (&acc)[CNT],
                                             const float* bias_s = nullptr) {
  if (m >= ep.M || n0 >= ep.N) return false;

  if (bias_s != nullptr) {
    // the tile's bias slice was staged in shared memory (zero beyond N): broadcast 16-byte reads
#pragma unroll
    for (int j = 0; j < CNT; j += 4) {
      const float4 b4 = *reinterpret_cast<const float4*>(bias_s + j);
      acc[j] += b4.x; acc[j + 1] += b4.y; acc[j + 2] += b4.z; acc[j + 3] += b4.w;
    }
  } else if (ep.bias != nullptr) {
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
  if (ep.mode == PTJ_EPI_GELU && sizeof(TOut) == 2) {
    // the activation sees the pre-activation as stored (rounded to the output type), like a separate GELU kernel would
#pragma unroll
    for (int j = 0; j < CNT; j += 2) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(acc[j], acc[j + 1]);
      const uint32_t w = *reinterpret_cast<const uint32_t*>(&h);
      acc[j] = __uint_as_float(w << 16);
      acc[j + 1] = __uint_as_float(w & 0xffff0000u);
    }
  }
  return true;
}

// which tensor the second phase reads next to the accumulator (nullptr: none)
__device__ __forceinline__ const void* epilogue_side_input(const EpilogueParams& ep) {
  if (ep.mode == PTJ_EPI_GELU_BWD || ep.mode == PTJ_EPI_DROPOUT_RESID) return ep.aux;
  if (ep.mode == PTJ_EPI_ACCUM) return ep.c;
  return nullptr;
}

// a[] = the side input's values at (m, n0 .. n0+CNT-1) (ignored when the mode has no side input)
// seed: ep.seed resolved by the caller (resolve_seed), once per thread
template <typename TOut, int CNT>
__device__ __forceinline__ void epilogue_post(const EpilogueParams& ep, int64_t m, int64_t n0, float (&acc)[CNT],
                                              const float (&a)[CNT], uint64_t seed) {
  constexpr bool kFast = sizeof(TOut) == 2;  // bf16 output: hardware tanh is exact enough after rounding
  if (ep.mode == PTJ_EPI_GELU) {
    if (kFast) {
#pragma unroll
      for (int j = 0; j < CNT; j += 2) gelu_tanh_x2(acc[j], acc[j + 1]);
    } else {
#pragma unroll
      for (int j = 0; j < CNT; ++j) acc[j] = gelu_tanh<kFast>(acc[j]);
    }
  } else if (ep.mode == PTJ_EPI_GELU_BWD) {
    if (kFast) {
#pragma unroll
      for (int j = 0; j < CNT; j += 2) gelu_tanh_grad_mul_x2(acc[j], acc[j + 1], a[j], a[j + 1]);
    } else {
#pragma unroll
      for (int j = 0; j < CNT; ++j) acc[j] *= gelu_tanh_grad<kFast>(a[j]);
    }
  } else if (ep.mode == PTJ_EPI_ACCUM) {
#pragma unroll
    for (int j = 0; j < CNT; ++j) acc[j] += a[j];
  } else if (ep.mode == PTJ_EPI_DROPOUT_RESID) {
    // mask indexed by the logical element position m * N + n (the stream ptj_dropout uses on a contiguous [M, N])
    const uint64_t base = static_cast<uint64_t>(m + ep.mask_row0) * static_cast<uint64_t>(ep.N) + static_cast<uint64_t>(n0);
    if (!ep.train) {
#pragma unroll
      for (int j = 0; j < CNT; ++j) acc[j] = fmaf(acc[j], ep.eval_scale, a[j]);
    } else if (ep.drop_thr == 0u) {
#pragma unroll
      for (int j = 0; j < CNT; ++j) acc[j] += a[j];
    } else if ((base & 7) == 0) {
#pragma unroll
      for (int j = 0; j < CNT; j += 8) {
        const uint32_t keep = dropout_keep_bits8(seed, ep.stream_id, (base + j) >> 3, ep.drop_thr);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[j + e] = a[j + e] + (((keep >> e) & 1u) ? acc[j + e] : 0.f);
      }
    } else {
#pragma unroll
      for (int j = 0; j < CNT; ++j)
        acc[j] = a[j] + (dropout_keep(seed, ep.stream_id, base + j, ep.drop_thr) ? acc[j] : 0.f);
    }
  }
}

// both phases + per-thread stores (used where one thread owns a short row segment)
template <typename TOut, int CNT>
__device__ __forceinline__ void epilogue_row_segment(const EpilogueParams& ep, int64_t m, int64_t n0, float (&acc)[CNT],
                                                     uint64_t seed) {
  if (!epilogue_pre<TOut, CNT>(ep, m, n0, acc)) return;
  const bool full = ep.vec_ok && n0 + CNT <= ep.N;
  if (ep.mode == PTJ_EPI_GELU && ep.aux_out != nullptr)
    store_row<TOut, CNT>(static_cast<TOut*>(ep.aux_out) + m * ep.ldc, n0, ep.N, full, acc);
  float a[CNT];
  if (const void* side = epilogue_side_input(ep)) load_row<TOut, CNT>(static_cast<const TOut*>(side) + m * ep.ldc, n0, ep.N, full, a);
  epilogue_post<TOut, CNT>(ep, m, n0, acc, a, seed);
  store_row<TOut, CNT>(static_cast<TOut*>(ep.c) + m * ep.ldc, n0, ep.N, full, acc);
}

// Warp-cooperative store of a 32-row x 32-column block whose rows are held one per lane: each lane parks its row in a
// padded shared-memory strip, then the warp writes it out 8 rows at a time with four lanes per row, so every global
// store instruction covers whole 64-byte row segments (full 32-byte sectors) instead of 32 scattered 16-byte pieces.
// `strip` is this warp's 32 x 80 bytes. Rows >= M are skipped. Requires 16-byte aligned rows (vec_ok) and a full
// 32-column block; all lanes of the warp must call it.
constexpr int kStripRowBytes = 80;  // 64 data bytes + 16 padding: conflict-free 16-byte accesses
constexpr int kStripBytes = 32 * kStripRowBytes;
template <typename TOut>
__device__ __forceinline__ void warp_store_block(uint8_t* strip, TOut* base, int64_t ld, int64_t row0, int64_t n0,
                                                 int64_t M, const float (&v)[32], int lane) {
  constexpr int kElemsPerPass = 64 / sizeof(TOut);  // 32 bf16 or 16 floats per 64-byte pass
#pragma unroll
  for (int pass = 0; pass < 32 / kElemsPerPass; ++pass) {
    uint8_t* mine = strip + lane * kStripRowBytes;
    if (sizeof(TOut) == 2) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const __nv_bfloat162 h = __floats2bfloat162_rn(v[q * 8 + 2 * i], v[q * 8 + 2 * i + 1]);
          w[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(mine + q * 16) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q)
        *reinterpret_cast<float4*>(mine + q * 16) =
            make_float4(v[pass * 16 + q * 4], v[pass * 16 + q * 4 + 1], v[pass * 16 + q * 4 + 2], v[pass * 16 + q * 4 + 3]);
    }
    __syncwarp();
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int rr = it * 8 + (lane >> 2), q = lane & 3;
      const uint4 t = *reinterpret_cast<const uint4*>(strip + rr * kStripRowBytes + q * 16);
      if (row0 + rr < M) {
        uint8_t* dst = reinterpret_cast<uint8_t*>(base + (row0 + rr) * ld + n0) + pass * 64 + q * 16;
        *reinterpret_cast<uint4*>(dst) = t;
      }
    }
    __syncwarp();
  }
}

// The mirror image: the warp reads a 32 x 32 block with whole 64-byte row segments per quad of lanes, parks it in the
// strip, and every lane picks up its own row. Rows >= M read as zero.
template <typename TOut>
__device__ __forceinline__ void warp_load_block(uint8_t* strip, const TOut* base, int64_t ld, int64_t row0, int64_t n0,
                                                int64_t M, float (&v)[32], int lane) {
  constexpr int kElemsPerPass = 64 / sizeof(TOut);
#pragma unroll
  for (int pass = 0; pass < 32 / kElemsPerPass; ++pass) {
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int rr = it * 8 + (lane >> 2), q = lane & 3;
      uint4 t = make_uint4(0u, 0u, 0u, 0u);
      if (row0 + rr < M)
        t = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(base + (row0 + rr) * ld + n0) + pass * 64 + q * 16);
      *reinterpret_cast<uint4*>(strip + rr * kStripRowBytes + q * 16) = t;
    }
    __syncwarp();
    const uint8_t* mine = strip + lane * kStripRowBytes;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint4 t = *reinterpret_cast<const uint4*>(mine + q * 16);
      const uint32_t w[4] = {t.x, t.y, t.z, t.w};
      if (sizeof(TOut) == 2) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          v[q * 8 + 2 * i] = __uint_as_float(w[i] << 16);
          v[q * 8 + 2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) v[pass * 16 + q * 4 + i] = __uint_as_float(w[i]);
      }
    }
    __syncwarp();
  }
}

}  // namespace ptj
