// Device and host helpers shared by the tcgen05 attention kernels (forward and backward translation units).
#pragma once
#include "attn_common.cuh"
#include "tc_common.cuh"
#include "tc_runtime.h"

namespace ptj {
namespace attn_tc {

using namespace tc;

constexpr int T = 128;            // tile edge along queries and keys
constexpr int DH = 64;            // head size
constexpr int kTileBytes = T * DH * 2;  // one [128][64] bf16 tile
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct RowView {  // a [batch, heads, seq, 64] view with 64 contiguous
  __nv_bfloat16* base;
  int64_t sb, sh, sr;
  __device__ __forceinline__ __nv_bfloat16* row(int64_t b, int64_t h, int64_t r) const {
    return base + b * sb + h * sh + r * sr;
  }
};

struct AttnParams {
  int S, H, BH, nq;
  float scale_log2;  // log2(e) / sqrt(d_head)
  float scale;       // 1 / sqrt(d_head)
  AttnDropout dr;
  const uint4* keep_bits;  // optional precomputed keep flags, one uint4 per (batch*head, tile, row): see attn_keep_bits_tc
  const int32_t* kstart;   // optional [batch, seq]: first key a query row may attend to (document start); NULL = 0
  unsigned int* fault;
};

// Philox round keys of a seed (round r uses rk[2r], rk[2r+1]): the same for every call of a kernel, so one thread
// writes them to shared memory at start-up, after resolving the seed argument (it may be the address of the seed).
__device__ __forceinline__ void philox_round_keys(uint64_t seed_arg, uint32_t* rk) {
  const uint64_t seed = resolve_seed(seed_arg);
  for (int r = 0; r < 10; ++r) {
    rk[2 * r] = static_cast<uint32_t>(seed) + static_cast<uint32_t>(r) * 0x9E3779B9u;
    rk[2 * r + 1] = static_cast<uint32_t>(seed >> 32) + static_cast<uint32_t>(r) * 0xBB67AE85u;
  }
}
// philox4x32_10 of common.cuh with the key schedule taken from a table
__device__ __forceinline__ void philox_rk(const uint32_t* rk, uint64_t ctr, uint32_t stream_id, uint32_t (&out)[4]) {
  uint32_t c0 = static_cast<uint32_t>(ctr), c1 = static_cast<uint32_t>(ctr >> 32), c2 = stream_id, c3 = 0x5054'4a31u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = static_cast<uint64_t>(0xD2511F53u) * c0;
    const uint64_t p1 = static_cast<uint64_t>(0xCD9E8D57u) * c2;
    const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c1 ^ rk[2 * r];
    const uint32_t n2 = static_cast<uint32_t>(p0 >> 32) ^ c3 ^ rk[2 * r + 1];
    c1 = static_cast<uint32_t>(p1);
    c3 = static_cast<uint32_t>(p0);
    c0 = n0;
    c2 = n2;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// keep flags of 32 consecutive probability elements starting at flat index idx0 (a multiple of 8)
__device__ __forceinline__ uint32_t keep_bits32(const AttnDropout& dr, uint64_t idx0) {
  uint32_t bits = 0;
#pragma unroll
  for (int c = 0; c < 4; ++c) bits |= dropout_keep_bits8(dr.seed, dr.stream_id, (idx0 >> 3) + c, dr.thr16) << (c * 8);
  return bits;
}

// Write 32 consecutive columns (col0 % 32 == 0) of row r of a [128][128] bf16 tile stored as two [128][64]
// 128-byte-swizzled sub-tiles that are kTileBytes apart.
__device__ __forceinline__ void store_row32_sw128(uint8_t* tile, int r, int col0, const float (&v)[32]) {
  uint8_t* line = tile + (col0 >> 6) * kTileBytes + r * 128;
  const int cb = (col0 & 63) >> 3;
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(v[t * 8 + 2 * i], v[t * 8 + 2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(line + (((cb + t) ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

__device__ __forceinline__ void tmem_ld_row32(uint32_t taddr, float (&f)[32]) {
  uint32_t r[32];
  tmem_ld_32x32(taddr, r);
  tmem_ld_wait();
#pragma unroll
  for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(r[j]);
}

// 2^x on the special-function unit (inputs here are <= 0 or small; subnormal results flush to zero)
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// NCALL consecutive counters at once, rounds in a rolled loop (small code, the calls give the instruction-level
// parallelism), round keys read from shared memory (rk_s[2r], rk_s[2r+1]).
template <int NCALL>
__device__ __forceinline__ void philox_rolled(const uint32_t* rk_s, uint64_t ctr0, uint32_t stream_id, uint32_t (&out)[NCALL][4]) {
  uint32_t c0[NCALL], c1[NCALL], c2[NCALL], c3[NCALL];
#pragma unroll
  for (int q = 0; q < NCALL; ++q) {
    const uint64_t ctr = ctr0 + q;
    c0[q] = static_cast<uint32_t>(ctr);
    c1[q] = static_cast<uint32_t>(ctr >> 32);
    c2[q] = stream_id;
    c3[q] = 0x5054'4a31u;
  }
#pragma unroll 1
  for (int r = 0; r < 10; ++r) {
    const uint32_t k0 = rk_s[2 * r], k1 = rk_s[2 * r + 1];
#pragma unroll
    for (int q = 0; q < NCALL; ++q) {
      const uint64_t p0 = static_cast<uint64_t>(0xD2511F53u) * c0[q];
      const uint64_t p1 = static_cast<uint64_t>(0xCD9E8D57u) * c2[q];
      const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c1[q] ^ k0;
      const uint32_t n2 = static_cast<uint32_t>(p0 >> 32) ^ c3[q] ^ k1;
      c1[q] = static_cast<uint32_t>(p1);
      c3[q] = static_cast<uint32_t>(p0);
      c0[q] = n0;
      c2[q] = n2;
    }
  }
#pragma unroll
  for (int q = 0; q < NCALL; ++q) {
    out[q][0] = c0[q]; out[q][1] = c1[q]; out[q][2] = c2[q]; out[q][3] = c3[q];
  }
}

// packed pairs of floats for the two-wide fp32 instructions of sm_100 (fma.rn.f32x2, add.f32x2)
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// descriptors of the five operand flavours used below (all tiles are 128-byte swizzled, 8-line groups 1024 B apart)
__device__ __forceinline__ uint64_t desc_kmajor_d(uint32_t tile, int k16) {  // [rows][64 d], K = d
  return smem_desc_sw128(tile + k16 * 32, 16, 1024);
}
__device__ __forceinline__ uint64_t desc_rows_as_k(uint32_t tile, int k16) {  // [128 rows][64 d], K = rows, MN = d
  return smem_desc_sw128(tile + k16 * 2048, kTileBytes, 1024);
}
__device__ __forceinline__ uint64_t desc_p_kmajor(uint32_t tile, int k16) {  // [128 q][128 kv], M = q, K = kv
  return smem_desc_sw128(tile + (k16 >> 2) * kTileBytes + (k16 & 3) * 32, 16, 1024);
}
__device__ __forceinline__ uint64_t desc_p_transposed(uint32_t tile, int k16) {  // same bytes, M = kv, K = q rows
  return smem_desc_sw128(tile + k16 * 2048, kTileBytes, 1024);
}

__device__ __forceinline__ uint8_t* align1024(uint8_t* raw) {
  return raw + ((1024u - (smem_u32(raw) & 1023u)) & 1023u);
}

// ---- host side -------------------------------------------------------------------------------------------------
inline bool make_map(CUtensorMap* m, const void* base, const ptj_attn_shape& sh, const int64_t (&st)[3]) {
  const uint64_t dims[4] = {static_cast<uint64_t>(DH), static_cast<uint64_t>(sh.seq), static_cast<uint64_t>(sh.heads),
                            static_cast<uint64_t>(sh.batch)};
  // a size-1 dimension may come with a zero stride; the encoder wants positive multiples of 16 bytes
  auto fix = [&](int64_t s) { return static_cast<uint64_t>(s > 0 ? s : DH) * 2; };
  const uint64_t strides[3] = {fix(st[2]), fix(st[1]), fix(st[0])};
  const uint32_t box[4] = {DH, T, 1, 1};
  return make_tmap_bf16(m, base, 4, dims, strides, box);
}

inline RowView make_view(const void* base, const int64_t (&st)[3]) {
  return RowView{static_cast<__nv_bfloat16*>(const_cast<void*>(base)), st[0], st[1], st[2]};
}

inline AttnParams make_params(const ptj_attn_shape& sh, const AttnDropout& dr) {
  AttnParams p{};
  p.S = static_cast<int>(sh.seq);
  p.H = static_cast<int>(sh.heads);
  p.BH = static_cast<int>(sh.batch * sh.heads);
  p.nq = p.S / T;
  p.scale = 1.f / sqrtf(static_cast<float>(DH));
  p.scale_log2 = p.scale * kLog2e;
  p.dr = dr;
  p.fault = tc::fault_word();
  return p;
}

}  // namespace attn_tc
}  // namespace ptj
