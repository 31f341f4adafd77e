// Causal flash attention backward on tcgen05 tensor cores (bf16 in, fp32 accumulate), d_head = 64, seq % 128 == 0.
// Semantics: model_triton.py:801-811 / 550-577: with P = softmax(causal(Q K^T / sqrt(d))) recomputed from the saved row
// statistics and Pd = dropout(P):  dV = Pd^T dO,  dP = dO V^T,  dS = P o (dP o keep - delta) / sqrt(d) with
// delta = rowsum(dO o O),  dK = dS^T Q,  dQ = dS K.
//
// Three launches:
//   1. prep:   delta[q] and the log2-domain log-sum-exp of every query row (one warp per four rows)
//   2. main:   persistent, warp-specialised block per SM. A work item is a (KV tile j, batch*head); its tiles are the
//              query tiles i >= j. dK_j and dV_j accumulate in tensor memory over the item; the 128 x 64 product
//              dS_ij K_j (tile i's share of dQ_i) is written to an fp32 workspace.
//   3. reduce: dQ_i = sum over j <= i of the workspace tiles, in a fixed order, to bf16.
// No atomics anywhere, so every result is bit-reproducible (the reference adds dQ with tl.atomic_add, :938).
//
// Main kernel, 384 threads:
//   warp 0      one thread issues the TMA copies: K_j, V_j of an item (2 buffers), Q_i and dO_i of a tile (3 stages)
//   warp 1      issues S = Q_i K_j^T and dP = dO_i V_j^T (dP goes into the columns S occupied once the scores have
//               been read out)
//   warp 2      issues dV += Pd^T dO_i for every tile in stream order
//   warp 3      issues dK += dS^T Q_i in stream order, then the tile's dQ share dS K_j (one issuer per accumulator
//               keeps the accumulation order fixed)
//   warps 4..7 / 8..11  two compute groups; group x takes the tiles of the block's tile stream with g % 2 == x, so one
//               group's exponentials overlap the other's loads, stores and barriers. Thread t owns query row t of
//               the tile (tensor-memory lane t). It forms P (kept as packed bf16 whose sign bit marks a dropped
//               element), writes Pd to shared memory, then turns dP into dS in the same buffer.
// Tensor memory (512 columns): [0,256) S / dP of the two groups, [256,384) the dQ shares of the two groups,
// [384,448) dV, [448,512) dK.
#include "attn_tc_dev.cuh"

namespace ptj {
namespace {

using namespace attn_tc;

constexpr int kThreads = 384;
constexpr int kOffKV = 0;                                  // K[2], V[2] (item buffers)
constexpr int kQGStages = 3;
constexpr int kOffQG = 4 * kTileBytes;                     // per stage: Q then dO
constexpr int kOffW = kOffQG + kQGStages * 2 * kTileBytes; // per group: one [128][128] bf16 tile, Pd then dS
constexpr int kOffBars = kOffW + 4 * kTileBytes;
constexpr int kNumBars = 32;
constexpr int kSmemBytes = kOffBars + kNumBars * 8 + 16 + 80 + 4 * 32 + 1024;  // (+ 32 last-tile entries, VARLEN)
constexpr int kTmemCols = 512;
constexpr uint32_t kColS = 0, kColDQ = 256, kColDV = 384, kColDK = 448;

struct Sched {
  int total, rounds, nq, BH;
  uint32_t bh_magic;  // ceil(2^32 / BH): x / BH == umulhi(x, bh_magic) for every x the kernel meets (checked on the host)
};

// Position in the stream of (item, query tile) pairs of one thread block; every role walks the same stream.
// Items are ordered heaviest first (KV tile 0 has the most query tiles) and dealt in boustrophedon order.
// last_tile (VARLEN): per round of this block, the last query tile whose rows reach into the item's KV tile (later
// query tiles mask all of its keys: they are skipped); nullptr = every item runs to the last query tile.
constexpr int kMaxRoundsTabled = 32;
struct Cursor {
  int n, ord, kt, bh, i, i1, g;
  bool valid;
  const int* last_tile;
  __device__ __forceinline__ void next_item(const Sched& s) {
    valid = false;
    while (++n < s.rounds) {
      const int pos = (n & 1) ? static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x);
      const int sp = n * static_cast<int>(gridDim.x) + pos;
      if (sp < s.total) {
        kt = s.BH == 1 ? sp : static_cast<int>(__umulhi(static_cast<uint32_t>(sp), s.bh_magic));  // sp / BH
        bh = sp - kt * s.BH;
        i = kt;
        i1 = last_tile != nullptr ? last_tile[n] : s.nq - 1;
        ++ord;
        valid = true;
        return;
      }
    }
  }
  __device__ __forceinline__ void init(const Sched& s, const int* last = nullptr) {
    n = -1; ord = -1; g = 0; kt = 0; bh = 0; i = 0; i1 = 0;
    last_tile = last;
    next_item(s);
  }
  __device__ __forceinline__ bool first(const Sched&) const { return i == kt; }
  __device__ __forceinline__ bool last(const Sched&) const { return i == i1; }
  __device__ __forceinline__ void advance(const Sched& s) {
    ++g;
    if (i == i1) next_item(s); else ++i;
  }
};

// ---- 1. per-row constants ------------------------------------------------------------------------------------------
// Eight lanes per query row: delta = sum_d dO[q,d] O[q,d]; lse2 = (row_max + log(row_sum)) * log2(e).
__global__ void __launch_bounds__(256)
attn_bwd_prep_kernel(const RowView d_o, const RowView o_view, const float* __restrict__ row_max,
                     const float* __restrict__ row_sum, float* __restrict__ delta, float* __restrict__ lse2, int S, int H,
                     int64_t rows) {
  grid_dep_sync();
  const int64_t r = (static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x) >> 3;
  const int part = threadIdx.x & 7;
  float acc = 0.f;
  if (r < rows) {
    const int64_t bh = r / S, q = r % S;
    const __nv_bfloat16* g = d_o.row(bh / H, bh % H, q) + part * 8;
    const __nv_bfloat16* o = o_view.row(bh / H, bh % H, q) + part * 8;
    float x[8], y[8];
    Elem<__nv_bfloat16>::load_vec(g, x);
    Elem<__nv_bfloat16>::load_vec(o, y);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc = fmaf(x[i], y[i], acc);
  }
  acc += __shfl_xor_sync(0xffffffffu, acc, 1);
  acc += __shfl_xor_sync(0xffffffffu, acc, 2);
  acc += __shfl_xor_sync(0xffffffffu, acc, 4);
  if (r < rows && part == 0) {
    delta[r] = acc;
    lse2[r] = (row_max[r] + logf(row_sum[r])) * kLog2e;
  }
}

// ---- 3. dQ = sum of the per-KV-tile shares ---------------------------------------------------------------------------
// A share is stored as 16 blocks of four columns, 128 rows each (a warp of the main kernel writes 512 contiguous
// bytes per store): float4 index ((bh * ntri + qt (qt + 1) / 2 + kt) * 16 + c4) * 128 + row. One thread sums one
// float4 over kt; consecutive threads take consecutive rows.
__global__ void __launch_bounds__(256)
attn_dq_reduce_kernel(const float* __restrict__ part, const RowView dq, const int32_t* __restrict__ kstart, int S, int H,
                      int nq, int64_t total_vec) {
  grid_dep_sync();
  const int64_t v = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
  if (v >= total_vec) return;
  const int row = static_cast<int>(v % T);
  const int c4 = static_cast<int>((v / T) % (DH / 4));
  const int64_t tile_id = v / (T * (DH / 4));  // bh * nq + qt
  const int64_t bh = tile_id / nq;
  const int qt = static_cast<int>(tile_id % nq);
  const int64_t q = static_cast<int64_t>(qt) * T + row;
  const int64_t ntri = static_cast<int64_t>(nq) * (nq + 1) / 2;
  const float4* src = reinterpret_cast<const float4*>(part) +
                      ((bh * ntri + static_cast<int64_t>(qt) * (qt + 1) / 2) * (DH / 4) + c4) * T + row;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  // packed / padded batches: shares of KV tiles before the row's first key were either skipped by the main kernel (not
  // written) or are exact zeros; a row without keys sums nothing
  int kt0 = 0;
  if (kstart != nullptr) {
    const int k = __ldg(kstart + (bh / H) * S + q);
    kt0 = k > q ? qt + 1 : max(k, 0) / T;
  }
  for (int kt = kt0; kt <= qt; ++kt) {
    const float4 t = __ldcs(src + static_cast<int64_t>(kt) * T * (DH / 4));
    acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
  }
  __nv_bfloat16* dst = dq.row(bh / H, bh % H, q) + c4 * 4;
  const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
  uint2 pk;
  pk.x = *reinterpret_cast<const uint32_t*>(&lo);
  pk.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(dst) = pk;
}

// ---- per-thread phases of the main kernel: straight-line code (no branch inside the unrolled loops) ------------------
// P phase of one 32-column chunk: s holds the raw scores on entry (-inf where the causal mask applies) and Pd (what
// goes to shared memory) on exit;
// pk receives P as packed bf16 pairs whose sign bit marks a dropped element. rw: the four Philox calls of the chunk.
// MODE 0: no mask; 1: raw Philox words in rw; 2: precomputed keep flags of the chunk in keepw (bit i = column i).
template <int MODE>
__device__ __forceinline__ void p_chunk(float (&s)[32], uint32_t* pk, const uint32_t (&rw)[4][4], uint32_t keepw,
                                        uint64_t sc2, uint64_t nl2, uint32_t thr_hi, float f_keep) {
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    float a, b;
    unpack2(fma2(pack2(s[i], s[i + 1]), sc2, nl2), a, b);
    a = ex2_approx(a);
    b = ex2_approx(b);
    float sa = a, sb = b;
    if (MODE != 0) {
      bool drop_a, drop_b;
      if (MODE == 1) {  // 16-bit lanes of word (i % 8) / 2 of call i / 8: low half = even element, high half = odd
        const uint32_t w = rw[i >> 3][(i & 7) >> 1];
        drop_a = (w << 16) < thr_hi;
        drop_b = w < thr_hi;
      } else {
        drop_a = (keepw & (1u << i)) == 0u;
        drop_b = (keepw & (2u << i)) == 0u;
      }
      sa = drop_a ? -a : a;
      sb = drop_b ? -b : b;
      a = drop_a ? 0.f : a;
      b = drop_b ? 0.f : b;
    }
    const __nv_bfloat162 h2 = __floats2bfloat162_rn(sa, sb);
    pk[i >> 1] = *reinterpret_cast<const uint32_t*>(&h2);
    s[i] = a * f_keep;
    s[i + 1] = b * f_keep;
  }
}
// dS phase of one chunk: s holds dP on entry and dS = P o (dP o keep * f_keep - delta) / sqrt(d) on exit.
template <bool MASKED>
__device__ __forceinline__ void ds_chunk(float (&s)[32], const uint32_t* pk, float ksc, float dsc) {
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    const uint32_t w = pk[i >> 1];
    const float xa = __uint_as_float(w << 16), xb = __uint_as_float(w & 0xffff0000u);
    float da = s[i], db = s[i + 1];
    if (MASKED) {
      da = xa < 0.f ? 0.f : da;
      db = xb < 0.f ? 0.f : db;
    }
    s[i] = fabsf(xa) * fmaf(da, ksc, -dsc);
    s[i + 1] = fabsf(xb) * fmaf(db, ksc, -dsc);
  }
}

// ---- 2. main kernel --------------------------------------------------------------------------------------------------
struct BwdViews {
  RowView dk, dv;
};

// VARLEN: query row i attends keys [p.kstart[b, i], i] only (see the forward kernel); masked scores are -inf, so their
// probabilities, and with them every product they enter, are exact zeros.
template <int MODE, bool VARLEN>
__global__ void __launch_bounds__(kThreads, 1)
attn_bwd_ws_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_g,
                   const float* __restrict__ delta, const float* __restrict__ lse2, float* __restrict__ dq_part,
                   const BwdViews outv, const AttnParams p, const Sched sched) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = align1024(smem_raw);
  uint8_t* kv_s = sm + kOffKV;  // item buffer b: K at b * 2 tiles, V right behind it
  uint8_t* qg_s = sm + kOffQG;  // stage x: Q at x * 2 tiles, dO right behind it
  uint8_t* w_s = sm + kOffW;    // group x: [128][128] bf16 at x * 2 tiles
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + kOffBars);
  uint64_t* kv_full = bars;            // [2]
  uint64_t* kv_empty = bars + 2;       // [2] two arrivals: last dP and last dQ share of the item
  uint64_t* s_full = bars + 4;         // [2] per group from here on
  uint64_t* s_free = bars + 6;         //     scores are in registers (one arrival per warp)
  uint64_t* dp_full = bars + 8;
  uint64_t* dp_free = bars + 10;       //     dP is in registers (one arrival per warp)
  uint64_t* pd_ready = bars + 12;      //     Pd is in the group's shared-memory tile (one arrival per warp)
  uint64_t* dv_done = bars + 14;       //     the dV MMA has read it
  uint64_t* ds_ready = bars + 16;      //     dS is in the group's shared-memory tile (one arrival per warp)
  uint64_t* dkq_done = bars + 18;      //     the dK and dQ-share MMAs (one issuer, one commit) have read it
  uint64_t* dq_full = bars + 20;
  uint64_t* dq_free = bars + 22;       //     the dQ share has been copied out (one arrival per warp)
  uint64_t* acc_full = bars + 24;      // the item's last dV and last dK MMAs are done (two arrivals)
  uint64_t* acc_free = bars + 25;      // dV / dK have been copied out (one arrival per warp of the finishing group)
  uint64_t* qg_full = bars + 26;       // [kQGStages]
  uint64_t* qg_empty = bars + 29;      // [kQGStages] the tile's dV and dK MMAs are done (two arrivals; S, dP came before)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint32_t* rk_s = tmem_slot + 2;  // Philox round keys
  int* last_tab = reinterpret_cast<int*>(rk_s + 20);  // [kMaxRoundsTabled] last query tile of this block's items (VARLEN)

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const AbortCtx ctx{abort_flag, p.fault};

  if (tid == 0) {
    for (int i = 0; i < kNumBars; ++i) {
      uint64_t* b = &bars[i];
      const int pair = i >> 1;  // the per-group barriers come in pairs
      uint32_t count = 1;       // TMA transactions and MMA commits
      if (b == acc_free || pair == 3 || pair == 5 || pair == 6 || pair == 8 || pair == 11) count = 4;  // compute warps
      if (pair == 1 || b == acc_full || i >= 29) count = 2;  // kv_empty, acc_full, qg_empty[]: two MMA commits each
      mbar_init(b, count);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_k);
    prefetch_tensormap(&tm_v);
    prefetch_tensormap(&tm_g);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  grid_dep_sync();  // set-up above touches no global memory; everything below may
  const uint32_t tmem = *tmem_slot;
  if (MODE == 1) {  // the kernel draws its own keep flags: round keys of the (possibly device-resident) seed
    if (tid == 0) philox_round_keys(p.dr.seed, rk_s);
    __syncthreads();
  }
  // VARLEN: query tiles none of whose rows reach into the item's KV tile are skipped. Warp w looks at the item of round
  // w, w + 12, ...: the last query tile with a row whose first key lies in or before the KV tile (the diagonal tile is
  // always visited).
  const int* last_tile = nullptr;
  if (VARLEN && sched.rounds <= kMaxRoundsTabled) {
    for (int n = warp; n < sched.rounds; n += kThreads / 32) {
      const int pos = (n & 1) ? static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x);
      const int sp = n * static_cast<int>(gridDim.x) + pos;
      int last = 0;
      if (sp < sched.total) {
        const int kt = sp / sched.BH, bh = sp - kt * sched.BH;
        const int32_t* ks = p.kstart + static_cast<int64_t>(bh / p.H) * p.S;
        const int kv_end = kt * T + T;  // keys of the tile are < kv_end
        last = kt;
        for (int i = kt + 1; i < sched.nq; ++i) {
          bool reach = false;
          for (int r = lane; r < T; r += 32) {
            const int row = i * T + r, k = __ldg(ks + row);
            reach = reach || (k <= row && k < kv_end);  // the row has keys and its first one is in or before the tile
          }
          if (__any_sync(0xffffffffu, reach)) last = i;
        }
      }
      if (lane == 0) last_tab[n] = last;
    }
    __syncthreads();
    last_tile = last_tab;
  }
  constexpr uint32_t idesc_s = idesc_bf16_f32(T, T, false, false);  // Q K^T and dO V^T
  constexpr uint32_t idesc_t = idesc_bf16_f32(T, DH, true, true);   // Pd^T dO and dS^T Q
  constexpr uint32_t idesc_q = idesc_bf16_f32(T, DH, false, true);  // dS K

  // the copy / MMA warps hand most of their registers to the compute warps (whole groups of four warps switch together)
  if (warp < 4) asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");

  // A polling role gives up when nothing has moved for the wait limit, or when another thread already aborted.
  auto stalled = [&](bool progress, long long& t_idle, unsigned int site) {
    if (progress) {
      t_idle = clock64();
      return false;
    }
    if (*abort_flag) return true;
    if (clock64() - t_idle > kWaitLimitCycles) {
      *abort_flag = 1;
      record_fault(p.fault, site);
      return true;
    }
    return false;
  };

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      Cursor ci, ct;  // items (K_j, V_j) and tiles (Q_i, dO_i) are two independent sequences
      ci.init(sched, last_tile);
      ct.init(sched, last_tile);
      long long t_idle = clock64();
      while (ci.valid || ct.valid) {
        bool progress = false;
        if (ci.valid) {
          const int b = ci.ord & 1;
          if (mbar_try_wait(&kv_empty[b], ((ci.ord >> 1) & 1) ^ 1u)) {
            mbar_expect_tx(&kv_full[b], 2 * kTileBytes);
            tma_load_4d(kv_s + b * 2 * kTileBytes, &tm_k, &kv_full[b], 0, ci.kt * T, ci.bh % p.H, ci.bh / p.H);
            tma_load_4d(kv_s + b * 2 * kTileBytes + kTileBytes, &tm_v, &kv_full[b], 0, ci.kt * T, ci.bh % p.H, ci.bh / p.H);
            ci.g += sched.nq - ci.i;  // skip the item's tiles
            ci.next_item(sched);
            progress = true;
          }
        }
        if (ct.valid) {
          const int x = ct.g % kQGStages;
          if (mbar_try_wait(&qg_empty[x], ((ct.g / kQGStages) & 1) ^ 1u)) {
            mbar_expect_tx(&qg_full[x], 2 * kTileBytes);
            tma_load_4d(qg_s + x * 2 * kTileBytes, &tm_q, &qg_full[x], 0, ct.i * T, ct.bh % p.H, ct.bh / p.H);
            tma_load_4d(qg_s + x * 2 * kTileBytes + kTileBytes, &tm_g, &qg_full[x], 0, ct.i * T, ct.bh % p.H, ct.bh / p.H);
            ct.advance(sched);
            progress = true;
          }
        }
        if (stalled(progress, t_idle, 0x2101u)) break;
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer: S = Q K^T, then dP = dO V^T over it
    // (all lanes walk the streams so that addresses and descriptors stay warp-uniform; an elected lane issues)
    Cursor cs, cd;
    cs.init(sched, last_tile);
    cd.init(sched, last_tile);
    long long t_idle = clock64();
    while (cs.valid || cd.valid) {
      bool progress = false;
      if (cs.valid) {
        const int x = cs.g & 1, st = cs.g % kQGStages;
        const uint32_t ph = (cs.g >> 1) & 1;
        bool ready = mbar_try_wait(&qg_full[st], (cs.g / kQGStages) & 1) &&
                     mbar_try_wait(&dp_free[x], ph ^ 1u);  // dP of tile g - 2 was read
        if (ready && cs.first(sched)) ready = mbar_try_wait(&kv_full[cs.ord & 1], (cs.ord >> 1) & 1);
        if (__all_sync(0xffffffffu, ready)) {
          tc_fence_after_sync();
          const uint32_t qa = smem_u32(qg_s + st * 2 * kTileBytes), ka = smem_u32(kv_s + (cs.ord & 1) * 2 * kTileBytes);
#pragma unroll
          for (int k16 = 0; k16 < DH / 16; ++k16)
            mma_bf16_ss_elect(tmem + kColS + x * T, desc_kmajor_d(qa, k16), desc_kmajor_d(ka, k16), idesc_s, k16 > 0);
          mma_commit_elect(&s_full[x]);
          cs.advance(sched);
          progress = true;
        }
      }
      if (cd.valid && (!cs.valid || cd.g < cs.g)) {
        const int x = cd.g & 1;
        const uint32_t ph = (cd.g >> 1) & 1;
        if (__all_sync(0xffffffffu, mbar_try_wait(&s_free[x], ph))) {
          tc_fence_after_sync();
          const uint32_t ga = smem_u32(qg_s + (cd.g % kQGStages) * 2 * kTileBytes + kTileBytes);
          const uint32_t va = smem_u32(kv_s + (cd.ord & 1) * 2 * kTileBytes + kTileBytes);
#pragma unroll
          for (int k16 = 0; k16 < DH / 16; ++k16)
            mma_bf16_ss_elect(tmem + kColS + x * T, desc_kmajor_d(ga, k16), desc_kmajor_d(va, k16), idesc_s, k16 > 0);
          mma_commit_elect(&dp_full[x]);
          if (cd.last(sched)) mma_commit_elect(&kv_empty[cd.ord & 1]);
          cd.advance(sched);
          progress = true;
        }
      }
      if (__any_sync(0xffffffffu, stalled(progress, t_idle, 0x2201u))) break;
    }
  } else if (warp == 2) {
    // ---------------------------------------------------------------- MMA issuer: dV += Pd^T dO (stream order)
    Cursor c;
    c.init(sched, last_tile);
    bool ok = true;
    while (c.valid && ok) {
      const int x = c.g & 1, st = c.g % kQGStages;
      bool w = mbar_wait(&pd_ready[x], (c.g >> 1) & 1, ctx, 0x2301u);
      if (w && c.first(sched)) w = mbar_wait(acc_free, (c.ord & 1) ^ 1u, ctx, 0x2302u);  // previous item copied out
      ok = __all_sync(0xffffffffu, w);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t wa = smem_u32(w_s + x * 2 * kTileBytes), ga = smem_u32(qg_s + st * 2 * kTileBytes + kTileBytes);
      const uint32_t acc = c.first(sched) ? 0u : 1u;
#pragma unroll
      for (int k16 = 0; k16 < T / 16; ++k16)
        mma_bf16_ss_elect(tmem + kColDV, desc_p_transposed(wa, k16), desc_rows_as_k(ga, k16), idesc_t, k16 > 0 ? 1u : acc);
      mma_commit_elect(&dv_done[x]);
      mma_commit_elect(&qg_empty[st]);
      if (c.last(sched)) mma_commit_elect(acc_full);
      c.advance(sched);
    }
  } else if (warp == 3) {
    // ---------------------------------------------------------------- MMA issuer: dK += dS^T Q (stream order) and the
    // tile's dQ share dS K_j; both read dS, so one warp issues them back to back
    Cursor c;
    c.init(sched, last_tile);
    bool ok = true;
    while (c.valid && ok) {
      const int x = c.g & 1, st = c.g % kQGStages;
      const uint32_t ph = (c.g >> 1) & 1;
      bool w = mbar_wait(&ds_ready[x], ph, ctx, 0x2401u);
      // the first dK of an item overwrites the accumulator: the previous item must have been copied out (the dV
      // issuer waits for the same barrier)
      if (w && c.first(sched)) w = mbar_wait(acc_free, (c.ord & 1) ^ 1u, ctx, 0x2403u);
      ok = __all_sync(0xffffffffu, w);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t wa = smem_u32(w_s + x * 2 * kTileBytes), qa = smem_u32(qg_s + st * 2 * kTileBytes);
      const uint32_t ka = smem_u32(kv_s + (c.ord & 1) * 2 * kTileBytes);
      const uint32_t acc = c.first(sched) ? 0u : 1u;
#pragma unroll
      for (int k16 = 0; k16 < T / 16; ++k16)
        mma_bf16_ss_elect(tmem + kColDK, desc_p_transposed(wa, k16), desc_rows_as_k(qa, k16), idesc_t, k16 > 0 ? 1u : acc);
      mma_commit_elect(&qg_empty[st]);
      if (c.last(sched)) mma_commit_elect(acc_full);
      ok = __all_sync(0xffffffffu, mbar_wait(&dq_free[x], ph ^ 1u, ctx, 0x2402u));  // previous own share copied out
      if (!ok) break;
#pragma unroll
      for (int k16 = 0; k16 < T / 16; ++k16)
        mma_bf16_ss_elect(tmem + kColDQ + x * DH, desc_p_kmajor(wa, k16), desc_rows_as_k(ka, k16), idesc_q, k16 > 0);
      mma_commit_elect(&dq_full[x]);
      mma_commit_elect(&dkq_done[x]);
      if (c.last(sched)) mma_commit_elect(&kv_empty[c.ord & 1]);
      c.advance(sched);
    }
  } else if (warp >= 4) {
    // ---------------------------------------------------------------- compute groups
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    const int quarter = warp & 3;            // tensor-memory lane quarter this warp may read
    const int grp = (warp - 4) >> 2;         // this group handles the stream's tiles with (g & 1) == grp
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t t_s = tmem + lane_base + kColS + grp * T;     // S, then dP
    const uint32_t t_q = tmem + lane_base + kColDQ + grp * DH;   // the tile's dQ share
    uint8_t* w_tile = w_s + grp * 2 * kTileBytes;
    const float f_keep = p.dr.train ? 1.f : p.dr.eval_scale;
    const uint32_t thr_hi = p.dr.thr16 << 16;
    const int ntri = p.nq * (p.nq + 1) / 2;

    Cursor c;
    c.init(sched, last_tile);
    bool ok = true;
    int64_t pend_part = -1;  // workspace tile that takes the dQ share still sitting in tensor memory
    int pend_g = 0;
    auto drain_dq = [&]() {  // copy the previous own tile's dQ share (its MMA finished long ago) to the workspace
      if (pend_part < 0) return;
      ok = mbar_wait(&dq_full[grp], (pend_g >> 1) & 1, ctx, 0x2501u);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) return;
      tc_fence_after_sync();
      float4* dst = reinterpret_cast<float4*>(dq_part) + pend_part * (T * DH / 4) + row;  // [16 column blocks][128 rows]
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        float t[32];
        tmem_ld_32x32f(t_q + cc * 32, t);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 8; ++i)
          __stcs(dst + (cc * 8 + i) * T, make_float4(t[4 * i], t[4 * i + 1], t[4 * i + 2], t[4 * i + 3]));
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&dq_free[grp]);
      pend_part = -1;
    };

    while (c.valid && ok) {
      if ((c.g & 1) == grp) {
        const uint32_t ph = (c.g >> 1) & 1;
        const int64_t q_row = static_cast<int64_t>(c.i) * T + row;
        const int64_t ri = static_cast<int64_t>(c.bh) * p.S + q_row;
        const float lse = lse2[ri];
        const float dsc = delta[ri] * p.scale;  // delta / sqrt(d)
        // dropout random words of this thread's row, one 32-column chunk ahead of their use
        uint32_t rw[2][4][4];
        const uint64_t call0 = ((static_cast<uint64_t>(c.bh) * p.S + q_row) * p.S + static_cast<uint64_t>(c.kt) * T) >> 3;
        if (MODE == 1) philox_rolled<4>(rk_s, call0, p.dr.stream_id, rw[0]);
        uint4 kb = make_uint4(0u, 0u, 0u, 0u);
        if (MODE == 2)
          kb = __ldg(p.keep_bits + (static_cast<int64_t>(c.bh) * ntri + c.i * (c.i + 1) / 2 + c.kt) * T + row);
        const uint32_t keepw[4] = {kb.x, kb.y, kb.z, kb.w};
        // ---- P from the scores; Pd to shared memory; P kept as packed bf16, sign bit set where dropped ----
        ok = mbar_wait(&s_full[grp], ph, ctx, 0x2502u);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
        float s[4][32];
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) tmem_ld_32x32f(t_s + cc * 32, s[cc]);
        tmem_ld_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_free[grp]);  // dP may now overwrite the scores
        // the group's shared-memory tile was last read by the previous own tile's dK and dQ-share MMAs
        ok = mbar_wait(&dkq_done[grp], ph ^ 1u, ctx, 0x2503u);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (c.i == c.kt) {  // causal mask: only the diagonal tile (an item's first) has columns beyond the row
#pragma unroll
          for (int cc = 0; cc < 4; ++cc)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (cc * 32 + i > row) s[cc][i] = -INFINITY;
        }
        if (VARLEN) {  // keys before the row's document
          const int rel = __ldg(p.kstart + static_cast<int64_t>(c.bh / p.H) * p.S + q_row) - c.kt * T;
          if (__any_sync(0xffffffffu, rel > 0)) {  // (most tiles hold no document boundary for any row of the warp)
#pragma unroll
            for (int cc = 0; cc < 4; ++cc)
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (cc * 32 + i < rel) s[cc][i] = -INFINITY;
          }
        }
        const uint64_t sc2 = pack2(p.scale_log2, p.scale_log2), nl2 = pack2(-lse, -lse);
        uint32_t pk[T / 2];
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          if (MODE == 1 && cc + 1 < 4) philox_rolled<4>(rk_s, call0 + (cc + 1) * 4, p.dr.stream_id, rw[(cc + 1) & 1]);
          p_chunk<MODE>(s[cc], pk + cc * 16, rw[cc & 1], keepw[cc], sc2, nl2, thr_hi, f_keep);
          store_row32_sw128(w_tile, row, cc * 32, s[cc]);
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&pd_ready[grp]);
        drain_dq();  // the previous own tile's dQ share: its MMA has long finished by now
        if (!ok) break;

        // ---- dS = P o (dP o keep - delta) / sqrt(d) into the same tile, once the dV MMA has read Pd ----
        ok = mbar_wait(&dp_full[grp], ph, ctx, 0x2504u);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) tmem_ld_32x32f(t_s + cc * 32, s[cc]);
        tmem_ld_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&dp_free[grp]);  // the next own tile's scores may now overwrite dP
        ok = mbar_wait(&dv_done[grp], ph, ctx, 0x2505u);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const float ksc = f_keep * p.scale;
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          ds_chunk<(MODE != 0)>(s[cc], pk + cc * 16, ksc, dsc);
          store_row32_sw128(w_tile, row, cc * 32, s[cc]);
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ds_ready[grp]);
        pend_part = static_cast<int64_t>(c.bh) * ntri + c.i * (c.i + 1) / 2 + c.kt;
        pend_g = c.g;

        if (c.last(sched)) {
          // The item ends with this tile. Its last dV MMA is already complete (dv_done was awaited before the dS phase),
          // so dV is copied out first, while the last dK MMA is still running; dK follows once acc_full says so.
          const int64_t kv_row = static_cast<int64_t>(c.kt) * T + row;
#pragma unroll
          for (int which = 0; which < 2; ++which) {
            if (which == 1) {
              ok = mbar_wait(acc_full, c.ord & 1, ctx, 0x2506u);
              ok = __all_sync(0xffffffffu, ok);
              if (!ok) break;
            }
            tc_fence_after_sync();
            const RowView& view = which == 0 ? outv.dv : outv.dk;
            __nv_bfloat16* dst = view.row(c.bh / p.H, c.bh % p.H, kv_row);
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
              float t[32];
              tmem_ld_32x32f(tmem + lane_base + (which == 0 ? kColDV : kColDK) + cc * 32, t);
              tmem_ld_wait();
#pragma unroll
              for (int c8 = 0; c8 < 4; ++c8) {
                float t8[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) t8[i] = t[c8 * 8 + i];
                Elem<__nv_bfloat16>::store_vec(dst + cc * 32 + c8 * 8, t8);
              }
            }
          }
          if (!ok) break;
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(acc_free);
        }
      }
      c.advance(sched);
    }
    if (ok) drain_dq();
  }

  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);  // let copies in flight land before shared memory is released
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace

bool attn_tc_supported(const ptj_attn_shape& sh, const void* const* ptrs, int nptrs) {
  if (sh.d_head != DH || sh.seq % T != 0 || sh.seq < T || sh.seq > (1 << 20)) return false;
  const int64_t bh = sh.batch * sh.heads, items = bh * (sh.seq / T);
  if (items * bh >= (1LL << 32)) return false;  // exactness bound of the kernels' reciprocal division by bh
  for (int i = 0; i < nptrs; ++i)
    if (!aligned16(ptrs[i])) return false;
  const int64_t* sts[4] = {sh.q_strides, sh.k_strides, sh.v_strides, sh.o_strides};
  for (const int64_t* st : sts) {
    if (st[0] % 8 != 0 || st[1] % 8 != 0 || st[2] % 8 != 0 || st[2] < DH) return false;
    if ((sh.batch > 1 && st[0] <= 0) || (sh.heads > 1 && st[1] <= 0)) return false;
  }
  return ptj_device_check() == PTJ_OK;
}

size_t attn_bwd_tc_workspace_bytes(const ptj_attn_shape& sh) {
  const int64_t nq = sh.seq / T, bh = sh.batch * sh.heads;
  const int64_t part = bh * (nq * (nq + 1) / 2) * T * DH;  // dQ shares
  const int64_t rows = bh * sh.seq;                        // delta, lse2
  return static_cast<size_t>(part + 2 * rows) * sizeof(float);
}

int attn_bwd_tc(const void* d_o, const void* q, const void* k, const void* v, const void* o, const float* row_max,
                const float* row_sum, void* dq, void* dk, void* dv, const ptj_attn_shape& sh,
                const ptj_attn_shape& dsh, const AttnDropout& dr, const uint32_t* keep_bits,
                const int32_t* row_kstart, void* workspace, size_t workspace_bytes, cudaStream_t st) {
  if (workspace == nullptr || workspace_bytes < attn_bwd_tc_workspace_bytes(sh) || !aligned16(workspace))
    return PTJ_ERR_WORKSPACE;
  CUtensorMap tq, tk, tv, tg;
  if (!make_map(&tq, q, sh, sh.q_strides) || !make_map(&tk, k, sh, sh.k_strides) ||
      !make_map(&tv, v, sh, sh.v_strides) || !make_map(&tg, d_o, sh, sh.o_strides))
    return PTJ_ERR_LAUNCH;
  AttnParams p = make_params(sh, dr);
  if (p.fault == nullptr) return PTJ_ERR_DEVICE;
  p.keep_bits = reinterpret_cast<const uint4*>(keep_bits);
  p.kstart = row_kstart;
  const bool masked = dr.train && dr.thr16 != 0u;
  const int mode = !masked ? 0 : (p.keep_bits != nullptr ? 2 : 1);
  using Kern = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap, const float*,
                        const float*, float*, const BwdViews, const AttnParams, const Sched);
  static const Kern kerns[2][3] = {
      {attn_bwd_ws_kernel<0, false>, attn_bwd_ws_kernel<1, false>, attn_bwd_ws_kernel<2, false>},
      {attn_bwd_ws_kernel<0, true>, attn_bwd_ws_kernel<1, true>, attn_bwd_ws_kernel<2, true>}};
  const Kern kern = kerns[row_kstart != nullptr ? 1 : 0][mode];
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess) {
    (void)cudaGetLastError();
    return PTJ_ERR_LAUNCH;
  }
  const int64_t rows = static_cast<int64_t>(p.BH) * p.S;
  float* part = static_cast<float*>(workspace);
  float* delta = part + static_cast<int64_t>(p.BH) * (p.nq * (p.nq + 1) / 2) * T * DH;
  float* lse2 = delta + rows;
  const RowView g_view = make_view(d_o, sh.o_strides), o_view = make_view(o, sh.o_strides);
  launch_k(attn_bwd_prep_kernel, static_cast<unsigned>((rows * 8 + 255) / 256), 256, 0, st, g_view, o_view, row_max, row_sum,
                                                                                     delta, lse2, p.S, p.H, rows);
  PTJ_CHECK_LAUNCH();
  Sched s;
  s.nq = p.nq;
  s.BH = p.BH;
  s.total = p.nq * p.BH;
  const int grid = s.total < kNumSMs ? s.total : kNumSMs;
  s.rounds = (s.total + grid - 1) / grid;
  s.bh_magic = static_cast<uint32_t>(((1ull << 32) + s.BH - 1) / s.BH);
  BwdViews views{make_view(dk, dsh.k_strides), make_view(dv, dsh.v_strides)};
  launch_k(kern, grid, kThreads, kSmemBytes, st, tq, tk, tv, tg, delta, lse2, part, views, p, s);
  PTJ_CHECK_LAUNCH();
  const int64_t total_vec = rows * (DH / 4);
  launch_k(attn_dq_reduce_kernel, static_cast<unsigned>((total_vec + 255) / 256), 256, 0, st, part, make_view(dq, dsh.q_strides),
                                                                                        row_kstart, p.S, p.H, p.nq, total_vec);
  PTJ_CHECK_LAUNCH();
  return PTJ_OK;
}

}  // namespace ptj
