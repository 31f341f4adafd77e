// GEMM for the training path.
//
// bf16 inputs: persistent, warp-specialised tcgen05 kernel. One warp issues TMA tensor copies into a ring of
// 128-byte-swizzled shared-memory stages, one thread issues tcgen05.mma (128 x BN x 16 per instruction, fp32
// accumulators in tensor memory, two accumulator buffers), eight warps drain finished accumulators with tcgen05.ld
// and run the elementwise epilogue while the next tile is already being multiplied. Either operand may be K-major
// or MN-major, which covers forward (x W^T), input-gradient (dy W) and weight-gradient (dy^T x) products without
// any transposed copy. Work items = output tiles x K splits, walked by a static persistent schedule.
//
// fp32 inputs: plain shared-memory tiled FMA kernel (exact fp32, any shape) for the fp32 parity path.
#include <atomic>

#include "common.cuh"
#include "gemm_epilogue.cuh"
#include "tc_common.cuh"
#include "tc_runtime.h"

namespace ptj {
namespace {

using namespace tc;

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kEpilogueWarps = 8;     // a multiple of 4: warp w may only read tensor-memory lanes 32*(w%4)..
constexpr int kWarpsPerQuarter = kEpilogueWarps / 4;   // these warps share a lane quarter and take its 32-column chunks in turn
constexpr int kFirstEpilogueWarp = 4;  // warps 0-3 form one warp group: warp 0 TMA, warp 1 MMA + TMEM owner, 2-3 idle
constexpr int kGemmThreads = 32 * (kFirstEpilogueWarp + kEpilogueWarps);
// Registers are re-split between the warp groups (setmaxnreg works on whole groups of four warps): the copy / MMA group
// keeps 40 per thread, the two epilogue groups get 232. A block of 10 warps is allocated like 12 and held to 168
// registers per thread, where the epilogue spilled a few values; with all but a sliver of the SM's L1 configured as
// shared memory a spill is a round trip to L2 under the load of the operand copies, in the one part of the kernel that
// has to keep up with the tensor pipe.
constexpr int kRegsIssue = 40, kRegsEpilogue = 232;  // warp 0: TMA, warp 1: MMA + TMEM owner, the rest: epilogue
constexpr int kSmemLimit = 227 * 1024;
static_assert(kStripBytes % 512 == 0, "tile stores with the 64-byte swizzle need 512-byte aligned strips");
constexpr int chunks_per_warp(int bn) { return (bn / 32 + kWarpsPerQuarter - 1) / kWarpsPerQuarter; }

template <int BN>
struct GemmCfg {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kBiasBytes = kEpilogueWarps * chunks_per_warp(BN) * 128;  // each epilogue warp's bias slices
  static constexpr int fixed_bytes(int strip) { return kEpilogueWarps * strip + kBiasBytes + 1024 + kBarrierBytes; }
  static constexpr int stages(int strip) {
    const int fit = (kSmemLimit - fixed_bytes(strip)) / kStageBytes;
    return fit < 6 ? fit : 6;
  }
  static constexpr int smem_bytes(int strip) { return stages(strip) * kStageBytes + fixed_bytes(strip); }
  static constexpr int kTmemCols = 512;     // two accumulator buffers, the second at column 256
  static constexpr int kAccStride = 256;
};

struct GemmParams {
  EpilogueParams ep;
  int64_t M, N, K;
  int num_m, num_n, num_kb, split_k;
  float* workspace;  // [split_k, M, N] partial sums when split_k > 1
  int out_bf16;
  int tma_store;  // outputs leave through tensor-map tile stores (bf16 output, 16-byte aligned rows, K not split)
  int tma_side;   // ... and the epilogue's side input arrives through tile loads, one block ahead
  unsigned int* fault;
};

// Tensor maps of the outputs (C and, for the GELU epilogue, the saved pre-activation): boxes of 32 rows x 32 bf16,
// 64-byte swizzle.
struct alignas(64) StoreMaps {
  CUtensorMap c, x;
  CUtensorMap s;  // the epilogue's side input (residual / saved pre-activation), same boxes
};

constexpr int kEpiBlockBytes = 2048;  // one 32 x 32 bf16 block

// The side input of a warp's blocks arrives through tile loads issued one block ahead into a landing buffer behind the
// warp's store strip, so that its latency hides under the previous block's arithmetic and the accumulator wait.
struct SidePrefetch {
  uint8_t* buf;    // kEpiBlockBytes, 512-byte aligned; nullptr: side inputs are read with plain loads
  uint64_t* bar;   // completes when a block has landed
  uint32_t waits;  // blocks waited for so far (the barrier's parity)
};

// Lane 0 requests the side-input block at (row0, n0). All lanes call.
__device__ __forceinline__ void side_prefetch_issue(const SidePrefetch& sp, const CUtensorMap* map, int64_t row0,
                                                    int64_t n0, int lane) {
  if (lane == 0) {
    mbar_expect_tx(sp.bar, kEpiBlockBytes);
    tma_load_2d(sp.buf, map, sp.bar, static_cast<int>(n0), static_cast<int>(row0));
  }
}

// One 32 x 32 bf16 block, one row per lane, leaves through the tensor map: rows are parked densely (64 bytes each) in
// the warp's strip (swizzled) and ONE lane issues an asynchronous tile store, so no warp waits on the memory system. The strip
// may only be rewritten after bulk_wait_read_all() by that lane. All lanes must call.
__device__ __forceinline__ void warp_store_block_tma(uint8_t* strip, const CUtensorMap* map, int64_t row0, int64_t n0,
                                                     const float (&v)[32], int lane) {
  // 64-byte swizzle of the tensor map: the 16-byte piece q of row r lies at piece q ^ ((r >> 1) & 3), which also makes
  // the eight lanes of a store phase hit eight different bank groups (the strip starts on a 512-byte boundary)
  uint8_t* mine = strip + lane * 64;
  const int sw = (lane >> 1) & 3;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(v[q * 8 + 2 * i], v[q * 8 + 2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(mine + ((q ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
  }
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0) {
    tma_store_2d(map, strip, static_cast<int>(n0), static_cast<int>(row0));
    bulk_commit_group();
  }
}

// Epilogue of one 32-row x 32-column block of an accumulator tile (one row per lane): arithmetic per thread, stores
// through the warp's staging strip when the block is full and rows are 16-byte aligned, else per thread.
template <typename TOut, bool SIDE>
__device__ __forceinline__ void tile_epilogue(const EpilogueParams& ep, uint8_t* strip, int64_t row0, int64_t row,
                                              int64_t n0, float (&acc)[32], int lane, const float* bias_s,
                                              const StoreMaps* maps, SidePrefetch& sp, const AbortCtx& ctx,
                                              int64_t next_n0, bool& ok, uint64_t seed) {
  // (warp-uniform) only full-width blocks: at a ragged right edge the tile store was seen to write the whole 16-byte
  // piece that holds the last valid column, i.e. up to seven padding columns
  const bool use_tma = maps != nullptr && sizeof(TOut) == 2 && row0 < ep.M && n0 + 32 <= ep.N;
  if (maps != nullptr) {
    // the previous block's tile store must have read the strip before anything overwrites it
    if (lane == 0) bulk_wait_read_all();
    __syncwarp();
  }
  const bool inside = epilogue_pre<TOut, 32>(ep, row, n0, acc, bias_s);
  TOut* c = static_cast<TOut*>(ep.c);
  TOut* aux_out = static_cast<TOut*>(ep.aux_out);
  const bool want_pre = ep.mode == PTJ_EPI_GELU && aux_out != nullptr;
  const bool staged = ep.vec_ok && n0 + 32 <= ep.N;  // warp-uniform
  if (want_pre && use_tma) {
    warp_store_block_tma(strip, &maps->x, row0, n0, acc, lane);
  } else if (want_pre) {
    if (staged) warp_store_block<TOut>(strip, aux_out, ep.ldc, row0, n0, ep.M, acc, lane);
    else if (inside) store_row<TOut, 32>(aux_out + row * ep.ldc, n0, ep.N, false, acc);
  }
  float side[32];
  if (SIDE) {
    // (warp-uniform) a block inside the matrix was requested one block ago (or at the start of the tile)
    if (row0 < ep.M && n0 < ep.N) {
      ok = __all_sync(0xffffffffu, mbar_wait(sp.bar, sp.waits & 1u, ctx, 0x0302u));
      if (!ok) return;
      ++sp.waits;
#pragma unroll
      for (int q = 0; q < 4; ++q) {  // this lane's row, stored with the tensor map's 64-byte swizzle
        const uint4 t = *reinterpret_cast<const uint4*>(sp.buf + lane * 64 + ((q ^ ((lane >> 1) & 3)) << 4));
        const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          side[q * 8 + 2 * i] = __uint_as_float(w[i] << 16);
          side[q * 8 + 2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
      }
      __syncwarp();
      if (next_n0 >= 0 && next_n0 < ep.N) side_prefetch_issue(sp, &maps->s, row0, next_n0, lane);
    }
  } else if (const void* sptr = epilogue_side_input(ep)) {
    if (staged) warp_load_block<TOut>(strip, static_cast<const TOut*>(sptr), ep.ldc, row0, n0, ep.M, side, lane);
    else if (inside) load_row<TOut, 32>(static_cast<const TOut*>(sptr) + row * ep.ldc, n0, ep.N, false, side);
  }
  if (inside) epilogue_post<TOut, 32>(ep, row, n0, acc, side, seed);
  if (use_tma) {
    if (want_pre) {
      if (lane == 0) bulk_wait_read_all();
      __syncwarp();
    }
    warp_store_block_tma(strip, &maps->c, row0, n0, acc, lane);
    return;
  }
  if (staged) warp_store_block<TOut>(strip, c, ep.ldc, row0, n0, ep.M, acc, lane);
  else if (inside) store_row<TOut, 32>(c + row * ep.ldc, n0, ep.N, false, acc);
}

template <int BN, bool A_KMAJOR, bool B_KMAJOR, bool SIDE>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ StoreMaps smaps, const GemmParams p) {
  using Cfg = GemmCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  // SIDE: the epilogue's side input arrives through tile loads, which takes a landing buffer per epilogue warp behind
  // its store strip (and, for the widest tiles, a stage of the operand ring)
  constexpr int kStrip = SIDE ? 2 * kEpiBlockBytes : kStripBytes;
  constexpr int nst = Cfg::stages(kStrip);
  uint8_t* strips = smem + nst * Cfg::kStageBytes;
  float* bias_smem = reinterpret_cast<float*>(strips + kEpilogueWarps * kStrip);
  uint64_t* bars = reinterpret_cast<uint64_t*>(strips + kEpilogueWarps * kStrip + Cfg::kBiasBytes);
  uint64_t* side_bars = bars + 24;  // one per epilogue warp
  uint64_t* full = bars;
  uint64_t* empty = bars + nst;
  uint64_t* tmem_full = bars + 2 * nst;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const AbortCtx ctx{abort_flag, p.fault};

  if (threadIdx.x == 0) {
    for (int s = 0; s < nst; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int w = 0; w < kEpilogueWarps; ++w) mbar_init(&side_bars[w], 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], kEpilogueWarps);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
    if (SIDE) prefetch_tensormap(&smaps.s);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  grid_dep_sync();  // set-up above touches no global memory; everything below may
  const uint32_t tmem_base = *tmem_slot;

  const int tiles = p.num_m * p.num_n;
  const int total = tiles * p.split_k;
  if (warp < kFirstEpilogueWarp) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsIssue));

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total && ok; item += gridDim.x) {
        const int split = item / tiles, tile = item - split * tiles;
        const int m_blk = tile % p.num_m, n_blk = tile / p.num_m;
        int kb0 = 0, kb1 = p.num_kb;  // (64-bit divisions only when K is split)
        if (p.split_k > 1) {
          kb0 = static_cast<int>(static_cast<int64_t>(split) * p.num_kb / p.split_k);
          kb1 = static_cast<int>(static_cast<int64_t>(split + 1) * p.num_kb / p.split_k);
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, ctx, 0x0101u)) { ok = false; break; }
          mbar_expect_tx(&full[stage], Cfg::kStageBytes);
          uint8_t* sa = smem + stage * Cfg::kStageBytes;
          uint8_t* sb = sa + Cfg::kABytes;
          if (A_KMAJOR) {
            tma_load_2d(sa, &tmap_a, &full[stage], kb * BK, m_blk * BM);
          } else {
#pragma unroll
            for (int h = 0; h < BM / 64; ++h)
              tma_load_2d(sa + h * 8192, &tmap_a, &full[stage], m_blk * BM + h * 64, kb * BK);
          }
          if (B_KMAJOR) {
            tma_load_2d(sb, &tmap_b, &full[stage], kb * BK, n_blk * BN);
          } else {
#pragma unroll
            for (int h = 0; h < BN / 64; ++h)
              tma_load_2d(sb + h * 8192, &tmap_b, &full[stage], n_blk * BN + h * 64, kb * BK);
          }
          if (++stage == nst) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_bf16_f32(BM, BN, !A_KMAJOR, !B_KMAJOR);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total && ok; item += gridDim.x, ++it) {
        const int split = item / tiles;
        int kb0 = 0, kb1 = p.num_kb;  // (64-bit divisions only when K is split)
        if (p.split_k > 1) {
          kb0 = static_cast<int>(static_cast<int64_t>(split) * p.num_kb / p.split_k);
          kb1 = static_cast<int>(static_cast<int64_t>(split + 1) * p.num_kb / p.split_k);
        }
        const int buf = it & 1;
        const uint32_t aphase = (it >> 1) & 1u;
        if (!mbar_wait(&tmem_empty[buf], aphase ^ 1u, ctx, 0x0201u)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * Cfg::kAccStride);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full[stage], phase, ctx, 0x0202u)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint32_t sb = sa + Cfg::kABytes;
#pragma unroll
          for (int k4 = 0; k4 < BK / 16; ++k4) {
            const uint64_t adesc = A_KMAJOR ? smem_desc_sw128(sa + k4 * 32, 16, 1024)
                                            : smem_desc_sw128(sa + k4 * 2048, 8192, 1024);
            const uint64_t bdesc = B_KMAJOR ? smem_desc_sw128(sb + k4 * 32, 16, 1024)
                                            : smem_desc_sw128(sb + k4 * 2048, 8192, 1024);
            mma_bf16_ss(d_tmem, adesc, bdesc, idesc, (kb > kb0 || k4 > 0) ? 1u : 0u);
          }
          mma_commit(&empty[stage]);  // the stage is free once these MMAs have read it
          if (++stage == nst) { stage = 0; phase ^= 1u; }
        }
        if (ok) mma_commit(&tmem_full[buf]);
      }
    }
  } else if (warp >= kFirstEpilogueWarp) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsEpilogue));
    const int quarter = warp & 3;  // tensor-memory lanes [32*quarter, 32*quarter+32) belong to this warp
    const int sub = (warp - kFirstEpilogueWarp) >> 2;   // position among the warps that share this lane quarter
    constexpr int kChunks = chunks_per_warp(BN);  // this warp takes chunks sub, sub + kWarpsPerQuarter, ...
    int it = 0;
    bool ok = true;
    const uint64_t seed = p.ep.mode == PTJ_EPI_DROPOUT_RESID ? resolve_seed(p.ep.seed) : 0ull;
    SidePrefetch sp{SIDE ? strips + (warp - kFirstEpilogueWarp) * kStrip + kEpiBlockBytes : nullptr, &side_bars[warp - kFirstEpilogueWarp], 0u};
    for (int item = blockIdx.x; item < total && ok; item += gridDim.x, ++it) {
      const int split = item / tiles, tile = item - split * tiles;
      const int m_blk = tile % p.num_m, n_blk = tile / p.num_m;
      const int buf = it & 1;
      const uint32_t aphase = (it >> 1) & 1u;
      float* wbias = bias_smem + (warp - kFirstEpilogueWarp) * (kChunks * 32);
      const bool bias_staged = p.ep.bias != nullptr && p.split_k == 1;
      if (bias_staged) {
        // this warp's slice of the tile's bias, fetched while the tile is still being multiplied
        __syncwarp();
#pragma unroll
        for (int j = 0; j < kChunks; ++j) {
          const int64_t n = static_cast<int64_t>(n_blk) * BN + (sub + j * kWarpsPerQuarter) * 32 + lane;
          wbias[j * 32 + lane] = n < p.N ? __ldg(p.ep.bias + n) : 0.f;
        }
        __syncwarp();
      }
      const int64_t row0 = static_cast<int64_t>(m_blk) * BM + quarter * 32;
      const int64_t row = row0 + lane;
      if (SIDE) {
        // the side input of this warp's first block of the tile, requested before the accumulator is even complete
        const int64_t nf = static_cast<int64_t>(n_blk) * BN + sub * 32;
        if (row0 < p.M && nf < p.N) side_prefetch_issue(sp, &smaps.s, row0, nf, lane);
      }
      ok = mbar_wait(&tmem_full[buf], aphase, ctx, 0x0301u);
      ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld below needs the whole warp
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                             static_cast<uint32_t>(buf * Cfg::kAccStride);
#pragma unroll 1
      for (int chunk = 0; chunk < kChunks; ++chunk) {
        const int col = (sub + chunk * kWarpsPerQuarter) * 32;  // first column of this chunk within the tile
        if (col >= BN) break;
        uint32_t r[32];
        tmem_ld_32x32(taddr + col, r);
        tmem_ld_wait();
        float acc[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = __uint_as_float(r[j]);
        const int64_t n0 = static_cast<int64_t>(n_blk) * BN + col;
        uint8_t* strip = strips + (warp - kFirstEpilogueWarp) * kStrip;
        const float* bias_c = bias_staged ? wbias + chunk * 32 : nullptr;
        if (p.split_k > 1) {
          float* w = p.workspace + static_cast<int64_t>(split) * p.M * p.N;
          if ((p.N & 3) == 0 && n0 + 32 <= p.N) {
            warp_store_block<float>(strip, w, p.N, row0, n0, p.M, acc, lane);
          } else if (row < p.M) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (n0 + j < p.N) w[row * p.N + n0 + j] = acc[j];
          }
        } else if (p.out_bf16) {
          const int ncol = (sub + (chunk + 1) * kWarpsPerQuarter) * 32;  // this warp's next block of the tile, if any
          const int64_t next_n0 = ncol < BN ? static_cast<int64_t>(n_blk) * BN + ncol : -1;
          tile_epilogue<__nv_bfloat16, SIDE>(p.ep, strip, row0, row, n0, acc, lane, bias_c,
                                             p.tma_store ? &smaps : nullptr, sp, ctx, next_n0, ok, seed);
          if (!ok) break;
        } else {
          tile_epilogue<float, false>(p.ep, strip, row0, row, n0, acc, lane, bias_c, nullptr, sp, ctx, -1, ok, seed);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[buf]);
    }
    if (lane == 0) bulk_wait_all();  // this lane's tile stores are complete before the block may exit
  }

  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    // give copies still in flight time to land before shared memory is handed back
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// ---- CTA-pair kernel -------------------------------------------------------------------------------------------
// Two CTAs of a cluster (two neighbouring SMs) share one 256 x BN output tile through tcgen05.mma.cta_group::2:
// CTA r of the pair loads A rows [r*128, r*128+128) and B rows [r*BN/2, (r+1)*BN/2) of the tile into its own
// shared memory and keeps rows r*128.. of the accumulator in its own tensor memory; one thread of the leader (rank 0)
// issues the MMAs for both. Per CTA and 16-deep K step that is 8 KB of TMA writes + 8 KB of operand reads instead
// of 12 + 12 in the single-CTA kernel, which is what the shared-memory port can sustain at full tensor rate.
// Signals: both CTAs' TMA loads complete on the LEADER's full barrier; tcgen05.commit multicasts the "stage free"
// and "accumulator ready" arrivals to both CTAs; the peer's epilogue warps arrive remotely on the leader's
// "accumulator drained" barrier. No TMA multicast is used anywhere.
template <int BN>
struct PairCfg {
  static constexpr int kABytes = BM * BK * 2;        // per CTA: 128 rows of A
  static constexpr int kBBytes = (BN / 2) * BK * 2;  // per CTA: half of the tile's B rows
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kBiasBytes = kEpilogueWarps * chunks_per_warp(BN) * 128;  // each epilogue warp's bias slices
  static constexpr int fixed_bytes(int strip) { return kEpilogueWarps * strip + kBiasBytes + 1024 + kBarrierBytes; }
  static constexpr int stages(int strip) {
    const int fit = (kSmemLimit - fixed_bytes(strip)) / kStageBytes;
    return fit < 6 ? fit : 6;
  }
  static constexpr int smem_bytes(int strip) { return stages(strip) * kStageBytes + fixed_bytes(strip); }
  static constexpr int kTmemCols = 512;
  static constexpr int kAccStride = 256;
};

// GROUPED: the launch carries a second product (its own operand maps and parameters; same K-block size, operand layouts
// and template arguments): work items [0, items1) belong to the first product, the rest to the second, dealt to the
// pairs as one list. Two products that would each occupy half of the pairs then run side by side in one round.
template <int BN, bool A_KMAJOR, bool B_KMAJOR, bool SIDE, bool GROUPED = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ StoreMaps smaps, const __grid_constant__ GemmParams p,
                    const __grid_constant__ CUtensorMap tmap_a2, const __grid_constant__ CUtensorMap tmap_b2,
                    const __grid_constant__ GemmParams p2, const int items1) {
  using Cfg = PairCfg<BN>;
  constexpr int HB = BN / 2;  // B rows held by one CTA
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  // SIDE: the epilogue's side input arrives through tile loads, which takes a landing buffer per epilogue warp behind
  // its store strip (and, for the widest tiles, a stage of the operand ring)
  constexpr int kStrip = SIDE ? 2 * kEpiBlockBytes : kStripBytes;
  constexpr int nst = Cfg::stages(kStrip);
  uint8_t* strips = smem + nst * Cfg::kStageBytes;
  float* bias_smem = reinterpret_cast<float*>(strips + kEpilogueWarps * kStrip);
  uint64_t* bars = reinterpret_cast<uint64_t*>(strips + kEpilogueWarps * kStrip + Cfg::kBiasBytes);
  uint64_t* side_bars = bars + 24;  // one per epilogue warp
  uint64_t* full = bars;                      // used in the leader only
  uint64_t* empty = bars + nst;      // one set per CTA, both signalled by the leader's commits
  uint64_t* tmem_full = bars + 2 * nst;
  uint64_t* tmem_empty = tmem_full + 2;       // used in the leader only: 8 local + 8 remote epilogue warps
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const AbortCtx ctx{abort_flag, p.fault};

  if (threadIdx.x == 0) {
    for (int s = 0; s < nst; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int w = 0; w < kEpilogueWarps; ++w) mbar_init(&side_bars[w], 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 2 * kEpilogueWarps);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
    if (GROUPED) {
      prefetch_tensormap(&tmap_a2);
      prefetch_tensormap(&tmap_b2);
    }
    if (SIDE) prefetch_tensormap(&smaps.s);
  }
  __syncthreads();
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before anyone signals across the pair
  tc_fence_after_sync();
  grid_dep_sync();  // set-up above touches no global memory; everything below may
  const uint32_t tmem_base = *tmem_slot;

  // (num_m counts 256-row tiles here)
  const int total = GROUPED ? items1 + p2.num_m * p2.num_n * p2.split_k : items1;
  const int pair = static_cast<int>(blockIdx.x) >> 1, npairs = static_cast<int>(gridDim.x) >> 1;
  if (warp < kFirstEpilogueWarp) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsIssue));

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = pair; item < total && ok; item += npairs) {
        const bool second = GROUPED && item >= items1;
        const GemmParams& q = second ? p2 : p;
        const CUtensorMap* map_a = second ? &tmap_a2 : &tmap_a;
        const CUtensorMap* map_b = second ? &tmap_b2 : &tmap_b;
        const int li = second ? item - items1 : item;
        const int tiles = q.num_m * q.num_n;
        const int split = li / tiles, tile = li - split * tiles;
        const int m_blk = tile % q.num_m, n_blk = tile / q.num_m;
        int kb0 = 0, kb1 = q.num_kb;  // (64-bit divisions only when K is split)
        if (q.split_k > 1) {
          kb0 = static_cast<int>(static_cast<int64_t>(split) * q.num_kb / q.split_k);
          kb1 = static_cast<int>(static_cast<int64_t>(split + 1) * q.num_kb / q.split_k);
        }
        const int m0 = m_blk * 2 * BM + static_cast<int>(rank) * BM;
        const int n0 = n_blk * BN + static_cast<int>(rank) * HB;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, ctx, 0x0401u)) { ok = false; break; }
          const uint32_t leader_full = mapa_shared(smem_u32(&full[stage]), 0);
          if (rank == 0) mbar_expect_tx(&full[stage], 2 * Cfg::kStageBytes);  // both CTAs' bytes land here
          uint8_t* sa = smem + stage * Cfg::kStageBytes;
          uint8_t* sb = sa + Cfg::kABytes;
          if (A_KMAJOR) {
            tma_load_2d_pair(sa, map_a, leader_full, kb * BK, m0);
          } else {
#pragma unroll
            for (int h = 0; h < BM / 64; ++h) tma_load_2d_pair(sa + h * 8192, map_a, leader_full, m0 + h * 64, kb * BK);
          }
          if (B_KMAJOR) {
            tma_load_2d_pair(sb, map_b, leader_full, kb * BK, n0);
          } else {
#pragma unroll
            for (int h = 0; h < HB / 64; ++h) tma_load_2d_pair(sb + h * 8192, map_b, leader_full, n0 + h * 64, kb * BK);
          }
          if (++stage == nst) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = idesc_bf16_f32(2 * BM, BN, !A_KMAJOR, !B_KMAJOR);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int item = pair; item < total && ok; item += npairs, ++it) {
        const bool second = GROUPED && item >= items1;
        const GemmParams& q = second ? p2 : p;
        const int split = (second ? item - items1 : item) / (q.num_m * q.num_n);
        int kb0 = 0, kb1 = q.num_kb;  // (64-bit divisions only when K is split)
        if (q.split_k > 1) {
          kb0 = static_cast<int>(static_cast<int64_t>(split) * q.num_kb / q.split_k);
          kb1 = static_cast<int>(static_cast<int64_t>(split + 1) * q.num_kb / q.split_k);
        }
        const int buf = it & 1;
        const uint32_t aphase = (it >> 1) & 1u;
        if (!mbar_wait_cluster(&tmem_empty[buf], aphase ^ 1u, ctx, 0x0501u)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * Cfg::kAccStride);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_cluster(&full[stage], phase, ctx, 0x0502u)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint32_t sb = sa + Cfg::kABytes;
#pragma unroll
          for (int k4 = 0; k4 < BK / 16; ++k4) {
            const uint64_t adesc = A_KMAJOR ? smem_desc_sw128(sa + k4 * 32, 16, 1024)
                                            : smem_desc_sw128(sa + k4 * 2048, 8192, 1024);
            const uint64_t bdesc = B_KMAJOR ? smem_desc_sw128(sb + k4 * 32, 16, 1024)
                                            : smem_desc_sw128(sb + k4 * 2048, 8192, 1024);
            mma_bf16_ss_pair(d_tmem, adesc, bdesc, idesc, (kb > kb0 || k4 > 0) ? 1u : 0u);
          }
          mma_commit_pair(&empty[stage], 3);  // stage free in both CTAs once these MMAs have read it
          if (++stage == nst) { stage = 0; phase ^= 1u; }
        }
        if (ok) mma_commit_pair(&tmem_full[buf], 3);
      }
    }
  } else if (warp >= kFirstEpilogueWarp) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsEpilogue));
    const int quarter = warp & 3;
    const int sub = (warp - kFirstEpilogueWarp) >> 2;
    constexpr int kChunks = chunks_per_warp(BN);
    const uint32_t leader_empty0 = mapa_shared(smem_u32(&tmem_empty[0]), 0);
    const uint32_t leader_empty1 = mapa_shared(smem_u32(&tmem_empty[1]), 0);
    int it = 0;
    bool ok = true;
    const uint64_t seed = p.ep.mode == PTJ_EPI_DROPOUT_RESID ? resolve_seed(p.ep.seed) : 0ull;
    SidePrefetch sp{SIDE ? strips + (warp - kFirstEpilogueWarp) * kStrip + kEpiBlockBytes : nullptr, &side_bars[warp - kFirstEpilogueWarp], 0u};
    for (int item = pair; item < total && ok; item += npairs, ++it) {
      const bool second = GROUPED && item >= items1;
      const GemmParams& q = second ? p2 : p;
      const int li = second ? item - items1 : item;
      const int tiles = q.num_m * q.num_n;
      const int split = li / tiles, tile = li - split * tiles;
      const int m_blk = tile % q.num_m, n_blk = tile / q.num_m;
      const int buf = it & 1;
      const uint32_t aphase = (it >> 1) & 1u;
      float* wbias = bias_smem + (warp - kFirstEpilogueWarp) * (kChunks * 32);
      const bool bias_staged = q.ep.bias != nullptr && q.split_k == 1;
      if (bias_staged) {
        // this warp's slice of the tile's bias, fetched while the tile is still being multiplied
        __syncwarp();
#pragma unroll
        for (int j = 0; j < kChunks; ++j) {
          const int64_t n = static_cast<int64_t>(n_blk) * BN + (sub + j * kWarpsPerQuarter) * 32 + lane;
          wbias[j * 32 + lane] = n < q.N ? __ldg(q.ep.bias + n) : 0.f;
        }
        __syncwarp();
      }
      const int64_t row0 = static_cast<int64_t>(m_blk) * 2 * BM + static_cast<int64_t>(rank) * BM + quarter * 32;
      const int64_t row = row0 + lane;
      if (SIDE && (!GROUPED || q.tma_side)) {
        // the side input of this warp's first block of the tile, requested before the accumulator is even complete
        // (a second product that is split over K leaves its epilogue to the finishing kernel: nothing to fetch)
        const int64_t nf = static_cast<int64_t>(n_blk) * BN + sub * 32;
        if (row0 < q.M && nf < q.N) side_prefetch_issue(sp, &smaps.s, row0, nf, lane);
      }
      ok = mbar_wait(&tmem_full[buf], aphase, ctx, 0x0601u);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                             static_cast<uint32_t>(buf * Cfg::kAccStride);
#pragma unroll 1
      for (int chunk = 0; chunk < kChunks; ++chunk) {
        const int col = (sub + chunk * kWarpsPerQuarter) * 32;  // first column of this chunk within the tile
        if (col >= BN) break;
        uint32_t r[32];
        tmem_ld_32x32(taddr + col, r);
        tmem_ld_wait();
        float acc[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] = __uint_as_float(r[j]);
        const int64_t n0 = static_cast<int64_t>(n_blk) * BN + col;
        uint8_t* strip = strips + (warp - kFirstEpilogueWarp) * kStrip;
        const float* bias_c = bias_staged ? wbias + chunk * 32 : nullptr;
        if (q.split_k > 1) {
          float* w = q.workspace + static_cast<int64_t>(split) * q.M * q.N;
          if ((q.N & 3) == 0 && n0 + 32 <= q.N) {
            warp_store_block<float>(strip, w, q.N, row0, n0, q.M, acc, lane);
          } else if (row < q.M) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (n0 + j < q.N) w[row * q.N + n0 + j] = acc[j];
          }
        } else if (q.out_bf16) {
          const int ncol = (sub + (chunk + 1) * kWarpsPerQuarter) * 32;  // this warp's next block of the tile, if any
          const int64_t next_n0 = ncol < BN ? static_cast<int64_t>(n_blk) * BN + ncol : -1;
          tile_epilogue<__nv_bfloat16, SIDE>(q.ep, strip, row0, row, n0, acc, lane, bias_c,
                                             q.tma_store ? &smaps : nullptr, sp, ctx, next_n0, ok, seed);
          if (!ok) break;
        } else {
          tile_epilogue<float, false>(q.ep, strip, row0, row, n0, acc, lane, bias_c, nullptr, sp, ctx, -1, ok, seed);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(buf == 0 ? leader_empty0 : leader_empty1);
    }
    if (lane == 0) bulk_wait_all();  // this lane's tile stores are complete before the block may exit
  }

  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  cluster_sync_all();  // neither CTA leaves (or frees tensor memory) while its peer may still signal it
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
  }
}

// c[m, n] = (accumulate ? c : 0) + bias[n] + sum_s ws[s, m, n]; four columns per thread (N % 4 == 0) or one.
template <typename TOut, int W>
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ ws, TOut* __restrict__ c, const float* __restrict__ bias, int64_t M,
                     int64_t N, int64_t ldc, int split_k, int accumulate) {
  grid_dep_sync();
  const int64_t total = M * N;
  for (int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * W; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x * W) {
    const int64_t m = i / N, n = i - m * N;
    float s[W];
#pragma unroll
    for (int j = 0; j < W; ++j) s[j] = 0.f;
    for (int k = 0; k < split_k; ++k) {
      const float* src = ws + static_cast<int64_t>(k) * total + i;
      if (W == 4) {
        const float4 v = *reinterpret_cast<const float4*>(src);
        s[0] += v.x; s[1] += v.y; s[2] += v.z; s[3] += v.w;
      } else {
        s[0] += *src;
      }
    }
    TOut* dst = c + m * ldc + n;
#pragma unroll
    for (int j = 0; j < W; ++j) {
      if (bias != nullptr) s[j] += bias[n + j];
      if (accumulate) s[j] += Elem<TOut>::load(dst + j);
      Elem<TOut>::store(dst + j, s[j]);
    }
  }
}

// ---- exact fp32 kernel -----------------------------------------------------------------------------------------
constexpr int SM_BM = 64, SM_BN = 64, SM_BK = 16;
template <typename TOut>
__global__ void __launch_bounds__(128)
gemm_simt_kernel(const float* __restrict__ A, const float* __restrict__ B, int64_t sam, int64_t sak, int64_t sbn,
                 int64_t sbk, int64_t M, int64_t N, int64_t K, const EpilogueParams ep) {
  grid_dep_sync();
  __shared__ float As[SM_BK][SM_BM + 4];
  __shared__ float Bs[SM_BK][SM_BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 7, ty = tid >> 3;  // 8 column groups of 8, 16 row groups of 4
  const int64_t m0 = static_cast<int64_t>(blockIdx.y) * SM_BM, n0 = static_cast<int64_t>(blockIdx.x) * SM_BN;
  float acc[4][8];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
  for (int64_t k0 = 0; k0 < K; k0 += SM_BK) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int idx = tid + i * 128;
      int mm, kk;
      if (sak == 1) { mm = idx / SM_BK; kk = idx % SM_BK; } else { kk = idx / SM_BM; mm = idx % SM_BM; }
      const int64_t gm = m0 + mm, gk = k0 + kk;
      As[kk][mm] = (gm < M && gk < K) ? A[gm * sam + gk * sak] : 0.f;
      int nn, kb;
      if (sbk == 1) { nn = idx / SM_BK; kb = idx % SM_BK; } else { kb = idx / SM_BN; nn = idx % SM_BN; }
      const int64_t gn = n0 + nn, gkb = k0 + kb;
      Bs[kb][nn] = (gn < N && gkb < K) ? B[gn * sbn + gkb * sbk] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < SM_BK; ++kk) {
      float a[4], b[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 8; ++j) b[j] = Bs[kk][tx * 8 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  const uint64_t seed = ep.mode == PTJ_EPI_DROPOUT_RESID ? resolve_seed(ep.seed) : 0ull;
#pragma unroll
  for (int i = 0; i < 4; ++i) epilogue_row_segment<TOut, 8>(ep, m0 + ty * 4 + i, n0 + tx * 8, acc[i], seed);
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) is needed once per kernel instantiation and device, not per launch.
template <typename Kern>
bool ensure_max_smem(Kern kern, std::atomic<uint64_t>& done) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    (void)cudaGetLastError();
    return false;
  }
  const uint64_t bit = 1ull << dev;
  if (done.load(std::memory_order_acquire) & bit) return true;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  done.fetch_or(bit, std::memory_order_release);
  return true;
}

template <int BN, bool AK, bool BK_, bool SIDE>
int launch_tc(const CUtensorMap& ta, const CUtensorMap& tb, const StoreMaps& sm, const GemmParams& p, cudaStream_t st) {
  using Cfg = GemmCfg<BN>;
  // per epilogue warp: the store strip, plus a landing buffer when side inputs arrive through tile loads
  const int smem_bytes = Cfg::smem_bytes(SIDE ? 2 * kEpiBlockBytes : kStripBytes);
  auto kern = gemm_tc_kernel<BN, AK, BK_, SIDE>;
  static std::atomic<uint64_t> attr_done{0};
  if (!ensure_max_smem(kern, attr_done)) return PTJ_ERR_LAUNCH;
  const int total = p.num_m * p.num_n * p.split_k;
  const int grid = total < kNumSMs ? total : kNumSMs;
  launch_k(kern, grid, kGemmThreads, smem_bytes, st, ta, tb, sm, p);
  PTJ_CHECK_LAUNCH();
  return PTJ_OK;
}

// Sum of the K-split partial tiles (fixed order) followed by the FULL epilogue of the product: one thread per row and
// group of eight columns. Used for the row range that a product's mostly-empty last round of tiles is turned into.
template <typename TOut>
__global__ void __launch_bounds__(256)
splitk_finish_kernel(const float* __restrict__ ws, const EpilogueParams ep, int split_k) {
  grid_dep_sync();
  const uint64_t seed = ep.mode == PTJ_EPI_DROPOUT_RESID ? resolve_seed(ep.seed) : 0ull;
  const int64_t groups = (ep.N + 7) / 8, total = ep.M * groups;
  const bool vec = (ep.N & 3) == 0;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t m = i / groups, n0 = (i - m * groups) * 8;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int k = 0; k < split_k; ++k) {
      const float* src = ws + (static_cast<int64_t>(k) * ep.M + m) * ep.N + n0;
      if (vec && n0 + 8 <= ep.N) {
        const float4 a = reinterpret_cast<const float4*>(src)[0], b = reinterpret_cast<const float4*>(src)[1];
        acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
        acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (n0 + j < ep.N) acc[j] += src[j];
      }
    }
    epilogue_row_segment<TOut, 8>(ep, m, n0, acc, seed);
  }
}

// A product whose last round of 256 x 256 tiles would leave most of the 74 thread-block pairs idle (96 tiles: 74 + 22):
// head rows that fill whole rounds, and the K parts for the remaining rows so that they fill one more round of short
// work items. parts == 0: no split (the product does not go to the pair kernel, or its last round is >= 60 % full).
struct TailPlan { int64_t head_rows; int parts; };
TailPlan tail_split_plan(int64_t M, int64_t N, int64_t K) {
  TailPlan none{0, 0};
  if (M < 256 || N < 256 || K < 2048) return none;
  const int64_t pairs = kNumSMs / 2;
  const int64_t num_m = ceil_div(M, 256), num_n = ceil_div(N, 256), tiles = num_m * num_n;
  const int64_t full = tiles / pairs, rest = tiles % pairs;
  if (full < 1 || rest == 0 || rest > 44) return none;
  const int64_t head_mb = full * pairs / num_n, tail_tiles = (num_m - head_mb) * num_n;
  if (head_mb < 1 || tail_tiles < 1) return none;
  int64_t parts = (2 * pairs + tail_tiles) / (2 * tail_tiles);  // pairs / tail_tiles, rounded
  if (parts > 8) parts = 8;
  if (parts > K / 64 / 4) parts = K / 64 / 4;
  if (parts < 2) return none;
  return TailPlan{head_mb * 256, static_cast<int>(parts)};
}

// sums the K-split partial tiles in a fixed order (no-op when split_k == 1)
int finish_split_k(float* workspace, void* c, const float* bias, int64_t M, int64_t N, int64_t ldc, int split_k,
                   int epilogue, int out_dtype, cudaStream_t st) {
  if (split_k <= 1) return PTJ_OK;
  const int64_t total = M * N;
  const bool w4 = N % 4 == 0;
  int64_t blocks = ceil_div(total, 256 * (w4 ? 4 : 1));
  if (blocks > kNumSMs * 8) blocks = kNumSMs * 8;
  const int acc = epilogue == PTJ_EPI_ACCUM;
  const int g = static_cast<int>(blocks);
  if (out_dtype == PTJ_F32) {
    if (w4) launch_k(splitk_reduce_kernel<float, 4>, g, 256, 0, st, workspace, static_cast<float*>(c), bias, M, N, ldc, split_k, acc);
    else launch_k(splitk_reduce_kernel<float, 1>, g, 256, 0, st, workspace, static_cast<float*>(c), bias, M, N, ldc, split_k, acc);
  } else {
    if (w4) launch_k(splitk_reduce_kernel<__nv_bfloat16, 4>, g, 256, 0, st, workspace, static_cast<__nv_bfloat16*>(c), bias, M, N, ldc, split_k, 0);
    else launch_k(splitk_reduce_kernel<__nv_bfloat16, 1>, g, 256, 0, st, workspace, static_cast<__nv_bfloat16*>(c), bias, M, N, ldc, split_k, 0);
  }
  PTJ_CHECK_LAUNCH();
  return PTJ_OK;
}

// p2 != nullptr: a second product in the same launch (see GROUPED above)
template <int BN, bool AK, bool BK_, bool SIDE, bool GROUPED = false>
int launch_tc_pair(const CUtensorMap& ta, const CUtensorMap& tb, const StoreMaps& sm, const GemmParams& p,
                   cudaStream_t st, const CUtensorMap* ta2 = nullptr, const CUtensorMap* tb2 = nullptr,
                   const GemmParams* p2 = nullptr) {
  using Cfg = PairCfg<BN>;
  const int smem_bytes = Cfg::smem_bytes(SIDE ? 2 * kEpiBlockBytes : kStripBytes);
  auto kern = gemm_tc_pair_kernel<BN, AK, BK_, SIDE, GROUPED>;
  static std::atomic<uint64_t> attr_done{0};
  if (!ensure_max_smem(kern, attr_done)) return PTJ_ERR_LAUNCH;
  const int items1 = p.num_m * p.num_n * p.split_k;
  const int total = items1 + (GROUPED ? p2->num_m * p2->num_n * p2->split_k : 0);
  const int pairs = total < kNumSMs / 2 ? total : kNumSMs / 2;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs));
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  if (cudaLaunchKernelEx(&cfg, kern, ta, tb, sm, p, GROUPED ? *ta2 : ta, GROUPED ? *tb2 : tb, GROUPED ? *p2 : p, items1) !=
      cudaSuccess) {
    (void)cudaGetLastError();
    return PTJ_ERR_LAUNCH;
  }
  count_launch(1);
  return PTJ_OK;
}

// Operand tensor maps of the thread-block-pair kernel (256 x 256 tiles: each CTA loads 128 rows of A and 128 of B).
bool make_pair_operand_maps(CUtensorMap* ta, CUtensorMap* tb, const void* a, const void* b, int64_t M, int64_t N,
                            int64_t K, int64_t lda, int64_t ldb, bool a_kmajor, bool b_kmajor) {
  const int pbn = 256;
  {
    const uint64_t dims_k[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
    const uint64_t dims_mn[2] = {static_cast<uint64_t>(M), static_cast<uint64_t>(K)};
    const uint64_t str[1] = {static_cast<uint64_t>(lda) * 2};
    const uint32_t box_k[2] = {64, 128}, box_mn[2] = {64, 64};
    if (!make_tmap_bf16(ta, a, 2, a_kmajor ? dims_k : dims_mn, str, a_kmajor ? box_k : box_mn)) return false;
  }
  {
    const uint64_t dims_k[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N)};
    const uint64_t dims_mn[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(K)};
    const uint64_t str[1] = {static_cast<uint64_t>(ldb) * 2};
    const uint32_t box_k[2] = {64, static_cast<uint32_t>(pbn / 2)}, box_mn[2] = {64, 64};
    if (!make_tmap_bf16(tb, b, 2, b_kmajor ? dims_k : dims_mn, str, b_kmajor ? box_k : box_mn)) return false;
  }
  return true;
}

// Which kernel: the CTA-pair kernel halves the shared-memory traffic per FLOP and wins wherever the main loop is
// long (K >= 2048: weight gradients, the second FFN matrix) or the output is huge (LM head); its 256 x 256 tiles
// quantise worse on the small N = 768 products, which stay on the single-CTA kernel.
bool use_pair_kernel(int64_t M, int64_t N, int64_t K) {
  if (M < 256 || N < 256) return false;
  return K >= 2048 || N >= 8192;
}

}  // namespace
}  // namespace ptj

using namespace ptj;

extern "C" int ptj_gemm(const void* a, const void* b, void* c, const float* bias, const void* aux, void* aux_out,
                        int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int a_kmajor,
                        int b_kmajor, int in_dtype, int out_dtype, int epilogue, const ptj_dropout_args* dropout,
                        int split_k, float* workspace, size_t workspace_floats, void* stream) {
  if (M < 1 || N < 1 || K < 1 || M > (1LL << 30) || N > (1LL << 30) || K > (1LL << 30)) return PTJ_ERR_BAD_SHAPE;
  if (!a || !b || !c) return PTJ_ERR_BAD_SHAPE;
  if (lda < (a_kmajor ? K : M) || ldb < (b_kmajor ? K : N) || ldc < N) return PTJ_ERR_BAD_SHAPE;
  if (out_dtype != PTJ_F32 && out_dtype != PTJ_BF16) return PTJ_ERR_DTYPE;
  if (epilogue < PTJ_EPI_NONE || epilogue > PTJ_EPI_ACCUM) return PTJ_ERR_UNSUPPORTED;
  if ((epilogue == PTJ_EPI_GELU_BWD || epilogue == PTJ_EPI_DROPOUT_RESID) && aux == nullptr) return PTJ_ERR_BAD_SHAPE;
  if (epilogue == PTJ_EPI_DROPOUT_RESID && dropout == nullptr) return PTJ_ERR_BAD_SHAPE;
  if (epilogue == PTJ_EPI_ACCUM && out_dtype != PTJ_F32) return PTJ_ERR_UNSUPPORTED;
  const bool tail_requested = split_k == PTJ_SPLIT_TAIL;
  if (split_k < 1) split_k = 1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  EpilogueParams ep{};
  ep.c = c;
  ep.bias = bias;
  ep.aux = aux;
  ep.aux_out = aux_out;
  ep.M = M;
  ep.N = N;
  ep.ldc = ldc;
  ep.mode = epilogue;
  const size_t osz = dtype_size(out_dtype);
  ep.bias_vec_ok = bias != nullptr && aligned16(bias);
  ep.vec_ok = aligned16(c) && (ldc * osz) % 16 == 0 && (aux == nullptr || aligned16(aux)) &&
              (aux_out == nullptr || aligned16(aux_out));
  if (dropout != nullptr) {
    if (!(dropout->p >= 0.f && dropout->p <= 1.f)) return PTJ_ERR_BAD_SHAPE;
    ep.drop_thr = dropout_threshold16(dropout->p);
    ep.eval_scale = 1.f - dropout->p;
    ep.train = dropout->train;
    ep.seed = dropout->seed;
    ep.stream_id = dropout->stream_id;
  }

  if (in_dtype == PTJ_F32) {
    if (split_k != 1) return PTJ_ERR_UNSUPPORTED;
    const int64_t sam = a_kmajor ? lda : 1, sak = a_kmajor ? 1 : lda;
    const int64_t sbn = b_kmajor ? ldb : 1, sbk = b_kmajor ? 1 : ldb;
    dim3 grid(static_cast<unsigned>(ceil_div(N, SM_BN)), static_cast<unsigned>(ceil_div(M, SM_BM)));
    if (grid.y > 65535) return PTJ_ERR_BAD_SHAPE;
    if (out_dtype == PTJ_F32)
      launch_k(gemm_simt_kernel<float>, grid, 128, 0, st, static_cast<const float*>(a), static_cast<const float*>(b), sam, sak,
                                                    sbn, sbk, M, N, K, ep);
    else
      launch_k(gemm_simt_kernel<__nv_bfloat16>, grid, 128, 0, st, static_cast<const float*>(a), static_cast<const float*>(b),
                                                            sam, sak, sbn, sbk, M, N, K, ep);
    PTJ_CHECK_LAUNCH();
    return PTJ_OK;
  }
  if (in_dtype != PTJ_BF16) return PTJ_ERR_DTYPE;

  if (!aligned16(a) || !aligned16(b) || lda % 8 != 0 || ldb % 8 != 0) return PTJ_ERR_MISALIGNED;
  if (ptj_device_check() != PTJ_OK) return PTJ_ERR_DEVICE;
  const int num_kb = static_cast<int>(ceil_div(K, BK));
  if (split_k > num_kb) split_k = num_kb;
  if (split_k > 1) {
    if (epilogue != PTJ_EPI_NONE && epilogue != PTJ_EPI_ACCUM) return PTJ_ERR_UNSUPPORTED;
    if (!workspace || workspace_floats < static_cast<size_t>(split_k) * M * N || !aligned16(workspace))
      return PTJ_ERR_WORKSPACE;
  }
  GemmParams p{};
  p.ep = ep;
  p.M = M;
  p.N = N;
  p.K = K;
  p.num_m = static_cast<int>(ceil_div(M, BM));
  p.num_kb = num_kb;
  p.split_k = split_k;
  p.workspace = workspace;
  p.out_bf16 = out_dtype == PTJ_BF16;
  p.fault = tc::fault_word();
  if (p.fault == nullptr) return PTJ_ERR_DEVICE;

  StoreMaps smaps{};
  if (p.out_bf16 && ep.vec_ok && split_k == 1) {
    const uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(M)};
    const uint64_t str[1] = {static_cast<uint64_t>(ldc) * 2};
    const uint32_t box[2] = {32, 32};
    if (!make_tmap_bf16_sw64(&smaps.c, c, 2, dims, str, box)) return PTJ_ERR_LAUNCH;
    if (epilogue == PTJ_EPI_GELU && aux_out != nullptr && !make_tmap_bf16_sw64(&smaps.x, aux_out, 2, dims, str, box))
      return PTJ_ERR_LAUNCH;
    p.tma_store = 1;
    if (a_kmajor && (epilogue == PTJ_EPI_GELU_BWD || epilogue == PTJ_EPI_DROPOUT_RESID)) {
      if (!make_tmap_bf16_sw64(&smaps.s, aux, 2, dims, str, box)) return PTJ_ERR_LAUNCH;
      p.tma_side = 1;
    }
  }

  if (use_pair_kernel(M, N, K)) {
    p.num_m = static_cast<int>(ceil_div(M, 2 * BM));
    p.num_n = static_cast<int>(ceil_div(N, 256));
    CUtensorMap ta, tb;
    if (!make_pair_operand_maps(&ta, &tb, a, b, M, N, K, lda, ldb, a_kmajor != 0, b_kmajor != 0)) return PTJ_ERR_LAUNCH;
    // PTJ_SPLIT_TAIL: the rows of a mostly-empty last round of tiles become a second product of the same launch,
    // split over K; their epilogue runs in the finishing kernel
    const TailPlan tp = tail_requested ? tail_split_plan(M, N, K) : TailPlan{0, 0};
    const bool tail_epilogue_ok = (epilogue == PTJ_EPI_NONE && bias == nullptr) ||
                                  (epilogue == PTJ_EPI_DROPOUT_RESID && p.tma_side && a_kmajor && b_kmajor);
    if (tp.parts >= 2 && tail_epilogue_ok && workspace != nullptr && aligned16(workspace) &&
        workspace_floats >= static_cast<size_t>(tp.parts) * (M - tp.head_rows) * N) {
      const int64_t head = tp.head_rows, tail = M - head;
      GemmParams ph = p, pt = p;
      ph.M = ph.ep.M = head;
      ph.num_m = static_cast<int>(head / 256);
      pt.M = pt.ep.M = tail;
      pt.num_m = static_cast<int>(ceil_div(tail, 2 * BM));
      pt.split_k = tp.parts;
      pt.workspace = workspace;
      pt.tma_store = pt.tma_side = 0;
      pt.ep.c = static_cast<char*>(c) + head * ldc * osz;
      if (aux != nullptr) pt.ep.aux = static_cast<const char*>(aux) + head * ldc * osz;
      pt.ep.mask_row0 = head;
      pt.ep.vec_ok = ep.vec_ok;
      const char* a_tail = static_cast<const char*>(a) + (a_kmajor ? head * lda : head) * 2;
      CUtensorMap ta_t, tb_t;
      if (!make_pair_operand_maps(&ta_t, &tb_t, a_tail, b, tail, N, K, lda, ldb, a_kmajor != 0, b_kmajor != 0))
        return PTJ_ERR_LAUNCH;
      int grc;
      if (ph.tma_side)
        grc = launch_tc_pair<256, true, true, true, true>(ta, tb, smaps, ph, st, &ta_t, &tb_t, &pt);
      else
        grc = a_kmajor ? (b_kmajor ? launch_tc_pair<256, true, true, false, true>(ta, tb, smaps, ph, st, &ta_t, &tb_t, &pt)
                                   : launch_tc_pair<256, true, false, false, true>(ta, tb, smaps, ph, st, &ta_t, &tb_t, &pt))
                       : (b_kmajor ? launch_tc_pair<256, false, true, false, true>(ta, tb, smaps, ph, st, &ta_t, &tb_t, &pt)
                                   : launch_tc_pair<256, false, false, false, true>(ta, tb, smaps, ph, st, &ta_t, &tb_t, &pt));
      if (grc != PTJ_OK) return grc;
      const int64_t threads = tail * ceil_div(N, 8);
      int64_t blocks = ceil_div(threads, 256);
      if (blocks > kNumSMs * 8) blocks = kNumSMs * 8;
      if (p.out_bf16)
        launch_k(splitk_finish_kernel<__nv_bfloat16>, static_cast<int>(blocks), 256, 0, st, workspace, pt.ep, tp.parts);
      else
        launch_k(splitk_finish_kernel<float>, static_cast<int>(blocks), 256, 0, st, workspace, pt.ep, tp.parts);
      PTJ_CHECK_LAUNCH();
      return PTJ_OK;
    }
    int prc;
    if (p.tma_side)  // (A is K-major whenever tma_side is set)
      prc = b_kmajor ? launch_tc_pair<256, true, true, true>(ta, tb, smaps, p, st)
                     : launch_tc_pair<256, true, false, true>(ta, tb, smaps, p, st);
    else
      prc = a_kmajor ? (b_kmajor ? launch_tc_pair<256, true, true, false>(ta, tb, smaps, p, st)
                                 : launch_tc_pair<256, true, false, false>(ta, tb, smaps, p, st))
                     : (b_kmajor ? launch_tc_pair<256, false, true, false>(ta, tb, smaps, p, st)
                                 : launch_tc_pair<256, false, false, false>(ta, tb, smaps, p, st));
    if (prc != PTJ_OK) return prc;
    return finish_split_k(workspace, c, bias, M, N, ldc, split_k, epilogue, out_dtype, st);
  }

  // tile width: fewer, fatter tiles (less operand traffic per FLOP) unless that leaves SMs idle in the last wave.
  // cost = waves x tile width x relative cost per column of that width
  auto waves_cost = [&](int bn, double penalty) {
    const int64_t items = static_cast<int64_t>(p.num_m) * ceil_div(N, bn) * split_k;
    return static_cast<double>(ceil_div(items, kNumSMs)) * bn * penalty;
  };
  int bn = 256;
  double best = waves_cost(256, 1.0);
  if (waves_cost(192, 1.08) < best) { bn = 192; best = waves_cost(192, 1.08); }
  if (waves_cost(128, 1.35) < best) { bn = 128; }
  p.num_n = static_cast<int>(ceil_div(N, bn));
  if (static_cast<int64_t>(p.num_m) * p.num_n * split_k > 0x7fffffffLL) return PTJ_ERR_BAD_SHAPE;

  CUtensorMap ta, tb;
  {
    const uint64_t dims_k[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
    const uint64_t dims_mn[2] = {static_cast<uint64_t>(M), static_cast<uint64_t>(K)};
    const uint64_t str[1] = {static_cast<uint64_t>(lda) * 2};
    const uint32_t box_k[2] = {64, 128}, box_mn[2] = {64, 64};
    if (!make_tmap_bf16(&ta, a, 2, a_kmajor ? dims_k : dims_mn, str, a_kmajor ? box_k : box_mn)) return PTJ_ERR_LAUNCH;
  }
  {
    const uint64_t dims_k[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N)};
    const uint64_t dims_mn[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(K)};
    const uint64_t str[1] = {static_cast<uint64_t>(ldb) * 2};
    const uint32_t box_k[2] = {64, static_cast<uint32_t>(bn)}, box_mn[2] = {64, 64};
    if (!make_tmap_bf16(&tb, b, 2, b_kmajor ? dims_k : dims_mn, str, b_kmajor ? box_k : box_mn)) return PTJ_ERR_LAUNCH;
  }

  int rc;
#define PTJ_TC(BN_)                                                              \
  (p.tma_side ? (b_kmajor ? launch_tc<BN_, true, true, true>(ta, tb, smaps, p, st)                \
                          : launch_tc<BN_, true, false, true>(ta, tb, smaps, p, st))              \
   : a_kmajor ? (b_kmajor ? launch_tc<BN_, true, true, false>(ta, tb, smaps, p, st)               \
                          : launch_tc<BN_, true, false, false>(ta, tb, smaps, p, st))             \
              : (b_kmajor ? launch_tc<BN_, false, true, false>(ta, tb, smaps, p, st)              \
                          : launch_tc<BN_, false, false, false>(ta, tb, smaps, p, st)))
  rc = bn == 128 ? PTJ_TC(128) : (bn == 192 ? PTJ_TC(192) : PTJ_TC(256));
#undef PTJ_TC
  if (rc != PTJ_OK) return rc;

  return finish_split_k(workspace, c, bias, M, N, ldc, split_k, epilogue, out_dtype, st);
}

extern "C" size_t ptj_gemm_tail_split_floats(int64_t M, int64_t N, int64_t K) {
  if (M < 1 || N < 1 || K < 1) return 0;
  const TailPlan tp = tail_split_plan(M, N, K);
  return tp.parts >= 2 ? static_cast<size_t>(tp.parts) * (M - tp.head_rows) * N : 0;
}

extern "C" int64_t ptj_gemm_tail_split_rows(int64_t M, int64_t N, int64_t K) {
  if (M < 1 || N < 1 || K < 1) return 0;
  const TailPlan tp = tail_split_plan(M, N, K);
  return tp.parts >= 2 ? tp.head_rows : 0;
}

// ---- two products in one launch -----------------------------------------------------------------------------------
namespace {
// parameters of one product of ptj_gemm_grouped2 for the thread-block-pair kernel (no bias, no side input).
// store_maps: where the product may leave through tensor-map tile stores (bf16 output, K not split): the first
// product only, the kernel has one set of output maps.
int make_grouped_problem(const ptj_gemm_problem& g, int64_t K, int a_kmajor, int b_kmajor, CUtensorMap* ta,
                         CUtensorMap* tb, GemmParams* out, StoreMaps* store_maps) {
  if (!g.a || !g.b || !g.c || g.M < 1 || g.N < 1) return PTJ_ERR_BAD_SHAPE;
  if (g.M > (1LL << 30) || g.N > (1LL << 30)) return PTJ_ERR_BAD_SHAPE;
  if (g.lda < (a_kmajor ? K : g.M) || g.ldb < (b_kmajor ? K : g.N) || g.ldc < g.N) return PTJ_ERR_BAD_SHAPE;
  if (g.epilogue != PTJ_EPI_NONE && g.epilogue != PTJ_EPI_ACCUM) return PTJ_ERR_UNSUPPORTED;
  if (g.out_dtype != PTJ_F32 && g.out_dtype != PTJ_BF16) return PTJ_ERR_DTYPE;
  if (g.epilogue == PTJ_EPI_ACCUM && g.out_dtype != PTJ_F32) return PTJ_ERR_UNSUPPORTED;
  if (!aligned16(g.a) || !aligned16(g.b) || g.lda % 8 != 0 || g.ldb % 8 != 0) return PTJ_ERR_MISALIGNED;
  if (!use_pair_kernel(g.M, g.N, K)) return PTJ_ERR_UNSUPPORTED;
  const int num_kb = static_cast<int>(ceil_div(K, BK));
  int split_k = g.split_k < 1 ? 1 : g.split_k;
  if (split_k > num_kb) split_k = num_kb;
  if (split_k > 1 && (!g.workspace || g.workspace_floats < static_cast<size_t>(split_k) * g.M * g.N ||
                      !aligned16(g.workspace)))
    return PTJ_ERR_WORKSPACE;
  GemmParams p{};
  p.ep.c = g.c;
  p.ep.M = g.M;
  p.ep.N = g.N;
  p.ep.ldc = g.ldc;
  p.ep.mode = g.epilogue;
  const size_t osz = dtype_size(g.out_dtype);
  p.ep.vec_ok = aligned16(g.c) && (g.ldc * osz) % 16 == 0;
  p.out_bf16 = g.out_dtype == PTJ_BF16;
  p.M = g.M;
  p.N = g.N;
  p.K = K;
  p.num_m = static_cast<int>(ceil_div(g.M, 2 * BM));
  p.num_n = static_cast<int>(ceil_div(g.N, 256));
  p.num_kb = num_kb;
  p.split_k = split_k;
  p.workspace = g.workspace;
  p.fault = tc::fault_word();
  if (p.fault == nullptr) return PTJ_ERR_DEVICE;
  if (static_cast<int64_t>(p.num_m) * p.num_n * split_k > 0x3fffffffLL) return PTJ_ERR_BAD_SHAPE;
  if (!make_pair_operand_maps(ta, tb, g.a, g.b, g.M, g.N, K, g.lda, g.ldb, a_kmajor != 0, b_kmajor != 0))
    return PTJ_ERR_LAUNCH;
  if (store_maps != nullptr && p.out_bf16 && p.ep.vec_ok && split_k == 1) {
    const uint64_t dims[2] = {static_cast<uint64_t>(g.N), static_cast<uint64_t>(g.M)};
    const uint64_t str[1] = {static_cast<uint64_t>(g.ldc) * 2};
    const uint32_t box[2] = {32, 32};
    if (!make_tmap_bf16_sw64(&store_maps->c, g.c, 2, dims, str, box)) return PTJ_ERR_LAUNCH;
    p.tma_store = 1;
  }
  *out = p;
  return PTJ_OK;
}
}  // namespace

extern "C" int ptj_gemm_grouped2(const ptj_gemm_problem* g0, const ptj_gemm_problem* g1, int64_t K, int a_kmajor,
                                 int b_kmajor, void* stream) {
  if (!g0 || !g1 || K < 1 || K > (1LL << 30)) return PTJ_ERR_BAD_SHAPE;
  if (ptj_device_check() != PTJ_OK) return PTJ_ERR_DEVICE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  CUtensorMap ta0, tb0, ta1, tb1;
  GemmParams p0, p1;
  StoreMaps none{};  // (holds the first product's output map when that product stores through it)
  int rc = make_grouped_problem(*g0, K, a_kmajor, b_kmajor, &ta0, &tb0, &p0, &none);
  if (rc != PTJ_OK) return rc;
  rc = make_grouped_problem(*g1, K, a_kmajor, b_kmajor, &ta1, &tb1, &p1, nullptr);
  if (rc != PTJ_OK) return rc;
  rc = a_kmajor ? (b_kmajor ? launch_tc_pair<256, true, true, false, true>(ta0, tb0, none, p0, st, &ta1, &tb1, &p1)
                            : launch_tc_pair<256, true, false, false, true>(ta0, tb0, none, p0, st, &ta1, &tb1, &p1))
                : (b_kmajor ? launch_tc_pair<256, false, true, false, true>(ta0, tb0, none, p0, st, &ta1, &tb1, &p1)
                            : launch_tc_pair<256, false, false, false, true>(ta0, tb0, none, p0, st, &ta1, &tb1, &p1));
  if (rc != PTJ_OK) return rc;
  rc = finish_split_k(p0.workspace, g0->c, nullptr, g0->M, g0->N, g0->ldc, p0.split_k, g0->epilogue, g0->out_dtype, st);
  if (rc != PTJ_OK) return rc;
  return finish_split_k(p1.workspace, g1->c, nullptr, g1->M, g1->N, g1->ldc, p1.split_k, g1->epilogue, g1->out_dtype, st);
}
