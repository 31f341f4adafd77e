// Causal flash attention on tcgen05 tensor cores (bf16 in, fp32 accumulate), d_head = 64, seq % 128 == 0.
// Semantics: model_triton.py:608-611 / 510-517 (forward), :801-811 / 550-577 (backward): softmax of the causally
// masked scaled scores, dropout on the probabilities (no rescale), times V. The row maximum and row sum of
// exponentials are saved (the reference's acts0 / acts1, :699-700) and the backward recomputes the probabilities.
//
// One thread block = 128 threads = 128 query rows; thread t owns row t of the 128 x 128 score tile that
// tcgen05.mma leaves in tensor memory (lane t), so row maxima and sums need no shuffles. Q/K/V/dO tiles come in
// through 4-D TMA maps over the caller's strided [batch, heads, seq, 64] views (128-byte swizzle); the probability
// and score-gradient tiles are written back to shared memory in the same swizzled layout and fed to the next MMA
// either K-major (P V, dS K) or MN-major (P^T dO, dS^T Q) by changing only the descriptor.
//
//   forward : per KV tile  S = Q K^T -> softmax in registers -> P to smem -> O_j = P V -> o = o * alpha + O_j
//   backward: kernel A (one block per KV tile, loops over query tiles): dV += Pd^T dO, dK += dS^T Q  (tensor memory)
//             kernel B (one block per query tile, loops over KV tiles): dQ += dS K
//             both recompute S and dP = dO V^T; no atomics, so results are bit-reproducible.
#include "attn_tc_dev.cuh"

namespace ptj {
namespace {

using namespace attn_tc;

// ---------------------------------------------------------------------------------------------------------------------
// backward. MODE 0: block owns a KV tile, loops over query tiles >= it, produces dK and dV.
//           MODE 1: block owns a query tile, loops over KV tiles <= it, produces dQ.
// Tensor memory (256 columns, so two blocks share an SM): [0,128) holds S and is then overwritten by dP (every
// thread keeps its row of probabilities in registers as packed bf16), [128,192) and [192,256) are the accumulators.
// Shared memory (96 KB): Q, K, V, dO tiles and ONE 32 KB buffer that first carries Pd (for dV) and then dS.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kBwdSmem = 4 * kTileBytes + 2 * kTileBytes + 1024 + 128;
constexpr int kBwdTmemCols = 256;

template <int MODE>
__global__ void __launch_bounds__(128, 2)
attn_bwd_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_g,
                   const RowView d_o, const RowView o_view, const float* __restrict__ row_max,
                   const float* __restrict__ row_sum, const RowView out0, const RowView out1, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = align1024(smem_raw);
  uint8_t* q_s = sm;
  uint8_t* k_s = sm + kTileBytes;
  uint8_t* v_s = sm + 2 * kTileBytes;
  uint8_t* g_s = sm + 3 * kTileBytes;
  uint8_t* w_s = sm + 4 * kTileBytes;  // Pd, then dS (two [128][64] sub-tiles)
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + 6 * kTileBytes);
  // bar_fix: resident tiles; bar_m0 / bar_m1: the two moving tiles; bar_s: S ready; bar_p: dP ready (and, MODE 0, the
  // dV MMA has consumed Pd); bar_acc: last accumulation MMA of the iteration done
  uint64_t *bar_fix = bars, *bar_m0 = bars + 1, *bar_m1 = bars + 2, *bar_s = bars + 3, *bar_p = bars + 4, *bar_acc = bars + 5;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5;
  // MODE 0: heavy KV tiles (early ones, many query tiles) first; MODE 1: heavy (late) query tiles first
  const int own = MODE == 0 ? static_cast<int>(blockIdx.x) / p.BH : p.nq - 1 - static_cast<int>(blockIdx.x) / p.BH;
  const int bh = static_cast<int>(blockIdx.x) % p.BH;
  const int b = bh / p.H, h = bh % p.H;
  const AbortCtx ctx{abort_flag, p.fault};

  if (tid == 0) {
    for (int i = 0; i < 6; ++i) mbar_init(&bars[i], 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc(tmem_slot, kBwdTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
  constexpr uint32_t idesc_s = idesc_bf16_f32(T, T, false, false);   // Q K^T and dO V^T
  constexpr uint32_t idesc_t = idesc_bf16_f32(T, DH, true, true);    // Pd^T dO, dS^T Q
  constexpr uint32_t idesc_q = idesc_bf16_f32(T, DH, false, true);   // dS K

  const int lo = MODE == 0 ? own : 0;
  const int hi = MODE == 0 ? p.nq : own + 1;
  // moving tile 0 feeds the S MMA and stays busy until the end of the iteration (MODE 0: Q, MODE 1: K);
  // moving tile 1 is only needed until dP (MODE 0: dO, also read by the dV MMA; MODE 1: V)
  uint8_t* m0_s = MODE == 0 ? q_s : k_s;
  uint8_t* m1_s = MODE == 0 ? g_s : v_s;
  const CUtensorMap* m0_map = MODE == 0 ? &tm_q : &tm_k;
  const CUtensorMap* m1_map = MODE == 0 ? &tm_g : &tm_v;
  bool dead = false;
  if (tid == 0) {
    mbar_expect_tx(bar_fix, 2 * kTileBytes);
    if (MODE == 0) {
      tma_load_4d(k_s, &tm_k, bar_fix, 0, own * T, h, b);
      tma_load_4d(v_s, &tm_v, bar_fix, 0, own * T, h, b);
    } else {
      tma_load_4d(q_s, &tm_q, bar_fix, 0, own * T, h, b);
      tma_load_4d(g_s, &tm_g, bar_fix, 0, own * T, h, b);
    }
    mbar_expect_tx(bar_m0, kTileBytes);
    tma_load_4d(m0_s, m0_map, bar_m0, 0, lo * T, h, b);
    mbar_expect_tx(bar_m1, kTileBytes);
    tma_load_4d(m1_s, m1_map, bar_m1, 0, lo * T, h, b);
    dead = !mbar_wait(bar_fix, 0, ctx, 0x2001u);
  }

  // per-row constants of a query row: log2-domain row maximum, 1 / row sum, delta = sum_d dO[q,d] O[q,d]
  struct RowConsts { float m2, inv_l, delta; };
  auto load_row_consts = [&](int q_tile) {
    const int64_t qr = static_cast<int64_t>(q_tile) * T + tid;
    const int64_t ri = static_cast<int64_t>(bh) * p.S + qr;
    RowConsts rc;
    rc.m2 = row_max[ri] * kLog2e;
    rc.inv_l = 1.f / row_sum[ri];
    const __nv_bfloat16* go = d_o.row(b, h, qr);
    const __nv_bfloat16* oo = o_view.row(b, h, qr);
    float acc = 0.f;
#pragma unroll
    for (int c = 0; c < DH / 8; ++c) {
      float x[8], y[8];
      Elem<__nv_bfloat16>::load_vec(go + c * 8, x);
      Elem<__nv_bfloat16>::load_vec(oo + c * 8, y);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc = fmaf(x[i], y[i], acc);
    }
    rc.delta = acc;
    return rc;
  };
  RowConsts rc = load_row_consts(MODE == 0 ? lo : own);

  int it = 0;
  for (int t = lo; t < hi; ++t, ++it) {
    const uint32_t ph = it & 1;
    const int qt = MODE == 0 ? t : own;
    const int kt = MODE == 0 ? own : t;
    const bool diag = qt == kt;
    const int64_t q_row = static_cast<int64_t>(qt) * T + tid;
    const uint64_t idx_row = (static_cast<uint64_t>(bh) * p.S + q_row) * p.S + static_cast<uint64_t>(kt) * T;
    const bool masked = p.dr.train && p.dr.thr16 != 0u;
    const float f_keep = p.dr.train ? 1.f : p.dr.eval_scale;

    // ---- S = Q K^T ----
    if (tid == 0 && !dead) {
      dead = !mbar_wait(bar_m0, ph, ctx, 0x2002u);
      if (!dead) {
        tc_fence_after_sync();
#pragma unroll
        for (int k16 = 0; k16 < DH / 16; ++k16)
          mma_bf16_ss(tmem, desc_kmajor_d(smem_u32(q_s), k16), desc_kmajor_d(smem_u32(k_s), k16), idesc_s, k16 > 0);
        mma_commit(bar_s);
      }
    }
    if (!dead) dead = !mbar_wait(bar_s, ph, ctx, 0x2003u);
    tc_fence_after_sync();
    dead = __any_sync(0xffffffffu, dead);

    // probabilities of this thread's row, kept in registers as packed bf16 pairs, and the dropout keep bits
    uint32_t pk[T / 2];
    uint32_t keep[4] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
    if (!dead) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float s[32];
        tmem_ld_row32(tmem + lane_base + c * 32, s);
        if (masked) keep[c] = keep_bits32(p.dr, idx_row + c * 32);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float pr = ex2_approx(fmaf(s[i], p.scale_log2, -rc.m2)) * rc.inv_l;
          if (diag && c * 32 + i > tid) pr = 0.f;
          s[i] = pr;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const __nv_bfloat162 h2 = __floats2bfloat162_rn(s[2 * i], s[2 * i + 1]);
          pk[c * 16 + i] = *reinterpret_cast<const uint32_t*>(&h2);
        }
        if (MODE == 0) {  // Pd = P * keep (* (1-p) in evaluation) for dV += Pd^T dO
#pragma unroll
          for (int i = 0; i < 32; ++i) s[i] = ((keep[c] >> i) & 1u) ? s[i] * f_keep : 0.f;
          store_row32_sw128(w_s, tid, c * 32, s);
        }
      }
    }
    if (MODE == 0) fence_proxy_async_smem();
    tc_fence_before_sync();
    if (__syncthreads_or(dead ? 1 : 0)) { dead = true; break; }  // S consumed by every thread, Pd complete

    // ---- dP = dO V^T into the columns S occupied (MODE 0: preceded by dV += Pd^T dO) ----
    if (tid == 0) {
      tc_fence_after_sync();
      dead = !mbar_wait(bar_m1, ph, ctx, 0x2004u);
      if (!dead) {
        tc_fence_after_sync();
        if (MODE == 0) {
#pragma unroll
          for (int k16 = 0; k16 < T / 16; ++k16)
            mma_bf16_ss(tmem + 128, desc_p_transposed(smem_u32(w_s), k16), desc_rows_as_k(smem_u32(g_s), k16), idesc_t,
                        (it > 0 || k16 > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int k16 = 0; k16 < DH / 16; ++k16)
          mma_bf16_ss(tmem, desc_kmajor_d(smem_u32(g_s), k16), desc_kmajor_d(smem_u32(v_s), k16), idesc_s, k16 > 0);
        mma_commit(bar_p);
      }
    }
    if (!dead) dead = !mbar_wait(bar_p, ph, ctx, 0x2005u);
    tc_fence_after_sync();
    if (tid == 0 && !dead && t + 1 < hi) {  // moving tile 1 is free: fetch the next one while dS is being formed
      mbar_expect_tx(bar_m1, kTileBytes);
      tma_load_4d(m1_s, m1_map, bar_m1, 0, (t + 1) * T, h, b);
    }
    // the buffer that receives dS was last read by the previous iteration's accumulation MMA (MODE 1) or by this
    // iteration's dV MMA (MODE 0, covered by bar_p)
    if (MODE == 1 && it > 0 && !dead) dead = !mbar_wait(bar_acc, ph ^ 1u, ctx, 0x2006u);
    dead = __any_sync(0xffffffffu, dead);
    if (!dead) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float dp[32];
        tmem_ld_row32(tmem + lane_base + c * 32, dp);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const uint32_t w = pk[c * 16 + (i >> 1)];
          const float pr = __uint_as_float((i & 1) ? (w & 0xffff0000u) : (w << 16));
          const float f = ((keep[c] >> i) & 1u) ? f_keep : 0.f;
          dp[i] = pr * (dp[i] * f - rc.delta) * p.scale;  // gradient w.r.t. the raw score q.k
        }
        store_row32_sw128(w_s, tid, c * 32, dp);
      }
    }
    // constants of the next query row (MODE 0): issue the loads now, they are consumed after the barrier
    RowConsts rc_next = rc;
    if (MODE == 0 && t + 1 < hi) rc_next = load_row_consts(t + 1);
    fence_proxy_async_smem();
    tc_fence_before_sync();
    if (__syncthreads_or(dead ? 1 : 0)) { dead = true; break; }  // dP consumed, dS complete

    // ---- accumulate: MODE 0 dK += dS^T Q ; MODE 1 dQ += dS K ----
    if (tid == 0) {
      tc_fence_after_sync();
      if (MODE == 0) {
#pragma unroll
        for (int k16 = 0; k16 < T / 16; ++k16)
          mma_bf16_ss(tmem + 192, desc_p_transposed(smem_u32(w_s), k16), desc_rows_as_k(smem_u32(q_s), k16), idesc_t,
                      (it > 0 || k16 > 0) ? 1u : 0u);
      } else {
#pragma unroll
        for (int k16 = 0; k16 < T / 16; ++k16)
          mma_bf16_ss(tmem + 128, desc_p_kmajor(smem_u32(w_s), k16), desc_rows_as_k(smem_u32(k_s), k16), idesc_q,
                      (it > 0 || k16 > 0) ? 1u : 0u);
      }
      mma_commit(bar_acc);
      if (t + 1 < hi) {  // moving tile 0 is reusable once this MMA has read it
        dead = !mbar_wait(bar_acc, ph, ctx, 0x2007u);
        if (!dead) {
          mbar_expect_tx(bar_m0, kTileBytes);
          tma_load_4d(m0_s, m0_map, bar_m0, 0, (t + 1) * T, h, b);
        }
      }
    }
    // MODE 0 overwrites the Pd/dS buffer early in the next iteration: every thread waits for the MMA that reads it
    if (MODE == 0 && tid != 0 && !dead && t + 1 < hi) dead = !mbar_wait(bar_acc, ph, ctx, 0x2008u);
    rc = rc_next;
  }

  if (!dead) dead = !mbar_wait(bar_acc, (it - 1) & 1, ctx, 0x2009u);  // the last accumulation MMA
  if (!__syncthreads_or(dead ? 1 : 0)) {
    tc_fence_after_sync();
    const int64_t r = static_cast<int64_t>(own) * T + tid;
#pragma unroll
    for (int which = 0; which < (MODE == 0 ? 2 : 1); ++which) {
      // MODE 0: which 0 = dV (columns 128.. -> out1), which 1 = dK (columns 192.. -> out0); MODE 1: dQ -> out0
      const RowView& dst_view = (MODE == 0 && which == 0) ? out1 : out0;
      __nv_bfloat16* dst = dst_view.row(b, h, r);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float v[32];
        tmem_ld_row32(tmem + lane_base + 128 + which * 64 + c * 32, v);
#pragma unroll
        for (int q8 = 0; q8 < 4; ++q8) {
          float t8[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) t8[i] = v[q8 * 8 + i];
          Elem<__nv_bfloat16>::store_vec(dst + c * 32 + q8 * 8, t8);
        }
      }
    }
  } else {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, kBwdTmemCols);
  }
}

}  // namespace

bool attn_tc_supported(const ptj_attn_shape& sh, const void* const* ptrs, int nptrs) {
  if (sh.d_head != DH || sh.seq % T != 0 || sh.seq < T || sh.seq > (1 << 20)) return false;
  if (sh.batch * sh.heads * (sh.seq / T) > 0x7fffffffLL) return false;
  for (int i = 0; i < nptrs; ++i)
    if (!aligned16(ptrs[i])) return false;
  const int64_t* sts[4] = {sh.q_strides, sh.k_strides, sh.v_strides, sh.o_strides};
  for (const int64_t* st : sts) {
    if (st[0] % 8 != 0 || st[1] % 8 != 0 || st[2] % 8 != 0 || st[2] < DH) return false;
    if ((sh.batch > 1 && st[0] <= 0) || (sh.heads > 1 && st[1] <= 0)) return false;
  }
  return ptj_device_check() == PTJ_OK;
}

int attn_bwd_tc(const void* d_o, const void* q, const void* k, const void* v, const void* o, const float* row_max,
                const float* row_sum, void* dq, void* dk, void* dv, const ptj_attn_shape& sh,
                const ptj_attn_shape& dsh, const AttnDropout& dr, cudaStream_t st) {
  CUtensorMap tq, tk, tv, tg;
  if (!make_map(&tq, q, sh, sh.q_strides) || !make_map(&tk, k, sh, sh.k_strides) ||
      !make_map(&tv, v, sh, sh.v_strides) || !make_map(&tg, d_o, sh, sh.o_strides))
    return PTJ_ERR_LAUNCH;
  const AttnParams p = make_params(sh, dr);
  if (p.fault == nullptr) return PTJ_ERR_DEVICE;
  for (auto kern : {attn_bwd_tc_kernel<0>, attn_bwd_tc_kernel<1>})
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwdSmem) != cudaSuccess) {
      (void)cudaGetLastError();
      return PTJ_ERR_LAUNCH;
    }
  const RowView g_view = make_view(d_o, sh.o_strides), o_view = make_view(o, sh.o_strides);
  attn_bwd_tc_kernel<0><<<p.nq * p.BH, 128, kBwdSmem, st>>>(tq, tk, tv, tg, g_view, o_view, row_max, row_sum,
                                                           make_view(dk, dsh.k_strides), make_view(dv, dsh.v_strides), p);
  PTJ_CHECK_LAUNCH();
  attn_bwd_tc_kernel<1><<<p.nq * p.BH, 128, kBwdSmem, st>>>(tq, tk, tv, tg, g_view, o_view, row_max, row_sum,
                                                           make_view(dq, dsh.q_strides), make_view(dq, dsh.q_strides), p);
  PTJ_CHECK_LAUNCH();
  return PTJ_OK;
}

}  // namespace ptj
