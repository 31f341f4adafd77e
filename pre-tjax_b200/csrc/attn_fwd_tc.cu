// Causal flash attention forward on tcgen05 tensor cores (bf16 in, fp32 accumulate), d_head = 64, seq % 128 == 0.
// Semantics: model_triton.py:608-611 / 510-517: softmax of the causally masked scaled scores, dropout on the
// probabilities (no rescale), times V; the row maximum and row sum of exponentials are saved (acts0 / acts1, :699-700).
//
// Persistent, warp-specialised thread block (one per SM, 384 threads):
//   warp 0      one thread issues the TMA copies: Q of a work item (2 buffers), K tiles (3-deep ring), V tiles (2-deep
//               ring), K and V as independent sequences
//   warp 1      issues the score MMAs S_g = Q K_g^T, up to three tiles ahead of the softmax
//   warps 2, 3  issue the output MMAs O += P_g V_g, one warp per softmax group
//   warps 4..7 / 8..11  two softmax groups; group x takes the tiles g of the block's tile stream with g % 2 == x, so
//               one group's exponentials overlap the other group's tensor-memory loads, barriers and bookkeeping.
//               Thread t of a group owns row t of the 128 x 128 score tile (tensor-memory lane t): no shuffles. Each
//               group accumulates its own output rows in tensor memory (the P V product adds onto them) with its
//               own reference exponent and row sums; when the item ends, the group that did not get the last tile
//               hands its state over through shared memory and the other one merges the two (log-sum-exp merge in
//               a fixed order) and writes the rows out.
// Work items = (query tile, batch*head), heaviest first, dealt to the blocks in boustrophedon order; all tiles of a
// block's items form one stream, so the next item's first tiles overlap the tail of the current one.
// Tensor memory: three S buffers at columns [0,384), one output accumulator per group at [384,512).
#include "attn_tc_dev.cuh"

namespace ptj {
namespace {

using namespace attn_tc;

constexpr int kThreads = 384;  // warps 0-3: TMA and MMA issue; warps 4-7 and 8-11: the softmax groups
constexpr int kKStages = 3, kVStages = 2, kSBufs = 3;
constexpr int kOffK = 2 * kTileBytes;                     // after Q[2]
constexpr int kOffV = kOffK + kKStages * kTileBytes;
constexpr int kOffP = kOffV + kVStages * kTileBytes;     // P[2 groups][2 sub-tiles]
constexpr int kOffDump = kOffP + 4 * kTileBytes;          // float[64 + 3][128]: hand-over of one group's state
constexpr int kOffBars = kOffDump + (DH + 3) * T * 4;
constexpr int kNumBars = 4 + 2 * kKStages + 2 * kVStages + 2 * kSBufs + 6 + 2;
constexpr int kSmemBytes = kOffBars + kNumBars * 8 + 16 + 80 + 4 * 32 + 1024;  // (+ 32 first-tile entries, VARLEN)
constexpr int kTmemCols = 512;

struct Sched {
  int total, rounds, nq, BH;
  uint32_t bh_magic;  // ceil(2^32 / BH): x / BH == umulhi(x, bh_magic) for every x the kernel meets (checked on the host)
};

// Position in the stream of (item, kv tile) pairs of one thread block; every role walks the same stream.
// first_tile (VARLEN): per round of this block, the first KV tile its item needs (keys before the first key of every
// row of the query tile are masked anyway: those tiles are skipped); nullptr = every item starts at tile 0.
constexpr int kMaxRoundsTabled = 32;
struct Cursor {
  int n, ord, qt, bh, j, j0, g;
  bool valid;
  const int* first_tile;
  __device__ __forceinline__ void next_item(const Sched& s) {
    valid = false;
    while (++n < s.rounds) {
      const int pos = (n & 1) ? static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x);
      const int sp = n * static_cast<int>(gridDim.x) + pos;
      if (sp < s.total) {
        const int t = s.BH == 1 ? sp : static_cast<int>(__umulhi(static_cast<uint32_t>(sp), s.bh_magic));  // sp / BH
        qt = s.nq - 1 - t;
        bh = sp - t * s.BH;
        j0 = first_tile != nullptr ? first_tile[n] : 0;
        j = j0;
        ++ord;
        valid = true;
        return;
      }
    }
  }
  __device__ __forceinline__ void init(const Sched& s, const int* first = nullptr) {
    n = -1; ord = -1; g = 0; qt = 0; bh = 0; j = 0; j0 = 0;
    first_tile = first;
    next_item(s);
  }
  __device__ __forceinline__ void advance(const Sched& s) {
    ++g;
    if (j == qt) next_item(s); else ++j;
  }
};

// MODE 0: no dropout mask; 1: Philox drawn in the kernel; 2: precomputed keep flags (p.keep_bits).
// VARLEN: query row i attends keys [p.kstart[b, i], i] only (packed documents / padding, the block-diagonal x causal x
// padding masks of the reference's collator, tokenized_dataset.py:110-131); a row whose range is empty gets a zero
// output row and the statistics (row_max, row_sum) = (0, 1). The tile stream is the causal one: keys outside a row's
// range are masked, whole tiles outside it contribute exact zeros.
template <int MODE, bool VARLEN>
__global__ void __launch_bounds__(kThreads, 1)
attn_fwd_ws_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const RowView out, float* __restrict__ row_max,
                   float* __restrict__ row_sum, const AttnParams p, const Sched sched) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = align1024(smem_raw);
  uint8_t* q_s = sm;
  uint8_t* k_s = sm + kOffK;
  uint8_t* v_s = sm + kOffV;
  uint8_t* p_s = sm + kOffP;
  float* dump = reinterpret_cast<float*>(sm + kOffDump);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + kOffBars);
  uint64_t* q_full = bars;                  // [2]
  uint64_t* q_empty = bars + 2;             // [2]
  uint64_t* k_full = bars + 4;              // [kKStages]
  uint64_t* k_empty = k_full + kKStages;
  uint64_t* v_full = k_empty + kKStages;    // [kVStages]
  uint64_t* v_empty = v_full + kVStages;
  uint64_t* s_full = v_empty + kVStages;    // [kSBufs]
  uint64_t* s_free = s_full + kSBufs;       // [kSBufs] one arrival per warp of the group that read the tile
  uint64_t* p_ready = s_free + kSBufs;      // [2] per group, one arrival per warp
  uint64_t* o_full = p_ready + 2;           // [2] per group
  uint64_t* o_free = o_full + 2;            // [2] per group, one arrival per warp
  uint64_t* dump_full = o_free + 2;         // one arrival per warp of the group that hands over
  uint64_t* dump_free = dump_full + 1;      // one arrival per warp of the group that merges
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dump_free + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint32_t* rk_s = tmem_slot + 2;  // Philox round keys (MODE 1)
  int* first_tab = reinterpret_cast<int*>(rk_s + 20);  // [kMaxRoundsTabled] first KV tile of this block's items (VARLEN)

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const AbortCtx ctx{abort_flag, p.fault};

  if (tid == 0) {
    for (int i = 0; i < 4 + 2 * kKStages + 2 * kVStages + kSBufs; ++i) mbar_init(&bars[i], 1);  // TMA / MMA completions
    for (int i = 0; i < kSBufs; ++i) mbar_init(&s_free[i], 4);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&p_ready[i], 4);
      mbar_init(&o_full[i], 1);
      mbar_init(&o_free[i], 4);
    }
    mbar_init(dump_full, 4);
    mbar_init(dump_free, 4);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_k);
    prefetch_tensormap(&tm_v);
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
  // VARLEN: whole KV tiles before the first key of every row of a query tile are skipped. Warp w looks at the item of
  // round w, w + 12, ...: the smallest first key over the tile's rows that have keys at all (none: only the diagonal
  // tile is visited, it masks everything).
  const int* first_tile = nullptr;
  if (VARLEN && sched.rounds <= kMaxRoundsTabled) {
    for (int n = warp; n < sched.rounds; n += kThreads / 32) {
      const int pos = (n & 1) ? static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x);
      const int sp = n * static_cast<int>(gridDim.x) + pos;
      int first = 0;
      if (sp < sched.total) {
        const int t = sp / sched.BH;
        const int qt = sched.nq - 1 - t, bh = sp - t * sched.BH;
        const int32_t* ks = p.kstart + static_cast<int64_t>(bh / p.H) * p.S + static_cast<int64_t>(qt) * T;
        int lo = 0x7fffffff;
        for (int r = lane; r < T; r += 32) {
          const int k = __ldg(ks + r);
          if (k <= qt * T + r) lo = min(lo, k);  // (k > row: the row has no keys)
        }
        lo = __reduce_min_sync(0xffffffffu, lo);
        first = lo == 0x7fffffff ? qt : min(max(lo, 0) / T, qt);
      }
      if (lane == 0) first_tab[n] = first;
    }
    __syncthreads();
    first_tile = first_tab;
  }

  // the copy / MMA warps hand most of their registers to the softmax warps (whole groups of four warps switch together)
  if (warp < 4) asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    // K (with Q at an item's first tile) and V are two independent sequences over the same stream: whichever has a
    // free slot is fetched next, so the K tiles run as far ahead as their ring allows.
    if (lane == 0) {
      Cursor ck, cv;
      ck.init(sched, first_tile);
      cv.init(sched, first_tile);
      bool q_done = false;  // Q of ck's item has been requested
      long long t_idle = clock64();
      while (ck.valid || cv.valid) {
        bool progress = false;
        if (ck.valid) {
          const int b = ck.bh / p.H, h = ck.bh % p.H;
          const int qb = ck.ord & 1;
          if (ck.j == ck.j0 && !q_done && mbar_try_wait(&q_empty[qb], ((ck.ord >> 1) & 1) ^ 1u)) {
            mbar_expect_tx(&q_full[qb], kTileBytes);
            tma_load_4d(q_s + qb * kTileBytes, &tm_q, &q_full[qb], 0, ck.qt * T, h, b);
            q_done = true;
            progress = true;
          }
          const int st = ck.g % kKStages;
          if ((ck.j > ck.j0 || q_done) && mbar_try_wait(&k_empty[st], ((ck.g / kKStages) & 1) ^ 1u)) {
            mbar_expect_tx(&k_full[st], kTileBytes);
            tma_load_4d(k_s + st * kTileBytes, &tm_k, &k_full[st], 0, ck.j * T, h, b);
            ck.advance(sched);
            q_done = false;
            progress = true;
          }
        }
        if (cv.valid) {
          const int st = cv.g % kVStages;
          if (mbar_try_wait(&v_empty[st], ((cv.g / kVStages) & 1) ^ 1u)) {
            mbar_expect_tx(&v_full[st], kTileBytes);
            tma_load_4d(v_s + st * kTileBytes, &tm_v, &v_full[st], 0, cv.j * T, cv.bh % p.H, cv.bh / p.H);
            cv.advance(sched);
            progress = true;
          }
        }
        if (progress) {
          t_idle = clock64();
        } else {
          if (*abort_flag) break;
          if (clock64() - t_idle > kWaitLimitCycles) {
            *abort_flag = 1;
            record_fault(p.fault, 0x1101u);
            break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer, scores: S_g = Q K_g^T
    // every lane walks the stream and waits (addresses and descriptors stay warp-uniform); an elected lane issues
    constexpr uint32_t idesc_s = idesc_bf16_f32(T, T, false, false);
    Cursor a;
    a.init(sched, first_tile);
    bool ok = true;
    while (a.valid && ok) {
      const int st = a.g % kKStages;
      const int qb = a.ord & 1;
      const int sb = a.g % kSBufs;
      bool w = true;
      if (a.j == a.j0) w = mbar_wait(&q_full[qb], (a.ord >> 1) & 1, ctx, 0x1201u);
      if (w) w = mbar_wait(&k_full[st], (a.g / kKStages) & 1, ctx, 0x1202u);
      if (w) w = mbar_wait(&s_free[sb], ((a.g / kSBufs) & 1) ^ 1u, ctx, 0x1203u);  // tile g - 3 has been read out
      ok = __all_sync(0xffffffffu, w);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t qa = smem_u32(q_s + qb * kTileBytes), ka = smem_u32(k_s + st * kTileBytes);
      uint64_t da[DH / 16], db[DH / 16];  // built by every lane: warp-uniform values
#pragma unroll
      for (int k16 = 0; k16 < DH / 16; ++k16) {
        da[k16] = desc_kmajor_d(qa, k16);
        db[k16] = desc_kmajor_d(ka, k16);
      }
      const uint32_t dst = tmem + sb * T;
#pragma unroll
      for (int k16 = 0; k16 < DH / 16; ++k16) mma_bf16_ss_elect(dst, da[k16], db[k16], idesc_s, k16 > 0);
      mma_commit_elect(&s_full[sb]);
      mma_commit_elect(&k_empty[st]);
      if (a.j == a.qt) mma_commit_elect(&q_empty[qb]);
      a.advance(sched);
    }
  } else if (warp < 4) {
    // ---------------------------------------------------------------- MMA issuers, output: O += P_g V_g, one warp
    // per softmax group (warp 2: even tiles of the stream, warp 3: odd tiles)
    constexpr uint32_t idesc_o = idesc_bf16_f32(T, DH, false, true);
    const int grp = warp - 2;
    Cursor b;
    b.init(sched, first_tile);
    bool ok = true;
    uint32_t items = 0;  // items this group has taken part in
    while (b.valid && ok) {
      if ((b.g & 1) == grp) {
        const int st = b.g % kVStages;
        const bool first = b.j - b.j0 <= 1;  // the group's first tile of this item: start a fresh accumulator ...
        bool w = mbar_wait(&p_ready[grp], (b.g >> 1) & 1, ctx, 0x1204u) &&
                 mbar_wait(&v_full[st], (b.g / kVStages) & 1, ctx, 0x1205u);
        if (first) {  // ... once the group has read the previous item's result out of it
          if (w) w = mbar_wait(&o_free[grp], (items & 1) ^ 1u, ctx, 0x1206u);
          ++items;
        }
        ok = __all_sync(0xffffffffu, w);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t pa = smem_u32(p_s + grp * 2 * kTileBytes), va = smem_u32(v_s + st * kTileBytes);
        uint64_t da[T / 16], db[T / 16];  // built by every lane: warp-uniform values
#pragma unroll
        for (int k16 = 0; k16 < T / 16; ++k16) {
          da[k16] = desc_p_kmajor(pa, k16);
          db[k16] = desc_rows_as_k(va, k16);
        }
        const uint32_t dst = tmem + kSBufs * T + grp * DH;
#pragma unroll
        for (int k16 = 0; k16 < T / 16; ++k16)
          mma_bf16_ss_elect(dst, da[k16], db[k16], idesc_o, (k16 > 0 || !first) ? 1u : 0u);
        mma_commit_elect(&o_full[grp]);
        mma_commit_elect(&v_empty[st]);
      }
      b.advance(sched);
    }
  } else if (warp >= 4) {
    // ---------------------------------------------------------------- softmax warps
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    const int quarter = warp & 3;            // tensor-memory lane quarter this warp may read
    const int grp = (warp - 4) >> 2;         // this group handles the stream's tiles with (g & 1) == grp
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t t_o = tmem + lane_base + kSBufs * T + grp * DH;  // this group's output accumulator
    uint8_t* p_tile = p_s + grp * 2 * kTileBytes;
    const float f_eval = p.dr.train ? 1.f : p.dr.eval_scale;  // evaluation: P * (1 - p), applied to the final rows
    const uint32_t thr_hi = p.dr.thr16 << 16;

    Cursor c;
    c.init(sched, first_tile);
    bool ok = true;
    float m_ref = 0.f, l = 0.f;  // reference exponent (log2 domain) and sum of 2^(s - m_ref) of this group's tiles
    float m_true = 0.f;          // true running row maximum (log2 domain), only reported
    bool have = false;           // the group holds tiles of the current item
    int pend_g = -1;             // own tile whose P V product may still be running
    uint32_t nd = 0;             // hand-overs (items with at least two tiles) seen so far
    auto wait_pv = [&]() {       // the group's last P V product is complete: accumulator and P buffer are quiet
      if (pend_g < 0) return;
      ok = mbar_wait(&o_full[grp], (pend_g >> 1) & 1, ctx, 0x1302u);
      ok = __all_sync(0xffffffffu, ok);
      tc_fence_after_sync();
      pend_g = -1;
    };

    while (c.valid && ok) {
      const bool mine = (c.g & 1) == grp;
      const int64_t q_row = static_cast<int64_t>(c.qt) * T + row;
      if (c.j == c.j0) have = false;
      if (mine) {
        const int sb = c.g % kSBufs;
        // dropout random words of this thread's row of the tile: independent of the scores, so they are drawn one
        // 32-column chunk ahead of their use (the first chunk while the score MMA may still be running)
        uint32_t rw[2][4][4];  // raw words of the four Philox calls of a 32-column chunk, drawn one chunk ahead
        const uint64_t call0 = ((static_cast<uint64_t>(c.bh) * p.S + q_row) * p.S + static_cast<uint64_t>(c.j) * T) >> 3;
        if (MODE == 1) {
#pragma unroll
          for (int q = 0; q < 4; ++q) philox_rk(rk_s, call0 + q, p.dr.stream_id, rw[0][q]);
        }
        uint4 kb = make_uint4(0u, 0u, 0u, 0u);
        if (MODE == 2)
          kb = __ldg(p.keep_bits + (static_cast<int64_t>(c.bh) * (p.nq * (p.nq + 1) / 2) + c.qt * (c.qt + 1) / 2 + c.j) * T + row);
        const uint32_t keepw[4] = {kb.x, kb.y, kb.z, kb.w};
        ok = mbar_wait(&s_full[sb], (c.g / kSBufs) & 1, ctx, 0x1303u);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
        float s[4][32];
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) tmem_ld_32x32f(tmem + lane_base + sb * T + cc * 32, s[cc]);
        tmem_ld_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_free[sb]);  // the scores are in registers: the buffer may take tile g + 3
        const bool diag = c.j == c.qt;
        if (diag) {  // causal mask: only the diagonal tile has columns beyond the row
#pragma unroll
          for (int cc = 0; cc < 4; ++cc)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (cc * 32 + i > row) s[cc][i] = -INFINITY;
        }
        if (VARLEN) {  // keys before the row's document: columns below rel (any tile may hold a boundary)
          const int rel = __ldg(p.kstart + static_cast<int64_t>(c.bh / p.H) * p.S + q_row) - c.j * T;
          if (__any_sync(0xffffffffu, rel > 0)) {  // (most tiles hold no document boundary for any row of the warp)
#pragma unroll
            for (int cc = 0; cc < 4; ++cc)
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (cc * 32 + i < rel) s[cc][i] = -INFINITY;
          }
        }
        float mp[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // four independent chains of three-input maxima
#pragma unroll
        for (int cc = 0; cc < 4; ++cc)
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
#pragma unroll
            for (int k = 0; k < 4; ++k) mp[k] = max3(mp[k], s[cc][i + 2 * k], s[cc][i + 2 * k + 1]);
          }
        const float mloc = fmaxf(fmaxf(mp[0], mp[1]), fmaxf(mp[2], mp[3])) * p.scale_log2;
        // The reference exponent only moves when the row maximum outgrows it by more than 2^8: probabilities then
        // stay below 256 (exact in fp32, same relative precision in bf16) and the accumulator in tensor memory is
        // rescaled rarely. Any reference gives the same quotient sum(P V) / sum(P).
        bool grow = false;
        if (!have) {
          m_ref = mloc;
          m_true = mloc;
          l = 0.f;
          have = true;
        } else {
          grow = mloc > m_ref + 8.f;
          m_true = fmaxf(m_true, mloc);
        }
        wait_pv();
        if (!ok) break;
        const float alpha = grow ? ex2_approx(m_ref - mloc) : 1.f;
        if (grow) {
          m_ref = mloc;
          l *= alpha;
        }
        // (VARLEN: a row that has met no key yet carries m_ref = -inf; its scores are all -inf too and must give 0)
        const float nm = (VARLEN && m_ref == -INFINITY) ? 0.f : -m_ref;
        const uint64_t sc2 = pack2(p.scale_log2, p.scale_log2), nm2 = pack2(nm, nm);
        uint64_t rp[2] = {0ull, 0ull};  // two packed running sums (four chains)
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          if (MODE == 1 && cc + 1 < 4) {
#pragma unroll
            for (int q = 0; q < 4; ++q) philox_rk(rk_s, call0 + (cc + 1) * 4 + q, p.dr.stream_id, rw[(cc + 1) & 1][q]);
          }
#pragma unroll
          for (int i = 0; i < 32; i += 2) {  // exp2(-inf) = 0 takes care of the masked columns
            float a, b;
            unpack2(fma2(pack2(s[cc][i], s[cc][i + 1]), sc2, nm2), a, b);
            a = ex2_approx(a);
            b = ex2_approx(b);
            rp[(i >> 1) & 1] = add2(rp[(i >> 1) & 1], pack2(a, b));
            if (MODE == 1) {  // 16-bit lanes of word (i % 8) / 2 of call i / 8: low half = even element, high half = odd
              const uint32_t w = rw[cc & 1][i >> 3][(i & 7) >> 1];
              if ((w << 16) < thr_hi) a = 0.f;
              if (w < thr_hi) b = 0.f;
            } else if (MODE == 2) {
              if ((keepw[cc] & (1u << i)) == 0u) a = 0.f;
              if ((keepw[cc] & (2u << i)) == 0u) b = 0.f;
            }
            s[cc][i] = a;
            s[cc][i + 1] = b;
          }
          store_row32_sw128(p_tile, row, cc * 32, s[cc]);
        }
        float rsum;
        {
          float a, b;
          unpack2(add2(rp[0], rp[1]), a, b);
          rsum = a + b;
        }
        if (__any_sync(0xffffffffu, grow)) {  // rare: bring the accumulated rows to the new reference exponent
#pragma unroll
          for (int cc = 0; cc < 2; ++cc) {
            uint32_t t[32];
            tmem_ld_32x32(t_o + cc * 32, t);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) t[i] = __float_as_uint(__uint_as_float(t[i]) * alpha);
            tmem_st_32x32(t_o + cc * 32, t);
          }
          tmem_st_wait();
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_ready[grp]);
        l += rsum;
        pend_g = c.g;
      }
      if (c.j == c.qt) {  // the item ends with this tile: its owner finishes the rows, the other group hands over
        float o[DH];
        if (have) {
          wait_pv();
          if (!ok) break;
#pragma unroll
          for (int cc = 0; cc < 2; ++cc) {
            float t[32];
            tmem_ld_row32(t_o + cc * 32, t);
#pragma unroll
            for (int i = 0; i < 32; ++i) o[cc * 32 + i] = t[i];
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&o_free[grp]);  // the next item may overwrite the accumulator
        }
        if (c.qt > c.j0) {  // (an item of a single tile has nothing to merge)
          if (!mine) {
            ok = mbar_wait(dump_free, (nd & 1) ^ 1u, ctx, 0x1304u);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
#pragma unroll
            for (int i = 0; i < DH; ++i) dump[i * T + row] = o[i];
            dump[DH * T + row] = m_ref;
            dump[(DH + 1) * T + row] = l;
            dump[(DH + 2) * T + row] = m_true;
            __syncwarp();
            if (lane == 0) mbar_arrive(dump_full);
          } else {
            ok = mbar_wait(dump_full, nd & 1, ctx, 0x1305u);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const float m_o = dump[DH * T + row], l_o = dump[(DH + 1) * T + row];
            const float mm = fmaxf(m_ref, m_o);
            float fa = ex2_approx(m_ref - mm), fb = ex2_approx(m_o - mm);
            if (VARLEN) {  // a group that met no key of this row (-inf - -inf is not a number)
              if (m_ref == -INFINITY) fa = 0.f;
              if (m_o == -INFINITY) fb = 0.f;
            }
#pragma unroll
            for (int i = 0; i < DH; ++i) o[i] = o[i] * fa + dump[i * T + row] * fb;
            l = l * fa + l_o * fb;
            m_ref = mm;
            m_true = fmaxf(m_true, dump[(DH + 2) * T + row]);
            __syncwarp();
            if (lane == 0) mbar_arrive(dump_free);
          }
          ++nd;
        }
        if (mine) {
          const bool empty = VARLEN && !(l > 0.f);  // the row attends nothing: zero output, neutral statistics
          const float inv = empty ? 0.f : f_eval / l;
          __nv_bfloat16* dst = out.row(c.bh / p.H, c.bh % p.H, q_row);
#pragma unroll
          for (int c8 = 0; c8 < DH / 8; ++c8) {
            float t[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) t[i] = o[c8 * 8 + i] * inv;
            Elem<__nv_bfloat16>::store_vec(dst + c8 * 8, t);
          }
          const int64_t ri = static_cast<int64_t>(c.bh) * p.S + q_row;
          row_max[ri] = empty ? 0.f : m_true * kLn2;                   // acts0: row maximum of the scaled scores
          row_sum[ri] = empty ? 1.f : l * ex2_approx(m_ref - m_true);  // acts1: sum of exp(score - maximum)
        }
        have = false;
      }
      c.advance(sched);
    }
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

// Keep flags of the attention-probability dropout for one call, computed once and shared by the forward and the
// backward kernel: word c of the uint4 at ((bh * ntri + qt (qt + 1) / 2 + kt) * 128 + row) holds the flags of
// columns 32 c .. 32 c + 31 of row `row` of tile (qt, kt); ntri = nq (nq + 1) / 2. One thread per word.
__global__ void __launch_bounds__(512)
attn_keep_bits_kernel(uint32_t* __restrict__ bits, const AttnDropout dr, int S, int nq) {
  grid_dep_sync();
  __shared__ uint32_t rk_s[20];
  if (threadIdx.x == 0) philox_round_keys(dr.seed, rk_s);
  __syncthreads();
  uint32_t rk[20];  // in registers: the kernel is bound by its integer instructions, keys as plain operands
#pragma unroll
  for (int i = 0; i < 20; ++i) rk[i] = rk_s[i];
  // one block per tile (its position is decoded once), one thread per word: 128 rows x 4 words
  const int ntri = nq * (nq + 1) / 2;
  const int64_t tile = blockIdx.x;  // bh * ntri + tri
  const int64_t bh = tile / ntri;
  const int tri = static_cast<int>(tile % ntri);
  int qt = static_cast<int>((sqrtf(8.f * tri + 1.f) - 1.f) * 0.5f);
  while ((qt + 1) * (qt + 2) / 2 <= tri) ++qt;
  while (qt * (qt + 1) / 2 > tri) --qt;
  const int kt = tri - qt * (qt + 1) / 2;
  const int cc = threadIdx.x & 3, row = threadIdx.x >> 2;
  const uint64_t idx0 = (static_cast<uint64_t>(bh) * S + static_cast<uint64_t>(qt) * T + row) * S +
                        static_cast<uint64_t>(kt) * T + cc * 32;
  // four Philox calls (round keys from the kernel parameters), eight 16-bit lanes each: bit e of a call's byte is set
  // when lane e (low half of word e / 2 for even e, high half for odd e) is >= the threshold
  const uint32_t thr_hi = dr.thr16 << 16;
  uint32_t word = 0;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint32_t w[4];
    philox_rk(rk, (idx0 >> 3) + q, dr.stream_id, w);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      word |= ((w[e] << 16) >= thr_hi ? 1u : 0u) << (8 * q + 2 * e);
      word |= (w[e] >= thr_hi ? 1u : 0u) << (8 * q + 2 * e + 1);
    }
  }
  bits[tile * 512 + threadIdx.x] = word;
}

}  // namespace

size_t attn_keep_bits_bytes(const ptj_attn_shape& sh) {
  const int64_t nq = sh.seq / T;
  return static_cast<size_t>(sh.batch * sh.heads * (nq * (nq + 1) / 2) * T) * 16;
}

int attn_keep_bits_tc(uint32_t* bits, const ptj_attn_shape& sh, const AttnDropout& dr, cudaStream_t st) {
  const int64_t tiles = static_cast<int64_t>(attn_keep_bits_bytes(sh) / 2048);
  launch_k(attn_keep_bits_kernel, static_cast<unsigned>(tiles), 512, 0, st, bits, dr, static_cast<int>(sh.seq),
                                                                      static_cast<int>(sh.seq / T));
  PTJ_CHECK_LAUNCH();
  return PTJ_OK;
}

int attn_fwd_tc(const void* q, const void* k, const void* v, void* o, float* row_max, float* row_sum,
                const uint32_t* keep_bits, const int32_t* row_kstart, const ptj_attn_shape& sh, const AttnDropout& dr,
                cudaStream_t st) {
  CUtensorMap tq, tk, tv;
  if (!make_map(&tq, q, sh, sh.q_strides) || !make_map(&tk, k, sh, sh.k_strides) || !make_map(&tv, v, sh, sh.v_strides))
    return PTJ_ERR_LAUNCH;
  AttnParams p = make_params(sh, dr);
  if (p.fault == nullptr) return PTJ_ERR_DEVICE;
  p.keep_bits = reinterpret_cast<const uint4*>(keep_bits);
  p.kstart = row_kstart;
  const bool masked = dr.train && dr.thr16 != 0u;
  const int mode = !masked ? 0 : (keep_bits != nullptr ? 2 : 1);
  using Kern = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const RowView, float*, float*,
                        const AttnParams, const Sched);
  static const Kern kerns[2][3] = {
      {attn_fwd_ws_kernel<0, false>, attn_fwd_ws_kernel<1, false>, attn_fwd_ws_kernel<2, false>},
      {attn_fwd_ws_kernel<0, true>, attn_fwd_ws_kernel<1, true>, attn_fwd_ws_kernel<2, true>}};
  const Kern kern = kerns[row_kstart != nullptr ? 1 : 0][mode];
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess) {
    (void)cudaGetLastError();
    return PTJ_ERR_LAUNCH;
  }
  Sched s;
  s.nq = p.nq;
  s.BH = p.BH;
  s.total = p.nq * p.BH;
  const int grid = s.total < kNumSMs ? s.total : kNumSMs;
  s.rounds = (s.total + grid - 1) / grid;
  s.bh_magic = static_cast<uint32_t>(((1ull << 32) + s.BH - 1) / s.BH);
  launch_k(kern, grid, kThreads, kSmemBytes, st, tq, tk, tv, make_view(o, sh.o_strides), row_max, row_sum, p, s);
  PTJ_CHECK_LAUNCH();
  return PTJ_OK;
}

}  // namespace ptj
