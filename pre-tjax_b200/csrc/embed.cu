// Token + position embedding forward (gather, scale by sqrt(dim), add positions, dropout) and its backward
// (deterministic segmented scatter into the embedding table, batch-sum into the position table), and the
// deterministic column sum used for bias gradients.
#include "common.cuh"
#include "tc_common.cuh"

namespace ptj {
namespace {

// y[t, :] = dropout(w_emb[ids[t], :] * sqrt(dim) + w_pos[t % seq, :])   (model_triton.py:166-167, 2338-2341)
template <typename TW, typename T>
__global__ void __launch_bounds__(256)
embed_fwd_kernel(const int32_t* __restrict__ ids, const TW* __restrict__ w_emb, const TW* __restrict__ w_pos,
                 T* __restrict__ y, int64_t tokens, int64_t seq, int dim, int64_t vocab, float scale, uint32_t thr,
                 float eval_scale, int train, uint64_t seed, uint32_t stream_id) {
  grid_dep_sync();
  seed = resolve_seed(seed);
  const int64_t total = tokens * dim;
  for (int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x * 4) {
    // dim % 4 == 0 is checked on the host, so the 4 elements share a token
    const int64_t t = i / dim;
    const int c = static_cast<int>(i - t * dim);
    int64_t id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const TW* e = w_emb + id * dim + c;
    const TW* p = w_pos + (t % seq) * dim + c;
    float k[4] = {eval_scale, eval_scale, eval_scale, eval_scale};
    if (train) {  // i is a multiple of 4: these four elements are the low or the high half of one Philox call
      const uint32_t keep = thr != 0u ? dropout_keep_bits8(seed, stream_id, static_cast<uint64_t>(i) >> 3, thr) >> (i & 4) : 0xfu;
#pragma unroll
      for (int j = 0; j < 4; ++j) k[j] = ((keep >> j) & 1u) ? 1.f : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
      Elem<T>::store(y + i + j, (Elem<TW>::load(e + j) * scale + Elem<TW>::load(p + j)) * k[j]);
  }
}

// eight consecutive elements starting at a 16-byte (bf16) / 32-byte (float) aligned address
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) { Elem<__nv_bfloat16>::load_vec(p, v); }
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

// Gradient w.r.t. the position table: d_w_pos[s, c] = sum_b mask * dy[b, s, c]   (model_triton.py:2518)
template <typename T>
__global__ void __launch_bounds__(256)
pos_bwd_kernel(const T* __restrict__ dy, float* __restrict__ d_w_pos, int64_t batch, int64_t seq, int dim,
               uint32_t thr, float eval_scale, int train, uint64_t seed, uint32_t stream_id) {
  grid_dep_sync();
  seed = resolve_seed(seed);
  const int64_t total = seq * dim;  // a multiple of 8 (the host checks dim % 8 == 0)
  const bool masked = train && thr != 0u;
  const float k_all = train ? 1.f : eval_scale;
  // eight consecutive features per thread: one 16-byte (bf16) load and one Philox call per batch row
  for (int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 8; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x * 8) {
    float s[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) s[e] = 0.f;
    for (int64_t b = 0; b < batch; ++b) {
      const int64_t idx = b * total + i;
      float x[8];
      load8(dy + idx, x);
      uint32_t keep = 0xffu;
      if (masked) keep = dropout_keep_bits8(seed, stream_id, static_cast<uint64_t>(idx) >> 3, thr);
#pragma unroll
      for (int e = 0; e < 8; ++e) s[e] += ((keep >> e) & 1u) ? x[e] * k_all : 0.f;
    }
    *reinterpret_cast<float4*>(d_w_pos + i) = make_float4(s[0], s[1], s[2], s[3]);
    *reinterpret_cast<float4*>(d_w_pos + i + 4) = make_float4(s[4], s[5], s[6], s[7]);
  }
}

// Adds rows pos_s[first], pos_s[first + step], ... (< n) of dy (masked, scaled) into acc; lanes run across the
// features, 8 per vector = one Philox call. A block's 8 warps share a batch with (first, step) = (warp, 8); a warp that
// owns a whole run passes (0, 1). Several rows per step: their loads are independent (kept as raw 16-byte
// pieces until they are added, in row order, so the sums do not depend on the grouping).
template <typename T, int NV>
__device__ __forceinline__ void add_rows(const T* __restrict__ dy, const int32_t* pos_s, int n, int dim, int nvec,
                                     bool masked, float k_all, uint64_t seed, uint32_t stream_id, uint32_t thr,
                                     float (&acc)[NV][8], int lane, int first, int step) {
  constexpr int U = sizeof(T) == 2 ? 4 : 2;    // rows per step
  constexpr int PV = sizeof(T) == 2 ? 1 : 2;   // 16-byte pieces per 8-element vector
  for (int r0 = first; r0 < n; r0 += step * U) {
    uint4 raw[U][NV][PV];
    int64_t rows_u[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int r = r0 + step * u;
      rows_u[u] = r < n ? static_cast<int64_t>(pos_s[r]) * dim : -1;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int v = lane + 32 * i;
        if (rows_u[u] >= 0 && v < nvec) {
          const uint4* src = reinterpret_cast<const uint4*>(dy + rows_u[u] + v * 8);
#pragma unroll
          for (int q = 0; q < PV; ++q) raw[u][i][q] = src[q];
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (rows_u[u] < 0) continue;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int v = lane + 32 * i;
        if (v < nvec) {
          float x[8];
          if (sizeof(T) == 2) {
            const uint32_t w[4] = {raw[u][i][0].x, raw[u][i][0].y, raw[u][i][0].z, raw[u][i][0].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              x[2 * e] = __uint_as_float(w[e] << 16);
              x[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
            }
          } else {
#pragma unroll
            for (int q = 0; q < PV; ++q) {
              x[4 * q] = __uint_as_float(raw[u][i][q].x);
              x[4 * q + 1] = __uint_as_float(raw[u][i][q].y);
              x[4 * q + 2] = __uint_as_float(raw[u][i][q].z);
              x[4 * q + 3] = __uint_as_float(raw[u][i][q].w);
            }
          }
          uint32_t keep = 0xffu;
          if (masked) keep = dropout_keep_bits8(seed, stream_id, static_cast<uint64_t>(rows_u[u] + v * 8) >> 3, thr);
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[i][e] += ((keep >> e) & 1u) ? x[e] * k_all : 0.f;
        }
      }
    }
  }
}

constexpr int kHeavyRun = 32;
constexpr int kHeavyCluster = 8;

// Gradient w.r.t. the embedding table (model_triton.py:183-185, 205-213). Token positions arrive stably sorted by
// token id, so the rows of one table row form a run of equal ids. A block looks at kChunk consecutive sorted positions:
// 64 threads mark the run heads among them (both neighbours' ids are two dependent loads, taken for all positions at
// once rather than by one block per position), and each of the 8 warps then sums whole runs on its own - lanes across
// the features, 8 per vector = one Philox call, four rows in flight, rows added in order - and adds the result onto
// the table row. One warp, fixed order, no atomics => every table row is reproducible. Runs longer than kHeavyRun rows
// (a Zipf head makes runs of ~1000) are left to the cluster kernel below.
constexpr int kChunk = 64;

template <typename T, int NV>
__global__ void __launch_bounds__(256, NV <= 4 ? 2 : 1)
embed_bwd_kernel(const T* __restrict__ dy, const int32_t* __restrict__ ids, const int32_t* __restrict__ sorted_pos,
                 float* __restrict__ d_w_emb, int accumulate, int64_t tokens, int dim, int64_t vocab, float scale,
                 uint32_t thr, float eval_scale, int train, uint64_t seed, uint32_t stream_id) {
  grid_dep_sync();
  seed = resolve_seed(seed);
  __shared__ uint32_t head_mask[kChunk / 32];
  __shared__ int32_t pos_w[8][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool masked = train && thr != 0u;
  const float k_all = train ? 1.f : eval_scale;
  const int nvec = dim / 8;  // dim % 8 == 0 is checked on the host
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kChunk;
  if (warp < kChunk / 32) {
    const int64_t j = base + threadIdx.x;
    bool head = false;
    if (j < tokens) {
      const int32_t id = ids[sorted_pos[j]];
      head = (j == 0 || ids[sorted_pos[j - 1]] != id) && id >= 0 && id < vocab &&
             !(j + kHeavyRun < tokens && ids[sorted_pos[j + kHeavyRun]] == id);  // (long runs: the cluster kernel)
    }
    const uint32_t m = __ballot_sync(0xffffffffu, head);
    if (lane == 0) head_mask[warp] = m;
  }
  __syncthreads();
  const uint32_t m0 = head_mask[0], m1 = head_mask[1];
  const int n0 = __popc(m0), nheads = n0 + __popc(m1);
  int32_t* my_pos = pos_w[warp];
  for (int h = warp; h < nheads; h += 8) {
    const int off = h < n0 ? static_cast<int>(__fns(m0, 0, h + 1)) : 32 + static_cast<int>(__fns(m1, 0, h - n0 + 1));
    const int64_t j = base + off;
    const int32_t id = ids[sorted_pos[j]];
    float acc[NV][8];
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[i][e] = 0.f;
    for (int64_t w0 = j;; w0 += 32) {  // the run, 32 positions at a time (matches are a prefix of each window)
      const int64_t q = w0 + lane;
      int32_t pos = -1;
      if (q < tokens) {
        pos = sorted_pos[q];
        if (ids[pos] != id) pos = -1;
      }
      __syncwarp();  // the previous window has been consumed
      my_pos[lane] = pos;
      const int n = __popc(__ballot_sync(0xffffffffu, pos >= 0));
      __syncwarp();
      add_rows<T, NV>(dy, my_pos, n, dim, nvec, masked, k_all, seed, stream_id, thr, acc, lane, 0, 1);
      if (n < 32) break;
    }
    float* out = d_w_emb + static_cast<int64_t>(id) * dim;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = lane + 32 * i;
      if (v < nvec) {
        float4* o4 = reinterpret_cast<float4*>(out + v * 8);
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
        if (accumulate) {
          a = o4[0];
          b = o4[1];
        }
        a.x += acc[i][0] * scale; a.y += acc[i][1] * scale; a.z += acc[i][2] * scale; a.w += acc[i][3] * scale;
        b.x += acc[i][4] * scale; b.y += acc[i][5] * scale; b.z += acc[i][6] * scale; b.w += acc[i][7] * scale;
        o4[0] = a;
        o4[1] = b;
      }
    }
  }
}

// The long runs (a Zipf head: the most frequent token of a GPT-2 batch of 8192 tokens occurs about 1 100 times) would
// each keep one warp busy for 100 us and more while the rest of the GPU idles. Here a cluster of kHeavyCluster blocks shares
// one run: block r of the cluster sums the r-th slice of the run's rows, the slices' sums meet in block 0 through
// distributed shared memory and are added in slice order (fixed order, no atomics => reproducible).
// Work assignment without any helper tensor: cluster k looks at sorted position a = k * kHeavyRun. A run longer than
// kHeavyRun contains at least one multiple of kHeavyRun; the cluster at the FIRST such multiple owns the run. Every
// block of a cluster evaluates the same conditions, so a cluster leaves or stays as a whole.
template <typename T, int NV>
__global__ void __launch_bounds__(256, NV <= 4 ? 2 : 1)
embed_bwd_heavy_kernel(const T* __restrict__ dy, const int32_t* __restrict__ ids,
                       const int32_t* __restrict__ sorted_pos, float* __restrict__ d_w_emb, int accumulate,
                       int64_t tokens, int dim, int64_t vocab, float scale, uint32_t thr, float eval_scale, int train,
                       uint64_t seed, uint32_t stream_id) {
  grid_dep_sync();
  seed = resolve_seed(seed);
  extern __shared__ float part[];  // [8][dim] per-warp sums, then [dim] this block's sum
  __shared__ int32_t pos_s[256];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const unsigned rank = tc::cluster_ctarank();
  const int64_t a = static_cast<int64_t>(blockIdx.x) * kHeavyRun;
  if (a >= tokens) return;
  const int32_t id = ids[sorted_pos[a]];
  if (id < 0 || id >= vocab) return;
  if (a >= kHeavyRun && ids[sorted_pos[a - kHeavyRun]] == id) return;  // an earlier multiple lies in the same run
  // head of the run: the matches among positions a, a - 1, ..., a - kHeavyRun + 1 are a prefix (ids are sorted)
  const bool back = tid < kHeavyRun && a - tid >= 0 && ids[sorted_pos[a - tid]] == id;
  const int64_t head = a - (__syncthreads_count(back) - 1);
  if (head + kHeavyRun >= tokens || ids[sorted_pos[head + kHeavyRun]] != id) return;  // a short run: the other kernel's
  // end of the run: probes every 32 positions, then the 32 positions after the last probe that matched
  int64_t inside = head + kHeavyRun;
  for (;;) {
    const int64_t q = inside + (tid + 1) * 32;
    const int c = __syncthreads_count(q < tokens && ids[sorted_pos[q]] == id);
    inside += static_cast<int64_t>(c) * 32;
    if (c < 256) break;
  }
  const int64_t qf = inside + 1 + tid;
  const int64_t end = inside + 1 + __syncthreads_count(tid < 32 && qf < tokens && ids[sorted_pos[qf]] == id);
  const int64_t len = end - head;
  const int64_t s0 = head + len * rank / kHeavyCluster, s1 = head + len * (rank + 1) / kHeavyCluster;

  const bool masked = train && thr != 0u;
  const float k_all = train ? 1.f : eval_scale;
  const int nvec = dim / 8;
  float acc[NV][8];
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[i][e] = 0.f;
  for (int64_t base = s0; base < s1; base += 256) {
    const int64_t q = base + tid;
    __syncthreads();  // previous batch fully consumed
    pos_s[tid] = q < s1 ? sorted_pos[q] : -1;
    __syncthreads();
    const int n = static_cast<int>(s1 - base < 256 ? s1 - base : 256);
    add_rows<T, NV>(dy, pos_s, n, dim, nvec, masked, k_all, seed, stream_id, thr, acc, lane, warp, 8);
  }
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = lane + 32 * i;
    if (v < nvec) {
#pragma unroll
      for (int e = 0; e < 8; ++e) part[warp * dim + v * 8 + e] = acc[i][e];
    }
  }
  __syncthreads();
  float* mine = part + 8 * dim;  // this block's slice sum, warps added in order
  for (int c = tid; c < dim; c += blockDim.x) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += part[w * dim + c];
    mine[c] = t;
  }
  tc::cluster_sync_all();  // every block's slice sum is in its shared memory
  if (rank == 0) {
    float* out = d_w_emb + static_cast<int64_t>(id) * dim;
    for (int c = tid; c < dim; c += blockDim.x) {
      float t = 0.f;
#pragma unroll
      for (int r = 0; r < kHeavyCluster; ++r) {
        float v;
        asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(tc::mapa_shared(tc::smem_u32(mine + c), r)));
        t += v;
      }
      out[c] = (accumulate ? out[c] : 0.f) + t * scale;
    }
  }
  tc::cluster_sync_all();  // nobody leaves (and frees its shared memory) before block 0 has read it
}

// rows of the table that no token hit are zeroed when not accumulating
__global__ void zero_kernel(float* __restrict__ p, int64_t n) {
  grid_dep_sync();
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    p[i] = 0.f;
}

// stage 1: block (bx, by) sums rows [by*chunk, (by+1)*chunk) of the 16-byte column groups bx*128 + tid
// (VEC = true) or of single columns (VEC = false, any alignment).
template <typename T, bool VEC>
__global__ void __launch_bounds__(128)
colsum_stage1_kernel(const T* __restrict__ x, float* __restrict__ partial, int64_t rows, int64_t cols, int64_t ld,
                     int64_t chunk) {
  grid_dep_sync();
  constexpr int V = VEC ? Elem<T>::kVec : 1;
  const int64_t g = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;  // column group
  const int64_t c0 = g * V;
  if (c0 >= cols) return;
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * chunk;
  const int64_t r1 = r0 + chunk < rows ? r0 + chunk : rows;
  float s[V];
#pragma unroll
  for (int j = 0; j < V; ++j) s[j] = 0.f;
#pragma unroll 4
  for (int64_t r = r0; r < r1; ++r) {
    if (VEC) {
      float v[Elem<T>::kVec];
      Elem<T>::load_vec(x + r * ld + c0, v);  // may read padding columns (ld is a multiple of the vector), never writes them
#pragma unroll
      for (int j = 0; j < V; ++j) s[j] += v[j];
    } else {
      s[0] += Elem<T>::load(x + r * ld + c0);
    }
  }
  float* out = partial + static_cast<int64_t>(blockIdx.y) * cols;
#pragma unroll
  for (int j = 0; j < V; ++j)
    if (c0 + j < cols) out[c0 + j] = s[j];
}
// stage 1, vector path: a block of 8 warps owns 32 column groups of 16 bytes (a warp reads 512 contiguous bytes of a
// row) and one chunk of rows; warp w takes rows r0 + w, r0 + w + 8, ...; the eight per-warp sums are added in warp
// order through shared memory, so the result depends only on the shapes.
template <typename T>
__global__ void __launch_bounds__(256)
colsum_stage1_rows_kernel(const T* __restrict__ x, float* __restrict__ partial, int64_t rows, int64_t cols, int64_t ld,
                          int64_t chunk) {
  grid_dep_sync();
  constexpr int V = Elem<T>::kVec;
  __shared__ float red[8][32][V + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t c0 = (static_cast<int64_t>(blockIdx.x) * 32 + lane) * V;
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * chunk;
  const int64_t r1 = r0 + chunk < rows ? r0 + chunk : rows;
  float s[V];
#pragma unroll
  for (int j = 0; j < V; ++j) s[j] = 0.f;
  if (c0 < cols) {
#pragma unroll 4
    for (int64_t r = r0 + warp; r < r1; r += 8) {
      float v[V];
      Elem<T>::load_vec(x + r * ld + c0, v);  // may read padding columns (ld is a multiple of the vector), never writes them
#pragma unroll
      for (int j = 0; j < V; ++j) s[j] += v[j];
    }
  }
#pragma unroll
  for (int j = 0; j < V; ++j) red[warp][lane][j] = s[j];
  __syncthreads();
  // 32 x V sums to write: thread t takes element t (and t + 256, ...) and adds the eight warps in order
  float* out = partial + static_cast<int64_t>(blockIdx.y) * cols;
  for (int e = threadIdx.x; e < 32 * V; e += 256) {
    const int g = e / V, j = e - g * V;
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += red[w][g][j];
    const int64_t c = (static_cast<int64_t>(blockIdx.x) * 32 + g) * V + j;
    if (c < cols) out[c] = t;
  }
}
// The same walk with the GELU backward folded in: dx = dy * gelu'(x) is written and the column sums of dx AS STORED
// (rounded to T) are accumulated, i.e. one pass gives the FFN's hidden gradient and its first bias gradient
// (t_gelu_bkwd2 followed by the db of t_linear_bkwd2_p in the reference, model_triton.py:296-304, 423-434).
// Needs 16-byte aligned rows and cols a multiple of the vector; dx may alias dy.
template <typename T>
__global__ void __launch_bounds__(256)
gelu_bwd_colsum_stage1_kernel(const T* dy, const T* __restrict__ x, T* dx, float* __restrict__ partial, int64_t rows,
                              int64_t cols, int64_t ld, int64_t chunk) {
  grid_dep_sync();
  constexpr int V = Elem<T>::kVec;
  constexpr bool kFast = sizeof(T) == 2;
  __shared__ float red[8][32][V + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t c0 = (static_cast<int64_t>(blockIdx.x) * 32 + lane) * V;
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * chunk;
  const int64_t r1 = r0 + chunk < rows ? r0 + chunk : rows;
  float s[V];
#pragma unroll
  for (int j = 0; j < V; ++j) s[j] = 0.f;
  if (c0 < cols) {
#pragma unroll 4
    for (int64_t r = r0 + warp; r < r1; r += 8) {
      float g[V], v[V];
      Elem<T>::load_vec(dy + r * ld + c0, g);
      Elem<T>::load_vec(x + r * ld + c0, v);
#pragma unroll
      for (int j = 0; j < V; ++j) {
        g[j] = Elem<T>::round(g[j] * gelu_tanh_grad<kFast>(v[j]));
        s[j] += g[j];
      }
      Elem<T>::store_vec(dx + r * ld + c0, g);
    }
  }
#pragma unroll
  for (int j = 0; j < V; ++j) red[warp][lane][j] = s[j];
  __syncthreads();
  float* out = partial + static_cast<int64_t>(blockIdx.y) * cols;
  for (int e = threadIdx.x; e < 32 * V; e += 256) {
    const int gi = e / V, j = e - gi * V;
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += red[w][gi][j];
    const int64_t c = (static_cast<int64_t>(blockIdx.x) * 32 + gi) * V + j;
    if (c < cols) out[c] = t;
  }
}
// stage 2: a block owns 32 columns; its 8 warps sum strided subsets of the chunk rows, added in warp order.
__global__ void __launch_bounds__(256)
colsum_stage2_kernel(const float* __restrict__ partial, float* __restrict__ out, int64_t cols, int nchunks) {
  grid_dep_sync();
  __shared__ float red[8][33];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t c = static_cast<int64_t>(blockIdx.x) * 32 + lane;
  float s = 0.f;
  if (c < cols)
    for (int k = warp; k < nchunks; k += 8) s += partial[static_cast<int64_t>(k) * cols + c];
  red[warp][lane] = s;
  __syncthreads();
  if (warp == 0 && c < cols) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += red[w][lane];
    out[c] = t;
  }
}

// Narrow matrices (the hidden-size bias gradients) split the rows of a chunk over a block's warps; wide ones (the
// vocabulary) have enough columns to fill the machine with one thread per column group.
inline bool colsum_split_rows(int64_t cols) { return cols <= 8192; }
inline int colsum_chunks(int64_t rows, int64_t cols) {
  // enough row chunks to fill the machine (about 8 blocks per SM), at least 32 rows per chunk
  const int64_t strips = colsum_split_rows(cols) ? ceil_div(ceil_div(cols, 4), 32) : ceil_div(ceil_div(cols, 8), 128);
  int64_t want = ceil_div(static_cast<int64_t>(kNumSMs) * 8, strips);
  const int64_t max_chunks = ceil_div(rows, 32);
  if (want > max_chunks) want = max_chunks;
  if (want > 1024) want = 1024;
  if (want < 1) want = 1;
  return static_cast<int>(want);
}

inline int flat_grid(int64_t work, int per_block) {
  int64_t b = ceil_div(work, per_block);
  const int64_t cap = static_cast<int64_t>(kNumSMs) * 8;
  if (b < 1) b = 1;
  return static_cast<int>(b < cap ? b : cap);
}

template <typename T>
int launch_embed_bwd(const void* dy, const int32_t* ids, const int32_t* sorted_pos, float* d_w_emb, int64_t tokens,
                     int dim, int64_t vocab, float scale, uint32_t thr, float eval_scale, int train, uint64_t seed,
                     uint32_t stream_id, int grid, cudaStream_t st) {
  const int nv = (dim / 8 + 31) / 32;
#define PTJ_EMB(NV)                                                                                              \
  {                                                                                                              \
    launch_k(embed_bwd_kernel<T, NV>, grid, 256, 0, st, static_cast<const T*>(dy), ids, sorted_pos, d_w_emb, 1, tokens, \
                                                     dim, vocab, scale, thr, eval_scale, train, seed, stream_id); \
  }
  if (nv <= 1) PTJ_EMB(1) else if (nv <= 2) PTJ_EMB(2) else if (nv <= 4) PTJ_EMB(4) else if (nv <= 8) PTJ_EMB(8) else PTJ_EMB(16)
#undef PTJ_EMB
  PTJ_CHECK_LAUNCH();
  if (tokens <= kHeavyRun) return PTJ_OK;  // no run can be longer than kHeavyRun
  // the long runs: one cluster of kHeavyCluster blocks per multiple of kHeavyRun among the sorted positions
  const size_t smem_h = static_cast<size_t>(9) * dim * sizeof(float);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(ceil_div(tokens, kHeavyRun)), kHeavyCluster);
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = smem_h;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = kHeavyCluster;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
#define PTJ_EMB_H(NV)                                                                                                \
  {                                                                                                                  \
    if (smem_h > 48 * 1024)                                                                                          \
      cudaFuncSetAttribute(embed_bwd_heavy_kernel<T, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_h); \
    (void)cudaLaunchKernelEx(&cfg, embed_bwd_heavy_kernel<T, NV>, static_cast<const T*>(dy), ids, sorted_pos, d_w_emb, 1, \
                             tokens, dim, vocab, scale, thr, eval_scale, train, seed, stream_id);                   \
  }
  if (nv <= 1) PTJ_EMB_H(1) else if (nv <= 2) PTJ_EMB_H(2) else if (nv <= 4) PTJ_EMB_H(4) else if (nv <= 8) PTJ_EMB_H(8) else PTJ_EMB_H(16)
#undef PTJ_EMB_H
  PTJ_CHECK_LAUNCH();
  return PTJ_OK;
}

}  // namespace
}  // namespace ptj

using namespace ptj;

extern "C" int ptj_embed_fwd(const int32_t* ids, const void* w_emb, const void* w_pos, void* y, int64_t batch,
                             int64_t seq, int64_t dim, int64_t vocab, float p, int train, uint64_t seed,
                             uint32_t stream_id, int wdtype, int dtype, void* stream) {
  if (batch < 0 || seq < 1 || dim < 4 || dim % 4 != 0 || vocab < 1 || !(p >= 0.f && p <= 1.f)) return PTJ_ERR_BAD_SHAPE;
  if (batch == 0) return PTJ_OK;
  if (!ids || !w_emb || !w_pos || !y) return PTJ_ERR_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t tokens = batch * seq;
  const int grid = flat_grid(tokens * dim / 4, 256);
  const float scale = sqrtf(static_cast<float>(dim));
  const uint32_t thr = dropout_threshold16(p);
#define PTJ_EMBED(TW, T)                                                                                      \
  launch_k(embed_fwd_kernel<TW, T>, grid, 256, 0, st, ids, static_cast<const TW*>(w_emb), static_cast<const TW*>(w_pos), \
                                                static_cast<T*>(y), tokens, seq, (int)dim, vocab, scale, thr,  \
                                                1.f - p, train, seed, stream_id)
  if (wdtype == PTJ_F32 && dtype == PTJ_F32) PTJ_EMBED(float, float);
  else if (wdtype == PTJ_F32 && dtype == PTJ_BF16) PTJ_EMBED(float, __nv_bfloat16);
  else if (wdtype == PTJ_BF16 && dtype == PTJ_BF16) PTJ_EMBED(__nv_bfloat16, __nv_bfloat16);
  else return PTJ_ERR_DTYPE;
#undef PTJ_EMBED
  PTJ_CHECK_LAUNCH();
  return PTJ_OK;
}

extern "C" int ptj_embed_bwd(const void* dy, const int32_t* ids, const int32_t* sorted_pos, float* d_w_emb,
                             float* d_w_pos, int accumulate, int64_t batch, int64_t seq, int64_t dim, int64_t vocab,
                             float p, int train, uint64_t seed, uint32_t stream_id, int dtype, void* stream) {
  if (batch < 1 || seq < 1 || dim < 8 || dim % 8 != 0 || dim > 4096 || vocab < 1 || !(p >= 0.f && p <= 1.f))
    return PTJ_ERR_BAD_SHAPE;
  if (batch * seq > 0x7fffffffLL) return PTJ_ERR_BAD_SHAPE;
  if (!dy || !ids || !sorted_pos || !d_w_emb || !d_w_pos) return PTJ_ERR_BAD_SHAPE;
  if (!aligned16(dy)) return PTJ_ERR_MISALIGNED;
  if (dtype != PTJ_F32 && dtype != PTJ_BF16) return PTJ_ERR_DTYPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t tokens = batch * seq;
  const float scale = sqrtf(static_cast<float>(dim));
  const uint32_t thr = dropout_threshold16(p);
  if (!accumulate) {
    launch_k(zero_kernel, flat_grid(vocab * dim, 256 * 4), 256, 0, st, d_w_emb, vocab * dim);
    PTJ_CHECK_LAUNCH();
  }
  if (!aligned16(d_w_emb)) return PTJ_ERR_MISALIGNED;
  const int grid_e = static_cast<int>(ceil_div(tokens, kChunk));  // one block per kChunk sorted positions
  if (!aligned16(d_w_pos)) return PTJ_ERR_MISALIGNED;
  const int grid_p = flat_grid(seq * dim / 8, 256);
  if (dtype == PTJ_F32) {
    if (launch_embed_bwd<float>(dy, ids, sorted_pos, d_w_emb, tokens, (int)dim, vocab, scale, thr, 1.f - p, train, seed,
                                stream_id, grid_e, st) != PTJ_OK)
      return PTJ_ERR_LAUNCH;
    PTJ_CHECK_LAUNCH();
    launch_k(pos_bwd_kernel<float>, grid_p, 256, 0, st, static_cast<const float*>(dy), d_w_pos, batch, seq, (int)dim, thr,
                                                  1.f - p, train, seed, stream_id);
  } else {
    if (launch_embed_bwd<__nv_bfloat16>(dy, ids, sorted_pos, d_w_emb, tokens, (int)dim, vocab, scale, thr, 1.f - p, train,
                                        seed, stream_id, grid_e, st) != PTJ_OK)
      return PTJ_ERR_LAUNCH;
    PTJ_CHECK_LAUNCH();
    launch_k(pos_bwd_kernel<__nv_bfloat16>, grid_p, 256, 0, st, static_cast<const __nv_bfloat16*>(dy), d_w_pos, batch, seq,
                                                          (int)dim, thr, 1.f - p, train, seed, stream_id);
  }
  PTJ_CHECK_LAUNCH();
  return PTJ_OK;
}

extern "C" size_t ptj_colsum_scratch_floats(int64_t rows, int64_t cols) {
  if (rows <= 0 || cols <= 0) return 0;
  return static_cast<size_t>(colsum_chunks(rows, cols)) * static_cast<size_t>(cols);
}

extern "C" int ptj_colsum(const void* x, float* out, float* scratch, size_t scratch_floats, int64_t rows,
                          int64_t cols, int64_t ld, int dtype, void* stream) {
  if (rows < 1 || cols < 1 || ld < cols) return PTJ_ERR_BAD_SHAPE;
  if (!x || !out) return PTJ_ERR_BAD_SHAPE;
  if (!scratch || scratch_floats < ptj_colsum_scratch_floats(rows, cols)) return PTJ_ERR_WORKSPACE;
  if (dtype != PTJ_F32 && dtype != PTJ_BF16) return PTJ_ERR_DTYPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int nchunks = colsum_chunks(rows, cols);
  const int64_t chunk = ceil_div(rows, nchunks);
  const int V = dtype == PTJ_F32 ? 4 : 8;
  const bool vec = aligned16(x) && ld % V == 0 && ceil_div(cols, V) * V <= ld;
  const int64_t groups = vec ? ceil_div(cols, V) : cols;
  dim3 grid(static_cast<unsigned>(ceil_div(groups, 128)), static_cast<unsigned>(nchunks));
  dim3 grid_rows(static_cast<unsigned>(ceil_div(groups, 32)), static_cast<unsigned>(nchunks));
  if (dtype == PTJ_F32) {
    if (vec && colsum_split_rows(cols)) launch_k(colsum_stage1_rows_kernel<float>, grid_rows, 256, 0, st, static_cast<const float*>(x), scratch, rows, cols, ld, chunk);
    else if (vec) launch_k(colsum_stage1_kernel<float, true>, grid, 128, 0, st, static_cast<const float*>(x), scratch, rows, cols, ld, chunk);
    else launch_k(colsum_stage1_kernel<float, false>, grid, 128, 0, st, static_cast<const float*>(x), scratch, rows, cols, ld, chunk);
  } else {
    if (vec && colsum_split_rows(cols)) launch_k(colsum_stage1_rows_kernel<__nv_bfloat16>, grid_rows, 256, 0, st, static_cast<const __nv_bfloat16*>(x), scratch, rows, cols, ld, chunk);
    else if (vec) launch_k(colsum_stage1_kernel<__nv_bfloat16, true>, grid, 128, 0, st, static_cast<const __nv_bfloat16*>(x), scratch, rows, cols, ld, chunk);
    else launch_k(colsum_stage1_kernel<__nv_bfloat16, false>, grid, 128, 0, st, static_cast<const __nv_bfloat16*>(x), scratch, rows, cols, ld, chunk);
  }
  PTJ_CHECK_LAUNCH();
  launch_k(colsum_stage2_kernel, static_cast<unsigned>(ceil_div(cols, 32)), 256, 0, st, scratch, out, cols, nchunks);
  PTJ_CHECK_LAUNCH();
  return PTJ_OK;
}

extern "C" int ptj_gelu_bwd_colsum(const void* dy, const void* x_preact, void* dx, float* colsum, float* scratch,
                                   size_t scratch_floats, int64_t rows, int64_t cols, int64_t ld, int dtype,
                                   void* stream) {
  if (rows < 1 || cols < 1 || ld < cols) return PTJ_ERR_BAD_SHAPE;
  if (!dy || !x_preact || !dx || !colsum) return PTJ_ERR_BAD_SHAPE;
  if (!scratch || scratch_floats < ptj_colsum_scratch_floats(rows, cols)) return PTJ_ERR_WORKSPACE;
  if (dtype != PTJ_F32 && dtype != PTJ_BF16) return PTJ_ERR_DTYPE;
  const int V = dtype == PTJ_F32 ? 4 : 8;
  if (!aligned16(dy) || !aligned16(x_preact) || !aligned16(dx) || ld % V != 0 || cols % V != 0) return PTJ_ERR_UNSUPPORTED;
  if (!colsum_split_rows(cols)) return PTJ_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int nchunks = colsum_chunks(rows, cols);
  const int64_t chunk = ceil_div(rows, nchunks);
  dim3 grid(static_cast<unsigned>(ceil_div(cols / V, 32)), static_cast<unsigned>(nchunks));
  if (dtype == PTJ_F32)
    launch_k(gelu_bwd_colsum_stage1_kernel<float>, grid, 256, 0, st, static_cast<const float*>(dy),
             static_cast<const float*>(x_preact), static_cast<float*>(dx), scratch, rows, cols, ld, chunk);
  else
    launch_k(gelu_bwd_colsum_stage1_kernel<__nv_bfloat16>, grid, 256, 0, st, static_cast<const __nv_bfloat16*>(dy),
             static_cast<const __nv_bfloat16*>(x_preact), static_cast<__nv_bfloat16*>(dx), scratch, rows, cols, ld, chunk);
  PTJ_CHECK_LAUNCH();
  launch_k(colsum_stage2_kernel, static_cast<unsigned>(ceil_div(cols, 32)), 256, 0, st, scratch, colsum, cols, nchunks);
  PTJ_CHECK_LAUNCH();
  return PTJ_OK;
}
