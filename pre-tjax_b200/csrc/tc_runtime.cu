// Host-side runtime shared by the tensor-core kernels: the device fault word, the driver entry point that encodes
// TMA tensor maps, library-level bookkeeping entry points.
#include <atomic>
#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "tc_common.cuh"
#include "tc_runtime.h"

namespace ptj {

static std::atomic<int64_t> g_launches{0};
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

namespace tc {

__device__ unsigned int g_fault_word;

unsigned int* fault_word() {
  constexpr int kMaxDev = 64;
  static unsigned int* cache[kMaxDev] = {};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (cache[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_fault_word) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    cache[dev] = static_cast<unsigned int*>(p);
  }
  return cache[dev];
}

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    else
      (void)cudaGetLastError();
  });
  return fn;
}

// Encoded tensor maps are cached per host thread, keyed by everything that goes into the encoding (base address,
// extents, strides, box, swizzle): a training step issues the same few hundred (tensor, box) combinations every
// iteration, and cuTensorMapEncodeTiled costs more than the rest of a launch's host work. A map is a pure function
// of its key (it holds no reference to the allocation's contents), so a stale entry can only be hit by a request that
// would encode the identical map again. Direct-mapped, 2048 entries per thread.
namespace {
struct TmapKey {
  const void* base;
  uint64_t dims[4];
  uint64_t strides[3];
  uint32_t box[4];
  uint32_t rank_swizzle;
  uint32_t pad;  // keeps the struct free of padding bytes, so memcmp compares only fields
  bool operator==(const TmapKey& o) const { return std::memcmp(this, &o, sizeof(TmapKey)) == 0; }
};
static_assert(sizeof(TmapKey) == 8 + 32 + 24 + 16 + 8, "TmapKey must have no padding");
struct TmapEntry {
  TmapKey key;
  bool valid;
  CUtensorMap map;
};
constexpr size_t kTmapCacheEntries = 2048;
inline uint64_t mix64(uint64_t h, uint64_t v) {
  h ^= v + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
  return h;
}
}  // namespace

static bool make_tmap_bf16_sw(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                             const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn enc = get_encode_tiled();
  if (enc == nullptr || rank < 1 || rank > 4) return false;
  TmapKey key;
  std::memset(&key, 0, sizeof(key));
  key.base = base;
  key.rank_swizzle = static_cast<uint32_t>(rank) | (static_cast<uint32_t>(swizzle) << 8);
  uint64_t h = mix64(reinterpret_cast<uint64_t>(base), key.rank_swizzle);
  for (int i = 0; i < rank; ++i) {
    key.dims[i] = dims[i];
    key.box[i] = box[i];
    h = mix64(h, dims[i] * 0x100000001B3ull + box[i]);
    if (i + 1 < rank) {
      key.strides[i] = strides_bytes[i];
      h = mix64(h, strides_bytes[i]);
    }
  }
  thread_local std::vector<TmapEntry> cache;
  if (cache.empty()) cache.resize(kTmapCacheEntries);
  TmapEntry& slot = cache[(h ^ (h >> 29)) % kTmapCacheEntries];
  if (slot.valid && slot.key == key) {
    *out = slot.map;
    return true;
  }
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (i + 1 < rank) gstr[i] = strides_bytes[i];
  }
  const CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, static_cast<cuuint32_t>(rank), const_cast<void*>(base),
                         gdim, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  slot.key = key;
  slot.map = *out;
  slot.valid = true;
  return true;
}

bool make_tmap_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                    const uint32_t* box) {
  return make_tmap_bf16_sw(out, base, rank, dims, strides_bytes, box, CU_TENSOR_MAP_SWIZZLE_128B);
}
bool make_tmap_bf16_sw64(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                         const uint64_t* strides_bytes, const uint32_t* box) {
  return make_tmap_bf16_sw(out, base, rank, dims, strides_bytes, box, CU_TENSOR_MAP_SWIZZLE_64B);
}

}  // namespace tc
}  // namespace ptj

using namespace ptj;

extern "C" int ptj_version(void) { return 100; }

extern "C" const char* ptj_status_string(int status) {
  switch (status) {
    case PTJ_OK: return "ok";
    case PTJ_ERR_BAD_SHAPE: return "bad shape or null pointer";
    case PTJ_ERR_MISALIGNED: return "pointer or leading dimension not aligned as required";
    case PTJ_ERR_DTYPE: return "unsupported dtype";
    case PTJ_ERR_LAUNCH: return "CUDA launch or driver call failed";
    case PTJ_ERR_WORKSPACE: return "scratch buffer missing or too small";
    case PTJ_ERR_UNSUPPORTED: return "unsupported combination of options";
    case PTJ_ERR_DEVICE: return "device is not sm_100 or a driver entry point is missing";
    case PTJ_ERR_TIMEOUT: return "a bounded wait inside a kernel ran out";
    case PTJ_ERR_TOO_LARGE: return "size exceeds the fixed capacity of the no-allocation entry point";
    default: return "unknown status";
  }
}

extern "C" int ptj_device_check(void) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) { (void)cudaGetLastError(); return PTJ_ERR_DEVICE; }
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return PTJ_ERR_DEVICE;
  }
  return major == 10 ? PTJ_OK : PTJ_ERR_DEVICE;
}

extern "C" int64_t ptj_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

extern "C" int ptj_last_kernel_fault(void* stream, unsigned int* code_out) {
  if (code_out == nullptr) return PTJ_ERR_BAD_SHAPE;
  unsigned int* w = tc::fault_word();
  if (w == nullptr) return PTJ_ERR_DEVICE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned int v = 0;
  if (cudaMemcpyAsync(&v, w, sizeof(v), cudaMemcpyDeviceToHost, st) != cudaSuccess) return PTJ_ERR_LAUNCH;
  if (cudaStreamSynchronize(st) != cudaSuccess) return PTJ_ERR_LAUNCH;
  if (v != 0) cudaMemsetAsync(w, 0, sizeof(v), st);
  *code_out = v;
  return PTJ_OK;
}
