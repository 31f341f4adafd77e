// Host-side runtime shared by the tensor-core kernels: the device fault word, the driver entry point that encodes
// TMA tensor maps, library-level bookkeeping entry points.
#include <atomic>
#include <mutex>

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

static bool make_tmap_bf16_sw(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                             const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn enc = get_encode_tiled();
  if (enc == nullptr) return false;
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
  return r == CUDA_SUCCESS;
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
