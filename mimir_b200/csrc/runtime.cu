// Host runtime of libmimir_b200: error word, launch counter, tensor-map
// encoding through the driver entry point (no link-time libcuda dependency).
//
// The error word follows the reference's design (backend/cuda/cuda_linux.go:
// 163-170): one word per device in host-mapped pinned memory, OR-ed by kernels,
// read by the host after a synchronisation, never a trap.
#include "runtime.h"

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace mimir {

namespace {
constexpr int kMaxDevices = 64;
unsigned* g_err_host[kMaxDevices] = {};
unsigned* g_err_dev[kMaxDevices] = {};
int g_sm_count[kMaxDevices] = {};
std::mutex g_mu;
std::atomic<long long> g_launches{0};
thread_local char g_last_error[512] = "";

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

int current_device() {
  int d = 0;
  cudaGetDevice(&d);
  return d < 0 || d >= kMaxDevices ? 0 : d;
}

void ensure_device(int d) {
  if (g_err_dev[d]) return;
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_err_dev[d]) return;
  unsigned* h = nullptr;
  unsigned* dp = nullptr;
  if (cudaHostAlloc(reinterpret_cast<void**>(&h), sizeof(unsigned) * 16, cudaHostAllocMapped) !=
      cudaSuccess)
    return;
  memset(h, 0, sizeof(unsigned) * 16);
  cudaHostGetDevicePointer(reinterpret_cast<void**>(&dp), h, 0);
  cudaDeviceProp prop;
  cudaGetDeviceProperties(&prop, d);
  g_sm_count[d] = prop.multiProcessorCount;
  g_err_host[d] = h;
  g_err_dev[d] = dp;
}
}  // namespace

unsigned* error_word_dev() {
  int d = current_device();
  ensure_device(d);
  return g_err_dev[d];
}

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int sm_count() {
  int d = current_device();
  ensure_device(d);
  return g_sm_count[d] > 0 ? g_sm_count[d] : 148;
}

int refuse(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return -1;
}

int encode_tmap(CUtensorMap* out, const void* base, int elem_bytes, int rank, const uint64_t* dims,
                const uint64_t* strides_bytes, const uint32_t* box, int swizzle) {
  if (!g_encode) {
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_encode) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult q;
      if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) !=
              cudaSuccess ||
          !fn)
        return refuse("cuTensorMapEncodeTiled entry point not found");
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0)
    return refuse("tensor map base %p is not 16-byte aligned", base);
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t gbox[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
    if (i > 0) {
      gstr[i - 1] = strides_bytes[i - 1];
      if (gstr[i - 1] % 16 != 0)
        return refuse("tensor map stride %llu is not a multiple of 16 bytes",
                      (unsigned long long)gstr[i - 1]);
    }
  }
  CUtensorMapDataType dt = elem_bytes == 2   ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                             : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUtensorMapSwizzle sw = swizzle == 3   ? CU_TENSOR_MAP_SWIZZLE_128B
                          : swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_64B
                          : swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_32B
                                         : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUresult r = g_encode(out, dt, rank, const_cast<void*>(base), gdim, gstr, gbox, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return refuse("cuTensorMapEncodeTiled failed with code %d", (int)r);
  return 0;
}

}  // namespace mimir

// ---------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------
MIMIR_API int mimir_version() { return 100; }

MIMIR_API int mimir_set_device(int dev) { return cudaSetDevice(dev) == cudaSuccess ? 0 : -1; }

// Reads and clears the current device's error word.  Call after synchronising
// the streams whose kernels should be covered.
MIMIR_API unsigned mimir_error_word(int clear) {
  int d = mimir::current_device();
  mimir::ensure_device(d);
  if (!mimir::g_err_host[d]) return 0;
  unsigned v = *reinterpret_cast<volatile unsigned*>(mimir::g_err_host[d]);
  if (clear) *reinterpret_cast<volatile unsigned*>(mimir::g_err_host[d]) = 0;
  return v;
}

MIMIR_API long long mimir_launch_count() { return mimir::g_launches.load(); }
MIMIR_API void mimir_launch_count_add(long long n) { mimir::g_launches.fetch_add(n); }

MIMIR_API const char* mimir_last_error() { return mimir::g_last_error; }

MIMIR_API int mimir_sm_count() { return mimir::sm_count(); }
