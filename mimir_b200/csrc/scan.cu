// ---------------------------------------------------------------------------
// Inclusive scans along the last axis of a [rows, n] matrix: running sum, running
// maximum and running log-sum-exp, fp32 or bf16 in and out, fp32 arithmetic.
//
// One block of 256 threads per row.  The row is walked in chunks of 1024 values:
// each thread scans 4 consecutive values in registers, a warp shuffle scans the
// thread totals, one shared-memory step scans the 8 warp totals, and the chunk's
// total is carried into the next chunk.  Rows shorter than a chunk take one pass;
// there is no second kernel and no look-back between blocks, because a row is one
// block's work (many short rows is the shape scans have in this framework: token
// positions, nucleus cuts, CTC / CRF recursions).
//
// Replaces the reference's scan kernel (backend/internal/gen/scan.go:85-168: thread
// per line up to 64 values, else block per line with 4 x 256 chunks, Hillis-Steele
// over thread totals and a carry; sum / max / logsumexp).
// ---------------------------------------------------------------------------
#include <cuda_bf16.h>
#include <float.h>

#include "common.cuh"
#include "runtime.h"

namespace mimir {

namespace {

constexpr int kScanThreads = 256;
constexpr int kScanPer = 4;
constexpr int kScanChunk = kScanThreads * kScanPer;

enum ScanMode { kScanSum = 0, kScanMax = 1, kScanLogSumExp = 2 };

template <int MODE>
__device__ __forceinline__ float scan_identity() {
  return MODE == kScanSum ? 0.f : -INFINITY;
}

template <int MODE>
__device__ __forceinline__ float scan_combine(float a, float b) {
  if constexpr (MODE == kScanSum) return a + b;
  if constexpr (MODE == kScanMax) return (a != a || b != b) ? NAN : fmaxf(a, b);
  // log(exp(a) + exp(b)) without overflow; -inf is the identity
  const float m = fmaxf(a, b);
  if (m == -INFINITY) return -INFINITY;
  return m + log1pf(__expf(fminf(a, b) - m));
}

__device__ __forceinline__ float scan_ld(const float* p) { return *p; }
__device__ __forceinline__ float scan_ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void scan_st(float* p, float v) { *p = v; }
__device__ __forceinline__ void scan_st(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

template <int MODE, typename T>
__global__ void __launch_bounds__(kScanThreads)
scan_rows_kernel(const T* __restrict__ x, T* __restrict__ y, int n, long long ldx, long long ldy, int reverse) {
  __shared__ float warp_tot[kScanThreads / 32];
  __shared__ float carry_s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const T* xr = x + static_cast<size_t>(blockIdx.x) * ldx;
  T* yr = y + static_cast<size_t>(blockIdx.x) * ldy;
  if (tid == 0) carry_s = scan_identity<MODE>();
  __syncthreads();
  for (int base = 0; base < n; base += kScanChunk) {
    float v[kScanPer];
    const int i0 = base + tid * kScanPer;
#pragma unroll
    for (int j = 0; j < kScanPer; ++j) {
      const int i = i0 + j;
      v[j] = i < n ? scan_ld(xr + (reverse ? n - 1 - i : i)) : scan_identity<MODE>();
    }
#pragma unroll
    for (int j = 1; j < kScanPer; ++j) v[j] = scan_combine<MODE>(v[j - 1], v[j]);
    // exclusive scan of the thread totals across the warp
    float incl = v[kScanPer - 1];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl = scan_combine<MODE>(up, incl);
    }
    float excl = __shfl_up_sync(0xffffffffu, incl, 1);
    if (lane == 0) excl = scan_identity<MODE>();
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    float before = carry_s;
    for (int w = 0; w < warp; ++w) before = scan_combine<MODE>(before, warp_tot[w]);
    before = scan_combine<MODE>(before, excl);
#pragma unroll
    for (int j = 0; j < kScanPer; ++j) {
      const int i = i0 + j;
      if (i < n) scan_st(yr + (reverse ? n - 1 - i : i), scan_combine<MODE>(before, v[j]));
    }
    __syncthreads();
    if (tid == kScanThreads - 1) carry_s = scan_combine<MODE>(before, v[kScanPer - 1]);
    __syncthreads();
  }
}

template <int MODE>
int launch_scan(const void* x, void* y, int is_f32, int rows, int n, long long ldx, long long ldy, int reverse,
                cudaStream_t st) {
  if (is_f32)
    scan_rows_kernel<MODE, float><<<rows, kScanThreads, 0, st>>>(static_cast<const float*>(x), static_cast<float*>(y),
                                                                 n, ldx, ldy, reverse);
  else
    scan_rows_kernel<MODE, __nv_bfloat16><<<rows, kScanThreads, 0, st>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), n, ldx, ldy, reverse);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : refuse("scan launch failed");
}

}  // namespace

}  // namespace mimir

using namespace mimir;

// mode 0 running sum, 1 running maximum, 2 running log-sum-exp; x and y are [rows, n] with row
// pitches ldx / ldy (elements) and may be the same buffer.  reverse != 0 scans from the end.
MIMIR_API int mimir_scan_rows(const void* x, void* y, int is_f32, int rows, int n, long long ldx, long long ldy, int mode,
                              int reverse, cudaStream_t st) {
  if (rows <= 0 || n <= 0) return 0;
  switch (mode) {
    case 0: return launch_scan<kScanSum>(x, y, is_f32, rows, n, ldx, ldy, reverse, st);
    case 1: return launch_scan<kScanMax>(x, y, is_f32, rows, n, ldx, ldy, reverse, st);
    case 2: return launch_scan<kScanLogSumExp>(x, y, is_f32, rows, n, ldx, ldy, reverse, st);
    default: return refuse("scan: unknown mode %d", mode);
  }
}
