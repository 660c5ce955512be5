// ---------------------------------------------------------------------------
// y[b, n] = sum_k x[b, k] * dequant(W)[n, k] for a weight kept in its ggml block
// encoding (Q8_0, Q4_0, Q4_K, Q6_K), read in place: no dequantised copy of the
// weight is made.  This is the small-batch path of the lazy tensor layer's
// quantised product (decode of a model whose file stores K-quants); the
// tensor-parallel decoder's Q4_0 path uses the planar / tiled layouts instead.
//
// One warp per weight row.  The row is walked in units of 32 values (a Q8_0 /
// Q4_0 block, or one of the eight sub-blocks of a 256-value K-quant super-block);
// four lanes share a unit, eight values each, so a warp covers 256 values per
// iteration and every lane's eight weights come from 8 consecutive bytes (Q6_K: 8
// low-nibble bytes plus 8 high-bit bytes).  Up to four activation rows are held per
// pass; larger batches loop.  fp32 accumulation, one shuffle reduction per
// row at the end.
//
// Replaces the reference's qmatmul kernel (backend/internal/gen/quant.go:156-209:
// 8 outputs per block, 32 threads per output, fp32 dequant, shared-memory tree sum),
// which covers Q8_0, Q4_K and Q6_K; Q4_0 is added here.
// ---------------------------------------------------------------------------
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "runtime.h"

namespace mimir {

namespace {

// Every block format has an even block size and even field offsets, and rows start on even
// addresses, so scales and 8-byte groups of quants can be read as 16-bit words.
__device__ __forceinline__ float h2f(const uint8_t* p) {
  return __half2float(__ushort_as_half(*reinterpret_cast<const uint16_t*>(p)));
}

// eight consecutive bytes from a 2-byte aligned address
__device__ __forceinline__ void ld_bytes8(const uint8_t* p, uint8_t out[8]) {
  const uint16_t* q = reinterpret_cast<const uint16_t*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint16_t w = q[i];
    out[2 * i] = static_cast<uint8_t>(w & 0xFF);
    out[2 * i + 1] = static_cast<uint8_t>(w >> 8);
  }
}

__device__ __forceinline__ void k4_scale_min(int j, const uint8_t* q, int& sc, int& mn) {
  if (j < 4) {
    sc = q[j] & 63;
    mn = q[j + 4] & 63;
  } else {
    sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
    mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
  }
}

// Eight consecutive values of unit `unit` of a row, starting at `off` (0, 8, 16, 24) inside the
// unit.  CODE is the file's dtype code: 64 Q8_0, 65 Q4_0, 66 Q4_K, 67 Q6_K.
template <int CODE>
__device__ __forceinline__ void decode8(const uint8_t* __restrict__ row, int unit, int off, float v[8]) {
  if constexpr (CODE == 64) {
    const uint8_t* b = row + static_cast<size_t>(unit) * 34;
    const float d = h2f(b);
    uint8_t q[8];
    ld_bytes8(b + 2 + off, q);
#pragma unroll
    for (int t = 0; t < 8; ++t) v[t] = d * static_cast<float>(static_cast<int8_t>(q[t]));
  } else if constexpr (CODE == 65) {
    const uint8_t* b = row + static_cast<size_t>(unit) * 18;
    const float d = h2f(b);
    const int sh = off < 16 ? 0 : 4;
    uint8_t q[8];
    ld_bytes8(b + 2 + (off & 15), q);
#pragma unroll
    for (int t = 0; t < 8; ++t) v[t] = d * static_cast<float>(((q[t] >> sh) & 0xF) - 8);
  } else if constexpr (CODE == 66) {
    const int sb = unit >> 3, sub = unit & 7;
    const uint8_t* b = row + static_cast<size_t>(sb) * 144;
    const float d = h2f(b), dmin = h2f(b + 2);
    int sc, mn;
    k4_scale_min(sub, b + 4, sc, mn);
    const float ds = d * sc, m = dmin * mn;
    const int sh = (sub & 1) ? 4 : 0;
    uint8_t q[8];
    ld_bytes8(b + 16 + (sub >> 1) * 32 + off, q);
#pragma unroll
    for (int t = 0; t < 8; ++t) v[t] = ds * static_cast<float>((q[t] >> sh) & 0xF) - m;
  } else {
    const int sb = unit >> 3, sub = unit & 7;
    const uint8_t* b = row + static_cast<size_t>(sb) * 210;
    const int half = sub >> 2, quarter = sub & 3;
    uint8_t ql[8], qh[8];
    ld_bytes8(b + 64 * half + ((quarter & 1) ? 32 : 0) + off, ql);
    ld_bytes8(b + 128 + 32 * half + off, qh);
    const int8_t* sc = reinterpret_cast<const int8_t*>(b + 192) + 8 * half + 2 * quarter;
    const float d = h2f(b + 208);
    const int sh = (quarter & 2) ? 4 : 0;
    // the lane's eight values lie inside one group of 16, so they share one scale
    const float ds = d * static_cast<float>(sc[off >> 4]);
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      const int lo = (ql[t] >> sh) & 0xF;
      const int hi = (qh[t] >> (2 * quarter)) & 3;
      v[t] = ds * static_cast<float>((lo | (hi << 4)) - 32);
    }
  }
}

template <int CODE>
__device__ __forceinline__ size_t row_bytes(int K) {
  if constexpr (CODE == 64) return static_cast<size_t>(K / 32) * 34;
  if constexpr (CODE == 65) return static_cast<size_t>(K / 32) * 18;
  if constexpr (CODE == 66) return static_cast<size_t>(K / 256) * 144;
  return static_cast<size_t>(K / 256) * 210;
}

__device__ __forceinline__ void load8(const float* p, float x[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float x[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    x[2 * i] = __uint_as_float(w[i] << 16);
    x[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}

constexpr int kRowsPerPass = 4;
constexpr int kWarpsPerBlock = 8;

template <int CODE, typename XT>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
qgemv_ggml_kernel(const uint8_t* __restrict__ w, const XT* __restrict__ x, int ldx, const float* __restrict__ bias,
                  float* __restrict__ out, int ldo, int N, int K, int B) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * kWarpsPerBlock + warp;
  if (n >= N) return;
  const uint8_t* row = w + static_cast<size_t>(n) * row_bytes<CODE>(K);
  const int units = K / 32;
  const int off = (lane & 3) * 8;
  for (int b0 = 0; b0 < B; b0 += kRowsPerPass) {
    float acc[kRowsPerPass];
#pragma unroll
    for (int r = 0; r < kRowsPerPass; ++r) acc[r] = 0.f;
    for (int u = lane >> 2; u < units; u += 8) {
      float v[8];
      decode8<CODE>(row, u, off, v);
      const int k = u * 32 + off;
#pragma unroll
      for (int r = 0; r < kRowsPerPass; ++r) {
        if (b0 + r < B) {
          float xv[8];
          load8(x + static_cast<size_t>(b0 + r) * ldx + k, xv);
#pragma unroll
          for (int t = 0; t < 8; ++t) acc[r] = fmaf(v[t], xv[t], acc[r]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < kRowsPerPass; ++r) {
      float s = acc[r];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
      if (lane == 0 && b0 + r < B) out[static_cast<size_t>(b0 + r) * ldo + n] = s + (bias ? bias[n] : 0.f);
    }
  }
}

template <int CODE>
int launch(const void* w, const void* x, int x_is_f32, int ldx, const float* bias, float* out, int ldo, int N, int K,
           int B, cudaStream_t st) {
  const int grid = ceil_div(N, kWarpsPerBlock);
  if (x_is_f32)
    qgemv_ggml_kernel<CODE, float><<<grid, kWarpsPerBlock * 32, 0, st>>>(
        static_cast<const uint8_t*>(w), static_cast<const float*>(x), ldx, bias, out, ldo, N, K, B);
  else
    qgemv_ggml_kernel<CODE, __nv_bfloat16><<<grid, kWarpsPerBlock * 32, 0, st>>>(
        static_cast<const uint8_t*>(w), static_cast<const __nv_bfloat16*>(x), ldx, bias, out, ldo, N, K, B);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : refuse("qgemv launch failed");
}

}  // namespace

}  // namespace mimir

using namespace mimir;

// w: ggml blocks of a [N, K] weight, rows contiguous.  x: [B, K] fp32 or bf16 with row pitch ldx
// (elements; a multiple of 8, base 16-byte aligned).  out: [B, N] fp32 with row pitch ldo.
MIMIR_API int mimir_qgemv_ggml(int code, const void* w, const void* x, int x_is_f32, int ldx, const float* bias,
                               float* out, int ldo, int N, int K, int B, cudaStream_t st) {
  if (code < 64 || code > 67) return refuse("qgemv: unknown dtype code %d", code);
  const int blk = code >= 66 ? 256 : 32;
  if (K <= 0 || K % blk) return refuse("qgemv: K = %d is not a multiple of the %d-value block", K, blk);
  if (N <= 0 || B <= 0) return refuse("qgemv: empty product");
  if (ldx % 8 || (reinterpret_cast<uintptr_t>(x) & 15)) return refuse("qgemv: activations must be 16-byte aligned rows");
  switch (code) {
    case 64: return launch<64>(w, x, x_is_f32, ldx, bias, out, ldo, N, K, B, st);
    case 65: return launch<65>(w, x, x_is_f32, ldx, bias, out, ldo, N, K, B, st);
    case 66: return launch<66>(w, x, x_is_f32, ldx, bias, out, ldo, N, K, B, st);
    default: return launch<67>(w, x, x_is_f32, ldx, bias, out, ldo, N, K, B, st);
  }
}
