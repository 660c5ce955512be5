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
// low-nibble bytes plus 8 high-bit bytes).  A lane fetches the bytes of two units before it
// decodes the first.  Quants become floats without conversion instructions (OR into the
// mantissa of 2^23, one subtraction that also removes the zero point); the block scale and
// Q4_K's constant term are applied once per unit to sum(q*x) and sum(x), so a weight costs one
// FMA per activation row.  Up to four activation rows are held per pass; larger batches loop.
// fp32 accumulation, one shuffle reduction per row at the end.
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
// addresses, so scales and groups of quants can be read as 16-bit words.
// The bytes one lane needs from one unit, fetched in one go so that a lane can have several units
// in flight before it decodes the first (the kernel is bound by memory latency).
//   Q8_0 / Q4_0: w[0] = scale (fp16), w[1..2] = 8 quant bytes
//   Q4_K       : w[0] = d | dmin << 16, w[1..3] = the 12 scale bytes, w[4..5] = 8 quant bytes
//   Q6_K       : w[0] = d | scale byte << 16, w[1..2] = 8 low-nibble bytes, w[3..4] = 8 high-bit bytes
struct RawUnit {
  uint32_t w[6];
};

__device__ __forceinline__ uint32_t ld_u16x2(const uint8_t* p) {   // 4 bytes from a 2-byte aligned address
  const uint16_t* q = reinterpret_cast<const uint16_t*>(p);
  return static_cast<uint32_t>(q[0]) | (static_cast<uint32_t>(q[1]) << 16);
}

// CODE is the file's dtype code: 64 Q8_0, 65 Q4_0, 66 Q4_K, 67 Q6_K.  `off` (0, 8, 16, 24) is the
// lane's position inside the unit of 32 values.
template <int CODE>
__device__ __forceinline__ void fetch_unit(const uint8_t* __restrict__ row, int unit, int off, RawUnit& r) {
  if constexpr (CODE == 64) {
    const uint8_t* b = row + static_cast<size_t>(unit) * 34;
    r.w[0] = *reinterpret_cast<const uint16_t*>(b);
    r.w[1] = ld_u16x2(b + 2 + off);
    r.w[2] = ld_u16x2(b + 6 + off);
  } else if constexpr (CODE == 65) {
    const uint8_t* b = row + static_cast<size_t>(unit) * 18;
    r.w[0] = *reinterpret_cast<const uint16_t*>(b);
    r.w[1] = ld_u16x2(b + 2 + (off & 15));
    r.w[2] = ld_u16x2(b + 6 + (off & 15));
  } else if constexpr (CODE == 66) {
    // super-blocks of 144 bytes in rows that start 16-byte aligned: 4- and 8-byte loads are aligned
    const uint8_t* b = row + static_cast<size_t>(unit >> 3) * 144;
    const uint32_t* h = reinterpret_cast<const uint32_t*>(b);
    r.w[0] = h[0];
    r.w[1] = h[1]; r.w[2] = h[2]; r.w[3] = h[3];
    const uint2 q = *reinterpret_cast<const uint2*>(b + 16 + ((unit & 7) >> 1) * 32 + off);
    r.w[4] = q.x; r.w[5] = q.y;
  } else {
    const int sub = unit & 7, half = sub >> 2, quarter = sub & 3;
    const uint8_t* b = row + static_cast<size_t>(unit >> 3) * 210;
    const uint32_t sc = b[192 + 8 * half + 2 * quarter + (off >> 4)];
    r.w[0] = static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(b + 208)) | (sc << 16);
    const uint8_t* ql = b + 64 * half + ((quarter & 1) ? 32 : 0) + off;
    const uint8_t* qh = b + 128 + 32 * half + off;
    r.w[1] = ld_u16x2(ql); r.w[2] = ld_u16x2(ql + 4);
    r.w[3] = ld_u16x2(qh); r.w[4] = ld_u16x2(qh + 4);
  }
}

__device__ __forceinline__ float half_bits(uint32_t lo16) {
  return __half2float(__ushort_as_half(static_cast<uint16_t>(lo16 & 0xFFFF)));
}

// An integer field below 2^23 as a float without a conversion instruction: OR it into the mantissa
// of 2^23 and subtract 2^23 plus the format's zero point.
__device__ __forceinline__ float field_to_float(uint32_t field, float magic_minus_zero) {
  return __uint_as_float(0x4B000000u | field) - magic_minus_zero;
}

// The unit's eight values as q[t] (integers held in floats, zero point already removed), a scale
// and a constant term: value t = scale * q[t] - minus.  The product with the activations then needs
// one FMA per value; scale and minus are applied once per unit on the sums.
template <int CODE>
__device__ __forceinline__ void decode_unit(const RawUnit& r, int unit, int off, float q[8], float& scale,
                                            float& minus) {
  constexpr float kTwo23 = 8388608.f;
  minus = 0.f;
  if constexpr (CODE == 64) {
    scale = half_bits(r.w[0]);
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      const uint32_t w = t < 4 ? r.w[1] : r.w[2];
      // a signed byte: flip its top bit to make it unsigned, remove 128 again with the magic constant
      q[t] = field_to_float(((w >> (8 * (t & 3))) & 0xFF) ^ 0x80, kTwo23 + 128.f);
    }
  } else if constexpr (CODE == 65) {
    scale = half_bits(r.w[0]);
    const int sh = off < 16 ? 0 : 4;
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      const uint32_t w = t < 4 ? r.w[1] : r.w[2];
      q[t] = field_to_float((w >> (8 * (t & 3) + sh)) & 0xF, kTwo23 + 8.f);
    }
  } else if constexpr (CODE == 66) {
    const int sub = unit & 7;
    const float d = half_bits(r.w[0]), dmin = half_bits(r.w[0] >> 16);
    // byte i of the 12 packed 6-bit scales / minimums, picked from the three words without an array
    auto sbyte = [&](int i) -> int {
      const uint32_t word = i < 4 ? r.w[1] : (i < 8 ? r.w[2] : r.w[3]);
      return static_cast<int>((word >> (8 * (i & 3))) & 0xFF);
    };
    int sc, mn;
    if (sub < 4) {
      sc = sbyte(sub) & 63;
      mn = sbyte(sub + 4) & 63;
    } else {
      sc = (sbyte(sub + 4) & 0xF) | ((sbyte(sub - 4) >> 6) << 4);
      mn = (sbyte(sub + 4) >> 4) | ((sbyte(sub) >> 6) << 4);
    }
    scale = d * static_cast<float>(sc);
    minus = dmin * static_cast<float>(mn);
    const int sh = (sub & 1) ? 4 : 0;
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      const uint32_t w = t < 4 ? r.w[4] : r.w[5];
      q[t] = field_to_float((w >> (8 * (t & 3) + sh)) & 0xF, kTwo23);
    }
  } else {
    const int quarter = unit & 3;
    // the lane's eight values lie inside one group of 16, so they share one scale
    scale = half_bits(r.w[0]) * static_cast<float>(static_cast<int8_t>((r.w[0] >> 16) & 0xFF));
    const int sh = (quarter & 2) ? 4 : 0;
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      const uint32_t wl = t < 4 ? r.w[1] : r.w[2], wh = t < 4 ? r.w[3] : r.w[4];
      const uint32_t lo = (wl >> (8 * (t & 3) + sh)) & 0xF;
      const uint32_t hi = (wh >> (8 * (t & 3) + 2 * quarter)) & 3;
      q[t] = field_to_float(lo | (hi << 4), kTwo23 + 32.f);
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
constexpr int kUnitsInFlight = 2;   // units a lane fetches before it decodes the first
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
    for (int u0 = lane >> 2; u0 < units; u0 += 8 * kUnitsInFlight) {
      RawUnit raw[kUnitsInFlight];
#pragma unroll
      for (int j = 0; j < kUnitsInFlight; ++j)
        if (u0 + 8 * j < units) fetch_unit<CODE>(row, u0 + 8 * j, off, raw[j]);
#pragma unroll
      for (int j = 0; j < kUnitsInFlight; ++j) {
        const int u = u0 + 8 * j;
        if (u >= units) break;
        float q[8], scale, minus;
        decode_unit<CODE>(raw[j], u, off, q, scale, minus);
        const int k = u * 32 + off;
#pragma unroll
        for (int r = 0; r < kRowsPerPass; ++r) {
          if (b0 + r < B) {
            float xv[8];
            load8(x + static_cast<size_t>(b0 + r) * ldx + k, xv);
            float dot = 0.f, sum = 0.f;
#pragma unroll
            for (int t = 0; t < 8; ++t) {
              dot = fmaf(q[t], xv[t], dot);
              if constexpr (CODE == 66) sum += xv[t];     // only Q4_K has a constant term
            }
            acc[r] = fmaf(scale, dot, acc[r]);
            if constexpr (CODE == 66) acc[r] = fmaf(-minus, sum, acc[r]);
          }
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
