// Pieces shared by the 1-CTA and the 2-CTA (cta_group::2) GEMM kernels: tile
// constants, epilogue flags, the fused epilogue applied to 8 columns of a row.
#pragma once
#include "common.cuh"
#include "runtime.h"

namespace mimir {

constexpr int kBM = 128;
constexpr int kBK = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr int kGemmThreads = 192;

enum GemmFlags : int {
  kOutF32 = 1,      // C is fp32 (default bf16)
  kAccumulate = 2,  // C += result
  kGelu = 4,        // C = gelu_tanh(acc + bias)
  kResidual = 8,    // C = acc + bias + aux
  kMulDGelu = 16,   // C = (acc) * gelu_tanh'(aux)
  kWritePre = 32,   // aux_out = acc + bias (pre-activation), with kGelu
};

struct GemmEpi {
  void* C;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* aux;
  __nv_bfloat16* aux_out;
  float* partial;  // split-K workspace [splits][M][N] (fp32) or nullptr
  int ldc, ldaux;
  int flags;
  float alpha;
};

// Applies the fused epilogue to 8 consecutive columns of one row and stores them.
__device__ __forceinline__ void epilogue_store8(const GemmEpi& ep, float (&v)[8], int row, int col) {
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] *= ep.alpha;
  if (ep.bias) {
    uint4 b = *reinterpret_cast<const uint4*>(ep.bias + col);
    float2 b0 = unpack_bf16x2(b.x), b1 = unpack_bf16x2(b.y), b2 = unpack_bf16x2(b.z),
           b3 = unpack_bf16x2(b.w);
    v[0] += b0.x; v[1] += b0.y; v[2] += b1.x; v[3] += b1.y;
    v[4] += b2.x; v[5] += b2.y; v[6] += b3.x; v[7] += b3.y;
  }
  if (ep.flags & (kResidual | kMulDGelu)) {
    uint4 a = *reinterpret_cast<const uint4*>(ep.aux + static_cast<size_t>(row) * ep.ldaux + col);
    float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z),
           a3 = unpack_bf16x2(a.w);
    float x[8] = {a0.x, a0.y, a1.x, a1.y, a2.x, a2.y, a3.x, a3.y};
    if (ep.flags & kMulDGelu) {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] *= gelu_tanh_grad(x[j]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] += x[j];
    }
  }
  if (ep.flags & kGelu) {
    if (ep.flags & kWritePre) {
      uint4 o;
      o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
      o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
      *reinterpret_cast<uint4*>(ep.aux_out + static_cast<size_t>(row) * ep.ldaux + col) = o;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = gelu_tanh(v[j]);
  }
  if (ep.flags & kOutF32) {
    float* c = reinterpret_cast<float*>(ep.C) + static_cast<size_t>(row) * ep.ldc + col;
    float4 lo = make_float4(v[0], v[1], v[2], v[3]), hi = make_float4(v[4], v[5], v[6], v[7]);
    if (ep.flags & kAccumulate) {
      float4 plo = *reinterpret_cast<float4*>(c), phi = *reinterpret_cast<float4*>(c + 4);
      lo.x += plo.x; lo.y += plo.y; lo.z += plo.z; lo.w += plo.w;
      hi.x += phi.x; hi.y += phi.y; hi.z += phi.z; hi.w += phi.w;
    }
    *reinterpret_cast<float4*>(c) = lo;
    *reinterpret_cast<float4*>(c + 4) = hi;
  } else {
    __nv_bfloat16* c = reinterpret_cast<__nv_bfloat16*>(ep.C) + static_cast<size_t>(row) * ep.ldc + col;
    if (ep.flags & kAccumulate) {
      uint4 p = *reinterpret_cast<uint4*>(c);
      float2 p0 = unpack_bf16x2(p.x), p1 = unpack_bf16x2(p.y), p2 = unpack_bf16x2(p.z),
             p3 = unpack_bf16x2(p.w);
      v[0] += p0.x; v[1] += p0.y; v[2] += p1.x; v[3] += p1.y;
      v[4] += p2.x; v[5] += p2.y; v[6] += p3.x; v[7] += p3.y;
    }
    uint4 o;
    o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
    o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
    *reinterpret_cast<uint4*>(c) = o;
  }
}


// Epilogue arithmetic on 8 consecutive columns of one row, without the store:
// v becomes the output values; pre (if the GELU side output is on) the pre-activation.
__device__ __forceinline__ void epilogue_math8(const GemmEpi& ep, float (&v)[8], float (&pre)[8], int row,
                                               int col) {
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] *= ep.alpha;
  if (ep.bias) {
    uint4 b = *reinterpret_cast<const uint4*>(ep.bias + col);
    float2 b0 = unpack_bf16x2(b.x), b1 = unpack_bf16x2(b.y), b2 = unpack_bf16x2(b.z), b3 = unpack_bf16x2(b.w);
    v[0] += b0.x; v[1] += b0.y; v[2] += b1.x; v[3] += b1.y;
    v[4] += b2.x; v[5] += b2.y; v[6] += b3.x; v[7] += b3.y;
  }
  if (ep.flags & (kResidual | kMulDGelu)) {
    uint4 a = *reinterpret_cast<const uint4*>(ep.aux + static_cast<size_t>(row) * ep.ldaux + col);
    float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z), a3 = unpack_bf16x2(a.w);
    float x[8] = {a0.x, a0.y, a1.x, a1.y, a2.x, a2.y, a3.x, a3.y};
    if (ep.flags & kMulDGelu) {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] *= gelu_tanh_grad(x[j]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] += x[j];
    }
  }
  if (ep.flags & kGelu) {
#pragma unroll
    for (int j = 0; j < 8; ++j) { pre[j] = v[j]; v[j] = gelu_tanh(v[j]); }
  }
}

// Stages a [32 rows x 64 columns] bf16 sub-tile (one row per lane, 8 x 16-byte units
// in pk) into a 128-byte-swizzled shared buffer and stores it with TMA.  Lane 0
// owns the bulk groups; at most one earlier store may still be reading the ring.
__device__ __forceinline__ void stage_and_store(const CUtensorMap* tm, uint8_t* wbuf, uint32_t& ring,
                                                const uint32_t (&pk)[32], int lane, int c0, int c1) {
  uint8_t* buf = wbuf + (ring & 1) * 4096;
  if (lane == 0) bulk_wait_group_read<1>();
  __syncwarp();
  const uint32_t base = smem_u32(buf) + lane * 128;
#pragma unroll
  for (int u = 0; u < 8; ++u)
    st_shared_v4(base + ((u ^ (lane & 7)) << 4), pk[4 * u], pk[4 * u + 1], pk[4 * u + 2], pk[4 * u + 3]);
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0) {
    tma_store_2d(tm, buf, c0, c1);
    bulk_commit_group();
  }
  ++ring;
}

// Split-K partial sums: NCH32 chunks of 32 fp32 columns leave through TMA stores into
// the workspace viewed as [splits][M][N] (3-D map, so rows past M are clipped per split).
template <int NCH32>
__device__ __forceinline__ void drain_partial_tma(const CUtensorMap* tmP, uint32_t taddr, int row0, int col_base,
                                                  int M, int N, int split, uint8_t* wbuf, uint32_t& ring,
                                                  int lane) {
#pragma unroll 1
  for (int c = 0; c < NCH32; ++c) {
    uint32_t r[32];
    tmem_ld32(taddr + c * 32, r);
    tmem_ld_wait();
    const int col0 = col_base + c * 32;
    if (col0 >= N || row0 >= M) continue;  // uniform over the warp
    uint8_t* buf = wbuf + (ring & 1) * 4096;
    if (lane == 0) bulk_wait_group_read<1>();
    __syncwarp();
    const uint32_t base = smem_u32(buf) + lane * 128;
#pragma unroll
    for (int u = 0; u < 8; ++u)
      st_shared_v4(base + ((u ^ (lane & 7)) << 4), r[4 * u], r[4 * u + 1], r[4 * u + 2], r[4 * u + 3]);
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_3d(tmP, buf, col0, row0, split);
      bulk_commit_group();
    }
    ++ring;
  }
}

// Epilogue modes of the straight-line (branch-free) chunk code below.
enum EpiMode : int { kEpiPlain = 0, kEpiGelu = 1, kEpiResidual = 2, kEpiDGelu = 3 };

__device__ __forceinline__ int epi_mode_of(int flags) {
  return (flags & kGelu) ? kEpiGelu : (flags & kResidual) ? kEpiResidual : (flags & kMulDGelu) ? kEpiDGelu : kEpiPlain;
}

// 64 columns of one row: accumulator bits in r0 | r1 -> packed bf16 output (pk) and,
// in GELU mode, packed pre-activation (pp).  No branches: loads for columns past N
// or rows past M are redirected to valid addresses and their results are clipped by
// the TMA store, so the whole chunk is one block of independent instructions and a
// lone warp per scheduler still keeps its pipelines busy.
template <int MODE, bool BIAS>
__device__ __forceinline__ void epilogue_chunk64(const GemmEpi& ep, const uint32_t (&r0)[32],
                                                 const uint32_t (&r1)[32], uint32_t (&pk)[32],
                                                 uint32_t (&pp)[32], int row_c, int col0, int N) {
  const float alpha = ep.alpha;
  uint4 bv[8], av[8];
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    const int cg = min(col0 + g * 8, N - 8);
    if (BIAS) bv[g] = *reinterpret_cast<const uint4*>(ep.bias + cg);
    if (MODE == kEpiResidual || MODE == kEpiDGelu)
      av[g] = *reinterpret_cast<const uint4*>(ep.aux + static_cast<size_t>(row_c) * ep.ldaux + cg);
  }
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = alpha * __uint_as_float(g < 4 ? r0[g * 8 + e] : r1[(g - 4) * 8 + e]);
    if (BIAS) {
      const uint32_t bw[4] = {bv[g].x, bv[g].y, bv[g].z, bv[g].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) { float2 t = unpack_bf16x2(bw[e]); v[2 * e] += t.x; v[2 * e + 1] += t.y; }
    }
    if (MODE == kEpiResidual || MODE == kEpiDGelu) {
      const uint32_t aw[4] = {av[g].x, av[g].y, av[g].z, av[g].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 t = unpack_bf16x2(aw[e]);
        if (MODE == kEpiResidual) { v[2 * e] += t.x; v[2 * e + 1] += t.y; }
        else { v[2 * e] *= gelu_tanh_grad(t.x); v[2 * e + 1] *= gelu_tanh_grad(t.y); }
      }
    }
    if (MODE == kEpiGelu) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        pp[4 * g + e] = pack_bf16x2(v[2 * e], v[2 * e + 1]);
        v[2 * e] = gelu_tanh(v[2 * e]);
        v[2 * e + 1] = gelu_tanh(v[2 * e + 1]);
      }
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) pk[4 * g + e] = pack_bf16x2(v[2 * e], v[2 * e + 1]);
  }
}

// Drains NCH 64-column chunks of an accumulator through the fused epilogue into TMA
// stores (bf16 outputs, no accumulate).  row0 = the warp's first row, lane's row =
// row0 + lane.  taddr / col_base point at the first chunk this warp owns.
template <int NCH, int MODE, bool BIAS>
__device__ __forceinline__ void drain_chunks_tma(const GemmEpi& ep, const CUtensorMap* tmC,
                                                 const CUtensorMap* tmPre, uint32_t taddr, int row0,
                                                 int col_base, int M, int N, uint8_t* wbuf, uint32_t& ring,
                                                 int lane) {
  const int row_c = min(row0 + lane, M - 1);
  const bool write_pre = MODE == kEpiGelu && (ep.flags & kWritePre);
#pragma unroll 1
  for (int c = 0; c < NCH; ++c) {
    uint32_t r0[32], r1[32];
    tmem_ld32(taddr + c * 64, r0);
    tmem_ld32(taddr + c * 64 + 32, r1);
    tmem_ld_wait();
    const int col0 = col_base + c * 64;
    if (col0 >= N || row0 >= M) continue;  // uniform over the warp
    uint32_t pk[32], pp[32];
    epilogue_chunk64<MODE, BIAS>(ep, r0, r1, pk, pp, row_c, col0, N);
    if (write_pre) stage_and_store(tmPre, wbuf, ring, pp, lane, col0, row0);
    stage_and_store(tmC, wbuf, ring, pk, lane, col0, row0);
  }
}

template <int NCH>
__device__ __forceinline__ void drain_accumulator_tma(const GemmEpi& ep, const CUtensorMap* tmC,
                                                      const CUtensorMap* tmPre, uint32_t taddr, int row0,
                                                      int col_base, int M, int N, uint8_t* wbuf, uint32_t& ring,
                                                      int lane) {
  const int mode = epi_mode_of(ep.flags);
  const bool bias = ep.bias != nullptr;
#define MIMIR_DRAIN(MODE_)                                                                                   \
  if (bias) drain_chunks_tma<NCH, MODE_, true>(ep, tmC, tmPre, taddr, row0, col_base, M, N, wbuf, ring, lane); \
  else drain_chunks_tma<NCH, MODE_, false>(ep, tmC, tmPre, taddr, row0, col_base, M, N, wbuf, ring, lane);
  if (mode == kEpiPlain) { MIMIR_DRAIN(kEpiPlain) }
  else if (mode == kEpiGelu) { MIMIR_DRAIN(kEpiGelu) }
  else if (mode == kEpiResidual) { MIMIR_DRAIN(kEpiResidual) }
  else { MIMIR_DRAIN(kEpiDGelu) }
#undef MIMIR_DRAIN
}

// Drains one accumulator buffer (128 lanes x BN columns of fp32 in TMEM) through
// the fused epilogue.  `row` is this thread's output row, taddr its TMEM address
// (lane quadrant included), col_base the first output column of the tile.
template <int BN>
__device__ __forceinline__ void drain_accumulator(const GemmEpi& ep, uint32_t taddr, int row, int col_base,
                                                  int M, int N, int split) {
#pragma unroll 1
  for (int c = 0; c < BN / 32; ++c) {
    uint32_t r[32];
    tmem_ld32(taddr + c * 32, r);
    tmem_ld_wait();
    const int col0 = col_base + c * 32;
    if (row < M) {
      if (ep.partial) {
        float* dst = ep.partial + (static_cast<size_t>(split) * M + row) * N + col0;
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          if (col0 + j < N)
            *reinterpret_cast<float4*>(dst + j) =
                make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                            __uint_as_float(r[j + 3]));
      } else {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          if (col0 + j < N) {
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[j + e]);
            epilogue_store8(ep, v, row, col0 + j);
          }
        }
      }
    }
  }
}

}  // namespace mimir
