// 2-D convolution as an implicit GEMM on the tcgen05 tensor cores, bf16 in NHWC
// with the channel count padded to a multiple of 64 (one 128-byte swizzle row).
//
// No window copy is ever materialised: the A tile of a filter tap is a plain
// tiled TMA load of an (Ht x Wt) patch of the image, 64 channels deep, at the
// tap's offset.  The patch's rows land in shared memory as consecutive 128-byte
// rows, which is exactly the K-major operand tile the tensor core wants (forward
// and input gradient: 128 pixels x 64 channels), or the MN-major one (weight
// gradient: 64 pixels of contraction x 64 channels).  Rows and columns of the
// patch that fall outside the image are filled with zeros by TMA, which is the
// convolution's zero padding.  Stride 1 (any dilation, any padding); strided
// convolutions are lowered to an explicit window gather plus the GEMM kernel by
// the caller.
//
//   forward          y[n,h,w,co]  = act(sum_{kh,kw,ci} x[n,h+kh*d-p,w+kw*d-p,ci] * W[co,(kh,kw,ci)] + b[co])
//   input gradient   the same kernel on dy with the flipped, transposed filter
//   weight gradient  dW[co,(kh,kw,ci)] = sum_{n,h,w} dy[n,h,w,co] * x[n,h+kh*d-p,w+kw*d-p,ci]
//                    split over pixel patches; fp32 partials summed by a second kernel
//
// Replaces the reference's tiled SIMT implicit-GEMM convolution kernels
// (backend/internal/gen/conv.go:99-177 forward, :182-266 weight gradient in parts
// plus a sum kernel, :275-376 input gradient) and its CPU-only max pooling
// (backend/cpu/pool.go:27).
#include "gemm_common.cuh"

namespace mimir {

struct ConvGeom {
  int N, H, W;      // input image
  int Ho, Wo;       // output image
  int Cp, Cop;      // padded input / output channels (multiples of 64)
  int KH, KW, pad_h, pad_w, dil;
  int Ht, Wt;       // pixel patch of a tile (Ht * Wt = 128 forward, 64 weight gradient)
  int h_tiles, w_tiles;
};

// ---------------------------------------------------------------------------
// Forward / input gradient.  warp 0 TMA, warp 1 MMA, warps 2..5 epilogue.
// ---------------------------------------------------------------------------
template <int BN, int STAGES>
__global__ void __launch_bounds__(kGemmThreads, 1)
conv_fwd_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, ConvGeom g,
                __nv_bfloat16* __restrict__ y, const float* __restrict__ bias, int relu, unsigned* err) {
  constexpr int A_BYTES = kBM * kBK * 2;
  constexpr int B_BYTES = BN * kBK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * BN;
  constexpr uint32_t IDESC = make_idesc_bf16(kBM, BN, false, false);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = g.Cop / BN;
  const int cchunks = g.Cp / kBK;
  const int kb_total = g.KH * g.KW * cchunks;
  const int units = g.N * g.h_tiles * g.w_tiles * n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 4);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmX);
      tma_prefetch_desc(&tmW);
      uint32_t it = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
        const int n_idx = u % n_tiles;
        int t = u / n_tiles;
        const int wt = t % g.w_tiles; t /= g.w_tiles;
        const int ht = t % g.h_tiles;
        const int img = t / g.h_tiles;
        for (int kb = 0; kb < kb_total; ++kb, ++it) {
          const int cc = kb % cchunks, tap = kb / cchunks;
          const int kw = tap % g.KW, kh = tap / g.KW;
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, err)) { ok = false; break; }
          uint8_t* sA = smem + s * STAGE_BYTES;
          uint8_t* sB = sA + A_BYTES;
          mbar_arrive_expect_tx(&full[s], STAGE_BYTES);
          // channel coordinate is a multiple of 64 elements (16-byte rule); the pixel
          // coordinates may be negative or past the edge: those rows read zeros
          tma_load_4d(sA, &tmX, &full[s], cc * kBK, wt * g.Wt + kw * g.dil - g.pad_w,
                      ht * g.Ht + kh * g.dil - g.pad_h, img);
          tma_load_2d(sB, &tmW, &full[s], kb * kBK, n_idx * BN);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t it = 0, ti = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < units && ok; u += gridDim.x, ++ti) {
        const uint32_t acc = ti & 1, acc_ph = (ti >> 1) & 1;
        if (!mbar_wait(&tempty[acc], acc_ph ^ 1, abort_flag, err)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kb_total; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full[s], ph, abort_flag, err)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sB = sA + A_BYTES;
          const uint64_t adesc = make_smem_desc_sw128(sA, 16, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(sB, 16, 1024);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k)
            umma_ss(d_tmem, adesc + k * 2, bdesc + k * 2, IDESC, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(&empty[s]);
        }
        if (ok) umma_commit(&tfull[acc]);
      }
    }
  } else {
    const int q = warp & 3;
    uint32_t ti = 0;
    for (int u = blockIdx.x; u < units; u += gridDim.x, ++ti) {
      const int n_idx = u % n_tiles;
      int t = u / n_tiles;
      const int wt = t % g.w_tiles; t /= g.w_tiles;
      const int ht = t % g.h_tiles;
      const int img = t / g.h_tiles;
      const uint32_t acc = ti & 1, acc_ph = (ti >> 1) & 1;
      if (!mbar_wait(&tfull[acc], acc_ph, abort_flag, err)) break;
      tc_fence_after();
      const int r = q * 32 + lane;
      const int oh = ht * g.Ht + r / g.Wt, ow = wt * g.Wt + r % g.Wt;
      const bool valid = oh < g.Ho && ow < g.Wo;
      __nv_bfloat16* dst = y + ((static_cast<size_t>(img) * g.Ho + oh) * g.Wo + ow) * g.Cop + n_idx * BN;
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t rr[32];
        tmem_ld32(taddr + c * 32, rr);
        tmem_ld_wait();
        if (valid) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              v[e] = __uint_as_float(rr[j + e]);
              if (bias) v[e] += bias[n_idx * BN + c * 32 + j + e];
              if (relu) v[e] = fmaxf(v[e], 0.f);
            }
            uint4 o;
            o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
            o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
            *reinterpret_cast<uint4*>(dst + c * 32 + j) = o;
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------
// Weight gradient.  A unit is (tap, 128 output channels, BN input channels,
// split); its contraction runs over the split's pixel patches (64 pixels each).
// Both operands are MN-major: pixels are rows of shared memory, channels the
// contiguous direction.  The accumulator goes to the fp32 partial buffer
// part[split][co][tap * Cp + ci].
// ---------------------------------------------------------------------------
template <int BN, int STAGES>
__global__ void __launch_bounds__(kGemmThreads, 1)
conv_wgrad_kernel(const __grid_constant__ CUtensorMap tmDy, const __grid_constant__ CUtensorMap tmX, ConvGeom g,
                  float* __restrict__ part, int Co, int splits, unsigned* err) {
  constexpr int A_BYTES = kBM * kBK * 2;
  constexpr int B_BYTES = BN * kBK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * BN;
  constexpr uint32_t IDESC = make_idesc_bf16(kBM, BN, true, true);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tfull = empty + STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int taps = g.KH * g.KW;
  const int m_tiles = (g.Cop + kBM - 1) / kBM, n_tiles = g.Cp / BN;
  const int patches = g.N * g.h_tiles * g.w_tiles;
  const int per = (patches + splits - 1) / splits;
  const int units = taps * m_tiles * n_tiles * splits;
  const int ldw = taps * g.Cp;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 4);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmDy);
      tma_prefetch_desc(&tmX);
      uint32_t it = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
        const int split = u % splits;
        int t = u / splits;
        const int n_idx = t % n_tiles; t /= n_tiles;
        const int m_idx = t % m_tiles;
        const int tap = t / m_tiles;
        const int kw = tap % g.KW, kh = tap / g.KW;
        const int p0 = split * per, p1 = min(patches, p0 + per);
        for (int p = p0; p < p1; ++p, ++it) {
          int tt = p;
          const int wt = tt % g.w_tiles; tt /= g.w_tiles;
          const int ht = tt % g.h_tiles;
          const int img = tt / g.h_tiles;
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, err)) { ok = false; break; }
          uint8_t* sA = smem + s * STAGE_BYTES;
          uint8_t* sB = sA + A_BYTES;
          mbar_arrive_expect_tx(&full[s], STAGE_BYTES);
#pragma unroll
          for (int c = 0; c < kBM / 64; ++c)  // channels past the tensor's extent read zeros
            tma_load_4d(sA + c * (kBK * 128), &tmDy, &full[s], m_idx * kBM + c * 64, wt * g.Wt, ht * g.Ht, img);
#pragma unroll
          for (int c = 0; c < BN / 64; ++c)
            tma_load_4d(sB + c * (kBK * 128), &tmX, &full[s], n_idx * BN + c * 64,
                        wt * g.Wt + kw * g.dil - g.pad_w, ht * g.Ht + kh * g.dil - g.pad_h, img);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t it = 0, ti = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < units && ok; u += gridDim.x, ++ti) {
        const int split = u % splits;
        const int p0 = split * per, p1 = min(patches, p0 + per);
        const uint32_t acc = ti & 1, acc_ph = (ti >> 1) & 1;
        if (!mbar_wait(&tempty[acc], acc_ph ^ 1, abort_flag, err)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int p = p0; p < p1; ++p, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full[s], ph, abort_flag, err)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sB = sA + A_BYTES;
          const uint64_t adesc = make_smem_desc_sw128(sA, kBK * 128, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(sB, kBK * 128, 1024);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k)
            umma_ss(d_tmem, adesc + k * 128, bdesc + k * 128, IDESC, (p > p0 || k > 0) ? 1u : 0u);
          umma_commit(&empty[s]);
        }
        if (ok) umma_commit(&tfull[acc]);
      }
    }
  } else {
    const int q = warp & 3;
    uint32_t ti = 0;
    for (int u = blockIdx.x; u < units; u += gridDim.x, ++ti) {
      const int split = u % splits;
      int t = u / splits;
      const int n_idx = t % n_tiles; t /= n_tiles;
      const int m_idx = t % m_tiles;
      const int tap = t / m_tiles;
      const int p0 = split * per, p1 = min(patches, p0 + per);
      const uint32_t acc = ti & 1, acc_ph = (ti >> 1) & 1;
      if (!mbar_wait(&tfull[acc], acc_ph, abort_flag, err)) break;
      tc_fence_after();
      const int co = m_idx * kBM + q * 32 + lane;
      float* dst = part + (static_cast<size_t>(split) * Co + co) * ldw + tap * g.Cp + n_idx * BN;
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t rr[32];
        tmem_ld32(taddr + c * 32, rr);
        tmem_ld_wait();
        if (co < Co) {
          const bool any = p1 > p0;  // a split without patches left its accumulator untouched
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4*>(dst + c * 32 + j) =
                any ? make_float4(__uint_as_float(rr[j]), __uint_as_float(rr[j + 1]), __uint_as_float(rr[j + 2]),
                                  __uint_as_float(rr[j + 3]))
                    : make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// dW[i] (+)= sum_s part[s][i]
__global__ void conv_wgrad_reduce_kernel(const float* __restrict__ part, float* __restrict__ dw, size_t n4, int splits,
                                         int accumulate) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  float4 a = accumulate ? reinterpret_cast<float4*>(dw)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s = 0; s < splits; ++s) {
    const float4 p = reinterpret_cast<const float4*>(part)[static_cast<size_t>(s) * n4 + i];
    a.x += p.x; a.y += p.y; a.z += p.z; a.w += p.w;
  }
  reinterpret_cast<float4*>(dw)[i] = a;
}

// ---------------------------------------------------------------------------
// Max pooling over NHWC bf16 (8 channels per thread).  The forward pass records
// the argmax as a byte (index inside the window) so that the backward pass is a
// gather with no comparison and no atomics: every input pixel looks at the
// windows that cover it.
// ---------------------------------------------------------------------------
__global__ void maxpool_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                   uint8_t* __restrict__ arg, int N, int H, int W, int C, int Ho, int Wo, int k, int s) {
  const int c8 = C / 8;
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<size_t>(N) * Ho * Wo * c8) return;
  const int c = static_cast<int>(idx % c8) * 8;
  size_t t = idx / c8;
  const int ow = static_cast<int>(t % Wo); t /= Wo;
  const int oh = static_cast<int>(t % Ho);
  const int n = static_cast<int>(t / Ho);
  float best[8];
  int bi[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) { best[e] = -INFINITY; bi[e] = 0; }
  for (int i = 0; i < k; ++i)
    for (int j = 0; j < k; ++j) {
      const int h = oh * s + i, w = ow * s + j;
      if (h >= H || w >= W) continue;
      const uint4 v = *reinterpret_cast<const uint4*>(x + ((static_cast<size_t>(n) * H + h) * W + w) * C + c);
      const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), cc = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
      const float f[8] = {a.x, a.y, b.x, b.y, cc.x, cc.y, d.x, d.y};
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if (f[e] > best[e]) { best[e] = f[e]; bi[e] = i * k + j; }
    }
  uint4 o;
  o.x = pack_bf16x2(best[0], best[1]); o.y = pack_bf16x2(best[2], best[3]);
  o.z = pack_bf16x2(best[4], best[5]); o.w = pack_bf16x2(best[6], best[7]);
  const size_t off = ((static_cast<size_t>(n) * Ho + oh) * Wo + ow) * C + c;
  *reinterpret_cast<uint4*>(y + off) = o;
  uint2 ab;
  ab.x = bi[0] | (bi[1] << 8) | (bi[2] << 16) | (bi[3] << 24);
  ab.y = bi[4] | (bi[5] << 8) | (bi[6] << 16) | (bi[7] << 24);
  *reinterpret_cast<uint2*>(arg + off) = ab;
}

__global__ void maxpool_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const uint8_t* __restrict__ arg,
                                   __nv_bfloat16* __restrict__ dx, int N, int H, int W, int C, int Ho, int Wo, int k,
                                   int s) {
  const int c8 = C / 8;
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<size_t>(N) * H * W * c8) return;
  const int c = static_cast<int>(idx % c8) * 8;
  size_t t = idx / c8;
  const int w = static_cast<int>(t % W); t /= W;
  const int h = static_cast<int>(t % H);
  const int n = static_cast<int>(t / H);
  float g[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  // windows (oh, ow) with oh*s <= h < oh*s + k
  const int oh_lo = h - k + 1 > 0 ? (h - k + s) / s : 0, oh_hi = min(Ho - 1, h / s);
  const int ow_lo = w - k + 1 > 0 ? (w - k + s) / s : 0, ow_hi = min(Wo - 1, w / s);
  for (int oh = oh_lo; oh <= oh_hi; ++oh)
    for (int ow = ow_lo; ow <= ow_hi; ++ow) {
      const int want = (h - oh * s) * k + (w - ow * s);
      const size_t off = ((static_cast<size_t>(n) * Ho + oh) * Wo + ow) * C + c;
      const uint2 ab = *reinterpret_cast<const uint2*>(arg + off);
      const uint4 v = *reinterpret_cast<const uint4*>(dy + off);
      const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), cc = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
      const float f[8] = {a.x, a.y, b.x, b.y, cc.x, cc.y, d.x, d.y};
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int which = ((e < 4 ? ab.x : ab.y) >> ((e & 3) * 8)) & 0xff;
        if (which == want) g[e] += f[e];
      }
    }
  uint4 o;
  o.x = pack_bf16x2(g[0], g[1]); o.y = pack_bf16x2(g[2], g[3]);
  o.z = pack_bf16x2(g[4], g[5]); o.w = pack_bf16x2(g[6], g[7]);
  *reinterpret_cast<uint4*>(dx + ((static_cast<size_t>(n) * H + h) * W + w) * C + c) = o;
}

// dx = dy where y > 0 (ReLU backward on the stored activation), 8 values per thread
__global__ void relu_bwd_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ dy,
                                __nv_bfloat16* __restrict__ dx, size_t n8) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  const uint4 yv = reinterpret_cast<const uint4*>(y)[i];
  uint4 g = reinterpret_cast<const uint4*>(dy)[i];
  const uint32_t ys[4] = {yv.x, yv.y, yv.z, yv.w};
  uint32_t gs[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 f = unpack_bf16x2(ys[e]);
    if (!(f.x > 0.f)) gs[e] &= 0xffff0000u;
    if (!(f.y > 0.f)) gs[e] &= 0x0000ffffu;
  }
  reinterpret_cast<uint4*>(dx)[i] = make_uint4(gs[0], gs[1], gs[2], gs[3]);
}

static int pick_patch(int Ho, int Wo, int pixels, int* Ht, int* Wt) {
  long long best = -1;
  for (int wt = 8; wt <= pixels; wt *= 2) {
    const int ht = pixels / wt;
    const long long tiles = static_cast<long long>(ceil_div(Wo, wt)) * ceil_div(Ho, ht);
    if (best < 0 || tiles < best) { best = tiles; *Ht = ht; *Wt = wt; }
  }
  return 0;
}

static int encode_nhwc(CUtensorMap* tm, const void* base, int N, int H, int W, int C, int Ht, int Wt) {
  uint64_t dims[4] = {static_cast<uint64_t>(C), static_cast<uint64_t>(W), static_cast<uint64_t>(H),
                      static_cast<uint64_t>(N)};
  uint64_t strides[3] = {static_cast<uint64_t>(C) * 2, static_cast<uint64_t>(W) * C * 2,
                         static_cast<uint64_t>(H) * W * C * 2};
  uint32_t box[4] = {64, static_cast<uint32_t>(Wt), static_cast<uint32_t>(Ht), 1};
  return encode_tmap(tm, base, 2, 4, dims, strides, box, 3);
}

template <int BN, int STAGES>
static int launch_conv_fwd(const CUtensorMap& tmX, const CUtensorMap& tmW, const ConvGeom& g, void* y, const float* bias,
                           int relu, cudaStream_t st) {
  constexpr int SMEM = STAGES * (kBM * kBK * 2 + BN * kBK * 2) + 1024 + 256;
  auto kern = conv_fwd_kernel<BN, STAGES>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
      return refuse("conv: cannot reserve %d bytes of shared memory", SMEM);
    configured = true;
  }
  const int units = g.N * g.h_tiles * g.w_tiles * (g.Cop / BN);
  const int grid = units < sm_count() ? units : sm_count();
  kern<<<grid, kGemmThreads, SMEM, st>>>(tmX, tmW, g, static_cast<__nv_bfloat16*>(y), bias, relu, error_word_dev());
  count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : refuse("conv forward launch failed");
}

template <int BN, int STAGES>
static int launch_conv_wgrad(const CUtensorMap& tmDy, const CUtensorMap& tmX, const ConvGeom& g, float* part, int Co,
                             int splits, cudaStream_t st) {
  constexpr int SMEM = STAGES * (kBM * kBK * 2 + BN * kBK * 2) + 1024 + 256;
  auto kern = conv_wgrad_kernel<BN, STAGES>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
      return refuse("conv: cannot reserve %d bytes of shared memory", SMEM);
    configured = true;
  }
  const int units = g.KH * g.KW * ceil_div(g.Cop, kBM) * (g.Cp / BN) * splits;
  const int grid = units < sm_count() ? units : sm_count();
  kern<<<grid, kGemmThreads, SMEM, st>>>(tmDy, tmX, g, part, Co, splits, error_word_dev());
  count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : refuse("conv weight-gradient launch failed");
}

}  // namespace mimir

using namespace mimir;

// y[N,Ho,Wo,Cop] = act(conv(x[N,H,W,Cp], w[Cop rows used: Co][KH*KW*Cp]) + bias), stride 1.
// Cp and Cop are multiples of 64; w has `w_rows` rows (rows past it read zeros) of KH*KW*Cp
// bf16 values each, ordered (kh, kw, ci).  bias: Cop floats or null.  Ho = H + 2*pad_h - dil*(KH-1),
// Wo likewise.  The input gradient is the same call on dy with the flipped, transposed filter
// and padding dil*(K-1) - pad.
MIMIR_API int mimir_conv2d_fwd(const void* x, const void* w, const float* bias, void* y, int N, int H, int W, int Cp,
                               int Cop, int w_rows, int KH, int KW, int pad_h, int pad_w, int dil, int relu,
                               cudaStream_t st) {
  if (Cp % 64 || Cop % 64 || Cp <= 0 || Cop <= 0) return refuse("conv: channel counts %d, %d must be multiples of 64", Cp, Cop);
  ConvGeom g;
  g.N = N; g.H = H; g.W = W; g.Cp = Cp; g.Cop = Cop; g.KH = KH; g.KW = KW; g.pad_h = pad_h; g.pad_w = pad_w; g.dil = dil;
  g.Ho = H + 2 * pad_h - dil * (KH - 1);
  g.Wo = W + 2 * pad_w - dil * (KW - 1);
  if (g.Ho <= 0 || g.Wo <= 0 || N <= 0) return refuse("conv: empty output %dx%d", g.Ho, g.Wo);
  pick_patch(g.Ho, g.Wo, kBM, &g.Ht, &g.Wt);
  g.h_tiles = ceil_div(g.Ho, g.Ht);
  g.w_tiles = ceil_div(g.Wo, g.Wt);
  CUtensorMap tmX, tmW;
  if (encode_nhwc(&tmX, x, N, H, W, Cp, g.Ht, g.Wt)) return -1;
  const int bn = Cop % 128 == 0 ? 128 : 64;
  {
    uint64_t dims[2] = {static_cast<uint64_t>(KH) * KW * Cp, static_cast<uint64_t>(w_rows)};
    uint64_t strides[1] = {static_cast<uint64_t>(KH) * KW * Cp * 2};
    uint32_t box[2] = {kBK, static_cast<uint32_t>(bn)};
    if (encode_tmap(&tmW, w, 2, 2, dims, strides, box, 3)) return -1;
  }
  return bn == 128 ? launch_conv_fwd<128, 6>(tmX, tmW, g, y, bias, relu, st)
                   : launch_conv_fwd<64, 8>(tmX, tmW, g, y, bias, relu, st);
}

// dw[Co][KH*KW*Cp] (fp32) (+)= sum over pixels of dy[N,Ho,Wo,Cop] (x) x[N,H,W,Cp] windows, stride 1.
// part: fp32 scratch of splits * Co * KH*KW*Cp values; splits <= 0 picks one that fills the GPU.
MIMIR_API int mimir_conv2d_wgrad(const void* dy, const void* x, float* dw, float* part, long long part_floats, int N,
                                 int H, int W, int Cp, int Cop, int Co, int KH, int KW, int pad_h, int pad_w, int dil,
                                 int splits, int accumulate, cudaStream_t st) {
  if (Cp % 64 || Cop % 64) return refuse("conv: channel counts %d, %d must be multiples of 64", Cp, Cop);
  if (Co > Cop || Co <= 0) return refuse("conv: %d output channels do not fit the padded %d", Co, Cop);
  ConvGeom g;
  g.N = N; g.H = H; g.W = W; g.Cp = Cp; g.Cop = Cop; g.KH = KH; g.KW = KW; g.pad_h = pad_h; g.pad_w = pad_w; g.dil = dil;
  g.Ho = H + 2 * pad_h - dil * (KH - 1);
  g.Wo = W + 2 * pad_w - dil * (KW - 1);
  if (g.Ho <= 0 || g.Wo <= 0 || N <= 0) return refuse("conv: empty output %dx%d", g.Ho, g.Wo);
  pick_patch(g.Ho, g.Wo, kBK, &g.Ht, &g.Wt);
  g.h_tiles = ceil_div(g.Ho, g.Ht);
  g.w_tiles = ceil_div(g.Wo, g.Wt);
  const int bn = Cp % 128 == 0 ? 128 : 64;
  const int patches = N * g.h_tiles * g.w_tiles;
  const long long per_split = static_cast<long long>(Co) * KH * KW * Cp;
  if (splits <= 0) {
    const int base_units = KH * KW * ceil_div(Cop, kBM) * (Cp / bn);
    splits = ceil_div(2 * sm_count(), base_units);
    if (splits > patches / 4) splits = patches / 4;
    if (splits < 1) splits = 1;
  }
  if (splits > patches) splits = patches;
  while (splits > 1 && static_cast<long long>(splits) * per_split > part_floats) --splits;
  if (static_cast<long long>(splits) * per_split > part_floats) return refuse("conv: weight-gradient scratch too small");
  while (splits > 1 && ceil_div(patches, splits) * (splits - 1) >= patches) --splits;
  CUtensorMap tmDy, tmX;
  if (encode_nhwc(&tmDy, dy, N, g.Ho, g.Wo, Cop, g.Ht, g.Wt)) return -1;
  if (encode_nhwc(&tmX, x, N, H, W, Cp, g.Ht, g.Wt)) return -1;
  const int rc = bn == 128 ? launch_conv_wgrad<128, 6>(tmDy, tmX, g, part, Co, splits, st)
                           : launch_conv_wgrad<64, 8>(tmDy, tmX, g, part, Co, splits, st);
  if (rc) return rc;
  const size_t n4 = static_cast<size_t>(per_split) / 4;
  conv_wgrad_reduce_kernel<<<static_cast<unsigned>((n4 + 255) / 256), 256, 0, st>>>(part, dw, n4, splits, accumulate);
  count_launch();
  return 0;
}

MIMIR_API int mimir_maxpool2d_fwd(const void* x, void* y, void* arg, int N, int H, int W, int C, int k, int s,
                                  cudaStream_t st) {
  if (C % 8 || k < 1 || s < 1 || k > 15) return refuse("maxpool: C %% 8 == 0 and 1 <= k <= 15 required");
  const int Ho = (H - k) / s + 1, Wo = (W - k) / s + 1;
  if (Ho <= 0 || Wo <= 0) return refuse("maxpool: window larger than the image");
  const size_t n = static_cast<size_t>(N) * Ho * Wo * (C / 8);
  maxpool_fwd_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), static_cast<uint8_t*>(arg), N, H, W, C, Ho, Wo,
      k, s);
  count_launch();
  return 0;
}
MIMIR_API int mimir_maxpool2d_bwd(const void* dy, const void* arg, void* dx, int N, int H, int W, int C, int k, int s,
                                  cudaStream_t st) {
  if (C % 8 || k < 1 || s < 1 || k > 15) return refuse("maxpool: C %% 8 == 0 and 1 <= k <= 15 required");
  const int Ho = (H - k) / s + 1, Wo = (W - k) / s + 1;
  const size_t n = static_cast<size_t>(N) * H * W * (C / 8);
  maxpool_bwd_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const uint8_t*>(arg), static_cast<__nv_bfloat16*>(dx), N, H, W, C,
      Ho, Wo, k, s);
  count_launch();
  return 0;
}
MIMIR_API int mimir_relu_bwd(const void* y, const void* dy, void* dx, long long n, cudaStream_t st) {
  if (n % 8) return refuse("relu_bwd: element count must be a multiple of 8");
  const size_t n8 = static_cast<size_t>(n / 8);
  relu_bwd_kernel<<<static_cast<unsigned>((n8 + 255) / 256), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(dy), static_cast<__nv_bfloat16*>(dx), n8);
  count_launch();
  return 0;
}
