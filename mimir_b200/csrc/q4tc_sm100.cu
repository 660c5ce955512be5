// Q4_0 weights x bf16 activations on the tcgen05 tensor cores, for decode batches
// (1..32 rows): out[b][n] = sum_k W[n][k] * x[b][k].
//
// The weight matrix is the MMA's M side (128 rows per tile), the batch its N side
// (16 or 32 columns), so a single instruction stream covers every row of the batch
// and the kernel stays bound by the 4.5-bit weight stream, not by arithmetic:
//
//   warp 0       bulk-copies raw weight tiles (4608 bytes per k-block: 2 x 128 x 16-byte quants +
//                2 x 128 fp16 scales), four k-blocks per copy, into a 6-deep shared-memory ring:
//                the weight stream is the only HBM traffic
//   warps 4..11  expand a raw tile to bf16 in the 128-byte-swizzled K-major layout the
//                tensor core reads (nibble -> 128 + n via a byte permute, -136, x scale) and
//                copy the k-block's activation tile [batch x 64] (L2 resident) beside it;
//                two groups of four warps take k-blocks in turn, because one tile's
//                expansion is a latency chain (shared load, convert, store, proxy fence)
//   warp 1       issues tcgen05.mma (accumulator 128 x batch in TMEM, double-buffered)
//   warps 12..15 read the accumulator and write fp32 partials [split][b][n]
//
// Work is split over (row tile, k range) so that every SM streams weights; after the
// main loop all blocks meet (they are co-resident: the grid never exceeds the SM
// count), optionally exchange flags with the other tensor-parallel ranks, and each
// block sums its slice of the output over the k-splits and the ranks' partial
// buffers (plain peer loads), adds the residual and writes bf16 or fp32.
// Every wait is bounded.
//
// Weight storage ("tiled Q4_0"): tile (row tile i, k-block j) is 4608 contiguous
// bytes at (i * K/64 + j) * 4608: quants[2][128][16] then scales[2][128] (fp16).
//
// Replaces the reference's SIMT qmatmul (backend/internal/gen/quant.go:163-209).
#include "quant_common.cuh"

namespace mimir {

constexpr int kTcRows = 128;
constexpr int kTcBK = 64;
constexpr int kTcRawBytes = 2 * kTcRows * 16 + 2 * kTcRows * 2;  // 4608
constexpr int kTcSub = 4;         // k-blocks per bulk copy (18 KB)
constexpr int kTcRawStages = 6;   // bulk copies in flight: ~110 KB per SM covers HBM latency at full bandwidth
constexpr int kTcAStages = 4;
constexpr int kTcGroups = 2;  // groups of four expanding warps; group g owns the k-blocks it % kTcGroups == g
constexpr int kTcThreads = (4 + 4 * kTcGroups + 4) * 32;

__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

struct TcTail {
  float* partial[kQMaxRanks];  // every rank's partial buffer [splits][B][N]
  unsigned* sig[kQMaxRanks];   // every rank's signal pad (only [rank] is used when world == 1)
  unsigned* epoch;
  unsigned* block_counter;
  const __nv_bfloat16* residual;
  __nv_bfloat16* out_bf16;
  float* out_f32;
  int ldo;
  int rank, world, slot;
  unsigned long long wait_ns;
};

// 8 nibbles of `w` selected by `shift` (0: low nibbles = values j, 4: high nibbles = values 16 + j)
// -> 4 bf16x2 words scaled by d2 = (d, d).
__device__ __forceinline__ void expand8(uint32_t w, int shift, __nv_bfloat162 d2, uint32_t (&o)[2]) {
  const uint32_t n = (w >> shift) & 0x0F0F0F0Fu;
  const uint32_t p0 = __byte_perm(n, 0x43434343u, 0x4140);  // (128 + n0, 128 + n1) as bf16x2
  const uint32_t p1 = __byte_perm(n, 0x43434343u, 0x4342);  // (128 + n2, 128 + n3)
  const __nv_bfloat162 c = __float2bfloat162_rn(136.f);
  __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&p0);
  __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&p1);
  a = __hmul2(__hsub2(a, c), d2);  // n - 8 is exact; one rounding in the product
  b = __hmul2(__hsub2(b, c), d2);
  o[0] = *reinterpret_cast<uint32_t*>(&a);
  o[1] = *reinterpret_cast<uint32_t*>(&b);
}

template <int BNB>
__global__ void __launch_bounds__(kTcThreads, 1)
q4_tc_kernel(const uint8_t* __restrict__ wt, const __nv_bfloat16* __restrict__ x, int ldx, TcTail tail, int N, int K,
             int B, int splits, unsigned* err) {
  constexpr int A_BYTES = kTcRows * kTcBK * 2;  // 16 KB expanded weight tile
  constexpr int ASTAGE = A_BYTES + 4096;        // + activation tile [BNB x 64] bf16 (1024-byte aligned slot)
  constexpr int BIG = kTcSub * kTcRawBytes;     // one bulk copy: the raw tiles of kTcSub consecutive k-blocks
  constexpr uint32_t TMEM_COLS = 2 * BNB < 32 ? 32 : 2 * BNB;
  constexpr uint32_t IDESC = make_idesc_bf16(kTcRows, BNB, false, false);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* a_ring = smem;                                    // kTcAStages x (weight tile | activation tile)
  uint8_t* raw_ring = smem + kTcAStages * ASTAGE;            // kTcRawStages x BIG
  uint64_t* raw_full = reinterpret_cast<uint64_t*>(raw_ring + kTcRawStages * BIG);
  uint64_t* raw_empty = raw_full + kTcRawStages;
  uint64_t* a_full = raw_empty + kTcRawStages;
  uint64_t* a_empty = a_full + kTcAStages;
  uint64_t* tfull = a_empty + kTcAStages;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = (N + kTcRows - 1) / kTcRows;
  const int kb_total = K / kTcBK;
  const int kb_per = (kb_total + splits - 1) / splits;
  const int units = n_tiles * splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kTcRawStages; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&raw_empty[s], 4 * kTcGroups);  // every expanding warp arrives once per bulk stage
    }
    for (int s = 0; s < kTcAStages; ++s) {
      mbar_init(&a_full[s], 4);                 // the four warps of the group that filled the stage
      mbar_init(&a_empty[s], 1);
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
    if (lane == 0) {  // raw weight tiles: one bulk copy per kTcSub k-blocks (the copy engine takes a fixed
                      // time per request, so small requests cap the bandwidth of an SM)
      uint32_t bit = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
        const int split = u % splits, tile = u / splits;
        const int kb0 = split * kb_per, kb1 = min(kb_total, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; kb += kTcSub, ++bit) {
          const int nsub = min(kTcSub, kb1 - kb);
          const int s = bit % kTcRawStages;
          const uint32_t ph = (bit / kTcRawStages) & 1;
          if (!mbar_wait(&raw_empty[s], ph ^ 1, abort_flag, err)) { ok = false; break; }
          mbar_arrive_expect_tx(&raw_full[s], nsub * kTcRawBytes);
          bulk_load_1d(raw_ring + s * BIG, wt + (static_cast<size_t>(tile) * kb_total + kb) * kTcRawBytes,
                       nsub * kTcRawBytes, &raw_full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t it = 0, ti = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < units && ok; u += gridDim.x, ++ti) {
        const int split = u % splits;
        const int kb0 = split * kb_per, kb1 = min(kb_total, kb0 + kb_per);
        const uint32_t acc = ti & 1, acc_ph = (ti >> 1) & 1;
        if (!mbar_wait(&tempty[acc], acc_ph ^ 1, abort_flag, err)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BNB;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % kTcAStages;
          const uint32_t ph = (it / kTcAStages) & 1;
          if (!mbar_wait(&a_full[s], ph, abort_flag, err)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sA = smem_u32(a_ring + s * ASTAGE);
          const uint64_t adesc = make_smem_desc_sw128(sA, 16, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(sA + A_BYTES, 16, 1024);
#pragma unroll
          for (int k = 0; k < kTcBK / 16; ++k)
            umma_ss(d_tmem, adesc + k * 2, bdesc + k * 2, IDESC, (kb > kb0 || k > 0) ? 1u : 0u);
          umma_commit(&a_empty[s]);
        }
        if (ok) umma_commit(&tfull[acc]);
      }
    }
  } else if (warp >= 4 && warp < 4 + 4 * kTcGroups) {
    // expand raw Q4_0 tiles to bf16 and stage the activation tile; thread t of the group owns row t
    const int group = (warp - 4) >> 2;
    const int t = ((warp - 4) & 3) * 32 + lane;
    uint32_t it = 0, bit = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
      const int split = u % splits;
      const int kb0 = split * kb_per, kb1 = min(kb_total, kb0 + kb_per);
      for (int kbb = kb0; kbb < kb1 && ok; kbb += kTcSub, ++bit) {
        const int nsub = min(kTcSub, kb1 - kbb);
        const int sb = bit % kTcRawStages;
        const uint32_t phb = (bit / kTcRawStages) & 1;
        bool waited = false;
        for (int j = 0; j < nsub; ++j) {
          const uint32_t itc = it + j;
          if (static_cast<int>(itc % kTcGroups) != group) continue;
          const int kb = kbb + j;
          // activation chunks (16 bytes = 8 values) this thread stages: chunk c = row * 8 + column chunk
          uint4 xv[BNB / 16];
#pragma unroll
          for (int c2 = 0; c2 < BNB / 16; ++c2) {
            const int c = t + c2 * 128, row = c >> 3;
            xv[c2] = row < B ? *reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * ldx + kb * kTcBK + (c & 7) * 8)
                             : make_uint4(0u, 0u, 0u, 0u);
          }
          if (!waited) {
            if (!mbar_wait(&raw_full[sb], phb, abort_flag, err)) { ok = false; break; }
            waited = true;
          }
          const int sa = itc % kTcAStages;
          const uint32_t pha = (itc / kTcAStages) & 1;
          if (!mbar_wait(&a_empty[sa], pha ^ 1, abort_flag, err)) { ok = false; break; }
          const uint8_t* raw = raw_ring + sb * BIG + j * kTcRawBytes;
          uint8_t* stage = a_ring + sa * ASTAGE;
          uint8_t* arow = stage + t * 128;
#pragma unroll
          for (int blk = 0; blk < 2; ++blk) {
            const uint4 q = *reinterpret_cast<const uint4*>(raw + (blk * kTcRows + t) * 16);
            const __half dh = *reinterpret_cast<const __half*>(raw + 2 * kTcRows * 16 + (blk * kTcRows + t) * 2);
            const __nv_bfloat162 d2 = __float2bfloat162_rn(__half2float(dh));
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
            // values 0..7 | 8..15 from the low nibbles of words 0,1 | 2,3; 16..23 | 24..31 from the high ones
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t lo[2], hi[2];
              expand8(w[(c & 1) * 2], (c >> 1) * 4, d2, lo);
              expand8(w[(c & 1) * 2 + 1], (c >> 1) * 4, d2, hi);
              const int chunk = (blk * 4 + c) ^ (t & 7);  // 128-byte swizzle of the 16-byte chunks
              *reinterpret_cast<uint4*>(arow + chunk * 16) = make_uint4(lo[0], lo[1], hi[0], hi[1]);
            }
          }
#pragma unroll
          for (int c2 = 0; c2 < BNB / 16; ++c2) {
            const int c = t + c2 * 128, row = c >> 3;
            *reinterpret_cast<uint4*>(stage + A_BYTES + row * 128 + (((c & 7) ^ (row & 7)) << 4)) = xv[c2];
          }
          fence_proxy_async_smem();  // the tensor core reads both tiles through the async proxy
          __syncwarp();
          if (lane == 0) mbar_arrive(&a_full[sa]);
        }
        it += nsub;
        __syncwarp();
        if (ok && lane == 0) mbar_arrive(&raw_empty[sb]);
      }
    }
  } else if (warp >= 4 + 4 * kTcGroups) {
    const int q = warp & 3;
    uint32_t ti = 0;
    float* mine = tail.partial[tail.rank];
    for (int u = blockIdx.x; u < units; u += gridDim.x, ++ti) {
      const int split = u % splits, tile = u / splits;
      const int kb0 = split * kb_per, kb1 = min(kb_total, kb0 + kb_per);
      const uint32_t acc = ti & 1, acc_ph = (ti >> 1) & 1;
      if (!mbar_wait(&tfull[acc], acc_ph, abort_flag, err)) break;
      tc_fence_after();
      const int n = tile * kTcRows + q * 32 + lane;
      const uint32_t taddr = tmem_base + acc * BNB + (static_cast<uint32_t>(q * 32) << 16);
      uint32_t r[BNB];
      if constexpr (BNB == 32) tmem_ld32(taddr, r); else tmem_ld16(taddr, r);
      tmem_ld_wait();
      if (n < N) {
        const bool any = kb1 > kb0;
#pragma unroll
        for (int b = 0; b < BNB; ++b)
          if (b < B) mine[(static_cast<size_t>(split) * B + b) * N + n] = any ? __uint_as_float(r[b]) : 0.f;
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

  // ---- all blocks (and, with world > 1, all ranks) meet, then reduce ----------------------
  __shared__ unsigned s_last;
  __shared__ int s_ok;
  const unsigned epoch = *tail.epoch + 1;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    s_ok = *abort_flag ? 0 : 1;
    s_last = atomicAdd(tail.block_counter, 1u) == gridDim.x - 1 ? 1u : 0u;
  }
  __syncthreads();
  if (s_last && threadIdx.x < tail.world) {
    __threadfence_system();
    st_release_sys_u32(tail.sig[threadIdx.x] + tail.slot * kQMaxRanks + tail.rank, epoch);
  }
  if (threadIdx.x < tail.world) {
    if (!wait_flag_ge(tail.sig[tail.rank] + tail.slot * kQMaxRanks + threadIdx.x, epoch, tail.wait_ns, err)) s_ok = 0;
  }
  __syncthreads();
  if (s_ok) {
    const int n4 = N / 4, total4 = B * n4;
    const size_t split_stride = static_cast<size_t>(B) * N;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += gridDim.x * blockDim.x) {
      const int b = i / n4, c = (i % n4) * 4;
      float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int r = 0; r < kQMaxRanks; ++r) {
        if (r < tail.world) {
          for (int sp = 0; sp < splits; ++sp) {
            const float4 v = ld_sys_f4(tail.partial[r] + sp * split_stride + static_cast<size_t>(b) * N + c);
            s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
          }
        }
      }
      if (tail.residual) {
        const uint2 rr = *reinterpret_cast<const uint2*>(tail.residual + static_cast<size_t>(b) * tail.ldo + c);
        const float2 r0 = unpack_bf16x2(rr.x), r1 = unpack_bf16x2(rr.y);
        s.x += r0.x; s.y += r0.y; s.z += r1.x; s.w += r1.y;
      }
      if (tail.out_f32) {
        *reinterpret_cast<float4*>(tail.out_f32 + static_cast<size_t>(b) * tail.ldo + c) = s;
      } else {
        uint2 o;
        o.x = pack_bf16x2(s.x, s.y);
        o.y = pack_bf16x2(s.z, s.w);
        *reinterpret_cast<uint2*>(tail.out_bf16 + static_cast<size_t>(b) * tail.ldo + c) = o;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned done = atomicAdd(tail.block_counter, 1u);
    if (done == 2 * gridDim.x - 1) {  // the last block to finish re-arms the counter and advances the epoch
      *tail.block_counter = 0;
      __threadfence();
      *tail.epoch = epoch;
    }
  }
}

// Activation rounding to Q8_0 (32-value blocks, scale = max|x| / 127) written back as bf16
// (q * scale), fused with RMSNorm (mode 1) or SwiGLU of a [rows][2K] gate|up matrix (mode 2).
// One block per (row, 2048-column slab); 8 values per thread, a Q8_0 block is 4 lanes.
__global__ void __launch_bounds__(256)
round_act_q8_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                    __nv_bfloat16* __restrict__ y, int ldy, int8_t* __restrict__ xq, float* __restrict__ xs, int K,
                    int mode, float eps) {
  const int row = blockIdx.y;
  const int ld = mode == 2 ? 2 * K : K;
  const __nv_bfloat16* xr = x + static_cast<size_t>(row) * ld;
  __shared__ float s_part[8];
  float rstd = 1.f;
  if (mode == 1) {  // every block of the row computes the row's sum of squares (K is small)
    float s = 0.f;
    for (int c = threadIdx.x * 8; c < K; c += 256 * 8) {
      const uint4 v = *reinterpret_cast<const uint4*>(xr + c);
      const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), cc = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
      s += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y + cc.x * cc.x + cc.y * cc.y + d.x * d.x + d.y * d.y;
    }
    s = warp_sum_f(s);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = s;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) tot += s_part[w];
    rstd = rsqrtf(tot / K + eps);
  }
  const int c = (blockIdx.x * 256 + threadIdx.x) * 8;
  if (c >= K) return;  // K % 32 == 0, so the four lanes of a Q8_0 block leave together
  float v[8];
  {
    const uint4 u = *reinterpret_cast<const uint4*>(xr + c);
    const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), cc = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = cc.x; v[5] = cc.y; v[6] = d.x; v[7] = d.y;
  }
  if (mode == 1) {
    const uint4 gu = *reinterpret_cast<const uint4*>(gamma + c);
    const float2 a = unpack_bf16x2(gu.x), b = unpack_bf16x2(gu.y), cc = unpack_bf16x2(gu.z), d = unpack_bf16x2(gu.w);
    const float g[8] = {a.x, a.y, b.x, b.y, cc.x, cc.y, d.x, d.y};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float t = __bfloat162float(__float2bfloat16_rn(v[j] * rstd)) * g[j];
      v[j] = __bfloat162float(__float2bfloat16_rn(t));
    }
  } else if (mode == 2) {
    const uint4 u = *reinterpret_cast<const uint4*>(xr + K + c);
    const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), cc = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
    const float up[8] = {a.x, a.y, b.x, b.y, cc.x, cc.y, d.x, d.y};
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = v[j] / (1.f + __expf(-v[j])) * up[j];
  }
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  const float d = amax / 127.f, inv = d > 0.f ? 1.f / d : 0.f;
  if (y) {
    uint4 o;
    o.x = pack_bf16x2(rintf(v[0] * inv) * d, rintf(v[1] * inv) * d);
    o.y = pack_bf16x2(rintf(v[2] * inv) * d, rintf(v[3] * inv) * d);
    o.z = pack_bf16x2(rintf(v[4] * inv) * d, rintf(v[5] * inv) * d);
    o.w = pack_bf16x2(rintf(v[6] * inv) * d, rintf(v[7] * inv) * d);
    *reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * ldy + c) = o;
  }
  if (xq) {   // planar Q8_0 for the integer dot-product path: int8 values and one fp32 scale per 32
    int q[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) q[j] = __float2int_rn(v[j] * inv);
    uint2 pk;
    pk.x = (q[0] & 0xff) | ((q[1] & 0xff) << 8) | ((q[2] & 0xff) << 16) | ((q[3] & 0xff) << 24);
    pk.y = (q[4] & 0xff) | ((q[5] & 0xff) << 8) | ((q[6] & 0xff) << 16) | ((q[7] & 0xff) << 24);
    *reinterpret_cast<uint2*>(xq + static_cast<size_t>(row) * K + c) = pk;
    if ((threadIdx.x & 3) == 0) xs[static_cast<size_t>(row) * (K / 32) + c / 32] = d;
  }
}

template <int BNB>
static int launch_q4_tc(const uint8_t* wt, const __nv_bfloat16* x, int ldx, const TcTail& tail, int N, int K, int B,
                        int splits, cudaStream_t st) {
  constexpr int SMEM = kTcAStages * (kTcRows * kTcBK * 2 + 4096) + kTcRawStages * kTcSub * kTcRawBytes + 1024 + 1024;
  auto kern = q4_tc_kernel<BNB>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
      return refuse("q4 tensor-core product: cannot reserve %d bytes of shared memory", SMEM);
    configured = true;
  }
  const int units = ceil_div(N, kTcRows) * splits;
  const int grid = units < sm_count() ? units : sm_count();  // one block per SM: all blocks are resident
  kern<<<grid, kTcThreads, SMEM, st>>>(wt, x, ldx, tail, N, K, B, splits, error_word_dev());
  count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : refuse("q4 tensor-core product: launch failed");
}

}  // namespace mimir

using namespace mimir;

// planar Q4_0 (scales [N][K/32] fp16, quants [N][K/32][16]) -> tiled layout; one thread per (tile, block, row)
__global__ void q4_planar_to_tiled_kernel(const __half* __restrict__ ws, const uint4* __restrict__ wq,
                                          uint8_t* __restrict__ out, int N, int K) {
  const int kb_total = K / kTcBK, n_tiles = (N + kTcRows - 1) / kTcRows;
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<size_t>(n_tiles) * kb_total * 2 * kTcRows) return;
  const int row = static_cast<int>(idx % kTcRows);
  const int blk = static_cast<int>((idx / kTcRows) % 2);
  const int kb = static_cast<int>((idx / (2 * kTcRows)) % kb_total);
  const int tile = static_cast<int>(idx / (2 * kTcRows * static_cast<size_t>(kb_total)));
  const int n = tile * kTcRows + row;
  uint8_t* base = out + (static_cast<size_t>(tile) * kb_total + kb) * kTcRawBytes;
  uint4 q = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);
  __half d = __float2half(0.f);
  if (n < N) {
    const size_t src = static_cast<size_t>(n) * (K / 32) + kb * 2 + blk;
    q = wq[src];
    d = ws[src];
  }
  *reinterpret_cast<uint4*>(base + (blk * kTcRows + row) * 16) = q;
  *reinterpret_cast<__half*>(base + 2 * kTcRows * 16 + (blk * kTcRows + row) * 2) = d;
}

MIMIR_API long long mimir_q4_tiled_bytes(int N, int K) {
  return static_cast<long long>(ceil_div(N, kTcRows)) * (K / kTcBK) * kTcRawBytes;
}
MIMIR_API int mimir_q4_planar_to_tiled(const void* ws, const void* wq, void* out, int N, int K, cudaStream_t st) {
  if (K % kTcBK) return refuse("tiled Q4_0: K must be a multiple of 64");
  const size_t n = static_cast<size_t>(ceil_div(N, kTcRows)) * (K / kTcBK) * 2 * kTcRows;
  q4_planar_to_tiled_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, st>>>(
      static_cast<const __half*>(ws), static_cast<const uint4*>(wq), static_cast<uint8_t*>(out), N, K);
  count_launch();
  return 0;
}

// y[rows][K] bf16 (row pitch ldy) = Q8_0-rounded activation (mode 0), of RMSNorm(x) * gamma (mode 1), or of
// silu(gate) * up for x = [rows][2K] (mode 2).  x rows are contiguous.
// xq / xs (both or neither): also the planar Q8_0 form, int8 [rows][K] and fp32 scales [rows][K/32]; y may be null then.
MIMIR_API int mimir_round_act_q8(const void* x, const void* gamma, void* y, int ldy, void* xq, float* xs, int rows, int K,
                                 int mode, float eps, cudaStream_t st) {
  if ((xq == nullptr) != (xs == nullptr) || (!y && !xq)) return refuse("activation rounding: no output given");
  if (K % 32 || ldy % 8) return refuse("activation rounding: K %% 32 == 0 and ldy %% 8 == 0 required");
  if (mode == 1 && !gamma) return refuse("activation rounding: RMSNorm needs gamma");
  dim3 grid(ceil_div(K, 2048), rows);
  round_act_q8_kernel<<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(gamma),
                                            static_cast<__nv_bfloat16*>(y), ldy, static_cast<int8_t*>(xq), xs, K, mode, eps);
  count_launch();
  return 0;
}

// out[b][n] (row pitch ldo; bf16, or fp32 when out_is_f32) = residual[b][n] + sum over ranks and k
// of W[n][k] x[b][k].  wt: tiled Q4_0 weights [N][K]; x: bf16 [B][K] (row pitch ldx), B <= 32.
// partial[r]: rank r's scratch of splits * B * N floats (peer-mapped when world > 1); sig[r]: rank r's
// signal pad; epoch / block_counter: device words of this slot.  N % 4 == 0, K % 64 == 0.
// splits <= 0 picks the k-split that fills the GPU (at most max_splits, which sizes `partial`).
MIMIR_API int mimir_q4_tc(const void* wt, const void* x, int ldx, void* const* partial, void* const* sig, void* epoch,
                          void* block_counter, const void* residual, void* out, int out_is_f32, int ldo, int N, int K,
                          int B, int splits, int max_splits, int rank, int world, int slot, cudaStream_t st) {
  if (B < 1 || B > 32) return refuse("q4 tensor-core product: batch %d outside 1..32", B);
  if (N % 4 || K % kTcBK || ldx % 8 || ldo % 4) return refuse("q4 tensor-core product: N %% 4, K %% 64, ldx %% 8, ldo %% 4 required");
  if (world < 1 || world > kQMaxRanks) return refuse("q4 tensor-core product: world %d outside 1..%d", world, kQMaxRanks);
  const int n_tiles = ceil_div(N, kTcRows), kb_total = K / kTcBK;
  if (splits <= 0) {
    // the makespan of a persistent grid is ceil(units / SMs) units of 1/splits of a row tile each;
    // a split costs one more partial to write and to sum
    const int sms = sm_count();
    int lim = kb_total / 4 < max_splits ? kb_total / 4 : max_splits;  // at least four k-blocks per unit
    if (lim < 1) lim = 1;
    double best = 1e30;
    splits = 1;
    for (int sp = 1; sp <= lim; ++sp) {
      const double cost = static_cast<double>(ceil_div(n_tiles * sp, sms)) / sp + (0.01 + 0.002 * B) * sp;
      if (cost < best - 1e-9) { best = cost; splits = sp; }
    }
  }
  if (splits > max_splits) splits = max_splits;
  if (splits < 1) splits = 1;
  while (splits > 1 && ceil_div(kb_total, splits) * (splits - 1) >= kb_total) --splits;
  const int bnb = B <= 16 ? 16 : 32;
  TcTail t;
  for (int r = 0; r < kQMaxRanks; ++r) {
    t.partial[r] = r < world ? static_cast<float*>(partial[r]) : nullptr;
    t.sig[r] = r < world ? static_cast<unsigned*>(sig[r]) : nullptr;
  }
  t.epoch = static_cast<unsigned*>(epoch);
  t.block_counter = static_cast<unsigned*>(block_counter);
  t.residual = static_cast<const __nv_bfloat16*>(residual);
  t.out_bf16 = out_is_f32 ? nullptr : static_cast<__nv_bfloat16*>(out);
  t.out_f32 = out_is_f32 ? static_cast<float*>(out) : nullptr;
  t.ldo = ldo;
  t.rank = rank; t.world = world; t.slot = slot; t.wait_ns = q_peer_wait_ns();
  const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(x);
  return bnb == 16 ? launch_q4_tc<16>(static_cast<const uint8_t*>(wt), xb, ldx, t, N, K, B, splits, st)
                   : launch_q4_tc<32>(static_cast<const uint8_t*>(wt), xb, ldx, t, N, K, B, splits, st);
}
