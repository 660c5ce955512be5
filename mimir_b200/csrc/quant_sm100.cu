// Quantized inference kernels.
//
// * dequantise Q8_0 / Q4_0 / Q4_K / Q6_K blocks (ggml layouts, same arithmetic as
//   the reference's dq_T helpers, backend/internal/gen/quant.go:41-131)
// * activation quantisation to Q8_0 fused with RMSNorm or SwiGLU
// * W4A8 product: Q4_0 weights x Q8_0 activations with int8 dot products (dp4a),
//   one warp per output row, every batch row reusing the weight registers
//   (replaces the reference's qmatmul, quant.go:163-209, which dequantises to fp32)
// * the same product fused with the tensor-parallel all-reduce: partial sums go
//   to a symmetric buffer, the last block signals the peers, and every block then
//   reduces a slice over all ranks' buffers by plain peer loads (one-shot), adds
//   the residual and writes the bf16 hidden state.  Waits on peers are bounded.
//
// GPU weight layout ("planar Q4_0"): the 18-byte ggml blocks of a [N, K] matrix
// are split at load time into scales[N][K/32] (fp16) and quants[N][K/32][16 bytes]
// so that a lane reads one aligned 16-byte vector per block.
#include "quant_common.cuh"

namespace mimir {

__device__ __forceinline__ float half_bits_to_float(uint16_t h) { return __half2float(__ushort_as_half(h)); }

// ---------------------------------------------------------------------------
// dequantise: one thread per output element (simple; off the hot path)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void q4k_scale_min(int j, const uint8_t* q, int& sc, int& mn) {
  if (j < 4) { sc = q[j] & 63; mn = q[j + 4] & 63; }
  else { sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4); mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
}

__global__ void dequant_kernel(int code, const uint8_t* __restrict__ raw, float* __restrict__ out, size_t n) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float v = 0.f;
  if (code == 64) {  // Q8_0
    const uint8_t* b = raw + (i / 32) * 34;
    v = half_bits_to_float(b[0] | (b[1] << 8)) * static_cast<float>(static_cast<int8_t>(b[2 + i % 32]));
  } else if (code == 65) {  // Q4_0
    const uint8_t* b = raw + (i / 32) * 18;
    const int j = static_cast<int>(i % 32);
    const int q = j < 16 ? (b[2 + j] & 0xF) : (b[2 + j - 16] >> 4);
    v = half_bits_to_float(b[0] | (b[1] << 8)) * static_cast<float>(q - 8);
  } else if (code == 66) {  // Q4_K
    const uint8_t* b = raw + (i / 256) * 144;
    const int j = static_cast<int>(i % 256), sub = j / 32, pair = sub / 2;
    const float d = half_bits_to_float(b[0] | (b[1] << 8)), dmin = half_bits_to_float(b[2] | (b[3] << 8));
    int sc, mn;
    q4k_scale_min(sub, b + 4, sc, mn);
    const uint8_t qq = b[16 + pair * 32 + j % 32];
    const int q = (sub & 1) ? (qq >> 4) : (qq & 0xF);
    v = d * sc * q - dmin * mn;
  } else if (code == 67) {  // Q6_K
    const uint8_t* b = raw + (i / 256) * 210;
    const int j = static_cast<int>(i % 256), half = j / 128, r = j % 128, quarter = r / 32, l = r % 32;
    const uint8_t* ql = b + 64 * half;
    const uint8_t* qh = b + 128 + 32 * half;
    const int8_t* sc = reinterpret_cast<const int8_t*>(b + 192) + 8 * half;
    const float d = half_bits_to_float(b[208] | (b[209] << 8));
    const int lo = quarter == 0 ? (ql[l] & 0xF) : quarter == 1 ? (ql[l + 32] & 0xF) : quarter == 2 ? (ql[l] >> 4) : (ql[l + 32] >> 4);
    const int hi = (qh[l] >> (2 * quarter)) & 3;
    v = d * sc[l / 16 + 2 * quarter] * ((lo | (hi << 4)) - 32);
  }
  out[i] = v;
}

// ggml Q4_0 blocks [nblocks][18] -> planar scales (fp16) + quants (16 bytes per block)
__global__ void q4_0_to_planar_kernel(const uint8_t* __restrict__ raw, __half* __restrict__ scales,
                                      uint4* __restrict__ quants, size_t nblocks) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= nblocks) return;
  const uint8_t* b = raw + i * 18;
  scales[i] = __ushort_as_half(static_cast<uint16_t>(b[0] | (b[1] << 8)));
  uint32_t w[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) w[k] = b[2 + 4 * k] | (b[3 + 4 * k] << 8) | (b[4 + 4 * k] << 16) | (b[5 + 4 * k] << 24);
  quants[i] = make_uint4(w[0], w[1], w[2], w[3]);
}

// ---------------------------------------------------------------------------
// Activation quantisation to planar Q8_0: xq [rows][K] int8, xs [rows][K/32] float.
// One warp per row.  mode 0: plain; mode 1: RMSNorm(x) * gamma first (also writes
// the normalised bf16 row when y != nullptr); mode 2: input is [rows][2K] gate|up,
// quantises silu(gate) * up.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float ld_act(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ float ld_act(const float* p) { return *p; }

template <typename TIn>
__global__ void __launch_bounds__(256)
quantize_act_kernel(const TIn* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                    __nv_bfloat16* __restrict__ y, int8_t* __restrict__ xq, float* __restrict__ xs, int rows,
                    int K, int mode, float eps) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int ld = mode == 2 ? 2 * K : K;
  const TIn* xr = x + static_cast<size_t>(row) * ld;
  float rstd = 1.f;
  if (mode == 1) {
    float s = 0.f;
    for (int c = lane; c < K; c += 32) { float v = ld_act(xr + c); s += v * v; }
    rstd = rsqrtf(warp_sum_f(s) / K + eps);
  }
  // each lane owns one 32-value block per iteration
  for (int blk = lane; blk < K / 32; blk += 32) {
    float v[32];
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const int c = blk * 32 + j;
      float t = ld_act(xr + c);
      if (mode == 1) {
        t = __bfloat162float(__float2bfloat16_rn(t * rstd)) * __bfloat162float(gamma[c]);
        t = __bfloat162float(__float2bfloat16_rn(t));
        if (y) y[static_cast<size_t>(row) * K + c] = __float2bfloat16_rn(t);
      } else if (mode == 2) {
        const float u = ld_act(xr + K + c);
        t = t / (1.f + __expf(-t)) * u;
      }
      v[j] = t;
      amax = fmaxf(amax, fabsf(t));
    }
    const float d = amax / 127.f, inv = d > 0.f ? 1.f / d : 0.f;
    xs[static_cast<size_t>(row) * (K / 32) + blk] = d;
    int8_t* q = xq + static_cast<size_t>(row) * K + blk * 32;
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      char4 c4;
      c4.x = static_cast<signed char>(__float2int_rn(v[j] * inv));
      c4.y = static_cast<signed char>(__float2int_rn(v[j + 1] * inv));
      c4.z = static_cast<signed char>(__float2int_rn(v[j + 2] * inv));
      c4.w = static_cast<signed char>(__float2int_rn(v[j + 3] * inv));
      *reinterpret_cast<char4*>(q + j) = c4;
    }
  }
}

// ---------------------------------------------------------------------------
// W4A8 dot products of one weight row with up to kQMaxBatch activation rows.
// Returns in acc[b] this lane's partial sums (to be warp-reduced by the caller).
// ---------------------------------------------------------------------------
template <int BT>
__device__ __forceinline__ void q4_row_dot(const __half* __restrict__ ws, const uint4* __restrict__ wq,
                                           const int8_t* __restrict__ xq, const float* __restrict__ xs, int K,
                                           int b0, int B, int lane, float (&acc)[BT]) {
  const int nblk = K / 32;
#pragma unroll
  for (int b = 0; b < BT; ++b) acc[b] = 0.f;
  // four blocks per lane and step: the four weight loads are issued before any arithmetic, so a
  // warp keeps 2 KB of the weight stream in flight instead of 512 bytes
  for (int blk0 = lane; blk0 < nblk; blk0 += 128) {
    uint4 qv[4];
    float dwv[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int blk = blk0 + 32 * u;
      const bool live = blk < nblk;
      qv[u] = live ? wq[blk] : make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);
      dwv[u] = live ? __half2float(ws[blk]) : 0.f;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int blk = blk0 + 32 * u;
      if (blk >= nblk) break;
      const uint4 q = qv[u];
      const float dw = dwv[u];
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
      // low nibbles are values 0..15 (bytes 0..15), high nibbles values 16..31
      int lo[4], hi[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        lo[k] = static_cast<int>(w[k] & 0x0F0F0F0Fu);
        hi[k] = static_cast<int>((w[k] >> 4) & 0x0F0F0F0Fu);
      }
#pragma unroll
      for (int b = 0; b < BT; ++b) {
        if (b0 + b < B) {
          const int4* xv = reinterpret_cast<const int4*>(xq + static_cast<size_t>(b0 + b) * K + blk * 32);
          const int4 x0 = xv[0], x1 = xv[1];
          int s = 0, sx = 0;
          s = __dp4a(lo[0], x0.x, s); s = __dp4a(lo[1], x0.y, s); s = __dp4a(lo[2], x0.z, s); s = __dp4a(lo[3], x0.w, s);
          s = __dp4a(hi[0], x1.x, s); s = __dp4a(hi[1], x1.y, s); s = __dp4a(hi[2], x1.z, s); s = __dp4a(hi[3], x1.w, s);
          // the stored nibbles carry an offset of 8: subtract 8 * sum(x)
          sx = __dp4a(0x01010101, x0.x, sx); sx = __dp4a(0x01010101, x0.y, sx); sx = __dp4a(0x01010101, x0.z, sx);
          sx = __dp4a(0x01010101, x0.w, sx); sx = __dp4a(0x01010101, x1.x, sx); sx = __dp4a(0x01010101, x1.y, sx);
          sx = __dp4a(0x01010101, x1.z, sx); sx = __dp4a(0x01010101, x1.w, sx);
          acc[b] += dw * xs[static_cast<size_t>(b0 + b) * nblk + blk] * static_cast<float>(s - 8 * sx);
        }
      }
    }
  }
}

// out[b][n] (fp32, pitch ldo) = sum_k W[n][k] x[b][k]; one warp per row n.
__global__ void __launch_bounds__(256)
q4_gemv_kernel(const __half* __restrict__ ws, const uint4* __restrict__ wq, const int8_t* __restrict__ xq,
               const float* __restrict__ xs, float* __restrict__ out, __nv_bfloat16* __restrict__ out_bf16, int N,
               int K, int B, int ldo) {
  const int lane = threadIdx.x & 31;
  const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (n >= N) return;
  const size_t wb = static_cast<size_t>(n) * (K / 32);
  for (int b0 = 0; b0 < B; b0 += 8) {
    float acc[8];
    q4_row_dot<8>(ws + wb, wq + wb, xq, xs, K, b0, B, lane, acc);
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      const float s = warp_sum_f(acc[b]);
      if (lane == 0 && b0 + b < B) {
        if (out_bf16) out_bf16[static_cast<size_t>(b0 + b) * ldo + n] = __float2bfloat16_rn(s);
        else out[static_cast<size_t>(b0 + b) * ldo + n] = s;
      }
    }
  }
}

// planar Q4_0 [N][K/32] -> bf16 [N][K] (prefill path: dequantise once, then tensor-core GEMM)
__global__ void q4_planar_to_bf16_kernel(const __half* __restrict__ ws, const uint4* __restrict__ wq,
                                         __nv_bfloat16* __restrict__ out, size_t nblocks) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= nblocks) return;
  const float d = __half2float(ws[i]);
  const uint4 q = wq[i];
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
  __nv_bfloat16* o = out + i * 32;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int byte = (w[k] >> (8 * j)) & 0xFF;
      o[4 * k + j] = __float2bfloat16_rn(d * static_cast<float>((byte & 0xF) - 8));
      o[16 + 4 * k + j] = __float2bfloat16_rn(d * static_cast<float>((byte >> 4) - 8));
    }
  }
}

// ---------------------------------------------------------------------------
// GEMV fused with the tensor-parallel all-reduce.
// ---------------------------------------------------------------------------
// All-gather by peer stores: this rank's slice [n bytes] goes to offset rank * n of
// every rank's destination buffer; then flags, then a bounded wait for all ranks.
struct AgArgs {
  uint8_t* dst[kQMaxRanks];
  unsigned* sig[kQMaxRanks];
  unsigned* epoch;
  unsigned* block_counter;
  int rank, world, slot;
  unsigned long long wait_ns;
};
__global__ void __launch_bounds__(256)
peer_allgather_kernel(const uint4* __restrict__ src, AgArgs a, size_t n16, unsigned* err) {
  __shared__ unsigned s_last;
  const unsigned epoch = *a.epoch + 1;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n16;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const uint4 v = src[i];
#pragma unroll
    for (int r = 0; r < kQMaxRanks; ++r)
      if (r < a.world) reinterpret_cast<uint4*>(a.dst[r] + static_cast<size_t>(a.rank) * n16 * 16)[i] = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(a.block_counter, 1u) == gridDim.x - 1 ? 1u : 0u;
  __syncthreads();
  if (s_last) {
    if (threadIdx.x < a.world) {
      __threadfence_system();
      st_release_sys_u32(a.sig[threadIdx.x] + a.slot * kQMaxRanks + a.rank, epoch);
    }
    __syncthreads();
    if (threadIdx.x < a.world) wait_flag_ge(a.sig[a.rank] + a.slot * kQMaxRanks + threadIdx.x, epoch, a.wait_ns, err);
    __syncthreads();
    if (threadIdx.x == 0) { *a.block_counter = 0; __threadfence(); *a.epoch = epoch; }
  }
}

// Phase 2 of the fused kernels: every block waits for all ranks' "partials written"
// flags, then reduces its slice of [B][N] over the ranks' buffers.
__device__ __forceinline__ void allreduce_tail(const QArArgs& a, int B, int N, unsigned* err) {
  __shared__ unsigned s_last;
  __shared__ int s_ok;
  const unsigned epoch = *a.epoch + 1;  // flag value of this call
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    s_ok = 1;
    s_last = atomicAdd(a.block_counter, 1u) == gridDim.x - 1 ? 1u : 0u;
  }
  __syncthreads();
  if (s_last && threadIdx.x < a.world) {
    __threadfence_system();
    st_release_sys_u32(a.sig[threadIdx.x] + a.slot * kQMaxRanks + a.rank, epoch);
  }
  if (threadIdx.x < a.world) {
    if (!wait_flag_ge(a.sig[a.rank] + a.slot * kQMaxRanks + threadIdx.x, epoch, a.wait_ns, err)) s_ok = 0;
  }
  __syncthreads();
  if (s_ok) {
    const int total4 = B * N / 4;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += gridDim.x * blockDim.x) {
      float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int r = 0; r < kQMaxRanks; ++r) {
        if (r < a.world) {
          const float4 v = ld_sys_f4(a.partial[r] + static_cast<size_t>(i) * 4);
          s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        }
      }
      if (a.residual) {
        const uint2 rr = *reinterpret_cast<const uint2*>(a.residual + static_cast<size_t>(i) * 4);
        const float2 r0 = unpack_bf16x2(rr.x), r1 = unpack_bf16x2(rr.y);
        s.x += r0.x; s.y += r0.y; s.z += r1.x; s.w += r1.y;
      }
      uint2 o;
      o.x = pack_bf16x2(s.x, s.y);
      o.y = pack_bf16x2(s.z, s.w);
      *reinterpret_cast<uint2*>(a.out + static_cast<size_t>(i) * 4) = o;
    }
  }
  // the last block to finish the reduction advances the epoch and re-arms the counter
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned done = atomicAdd(a.block_counter, 1u);
    if (done == 2 * gridDim.x - 1) {
      *a.block_counter = 0;
      __threadfence();
      *a.epoch = epoch;
    }
  }
}

__global__ void __launch_bounds__(256)
q4_gemv_allreduce_kernel(const __half* __restrict__ ws, const uint4* __restrict__ wq,
                         const int8_t* __restrict__ xq, const float* __restrict__ xs, QArArgs a, int N, int K,
                         int B, unsigned* err) {
  const int lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  float* mine = a.partial[a.rank];
  for (int n = blockIdx.x * warps + (threadIdx.x >> 5); n < N; n += gridDim.x * warps) {
    const size_t wb = static_cast<size_t>(n) * (K / 32);
    for (int b0 = 0; b0 < B; b0 += 8) {
      float acc[8];
      q4_row_dot<8>(ws + wb, wq + wb, xq, xs, K, b0, B, lane, acc);
#pragma unroll
      for (int b = 0; b < 8; ++b) {
        const float s = warp_sum_f(acc[b]);
        if (lane == 0 && b0 + b < B) mine[static_cast<size_t>(b0 + b) * N + n] = s;
      }
    }
  }
  allreduce_tail(a, B, N, err);
}

// The all-reduce alone, for partial sums another kernel produced (prefill GEMMs).
__global__ void __launch_bounds__(256) oneshot_allreduce_kernel(QArArgs a, int B, int N, unsigned* err) {
  allreduce_tail(a, B, N, err);
}

// ---------------------------------------------------------------------------
// Single-query attention over an fp16 KV cache (decode step), split over the keys.
// The number of valid keys comes from device memory, so one captured CUDA graph
// serves every decode step.
// q [B][Hq][D] bf16 with row pitch ldq, cache K/V [B][Hkv][cap][D] fp16, out [B][Hq][D] bf16.
// Grid (Hkv, B, S): a block owns one KV head (all G = Hq/Hkv query heads that share it,
// so each key and value row is read once) and the z-th of S equal key ranges.  A warp
// takes four keys per iteration, so four independent row loads are in flight per lane.
// Each block leaves an unnormalised partial (o, max, sum) in `ws`; the block that
// arrives last at the (batch, kv head) counter merges the S partials and resets the
// counter for the next launch.  With S == 1 the block writes the result directly.
// ---------------------------------------------------------------------------
constexpr int kDecWarps = 8;
constexpr int kDecKeys = 4;

template <int D, int G>
__global__ void __launch_bounds__(kDecWarps * 32)
attn_decode_kernel(const __nv_bfloat16* __restrict__ q, const __half* __restrict__ kc, const __half* __restrict__ vc,
                   __nv_bfloat16* __restrict__ out, int Hq, int Hkv, int cap, const int* __restrict__ len_ptr, float scale,
                   int ldq, float* __restrict__ ws, unsigned* __restrict__ counters, int S) {
  constexpr int PER = D / 32;  // elements of the head dimension per lane
  const int len = min(*len_ptr, cap);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int hk = blockIdx.x, b = blockIdx.y, z = blockIdx.z;
  const int chunk = (len + S - 1) / S;
  const int t_begin = z * chunk, t_end = min(len, t_begin + chunk);
  __shared__ float sm[kDecWarps][G], sl[kDecWarps][G];
  __shared__ float so[kDecWarps][G][D];
  __shared__ int s_last;

  float qv[G][PER], o[G][PER], m[G], l[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      qv[g][i] = __bfloat162float(q[static_cast<size_t>(b) * ldq + (hk * G + g) * D + lane * PER + i]) * scale;
      o[g][i] = 0.f;
    }
  }
  const __half* kb = kc + (static_cast<size_t>(b) * Hkv + hk) * cap * D + lane * PER;
  const __half* vb = vc + (static_cast<size_t>(b) * Hkv + hk) * cap * D + lane * PER;
  for (int t0 = t_begin + warp * kDecKeys; t0 < t_end; t0 += kDecWarps * kDecKeys) {
    float kf[kDecKeys][PER], vf[kDecKeys][PER];
#pragma unroll
    for (int u = 0; u < kDecKeys; ++u) {
      const int t = min(t0 + u, t_end - 1);  // a clamped row is read but its weight is zero
      if constexpr (PER == 4) {
        const uint2 kr = *reinterpret_cast<const uint2*>(kb + static_cast<size_t>(t) * D);
        const uint2 vr = *reinterpret_cast<const uint2*>(vb + static_cast<size_t>(t) * D);
        const __half2 k0 = *reinterpret_cast<const __half2*>(&kr.x), k1 = *reinterpret_cast<const __half2*>(&kr.y);
        const __half2 v0 = *reinterpret_cast<const __half2*>(&vr.x), v1 = *reinterpret_cast<const __half2*>(&vr.y);
        kf[u][0] = __low2float(k0); kf[u][1] = __high2float(k0); kf[u][2] = __low2float(k1); kf[u][3] = __high2float(k1);
        vf[u][0] = __low2float(v0); vf[u][1] = __high2float(v0); vf[u][2] = __low2float(v1); vf[u][3] = __high2float(v1);
      } else {
        const __half2 k0 = *reinterpret_cast<const __half2*>(kb + static_cast<size_t>(t) * D);
        const __half2 v0 = *reinterpret_cast<const __half2*>(vb + static_cast<size_t>(t) * D);
        kf[u][0] = __low2float(k0); kf[u][1] = __high2float(k0);
        vf[u][0] = __low2float(v0); vf[u][1] = __high2float(v0);
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float sc[kDecKeys];
#pragma unroll
      for (int u = 0; u < kDecKeys; ++u) {
        float d = 0.f;
#pragma unroll
        for (int i = 0; i < PER; ++i) d += qv[g][i] * kf[u][i];
        sc[u] = d;
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1)
#pragma unroll
        for (int u = 0; u < kDecKeys; ++u) sc[u] += __shfl_xor_sync(0xffffffffu, sc[u], off);
      float mn = m[g];
#pragma unroll
      for (int u = 0; u < kDecKeys; ++u)
        if (t0 + u < t_end) mn = fmaxf(mn, sc[u]);
      const float alpha = m[g] == -INFINITY ? 0.f : __expf(m[g] - mn);
      float pw[kDecKeys], psum = 0.f;
#pragma unroll
      for (int u = 0; u < kDecKeys; ++u) {
        pw[u] = t0 + u < t_end ? __expf(sc[u] - mn) : 0.f;
        psum += pw[u];
      }
      l[g] = l[g] * alpha + psum;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        float acc = o[g][i] * alpha;
#pragma unroll
        for (int u = 0; u < kDecKeys; ++u) acc += pw[u] * vf[u][i];
        o[g][i] = acc;
      }
      m[g] = mn;
    }
  }
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (lane == 0) { sm[warp][g] = m[g]; sl[warp][g] = l[g]; }
#pragma unroll
    for (int i = 0; i < PER; ++i) so[warp][g][lane * PER + i] = o[g][i];
  }
  __syncthreads();
  // warp g merges the block's warps for query head g
  float M = -INFINITY, L = 0.f, acc[PER];
  if (warp < G) {
    const int g = warp;
    for (int w = 0; w < kDecWarps; ++w) M = fmaxf(M, sm[w][g]);
#pragma unroll
    for (int i = 0; i < PER; ++i) acc[i] = 0.f;
    for (int w = 0; w < kDecWarps; ++w) {
      const float f = sm[w][g] == -INFINITY ? 0.f : __expf(sm[w][g] - M);
      L += sl[w][g] * f;
#pragma unroll
      for (int i = 0; i < PER; ++i) acc[i] += so[w][g][lane * PER + i] * f;
    }
    const int h = hk * G + g;
    if (S == 1) {
      const float inv = L > 0.f ? 1.f / L : 0.f;
#pragma unroll
      for (int i = 0; i < PER; ++i)
        out[(static_cast<size_t>(b) * Hq + h) * D + lane * PER + i] = __float2bfloat16_rn(acc[i] * inv);
    } else {
      float* part = ws + ((static_cast<size_t>(b) * Hq + h) * S + z) * (D + 2);
#pragma unroll
      for (int i = 0; i < PER; ++i) part[lane * PER + i] = acc[i];
      if (lane == 0) { part[D] = M; part[D + 1] = L; }
    }
  }
  if (S == 1) return;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(&counters[b * Hkv + hk], 1u);
    s_last = prev == static_cast<unsigned>(S - 1);
    if (s_last) counters[b * Hkv + hk] = 0u;  // ready for the next launch on this stream
  }
  __syncthreads();
  if (!s_last || warp >= G) return;
  __threadfence();
  const int h = hk * G + warp;
  const float* parts = ws + (static_cast<size_t>(b) * Hq + h) * S * (D + 2);
  float Mt = -INFINITY;
  for (int j = 0; j < S; ++j) Mt = fmaxf(Mt, __ldcg(parts + static_cast<size_t>(j) * (D + 2) + D));
  float Lt = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) acc[i] = 0.f;
  for (int j = 0; j < S; ++j) {
    const float* pj = parts + static_cast<size_t>(j) * (D + 2);
    const float mj = __ldcg(pj + D);
    const float f = mj == -INFINITY ? 0.f : __expf(mj - Mt);
    Lt += __ldcg(pj + D + 1) * f;
#pragma unroll
    for (int i = 0; i < PER; ++i) acc[i] += __ldcg(pj + lane * PER + i) * f;
  }
  const float inv = Lt > 0.f ? 1.f / Lt : 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i)
    out[(static_cast<size_t>(b) * Hq + h) * D + lane * PER + i] = __float2bfloat16_rn(acc[i] * inv);
}

// k, v [B][Hkv][D] bf16 (row pitch ld, column offsets kcol / vcol) -> fp16 cache at position pos
__global__ void kv_cache_write_kernel(const __nv_bfloat16* __restrict__ kv, int ld, int kcol, int vcol,
                                      __half* __restrict__ kc, __half* __restrict__ vc, int B, int Hkv, int D,
                                      int cap, const int* __restrict__ pos_ptr) {
  const int pos = *pos_ptr;
  if (pos < 0 || pos >= cap) return;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= B * Hkv * D) return;
  const int d = i % D, h = (i / D) % Hkv, b = i / (D * Hkv);
  const size_t dst = ((static_cast<size_t>(b) * Hkv + h) * cap + pos) * D + d;
  kc[dst] = __float2half(__bfloat162float(kv[static_cast<size_t>(b) * ld + kcol + h * D + d]));
  vc[dst] = __float2half(__bfloat162float(kv[static_cast<size_t>(b) * ld + vcol + h * D + d]));
}

// Decode-step rotary embedding and cache write in one launch: the (interleaved) pairs of the Hq query
// heads and Hkv key heads of qkv [B][(Hq + 2 Hkv) D] are rotated in place by the row's position, the
// rotated keys and the values go to the fp16 cache at the write position.  The arithmetic is the
// two-kernel sequence's: rotate in fp32, round to bf16 (what attention reads for q), bf16 -> fp16 for the cache.
__global__ void rope_kv_write_kernel(__nv_bfloat16* __restrict__ qkv, int ld, const int* __restrict__ pos_rows,
                                     const float* __restrict__ freqs, __half* __restrict__ kc, __half* __restrict__ vc,
                                     int B, int Hq, int Hkv, int D, int cap, const int* __restrict__ pos_ptr) {
  const int half = D / 2;
  const int n_rope = B * (Hq + Hkv) * half, n_v = B * Hkv * half;
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  const int wpos = *pos_ptr;
  const bool store = wpos >= 0 && wpos < cap;
  if (idx < n_rope) {
    const int i = idx % half, h = (idx / half) % (Hq + Hkv), b = idx / (half * (Hq + Hkv));
    float sn, cs;
    sincosf(static_cast<float>(pos_rows[b]) * freqs[i], &sn, &cs);
    __nv_bfloat16* base = qkv + static_cast<size_t>(b) * ld + h * D;
    const float x0 = __bfloat162float(base[2 * i]), x1 = __bfloat162float(base[2 * i + 1]);
    const __nv_bfloat16 r0 = __float2bfloat16_rn(x0 * cs - x1 * sn), r1 = __float2bfloat16_rn(x0 * sn + x1 * cs);
    base[2 * i] = r0;
    base[2 * i + 1] = r1;
    if (h >= Hq && store) {
      const size_t dst = ((static_cast<size_t>(b) * Hkv + (h - Hq)) * cap + wpos) * D + 2 * i;
      kc[dst] = __float2half(__bfloat162float(r0));
      kc[dst + 1] = __float2half(__bfloat162float(r1));
    }
  } else if (idx < n_rope + n_v && store) {
    const int j = idx - n_rope;
    const int i = j % half, h = (j / half) % Hkv, b = j / (half * Hkv);
    const __nv_bfloat16* src = qkv + static_cast<size_t>(b) * ld + (Hq + Hkv + h) * D + 2 * i;
    const size_t dst = ((static_cast<size_t>(b) * Hkv + h) * cap + wpos) * D + 2 * i;
    vc[dst] = __float2half(__bfloat162float(src[0]));
    vc[dst + 1] = __float2half(__bfloat162float(src[1]));
  }
}

// fp32 [rows][N] -> bf16
__global__ void f32_to_bf16_rows_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y, size_t n) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) y[i] = __float2bfloat16_rn(x[i]);
}

static unsigned long long g_q_wait_ns = 10000000000ull;
unsigned long long q_peer_wait_ns() { return g_q_wait_ns; }

}  // namespace mimir

using namespace mimir;

MIMIR_API void mimir_q_set_peer_wait_ms(long long ms) { g_q_wait_ns = static_cast<unsigned long long>(ms) * 1000000ull; }

MIMIR_API int mimir_dequant(int code, const void* raw, float* out, long long n, cudaStream_t st) {
  if (code < 64 || code > 67) return refuse("dequant: unknown dtype code %d", code);
  dequant_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, st>>>(code, static_cast<const uint8_t*>(raw), out, n);
  count_launch();
  return 0;
}
MIMIR_API int mimir_q4_0_to_planar(const void* raw, void* scales, void* quants, long long nblocks, cudaStream_t st) {
  q4_0_to_planar_kernel<<<static_cast<unsigned>((nblocks + 255) / 256), 256, 0, st>>>(
      static_cast<const uint8_t*>(raw), static_cast<__half*>(scales), static_cast<uint4*>(quants), nblocks);
  count_launch();
  return 0;
}
// mode 0 plain, 1 RMSNorm * gamma (y optional), 2 SwiGLU of [rows][2K]
MIMIR_API int mimir_quantize_act(const void* x, int x_is_f32, const void* gamma, void* y, void* xq, float* xs,
                                 int rows, int K, int mode, float eps, cudaStream_t st) {
  if (K % 32) return refuse("quantize: K must be a multiple of 32");
  if (x_is_f32)
    quantize_act_kernel<float><<<ceil_div(rows, 8), 256, 0, st>>>(static_cast<const float*>(x),
                                                                 static_cast<const __nv_bfloat16*>(gamma),
                                                                 static_cast<__nv_bfloat16*>(y),
                                                                 static_cast<int8_t*>(xq), xs, rows, K, mode, eps);
  else
    quantize_act_kernel<__nv_bfloat16><<<ceil_div(rows, 8), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(gamma),
        static_cast<__nv_bfloat16*>(y), static_cast<int8_t*>(xq), xs, rows, K, mode, eps);
  count_launch();
  return 0;
}
// out_is_bf16 selects the element type of `out`.
MIMIR_API int mimir_q4_gemv(const void* ws, const void* wq, const void* xq, const float* xs, void* out,
                            int out_is_bf16, int N, int K, int B, int ldo, cudaStream_t st) {
  if (K % 32) return refuse("q4 gemv: K must be a multiple of 32");
  q4_gemv_kernel<<<ceil_div(N, 8), 256, 0, st>>>(static_cast<const __half*>(ws), static_cast<const uint4*>(wq),
                                                 static_cast<const int8_t*>(xq), xs,
                                                 out_is_bf16 ? nullptr : static_cast<float*>(out),
                                                 out_is_bf16 ? static_cast<__nv_bfloat16*>(out) : nullptr, N, K, B,
                                                 ldo);
  count_launch();
  return 0;
}
// partial/sig: arrays of `world` device pointers (peer mapped).  N*B must be a multiple of 4.
MIMIR_API int mimir_q4_gemv_allreduce(const void* ws, const void* wq, const void* xq, const float* xs,
                                      void* const* partial, void* const* sig, void* epoch, void* block_counter,
                                      const void* residual, void* out, int N, int K, int B, int rank, int world,
                                      int slot, cudaStream_t st) {
  if (K % 32 || (static_cast<long long>(N) * B) % 4) return refuse("q4 gemv all-reduce: K %% 32 and N*B %% 4 must be 0");
  if (world < 1 || world > kQMaxRanks) return refuse("q4 gemv all-reduce: world %d not in 1..8", world);
  QArArgs a;
  for (int r = 0; r < kQMaxRanks; ++r) {
    a.partial[r] = r < world ? static_cast<float*>(partial[r]) : nullptr;
    a.sig[r] = r < world ? static_cast<unsigned*>(sig[r]) : nullptr;
  }
  a.epoch = static_cast<unsigned*>(epoch);
  a.block_counter = static_cast<unsigned*>(block_counter);
  a.residual = static_cast<const __nv_bfloat16*>(residual);
  a.out = static_cast<__nv_bfloat16*>(out);
  a.rank = rank; a.world = world; a.slot = slot; a.wait_ns = g_q_wait_ns;
  // every block must be resident at once (blocks wait on flags that the last block of the
  // grid sets): size the grid from the occupancy the kernel really gets
  static int blocks_per_sm = 0;
  if (blocks_per_sm == 0) {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, q4_gemv_allreduce_kernel, 256, 0) != cudaSuccess || n < 1) n = 1;
    blocks_per_sm = n;
  }
  int grid = ceil_div(N, 8);
  const int cap = sm_count() * blocks_per_sm;
  if (grid > cap) grid = cap;
  q4_gemv_allreduce_kernel<<<grid, 256, 0, st>>>(static_cast<const __half*>(ws), static_cast<const uint4*>(wq),
                                                 static_cast<const int8_t*>(xq), xs, a, N, K, B, error_word_dev());
  count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : refuse("q4 gemv all-reduce launch failed");
}
MIMIR_API int mimir_oneshot_allreduce(void* const* partial, void* const* sig, void* epoch, void* block_counter,
                                      const void* residual, void* out, int N, int B, int rank, int world, int slot,
                                      cudaStream_t st) {
  if ((static_cast<long long>(N) * B) % 4) return refuse("all-reduce: N*B must be a multiple of 4");
  QArArgs a;
  for (int r = 0; r < kQMaxRanks; ++r) {
    a.partial[r] = r < world ? static_cast<float*>(partial[r]) : nullptr;
    a.sig[r] = r < world ? static_cast<unsigned*>(sig[r]) : nullptr;
  }
  a.epoch = static_cast<unsigned*>(epoch);
  a.block_counter = static_cast<unsigned*>(block_counter);
  a.residual = static_cast<const __nv_bfloat16*>(residual);
  a.out = static_cast<__nv_bfloat16*>(out);
  a.rank = rank; a.world = world; a.slot = slot; a.wait_ns = g_q_wait_ns;
  oneshot_allreduce_kernel<<<sm_count(), 256, 0, st>>>(a, B, N, error_word_dev());  // one resident block per SM
  count_launch();
  return 0;
}
template <int D>
static int launch_attn_decode(const void* q, const void* kc, const void* vc, void* out, int B, int Hq, int Hkv, int cap,
                              const int* len_dev, float scale, int ldq, float* ws, unsigned* counters, int S,
                              cudaStream_t st) {
  dim3 grid(Hkv, B, S);
#define MIMIR_DEC(G)                                                                                                 \
  attn_decode_kernel<D, G><<<grid, kDecWarps * 32, 0, st>>>(                                                         \
      static_cast<const __nv_bfloat16*>(q), static_cast<const __half*>(kc), static_cast<const __half*>(vc),          \
      static_cast<__nv_bfloat16*>(out), Hq, Hkv, cap, len_dev, scale, ldq, ws, counters, S)
  switch (Hq / Hkv) {
    case 1: MIMIR_DEC(1); break;
    case 2: MIMIR_DEC(2); break;
    case 4: MIMIR_DEC(4); break;
    case 8: MIMIR_DEC(8); break;
    default: return refuse("decode attention: %d query heads per KV head not supported (1, 2, 4 or 8)", Hq / Hkv);
  }
#undef MIMIR_DEC
  count_launch();
  return 0;
}
// ws: B * Hq * splits * (D + 2) floats and counters: B * Hkv zeroed words, both needed only when splits > 1.
MIMIR_API int mimir_attn_decode(const void* q, const void* kc, const void* vc, void* out, int B, int Hq, int Hkv,
                                int D, int cap, const int* len_dev, float scale, int ldq, float* ws,
                                unsigned* counters, int splits, cudaStream_t st) {
  if (Hkv <= 0 || Hq % Hkv) return refuse("decode attention: %d query heads do not divide over %d KV heads", Hq, Hkv);
  if (splits < 1 || (splits > 1 && (!ws || !counters))) return refuse("decode attention: %d splits need a workspace", splits);
  if (D == 128) return launch_attn_decode<128>(q, kc, vc, out, B, Hq, Hkv, cap, len_dev, scale, ldq, ws, counters, splits, st);
  if (D == 64) return launch_attn_decode<64>(q, kc, vc, out, B, Hq, Hkv, cap, len_dev, scale, ldq, ws, counters, splits, st);
  return refuse("decode attention: head dim %d not supported (64 or 128)", D);
}
MIMIR_API int mimir_kv_cache_write(const void* kv, int ld, int kcol, int vcol, void* kc, void* vc, int B, int Hkv,
                                   int D, int cap, const int* pos_dev, cudaStream_t st) {
  const int n = B * Hkv * D;
  kv_cache_write_kernel<<<ceil_div(n, 256), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(kv), ld, kcol, vcol,
                                                          static_cast<__half*>(kc), static_cast<__half*>(vc), B, Hkv,
                                                          D, cap, pos_dev);
  count_launch();
  return 0;
}
MIMIR_API int mimir_rope_kv_write(void* qkv, int ld, const int* pos_rows, const float* freqs, void* kc, void* vc, int B,
                                  int Hq, int Hkv, int D, int cap, const int* pos_dev, cudaStream_t st) {
  if (D % 2) return refuse("rope: head dim must be even");
  const int n = B * (Hq + 2 * Hkv) * (D / 2);
  rope_kv_write_kernel<<<ceil_div(n, 256), 256, 0, st>>>(static_cast<__nv_bfloat16*>(qkv), ld, pos_rows, freqs,
                                                         static_cast<__half*>(kc), static_cast<__half*>(vc), B, Hq, Hkv, D,
                                                         cap, pos_dev);
  count_launch();
  return 0;
}
MIMIR_API int mimir_f32_to_bf16(const float* x, void* y, long long n, cudaStream_t st) {
  f32_to_bf16_rows_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, st>>>(x, static_cast<__nv_bfloat16*>(y), n);
  count_launch();
  return 0;
}

MIMIR_API int mimir_q4_planar_to_bf16(const void* ws, const void* wq, void* out, long long nblocks, cudaStream_t st) {
  q4_planar_to_bf16_kernel<<<static_cast<unsigned>((nblocks + 255) / 256), 256, 0, st>>>(
      static_cast<const __half*>(ws), static_cast<const uint4*>(wq), static_cast<__nv_bfloat16*>(out), nblocks);
  count_launch();
  return 0;
}
// nbytes (multiple of 16) of src land at dst[r] + rank * nbytes on every rank r.
MIMIR_API int mimir_peer_allgather(const void* src, void* const* dst, void* const* sig, void* epoch,
                                   void* block_counter, long long nbytes, int rank, int world, int slot,
                                   cudaStream_t st) {
  if (nbytes % 16) return refuse("all-gather: byte count must be a multiple of 16");
  AgArgs a;
  for (int r = 0; r < kQMaxRanks; ++r) {
    a.dst[r] = r < world ? static_cast<uint8_t*>(dst[r]) : nullptr;
    a.sig[r] = r < world ? static_cast<unsigned*>(sig[r]) : nullptr;
  }
  a.epoch = static_cast<unsigned*>(epoch);
  a.block_counter = static_cast<unsigned*>(block_counter);
  a.rank = rank; a.world = world; a.slot = slot; a.wait_ns = g_q_wait_ns;
  // small messages: 32 blocks keep the arrival counter cheap; large ones use every SM for link bandwidth
  int blocks = static_cast<int>(nbytes / 65536);
  if (blocks < 32) blocks = 32;
  if (blocks > sm_count()) blocks = sm_count();
  peer_allgather_kernel<<<blocks, 256, 0, st>>>(static_cast<const uint4*>(src), a, static_cast<size_t>(nbytes / 16),
                                            error_word_dev());
  count_launch();
  return 0;
}
