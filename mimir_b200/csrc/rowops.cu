// Row kernels: LayerNorm / RMSNorm forward+backward, softmax, fused
// softmax-cross-entropy (loss + gradient in place).  One warp (norms) or one
// block (vocabulary rows) per row, 128-bit loads, fp32 math, bf16 storage.
//
// Reference semantics: nn/layers.go:139 (LayerNorm), nn/transformer.go:28-61
// (RMSNorm: normalise in fp32, round to the input dtype, then scale),
// tensor/reduce.go:199-218 (softmax / log-softmax), nn/loss/loss.go:35-96
// (cross entropy over class indices).
#include "common.cuh"
#include "runtime.h"

namespace mimir {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 u;
  u.x = pack_bf16x2(v[0], v[1]); u.y = pack_bf16x2(v[2], v[3]);
  u.z = pack_bf16x2(v[4], v[5]); u.w = pack_bf16x2(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

// ---------------------------------------------------------------------------
// LayerNorm / RMSNorm forward.  Lane owns columns lane*8 + i*256.
// ---------------------------------------------------------------------------
template <int NCHUNK, bool RMS>
__global__ void __launch_bounds__(256)
norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                const __nv_bfloat16* __restrict__ beta, __nv_bfloat16* __restrict__ y,
                float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows, int C, float eps) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const __nv_bfloat16* xr = x + static_cast<size_t>(row) * C;
  float v[NCHUNK][8];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < NCHUNK; ++i) {
    const int c = lane * 8 + i * 256;
    if (c < C) {
      load8(xr + c, v[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) s += RMS ? v[i][j] * v[i][j] : v[i][j];
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] = 0.f;
    }
  }
  s = warp_sum(s);
  float mean = 0.f, rstd;
  if (RMS) {
    rstd = rsqrtf(s / C + eps);
  } else {
    mean = s / C;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < NCHUNK; ++i) {
      const int c = lane * 8 + i * 256;
      if (c < C) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { float d = v[i][j] - mean; q += d * d; }
      }
    }
    q = warp_sum(q);
    rstd = rsqrtf(q / C + eps);
  }
  if (lane == 0) {
    if (mean_out) mean_out[row] = mean;
    if (rstd_out) rstd_out[row] = rstd;
  }
  __nv_bfloat16* yr = y + static_cast<size_t>(row) * C;
#pragma unroll
  for (int i = 0; i < NCHUNK; ++i) {
    const int c = lane * 8 + i * 256;
    if (c < C) {
      float g[8], b[8], o[8];
      load8(gamma + c, g);
      if (!RMS && beta) load8(beta + c, b);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float n = (v[i][j] - mean) * rstd;
        if (RMS) n = __bfloat162float(__float2bfloat16_rn(n));  // round before the scale
        o[j] = n * g[j] + ((!RMS && beta) ? b[j] : 0.f);
      }
      store8(yr + c, o);
    }
  }
}

// ---------------------------------------------------------------------------
// LayerNorm / RMSNorm backward.  dx (+= residual gradient), and per-block
// partial sums of dgamma / dbeta in `partial` [gridDim.x][2][C] (fp32).
// ---------------------------------------------------------------------------
template <int NCHUNK, bool RMS>
__global__ void __launch_bounds__(256)
norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean_in,
                const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dres,
                __nv_bfloat16* __restrict__ dx, float* __restrict__ partial, int rows, int C) {
  extern __shared__ float red[];  // [warps][2][C] would be large: reduce through rounds instead
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  float dg[NCHUNK][8], db[NCHUNK][8], g[NCHUNK][8];
#pragma unroll
  for (int i = 0; i < NCHUNK; ++i) {
    const int c = lane * 8 + i * 256;
    if (c < C) load8(gamma + c, g[i]);
#pragma unroll
    for (int j = 0; j < 8; ++j) { dg[i][j] = 0.f; db[i][j] = 0.f; if (c >= C) g[i][j] = 0.f; }
  }
  for (int row = blockIdx.x * nwarp + warp; row < rows; row += gridDim.x * nwarp) {
    const size_t off = static_cast<size_t>(row) * C;
    const float mean = RMS ? 0.f : mean_in[row], rstd = rstd_in[row];
    float xh[NCHUNK][8], d[NCHUNK][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NCHUNK; ++i) {
      const int c = lane * 8 + i * 256;
      if (c < C) {
        load8(x + off + c, xh[i]);
        load8(dy + off + c, d[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] = (xh[i][j] - mean) * rstd;
          dg[i][j] += d[i][j] * xh[i][j];
          db[i][j] += d[i][j];
          d[i][j] *= g[i][j];
          s1 += d[i][j];
          s2 += d[i][j] * xh[i][j];
        }
      }
    }
    s1 = RMS ? 0.f : warp_sum(s1) / C;
    s2 = warp_sum(s2) / C;
#pragma unroll
    for (int i = 0; i < NCHUNK; ++i) {
      const int c = lane * 8 + i * 256;
      if (c < C) {
        float o[8];
        if (dres) load8(dres + off + c, o);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float t = rstd * (d[i][j] - s1 - xh[i][j] * s2);
          o[j] = dres ? o[j] + t : t;
        }
        store8(dx + off + c, o);
      }
    }
  }
  // Block reduce of dg / db over warps, one chunk at a time through shared memory.
  float* out = partial + static_cast<size_t>(blockIdx.x) * 2 * C;
#pragma unroll
  for (int i = 0; i < NCHUNK; ++i) {
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      red[(warp * 2 + 0) * 256 + lane * 8 + j] = dg[i][j];
      red[(warp * 2 + 1) * 256 + lane * 8 + j] = db[i][j];
    }
    __syncthreads();
    for (int t = threadIdx.x; t < 512; t += blockDim.x) {
      const int which = t >> 8, col = t & 255;
      float s = 0.f;
      for (int w = 0; w < nwarp; ++w) s += red[(w * 2 + which) * 256 + col];
      const int c = col + i * 256;
      if (c < C) out[which * C + c] = s;
    }
  }
}

// Sums `nparts` partial rows [nparts][width] into bf16 (optionally accumulating).
// Sums `nparts` partial rows [nparts][width] (fp32) column-wise.  Block = 32
// columns x 32 row lanes.  Columns [0, split) go to out0, [split, width) to out1
// (bf16, optionally accumulating), which finishes dgamma and dbeta in one launch.
__global__ void __launch_bounds__(1024)
reduce_partials_kernel(const float* __restrict__ partial, int nparts, int width, int split,
                       __nv_bfloat16* __restrict__ out0, __nv_bfloat16* __restrict__ out1, int accumulate) {
  __shared__ float red[32][33];
  const int cl = threadIdx.x & 31, rl = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cl;
  float s = 0.f;
  if (c < width)
    for (int p = rl; p < nparts; p += 32) s += partial[static_cast<size_t>(p) * width + c];
  red[rl][cl] = s;
  __syncthreads();
  if (rl == 0 && c < width) {
#pragma unroll
    for (int r = 1; r < 32; ++r) s += red[r][cl];
    __nv_bfloat16* o = c < split ? out0 + c : out1 + (c - split);
    if (c >= split && !out1) return;
    if (accumulate) s += __bfloat162float(*o);
    *o = __float2bfloat16_rn(s);
  }
}

// Column sums of a bf16 matrix [rows, N] (row pitch ld) into partial[gridDim.y][N].
__global__ void __launch_bounds__(256)
colsum_partial_kernel(const __nv_bfloat16* __restrict__ x, int rows, int N, int ld,
                      float* __restrict__ partial) {
  __shared__ float red[8][256];
  const int cg = threadIdx.x & 31, rl = threadIdx.x >> 5;
  const int col = blockIdx.x * 256 + cg * 8;
  const int rows_per = (rows + gridDim.y - 1) / gridDim.y;
  const int r0 = blockIdx.y * rows_per, r1 = min(rows, r0 + rows_per);
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (col < N) {
    for (int r = r0 + rl; r < r1; r += 8) {
      float v[8];
      load8(x + static_cast<size_t>(r) * ld + col, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += v[j];
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) red[rl][cg * 8 + j] = acc[j];
  __syncthreads();
  const int c = threadIdx.x;
  float s = 0.f;
#pragma unroll
  for (int r = 0; r < 8; ++r) s += red[r][c];
  if (blockIdx.x * 256 + c < N) partial[static_cast<size_t>(blockIdx.y) * N + blockIdx.x * 256 + c] = s;
}

// ---------------------------------------------------------------------------
// Fused softmax cross-entropy over a padded vocabulary.  One block per row.
// logits [rows, ld] bf16 (columns >= V are padding).  Writes loss[row] and, if
// dlogits != nullptr, (softmax - onehot) * gscale in bf16 (may alias logits).
// target < 0 means "ignore this row".
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(512)
cross_entropy_kernel(const __nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ target,
                     float* __restrict__ loss, __nv_bfloat16* __restrict__ dlogits, int V, int ld,
                     float gscale, unsigned* err) {
  __shared__ float smax[16], ssum[16];
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const __nv_bfloat16* lr = logits + static_cast<size_t>(row) * ld;
  const int64_t tgt = target[row];
  if (tgt >= V) { if (tid == 0) raise_error(err, kErrIndex); }
  // read before anyone may overwrite the row in place
  const float tgt_logit = (tid == 0 && tgt >= 0 && tgt < V) ? __bfloat162float(lr[tgt]) : 0.f;
  // two independent online-softmax chains over alternate chunks: two row loads in flight per
  // thread and half the dependent rescale chain
  float m = -INFINITY, s = 0.f, m2 = -INFINITY, s2 = 0.f;
  const int vfull = V & ~7;   // chunks below this bound lie entirely inside the row
  for (int c = tid * 8; c < V; c += 2 * 512 * 8) {
    const int c2 = c + 512 * 8;
    float v[8], w[8];
    load8(lr + c, v);
    const bool have2 = c2 < V;
    if (have2) load8(lr + c2, w);
    if (c + 8 > vfull) {
#pragma unroll
      for (int j = 0; j < 8; ++j) if (c + j >= V) v[j] = -INFINITY;
    }
    float cm = m;
#pragma unroll
    for (int j = 0; j < 8; ++j) cm = fmaxf(cm, v[j]);
    float add = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) add += __expf(v[j] - cm);
    s = s * __expf(m - cm) + add;
    m = cm;
    if (have2) {
      if (c2 + 8 > vfull) {
#pragma unroll
        for (int j = 0; j < 8; ++j) if (c2 + j >= V) w[j] = -INFINITY;
      }
      float dm = m2;
#pragma unroll
      for (int j = 0; j < 8; ++j) dm = fmaxf(dm, w[j]);
      float add2 = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) add2 += __expf(w[j] - dm);
      s2 = s2 * __expf(m2 - dm) + add2;
      m2 = dm;
    }
  }
  {
    const float mm = fmaxf(m, m2);
    s = (m == -INFINITY ? 0.f : s * __expf(m - mm)) + (m2 == -INFINITY ? 0.f : s2 * __expf(m2 - mm));
    m = mm;
  }
  // combine (m, s) pairs across the block
  // a thread or warp that saw no column has m = -inf: its weight is zero
  float wm = warp_max(m);
  s = warp_sum(m == -INFINITY ? 0.f : s * __expf(m - wm));
  if (lane == 0) { smax[warp] = wm; ssum[warp] = s; }
  __syncthreads();
  float bm = -INFINITY;
#pragma unroll
  for (int w = 0; w < 16; ++w) bm = fmaxf(bm, smax[w]);
  float bs = 0.f;
#pragma unroll
  for (int w = 0; w < 16; ++w) bs += smax[w] == -INFINITY ? 0.f : ssum[w] * __expf(smax[w] - bm);
  const float lse = bm + __logf(bs);
  const bool ignore = tgt < 0 || tgt >= V;
  if (tid == 0) loss[row] = ignore ? 0.f : lse - tgt_logit;
  if (dlogits) {
    __nv_bfloat16* dr = dlogits + static_cast<size_t>(row) * ld;
    const float gs = ignore ? 0.f : gscale;
    for (int c = tid * 8; c < ld; c += 512 * 8) {
      float v[8], o[8];
      load8(lr + c, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float p = (c + j < V) ? __expf(v[j] - lse) : 0.f;
        if (c + j == tgt) p -= 1.f;
        o[j] = p * gs;
      }
      store8(dr + c, o);
    }
  }
}

// out[0] = scale * sum(x[0..n)); single block.
__global__ void __launch_bounds__(1024) sum_scale_kernel(const float* __restrict__ x, int n, float scale,
                                                        float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += x[i];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    s = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    s = warp_sum(s);
    if (threadIdx.x == 0) out[0] = s * scale;
  }
}

// Row softmax (bf16 in/out), one warp per row for short rows, used by generic
// attention / classifier heads.  log != 0 writes log-softmax.
__global__ void __launch_bounds__(256)
softmax_rows_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, int rows,
                    int C, int log) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const __nv_bfloat16* xr = x + static_cast<size_t>(row) * C;
  float m = -INFINITY;
  for (int c = lane; c < C; c += 32) m = fmaxf(m, __bfloat162float(xr[c]));
  m = warp_max(m);
  float s = 0.f;
  for (int c = lane; c < C; c += 32) s += __expf(__bfloat162float(xr[c]) - m);
  s = warp_sum(s);
  const float inv = 1.f / s, ls = __logf(s);
  __nv_bfloat16* yr = y + static_cast<size_t>(row) * C;
  for (int c = lane; c < C; c += 32) {
    float v = __bfloat162float(xr[c]) - m;
    yr[c] = __float2bfloat16_rn(log ? v - ls : __expf(v) * inv);
  }
}

template <bool RMS>
static int norm_fwd_dispatch(const void* x, const void* g, const void* b, void* y, float* mean,
                             float* rstd, int rows, int C, float eps, cudaStream_t st) {
  const int wpb = 8, grid = ceil_div(rows, wpb);
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto G = static_cast<const __nv_bfloat16*>(g);
  auto B = static_cast<const __nv_bfloat16*>(b);
  auto Y = static_cast<__nv_bfloat16*>(y);
#define CASE(NC) norm_fwd_kernel<NC, RMS><<<grid, wpb * 32, 0, st>>>(X, G, B, Y, mean, rstd, rows, C, eps)
  if (C <= 256) CASE(1); else if (C <= 512) CASE(2); else if (C <= 768) CASE(3);
  else if (C <= 1024) CASE(4); else if (C <= 2048) CASE(8); else if (C <= 4096) CASE(16);
  else if (C <= 8192) CASE(32); else return refuse("norm: C=%d exceeds 8192", C);
#undef CASE
  count_launch();
  return 0;
}

// LayerNorm / RMSNorm backward, second form: a block spans the row (one thread per 8 columns),
// so every thread owns the same columns for all rows and keeps their dgamma / dbeta sums in 16
// registers whatever C is; the two row sums (sum d*g, sum d*g*xhat) go through one shared-memory
// exchange per kRowsPerIter rows.  Register use does not grow with C (the warp-per-row form
// above spills beyond C = 1024).  partial: [gridDim.x][2][C].
constexpr int kRowsPerIter = 4;
template <bool RMS, int MAXT>
__global__ void __launch_bounds__(MAXT)
norm_bwd_rows_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                     const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean_in,
                     const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dres,
                     __nv_bfloat16* __restrict__ dx, float* __restrict__ partial, int rows, int C) {
  __shared__ float red[2][32][2 * kRowsPerIter];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int c = threadIdx.x * 8;
  const bool active = c < C;
  float g[8], dg[8], db[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { g[j] = 0.f; dg[j] = 0.f; db[j] = 0.f; }
  if (active) load8(gamma + c, g);
  const float invC = 1.f / C;
  int parity = 0;
  for (int row0 = blockIdx.x * kRowsPerIter; row0 < rows; row0 += gridDim.x * kRowsPerIter, parity ^= 1) {
    float xh[kRowsPerIter][8], d[kRowsPerIter][8], sums[2 * kRowsPerIter], rs[kRowsPerIter];
#pragma unroll
    for (int r = 0; r < kRowsPerIter; ++r) {
      const int row = row0 + r;
      sums[2 * r] = 0.f; sums[2 * r + 1] = 0.f; rs[r] = 0.f;
      if (row < rows && active) {
        const size_t off = static_cast<size_t>(row) * C + c;
        const float mean = RMS ? 0.f : mean_in[row];
        rs[r] = rstd_in[row];
        load8(x + off, xh[r]);
        load8(dy + off, d[r]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[r][j] = (xh[r][j] - mean) * rs[r];
          dg[j] += d[r][j] * xh[r][j];
          db[j] += d[r][j];
          d[r][j] *= g[j];
          sums[2 * r] += d[r][j];
          sums[2 * r + 1] += d[r][j] * xh[r][j];
        }
      }
    }
#pragma unroll
    for (int k = 0; k < 2 * kRowsPerIter; ++k) sums[k] = warp_sum(sums[k]);
    if (lane == 0) {
#pragma unroll
      for (int k = 0; k < 2 * kRowsPerIter; ++k) red[parity][warp][k] = sums[k];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 2 * kRowsPerIter; ++k) {
      float t = 0.f;
      for (int w = 0; w < nwarp; ++w) t += red[parity][w][k];
      sums[k] = t * invC;
    }
#pragma unroll
    for (int r = 0; r < kRowsPerIter; ++r) {
      const int row = row0 + r;
      if (row < rows && active) {
        const size_t off = static_cast<size_t>(row) * C + c;
        const float s1 = RMS ? 0.f : sums[2 * r], s2 = sums[2 * r + 1];
        float o[8];
        if (dres) load8(dres + off, o);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float t = rs[r] * (d[r][j] - s1 - xh[r][j] * s2);
          o[j] = dres ? o[j] + t : t;
        }
        store8(dx + off, o);
      }
    }
  }
  if (active) {
    float* out = partial + static_cast<size_t>(blockIdx.x) * 2 * C + c;
#pragma unroll
    for (int j = 0; j < 8; j += 4) {
      *reinterpret_cast<float4*>(out + j) = make_float4(dg[j], dg[j + 1], dg[j + 2], dg[j + 3]);
      *reinterpret_cast<float4*>(out + C + j) = make_float4(db[j], db[j + 1], db[j + 2], db[j + 3]);
    }
  }
}

// The same block-spans-the-row form, software pipelined: the packed x / dy / dres values, mean and
// rstd of the next TWO groups of R rows are requested before the current group is reduced, exchanged
// through shared memory and stored, so loads stay in flight through the whole loop (the form above
// has none in flight while it reduces and stores: it measured 16 % of DRAM peak with the long
// scoreboard as its main stall).
__device__ __forceinline__ void unpack_bf16x8(const uint4& u, float (&v)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[2 * j] = __uint_as_float(w[j] << 16);
    v[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
  }
}

struct NormBwdRaw {
  uint4 x, dy, dr;
  float mean, rstd;
};

template <bool RMS, int MAXT, int R>
__global__ void __launch_bounds__(MAXT)
norm_bwd_rows_pipe_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                          const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean_in,
                          const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dres,
                          __nv_bfloat16* __restrict__ dx, float* __restrict__ partial, int rows, int C) {
  __shared__ float red[2][32][2 * R];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int c = threadIdx.x * 8;
  const bool active = c < C;
  float g[8], dg[8], db[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { g[j] = 0.f; dg[j] = 0.f; db[j] = 0.f; }
  if (active) load8(gamma + c, g);
  const float invC = 1.f / C;
  NormBwdRaw cur[R], nxt[R], nxt2[R];   // the current group and the two groups requested ahead of it
  auto fetch = [&](NormBwdRaw (&b)[R], int first) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int row = first + r;
      if (row < rows && active) {
        const size_t off = static_cast<size_t>(row) * C + c;
        b[r].x = *reinterpret_cast<const uint4*>(x + off);
        b[r].dy = *reinterpret_cast<const uint4*>(dy + off);
        if (dres) b[r].dr = *reinterpret_cast<const uint4*>(dres + off);
        b[r].mean = RMS ? 0.f : mean_in[row];
        b[r].rstd = rstd_in[row];
      }
    }
  };
  const int step = gridDim.x * R;
  int row0 = blockIdx.x * R;
  if (row0 < rows) fetch(cur, row0);
  if (row0 + step < rows) fetch(nxt, row0 + step);
  int parity = 0;
  for (; row0 < rows; row0 += step, parity ^= 1) {
    if (row0 + 2 * step < rows) fetch(nxt2, row0 + 2 * step);
    float xh[R][8], d[R][8], sums[2 * R], rs[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int row = row0 + r;
      sums[2 * r] = 0.f; sums[2 * r + 1] = 0.f; rs[r] = 0.f;
      if (row < rows && active) {
        unpack_bf16x8(cur[r].x, xh[r]);
        unpack_bf16x8(cur[r].dy, d[r]);
        const float mean = cur[r].mean;
        rs[r] = cur[r].rstd;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[r][j] = (xh[r][j] - mean) * rs[r];
          dg[j] += d[r][j] * xh[r][j];
          db[j] += d[r][j];
          d[r][j] *= g[j];
          sums[2 * r] += d[r][j];
          sums[2 * r + 1] += d[r][j] * xh[r][j];
        }
      }
    }
#pragma unroll
    for (int k = 0; k < 2 * R; ++k) sums[k] = warp_sum(sums[k]);
    if (lane == 0) {
#pragma unroll
      for (int k = 0; k < 2 * R; ++k) red[parity][warp][k] = sums[k];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 2 * R; ++k) {
      float t = 0.f;
      for (int w = 0; w < nwarp; ++w) t += red[parity][w][k];
      sums[k] = t * invC;
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int row = row0 + r;
      if (row < rows && active) {
        const size_t off = static_cast<size_t>(row) * C + c;
        const float s1 = RMS ? 0.f : sums[2 * r], s2 = sums[2 * r + 1];
        float o[8];
        if (dres) unpack_bf16x8(cur[r].dr, o);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float t = rs[r] * (d[r][j] - s1 - xh[r][j] * s2);
          o[j] = dres ? o[j] + t : t;
        }
        store8(dx + off, o);
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) { cur[r] = nxt[r]; nxt[r] = nxt2[r]; }
  }
  if (active) {
    float* out = partial + static_cast<size_t>(blockIdx.x) * 2 * C + c;
#pragma unroll
    for (int j = 0; j < 8; j += 4) {
      *reinterpret_cast<float4*>(out + j) = make_float4(dg[j], dg[j + 1], dg[j + 2], dg[j + 3]);
      *reinterpret_cast<float4*>(out + C + j) = make_float4(db[j], db[j + 1], db[j + 2], db[j + 3]);
    }
  }
}

// Returns the number of partial rows written (blocks launched) in *used.
template <bool RMS>
static int norm_bwd_dispatch(const void* dy, const void* x, const void* g, const float* mean,
                             const float* rstd, const void* dres, void* dx, float* partial,
                             int nblocks, int rows, int C, int* used, cudaStream_t st) {
  if (C > 8192) return refuse("norm backward: C=%d exceeds 8192", C);
  int threads = (C / 8 + 31) / 32 * 32;
  if (threads <= 128 && (reinterpret_cast<uintptr_t>(dy) & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
      (!dres || (reinterpret_cast<uintptr_t>(dres) & 15) == 0)) {
    // narrow rows (C <= 1024): the pipelined form, two rows per group
    constexpr int R = 2;
    int blocks = ceil_div(rows, R);
    if (blocks > nblocks) blocks = nblocks;
    *used = blocks;
    norm_bwd_rows_pipe_kernel<RMS, 128, R><<<blocks, threads, 0, st>>>(
        static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(g),
        mean, rstd, static_cast<const __nv_bfloat16*>(dres), static_cast<__nv_bfloat16*>(dx), partial, rows, C);
    count_launch();
    return 0;
  }
  int blocks = ceil_div(rows, kRowsPerIter);
  if (blocks > nblocks) blocks = nblocks;
  *used = blocks;
#define NB_CASE(MAXT)                                                                                                   \
  norm_bwd_rows_kernel<RMS, MAXT><<<blocks, threads, 0, st>>>(                                                           \
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(g), \
      mean, rstd, static_cast<const __nv_bfloat16*>(dres), static_cast<__nv_bfloat16*>(dx), partial, rows, C)
  if (threads <= 128) NB_CASE(128); else if (threads <= 256) NB_CASE(256); else if (threads <= 512) NB_CASE(512);
  else NB_CASE(1024);
#undef NB_CASE
  count_launch();
  return 0;
}

}  // namespace mimir

using namespace mimir;

// y = LayerNorm(x) * gamma + beta over the last dim C (C % 8 == 0); saves mean / rstd (fp32).
MIMIR_API int mimir_layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y,
                                  float* mean, float* rstd, int rows, int C, float eps,
                                  cudaStream_t st) {
  if (C % 8) return refuse("layernorm: C must be a multiple of 8");
  return norm_fwd_dispatch<false>(x, gamma, beta, y, mean, rstd, rows, C, eps, st);
}
MIMIR_API int mimir_rmsnorm_fwd(const void* x, const void* gamma, void* y, float* rstd, int rows,
                                int C, float eps, cudaStream_t st) {
  if (C % 8) return refuse("rmsnorm: C must be a multiple of 8");
  return norm_fwd_dispatch<true>(x, gamma, nullptr, y, nullptr, rstd, rows, C, eps, st);
}

// Number of blocks (and rows of `partial`) the backward kernels use.
MIMIR_API int mimir_norm_bwd_blocks() { return sm_count() * 4; }

// dx = dres + LN'(dy); dgamma/dbeta (bf16) written, or accumulated when accumulate != 0.
// partial: fp32 scratch of mimir_norm_bwd_blocks() * 2 * C floats.
MIMIR_API int mimir_layernorm_bwd(const void* dy, const void* x, const void* gamma,
                                  const float* mean, const float* rstd, const void* dres, void* dx,
                                  void* dgamma, void* dbeta, float* partial, int rows, int C,
                                  int accumulate, cudaStream_t st) {
  if (C % 8) return refuse("layernorm: C must be a multiple of 8");
  int nb = mimir_norm_bwd_blocks();
  if (norm_bwd_dispatch<false>(dy, x, gamma, mean, rstd, dres, dx, partial, nb, rows, C, &nb, st)) return -1;
  // partial rows are [dgamma (C) | dbeta (C)]
  reduce_partials_kernel<<<ceil_div(2 * C, 32), 1024, 0, st>>>(partial, nb, 2 * C, C,
                                                               static_cast<__nv_bfloat16*>(dgamma),
                                                               static_cast<__nv_bfloat16*>(dbeta), accumulate);
  count_launch();
  return 0;
}
MIMIR_API int mimir_rmsnorm_bwd(const void* dy, const void* x, const void* gamma, const float* rstd,
                                const void* dres, void* dx, void* dgamma, float* partial, int rows,
                                int C, int accumulate, cudaStream_t st) {
  if (C % 8) return refuse("rmsnorm: C must be a multiple of 8");
  int nb = mimir_norm_bwd_blocks();
  if (norm_bwd_dispatch<true>(dy, x, gamma, nullptr, rstd, dres, dx, partial, nb, rows, C, &nb, st)) return -1;
  reduce_partials_kernel<<<ceil_div(2 * C, 32), 1024, 0, st>>>(partial, nb, 2 * C, C,
                                                               static_cast<__nv_bfloat16*>(dgamma), nullptr,
                                                               accumulate);
  count_launch();
  return 0;
}

// out[N] (bf16) = column sums of x[rows, N]; partial: fp32 scratch of 64 * N floats.
MIMIR_API int mimir_colsum(const void* x, int rows, int N, int ld, void* out, float* partial,
                           int accumulate, cudaStream_t st) {
  if (N % 8 || ld % 8) return refuse("colsum: N and ld must be multiples of 8");
  const int parts = rows >= 64 * 8 ? 64 : 1;
  dim3 grid(ceil_div(N, 256), parts);
  colsum_partial_kernel<<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), rows, N, ld,
                                              partial);
  reduce_partials_kernel<<<ceil_div(N, 32), 1024, 0, st>>>(partial, parts, N, N,
                                                          static_cast<__nv_bfloat16*>(out), nullptr,
                                                          accumulate);
  count_launch(2);
  return 0;
}

// Per-row loss and (optionally) in-place gradient; then mean_loss[0] = sum(loss) * loss_scale.
MIMIR_API int mimir_cross_entropy(const void* logits, const void* target, float* loss_rows,
                                  void* dlogits, float* mean_loss, int rows, int V, int ld,
                                  float gscale, float loss_scale, cudaStream_t st) {
  if (ld % 8) return refuse("cross entropy: row pitch must be a multiple of 8");
  cross_entropy_kernel<<<rows, 512, 0, st>>>(static_cast<const __nv_bfloat16*>(logits),
                                             static_cast<const int64_t*>(target), loss_rows,
                                             static_cast<__nv_bfloat16*>(dlogits), V, ld, gscale,
                                             error_word_dev());
  count_launch();
  if (mean_loss) {
    sum_scale_kernel<<<1, 1024, 0, st>>>(loss_rows, rows, loss_scale, mean_loss);
    count_launch();
  }
  return 0;
}

MIMIR_API int mimir_softmax_rows(const void* x, void* y, int rows, int C, int log, cudaStream_t st) {
  softmax_rows_kernel<<<ceil_div(rows, 8), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x),
                                                        static_cast<__nv_bfloat16*>(y), rows, C, log);
  count_launch();
  return 0;
}

// ---------------------------------------------------------------------------
// Allocation-free column sums (declared in mimir_noalloc.h).
// ---------------------------------------------------------------------------
#include "mimir_noalloc.h"

#include <mutex>

namespace mimir {
namespace {
// Partial sums of one call: [64 row groups][MIMIR_COLSUM_NOALLOC_MAX_N] floats.
// In host code this name is only a handle for cudaGetSymbolAddress, never a pointer
// to pass to a kernel.
static __device__ __align__(256) float g_colsum_scratch[64 * MIMIR_COLSUM_NOALLOC_MAX_N];

constexpr int kNoAllocMaxDevices = 64;
float* g_colsum_scratch_addr[kNoAllocMaxDevices] = {};
std::mutex g_colsum_scratch_mu;

// Device address of the scratch array on the current device (looked up once per device).
float* colsum_scratch_for_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoAllocMaxDevices) {
    refuse("colsum_noalloc: cannot identify the current device");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_colsum_scratch_mu);
  if (!g_colsum_scratch_addr[dev]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_colsum_scratch);
    if (e != cudaSuccess || !p) {
      refuse("colsum_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return nullptr;
    }
    g_colsum_scratch_addr[dev] = static_cast<float*>(p);
  }
  return g_colsum_scratch_addr[dev];
}
}  // namespace
}  // namespace mimir

MIMIR_API int mimir_colsum_noalloc(const void* x, int rows, int N, int ld, void* out, int accumulate,
                                   cudaStream_t st) {
  if (rows <= 0 || N <= 0) return refuse("colsum_noalloc: empty input (%d x %d)", rows, N);
  if (N % 8 || ld % 8) return refuse("colsum_noalloc: N and ld must be multiples of 8");
  if (ld < N) return refuse("colsum_noalloc: row pitch %d is smaller than the %d columns", ld, N);
  if (N > MIMIR_COLSUM_NOALLOC_MAX_N)
    return refuse("colsum_noalloc: N = %d exceeds the built-in scratch (at most %d columns); "
                  "use mimir_colsum with your own buffer",
                  N, MIMIR_COLSUM_NOALLOC_MAX_N);
  float* scratch = mimir::colsum_scratch_for_current_device();
  if (!scratch) return -1;
  cudaGetLastError();  // an earlier, unrelated launch error must not be reported as this call's
  const int parts = rows >= 64 * 8 ? 64 : 1;  // same split as mimir_colsum, so results agree bit for bit
  dim3 grid(ceil_div(N, 256), parts);
  colsum_partial_kernel<<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), rows, N, ld, scratch);
  reduce_partials_kernel<<<ceil_div(N, 32), 1024, 0, st>>>(scratch, parts, N, N,
                                                          static_cast<__nv_bfloat16*>(out), nullptr,
                                                          accumulate);
  count_launch(2);
  return cudaGetLastError() == cudaSuccess ? 0 : refuse("colsum_noalloc: launch failed");
}
