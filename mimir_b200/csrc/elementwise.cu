// Vectorised (128-bit) elementwise families: embedding gather / scatter-add,
// GELU / SiLU / SwiGLU forward+backward, RoPE (interleaved and halves order),
// cast / scale / add, sum of squares, and the fused AdamW update over flat
// parameter buffers (bf16 parameter + fp32 master + m + v in one pass).
//
// Reference semantics: tensor/elementwise.go:556-594 (activations),
// nn/transformer.go:191-259 (RoPE), optim/optim.go:494-510 (AdamW rule),
// :198-215 (global-norm clip factor), :372-392 (master weights).
#include "common.cuh"
#include "philox.cuh"
#include "runtime.h"

namespace mimir {

__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float (&v)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
}
__device__ __forceinline__ void st8(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 u;
  u.x = pack_bf16x2(v[0], v[1]); u.y = pack_bf16x2(v[2], v[3]);
  u.z = pack_bf16x2(v[4], v[5]); u.w = pack_bf16x2(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

// ---------------------------------------------------------------------------
// Embedding
// ---------------------------------------------------------------------------
// out[m, :] = wte[tok[m], :] (+ wpe[m % T, :] when wpe != nullptr)
__global__ void embedding_fwd_kernel(const int64_t* __restrict__ tok, const __nv_bfloat16* __restrict__ wte,
                                     const __nv_bfloat16* __restrict__ wpe, __nv_bfloat16* __restrict__ out,
                                     int rows, int T, int C, int V, unsigned* err) {
  const int c8 = C / 8;
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<size_t>(rows) * c8) return;
  const int m = static_cast<int>(idx / c8), c = static_cast<int>(idx % c8) * 8;
  int64_t t = tok[m];
  if (t < 0 || t >= V) { raise_error(err, kErrIndex); t = 0; }
  float a[8];
  ld8(wte + static_cast<size_t>(t) * C + c, a);
  if (wpe) {
    float b[8];
    ld8(wpe + static_cast<size_t>(m % T) * C + c, b);
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] += b[j];
  }
  st8(out + static_cast<size_t>(m) * C + c, a);
}

// dwte[tok[m], :] += dx[m, :] with bf16x2 atomics (rows collide when a token repeats).
__global__ void embedding_bwd_kernel(const int64_t* __restrict__ tok, const __nv_bfloat16* __restrict__ dx,
                                     __nv_bfloat16* __restrict__ dwte, int rows, int C, int V) {
  const int c2 = C / 2;
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<size_t>(rows) * c2) return;
  const int m = static_cast<int>(idx / c2), c = static_cast<int>(idx % c2) * 2;
  const int64_t t = tok[m];
  if (t < 0 || t >= V) return;
  const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(dx + static_cast<size_t>(m) * C + c);
  atomicAdd(reinterpret_cast<__nv_bfloat162*>(dwte + static_cast<size_t>(t) * C + c), v);
}

// dwpe[t, :] (=|+=) sum_b dx[b*T + t, :]
__global__ void posemb_bwd_kernel(const __nv_bfloat16* __restrict__ dx, __nv_bfloat16* __restrict__ dwpe,
                                  int B, int T, int C, int accumulate) {
  const int c8 = C / 8;
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<size_t>(T) * c8) return;
  const int t = static_cast<int>(idx / c8), c = static_cast<int>(idx % c8) * 8;
  float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (accumulate) ld8(dwpe + static_cast<size_t>(t) * C + c, s);
  for (int b = 0; b < B; ++b) {
    float v[8];
    ld8(dx + (static_cast<size_t>(b) * T + t) * C + c, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) s[j] += v[j];
  }
  st8(dwpe + static_cast<size_t>(t) * C + c, s);
}

// ---------------------------------------------------------------------------
// Activations (standalone; the GEMM epilogue covers the fused cases)
// mode: 0 gelu_tanh, 1 silu, 2 relu
// ---------------------------------------------------------------------------
__device__ __forceinline__ float act_fwd(int mode, float x) {
  if (mode == 0) return gelu_tanh(x);
  if (mode == 1) return x / (1.f + __expf(-x));
  return fmaxf(x, 0.f);
}
__device__ __forceinline__ float act_bwd(int mode, float x) {
  if (mode == 0) return gelu_tanh_grad(x);
  if (mode == 1) { float s = 1.f / (1.f + __expf(-x)); return s * (1.f + x * (1.f - s)); }
  return x > 0.f ? 1.f : 0.f;
}
__global__ void act_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, size_t n8,
                               int mode) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  float v[8];
  ld8(x + i * 8, v);
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = act_fwd(mode, v[j]);
  st8(y + i * 8, v);
}
__global__ void act_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                               __nv_bfloat16* __restrict__ dx, size_t n8, int mode) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  float v[8], d[8];
  ld8(x + i * 8, v);
  ld8(dy + i * 8, d);
#pragma unroll
  for (int j = 0; j < 8; ++j) d[j] *= act_bwd(mode, v[j]);
  st8(dx + i * 8, d);
}

// SwiGLU over a fused [rows, 2F] gate|up matrix: y = silu(gate) * up.
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ y, int rows,
                                  int F) {
  const int f8 = F / 8;
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<size_t>(rows) * f8) return;
  const int r = static_cast<int>(idx / f8), c = static_cast<int>(idx % f8) * 8;
  float g[8], u[8];
  ld8(gu + static_cast<size_t>(r) * 2 * F + c, g);
  ld8(gu + static_cast<size_t>(r) * 2 * F + F + c, u);
#pragma unroll
  for (int j = 0; j < 8; ++j) g[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
  st8(y + static_cast<size_t>(r) * F + c, g);
}
// dgu[rows, 2F] from dy[rows, F]
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dy,
                                  __nv_bfloat16* __restrict__ dgu, int rows, int F) {
  const int f8 = F / 8;
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<size_t>(rows) * f8) return;
  const int r = static_cast<int>(idx / f8), c = static_cast<int>(idx % f8) * 8;
  float g[8], u[8], d[8], dg[8], du[8];
  ld8(gu + static_cast<size_t>(r) * 2 * F + c, g);
  ld8(gu + static_cast<size_t>(r) * 2 * F + F + c, u);
  ld8(dy + static_cast<size_t>(r) * F + c, d);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float s = 1.f / (1.f + __expf(-g[j]));
    du[j] = d[j] * g[j] * s;
    dg[j] = d[j] * u[j] * s * (1.f + g[j] * (1.f - s));
  }
  st8(dgu + static_cast<size_t>(r) * 2 * F + c, dg);
  st8(dgu + static_cast<size_t>(r) * 2 * F + F + c, du);
}

// The same product with gate and up in separate buffers (what two Linear layers produce).
__global__ void swiglu2_fwd_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up,
                                   __nv_bfloat16* __restrict__ y, size_t n8) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  float g[8], u[8];
  ld8(gate + i * 8, g);
  ld8(up + i * 8, u);
#pragma unroll
  for (int j = 0; j < 8; ++j) g[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
  st8(y + i * 8, g);
}
__global__ void swiglu2_bwd_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up,
                                   const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dgate,
                                   __nv_bfloat16* __restrict__ dup, size_t n8) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  float g[8], u[8], d[8], dg[8], du[8];
  ld8(gate + i * 8, g);
  ld8(up + i * 8, u);
  ld8(dy + i * 8, d);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float s = 1.f / (1.f + __expf(-g[j]));
    du[j] = d[j] * g[j] * s;
    dg[j] = d[j] * u[j] * s * (1.f + g[j] * (1.f - s));
  }
  st8(dgate + i * 8, dg);
  st8(dup + i * 8, du);
}

// ---------------------------------------------------------------------------
// RoPE applied in place to `nheads` heads of D dims starting at column col0 of
// x[rows, ld].  pos[row] gives the position.  interleaved: pairs (2i, 2i+1);
// otherwise halves (i, i + D/2).  inverse != 0 applies the transpose rotation
// (the backward pass).  freqs[D/2] are the per-pair angular frequencies.
// ---------------------------------------------------------------------------
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const int* __restrict__ pos,
                            const float* __restrict__ freqs, int rows, int ld, int col0, int nheads, int D,
                            int interleaved, int inverse) {
  const int half = D / 2;
  const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<size_t>(rows) * nheads * half) return;
  const int i = static_cast<int>(idx % half);
  const int h = static_cast<int>((idx / half) % nheads);
  const int r = static_cast<int>(idx / (static_cast<size_t>(half) * nheads));
  float ang = static_cast<float>(pos[r]) * freqs[i];
  float sn, cs;
  sincosf(ang, &sn, &cs);
  if (inverse) sn = -sn;
  __nv_bfloat16* base = x + static_cast<size_t>(r) * ld + col0 + h * D;
  const int i0 = interleaved ? 2 * i : i, i1 = interleaved ? 2 * i + 1 : i + half;
  const float a = __bfloat162float(base[i0]), b = __bfloat162float(base[i1]);
  base[i0] = __float2bfloat16_rn(a * cs - b * sn);
  base[i1] = __float2bfloat16_rn(a * sn + b * cs);
}

// ---------------------------------------------------------------------------
// cast / scale / add
// ---------------------------------------------------------------------------
__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y, size_t n,
                                        float scale) {
  const size_t i = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
  if (i + 8 <= n) {
    float4 a = *reinterpret_cast<const float4*>(x + i), b = *reinterpret_cast<const float4*>(x + i + 4);
    float v[8] = {a.x * scale, a.y * scale, a.z * scale, a.w * scale,
                  b.x * scale, b.y * scale, b.z * scale, b.w * scale};
    st8(y + i, v);
  } else {
    for (size_t j = i; j < n; ++j) y[j] = __float2bfloat16_rn(x[j] * scale);
  }
}
__global__ void cast_bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ y, size_t n,
                                        float scale) {
  const size_t i = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
  if (i + 8 <= n) {
    float v[8];
    ld8(x + i, v);
    *reinterpret_cast<float4*>(y + i) = make_float4(v[0] * scale, v[1] * scale, v[2] * scale, v[3] * scale);
    *reinterpret_cast<float4*>(y + i + 4) = make_float4(v[4] * scale, v[5] * scale, v[6] * scale, v[7] * scale);
  } else {
    for (size_t j = i; j < n; ++j) y[j] = __bfloat162float(x[j]) * scale;
  }
}
// y = a * alpha + b * beta (bf16), n % 8 == 0
__global__ void axpby_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                             __nv_bfloat16* __restrict__ y, size_t n8, float alpha, float beta) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  float u[8], v[8];
  ld8(a + i * 8, u);
  ld8(b + i * 8, v);
#pragma unroll
  for (int j = 0; j < 8; ++j) u[j] = u[j] * alpha + v[j] * beta;
  st8(y + i * 8, u);
}

// out[0] += sum(g^2) over bf16 (or fp32) grads; out must be zeroed by the caller.
template <typename T>
__global__ void __launch_bounds__(256) sumsq_kernel(const T* __restrict__ g, size_t n, float* __restrict__ out) {
  __shared__ float red[8];
  float s = 0.f;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x * 8;
  for (size_t i = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 8; i < n; i += stride) {
    if (i + 8 <= n) {
      float v[8];
      if constexpr (sizeof(T) == 2) {
        ld8(reinterpret_cast<const __nv_bfloat16*>(g) + i, v);
      } else {
        float4 a = *reinterpret_cast<const float4*>(g + i), b = *reinterpret_cast<const float4*>(g + i + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) s += v[j] * v[j];
    } else {
      for (size_t j = i; j < n; ++j) { float v = static_cast<float>(g[j]); s += v * v; }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += red[w];
    atomicAdd(out, t);
  }
}

// ---------------------------------------------------------------------------
// Fused AdamW over a flat range (n % 8 == 0, 16-byte aligned bases).
//   g = grad * gscale * clipcoef;  p *= 1 - lr*wd;  m = b1 m + (1-b1) g;
//   v = b2 v + (1-b2) g^2;  p -= (lr/bc1) * m / (sqrt(v)/sqrt(bc2) + eps)
// with p the fp32 master; the bf16 parameter is rewritten from it.
// clipcoef = min(1, clip / (sqrt(gnorm_sq[0]) * gscale + 1e-6)) when gnorm_sq != nullptr.
// ---------------------------------------------------------------------------
struct AdamArgs {
  float lr, beta1, beta2, eps, wd, bc1, bc2_sqrt, gscale, clip;
};
// Step-dependent values may instead come from device memory so that a captured
// CUDA graph can be replayed with a new learning rate and step count:
// hyper[0] = lr, hyper[1] = 1 - beta1^t, hyper[2] = sqrt(1 - beta2^t), hyper[3] = grad scale.
template <typename G>
__global__ void __launch_bounds__(256)
adamw_flat_kernel(float* __restrict__ master, __nv_bfloat16* __restrict__ param, const G* __restrict__ grad,
                  float* __restrict__ m, float* __restrict__ v, size_t n8, size_t decay_n8, AdamArgs a,
                  const float* __restrict__ gnorm_sq, const float* __restrict__ hyper) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  if (hyper) { a.lr = hyper[0]; a.bc1 = hyper[1]; a.bc2_sqrt = hyper[2]; a.gscale = hyper[3]; }
  if (i >= decay_n8) a.wd = 0.f;
  float gs = a.gscale;
  if (gnorm_sq) {
    const float norm = sqrtf(gnorm_sq[0]) * a.gscale;
    gs *= fminf(1.f, a.clip / (norm + 1e-6f));
  }
  float g[8];
  if constexpr (sizeof(G) == 2) {
    ld8(reinterpret_cast<const __nv_bfloat16*>(grad) + i * 8, g);
  } else {
    float4 x = *reinterpret_cast<const float4*>(grad + i * 8), y = *reinterpret_cast<const float4*>(grad + i * 8 + 4);
    g[0] = x.x; g[1] = x.y; g[2] = x.z; g[3] = x.w; g[4] = y.x; g[5] = y.y; g[6] = y.z; g[7] = y.w;
  }
  float4 p0 = *reinterpret_cast<float4*>(master + i * 8), p1 = *reinterpret_cast<float4*>(master + i * 8 + 4);
  float4 m0 = *reinterpret_cast<float4*>(m + i * 8), m1 = *reinterpret_cast<float4*>(m + i * 8 + 4);
  float4 v0 = *reinterpret_cast<float4*>(v + i * 8), v1 = *reinterpret_cast<float4*>(v + i * 8 + 4);
  float p[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
  float mm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
  float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
  const float decay = 1.f - a.lr * a.wd, step = a.lr / a.bc1;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float gj = g[j] * gs;
    p[j] *= decay;
    mm[j] = a.beta1 * mm[j] + (1.f - a.beta1) * gj;
    vv[j] = a.beta2 * vv[j] + (1.f - a.beta2) * gj * gj;
    p[j] -= step * mm[j] / (sqrtf(vv[j]) / a.bc2_sqrt + a.eps);
  }
  *reinterpret_cast<float4*>(master + i * 8) = make_float4(p[0], p[1], p[2], p[3]);
  *reinterpret_cast<float4*>(master + i * 8 + 4) = make_float4(p[4], p[5], p[6], p[7]);
  *reinterpret_cast<float4*>(m + i * 8) = make_float4(mm[0], mm[1], mm[2], mm[3]);
  *reinterpret_cast<float4*>(m + i * 8 + 4) = make_float4(mm[4], mm[5], mm[6], mm[7]);
  *reinterpret_cast<float4*>(v + i * 8) = make_float4(vv[0], vv[1], vv[2], vv[3]);
  *reinterpret_cast<float4*>(v + i * 8 + 4) = make_float4(vv[4], vv[5], vv[6], vv[7]);
  if (param) st8(param + i * 8, p);
}

static inline unsigned blocks_for(size_t n, int per_block) {
  return static_cast<unsigned>((n + per_block - 1) / per_block);
}

}  // namespace mimir


// ---------------------------------------------------------------------------
// Philox4x32-10 (counter = block index, key = the 64-bit seed).  Element i of a
// stream is word i % 4 of block i / 4; a thread produces one block.  Uniforms are
// the top 24 bits / 2^24, exactly as the host generator computes them, so a
// dropout mask drawn here matches the CPU's bit for bit
// (reference: backend/internal/gen/gen.go:577-610, backend/cpu/rand.go).
// ---------------------------------------------------------------------------
namespace mimir {
__global__ void philox_uniform_kernel(float* __restrict__ out, size_t n, uint64_t seed) {
  const size_t blk = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (blk * 4 >= n) return;
  const uint4 w = philox4x32_10(blk, seed);
  const uint32_t v[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int j = 0; j < 4; ++j)
    if (blk * 4 + j < n) out[blk * 4 + j] = static_cast<float>(v[j] >> 8) * (1.0f / 16777216.0f);
}
// y = x * keep / (1 - p) with keep = uniform >= p (bf16, 4 values per thread)
__global__ void philox_dropout_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, size_t n,
                                      uint64_t seed, float p, float scale) {
  const size_t blk = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (blk * 4 >= n) return;
  const uint4 w = philox4x32_10(blk, seed);
  const uint32_t v[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const size_t i = blk * 4 + j;
    if (i < n) {
      const float u = static_cast<float>(v[j] >> 8) * (1.0f / 16777216.0f);
      y[i] = u >= p ? __float2bfloat16_rn(__bfloat162float(x[i]) * scale) : __float2bfloat16_rn(0.f);
    }
  }
}
}  // namespace mimir

using namespace mimir;
typedef __nv_bfloat16 bf16;

MIMIR_API int mimir_embedding_fwd(const void* tok, const void* wte, const void* wpe, void* out, int rows,
                                  int T, int C, int V, cudaStream_t st) {
  if (C % 8) return refuse("embedding: C must be a multiple of 8");
  const size_t n = static_cast<size_t>(rows) * (C / 8);
  embedding_fwd_kernel<<<blocks_for(n, 256), 256, 0, st>>>(
      static_cast<const int64_t*>(tok), static_cast<const bf16*>(wte), static_cast<const bf16*>(wpe),
      static_cast<bf16*>(out), rows, T, C, V, error_word_dev());
  count_launch();
  return 0;
}
MIMIR_API int mimir_embedding_bwd(const void* tok, const void* dx, void* dwte, void* dwpe, int B, int T,
                                  int C, int V, int accumulate_wpe, cudaStream_t st) {
  if (C % 8) return refuse("embedding: C must be a multiple of 8");
  const int rows = B * T;
  const size_t n = static_cast<size_t>(rows) * (C / 2);
  embedding_bwd_kernel<<<blocks_for(n, 256), 256, 0, st>>>(static_cast<const int64_t*>(tok),
                                                           static_cast<const bf16*>(dx),
                                                           static_cast<bf16*>(dwte), rows, C, V);
  count_launch();
  if (dwpe) {
    const size_t np = static_cast<size_t>(T) * (C / 8);
    posemb_bwd_kernel<<<blocks_for(np, 128), 128, 0, st>>>(static_cast<const bf16*>(dx),
                                                           static_cast<bf16*>(dwpe), B, T, C, accumulate_wpe);
    count_launch();
  }
  return 0;
}
MIMIR_API int mimir_act_fwd(const void* x, void* y, long long n, int mode, cudaStream_t st) {
  if (n % 8) return refuse("activation: n must be a multiple of 8");
  act_fwd_kernel<<<blocks_for(n / 8, 256), 256, 0, st>>>(static_cast<const bf16*>(x), static_cast<bf16*>(y),
                                                         n / 8, mode);
  count_launch();
  return 0;
}
MIMIR_API int mimir_act_bwd(const void* x, const void* dy, void* dx, long long n, int mode, cudaStream_t st) {
  if (n % 8) return refuse("activation: n must be a multiple of 8");
  act_bwd_kernel<<<blocks_for(n / 8, 256), 256, 0, st>>>(static_cast<const bf16*>(x),
                                                         static_cast<const bf16*>(dy),
                                                         static_cast<bf16*>(dx), n / 8, mode);
  count_launch();
  return 0;
}
MIMIR_API int mimir_swiglu_fwd(const void* gu, void* y, int rows, int F, cudaStream_t st) {
  if (F % 8) return refuse("swiglu: F must be a multiple of 8");
  const size_t n = static_cast<size_t>(rows) * (F / 8);
  swiglu_fwd_kernel<<<blocks_for(n, 256), 256, 0, st>>>(static_cast<const bf16*>(gu), static_cast<bf16*>(y),
                                                        rows, F);
  count_launch();
  return 0;
}
MIMIR_API int mimir_swiglu_bwd(const void* gu, const void* dy, void* dgu, int rows, int F, cudaStream_t st) {
  if (F % 8) return refuse("swiglu: F must be a multiple of 8");
  const size_t n = static_cast<size_t>(rows) * (F / 8);
  swiglu_bwd_kernel<<<blocks_for(n, 256), 256, 0, st>>>(static_cast<const bf16*>(gu),
                                                        static_cast<const bf16*>(dy),
                                                        static_cast<bf16*>(dgu), rows, F);
  count_launch();
  return 0;
}
MIMIR_API int mimir_swiglu2_fwd(const void* gate, const void* up, void* y, long long n, cudaStream_t st) {
  if (n % 8) return refuse("swiglu: n must be a multiple of 8");
  swiglu2_fwd_kernel<<<blocks_for(n / 8, 256), 256, 0, st>>>(static_cast<const bf16*>(gate),
                                                             static_cast<const bf16*>(up), static_cast<bf16*>(y),
                                                             static_cast<size_t>(n / 8));
  count_launch();
  return 0;
}
MIMIR_API int mimir_swiglu2_bwd(const void* gate, const void* up, const void* dy, void* dgate, void* dup,
                                long long n, cudaStream_t st) {
  if (n % 8) return refuse("swiglu: n must be a multiple of 8");
  swiglu2_bwd_kernel<<<blocks_for(n / 8, 256), 256, 0, st>>>(
      static_cast<const bf16*>(gate), static_cast<const bf16*>(up), static_cast<const bf16*>(dy),
      static_cast<bf16*>(dgate), static_cast<bf16*>(dup), static_cast<size_t>(n / 8));
  count_launch();
  return 0;
}
MIMIR_API int mimir_rope(void* x, const int* pos, const float* freqs, int rows, int ld, int col0, int nheads,
                         int D, int interleaved, int inverse, cudaStream_t st) {
  if (D % 2) return refuse("rope: head dim must be even");
  const size_t n = static_cast<size_t>(rows) * nheads * (D / 2);
  rope_kernel<<<blocks_for(n, 256), 256, 0, st>>>(static_cast<bf16*>(x), pos, freqs, rows, ld, col0, nheads, D,
                                                  interleaved, inverse);
  count_launch();
  return 0;
}
MIMIR_API int mimir_cast_f32_bf16(const float* x, void* y, long long n, float scale, cudaStream_t st) {
  cast_f32_to_bf16_kernel<<<blocks_for((n + 7) / 8, 256), 256, 0, st>>>(x, static_cast<bf16*>(y), n, scale);
  count_launch();
  return 0;
}
MIMIR_API int mimir_cast_bf16_f32(const void* x, float* y, long long n, float scale, cudaStream_t st) {
  cast_bf16_to_f32_kernel<<<blocks_for((n + 7) / 8, 256), 256, 0, st>>>(static_cast<const bf16*>(x), y, n,
                                                                        scale);
  count_launch();
  return 0;
}
MIMIR_API int mimir_axpby(const void* a, const void* b, void* y, long long n, float alpha, float beta,
                          cudaStream_t st) {
  if (n % 8) return refuse("axpby: n must be a multiple of 8");
  axpby_kernel<<<blocks_for(n / 8, 256), 256, 0, st>>>(static_cast<const bf16*>(a), static_cast<const bf16*>(b),
                                                       static_cast<bf16*>(y), n / 8, alpha, beta);
  count_launch();
  return 0;
}
// out[0] += sum of squares; grad_is_f32 selects the element type.
MIMIR_API int mimir_sumsq(const void* g, long long n, int grad_is_f32, float* out, cudaStream_t st) {
  const unsigned grid = static_cast<unsigned>(sm_count() * 4);
  if (grad_is_f32)
    sumsq_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(g), n, out);
  else
    sumsq_kernel<bf16><<<grid, 256, 0, st>>>(static_cast<const bf16*>(g), n, out);
  count_launch();
  return 0;
}
// Elements [0, decay_n) get weight decay `wd`, the rest none.  hyper: optional
// device array {lr, 1-beta1^t, sqrt(1-beta2^t), grad scale} overriding lr/step/gscale.
MIMIR_API int mimir_adamw_flat(float* master, void* param, const void* grad, int grad_is_f32, float* m,
                               float* v, long long n, long long decay_n, float lr, float beta1, float beta2,
                               float eps, float wd, int step, float gscale, const float* gnorm_sq, float clip,
                               const float* hyper, cudaStream_t st) {
  if (n % 8 || decay_n % 8) return refuse("adamw: n and decay_n must be multiples of 8");
  if (n == 0) return 0;
  AdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.wd = wd;
  a.bc1 = 1.f - powf(beta1, static_cast<float>(step));
  a.bc2_sqrt = sqrtf(1.f - powf(beta2, static_cast<float>(step)));
  a.gscale = gscale; a.clip = clip;
  if (grad_is_f32)
    adamw_flat_kernel<float><<<blocks_for(n / 8, 256), 256, 0, st>>>(master, static_cast<bf16*>(param),
                                                                    static_cast<const float*>(grad), m, v,
                                                                    n / 8, decay_n / 8, a, gnorm_sq, hyper);
  else
    adamw_flat_kernel<bf16><<<blocks_for(n / 8, 256), 256, 0, st>>>(master, static_cast<bf16*>(param),
                                                                   static_cast<const bf16*>(grad), m, v,
                                                                   n / 8, decay_n / 8, a, gnorm_sq, hyper);
  count_launch();
  return 0;
}

MIMIR_API int mimir_philox_uniform(float* out, long long n, unsigned long long seed, cudaStream_t st) {
  if (n <= 0) return 0;
  const size_t blocks = (static_cast<size_t>(n) + 3) / 4;
  philox_uniform_kernel<<<static_cast<unsigned>((blocks + 255) / 256), 256, 0, st>>>(out, static_cast<size_t>(n), seed);
  count_launch();
  return 0;
}
// Inverted dropout with drop probability p; the same seed reproduces the mask (backward pass, other devices).
MIMIR_API int mimir_philox_dropout(const void* x, void* y, long long n, unsigned long long seed, float p,
                                   cudaStream_t st) {
  if (n <= 0) return 0;
  if (!(p >= 0.f && p < 1.f)) return refuse("dropout: probability %f outside [0, 1)", p);
  const size_t blocks = (static_cast<size_t>(n) + 3) / 4;
  philox_dropout_kernel<<<static_cast<unsigned>((blocks + 255) / 256), 256, 0, st>>>(
      static_cast<const bf16*>(x), static_cast<bf16*>(y), static_cast<size_t>(n), seed, p, 1.f / (1.f - p));
  count_launch();
  return 0;
}
