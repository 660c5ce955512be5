// ---------------------------------------------------------------------------
// Token sampling on the device: temperature, top-k, top-p (nucleus), min-p and a
// Philox draw in ONE kernel, one block per row of logits, so a decode loop reads
// back a 4-byte token id instead of a vocabulary of logits.
//
//   1. radix select (4 passes of 8 bits over order-preserving keys) finds the
//      k-th largest logit; k = top_k, at most 1024 (top_k <= 0 means 1024)
//   2. the candidates above the threshold are gathered, the ones equal to it are
//      taken in index order (a block-wide ordered count), so the set is the same
//      on every run
//   3. a bitonic sort in shared memory orders them by (logit descending, index
//      ascending)
//   4. softmax over the candidates (top_k > 0, or a vocabulary of at most 1024) or
//      over the whole vocabulary (top_k <= 0: the nucleus is then cut from the 1024
//      most probable tokens), min-p and top-p cuts as prefix conditions on the
//      sorted list, and one uniform from Philox4x32-10 (counter = draw index, word
//      = row % 4 of block row / 4) picks the token by inverse CDF
//
// temperature <= 0 or top_k == 1 is a plain arg-max (lowest index among equals).
//
// Replaces the host-side sampler of the reference (llm/sampler.go: sort of the whole
// vocabulary on the CPU after copying the logits back) and its GPU top-k / argsort
// kernels used for that purpose (backend/internal/gen/sort.go:62-180).
// ---------------------------------------------------------------------------
#include <cuda_bf16.h>
#include <float.h>

#include "common.cuh"
#include "philox.cuh"
#include "runtime.h"

namespace mimir {

namespace {

constexpr int kSampleThreads = 1024;
constexpr int kMaxCand = 1024;

__device__ __forceinline__ float ldf(const float* p) { return *p; }
__device__ __forceinline__ float ldf(const __nv_bfloat16* p) { return __bfloat162float(*p); }

// ascending order-preserving key of a float; NaN sorts below everything
__device__ __forceinline__ uint32_t fkey(float f) {
  if (f != f) return 0u;
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Calls f(index, value) for every logit of the row that belongs to this thread.  Rows that start on
// a 16-byte boundary are read eight values per 16-byte load, four loads in flight per thread (one
// block walks a whole row, so the bytes it keeps in flight set its speed); the order in which a
// thread sees its values is of no consequence to any caller.
constexpr int kLoadsInFlight = 4;

__device__ __forceinline__ void unpack8(const uint4& u, float v[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[2 * j] = __uint_as_float(w[j] << 16);
    v[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
  }
}

template <typename F>
__device__ __forceinline__ void for_each_logit(const __nv_bfloat16* x, int V, int tid, F f) {
  int done = 0;
  if ((reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    const int groups = V / 8;
    for (int g0 = tid; g0 < groups; g0 += kLoadsInFlight * kSampleThreads) {
      uint4 u[kLoadsInFlight];
#pragma unroll
      for (int j = 0; j < kLoadsInFlight; ++j) {
        const int g = g0 + j * kSampleThreads;
        if (g < groups) u[j] = *reinterpret_cast<const uint4*>(x + g * 8);
      }
#pragma unroll
      for (int j = 0; j < kLoadsInFlight; ++j) {
        const int g = g0 + j * kSampleThreads;
        if (g < groups) {
          float v[8];
          unpack8(u[j], v);
#pragma unroll
          for (int t = 0; t < 8; ++t) f(g * 8 + t, v[t]);
        }
      }
    }
    done = groups * 8;
  }
  for (int i = done + tid; i < V; i += kSampleThreads) f(i, __bfloat162float(x[i]));
}

template <typename F>
__device__ __forceinline__ void for_each_logit(const float* x, int V, int tid, F f) {
  int done = 0;
  if ((reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    const int groups = V / 4;
    for (int g0 = tid; g0 < groups; g0 += kLoadsInFlight * kSampleThreads) {
      float4 u[kLoadsInFlight];
#pragma unroll
      for (int j = 0; j < kLoadsInFlight; ++j) {
        const int g = g0 + j * kSampleThreads;
        if (g < groups) u[j] = *reinterpret_cast<const float4*>(x + g * 4);
      }
#pragma unroll
      for (int j = 0; j < kLoadsInFlight; ++j) {
        const int g = g0 + j * kSampleThreads;
        if (g < groups) {
          f(g * 4, u[j].x); f(g * 4 + 1, u[j].y); f(g * 4 + 2, u[j].z); f(g * 4 + 3, u[j].w);
        }
      }
    }
    done = groups * 4;
  }
  for (int i = done + tid; i < V; i += kSampleThreads) f(i, x[i]);
}

struct SampleSmem {
  uint32_t hist[32][256];     // one histogram per warp
  float cval[kMaxCand];
  int cidx[kMaxCand];
  float scan[kMaxCand];
  float red_f[32];
  int red_i[32];
  uint32_t prefix, need;
  int n_greater, tie_base, n_equal;
  float zfull, tie_val;
};

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float s = 0.f;
#pragma unroll
  for (int w = 0; w < kSampleThreads / 32; ++w) s += red[w];
  return s;
}

// candidate a sorts before candidate b
__device__ __forceinline__ bool before(float va, int ia, float vb, int ib) {
  return va > vb || (va == vb && ia < ib);
}

template <typename T>
__global__ void __launch_bounds__(kSampleThreads, 1)
sample_kernel(const T* __restrict__ logits, int ld, int V, float temperature, int top_k, float top_p, float min_p,
              uint64_t seed, uint64_t draw, const int* __restrict__ draw_dev, int* __restrict__ out_tok,
              float* __restrict__ out_prob) {
  extern __shared__ uint8_t smem_raw[];
  if (draw_dev) draw = static_cast<uint64_t>(*draw_dev);   // a step counter kept on the device (graph replays)
  SampleSmem& sm = *reinterpret_cast<SampleSmem*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row = blockIdx.x;
  const T* x = logits + static_cast<size_t>(row) * ld;

  // ---- arg-max
  if (temperature <= 0.f || top_k == 1) {
    float bv = -FLT_MAX;
    int bi = 0x7fffffff;
    for_each_logit(x, V, tid, [&](int i, float v) {
      if (before(v, i, bv, bi)) { bv = v; bi = i; }
    });
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (before(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { sm.red_f[warp] = bv; sm.red_i[warp] = bi; }
    __syncthreads();
    if (tid == 0) {
      for (int w = 1; w < kSampleThreads / 32; ++w)
        if (before(sm.red_f[w], sm.red_i[w], bv, bi)) { bv = sm.red_f[w]; bi = sm.red_i[w]; }
      out_tok[row] = bi == 0x7fffffff ? 0 : bi;
      if (out_prob) out_prob[row] = 1.f;
    }
    return;
  }

  const int k = min(min(top_k > 0 ? top_k : kMaxCand, kMaxCand), V);
  const float inv_t = 1.f / temperature;

  // ---- 1. radix select of the k-th largest key
  if (tid == 0) { sm.prefix = 0; sm.need = static_cast<uint32_t>(k); }
  uint32_t mask = 0;
  for (int pass = 3; pass >= 0; --pass) {
    for (int i = tid; i < 32 * 256; i += kSampleThreads) (&sm.hist[0][0])[i] = 0;
    __syncthreads();
    const uint32_t prefix = sm.prefix;
    const int shift = 8 * pass;
    for_each_logit(x, V, tid, [&](int, float v) {
      const uint32_t key = fkey(v);
      if ((key & mask) == prefix) atomicAdd(&sm.hist[warp][(key >> shift) & 255], 1u);
    });
    __syncthreads();
    if (tid < 256) {
      uint32_t s = 0;
#pragma unroll
      for (int w = 0; w < 32; ++w) s += sm.hist[w][tid];
      sm.hist[0][tid] = s;
    }
    __syncthreads();
    if (tid == 0) {
      uint32_t cum = 0, need = sm.need;
      int b = 255;
      for (; b > 0; --b) {
        if (cum + sm.hist[0][b] >= need) break;
        cum += sm.hist[0][b];
      }
      sm.need = need - cum;
      sm.prefix = prefix | (static_cast<uint32_t>(b) << shift);
    }
    mask |= 0xFFu << shift;
    __syncthreads();
  }
  const uint32_t thr = sm.prefix;            // key of the k-th largest logit
  const int need_ties = static_cast<int>(sm.need);
  const int n_greater_expected = k - need_ties;

  // ---- 2. gather: keys above the threshold in any order, equal keys in index order
  if (tid == 0) { sm.n_greater = 0; sm.tie_base = 0; sm.n_equal = 0; }
  for (int i = tid; i < kMaxCand; i += kSampleThreads) { sm.cval[i] = -FLT_MAX; sm.cidx[i] = 0x7fffffff; }
  __syncthreads();
  int* eq = reinterpret_cast<int*>(sm.scan);      // indices of the logits equal to the threshold (scan is free until step 4)
  for_each_logit(x, V, tid, [&](int i, float v) {
    const uint32_t key = fkey(v);
    if (key > thr) {
      const int pos = atomicAdd(&sm.n_greater, 1);
      if (pos < kMaxCand) { sm.cval[pos] = v; sm.cidx[pos] = i; }
    } else if (key == thr) {
      const int pos = atomicAdd(&sm.n_equal, 1);
      if (pos < kMaxCand) eq[pos] = i;
      sm.tie_val = v;                              // every such logit has the same bits
    }
  });
  __syncthreads();
  const int n_equal = sm.n_equal;
  if (n_equal <= kMaxCand) {
    // the usual case, a handful of equal logits: each one counts the equal logits with a smaller
    // index, and the need_ties lowest indices enter the candidate list
    if (tid < n_equal) {
      const int me = eq[tid];
      int rank = 0;
      for (int j = 0; j < n_equal; ++j) rank += eq[j] < me ? 1 : 0;
      if (rank < need_ties) { sm.cval[n_greater_expected + rank] = sm.tie_val; sm.cidx[n_greater_expected + rank] = me; }
    }
    __syncthreads();
  } else {
    // more than 1024 equal logits: walk the row in index order, tile by tile, until enough are taken
    for (int base = 0; base < V; base += kSampleThreads) {
      const int taken = sm.tie_base;
      if (taken >= need_ties) break;
      const int i = base + tid;
      float v = 0.f;
      bool tie = false;
      if (i < V) { v = ldf(x + i); tie = fkey(v) == thr; }
      const uint32_t ballot = __ballot_sync(0xffffffffu, tie);
      if (lane == 0) sm.red_i[warp] = __popc(ballot);
      __syncthreads();
      int before_me = taken;
      for (int w = 0; w < warp; ++w) before_me += sm.red_i[w];
      const int pos = before_me + __popc(ballot & ((1u << lane) - 1u));
      if (tie && pos < need_ties) { sm.cval[n_greater_expected + pos] = v; sm.cidx[n_greater_expected + pos] = i; }
      __syncthreads();
      if (tid == 0) {
        int t = taken;
        for (int w = 0; w < kSampleThreads / 32; ++w) t += sm.red_i[w];
        sm.tie_base = t;
      }
      __syncthreads();
    }
  }

  // ---- 3. bitonic sort of the first n_sort slots (the power of two that holds the k candidates;
  //         the slots behind them are padding) by (value descending, index ascending)
  int n_sort = 2;
  while (n_sort < k) n_sort <<= 1;
  for (int size = 2; size <= n_sort; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      const int other = tid ^ stride;
      if (other > tid && other < n_sort) {
        const float va = sm.cval[tid], vb = sm.cval[other];
        const int ia = sm.cidx[tid], ib = sm.cidx[other];
        const bool up = (tid & size) == 0;
        const bool swap = up ? before(vb, ib, va, ia) : before(va, ia, vb, ib);
        if (swap) { sm.cval[tid] = vb; sm.cval[other] = va; sm.cidx[tid] = ib; sm.cidx[other] = ia; }
      }
      __syncthreads();
    }
  }

  // ---- 4. probabilities, cuts and the draw
  const float vmax = sm.cval[0];
  const bool full_vocab = top_k <= 0 && V > kMaxCand;
  if (full_vocab) {
    float s = 0.f;
    for_each_logit(x, V, tid, [&](int, float v) { s += __expf((v - vmax) * inv_t); });
    s = block_sum(s, sm.red_f);
    if (tid == 0) sm.zfull = s;
    __syncthreads();
  }
  const float e = tid < k ? __expf((sm.cval[tid] - vmax) * inv_t) : 0.f;
  const float z = full_vocab ? sm.zfull : block_sum(e, sm.red_f);
  const float p = e / z;
  // inclusive scan of p over the sorted list
  float c = p;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float n = __shfl_up_sync(0xffffffffu, c, o);
    if (lane >= o) c += n;
  }
  __syncthreads();
  if (lane == 31) sm.red_f[warp] = c;
  __syncthreads();
  float warp_base = 0.f;
  for (int w = 0; w < warp; ++w) warp_base += sm.red_f[w];
  c += warp_base;
  sm.scan[tid] = c;
  __syncthreads();
  const float p0 = sm.scan[0];
  const bool keep = tid < k && (tid == 0 || ((c - p) < top_p && p >= min_p * p0));
  // both cuts are prefix conditions on the sorted list: the kept set is [0, nk)
  const uint32_t kb = __ballot_sync(0xffffffffu, keep);
  if (lane == 0) sm.red_i[warp] = __popc(kb);
  __syncthreads();
  int nk = 0;
  for (int w = 0; w < kSampleThreads / 32; ++w) {
    nk += sm.red_i[w];
    if (sm.red_i[w] < 32) break;
  }
  nk = max(nk, 1);
  const float total = sm.scan[nk - 1];
  const uint4 rnd = philox4x32_10(draw * ((gridDim.x + 3) / 4) + row / 4, seed);
  const uint32_t words[4] = {rnd.x, rnd.y, rnd.z, rnd.w};
  const float target = philox_unit(words[row & 3]) * total;
  // index = number of kept entries whose inclusive sum is <= target
  const bool below = tid < nk && c <= target;
  const uint32_t bb = __ballot_sync(0xffffffffu, below);
  __syncthreads();
  if (lane == 0) sm.red_i[warp] = __popc(bb);
  __syncthreads();
  if (tid == 0) {
    int idx = 0;
    for (int w = 0; w < kSampleThreads / 32; ++w) idx += sm.red_i[w];
    idx = min(idx, nk - 1);
    out_tok[row] = sm.cidx[idx];
    if (out_prob) out_prob[row] = (sm.scan[idx] - (idx ? sm.scan[idx - 1] : 0.f)) / total;
  }
}

}  // namespace

}  // namespace mimir

using namespace mimir;

// logits: [rows, V] fp32 or bf16 with row pitch ld (elements).  out_tok: int32 [rows];
// out_prob (optional): probability of the drawn token under the filtered distribution.
// `draw` numbers the call (a decode step), so one seed gives an independent uniform per
// (draw, row); when draw_dev is not null the number is read from that device int instead, which
// lets a captured decode step advance it between replays.
MIMIR_API int mimir_sample(const void* logits, int is_f32, int ld, int rows, int V, float temperature, int top_k,
                           float top_p, float min_p, unsigned long long seed, unsigned long long draw,
                           const int* draw_dev, int* out_tok, float* out_prob, cudaStream_t st) {
  if (rows <= 0 || V <= 0) return refuse("sample: empty logits");
  if (top_p <= 0.f) top_p = 1e-30f;
  const size_t smem = sizeof(SampleSmem);
  static_assert(sizeof(SampleSmem) <= 48 * 1024, "fits the default dynamic shared memory limit");
  if (is_f32)
    sample_kernel<float><<<rows, kSampleThreads, smem, st>>>(static_cast<const float*>(logits), ld, V, temperature,
                                                             top_k, top_p, min_p, seed, draw, draw_dev, out_tok, out_prob);
  else
    sample_kernel<__nv_bfloat16><<<rows, kSampleThreads, smem, st>>>(static_cast<const __nv_bfloat16*>(logits), ld, V,
                                                                     temperature, top_k, top_p, min_p, seed, draw,
                                                                     draw_dev, out_tok, out_prob);
  count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : refuse("sample launch failed");
}
