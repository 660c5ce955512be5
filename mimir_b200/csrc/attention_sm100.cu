// Fused attention forward and backward on tcgen05 tensor cores with the score
// and probability tiles held in TMEM (never in global memory).
//
// Semantics follow the reference's OpAttention / OpAttentionGrad
// (backend/op.go:117-135, backend/internal/gen/attention.go:234-662): softmax(
// scale * Q K^T + causal mask with offset) V, grouped-query heads, logsumexp
// (natural log) saved by the forward pass, probabilities recomputed from it in
// the backward pass, D = rowsum(dO * O) precomputed, and no atomics: like the
// reference's "key blocks" and "query blocks", one kernel owns dK/dV tiles and
// a second one owns dQ tiles.
//
// Layout: Q [B, Tq, Hq, D], K/V [B, Tk, Hkv, D] with arbitrary token pitch (so a
// fused [Q heads | K heads | V heads] projection output is read in place),
// O [B, Tq, Hq, D], LSE / Dsum [B, Hq, Tq] fp32.  D is 64 or 128.
//
// Forward CTA = 128 query rows of one (batch, head):
//   warp 0: TMA loads of Q once and of K/V tiles through a stage ring
//   warp 1: tcgen05.mma  S = Q K^T (smem x smem -> TMEM), O_part = P V (TMEM x smem)
//   warps 2-5: one thread per query row: online softmax out of TMEM, P written
//              back to TMEM as bf16 over S, running rescale of O in registers.
// S and O_part are double buffered in TMEM so that S(j+1) overlaps softmax(j).
#include "common.cuh"
#include "runtime.h"

namespace mimir {

constexpr int kAttFwdThreads = 320;   // every kernel here: TMA warp, MMA warp, 8 softmax warps (two per TMEM lane quadrant)
constexpr int kTile = 128;            // query rows and key rows per tile
constexpr int kChunkBytes = 128 * 128;  // 128 rows x 64 bf16

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct AttnParams {
  int B, Tq, Tk, Hq, Hkv;
  int causal, offset;  // key j visible to query i iff j <= i + offset
  float scale;         // softmax scale
  int ldo;             // token pitch of O / dQ output (elements)
  int ldkv;            // token pitch of dK / dV output (elements)
};

// K-major operand descriptor for a [128 x 64] bf16 chunk, k-step kk (16 elements)
__device__ __forceinline__ uint64_t kdesc(uint32_t chunk_addr, int kk) {
  return make_smem_desc_sw128(chunk_addr, 16, 1024) + static_cast<uint64_t>(kk * 2);
}
// MN-major operand descriptor over the same bytes: rows are the contraction
// index, ks selects rows [16 ks, 16 ks + 16); 64-column chunks are kChunkBytes apart.
__device__ __forceinline__ uint64_t mndesc(uint32_t tile_addr, int ks) {
  return make_smem_desc_sw128(tile_addr + ks * 2048, kChunkBytes, 1024);
}

template <int D>
__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* tm, uint64_t* bar, int h,
                                          int t0, int b) {
#pragma unroll
  for (int c = 0; c < D / 64; ++c) tma_load_4d(dst + c * kChunkBytes, tm, bar, c * 64, h, t0, b);
}

// S[128 x 128] = A[128 x D] * B[128 x D]^T, both K-major tiles in shared memory.
template <int D>
__device__ __forceinline__ void mma_scores(uint32_t d_tmem, uint32_t a_addr, uint32_t b_addr) {
  constexpr uint32_t idesc = make_idesc_bf16(128, 128, false, false);
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    const int chunk = ks / 4, kk = ks % 4;
    umma_ss(d_tmem, kdesc(a_addr + chunk * kChunkBytes, kk), kdesc(b_addr + chunk * kChunkBytes, kk),
            idesc, ks > 0 ? 1u : 0u);
  }
}
// Acc[128 x D] (+)= P[128 x 128] (bf16 in TMEM) * Bmn[128 x D] (rows = contraction index).
template <int D>
__device__ __forceinline__ void mma_from_tmem(uint32_t d_tmem, uint32_t p_tmem, uint32_t b_addr,
                                              bool accumulate) {
  constexpr uint32_t idesc = make_idesc_bf16(128, D, false, true);
#pragma unroll
  for (int ks = 0; ks < 8; ++ks)
    umma_ts(d_tmem, p_tmem + ks * 8, mndesc(b_addr, ks), idesc, (accumulate || ks > 0) ? 1u : 0u);
}

// Bounded rendezvous of the two warps that share a TMEM lane quadrant: publishes `seq` in *mine,
// waits until *theirs has reached it.  Returns false (and raises the abort flag) after two seconds,
// so a lost partner can never leave a warp spinning.
__device__ __forceinline__ bool pair_sync(volatile int* mine, volatile int* theirs, int seq, int lane,
                                          volatile int* abort_flag, unsigned* err) {
  __syncwarp();
  bool ok = true;
  if (lane == 0) {
    __threadfence_block();
    *mine = seq;
    uint64_t t0 = 0;
    for (uint32_t it = 1; *theirs < seq; ++it) {
      if ((it & 0xff) == 0) {
        if (*abort_flag) { ok = false; break; }
        const uint64_t now = global_timer_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > kWaitLimitNs) {
          *abort_flag = 1;
          raise_error(err, kErrWaitTimeout);
          ok = false;
          break;
        }
      }
    }
    __threadfence_block();
  }
  ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
  return ok;
}

// Half-tile forms used by the backward kernels: `hh` selects rows [64 hh, 64 hh + 64) of the B tile.
// S_half[128 x 64] = A[128 x D] * B_half[64 x D]^T
template <int D>
__device__ __forceinline__ void mma_scores_half(uint32_t d_tmem, uint32_t a_addr, uint32_t b_addr, int hh) {
  constexpr uint32_t idesc = make_idesc_bf16(128, 64, false, false);
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    const int chunk = ks / 4, kk = ks % 4;
    umma_ss(d_tmem, kdesc(a_addr + chunk * kChunkBytes, kk), kdesc(b_addr + chunk * kChunkBytes + hh * 8192, kk), idesc,
            ks > 0 ? 1u : 0u);
  }
}
// Acc[128 x D] (+)= P_half[128 x 64] (bf16 in TMEM) * Bmn_half[64 x D]
template <int D>
__device__ __forceinline__ void mma_from_tmem_half(uint32_t d_tmem, uint32_t p_tmem, uint32_t b_addr, int hh,
                                                   bool accumulate) {
  constexpr uint32_t idesc = make_idesc_bf16(128, D, false, true);
#pragma unroll
  for (int ks = 0; ks < 4; ++ks)
    umma_ts(d_tmem, p_tmem + ks * 8, mndesc(b_addr, hh * 4 + ks), idesc, (accumulate || ks > 0) ? 1u : 0u);
}

// ---------------------------------------------------------------------------
// Forward
// ---------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(kAttFwdThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, __nv_bfloat16* __restrict__ O,
                float* __restrict__ LSE, AttnParams p, unsigned* err) {
  constexpr int NST = D == 64 ? 3 : 2;
  constexpr int TB = (D / 64) * kChunkBytes;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + TB;
  uint8_t* sV = sK + NST * TB;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + NST * TB);
  uint64_t* q_full = bars;
  uint64_t* k_full = q_full + 1;
  uint64_t* k_empty = k_full + NST;
  uint64_t* v_full = k_empty + NST;
  uint64_t* v_empty = v_full + NST;
  uint64_t* s_full = v_empty + NST;
  uint64_t* p_ready = s_full + 2;   // [score buffer][key half]
  uint64_t* pv_done = p_ready + 4;  // [key half]: one completion per tile
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  __shared__ float xml[2][2][kTile];    // [m | l][half][row]: the halves' running maximum and sum, exchanged at the end
  __shared__ int xseq[2][4];            // [half][quadrant]: rendezvous counters of the partner warps

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = (p.Tq + kTile - 1) / kTile;
  const int qt = n_qt - 1 - blockIdx.x;  // heaviest (longest causal prefix) tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int q0 = qt * kTile;
  int n_kv = (p.Tk + kTile - 1) / kTile;
  if (p.causal) {
    const int last_key = q0 + kTile - 1 + p.offset;
    n_kv = last_key < 0 ? 0 : min(n_kv, last_key / kTile + 1);
  }

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < NST; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) { mbar_init(&s_full[i], 1); mbar_init(&pv_done[i], 1); }
    for (int i = 0; i < 4; ++i) mbar_init(&p_ready[i], 4);
    for (int i = 0; i < 8; ++i) (&xseq[0][0])[i] = 0;
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem;        // two 128-column score buffers
  const uint32_t tO = tmem + 256;  // two D-column output accumulators, one per key half

  if (warp == 0) {
    if (lane == 0 && n_kv > 0) {
      mbar_arrive_expect_tx(q_full, TB);
      load_tile<D>(sQ, &tmQ, q_full, h, q0, b);
      for (int j = 0; j < n_kv; ++j) {
        const int s = j % NST;
        const uint32_t ph = (j / NST) & 1;
        if (!mbar_wait(&k_empty[s], ph ^ 1, abort_flag, err)) break;
        mbar_arrive_expect_tx(&k_full[s], TB);
        load_tile<D>(sK + s * TB, &tmK, &k_full[s], hk, j * kTile, b);
        if (!mbar_wait(&v_empty[s], ph ^ 1, abort_flag, err)) break;
        mbar_arrive_expect_tx(&v_full[s], TB);
        load_tile<D>(sV + s * TB, &tmV, &v_full[s], hk, j * kTile, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_kv > 0) {
      bool ok = mbar_wait(q_full, 0, abort_flag, err);
      const uint32_t aQ = smem_u32(sQ);
      if (ok && (ok = mbar_wait(&k_full[0], 0, abort_flag, err))) {
        tc_fence_after();
        mma_scores<D>(tS, aQ, smem_u32(sK));
        umma_commit(&s_full[0]);
        umma_commit(&k_empty[0]);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) {
          const int s = (j + 1) % NST;
          if (!(ok = mbar_wait(&k_full[s], ((j + 1) / NST) & 1, abort_flag, err))) break;
          tc_fence_after();
          mma_scores<D>(tS + ((j + 1) & 1) * 128, aQ, smem_u32(sK + s * TB));
          umma_commit(&s_full[(j + 1) & 1]);
          umma_commit(&k_empty[s]);
        }
        const int s = j % NST, bi = j & 1;
        if (!(ok = mbar_wait(&v_full[s], (j / NST) & 1, abort_flag, err))) break;
        // the two key halves are independent streams: each accumulates P_half * V_half into its own
        // accumulator as soon as its softmax warps have written P_half
        for (int hh = 0; hh < 2 && ok; ++hh) {
          if (!(ok = mbar_wait(&p_ready[bi * 2 + hh], (j >> 1) & 1, abort_flag, err))) break;
          tc_fence_after();
          mma_from_tmem_half<D>(tO + hh * D, tS + bi * 128 + hh * 64, smem_u32(sV + s * TB), hh, j > 0);
          umma_commit(&pv_done[hh]);
        }
        if (ok) umma_commit(&v_empty[s]);
      }
    }
  } else {
    // Eight softmax warps: two per 32-row TMEM lane quadrant.  `half` 0 owns keys 0..63 of every key
    // tile, `half` 1 keys 64..127, and each half is an attention of its own over its keys: own
    // running maximum and row sum, own accumulator O_half in TMEM (P_half * V_half, accumulated by
    // the tensor core across tiles).  The halves never talk to each other inside the loop, so they
    // drift apart by up to one tile and the exponentials of one overlap the loads, maxima and
    // stores of the other; their results are merged once at the end.  The accumulator is rescaled
    // only when a row's maximum has grown by more than 2^8 since the last rescale (P stays below
    // 2^8, harmless in bf16 / fp32), which after the first tiles almost never happens.
    const int quad = warp & 3, half = (warp - 2) >> 2;
    const int r = quad * 32 + lane;
    const int q_pos = q0 + r;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const float sl2 = p.scale * 1.4426950408889634f;
    constexpr int DH = D / 2;
    float m = -INFINITY, l = 0.f;   // m: the maximum the probabilities are scaled by
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      const int bi = j & 1;
      if (!(ok = mbar_wait(&s_full[bi], (j >> 1) & 1, abort_flag, err))) break;
      tc_fence_after();
      const int kv0 = j * kTile + half * 64;
      const bool need_mask = (p.causal && kv0 + 63 > q0 + p.offset) || (kv0 + 64 > p.Tk);
      const int limit = p.causal ? min(p.Tk - 1, q_pos + p.offset) : p.Tk - 1;  // last visible key
      const uint32_t ts = tS + bi * 128 + half * 64 + lane_base;
      uint32_t s0[32], s1[32];
      tmem_ld32(ts, s0);
      tmem_ld32(ts + 32, s1);
      tmem_ld_wait();
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
      if (need_mask) {
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          if (kv0 + e > limit) s0[e] = 0xff800000u;
          if (kv0 + 32 + e > limit) s1[e] = 0xff800000u;
        }
      }
#pragma unroll
      for (int e = 0; e < 32; e += 2) {
        mx0 = fmaxf(mx0, __uint_as_float(s0[e]));
        mx1 = fmaxf(mx1, __uint_as_float(s0[e + 1]));
        mx2 = fmaxf(mx2, __uint_as_float(s1[e]));
        mx3 = fmaxf(mx3, __uint_as_float(s1[e + 1]));
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      const bool grow = mx != -INFINITY && (mx - m) * sl2 > 8.f;   // also the first finite maximum (m = -inf)
      if (__any_sync(0xffffffffu, grow)) {
        const float alpha = grow ? ex2((m - mx) * sl2) : 1.f;       // ex2(-inf) = 0 for the first one
        if (grow) m = mx;
        l *= alpha;
        if (j > 0) {
          // O_half *= alpha in TMEM, after the product of the previous tile has landed
          if (!(ok = mbar_wait(&pv_done[half], (j - 1) & 1, abort_flag, err))) break;
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t rr[32];
            tmem_ld32(tO + half * D + lane_base + c * 32, rr);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) rr[e] = __float_as_uint(__uint_as_float(rr[e]) * alpha);
            tmem_st32(tO + half * D + lane_base + c * 32, rr);
          }
        }
      }
      const float msl = (m == -INFINITY ? 0.f : m) * sl2;
      float rs0 = 0.f, rs1 = 0.f;
      uint32_t pk[32];
#pragma unroll
      for (int e = 0; e < 32; e += 2) {
        const float p0 = ex2(__uint_as_float(s0[e]) * sl2 - msl), p1 = ex2(__uint_as_float(s0[e + 1]) * sl2 - msl);
        const float p2 = ex2(__uint_as_float(s1[e]) * sl2 - msl), p3 = ex2(__uint_as_float(s1[e + 1]) * sl2 - msl);
        rs0 += p0 + p1;
        rs1 += p2 + p3;
        pk[e >> 1] = pack_bf16x2(p0, p1);
        pk[16 + (e >> 1)] = pack_bf16x2(p2, p3);
      }
      // P_half (bf16 pairs) goes over the first 32 columns of this half's own scores
      tmem_st32(ts, pk);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[bi * 2 + half]);
      l += rs0 + rs1;
    }
    // merge the halves: both products of the last tile must have landed
    if (ok && n_kv > 0) {
      ok = mbar_wait(&pv_done[0], (n_kv - 1) & 1, abort_flag, err) &&
           mbar_wait(&pv_done[1], (n_kv - 1) & 1, abort_flag, err);
      tc_fence_after();
    }
    xml[0][half][r] = m;
    xml[1][half][r] = l;
    if (ok) ok = pair_sync(&xseq[half][quad], &xseq[half ^ 1][quad], 1, lane, abort_flag, err);
    const float m_o = xml[0][half ^ 1][r], l_o = xml[1][half ^ 1][r];
    const float mm = fmaxf(m, m_o);
    const float f_me = m == -INFINITY ? 0.f : ex2((m - mm) * sl2);
    const float f_ot = m_o == -INFINITY ? 0.f : ex2((m_o - mm) * sl2);
    const float f0 = half == 0 ? f_me : f_ot, f1 = half == 0 ? f_ot : f_me;   // factors of O_0 and O_1
    const float lsum = l * f_me + l_o * f_ot;
    if (ok && n_kv > 0) {
      // the TMEM loads are warp-wide instructions: every lane takes part, only the stores to global
      // memory depend on whether the lane's row exists
      const bool row_ok = q_pos < p.Tq;
      const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
      __nv_bfloat16* dst = O + (static_cast<size_t>(b) * p.Tq + q_pos) * p.ldo + h * D + half * DH;
#pragma unroll
      for (int c = 0; c < DH / 32; ++c) {
        uint32_t ra[32], rb[32];
        tmem_ld32(tO + lane_base + half * DH + c * 32, ra);
        tmem_ld32(tO + D + lane_base + half * DH + c * 32, rb);
        tmem_ld_wait();
#pragma unroll
        for (int d = 0; d < 32; d += 8) {
          float v[8];
#pragma unroll
          for (int e = 0; e < 8; ++e)
            v[e] = (__uint_as_float(ra[d + e]) * f0 + __uint_as_float(rb[d + e]) * f1) * inv;
          uint4 u;
          u.x = pack_bf16x2(v[0], v[1]); u.y = pack_bf16x2(v[2], v[3]);
          u.z = pack_bf16x2(v[4], v[5]); u.w = pack_bf16x2(v[6], v[7]);
          if (row_ok) *reinterpret_cast<uint4*>(dst + c * 32 + d) = u;
        }
      }
      if (row_ok && LSE && half == 0)
        LSE[(static_cast<size_t>(b) * p.Hq + h) * p.Tq + q_pos] =
            lsum > 0.f ? (mm * sl2 + log2f(lsum)) * 0.6931471805599453f : -INFINITY;
    } else if (ok && n_kv == 0 && q_pos < p.Tq) {
      // no visible key at all: a zero row (the reference's zero-row rule) and -inf log-sum-exp
      __nv_bfloat16* dst = O + (static_cast<size_t>(b) * p.Tq + q_pos) * p.ldo + h * D + half * DH;
#pragma unroll
      for (int d = 0; d < DH; d += 8) *reinterpret_cast<uint4*>(dst + d) = make_uint4(0, 0, 0, 0);
      if (LSE && half == 0) LSE[(static_cast<size_t>(b) * p.Hq + h) * p.Tq + q_pos] = -INFINITY;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ---------------------------------------------------------------------------
// Dsum[b, h, i] = sum_d dO[b, i, h, d] * O[b, i, h, d]
// ---------------------------------------------------------------------------
__global__ void attn_dsum_kernel(const __nv_bfloat16* __restrict__ O, const __nv_bfloat16* __restrict__ dO,
                                 float* __restrict__ dsum, int B, int T, int H, int D, int ldo, int lddo) {
  const int per = D / 8;  // lanes per (token, head)
  const size_t gid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t item = gid / per;
  const int part = static_cast<int>(gid % per);
  const bool live = item < static_cast<size_t>(B) * T * H;
  float s = 0.f;
  size_t tok = 0;
  int h = 0;
  if (live) {
    tok = item / H;
    h = static_cast<int>(item % H);
    uint4 a = *reinterpret_cast<const uint4*>(O + tok * ldo + h * D + part * 8);
    uint4 g = *reinterpret_cast<const uint4*>(dO + tok * lddo + h * D + part * 8);
    float2 a0 = unpack_bf16x2(a.x), a1 = unpack_bf16x2(a.y), a2 = unpack_bf16x2(a.z), a3 = unpack_bf16x2(a.w);
    float2 g0 = unpack_bf16x2(g.x), g1 = unpack_bf16x2(g.y), g2 = unpack_bf16x2(g.z), g3 = unpack_bf16x2(g.w);
    s = a0.x * g0.x + a0.y * g0.y + a1.x * g1.x + a1.y * g1.y + a2.x * g2.x + a2.y * g2.y + a3.x * g3.x +
        a3.y * g3.y;
  }
  for (int o = per >> 1; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (live && part == 0) {
    const size_t bb = tok / T, t = tok % T;
    dsum[(bb * H + h) * T + t] = s;
  }
}

// ---------------------------------------------------------------------------
// Backward.  MODE 0: CTA owns a key tile, accumulates dV and dK over the query
// tiles (and over the query heads of its group); scores are built transposed
// (rows = keys) so that P^T and dS^T sit in TMEM as the A operand.
// MODE 1: CTA owns a query tile and accumulates dQ over the key tiles.
//   X tiles (loaded once):   MODE 0: K, V      MODE 1: Q, dO
//   Y tiles (ring):          MODE 0: Q, dO     MODE 1: K, V
//   S'  = X0 * Y0^T,  dP' = X1 * Y1^T
// ---------------------------------------------------------------------------
template <int D, int MODE>
__global__ void __launch_bounds__(kAttFwdThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmX0, const __grid_constant__ CUtensorMap tmX1,
                const __grid_constant__ CUtensorMap tmY0, const __grid_constant__ CUtensorMap tmY1,
                const float* __restrict__ LSE, const float* __restrict__ Dsum,
                __nv_bfloat16* __restrict__ out0, __nv_bfloat16* __restrict__ out1, AttnParams p,
                unsigned* err) {
  constexpr int NST = 2;
  constexpr int TB = (D / 64) * kChunkBytes;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sX0 = smem;
  uint8_t* sX1 = sX0 + TB;
  uint8_t* sY = sX1 + TB;  // NST x (Y0, Y1)
  // per softmax warp, double buffered: [2][8 warps][lse*log2e (128) | dsum (128)]
  float* vec = reinterpret_cast<float*>(sY + NST * 2 * TB);
  uint64_t* bars = reinterpret_cast<uint64_t*>(vec + 2 * 8 * 256);
  uint64_t* x_full = bars;
  uint64_t* y_full = x_full + 1;
  uint64_t* y_empty = y_full + NST;
  uint64_t* s_full = y_empty + NST;   // [2]: one per score / dP half-tile buffer
  uint64_t* p_ready = s_full + 2;     // [2]
  uint64_t* acc_full = p_ready + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  __shared__ int xseq[2][4];   // [half][quadrant]: rendezvous counters of the two warps sharing a lane quadrant

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = p.Hq / p.Hkv;
  const int b = blockIdx.z;
  const int xt = blockIdx.x;  // tile index of the owned (row) tile
  const int x0 = xt * kTile;
  const int n_qt = (p.Tq + kTile - 1) / kTile, n_kt = (p.Tk + kTile - 1) / kTile;
  // inner tile range [y_begin, y_end) and number of heads to loop over
  int y_begin, y_end, n_heads, hx;
  if (MODE == 0) {
    hx = blockIdx.y;  // kv head
    n_heads = group;
    y_end = n_qt;
    // first query tile that can see key x0: i + offset >= x0
    y_begin = p.causal ? max(0, (x0 - p.offset) / kTile) : 0;
    if (p.causal && x0 - p.offset < 0) y_begin = 0;
  } else {
    hx = blockIdx.y;  // query head
    n_heads = 1;
    y_begin = 0;
    y_end = n_kt;
    if (p.causal) {
      const int last_key = x0 + kTile - 1 + p.offset;
      y_end = last_key < 0 ? 0 : min(n_kt, last_key / kTile + 1);
    }
  }
  const int n_inner = max(0, y_end - y_begin);
  const int n_iter = n_inner * n_heads;

  if (threadIdx.x == 0) {
    mbar_init(x_full, 1);
    for (int s = 0; s < NST; ++s) { mbar_init(&y_full[s], 1); mbar_init(&y_empty[s], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&s_full[i], 1); mbar_init(&p_ready[i], 8); }
    mbar_init(acc_full, 1);
    for (int i = 0; i < 8; ++i) (&xseq[0][0])[i] = 0;
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // two half-tile buffers (64 score columns + 64 dP columns each) at 0 and 128, accumulators above:
  // the MMAs of half-tile j+1 run while the softmax warps work on half-tile j
  const uint32_t tBuf = tmem, tA0 = tmem + 256, tA1 = tmem + 256 + D;

  if (warp == 0) {
    if (lane == 0 && n_iter > 0) {
      mbar_arrive_expect_tx(x_full, 2 * TB);
      const int hx_load = hx;
      load_tile<D>(sX0, &tmX0, x_full, hx_load, x0, b);
      load_tile<D>(sX1, &tmX1, x_full, hx_load, x0, b);
      for (int it = 0; it < n_iter; ++it) {
        const int g = it / n_inner, yt = y_begin + it % n_inner;
        const int hy = MODE == 0 ? hx * group + g : hx / group;
        const int s = it % NST;
        if (!mbar_wait(&y_empty[s], ((it / NST) & 1) ^ 1, abort_flag, err)) break;
        mbar_arrive_expect_tx(&y_full[s], 2 * TB);
        load_tile<D>(sY + (s * 2) * TB, &tmY0, &y_full[s], hy, yt * kTile, b);
        load_tile<D>(sY + (s * 2 + 1) * TB, &tmY1, &y_full[s], hy, yt * kTile, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_iter > 0) {
      bool ok = mbar_wait(x_full, 0, abort_flag, err);
      const uint32_t aX0 = smem_u32(sX0), aX1 = smem_u32(sX1);
      const int n_half = 2 * n_iter;
      auto issue_scores = [&](int j) -> bool {
        const int it = j >> 1, hh = j & 1, s = it % NST;
        const uint32_t aY0 = smem_u32(sY + (s * 2) * TB), aY1 = aY0 + TB;
        if (hh == 0 && !mbar_wait(&y_full[s], (it / NST) & 1, abort_flag, err)) return false;
        tc_fence_after();
        const uint32_t tb = tBuf + (j & 1) * 128;
        mma_scores_half<D>(tb, aX0, aY0, hh);
        mma_scores_half<D>(tb + 64, aX1, aY1, hh);
        umma_commit(&s_full[j & 1]);
        return true;
      };
      if (ok && n_half > 0) ok = issue_scores(0);
      for (int j = 0; j < n_half && ok; ++j) {
        if (j + 1 < n_half && !(ok = issue_scores(j + 1))) break;   // overlaps the softmax of half-tile j
        const int it = j >> 1, hh = j & 1, s = it % NST;
        const uint32_t aY0 = smem_u32(sY + (s * 2) * TB), aY1 = aY0 + TB;
        const uint32_t tb = tBuf + (j & 1) * 128;
        if (!(ok = mbar_wait(&p_ready[j & 1], (j >> 1) & 1, abort_flag, err))) break;
        tc_fence_after();
        if (MODE == 0) {
          mma_from_tmem_half<D>(tA0, tb, aY1, hh, j > 0);        // dV += P^T dO
          mma_from_tmem_half<D>(tA1, tb + 64, aY0, hh, j > 0);   // dK += dS^T Q
        } else {
          mma_from_tmem_half<D>(tA0, tb + 64, aY0, hh, j > 0);   // dQ += dS K
        }
        if (hh == 1) umma_commit(&y_empty[s]);
      }
      if (ok) umma_commit(acc_full);
    }
  } else {
    // Two warps per TMEM lane quadrant.  A 128-column inner tile is processed as two 64-column
    // half-tiles in alternating TMEM buffers (the MMAs of one half run under the softmax of the
    // other); of a half-tile, `half` 0 takes columns 0..31 and `half` 1 columns 32..63, and in the
    // epilogue the two take alternate 32-column chunks of the accumulators.  Both read their columns
    // into registers, meet (bounded), and only then write P / dS over the score / dP buffers, whose
    // bf16 columns overlap the partner's unread fp32 columns.
    const int quad = warp & 3, half = (warp - 2) >> 2;
    const int r = quad * 32 + lane;  // row inside the owned tile
    const int x_pos = x0 + r;
    const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
    const float sl2 = p.scale * 1.4426950408889634f;
    const float kLog2e = 1.4426950408889634f;
    float my_lse2 = 0.f, my_dsum = 0.f;
    if (MODE == 1) {
      const bool live = x_pos < p.Tq;
      const size_t idx = (static_cast<size_t>(b) * p.Hq + hx) * p.Tq + (live ? x_pos : 0);
      my_lse2 = live ? LSE[idx] * kLog2e : INFINITY;
      my_dsum = live ? Dsum[idx] : 0.f;
    }
    bool ok = true;
    for (int j = 0; j < 2 * n_iter && ok; ++j) {
      const int it = j >> 1, hh = j & 1;
      const int g = it / n_inner, yt = y_begin + it % n_inner;
      const int y0 = yt * kTile;
      float* vbuf = vec + ((it & 1) * 8 + (warp - 2)) * 256;
      if (MODE == 0 && hh == 0) {
        // each warp stages its own copy of this query tile's logsumexp and Dsum vectors
        const int hq = hx * group + g;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int qi = i * 32 + lane, qp = y0 + qi;
          const bool live = qp < p.Tq;
          const size_t idx = (static_cast<size_t>(b) * p.Hq + hq) * p.Tq + (live ? qp : 0);
          vbuf[qi] = live ? LSE[idx] * kLog2e : INFINITY;
          vbuf[128 + qi] = live ? Dsum[idx] : 0.f;
        }
        __syncwarp();
      }
      if (!(ok = mbar_wait(&s_full[j & 1], (j >> 1) & 1, abort_flag, err))) break;
      tc_fence_after();
      // visibility of column c (position y0 + c) for this thread's row
      //   MODE 0: row = key, column = query: visible iff key <= query + offset
      //   MODE 1: row = query, column = key
      const bool row_live = MODE == 0 ? x_pos < p.Tk : x_pos < p.Tq;
      int c_lo = 0, c_hi = kTile;  // visible columns [c_lo, c_hi)
      if (MODE == 0) {
        c_hi = min(kTile, p.Tq - y0);
        if (p.causal) c_lo = max(0, x_pos - p.offset - y0);
      } else {
        c_hi = min(kTile, p.Tk - y0);
        if (p.causal) c_hi = min(c_hi, x_pos + p.offset - y0 + 1);
      }
      if (!row_live) c_hi = 0;
      // this warp's 32 columns of the half-tile: tile columns [cbase, cbase + 32)
      const int cbase = hh * 64 + half * 32;
      const uint32_t tb = tBuf + (j & 1) * 128 + lane_base;
      uint32_t rs[32], rd[32], pk[16], dk[16];
      tmem_ld32(tb + half * 32, rs);
      tmem_ld32(tb + 64 + half * 32, rd);
      tmem_ld_wait();
      // P / dS (bf16 pairs) go over columns 0..31 of the score / dP buffers, which the partner warp reads
      if (!(ok = pair_sync(&xseq[half][quad], &xseq[half ^ 1][quad], j + 1, lane, abort_flag, err))) break;
#pragma unroll
      for (int e = 0; e < 32; e += 2) {
        float pv[2], dv[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int col = cbase + e + u;
          const float lse2 = MODE == 0 ? vbuf[col] : my_lse2;
          const float ds = MODE == 0 ? vbuf[128 + col] : my_dsum;
          float pr = ex2(__uint_as_float(rs[e + u]) * sl2 - lse2);
          if (col < c_lo || col >= c_hi) pr = 0.f;
          pv[u] = pr;
          dv[u] = pr * (__uint_as_float(rd[e + u]) - ds);
        }
        pk[e >> 1] = pack_bf16x2(pv[0], pv[1]);
        dk[e >> 1] = pack_bf16x2(dv[0], dv[1]);
      }
      if (MODE == 0) tmem_st16(tb + half * 16, pk);
      tmem_st16(tb + 64 + half * 16, dk);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[j & 1]);
    }
    if (ok && n_iter > 0 && mbar_wait(acc_full, 0, abort_flag, err)) {
      tc_fence_after();
      const bool live = MODE == 0 ? x_pos < p.Tk : x_pos < p.Tq;
      const int T = MODE == 0 ? p.Tk : p.Tq;
      const int ld = MODE == 0 ? p.ldkv : p.ldo;
#pragma unroll
      for (int a = 0; a < (MODE == 0 ? 2 : 1); ++a) {
        // MODE 0: a = 0 is dV (unscaled), a = 1 is dK (times the softmax scale)
        const float mul = (MODE == 0 && a == 0) ? 1.f : p.scale;
        __nv_bfloat16* outp = a == 0 ? out0 : out1;
        __nv_bfloat16* dst = outp + (static_cast<size_t>(b) * T + (live ? x_pos : 0)) * ld + hx * D;
        const uint32_t ta = (a == 0 ? tA0 : tA1) + lane_base;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          if ((c & 1) != half) continue;   // the two warps of a quadrant take alternate 32-column chunks
          uint32_t rr[32];
          tmem_ld32(ta + c * 32, rr);
          tmem_ld_wait();
          if (live) {
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
              uint4 u;
              u.x = pack_bf16x2(__uint_as_float(rr[e]) * mul, __uint_as_float(rr[e + 1]) * mul);
              u.y = pack_bf16x2(__uint_as_float(rr[e + 2]) * mul, __uint_as_float(rr[e + 3]) * mul);
              u.z = pack_bf16x2(__uint_as_float(rr[e + 4]) * mul, __uint_as_float(rr[e + 5]) * mul);
              u.w = pack_bf16x2(__uint_as_float(rr[e + 6]) * mul, __uint_as_float(rr[e + 7]) * mul);
              *reinterpret_cast<uint4*>(dst + c * 32 + e) = u;
            }
          }
        }
      }
    } else if (n_iter == 0) {
      // nothing attends here (possible only with a negative causal offset): zero gradients
      const bool live = MODE == 0 ? x_pos < p.Tk : x_pos < p.Tq;
      if (live && half == 0) {
        const int T = MODE == 0 ? p.Tk : p.Tq;
        const int ld = MODE == 0 ? p.ldkv : p.ldo;
        for (int a = 0; a < (MODE == 0 ? 2 : 1); ++a) {
          __nv_bfloat16* outp = a == 0 ? out0 : out1;
          __nv_bfloat16* dst = outp + (static_cast<size_t>(b) * T + x_pos) * ld + hx * D;
          for (int d = 0; d < D; d += 8) *reinterpret_cast<uint4*>(dst + d) = make_uint4(0, 0, 0, 0);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

static int make_map4(CUtensorMap* tm, const void* base, int D, int H, int T, int B, int ld) {
  uint64_t dims[4] = {static_cast<uint64_t>(D), static_cast<uint64_t>(H), static_cast<uint64_t>(T),
                      static_cast<uint64_t>(B)};
  uint64_t strides[3] = {static_cast<uint64_t>(D) * 2, static_cast<uint64_t>(ld) * 2,
                         static_cast<uint64_t>(T) * ld * 2};
  uint32_t box[4] = {64, 1, 128, 1};
  return encode_tmap(tm, base, 2, 4, dims, strides, box, 3);
}

template <typename Kern>
static int set_smem(Kern kern, int bytes) {
  return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess
             ? 0
             : refuse("attention: cannot reserve %d bytes of shared memory", bytes);
}

static int check_common(int D, int Hq, int Hkv, int ldq, int ldk, int ldv) {
  if (D != 64 && D != 128) return refuse("attention: head dim %d not supported (64 or 128)", D);
  if (Hkv <= 0 || Hq % Hkv) return refuse("attention: %d query heads not a multiple of %d kv heads", Hq, Hkv);
  if (ldq % 8 || ldk % 8 || ldv % 8) return refuse("attention: token pitch must be a multiple of 8");
  return 0;
}

}  // namespace mimir

using namespace mimir;

// Fused attention forward.  Q/K/V/O are bf16; ldq/ldk/ldv/ldo are token pitches
// in elements; LSE (may be null) is [B, Hq, Tq] fp32.
MIMIR_API int mimir_attention_fwd(const void* Q, const void* K, const void* V, void* O, float* LSE, int B,
                                  int Tq, int Tk, int Hq, int Hkv, int D, int ldq, int ldk, int ldv, int ldo,
                                  int causal, int offset, float scale, cudaStream_t st) {
  if (check_common(D, Hq, Hkv, ldq, ldk, ldv) || ldo % 8) return -1;
  CUtensorMap tq, tk, tv;
  if (make_map4(&tq, Q, D, Hq, Tq, B, ldq) || make_map4(&tk, K, D, Hkv, Tk, B, ldk) ||
      make_map4(&tv, V, D, Hkv, Tk, B, ldv))
    return -1;
  AttnParams p{B, Tq, Tk, Hq, Hkv, causal, offset, scale, ldo, 0};
  dim3 grid(ceil_div(Tq, kTile), Hq, B);
  if (D == 64) {
    constexpr int SM = (1 + 2 * 3) * kChunkBytes + 1024 + 256;
    static bool cfg = false;
    if (!cfg) { if (set_smem(attn_fwd_kernel<64>, SM)) return -1; cfg = true; }
    attn_fwd_kernel<64><<<grid, kAttFwdThreads, SM, st>>>(tq, tk, tv, static_cast<__nv_bfloat16*>(O), LSE, p,
                                                       error_word_dev());
  } else {
    constexpr int SM = (1 + 2 * 2) * 2 * kChunkBytes + 1024 + 256;
    static bool cfg = false;
    if (!cfg) { if (set_smem(attn_fwd_kernel<128>, SM)) return -1; cfg = true; }
    attn_fwd_kernel<128><<<grid, kAttFwdThreads, SM, st>>>(tq, tk, tv, static_cast<__nv_bfloat16*>(O), LSE, p,
                                                        error_word_dev());
  }
  count_launch();
  return cudaGetLastError() == cudaSuccess ? 0 : refuse("attention forward launch failed");
}

// Fused attention backward: dQ [B,Tq,Hq,D] (pitch lddq), dK/dV [B,Tk,Hkv,D] (pitch lddkv).
// dsum: fp32 scratch [B, Hq, Tq].
MIMIR_API int mimir_attention_bwd(const void* Q, const void* K, const void* V, const void* O, const void* dO,
                                  const float* LSE, float* dsum, void* dQ, void* dK, void* dV, int B, int Tq,
                                  int Tk, int Hq, int Hkv, int D, int ldq, int ldk, int ldv, int ldo,
                                  int lddo, int lddq, int lddkv, int causal, int offset, float scale,
                                  cudaStream_t st) {
  if (check_common(D, Hq, Hkv, ldq, ldk, ldv) || ldo % 8 || lddo % 8 || lddq % 8 || lddkv % 8) return -1;
  CUtensorMap tq, tk, tv, tdo;
  if (make_map4(&tq, Q, D, Hq, Tq, B, ldq) || make_map4(&tk, K, D, Hkv, Tk, B, ldk) ||
      make_map4(&tv, V, D, Hkv, Tk, B, ldv) || make_map4(&tdo, dO, D, Hq, Tq, B, lddo))
    return -1;
  {
    const size_t n = static_cast<size_t>(B) * Tq * Hq * (D / 8);
    attn_dsum_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(O), static_cast<const __nv_bfloat16*>(dO), dsum, B, Tq, Hq, D, ldo,
        lddo);
  }
  AttnParams p{B, Tq, Tk, Hq, Hkv, causal, offset, scale, lddq, lddkv};
  dim3 grid_kv(ceil_div(Tk, kTile), Hkv, B), grid_q(ceil_div(Tq, kTile), Hq, B);
  auto dq = static_cast<__nv_bfloat16*>(dQ);
  auto dk = static_cast<__nv_bfloat16*>(dK);
  auto dv = static_cast<__nv_bfloat16*>(dV);
  if (D == 64) {
    constexpr int SM = (2 + 2 * 2) * kChunkBytes + 16384 + 1024 + 256;
    static bool cfg = false;
    if (!cfg) {
      if (set_smem(attn_bwd_kernel<64, 0>, SM) || set_smem(attn_bwd_kernel<64, 1>, SM)) return -1;
      cfg = true;
    }
    attn_bwd_kernel<64, 0><<<grid_kv, kAttFwdThreads, SM, st>>>(tk, tv, tq, tdo, LSE, dsum, dv, dk, p,
                                                             error_word_dev());
    attn_bwd_kernel<64, 1><<<grid_q, kAttFwdThreads, SM, st>>>(tq, tdo, tk, tv, LSE, dsum, dq, nullptr, p,
                                                            error_word_dev());
  } else {
    constexpr int SM = (2 + 2 * 2) * 2 * kChunkBytes + 16384 + 1024 + 256;
    static bool cfg = false;
    if (!cfg) {
      if (set_smem(attn_bwd_kernel<128, 0>, SM) || set_smem(attn_bwd_kernel<128, 1>, SM)) return -1;
      cfg = true;
    }
    attn_bwd_kernel<128, 0><<<grid_kv, kAttFwdThreads, SM, st>>>(tk, tv, tq, tdo, LSE, dsum, dv, dk, p,
                                                              error_word_dev());
    attn_bwd_kernel<128, 1><<<grid_q, kAttFwdThreads, SM, st>>>(tq, tdo, tk, tv, LSE, dsum, dq, nullptr, p,
                                                             error_word_dev());
  }
  count_launch(3);
  return cudaGetLastError() == cudaSuccess ? 0 : refuse("attention backward launch failed");
}
