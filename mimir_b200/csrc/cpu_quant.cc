// CPU kernels for block-quantized weights: y[b][n] = sum_k W[n][k] x[b][k] with W read in its ggml
// block encoding (Q8_0, Q4_0, Q4_K, Q6_K), for the few-row products of decoding on the host
// (reference: backend/cpu/quant.go, llm/decode.go:79-160: the reference's CPU decode step keeps the
// weights quantized and multiplies block by block).
//
// Two paths, chosen once at run time from the CPU's features:
//   * int8: the activation rows are rounded to int8 (one float scale per 32 values for Q8_0 / Q4_0
//     weights, one per 256 for the K-quants, whose super-blocks are then summed in integers: dot
//     products times their 6-bit or int8 sub-block scales), and every weight block is multiplied with
//     its activation block by 256-bit VNNI dot products (vpdpbusd: unsigned weight codes x signed
//     activations), the offsets (-8, -32, the K-quant minima) folded in through the block sums;
//   * exact: float activations, weights decoded value by value (any x86-64).  It computes exactly
//     x . dequant(W) and is what the int8 path is tested against.
// Rows of W are split over a small pool of worker threads that lives as long as the library.
// Plain C ABI; compiled by the host compiler (no CUDA in this file).
#include "cpu_pool.h"


#include <atomic>
#include <condition_variable>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <mutex>
#include <new>
#include <thread>
#include <vector>

#define MIMIR_CPU_API extern "C" __attribute__((visibility("default")))

namespace {

enum Code { Q8_0 = 64, Q4_0 = 65, Q4_K = 66, Q6_K = 67 };

inline float half_to_float(uint16_t h) {
  const uint32_t sign = static_cast<uint32_t>(h & 0x8000) << 16;
  uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ff, bits;
  if (exp == 0) {
    if (man == 0) bits = sign;
    else {
      exp = 127 - 15 + 1;
      while (!(man & 0x400)) { man <<= 1; --exp; }
      bits = sign | (exp << 23) | ((man & 0x3ff) << 13);
    }
  } else if (exp == 31) bits = sign | 0x7f800000u | (man << 13);
  else bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
  float f;
  memcpy(&f, &bits, 4);
  return f;
}
inline float ld_half(const uint8_t* p) {
  uint16_t h;
  memcpy(&h, p, 2);
  return half_to_float(h);
}

// bytes per row of K values
inline size_t row_bytes(int code, int K) {
  switch (code) {
    case Q8_0: return static_cast<size_t>(K / 32) * 34;
    case Q4_0: return static_cast<size_t>(K / 32) * 18;
    case Q4_K: return static_cast<size_t>(K / 256) * 144;
    case Q6_K: return static_cast<size_t>(K / 256) * 210;
  }
  return 0;
}

// 6-bit scale and minimum j (0..7) of a Q4_K super-block (12 packed bytes)
inline void q4k_scale_min(int j, const uint8_t* q, int& sc, int& mn) {
  if (j < 4) { sc = q[j] & 63; mn = q[j + 4] & 63; }
  else { sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4); mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
}

// ---------------------------------------------------------------------------
// exact path: decode one row into floats block by block and multiply
// ---------------------------------------------------------------------------
void decode_block(int code, const uint8_t* b, float* out) {   // 32 values (Q8_0 / Q4_0) or 256 (K-quants)
  if (code == Q8_0) {
    const float d = ld_half(b);
    const int8_t* q = reinterpret_cast<const int8_t*>(b + 2);
    for (int i = 0; i < 32; ++i) out[i] = d * q[i];
  } else if (code == Q4_0) {
    const float d = ld_half(b);
    for (int i = 0; i < 16; ++i) {
      out[i] = d * ((b[2 + i] & 0xF) - 8);
      out[16 + i] = d * ((b[2 + i] >> 4) - 8);
    }
  } else if (code == Q4_K) {
    const float d = ld_half(b), dmin = ld_half(b + 2);
    const uint8_t* qs = b + 16;
    for (int p = 0; p < 4; ++p) {
      int s1, m1, s2, m2;
      q4k_scale_min(2 * p, b + 4, s1, m1);
      q4k_scale_min(2 * p + 1, b + 4, s2, m2);
      for (int i = 0; i < 32; ++i) {
        out[64 * p + i] = d * s1 * (qs[32 * p + i] & 0xF) - dmin * m1;
        out[64 * p + 32 + i] = d * s2 * (qs[32 * p + i] >> 4) - dmin * m2;
      }
    }
  } else {
    const uint8_t *ql = b, *qh = b + 128;
    const int8_t* sc = reinterpret_cast<const int8_t*>(b + 192);
    const float d = ld_half(b + 208);
    for (int h = 0; h < 2; ++h) {
      const uint8_t *l = ql + 64 * h, *hq = qh + 32 * h;
      const int8_t* s = sc + 8 * h;
      for (int i = 0; i < 32; ++i) {
        const int g = i / 16;
        const int q1 = ((l[i] & 0xF) | (((hq[i] >> 0) & 3) << 4)) - 32;
        const int q2 = ((l[32 + i] & 0xF) | (((hq[i] >> 2) & 3) << 4)) - 32;
        const int q3 = ((l[i] >> 4) | (((hq[i] >> 4) & 3) << 4)) - 32;
        const int q4 = ((l[32 + i] >> 4) | (((hq[i] >> 6) & 3) << 4)) - 32;
        out[128 * h + i] = d * s[g] * q1;
        out[128 * h + 32 + i] = d * s[g + 2] * q2;
        out[128 * h + 64 + i] = d * s[g + 4] * q3;
        out[128 * h + 96 + i] = d * s[g + 6] * q4;
      }
    }
  }
}

void rows_exact(int code, const uint8_t* w, int K, const float* x, int B, float* y, int N, int n0, int n1) {
  const int vals = (code == Q8_0 || code == Q4_0) ? 32 : 256;
  const size_t bb = code == Q8_0 ? 34 : code == Q4_0 ? 18 : code == Q4_K ? 144 : 210;
  const size_t rb = row_bytes(code, K);
  float tmp[256];
  for (int n = n0; n < n1; ++n) {
    double acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    const uint8_t* row = w + static_cast<size_t>(n) * rb;
    for (int k0 = 0; k0 < K; k0 += vals) {
      decode_block(code, row + static_cast<size_t>(k0 / vals) * bb, tmp);
      for (int b = 0; b < B; ++b) {
        const float* xr = x + static_cast<size_t>(b) * K + k0;
        float s = 0.f;
        for (int i = 0; i < vals; ++i) s += tmp[i] * xr[i];
        acc[b] += s;
      }
    }
    for (int b = 0; b < B; ++b) y[static_cast<size_t>(b) * N + n] = static_cast<float>(acc[b]);
  }
}

// ---------------------------------------------------------------------------
// int8 path
// ---------------------------------------------------------------------------
struct ActQ {            // one activation row rounded to int8
  const int8_t* q;       // K values
  const float* d;        // K / 32 scales (one per 32 values for Q8_0 / Q4_0 weights; the K-quants share
                         // one per 256 values, repeated, so that a super-block is summed in integers)
  const float* ds;       // K / 32: scale x sum of the block's values
  const int32_t* isum;   // K / 32: sum of the block's int8 values
  const int32_t* isum16; // K / 16: sum of each half block (Q6_K has a scale per 16 values)
};

#define VNNI __attribute__((target("avx2,fma,avx512f,avx512bw,avx512vl,avx512vnni")))

VNNI inline float hsum8(__m256 v) {
  __m128 s = _mm_add_ps(_mm256_castps256_ps128(v), _mm256_extractf128_ps(v, 1));
  s = _mm_add_ps(s, _mm_movehl_ps(s, s));
  s = _mm_add_ss(s, _mm_movehdup_ps(s));
  return _mm_cvtss_f32(s);
}

template <int B>
VNNI void rows_int8_t(int code, const uint8_t* w, int K, const ActQ* act, float* y, int N, int n0, int n1) {
  const size_t rb = row_bytes(code, K);
  const __m256i low4 = _mm256_set1_epi8(0x0F);
  for (int n = n0; n < n1; ++n) {
    const uint8_t* row = w + static_cast<size_t>(n) * rb;
    __m256 acc[B];
    float off[B];
    _Pragma("GCC unroll 8") for (int b = 0; b < B; ++b) { acc[b] = _mm256_setzero_ps(); off[b] = 0.f; }
    if (code == Q8_0) {
      for (int blk = 0; blk < K / 32; ++blk) {
        const uint8_t* p = row + static_cast<size_t>(blk) * 34;
        const float dw = ld_half(p);
        const __m256i qw = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(p + 2));
        const __m256i aw = _mm256_abs_epi8(qw);                   // unsigned operand: |w|
        _Pragma("GCC unroll 8") for (int b = 0; b < B; ++b) {
          const __m256i qa = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(act[b].q + blk * 32));
          const __m256i sa = _mm256_sign_epi8(qa, qw);            // signed operand: a x sign(w)
          const __m256i dot = _mm256_dpbusd_epi32(_mm256_setzero_si256(), aw, sa);
          acc[b] = _mm256_fmadd_ps(_mm256_cvtepi32_ps(dot), _mm256_set1_ps(dw * act[b].d[blk]), acc[b]);
        }
      }
    } else if (code == Q4_0) {
      for (int blk = 0; blk < K / 32; ++blk) {
        const uint8_t* p = row + static_cast<size_t>(blk) * 18;
        const float dw = ld_half(p);
        const __m128i raw = _mm_loadu_si128(reinterpret_cast<const __m128i*>(p + 2));
        // values 0..15 are the low nibbles, 16..31 the high nibbles
        const __m256i nib = _mm256_and_si256(_mm256_set_m128i(_mm_srli_epi16(raw, 4), raw), low4);
        _Pragma("GCC unroll 8") for (int b = 0; b < B; ++b) {
          const __m256i qa = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(act[b].q + blk * 32));
          const __m256i dot = _mm256_dpbusd_epi32(_mm256_setzero_si256(), nib, qa);
          acc[b] = _mm256_fmadd_ps(_mm256_cvtepi32_ps(dot), _mm256_set1_ps(dw * act[b].d[blk]), acc[b]);
          off[b] += dw * 8.f * act[b].ds[blk];                     // codes carry an offset of 8
        }
      }
    } else if (code == Q4_K) {
      // a super-block is summed in integers: dot products x 6-bit scales, one float multiply at its end
      for (int sb = 0; sb < K / 256; ++sb) {
        const uint8_t* p = row + static_cast<size_t>(sb) * 144;
        const float d = ld_half(p), dmin = ld_half(p + 2);
        int sc[8], mn[8];
        {
          const uint8_t* q = p + 4;
          for (int j = 0; j < 4; ++j) {
            sc[j] = q[j] & 63;
            mn[j] = q[j + 4] & 63;
            sc[j + 4] = (q[j + 8] & 0xF) | ((q[j] >> 6) << 4);
            mn[j + 4] = (q[j + 8] >> 4) | ((q[j + 4] >> 6) << 4);
          }
        }
        __m256i acci[B];
        _Pragma("GCC unroll 8") for (int b = 0; b < B; ++b) acci[b] = _mm256_setzero_si256();
        const int b0 = sb * 8;
        for (int pr = 0; pr < 4; ++pr) {
          const __m256i raw = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(p + 16 + 32 * pr));
          const __m256i lo = _mm256_and_si256(raw, low4);
          const __m256i hi = _mm256_and_si256(_mm256_srli_epi16(raw, 4), low4);
          const __m256i s0 = _mm256_set1_epi32(sc[2 * pr]), s1 = _mm256_set1_epi32(sc[2 * pr + 1]);
          _Pragma("GCC unroll 8") for (int b = 0; b < B; ++b) {
            const int8_t* qa = act[b].q + (b0 + 2 * pr) * 32;
            const __m256i d0 = _mm256_dpbusd_epi32(_mm256_setzero_si256(), lo, _mm256_loadu_si256(reinterpret_cast<const __m256i*>(qa)));
            const __m256i d1 = _mm256_dpbusd_epi32(_mm256_setzero_si256(), hi, _mm256_loadu_si256(reinterpret_cast<const __m256i*>(qa + 32)));
            acci[b] = _mm256_add_epi32(acci[b], _mm256_add_epi32(_mm256_mullo_epi32(d0, s0), _mm256_mullo_epi32(d1, s1)));
          }
        }
        _Pragma("GCC unroll 8") for (int b = 0; b < B; ++b) {
          const float da = act[b].d[b0];
          acc[b] = _mm256_fmadd_ps(_mm256_cvtepi32_ps(acci[b]), _mm256_set1_ps(d * da), acc[b]);
          int ms = 0;
          for (int j = 0; j < 8; ++j) ms += mn[j] * act[b].isum[b0 + j];
          off[b] += dmin * da * static_cast<float>(ms);
        }
      }
    } else {  // Q6_K: 6-bit codes with an offset of 32 and an int8 scale per 16 values
      const __m256i two = _mm256_set1_epi8(3);
      for (int sb = 0; sb < K / 256; ++sb) {
        const uint8_t* p = row + static_cast<size_t>(sb) * 210;
        const int8_t* sc = reinterpret_cast<const int8_t*>(p + 192);
        const float d = ld_half(p + 208);
        __m256i acci[B];
        int ioff[B];
        _Pragma("GCC unroll 8") for (int b = 0; b < B; ++b) { acci[b] = _mm256_setzero_si256(); ioff[b] = 0; }
        for (int h = 0; h < 2; ++h) {
          const __m256i l0 = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(p + 64 * h));
          const __m256i l1 = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(p + 64 * h + 32));
          const __m256i hq = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(p + 128 + 32 * h));
          __m256i q[4];
          q[0] = _mm256_or_si256(_mm256_and_si256(l0, low4), _mm256_slli_epi16(_mm256_and_si256(hq, two), 4));
          q[1] = _mm256_or_si256(_mm256_and_si256(l1, low4),
                                 _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(hq, 2), two), 4));
          q[2] = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(l0, 4), low4),
                                 _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(hq, 4), two), 4));
          q[3] = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(l1, 4), low4),
                                 _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(hq, 6), two), 4));
          for (int g = 0; g < 4; ++g) {
            const int ab = sb * 8 + h * 4 + g;                     // activation block of these 32 values
            const int sa = sc[8 * h + 2 * g], sb2 = sc[8 * h + 2 * g + 1];   // a scale per 16 values
            const __m256i scale = _mm256_set_epi32(sb2, sb2, sb2, sb2, sa, sa, sa, sa);
            _Pragma("GCC unroll 8") for (int b = 0; b < B; ++b) {
              const __m256i qa = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(act[b].q + ab * 32));
              const __m256i dot = _mm256_dpbusd_epi32(_mm256_setzero_si256(), q[g], qa);
              acci[b] = _mm256_add_epi32(acci[b], _mm256_mullo_epi32(dot, scale));
              ioff[b] += sa * act[b].isum16[2 * ab] + sb2 * act[b].isum16[2 * ab + 1];   // codes carry an offset of 32
            }
          }
        }
        _Pragma("GCC unroll 8") for (int b = 0; b < B; ++b) {
          const float f = d * act[b].d[sb * 8];
          acc[b] = _mm256_fmadd_ps(_mm256_cvtepi32_ps(acci[b]), _mm256_set1_ps(f), acc[b]);
          off[b] += 32.f * f * static_cast<float>(ioff[b]);
        }
      }
    }
    _Pragma("GCC unroll 8") for (int b = 0; b < B; ++b) y[static_cast<size_t>(b) * N + n] = hsum8(acc[b]) - off[b];
  }
}

VNNI void rows_int8(int code, const uint8_t* w, int K, const ActQ* act, int B, float* y, int N, int n0, int n1) {
  // the row count is a template argument so that the accumulators of every row stay in registers
  switch (B) {
    case 1: rows_int8_t<1>(code, w, K, act, y, N, n0, n1); break;
    case 2: rows_int8_t<2>(code, w, K, act, y, N, n0, n1); break;
    case 3: rows_int8_t<3>(code, w, K, act, y, N, n0, n1); break;
    case 4: rows_int8_t<4>(code, w, K, act, y, N, n0, n1); break;
    case 5: rows_int8_t<5>(code, w, K, act, y, N, n0, n1); break;
    case 6: rows_int8_t<6>(code, w, K, act, y, N, n0, n1); break;
    case 7: rows_int8_t<7>(code, w, K, act, y, N, n0, n1); break;
    default: rows_int8_t<8>(code, w, K, act, y, N, n0, n1); break;
  }
}

// rounds one row of K floats to 32-value blocks
// group: values sharing one scale (32, or 256 for the K-quants)
void quantize_row(const float* x, int K, int group, int8_t* q, float* d, float* ds, int32_t* isum, int32_t* isum16) {
  for (int g0 = 0; g0 < K; g0 += group) {
    float amax = 0.f;
    for (int i = 0; i < group; ++i) amax = std::fmax(amax, std::fabs(x[g0 + i]));
    const float scale = amax / 127.f, inv = scale > 0.f ? 1.f / scale : 0.f;
    for (int blk = g0 / 32; blk < (g0 + group) / 32; ++blk) {
      const float* xb = x + blk * 32;
      int s0 = 0, s1 = 0;
      for (int i = 0; i < 32; ++i) {
        const int v = static_cast<int>(std::nearbyint(xb[i] * inv));
        q[blk * 32 + i] = static_cast<int8_t>(v);
        (i < 16 ? s0 : s1) += v;
      }
      d[blk] = scale;
      ds[blk] = scale * static_cast<float>(s0 + s1);
      isum[blk] = s0 + s1;
      isum16[2 * blk] = s0;
      isum16[2 * blk + 1] = s1;
    }
  }
}

// ---------------------------------------------------------------------------
// worker pool
// ---------------------------------------------------------------------------
}  // namespace

namespace mimir_cpu {

static std::mutex g_pool_mutex;
static Pool* g_pool = nullptr;
static int g_threads = 0;

// after fork() the child has none of the worker threads: it starts a pool of its own on first use
static void forget_pool_in_child() { g_pool = nullptr; new (&g_pool_mutex) std::mutex(); }

Pool& pool() {
  static const bool hooked = (pthread_atfork(nullptr, nullptr, forget_pool_in_child), true);
  (void)hooked;
  if (!g_pool) {
    int n = g_threads > 0 ? g_threads : static_cast<int>(std::thread::hardware_concurrency());
    if (n < 1) n = 1;
    if (n > 64) n = 64;
    g_pool = new Pool(n);
  }
  return *g_pool;
}

std::mutex& pool_mutex() { return g_pool_mutex; }

int set_threads(int n) {
  std::lock_guard<std::mutex> lk(g_pool_mutex);
  const int old = g_threads;
  g_threads = n < 0 ? 0 : n;
  if (g_pool) { delete g_pool; g_pool = nullptr; }
  return old;
}

}  // namespace mimir_cpu

namespace {

using mimir_cpu::pool;

bool has_vnni() {
  static const bool ok = __builtin_cpu_supports("avx512vnni") && __builtin_cpu_supports("avx512vl") &&
                         __builtin_cpu_supports("avx512bw") && __builtin_cpu_supports("avx2");
  return ok;
}

}  // namespace

// 1 when the int8 path (AVX-512 VNNI) is available on this CPU
MIMIR_CPU_API int mimir_cpu_qgemv_has_int8() { return has_vnni() ? 1 : 0; }

// Number of threads of the next products (0 = one per hardware thread).  Returns the previous setting.
MIMIR_CPU_API int mimir_cpu_set_threads(int n) { return mimir_cpu::set_threads(n); }

// y [B][N] (fp32) = x [B][K] (fp32) . W^T, W = N rows of K values in ggml blocks of `code`.
// mode 0: exact; 1: int8 activations; -1: int8 when the CPU has it.  scratch: B * (K + 5 * K / 32 * 4 + 64) bytes
// or null (allocated per call).  Returns 0, or -1 for a bad argument.
MIMIR_CPU_API int mimir_cpu_qgemv(int code, const void* w, int N, int K, const float* x, int B, float* y, int mode,
                                  void* scratch) {
  if (code < Q8_0 || code > Q6_K || N < 0 || B < 1 || B > 8) return -1;
  const int vals = (code == Q8_0 || code == Q4_0) ? 32 : 256;
  if (K <= 0 || K % vals) return -1;
  const bool int8 = mode == 1 || (mode == -1 && has_vnni());
  if (int8 && !has_vnni()) return -1;
  std::lock_guard<std::mutex> lk(mimir_cpu::pool_mutex());
  mimir_cpu::Pool& p = pool();
  const uint8_t* wb = static_cast<const uint8_t*>(w);
  // rows are handed out in chunks from a shared counter, so a thread that is held up (a busy core, a
  // hyper-thread sibling) takes fewer chunks instead of holding everyone back
  const int chunk = N >= 4096 ? 64 : N >= 512 ? 32 : 8;
  std::atomic<int> next{0};
  if (!int8) {
    p.run([&](int, int) {
      for (int n0 = next.fetch_add(chunk); n0 < N; n0 = next.fetch_add(chunk))
        rows_exact(code, wb, K, x, B, y, N, n0, n0 + chunk < N ? n0 + chunk : N);
    });
    return 0;
  }
  const int nb = K / 32;
  const size_t per_row = static_cast<size_t>(K) + static_cast<size_t>(nb) * 5 * 4 + 64;
  std::vector<uint8_t> own;
  uint8_t* s = static_cast<uint8_t*>(scratch);
  if (!s) { own.resize(per_row * B); s = own.data(); }
  ActQ act[8];
  for (int b = 0; b < B; ++b) {
    uint8_t* base = s + per_row * b;
    int8_t* q = reinterpret_cast<int8_t*>(base);
    float* f = reinterpret_cast<float*>(base + ((static_cast<size_t>(K) + 63) / 64) * 64);
    int32_t* is = reinterpret_cast<int32_t*>(f + 2 * nb);
    act[b] = ActQ{q, f, f + nb, is, is + nb};
    quantize_row(x + static_cast<size_t>(b) * K, K, vals == 256 ? 256 : 32, q, f, f + nb, is, is + nb);
  }
  p.run([&](int, int) {
    for (int n0 = next.fetch_add(chunk); n0 < N; n0 = next.fetch_add(chunk))
      rows_int8(code, wb, K, act, B, y, N, n0, n0 + chunk < N ? n0 + chunk : N);
  });
  return 0;
}

// out [N][K] (bfloat16, round to nearest even) = the values of W, N rows of K values in ggml blocks of `code`.
// For prompts: many activation rows amortise one expansion of the matrix, and the product then runs as a
// bfloat16 matrix product (on the matrix units where the CPU has them).  Returns 0, or -1 for a bad argument.
MIMIR_CPU_API int mimir_cpu_dequant_bf16(int code, const void* w, int N, int K, uint16_t* out) {
  if (code < Q8_0 || code > Q6_K || N < 0) return -1;
  const int vals = (code == Q8_0 || code == Q4_0) ? 32 : 256;
  if (K <= 0 || K % vals) return -1;
  const size_t bb = code == Q8_0 ? 34 : code == Q4_0 ? 18 : code == Q4_K ? 144 : 210;
  const size_t rb = row_bytes(code, K);
  const uint8_t* wb = static_cast<const uint8_t*>(w);
  std::lock_guard<std::mutex> lk(mimir_cpu::pool_mutex());
  mimir_cpu::Pool& p = pool();
  const int chunk = 16;
  std::atomic<int> next{0};
  p.run([&](int, int) {
    float tmp[256];
    for (int n0 = next.fetch_add(chunk); n0 < N; n0 = next.fetch_add(chunk)) {
      const int n1 = n0 + chunk < N ? n0 + chunk : N;
      for (int n = n0; n < n1; ++n) {
        const uint8_t* row = wb + static_cast<size_t>(n) * rb;
        uint16_t* o = out + static_cast<size_t>(n) * K;
        for (int k0 = 0; k0 < K; k0 += vals) {
          decode_block(code, row + static_cast<size_t>(k0 / vals) * bb, tmp);
          for (int i = 0; i < vals; ++i) {
            uint32_t u;
            memcpy(&u, &tmp[i], 4);
            u += 0x7FFFu + ((u >> 16) & 1u);          // round to nearest, ties to even (the values are finite)
            o[k0 + i] = static_cast<uint16_t>(u >> 16);
          }
        }
      }
    }
  });
  return 0;
}
