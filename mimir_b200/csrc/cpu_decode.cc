// One decoder layer of a Llama-family model for one new token per sequence, on the host (reference:
// llm/decode.go: the recorded CPU decode step with fused QKV and gate/up products).  Everything between the
// four products over quantized blocks (normalisations, rotary positions, the cache append, attention over
// the cache, SwiGLU, the residual sums) runs here too, so a token costs one call per layer instead of some
// forty small tensor operations: at eight threads those were more than a third of a token's time.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <mutex>
#include <vector>

#include "cpu_pool.h"

#define MIMIR_CPU_API extern "C" __attribute__((visibility("default")))

extern "C" int mimir_cpu_qgemv(int code, const void* w, int N, int K, const float* x, int B, float* y, int mode, void* scratch);

extern "C" {
// <c-abi>
struct MimirDecodeLayer {
  int32_t B, E, H, Hk, D, hidden, rope_dim, interleaved, pos, cap, mode, qkv_code, o_code, gate_up_code, down_code, pad_;
  float eps, pad2_;
  const float* attn_norm;   // [E]
  const float* ffn_norm;    // [E]
  const float* qkv_bias;    // [(H + 2 Hk) D] or null
  const float* inv_freq;    // [rope_dim / 2]
  const void* qkv;          // (H + 2 Hk) D rows of E values
  const void* o;            // E rows of H D values
  const void* gate_up;      // 2 hidden rows of E values (gate rows first)
  const void* down;         // E rows of hidden values
  float* k_cache;           // [B, Hk, cap, D] of this layer
  float* v_cache;
  float* x;                 // [B, E], updated in place
  float* scratch;           // mimir_cpu_decode_scratch(...) floats
};
// </c-abi>
}

namespace {

void rms_norm(const float* x, const float* g, float eps, int n, float* out) {
  double ss = 0;
  for (int i = 0; i < n; ++i) ss += static_cast<double>(x[i]) * x[i];
  const float r = 1.0f / std::sqrt(static_cast<float>(ss / n) + eps);
  for (int i = 0; i < n; ++i) out[i] = x[i] * r * g[i];
}

void rope(float* v, int heads, int D, int rope_dim, bool interleaved, int pos, const float* inv_freq) {
  const int half = rope_dim / 2;
  for (int i = 0; i < half; ++i) {
    const float ang = static_cast<float>(pos) * inv_freq[i];
    const float c = std::cos(ang), s = std::sin(ang);
    for (int h = 0; h < heads; ++h) {
      float* p = v + static_cast<size_t>(h) * D;
      float &a = interleaved ? p[2 * i] : p[i], &b = interleaved ? p[2 * i + 1] : p[i + half];
      const float a0 = a, b0 = b;
      a = a0 * c - b0 * s;
      b = a0 * s + b0 * c;
    }
  }
}

}  // namespace

// floats of scratch a layer call needs
MIMIR_CPU_API long long mimir_cpu_decode_scratch(int B, int E, int H, int Hk, int D, int hidden, int cap) {
  const long long nqkv = static_cast<long long>(H + 2 * Hk) * D;
  return static_cast<long long>(B) * (2LL * E + nqkv + static_cast<long long>(H) * D + 3LL * hidden) + static_cast<long long>(B) * H * cap + 64;
}

// Returns 0, or -1 for a bad argument (nothing is written then).
MIMIR_CPU_API int mimir_cpu_decode_layer(const MimirDecodeLayer* a) {
  const int B = a->B, E = a->E, H = a->H, Hk = a->Hk, D = a->D, hidden = a->hidden, pos = a->pos, cap = a->cap;
  if (B < 1 || B > 8 || E < 1 || H < 1 || Hk < 1 || H % Hk || D < 1 || hidden < 1 || pos < 0 || pos >= cap || a->rope_dim < 0 ||
      a->rope_dim > D || (a->rope_dim & 1))
    return -1;
  const int nqkv = (H + 2 * Hk) * D, HD = H * D;
  float* h = a->scratch;                                  // [B, E]
  float* qkv = h + static_cast<size_t>(B) * E;            // [B, nqkv]
  float* att = qkv + static_cast<size_t>(B) * nqkv;       // [B, H D]
  float* gu = att + static_cast<size_t>(B) * HD;          // [B, 2 hidden]
  float* act = gu + static_cast<size_t>(B) * 2 * hidden;  // [B, hidden]
  float* tmp = act + static_cast<size_t>(B) * hidden;     // [B, E]
  float* scores = tmp + static_cast<size_t>(B) * E;       // [B H, cap]
  for (int b = 0; b < B; ++b) rms_norm(a->x + static_cast<size_t>(b) * E, a->attn_norm, a->eps, E, h + static_cast<size_t>(b) * E);
  if (mimir_cpu_qgemv(a->qkv_code, a->qkv, nqkv, E, h, B, qkv, a->mode, nullptr) != 0) return -1;
  const size_t head_stride = static_cast<size_t>(cap) * D, seq_stride = static_cast<size_t>(Hk) * head_stride;
  for (int b = 0; b < B; ++b) {
    float* row = qkv + static_cast<size_t>(b) * nqkv;
    if (a->qkv_bias)
      for (int i = 0; i < nqkv; ++i) row[i] += a->qkv_bias[i];
    rope(row, H, D, a->rope_dim, a->interleaved != 0, pos, a->inv_freq);
    rope(row + HD, Hk, D, a->rope_dim, a->interleaved != 0, pos, a->inv_freq);
    for (int hk = 0; hk < Hk; ++hk) {
      memcpy(a->k_cache + b * seq_stride + hk * head_stride + static_cast<size_t>(pos) * D, row + HD + hk * D, sizeof(float) * D);
      memcpy(a->v_cache + b * seq_stride + hk * head_stride + static_cast<size_t>(pos) * D, row + HD + Hk * D + hk * D, sizeof(float) * D);
    }
  }
  // attention of the new token over the cache: one (sequence, head) per task
  const int n = pos + 1, group = H / Hk;
  const float scale = 1.0f / std::sqrt(static_cast<float>(D));
  auto head = [&](long long t) {
    const int b = static_cast<int>(t / H), hq = static_cast<int>(t % H), hk = hq / group;
    const float* q = qkv + static_cast<size_t>(b) * nqkv + static_cast<size_t>(hq) * D;
    const float* K = a->k_cache + b * seq_stride + hk * head_stride;
    const float* V = a->v_cache + b * seq_stride + hk * head_stride;
    float* s = scores + static_cast<size_t>(t) * cap;
    float top = -INFINITY;
    for (int j = 0; j < n; ++j) {
      const float* kj = K + static_cast<size_t>(j) * D;
      float d = 0;
      for (int i = 0; i < D; ++i) d += q[i] * kj[i];
      s[j] = d * scale;
      if (s[j] > top) top = s[j];
    }
    float sum = 0;
    for (int j = 0; j < n; ++j) { s[j] = std::exp(s[j] - top); sum += s[j]; }
    float* o = att + static_cast<size_t>(b) * HD + static_cast<size_t>(hq) * D;
    for (int i = 0; i < D; ++i) o[i] = 0;
    const float inv = 1.0f / sum;
    for (int j = 0; j < n; ++j) {
      const float p = s[j] * inv;
      const float* vj = V + static_cast<size_t>(j) * D;
      for (int i = 0; i < D; ++i) o[i] += p * vj[i];
    }
  };
  const long long tasks = static_cast<long long>(B) * H;
  if (static_cast<long long>(n) * D * tasks < (1 << 16)) {
    for (long long t = 0; t < tasks; ++t) head(t);
  } else {
    std::lock_guard<std::mutex> lk(mimir_cpu::pool_mutex());
    std::atomic<long long> next{0};
    mimir_cpu::pool().run_shared([&](int, int) {
      for (long long t = next.fetch_add(1); t < tasks; t = next.fetch_add(1)) head(t);
    });
  }
  if (mimir_cpu_qgemv(a->o_code, a->o, E, HD, att, B, tmp, a->mode, nullptr) != 0) return -1;
  for (size_t i = 0; i < static_cast<size_t>(B) * E; ++i) a->x[i] += tmp[i];
  for (int b = 0; b < B; ++b) rms_norm(a->x + static_cast<size_t>(b) * E, a->ffn_norm, a->eps, E, h + static_cast<size_t>(b) * E);
  if (mimir_cpu_qgemv(a->gate_up_code, a->gate_up, 2 * hidden, E, h, B, gu, a->mode, nullptr) != 0) return -1;
  for (int b = 0; b < B; ++b) {
    const float* g = gu + static_cast<size_t>(b) * 2 * hidden;
    const float* u = g + hidden;
    float* o = act + static_cast<size_t>(b) * hidden;
    for (int i = 0; i < hidden; ++i) o[i] = g[i] / (1.0f + std::exp(-g[i])) * u[i];
  }
  if (mimir_cpu_qgemv(a->down_code, a->down, E, hidden, act, B, tmp, a->mode, nullptr) != 0) return -1;
  for (size_t i = 0; i < static_cast<size_t>(B) * E; ++i) a->x[i] += tmp[i];
  return 0;
}
