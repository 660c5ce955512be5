// Dual coordinate descent for the linear support vector classifier (reference: svm/solve.go, after
// LIBLINEAR, Hsieh et al. 2008): min_a 0.5 |sum_i a_i y_i x_i|^2 - sum_i a_i, 0 <= a_i <= C, with the
// hinge loss.  One pass visits the rows in a seeded random order; rows whose multiplier sits at a bound
// with a gradient that keeps it there are skipped ("shrinking" without removing them).  No kernel
// matrix is needed, so the cost of a pass is one read of the table.
#include <cmath>
#include <cstdint>
#include <vector>

#define MIMIR_CPU_API extern "C" __attribute__((visibility("default")))

namespace {
inline uint64_t next(uint64_t& s) {          // xorshift64*
  s ^= s >> 12;
  s ^= s << 25;
  s ^= s >> 27;
  return s * 0x2545F4914F6CDD1DULL;
}
}  // namespace

// x [n, f] row-major float32 (the caller appends a constant 1 for the bias), y [n] in {-1, +1},
// alpha [n] and w [f] in/out (zero to start).  Returns the number of passes made, or -1 on bad sizes.
MIMIR_CPU_API int mimir_cpu_svm_dcd(const float* x, const float* y, long long n, int f, double c, double tol, int max_passes,
                                    uint64_t seed, double* alpha, double* w) {
  if (n <= 0 || f <= 0 || c <= 0 || max_passes < 1) return -1;
  std::vector<double> qd(n);
  for (long long i = 0; i < n; ++i) {
    const float* r = x + i * f;
    double s = 0;
    for (int j = 0; j < f; ++j) s += static_cast<double>(r[j]) * r[j];
    qd[i] = s;
  }
  std::vector<long long> order(n);
  for (long long i = 0; i < n; ++i) order[i] = i;
  uint64_t state = seed * 0x9E3779B97F4A7C15ULL + 0x1234567ULL;
  if (state == 0) state = 1;
  int pass = 0;
  for (; pass < max_passes; ++pass) {
    for (long long i = n - 1; i > 0; --i) {
      const long long j = static_cast<long long>(next(state) % static_cast<uint64_t>(i + 1));
      std::swap(order[i], order[j]);
    }
    double worst = 0;          // the largest projected gradient of the pass
    for (long long k = 0; k < n; ++k) {
      const long long i = order[k];
      if (qd[i] <= 0) continue;
      const float* r = x + i * f;
      double dot = 0;
      for (int j = 0; j < f; ++j) dot += w[j] * r[j];
      const double g = y[i] * dot - 1.0;
      double pg = g;
      if (alpha[i] <= 0) pg = g < 0 ? g : 0;
      else if (alpha[i] >= c) pg = g > 0 ? g : 0;
      if (std::fabs(pg) > worst) worst = std::fabs(pg);
      if (pg == 0) continue;
      double a = alpha[i] - g / qd[i];
      a = a < 0 ? 0 : (a > c ? c : a);
      const double d = (a - alpha[i]) * y[i];
      alpha[i] = a;
      if (d != 0)
        for (int j = 0; j < f; ++j) w[j] += d * r[j];
    }
    if (worst <= tol) { ++pass; break; }
  }
  return pass;
}
