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
// Shrinking as in LIBLINEAR: a row whose multiplier sits at a bound with a gradient beyond the previous
// pass's extremes leaves the active set; when the active set has converged the whole set is checked
// once more before stopping.
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
  long long active = n;
  double pg_max_old = INFINITY, pg_min_old = -INFINITY;
  int pass = 0;
  while (pass < max_passes) {
    ++pass;
    for (long long i = active - 1; i > 0; --i) {
      const long long j = static_cast<long long>(next(state) % static_cast<uint64_t>(i + 1));
      std::swap(order[i], order[j]);
    }
    double pg_max = -INFINITY, pg_min = INFINITY;
    for (long long k = 0; k < active; ++k) {
      const long long i = order[k];
      const float* r = x + i * f;
      double dot = 0;
      for (int j = 0; j < f; ++j) dot += w[j] * r[j];
      const double g = y[i] * dot - 1.0;
      double pg = 0;
      if (alpha[i] <= 0) {
        if (g > pg_max_old) {                 // stays at zero: out of the active set
          --active;
          std::swap(order[k], order[active]);
          --k;
          continue;
        }
        if (g < 0) pg = g;
      } else if (alpha[i] >= c) {
        if (g < pg_min_old) {
          --active;
          std::swap(order[k], order[active]);
          --k;
          continue;
        }
        if (g > 0) pg = g;
      } else {
        pg = g;
      }
      if (pg > pg_max) pg_max = pg;
      if (pg < pg_min) pg_min = pg;
      if (std::fabs(pg) > 1e-12 && qd[i] > 0) {
        double a = alpha[i] - g / qd[i];
        a = a < 0 ? 0 : (a > c ? c : a);
        const double d = (a - alpha[i]) * y[i];
        alpha[i] = a;
        if (d != 0)
          for (int j = 0; j < f; ++j) w[j] += d * r[j];
      }
    }
    if (pg_max - pg_min <= tol) {
      if (active == n) break;
      active = n;                              // converged on the active set: check every row once more
      pg_max_old = INFINITY;
      pg_min_old = -INFINITY;
      continue;
    }
    pg_max_old = pg_max <= 0 ? INFINITY : pg_max;
    pg_min_old = pg_min >= 0 ? -INFINITY : pg_min;
  }
  return pass;
}

// Sequential minimal optimization over a kernel matrix held in memory (reference: svm/solve.go, after
// libsvm): min 0.5 a'Qa + p'a with Q[s][t] = y_s y_t K[idx_s][idx_t], 0 <= a <= c, y'a = 0.  The working
// pair is the maximal violator and the partner that lowers the objective most (second-order selection).
// K is [m, m] float32 row-major, idx [l] maps variables to its rows.  alpha [l] (zero) and grad [l] (= p)
// in/out.  Returns the steps made, or -1 on bad sizes.
MIMIR_CPU_API long long mimir_cpu_svm_smo(const float* K, long long m, const int64_t* idx, const double* y, long long l, double c,
                                          double tol, long long max_iter, double* alpha, double* grad) {
  if (m <= 0 || l <= 0 || c <= 0 || max_iter < 0) return -1;
  const double tau = 1e-12;
  std::vector<double> diag(l);
  for (long long t = 0; t < l; ++t) diag[t] = K[idx[t] * m + idx[t]];
  // the maximal violator i and the extremes are found while the gradient is updated, so a step reads the
  // variables twice: once to choose j, once to update and choose the next i
  long long i = -1;
  double gmax = -INFINITY, gmin = INFINITY;
  auto scan = [&](long long t) {
    const double s = -y[t] * grad[t];
    const bool pos = y[t] > 0;
    const bool up = pos ? alpha[t] < c : alpha[t] > 0;
    const bool low = pos ? alpha[t] > 0 : alpha[t] < c;
    if (up && s > gmax) { gmax = s; i = t; }
    if (low && s < gmin) gmin = s;
  };
  for (long long t = 0; t < l; ++t) scan(t);
  long long it = 0;
  for (; it < max_iter; ++it) {
    if (i < 0 || gmax - gmin < tol) break;
    const float* Ki = K + idx[i] * m;
    long long j = -1;
    double best = INFINITY;
    const double di = diag[i];
    for (long long t = 0; t < l; ++t) {
      const double b = gmax + y[t] * grad[t];
      if (b <= 0) continue;
      const bool low = y[t] > 0 ? alpha[t] > 0 : alpha[t] < c;
      if (!low) continue;
      double q = di + diag[t] - 2.0 * Ki[idx[t]];
      if (q < tau) q = tau;
      const double gain = -(b * b) / q;
      if (gain < best) { best = gain; j = t; }
    }
    if (j < 0) break;
    const float* Kj = K + idx[j] * m;
    double q = di + diag[j] - 2.0 * Ki[idx[j]];
    if (q < tau) q = tau;
    double step = (gmax + y[j] * grad[j]) / q;
    const double room_i = y[i] > 0 ? c - alpha[i] : alpha[i];
    const double room_j = y[j] > 0 ? alpha[j] : c - alpha[j];
    if (step > room_i) step = room_i;
    if (step > room_j) step = room_j;
    alpha[i] += y[i] * step;
    alpha[j] -= y[j] * step;
    i = -1;
    gmax = -INFINITY;
    gmin = INFINITY;
    for (long long t = 0; t < l; ++t) {
      grad[t] += step * y[t] * (static_cast<double>(Ki[idx[t]]) - Kj[idx[t]]);
      scan(t);
    }
  }
  return it;
}

// Coordinate descent for the elastic net on a Gram matrix (reference: linear/fit.go):
// min 0.5 w'Gw - c'w + l1 |w|_1 + 0.5 l2 |w|^2, G [f, f] and c [f] double.  Stops once a pass moves no
// weight by more than tol.  Returns the passes made.
MIMIR_CPU_API int mimir_cpu_elastic_cd(const double* G, const double* c, int f, double l1, double l2, double tol, int max_passes,
                                       double* w) {
  if (f <= 0 || max_passes < 1) return -1;
  int pass = 0;
  for (; pass < max_passes; ++pass) {
    double moved = 0;
    for (int j = 0; j < f; ++j) {
      const double d = G[j * f + j];
      if (d <= 0) continue;
      double rho = c[j] + d * w[j];
      const double* row = G + static_cast<long long>(j) * f;
      for (int k = 0; k < f; ++k) rho -= row[k] * w[k];
      double v = std::fabs(rho) - l1;
      v = v <= 0 ? 0 : (rho > 0 ? v : -v) / (d + l2);
      const double delta = std::fabs(v - w[j]);
      if (delta > moved) moved = delta;
      w[j] = v;
    }
    if (moved <= tol) { ++pass; break; }
  }
  return pass;
}
