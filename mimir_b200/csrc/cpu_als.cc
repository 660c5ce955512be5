// One side of alternating least squares (reference: recommend/als.go): every row of A is set to the ridge
// solution against the fixed factors B of the events it has.  The normal equations of a row are built from its
// own events (k x k per row, on the worker that solves it) instead of one k x k block per EVENT in memory.
#include <atomic>
#include <cmath>
#include <cstdint>
#include <mutex>
#include <vector>

#include "cpu_pool.h"

#define MIMIR_CPU_API extern "C" __attribute__((visibility("default")))

// A: double [rows][k], written.  B: double [.][k].  start: int64 [rows + 1], the events of row r are
// start[r] .. start[r + 1]; col [events]: the row of B each event names; w [events]: the weight of its outer
// product; t [events]: the weight of its row of B on the right-hand side.  base: double [k][k] added to every
// row's matrix (B'B for implicit feedback) or null; l2 is added to the diagonal.  A row without events becomes
// zero.  Returns 0, or -1 for bad arguments; a matrix that is not positive definite is solved with a larger
// diagonal (its own trace * 1e-12, doubled until it is).
MIMIR_CPU_API int mimir_cpu_als_side(double* A, long long rows, const double* B, long long b_rows, int k, const int64_t* start,
                                     const int64_t* col, const double* w, const double* t, const double* base, double l2) {
  if (rows < 0 || k < 1 || k > 1024 || b_rows < 1 || l2 < 0) return -1;
  for (long long e = start[0]; e < start[rows]; ++e)
    if (col[e] < 0 || col[e] >= b_rows) return -1;
  std::lock_guard<std::mutex> lk(mimir_cpu::pool_mutex());
  mimir_cpu::Pool& pool = mimir_cpu::pool();
  const long long chunk = 16, chunks = (rows + chunk - 1) / chunk;
  std::atomic<long long> next{0};
  auto work = [&](int, int) {
    std::vector<double> G(static_cast<size_t>(k) * k), L(static_cast<size_t>(k) * k), rhs(k), y(k);
    for (long long c = next.fetch_add(1); c < chunks; c = next.fetch_add(1)) {
      for (long long r = c * chunk; r < rows && r < (c + 1) * chunk; ++r) {
        double* out = A + static_cast<size_t>(r) * k;
        if (start[r + 1] == start[r]) {
          for (int i = 0; i < k; ++i) out[i] = 0;
          continue;
        }
        for (int i = 0; i < k; ++i) {
          rhs[i] = 0;
          for (int j = 0; j < k; ++j) G[static_cast<size_t>(i) * k + j] = base ? base[static_cast<size_t>(i) * k + j] : 0.0;
          G[static_cast<size_t>(i) * k + i] += l2;
        }
        for (long long e = start[r]; e < start[r + 1]; ++e) {
          const double* b = B + static_cast<size_t>(col[e]) * k;
          const double we = w[e], te = t[e];
          for (int i = 0; i < k; ++i) {
            const double s = we * b[i];
            double* g = G.data() + static_cast<size_t>(i) * k;
            for (int j = 0; j <= i; ++j) g[j] += s * b[j];          // the lower triangle is enough
            rhs[i] += te * b[i];
          }
        }
        // Cholesky G = L L', then two triangular solves
        double bump = 0;
        for (int attempt = 0; attempt < 60; ++attempt) {
          bool ok = true;
          for (int i = 0; i < k && ok; ++i) {
            for (int j = 0; j <= i; ++j) {
              double s = G[static_cast<size_t>(i) * k + j] + (i == j ? bump : 0.0);
              for (int q = 0; q < j; ++q) s -= L[static_cast<size_t>(i) * k + q] * L[static_cast<size_t>(j) * k + q];
              if (i == j) {
                if (!(s > 0)) { ok = false; break; }
                L[static_cast<size_t>(i) * k + i] = std::sqrt(s);
              } else {
                L[static_cast<size_t>(i) * k + j] = s / L[static_cast<size_t>(j) * k + j];
              }
            }
          }
          if (ok) break;
          double trace = 0;
          for (int i = 0; i < k; ++i) trace += std::fabs(G[static_cast<size_t>(i) * k + i]);
          bump = bump > 0 ? bump * 2 : (trace > 0 ? trace : 1.0) * 1e-12;
        }
        for (int i = 0; i < k; ++i) {
          double s = rhs[i];
          for (int q = 0; q < i; ++q) s -= L[static_cast<size_t>(i) * k + q] * y[q];
          y[i] = s / L[static_cast<size_t>(i) * k + i];
        }
        for (int i = k - 1; i >= 0; --i) {
          double s = y[i];
          for (int q = i + 1; q < k; ++q) s -= L[static_cast<size_t>(q) * k + i] * out[q];
          out[i] = s / L[static_cast<size_t>(i) * k + i];
        }
      }
    }
  };
  if (rows * static_cast<long long>(k) * k < (1 << 16)) work(0, 1);
  else pool.run_shared(work);
  return 0;
}
