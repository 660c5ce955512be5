// Clustering on the host where the work is a loop over pairs of rows that tensor operations serve badly
// (reference: cluster/dbscan.go, cluster/agglomerative.go): density groups by a concurrent union of the core rows
// within reach of one another, and Ward's hierarchy by the nearest-neighbour chain over the clusters' means.
#include <immintrin.h>

#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <memory>
#include <mutex>
#include <vector>

#include "cpu_pool.h"

#define MIMIR_CPU_API extern "C" __attribute__((visibility("default")))

namespace {

template <class Fn>
void share(mimir_cpu::Pool& pool, long long count, bool parallel, const Fn& fn) {
  if (!parallel || count < 2 || pool.size() == 1) {
    for (long long i = 0; i < count; ++i) fn(i);
    return;
  }
  std::atomic<long long> next{0};
  pool.run_shared([&](int, int) {
    for (long long i = next.fetch_add(1); i < count; i = next.fetch_add(1)) fn(i);
  });
}

// d[j] = |row - column j|^2 for the columns j in [j0, j1) of the table held one feature per row (Zt [F][n])
void distances_plain(const float* Zt, long long n, int F, const float* row, long long j0, long long j1, float* d) {
  for (long long j = j0; j < j1; ++j) d[j - j0] = 0.f;
  for (int f = 0; f < F; ++f) {
    const float* col = Zt + static_cast<size_t>(f) * n;
    const float v = row[f];
    for (long long j = j0; j < j1; ++j) { const float t = col[j] - v; d[j - j0] += t * t; }
  }
}

__attribute__((target("avx2,fma"))) void distances_avx2(const float* Zt, long long n, int F, const float* row, long long j0, long long j1,
                                                         float* d) {
  const long long m = j1 - j0;
  long long k = 0;
  for (; k + 8 <= m; k += 8) {
    __m256 acc = _mm256_setzero_ps();
    for (int f = 0; f < F; ++f) {
      const __m256 t = _mm256_sub_ps(_mm256_loadu_ps(Zt + static_cast<size_t>(f) * n + j0 + k), _mm256_set1_ps(row[f]));
      acc = _mm256_fmadd_ps(t, t, acc);
    }
    _mm256_storeu_ps(d + k, acc);
  }
  for (; k < m; ++k) {
    float acc = 0.f;
    for (int f = 0; f < F; ++f) { const float t = Zt[static_cast<size_t>(f) * n + j0 + k] - row[f]; acc += t * t; }
    d[k] = acc;
  }
}

void distances(const float* Zt, long long n, int F, const float* row, long long j0, long long j1, float* d) {
  static const bool fast = __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma");
  if (fast) distances_avx2(Zt, n, F, row, j0, j1, d);
  else distances_plain(Zt, n, F, row, j0, j1, d);
}

// Roots of a forest over 0 .. n-1 that several threads join at once: a root only ever becomes the child of a
// SMALLER root, so the partition that results is the connected components whatever the order of the joins, and
// each component's root is its smallest member.
struct Joined {
  std::vector<std::atomic<int32_t>> parent;
  explicit Joined(long long n) : parent(n) {
    for (long long i = 0; i < n; ++i) parent[i].store(static_cast<int32_t>(i), std::memory_order_relaxed);
  }
  int32_t find(int32_t x) {
    for (;;) {
      const int32_t p = parent[x].load(std::memory_order_acquire);
      if (p == x) return x;
      const int32_t g = parent[p].load(std::memory_order_acquire);
      if (g != p) {                       // halve the path: x skips to its grandparent (an ancestor either way)
        int32_t expect = p;
        parent[x].compare_exchange_weak(expect, g, std::memory_order_release, std::memory_order_relaxed);
      }
      x = p;
    }
  }
  void join(int32_t a, int32_t b) {
    for (;;) {
      a = find(a);
      b = find(b);
      if (a == b) return;
      if (a < b) { const int32_t t = a; a = b; b = t; }      // a is the larger root: it goes under b
      int32_t want = a;
      if (parent[a].compare_exchange_strong(want, b, std::memory_order_acq_rel, std::memory_order_acquire)) return;
    }
  }
};

}  // namespace

// Density groups (DBSCAN) over Z float [n][F] (standardized rows): a row with at least min_rows rows within
// sqrt(eps2) of it (itself included) is a core; cores within reach of one another share a group; groups are
// numbered by their first core; a row that is no core takes the lowest group among the cores that reach it, or -1.
// labels: int64 [n]; core: uint8 [n].  Rows are compared in tiles of columns, the rows of a tile shared among the
// workers; no list of neighbours is kept, so memory stays at the table's size.  Returns the number of groups.
MIMIR_CPU_API long long mimir_cpu_dbscan(const float* Z, long long n, int F, float eps2, long long min_rows, int64_t* labels, uint8_t* core) {
  if (n < 0 || n > std::numeric_limits<int32_t>::max() || F < 1 || !(eps2 > 0) || min_rows < 1) return -1;
  if (n == 0) return 0;
  std::lock_guard<std::mutex> lk(mimir_cpu::pool_mutex());
  mimir_cpu::Pool& pool = mimir_cpu::pool();
  std::vector<float> Zt(static_cast<size_t>(n) * F);
  for (long long r = 0; r < n; ++r)
    for (int f = 0; f < F; ++f) Zt[static_cast<size_t>(f) * n + r] = Z[static_cast<size_t>(r) * F + f];
  // a band of rows meets one tile of columns at a time: the tile (F x 512 floats) stays in the first-level cache
  // while every row of the band is compared with it
  const long long tile = 512, band = 64, bands = (n + band - 1) / band;
  const bool wide = n * n >= (1 << 18);
  std::unique_ptr<mimir_cpu::Pool::Awake> awake(wide ? new mimir_cpu::Pool::Awake(pool) : nullptr);
  // (1) how many rows each row has within reach
  share(pool, bands, wide, [&](long long bi) {
    std::vector<float> d(tile);
    const long long i0 = bi * band, i1 = i0 + band < n ? i0 + band : n;
    long long count[64] = {0};
    for (long long j0 = 0; j0 < n; j0 += tile) {
      const long long j1 = j0 + tile < n ? j0 + tile : n;
      for (long long i = i0; i < i1; ++i) {
        distances(Zt.data(), n, F, Z + static_cast<size_t>(i) * F, j0, j1, d.data());
        long long c = 0;
        for (long long j = 0; j < j1 - j0; ++j) c += d[j] <= eps2;
        count[i - i0] += c;
      }
    }
    for (long long i = i0; i < i1; ++i) core[i] = count[i - i0] >= min_rows ? 1 : 0;
  });
  // (2) cores within reach of one another join (each pair is met from its later row)
  Joined groups(n);
  share(pool, bands, wide, [&](long long bi) {
    std::vector<float> d(tile);
    const long long i0 = bi * band, i1 = i0 + band < n ? i0 + band : n;
    for (long long j0 = 0; j0 < i1; j0 += tile) {
      for (long long i = i0; i < i1; ++i) {
        if (!core[i] || j0 >= i) continue;
        const long long j1 = j0 + tile < i ? j0 + tile : i;
        distances(Zt.data(), n, F, Z + static_cast<size_t>(i) * F, j0, j1, d.data());
        for (long long j = 0; j < j1 - j0; ++j)
          if (d[j] <= eps2 && core[j0 + j]) groups.join(static_cast<int32_t>(i), static_cast<int32_t>(j0 + j));
      }
    }
  });
  // (3) numbers in the order of each group's first core
  std::vector<int64_t> number(n, -1);
  long long count = 0;
  for (long long i = 0; i < n; ++i) {
    labels[i] = -1;
    if (!core[i]) continue;
    const int32_t root = groups.find(static_cast<int32_t>(i));
    if (number[root] < 0) number[root] = count++;
    labels[i] = number[root];
  }
  // (4) the other rows: the lowest group among the cores that reach them
  share(pool, bands, wide, [&](long long bi) {
    std::vector<float> d(tile);
    const long long i0 = bi * band, i1 = i0 + band < n ? i0 + band : n;
    bool any = false;
    for (long long i = i0; i < i1; ++i) any = any || !core[i];
    if (!any) return;
    for (long long j0 = 0; j0 < n; j0 += tile) {
      const long long j1 = j0 + tile < n ? j0 + tile : n;
      for (long long i = i0; i < i1; ++i) {
        if (core[i]) continue;
        distances(Zt.data(), n, F, Z + static_cast<size_t>(i) * F, j0, j1, d.data());
        int64_t best = labels[i];
        for (long long j = 0; j < j1 - j0; ++j)
          if (d[j] <= eps2 && core[j0 + j]) {
            const int64_t g = number[groups.find(static_cast<int32_t>(j0 + j))];
            if (best < 0 || g < best) best = g;
          }
        labels[i] = best;
      }
    }
  });
  return count;
}

namespace {

// out[j] = sa s_j / (sa + s_j) |c - column j|^2 for the clusters held one per column (C [F][cap], sizes s; a
// column of size 0 is a cluster that no longer exists and reads as infinity)
void ward_row_plain(const double* C, long long cap, long long m, int F, const double* c, double sa, const double* s, double* out) {
  for (long long j = 0; j < m; ++j) out[j] = 0.0;
  for (int f = 0; f < F; ++f) {
    const double* col = C + static_cast<size_t>(f) * cap;
    const double v = c[f];
    for (long long j = 0; j < m; ++j) { const double t = col[j] - v; out[j] += t * t; }
  }
  for (long long j = 0; j < m; ++j) out[j] = s[j] > 0 ? sa * s[j] / (sa + s[j]) * out[j] : std::numeric_limits<double>::infinity();
}

__attribute__((target("avx2,fma"))) void ward_row_avx2(const double* C, long long cap, long long m, int F, const double* c, double sa,
                                                        const double* s, double* out) {
  long long j = 0;
  for (; j + 4 <= m; j += 4) {
    __m256d acc = _mm256_setzero_pd();
    for (int f = 0; f < F; ++f) {
      const __m256d t = _mm256_sub_pd(_mm256_loadu_pd(C + static_cast<size_t>(f) * cap + j), _mm256_set1_pd(c[f]));
      acc = _mm256_fmadd_pd(t, t, acc);
    }
    _mm256_storeu_pd(out + j, acc);
  }
  for (; j < m; ++j) {
    double acc = 0.0;
    for (int f = 0; f < F; ++f) { const double t = C[static_cast<size_t>(f) * cap + j] - c[f]; acc += t * t; }
    out[j] = acc;
  }
  for (j = 0; j < m; ++j) out[j] = s[j] > 0 ? sa * s[j] / (sa + s[j]) * out[j] : std::numeric_limits<double>::infinity();
}

}  // namespace

// Ward's hierarchy by the nearest-neighbour chain WITHOUT a distance matrix: the Ward distance of two clusters
// is |A||B| / (|A| + |B|) |mean_A - mean_B|^2, so a cluster's nearest neighbour is one pass over the means of
// the clusters that exist (F multiply-adds per cluster instead of one load from an n x n matrix, and n F
// numbers of memory instead of n^2).  Z: double [n][F], standardized rows.  The table of means is packed again
// whenever half of its columns have died.  merges: int64 [n-1][2] (rows are clusters 0 .. n-1, merge s makes
// cluster n + s, in the order the chain finds them); heights: double [n-1].  A tie keeps the previous link, so a
// chain always ends.
MIMIR_CPU_API int mimir_cpu_ward_means(const double* Z, long long n, int F, int64_t* merges, double* heights) {
  if (n < 1 || F < 1) return -1;
  static const bool fast = __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma");
  // a large table's passes over the means are shared among the workers, who stay awake between them
  std::lock_guard<std::mutex> lk(mimir_cpu::pool_mutex());
  mimir_cpu::Pool& pool = mimir_cpu::pool();
  const bool wide = n >= 16384 && pool.size() > 1;
  std::unique_ptr<mimir_cpu::Pool::Awake> awake(wide ? new mimir_cpu::Pool::Awake(pool) : nullptr);
  long long cap = n, m = n, live = n;                 // columns allocated, columns in use, clusters that exist
  std::vector<double> C(static_cast<size_t>(F) * cap), size(n, 1.0), row(n), mean(F);
  std::vector<int64_t> name(n);
  for (long long r = 0; r < n; ++r) {
    name[r] = r;
    for (int f = 0; f < F; ++f) C[static_cast<size_t>(f) * cap + r] = Z[static_cast<size_t>(r) * F + f];
  }
  std::vector<long long> chain;
  long long first = 0;
  for (long long step = 0; step < n - 1; ++step) {
    if (live * 2 <= m && m > 64) {
      // pack the columns of the clusters that exist to the front; the chain's places move with them
      std::vector<long long> to(m, -1);
      long long k = 0;
      for (long long j = 0; j < m; ++j)
        if (size[j] > 0) to[j] = k++;
      for (int f = 0; f < F; ++f) {
        double* col = C.data() + static_cast<size_t>(f) * cap;
        for (long long j = 0; j < m; ++j)
          if (to[j] >= 0) col[to[j]] = col[j];
      }
      for (long long j = 0; j < m; ++j)
        if (to[j] >= 0) { size[to[j]] = size[j]; name[to[j]] = name[j]; }
      for (auto& c : chain) c = to[c];
      m = k;
      first = 0;
    }
    if (chain.empty()) {
      while (!(size[first] > 0)) ++first;
      chain.push_back(first);
    }
    double h = 0;
    for (;;) {
      const long long a = chain.back();
      for (int f = 0; f < F; ++f) mean[f] = C[static_cast<size_t>(f) * cap + a];
      const long long piece = 4096, pieces = (m + piece - 1) / piece;
      share(pool, pieces, wide && m >= 4 * piece, [&](long long p) {
        const long long j0 = p * piece, mj = j0 + piece < m ? piece : m - j0;
        if (fast) ward_row_avx2(C.data() + j0, cap, mj, F, mean.data(), size[a], size.data() + j0, row.data() + j0);
        else ward_row_plain(C.data() + j0, cap, mj, F, mean.data(), size[a], size.data() + j0, row.data() + j0);
      });
      row[a] = std::numeric_limits<double>::infinity();
      long long b = 0;
      double best = row[0];
      for (long long j = 1; j < m; ++j)
        if (row[j] < best) { best = row[j]; b = j; }
      if (chain.size() > 1) {
        const long long before = chain[chain.size() - 2];
        if (row[before] <= best) { b = before; best = row[before]; }      // a tie keeps the previous link
        if (b == before) { h = best; break; }
      }
      chain.push_back(b);
    }
    const long long a = chain.back();
    chain.pop_back();
    const long long b = chain.back();
    chain.pop_back();
    merges[2 * step] = name[a];
    merges[2 * step + 1] = name[b];
    heights[step] = h;
    const double sa = size[a], sb = size[b];
    for (int f = 0; f < F; ++f) {
      double* col = C.data() + static_cast<size_t>(f) * cap;
      col[a] = (sa * col[a] + sb * col[b]) / (sa + sb);
    }
    size[a] = sa + sb;
    size[b] = 0;
    name[a] = n + step;
    --live;
  }
  return 0;
}
