// Gradient histograms for tree learners on the host (reference: the hand-written histogram kernels
// behind tree/ and its forests: one pass over the rows of a node adds each row's gradient, hessian
// and count into the bin of every feature).
//
// bins: uint8 [rows_total][F] row-major; idx: the rows of the node (null = rows 0 .. n-1); out: double
// [3][F][nbins] = sums of g, sums of h, counts.  Rows are split evenly over the worker threads, each
// adds into a histogram of its own, and the partial histograms are summed in thread order, so the
// result does not depend on timing.
#include <cstring>

#include "cpu_pool.h"

#define MIMIR_CPU_API extern "C" __attribute__((visibility("default")))

MIMIR_CPU_API int mimir_cpu_hist(const uint8_t* bins, int F, const int64_t* idx, long long n, const float* g, const float* h,
                                 int nbins, double* out) {
  if (F < 1 || nbins < 1 || nbins > 256 || n < 0) return -1;
  const size_t cells = static_cast<size_t>(F) * nbins;
  memset(out, 0, sizeof(double) * 3 * cells);
  if (n == 0) return 0;
  std::lock_guard<std::mutex> lk(mimir_cpu::pool_mutex());
  mimir_cpu::Pool& pool = mimir_cpu::pool();
  const int parts = n < 4096 ? 1 : pool.size();
  std::vector<double> partial(static_cast<size_t>(parts) * 3 * cells, 0.0);
  auto work = [&](int part, int nparts) {
    if (part >= parts) return;
    (void)nparts;
    const long long per = (n + parts - 1) / parts, r0 = part * per, r1 = r0 + per < n ? r0 + per : n;
    double* hg = partial.data() + static_cast<size_t>(part) * 3 * cells;
    double* hh = hg + cells;
    double* hc = hh + cells;
    for (long long k = r0; k < r1; ++k) {
      const long long r = idx ? idx[k] : k;
      const uint8_t* row = bins + static_cast<size_t>(r) * F;
      const double gv = g[r], hv = h[r];
      for (int f = 0; f < F; ++f) {
        const size_t c = static_cast<size_t>(f) * nbins + row[f];
        hg[c] += gv;
        hh[c] += hv;
        hc[c] += 1.0;
      }
    }
  };
  if (parts == 1) work(0, 1);
  else pool.run(work);
  for (int p = 0; p < parts; ++p) {
    const double* src = partial.data() + static_cast<size_t>(p) * 3 * cells;
    for (size_t c = 0; c < 3 * cells; ++c) out[c] += src[c];
  }
  return 0;
}

// ---------------------------------------------------------------------------
// One regression tree on gradients / hessians, grown here from the root (reference: tree/: second-order
// gain with L2, histogram of the smaller child counted, the larger one = parent - sibling).
// ---------------------------------------------------------------------------
namespace {

struct Hist {
  std::vector<double> v;   // [3][F][nbins]
};

void build_hist(const uint8_t* bins, int F, const int64_t* idx, long long n, const float* g, const float* h, int nbins,
                mimir_cpu::Pool& pool, std::vector<double>& partial, double* out) {
  const size_t cells = static_cast<size_t>(F) * nbins;
  memset(out, 0, sizeof(double) * 3 * cells);
  const int parts = n < 8192 ? 1 : pool.size();
  if (parts == 1) {
    double *hg = out, *hh = out + cells, *hc = out + 2 * cells;
    for (long long k = 0; k < n; ++k) {
      const long long r = idx[k];
      const uint8_t* row = bins + static_cast<size_t>(r) * F;
      const double gv = g[r], hv = h[r];
      for (int f = 0; f < F; ++f) {
        const size_t c = static_cast<size_t>(f) * nbins + row[f];
        hg[c] += gv; hh[c] += hv; hc[c] += 1.0;
      }
    }
    return;
  }
  partial.assign(static_cast<size_t>(parts) * 3 * cells, 0.0);
  pool.run([&](int part, int) {
    if (part >= parts) return;
    const long long per = (n + parts - 1) / parts, r0 = part * per, r1 = r0 + per < n ? r0 + per : n;
    double* hg = partial.data() + static_cast<size_t>(part) * 3 * cells;
    double *hh = hg + cells, *hc = hh + cells;
    for (long long k = r0; k < r1; ++k) {
      const long long r = idx[k];
      const uint8_t* row = bins + static_cast<size_t>(r) * F;
      const double gv = g[r], hv = h[r];
      for (int f = 0; f < F; ++f) {
        const size_t c = static_cast<size_t>(f) * nbins + row[f];
        hg[c] += gv; hh[c] += hv; hc[c] += 1.0;
      }
    }
  });
  for (int p = 0; p < parts; ++p) {
    const double* src = partial.data() + static_cast<size_t>(p) * 3 * cells;
    for (size_t c = 0; c < 3 * cells; ++c) out[c] += src[c];
  }
}

inline uint64_t splitmix(uint64_t& s) {
  uint64_t z = (s += 0x9E3779B97F4A7C15ull);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

}  // namespace

// Grows a tree over the rows idx[0 .. n) (idx is reordered in place).  colsample_k: features tried per node
// (0 = all), drawn from `seed`.  nodes: double [max_nodes][5] = feature (-1: leaf), bin, left, right, value;
// importance: double [F], gains added per split feature.  Returns the number of nodes, or -1.
MIMIR_CPU_API int mimir_cpu_grow_tree(const uint8_t* bins, int F, int64_t* idx, long long n, const float* g, const float* h,
                                      int nbins, int max_depth, long long min_leaf, double min_gain, double l2, int colsample_k,
                                      unsigned long long seed, double* nodes, int max_nodes, double* importance) {
  if (F < 1 || nbins < 1 || nbins > 256 || n < 1 || max_nodes < 1 || max_depth < 0) return -1;
  std::lock_guard<std::mutex> lk(mimir_cpu::pool_mutex());
  mimir_cpu::Pool& pool = mimir_cpu::pool();
  const size_t cells = static_cast<size_t>(F) * nbins;
  struct Item { long long lo, hi; int depth, node; Hist* hist; double G, H; };   // hist == nullptr: a leaf, sums given
  std::vector<Item> stack;
  std::vector<double> partial;
  std::vector<int64_t> scratch(n);
  std::vector<int> feats(F);
  uint64_t rng = seed;
  int n_nodes = 0;
  auto new_node = [&](double value) {
    double* nd = nodes + static_cast<size_t>(n_nodes) * 5;
    nd[0] = -1; nd[1] = 0; nd[2] = -1; nd[3] = -1; nd[4] = value;
    return n_nodes++;
  };
  Hist* root = new Hist{std::vector<double>(3 * cells)};
  build_hist(bins, F, idx, n, g, h, nbins, pool, partial, root->v.data());
  stack.push_back({0, n, 0, -1, root, 0, 0});
  // the parent's child slots are patched when a child gets its number; children are numbered in
  // depth-first order, left before right, like a recursive builder numbers them
  struct Patch { int parent; int side; };
  std::vector<Patch> patch;
  patch.push_back({-1, 0});
  while (!stack.empty()) {
    Item it = stack.back();
    stack.pop_back();
    const Patch pt = patch.back();
    patch.pop_back();
    double G = it.G, H = it.H;
    const double* hg = it.hist ? it.hist->v.data() : nullptr;
    const double *hh = hg + cells, *hc = hh + cells;
    if (it.hist) {
      G = H = 0;
      for (int b = 0; b < nbins; ++b) { G += hg[b]; H += hh[b]; }
    }
    if (n_nodes >= max_nodes) { delete it.hist; return -1; }
    const int node = new_node(-G / (H + l2));
    if (pt.parent >= 0) nodes[static_cast<size_t>(pt.parent) * 5 + 2 + pt.side] = node;
    const long long cnt = it.hi - it.lo;
    if (!it.hist) continue;
    if (it.depth >= max_depth || cnt < 2 * min_leaf) { delete it.hist; continue; }
    // features tried at this node
    int nf = F;
    for (int f = 0; f < F; ++f) feats[f] = f;
    if (colsample_k > 0 && colsample_k < F) {
      for (int k = 0; k < colsample_k; ++k) {
        const int j = k + static_cast<int>(splitmix(rng) % static_cast<uint64_t>(F - k));
        const int t = feats[k]; feats[k] = feats[j]; feats[j] = t;
      }
      nf = colsample_k;
    }
    const double parent_score = G * G / (H + l2);
    double best_gain = -1, best_GL = 0, best_HL = 0;
    int best_f = -1, best_b = 0;
    for (int q = 0; q < nf; ++q) {
      const int f = feats[q];
      double GL = 0, HL = 0, CL = 0;
      for (int b = 0; b < nbins; ++b) {
        const size_t c = static_cast<size_t>(f) * nbins + b;
        GL += hg[c]; HL += hh[c]; CL += hc[c];
        const double CR = static_cast<double>(cnt) - CL;
        if (CL < static_cast<double>(min_leaf) || CR < static_cast<double>(min_leaf)) continue;
        const double GR = G - GL, HR = H - HL;
        const double gain = GL * GL / (HL + l2) + GR * GR / (HR + l2) - parent_score;
        if (gain > best_gain) { best_gain = gain; best_f = f; best_b = b; best_GL = GL; best_HL = HL; }
      }
    }
    if (best_f < 0 || !(best_gain > min_gain)) { delete it.hist; continue; }
    importance[best_f] += best_gain;
    nodes[static_cast<size_t>(node) * 5] = best_f;
    nodes[static_cast<size_t>(node) * 5 + 1] = best_b;
    // stable partition of the rows: left rows first, both sides in their old order
    long long nl = 0, nr = 0;
    for (long long k = it.lo; k < it.hi; ++k) {
      const int64_t r = idx[k];
      if (bins[static_cast<size_t>(r) * F + best_f] <= best_b) idx[it.lo + nl++] = r;
      else scratch[nr++] = r;
    }
    memcpy(idx + it.lo + nl, scratch.data(), sizeof(int64_t) * nr);
    const long long mid = it.lo + nl;
    Hist *lh = nullptr, *rh = nullptr;
    if (it.depth + 1 < max_depth) {
      // children that may split again need histograms: the smaller one is counted, the larger one is
      // the parent's minus it
      lh = new Hist{std::vector<double>(3 * cells)};
      rh = it.hist;
      if (nl <= nr) {
        build_hist(bins, F, idx + it.lo, nl, g, h, nbins, pool, partial, lh->v.data());
        for (size_t c = 0; c < 3 * cells; ++c) rh->v[c] -= lh->v[c];
      } else {
        build_hist(bins, F, idx + mid, nr, g, h, nbins, pool, partial, lh->v.data());
        for (size_t c = 0; c < 3 * cells; ++c) rh->v[c] -= lh->v[c];
        Hist* t = lh; lh = rh; rh = t;  // lh = left (larger, by subtraction), rh = right (counted)
      }
    } else {
      delete it.hist;                   // leaves: their sums are the split's prefix sums
    }
    // right is pushed first so that left is numbered first
    stack.push_back({mid, it.hi, it.depth + 1, node, rh, G - best_GL, H - best_HL});
    patch.push_back({node, 1});
    stack.push_back({it.lo, mid, it.depth + 1, node, lh, best_GL, best_HL});
    patch.push_back({node, 0});
  }
  return n_nodes;
}

// out[r] = value of the leaf row r of `bins` (uint8 [n][F]) reaches in the tree `nodes` (double [n_nodes][5]).
MIMIR_CPU_API int mimir_cpu_tree_predict(const uint8_t* bins, int F, long long n, const double* nodes, int n_nodes, float* out) {
  if (F < 1 || n < 0 || n_nodes < 1) return -1;
  std::lock_guard<std::mutex> lk(mimir_cpu::pool_mutex());
  mimir_cpu::Pool& pool = mimir_cpu::pool();
  std::atomic<long long> next{0};
  const long long chunk = 4096;
  std::atomic<int> bad{0};
  auto work = [&](int, int) {
    for (long long r0 = next.fetch_add(chunk); r0 < n; r0 = next.fetch_add(chunk)) {
      const long long r1 = r0 + chunk < n ? r0 + chunk : n;
      for (long long r = r0; r < r1; ++r) {
        const uint8_t* row = bins + static_cast<size_t>(r) * F;
        int node = 0, steps = 0;
        for (;;) {
          const double* nd = nodes + static_cast<size_t>(node) * 5;
          const int f = static_cast<int>(nd[0]);
          if (f < 0) { out[r] = static_cast<float>(nd[4]); break; }
          const int nxt = static_cast<int>(row[f] <= static_cast<int>(nd[1]) ? nd[2] : nd[3]);
          if (f >= F || nxt <= node || nxt >= n_nodes || ++steps > n_nodes) { bad.store(1); out[r] = 0.f; break; }   // not a tree
          node = nxt;
        }
      }
    }
  };
  if (n < 16384) work(0, 1);
  else pool.run(work);
  return bad.load() ? -1 : 0;
}
