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

// One (feature, bin) cell: the sums of gradients and hessians and the count of the rows that fall in it, side
// by side, so a row's update of a feature touches one cache line instead of three.
struct Cell {
  double g, h, c;
};

struct Hist {
  std::vector<Cell> v;   // [F][nbins]
};

// The histogram of the rows idx[0 .. n) over bins held one COLUMN per feature (colbins [F][total]): a
// feature's pass streams the node's gradients, gathered once into row order (og / oh), and touches only that
// feature's cells, which stay in the first-level cache.  Workers share the features, so nothing is cleared,
// summed or ordered afterwards and the result is the same for any number of workers.
void build_hist(const uint8_t* colbins, long long total, int F, const int64_t* idx, long long n, const float* g, const float* h,
                int nbins, mimir_cpu::Pool& pool, std::vector<float>& og, std::vector<float>& oh, Cell* out) {
  const size_t cells = static_cast<size_t>(F) * nbins;
  memset(static_cast<void*>(out), 0, sizeof(Cell) * cells);
  if (static_cast<long long>(og.size()) < n) { og.resize(n); oh.resize(n); }
  for (long long k = 0; k < n; ++k) { og[k] = g[idx[k]]; oh[k] = h[idx[k]]; }
  auto feature = [&](int f) {
    const uint8_t* col = colbins + static_cast<size_t>(f) * total;
    Cell* c = out + static_cast<size_t>(f) * nbins;
    for (long long k = 0; k < n; ++k) {
      Cell& cell = c[col[idx[k]]];
      cell.g += og[k];
      cell.h += oh[k];
      cell.c += 1.0;
    }
  };
  const int workers = pool.size();
  if (n * F < 65536 || workers == 1 || F < 2) {
    for (int f = 0; f < F; ++f) feature(f);
    return;
  }
  // half the workers take features: a feature's pass is bound by the latency of its own additions, which a
  // second hardware thread on the same core only slows down
  const int takers = workers > 2 ? workers / 2 : workers;
  std::atomic<int> next{0};
  pool.run([&](int part, int) {
    if (part >= takers) return;
    for (int f = next.fetch_add(1); f < F; f = next.fetch_add(1)) feature(f);
  });
}

inline uint64_t splitmix(uint64_t& s) {
  uint64_t z = (s += 0x9E3779B97F4A7C15ull);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

}  // namespace

// Grows a tree over the rows idx[0 .. n) (idx is reordered in place); bins are held one column per feature.  colsample_k: features tried per node
// (0 = all), drawn from `seed`.  nodes: double [max_nodes][5] = feature (-1: leaf), bin, left, right, value;
// importance: double [F], gains added per split feature.  Returns the number of nodes, or -1.
static int grow_tree(const uint8_t* bins, long long total, int F, int64_t* idx, long long n, const float* g, const float* h,
                     int nbins, int max_depth, long long min_leaf, double min_gain, double l2, int colsample_k,
                     unsigned long long seed, double* nodes, int max_nodes, double* importance, float* leaf_out) {
  if (F < 1 || nbins < 1 || nbins > 256 || n < 1 || max_nodes < 1 || max_depth < 0) return -1;
  std::lock_guard<std::mutex> lk(mimir_cpu::pool_mutex());
  mimir_cpu::Pool& pool = mimir_cpu::pool();
  const size_t cells = static_cast<size_t>(F) * nbins;
  struct Item { long long lo, hi; int depth, node; Hist* hist; double G, H; };   // hist == nullptr: a leaf, sums given
  std::vector<Item> stack;
  std::vector<float> og, oh;
  std::vector<int64_t> scratch(n);
  std::vector<int> feats(F);
  uint64_t rng = seed;
  int n_nodes = 0;
  auto new_node = [&](double value) {
    double* nd = nodes + static_cast<size_t>(n_nodes) * 5;
    nd[0] = -1; nd[1] = 0; nd[2] = -1; nd[3] = -1; nd[4] = value;
    return n_nodes++;
  };
  Hist* root = new Hist{std::vector<Cell>(cells)};
  build_hist(bins, total, F, idx, n, g, h, nbins, pool, og, oh, root->v.data());
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
    const Cell* hc = it.hist ? it.hist->v.data() : nullptr;
    if (it.hist) {
      G = H = 0;
      for (int b = 0; b < nbins; ++b) { G += hc[b].g; H += hc[b].h; }      // every row falls in some bin of feature 0
    }
    if (n_nodes >= max_nodes) { delete it.hist; return -1; }
    const int node = new_node(-G / (H + l2));
    if (pt.parent >= 0) nodes[static_cast<size_t>(pt.parent) * 5 + 2 + pt.side] = node;
    const long long cnt = it.hi - it.lo;
    // a node that stays a leaf tells its rows their value (when the caller wants the tree's answers for the
    // rows it was grown on, which saves a pass over the tree afterwards)
    auto settle = [&]() {
      if (!leaf_out) return;
      const float v = static_cast<float>(-G / (H + l2));
      for (long long k = it.lo; k < it.hi; ++k) leaf_out[idx[k]] = v;
    };
    if (!it.hist) { settle(); continue; }
    if (it.depth >= max_depth || cnt < 2 * min_leaf) { delete it.hist; settle(); continue; }
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
        const Cell& cell = hc[static_cast<size_t>(f) * nbins + b];
        GL += cell.g; HL += cell.h; CL += cell.c;
        const double CR = static_cast<double>(cnt) - CL;
        if (CL < static_cast<double>(min_leaf) || CR < static_cast<double>(min_leaf)) continue;
        const double GR = G - GL, HR = H - HL;
        const double gain = GL * GL / (HL + l2) + GR * GR / (HR + l2) - parent_score;
        if (gain > best_gain) { best_gain = gain; best_f = f; best_b = b; best_GL = GL; best_HL = HL; }
      }
    }
    if (best_f < 0 || !(best_gain > min_gain)) { delete it.hist; settle(); continue; }
    importance[best_f] += best_gain;
    nodes[static_cast<size_t>(node) * 5] = best_f;
    nodes[static_cast<size_t>(node) * 5 + 1] = best_b;
    // stable partition of the rows: left rows first, both sides in their old order.  Large nodes are cut
    // into one chunk per worker: each counts its left rows, then writes both kinds at the places the counts
    // before it give (the same order as a serial pass).
    long long nl = 0, nr = 0;
    const uint8_t* col = bins + static_cast<size_t>(best_f) * total;
    const long long cnt_rows = it.hi - it.lo;
    const int chunks = cnt_rows < 32768 ? 1 : pool.size();
    if (chunks == 1) {
      for (long long k = it.lo; k < it.hi; ++k) {
        const int64_t r = idx[k];
        const bool left = col[r] <= best_b;
        idx[it.lo + nl] = r;           // both stores are made and one of the two cursors moves: no branch to mispredict
        scratch[nr] = r;
        nl += left;
        nr += !left;
      }
      memcpy(idx + it.lo + nl, scratch.data(), sizeof(int64_t) * nr);
    } else {
      std::vector<long long> lefts(chunks + 1, 0);
      const long long per = (cnt_rows + chunks - 1) / chunks;
      pool.run([&](int part, int) {
        if (part >= chunks) return;
        const long long a = it.lo + part * per, b = a + per < it.hi ? a + per : it.hi;
        long long c = 0;
        for (long long k = a; k < b; ++k) c += col[idx[k]] <= best_b;
        lefts[part + 1] = c;
      });
      for (int p = 0; p < chunks; ++p) lefts[p + 1] += lefts[p];
      nl = lefts[chunks];
      nr = cnt_rows - nl;
      pool.run([&](int part, int) {
        if (part >= chunks) return;
        const long long a = it.lo + part * per, b = a + per < it.hi ? a + per : it.hi;
        if (a >= b) return;
        long long wl = lefts[part], wr = nl + (a - it.lo) - lefts[part];       // rights before this chunk = rows before - lefts before
        for (long long k = a; k < b; ++k) {
          const int64_t r = idx[k];
          if (col[r] <= best_b) scratch[wl++] = r;
          else scratch[wr++] = r;
        }
      });
      memcpy(idx + it.lo, scratch.data(), sizeof(int64_t) * cnt_rows);
    }
    const long long mid = it.lo + nl;
    Hist *lh = nullptr, *rh = nullptr;
    if (it.depth + 1 < max_depth) {
      // children that may split again need histograms: the smaller one is counted, the larger one is
      // the parent's minus it
      lh = new Hist{std::vector<Cell>(cells)};
      rh = it.hist;
      auto subtract = [&]() {
        for (size_t c = 0; c < cells; ++c) { rh->v[c].g -= lh->v[c].g; rh->v[c].h -= lh->v[c].h; rh->v[c].c -= lh->v[c].c; }
      };
      if (nl <= nr) {
        build_hist(bins, total, F, idx + it.lo, nl, g, h, nbins, pool, og, oh, lh->v.data());
        subtract();
      } else {
        build_hist(bins, total, F, idx + mid, nr, g, h, nbins, pool, og, oh, lh->v.data());
        subtract();
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

// bins: one COLUMN per feature, uint8 [F][total]; idx [n] holds row numbers in [0, total).
// leaf_out (float [total], may be null) receives the value of the leaf each grown-on row reached.
MIMIR_CPU_API int mimir_cpu_grow_tree_answers(const uint8_t* colbins, long long total, int F, int64_t* idx, long long n, const float* g,
                                              const float* h, int nbins, int max_depth, long long min_leaf, double min_gain, double l2,
                                              int colsample_k, unsigned long long seed, double* nodes, int max_nodes,
                                              double* importance, float* leaf_out) {
  if (total < 1) return -1;
  for (long long k = 0; k < n; ++k)
    if (idx[k] < 0 || idx[k] >= total) return -1;
  return grow_tree(colbins, total, F, idx, n, g, h, nbins, max_depth, min_leaf, min_gain, l2, colsample_k, seed, nodes, max_nodes,
                   importance, leaf_out);
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
