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
struct alignas(32) Cell {
  double g, h, c, pad;     // four doubles: one 256-bit load, add and store per update
};

inline uint64_t mix(uint64_t z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

// A node while the tree grows, level by level.
struct Grow {
  long long lo = 0, hi = 0;        // its rows are idx[lo .. hi)
  int depth = 0;
  uint64_t path = 1;               // 1 for the root, 2p / 2p + 1 for the children of p: seeds the feature draw
  int left = -1, right = -1;       // indices into the growing list, -1 for a leaf
  int feature = -1, bin = 0;
  double G = 0, H = 0, gain = 0, GL = 0, HL = 0;
  long long nl = 0;                // rows that go left
  std::vector<Cell> hist;          // empty for a node that cannot split (depth limit): its sums are given
  bool counted = false;            // its histogram is counted from its rows (the smaller child); else parent - sibling
};

// One feature's pass over the rows idx[lo .. hi): the cell of each row's bin takes (gradient, hessian, 1).
// With AVX2 the three additions are one 256-bit add on the padded cell.
__attribute__((target("avx2"))) void count_cells_avx2(const uint8_t* col, const int64_t* idx, const float* og, const float* oh,
                                                       long long lo, long long hi, Cell* c) {
  for (long long k = lo; k < hi; ++k) {
    double* cell = reinterpret_cast<double*>(c + col[idx[k]]);
    const __m256d inc = _mm256_set_pd(0.0, 1.0, static_cast<double>(oh[k]), static_cast<double>(og[k]));
    _mm256_store_pd(cell, _mm256_add_pd(_mm256_load_pd(cell), inc));
  }
}

void count_cells(const uint8_t* col, const int64_t* idx, const float* og, const float* oh, long long lo, long long hi, Cell* c) {
  static const bool avx2 = __builtin_cpu_supports("avx2");
  if (avx2) {
    count_cells_avx2(col, idx, og, oh, lo, hi, c);
    return;
  }
  for (long long k = lo; k < hi; ++k) {
    Cell& cell = c[col[idx[k]]];
    cell.g += og[k];
    cell.h += oh[k];
    cell.c += 1.0;
  }
}

// runs fn(i) for i in [0, count) on the pool, items handed out one by one; serial when there is little to share
template <class Fn>
void for_each(mimir_cpu::Pool& pool, long long count, bool parallel, const Fn& fn) {
  if (!parallel || count < 2 || pool.size() == 1) {
    for (long long i = 0; i < count; ++i) fn(i);
    return;
  }
  // pieces come from one counter and the job does not wait for sleeping workers: whoever is awake takes them
  std::atomic<long long> next{0};
  pool.run_shared([&](int, int) {
    for (long long i = next.fetch_add(1); i < count; i = next.fetch_add(1)) fn(i);
  });
}

}  // namespace

// Grows a tree over the rows idx[0 .. n) (idx is reordered in place); bins are held one column per feature.
// colsample_k: features tried per node (0 = all), drawn from `seed` and the node's place in the tree.
// nodes: double [max_nodes][5] = feature (-1: leaf), bin, left, right, value, numbered depth first, left before
// right; importance: double [F], gains added per split feature.  Returns the number of nodes, or -1.
//
// The tree grows one LEVEL at a time, so the pool is entered a few times per level instead of a few times per
// node: (1) every node of the level finds its best split, (2) the rows of the splitting nodes are partitioned,
// (3) the gradients are gathered into row order once for the whole level, (4) the histograms of the smaller
// children are counted, one (child, feature) pass per task, each pass touching one feature's cells only,
// (5) the larger children take the parent's histogram minus the sibling's.  Every sum is made by one worker in
// row order, so the tree does not depend on the number of workers.
static int grow_tree(const uint8_t* bins, long long total, int F, int64_t* idx, long long n, const float* g, const float* h,
                     int nbins, int max_depth, long long min_leaf, double min_gain, double l2, int colsample_k,
                     unsigned long long seed, double* nodes, int max_nodes, double* importance, float* leaf_out) {
  if (F < 1 || nbins < 1 || nbins > 256 || n < 1 || max_nodes < 1 || max_depth < 0) return -1;
  std::lock_guard<std::mutex> lk(mimir_cpu::pool_mutex());
  mimir_cpu::Pool& pool = mimir_cpu::pool();
  const size_t cells = static_cast<size_t>(F) * nbins;
  std::vector<Grow> all;
  all.reserve(static_cast<size_t>(max_nodes < 4096 ? max_nodes : 4096));
  std::vector<float> og(n), oh(n);
  std::vector<int64_t> scratch(n);
  const bool wide = n * static_cast<long long>(F) >= 65536;      // enough work to share at all

  auto gather = [&](long long lo, long long hi) {
    const long long chunk = 16384, count = (hi - lo + chunk - 1) / chunk;
    for_each(pool, count, wide, [&](long long c) {
      const long long a = lo + c * chunk, b = a + chunk < hi ? a + chunk : hi;
      for (long long k = a; k < b; ++k) { og[k] = g[idx[k]]; oh[k] = h[idx[k]]; }
    });
  };
  auto count_feature = [&](Grow& nd, int f) { count_cells(bins + static_cast<size_t>(f) * total, idx, og.data(), oh.data(), nd.lo, nd.hi,
                                                          nd.hist.data() + static_cast<size_t>(f) * nbins); };

  all.emplace_back();
  all[0].lo = 0;
  all[0].hi = n;
  all[0].hist.assign(cells, Cell{0, 0, 0, 0});
  gather(0, n);
  for_each(pool, F, wide, [&](long long f) { count_feature(all[0], static_cast<int>(f)); });
  {
    double G = 0, H = 0;
    for (int b = 0; b < nbins; ++b) { G += all[0].hist[b].g; H += all[0].hist[b].h; }      // every row falls in some bin of feature 0
    all[0].G = G;
    all[0].H = H;
  }
  std::vector<int> level{0}, next_level;
  while (!level.empty()) {
    // (1) the best split of every node of the level that may split
    for_each(pool, static_cast<long long>(level.size()), wide && level.size() >= 4, [&](long long li) {
      Grow& nd = all[level[li]];
      const long long cnt = nd.hi - nd.lo;
      if (nd.hist.empty() || nd.depth >= max_depth || cnt < 2 * min_leaf) return;
      std::vector<int> feats(F);
      int nf = F;
      for (int f = 0; f < F; ++f) feats[f] = f;
      if (colsample_k > 0 && colsample_k < F) {
        uint64_t rng = mix(seed ^ (nd.path * 0x9E3779B97F4A7C15ull));
        for (int k = 0; k < colsample_k; ++k) {
          rng = mix(rng + 0x9E3779B97F4A7C15ull);
          const int j = k + static_cast<int>(rng % static_cast<uint64_t>(F - k));
          const int t = feats[k]; feats[k] = feats[j]; feats[j] = t;
        }
        nf = colsample_k;
      }
      const double parent_score = nd.G * nd.G / (nd.H + l2);
      double best_gain = -1, best_GL = 0, best_HL = 0, best_CL = 0;
      int best_f = -1, best_b = 0;
      for (int q = 0; q < nf; ++q) {
        const int f = feats[q];
        const Cell* hc = nd.hist.data() + static_cast<size_t>(f) * nbins;
        double GL = 0, HL = 0, CL = 0;
        for (int b = 0; b < nbins; ++b) {
          GL += hc[b].g; HL += hc[b].h; CL += hc[b].c;
          const double CR = static_cast<double>(cnt) - CL;
          if (CL < static_cast<double>(min_leaf) || CR < static_cast<double>(min_leaf)) continue;
          const double GR = nd.G - GL, HR = nd.H - HL;
          const double gain = GL * GL / (HL + l2) + GR * GR / (HR + l2) - parent_score;
          if (gain > best_gain || (gain == best_gain && best_f >= 0 && f < best_f)) {
            best_gain = gain; best_f = f; best_b = b; best_GL = GL; best_HL = HL; best_CL = CL;
          }
        }
      }
      if (best_f < 0 || !(best_gain > min_gain)) return;
      nd.feature = best_f;
      nd.bin = best_b;
      nd.gain = best_gain;
      nd.GL = best_GL;
      nd.HL = best_HL;
      nd.nl = static_cast<long long>(best_CL + 0.5);
    });
    // children get their places in the list (serially: the list may move in memory)
    next_level.clear();
    for (int id : level) {
      if (all[id].feature < 0) {
        std::vector<Cell>().swap(all[id].hist);          // a leaf: its histogram is not needed again
        continue;
      }
      if (static_cast<int>(all.size()) + 2 > max_nodes) return -1;
      const Grow p = Grow{all[id].lo, all[id].hi, all[id].depth, all[id].path};
      const long long mid = p.lo + all[id].nl;
      Grow l, r;
      l.lo = p.lo; l.hi = mid; r.lo = mid; r.hi = p.hi;
      l.depth = r.depth = p.depth + 1;
      l.path = p.path * 2; r.path = p.path * 2 + 1;
      l.G = all[id].GL; l.H = all[id].HL; r.G = all[id].G - all[id].GL; r.H = all[id].H - all[id].HL;
      all[id].left = static_cast<int>(all.size());
      all.push_back(std::move(l));
      all[id].right = static_cast<int>(all.size());
      all.push_back(std::move(r));
      importance[all[id].feature] += all[id].gain;
      next_level.push_back(id);           // parents for now; replaced by their children below
    }
    if (next_level.empty()) break;
    // (2) the rows of each splitting node: left rows first, both sides in their old order.  Few, large nodes are
    // cut into chunks (counted, then written at the places the counts before them give); many nodes go one per task.
    const long long parents = static_cast<long long>(next_level.size());
    const int workers = pool.size();
    if (wide && parents < workers) {
      for (int id : next_level) {
        Grow& nd = all[id];
        const uint8_t* col = bins + static_cast<size_t>(nd.feature) * total;
        const long long rows = nd.hi - nd.lo;
        const int chunks = rows < 32768 ? 1 : workers;
        if (chunks == 1) {
          long long nl = 0, nr = 0;
          for (long long k = nd.lo; k < nd.hi; ++k) {
            const int64_t r = idx[k];
            const bool left = col[r] <= nd.bin;
            idx[nd.lo + nl] = r;          // both stores are made and one cursor moves: no branch to mispredict
            scratch[nd.lo + nr] = r;
            nl += left;
            nr += !left;
          }
          memcpy(idx + nd.lo + nl, scratch.data() + nd.lo, sizeof(int64_t) * nr);
          continue;
        }
        std::vector<long long> lefts(chunks + 1, 0);
        const long long per = (rows + chunks - 1) / chunks;
        for_each(pool, chunks, true, [&](long long part) {
          const long long a = nd.lo + part * per, b = a + per < nd.hi ? a + per : nd.hi;
          long long c = 0;
          for (long long k = a; k < b; ++k) c += col[idx[k]] <= nd.bin;
          lefts[part + 1] = c;
        });
        for (int p = 0; p < chunks; ++p) lefts[p + 1] += lefts[p];
        const long long nl = lefts[chunks];
        for_each(pool, chunks, true, [&](long long part) {
          const long long a = nd.lo + part * per, b = a + per < nd.hi ? a + per : nd.hi;
          long long wl = nd.lo + lefts[part], wr = nd.lo + nl + (a - nd.lo) - lefts[part];
          for (long long k = a; k < b; ++k) {
            const int64_t r = idx[k];
            if (col[r] <= nd.bin) scratch[wl++] = r;
            else scratch[wr++] = r;
          }
        });
        memcpy(idx + nd.lo, scratch.data() + nd.lo, sizeof(int64_t) * rows);
      }
    } else {
      for_each(pool, parents, wide, [&](long long pi) {
        Grow& nd = all[next_level[pi]];
        const uint8_t* col = bins + static_cast<size_t>(nd.feature) * total;
        long long nl = 0, nr = 0;
        for (long long k = nd.lo; k < nd.hi; ++k) {
          const int64_t r = idx[k];
          const bool left = col[r] <= nd.bin;
          idx[nd.lo + nl] = r;
          scratch[nd.lo + nr] = r;
          nl += left;
          nr += !left;
        }
        memcpy(idx + nd.lo + nl, scratch.data() + nd.lo, sizeof(int64_t) * nr);
      });
    }
    // children that may split again need histograms: the smaller one is counted, the larger one is the
    // parent's minus it
    std::vector<int> counted, parents_of;
    std::vector<int> children;
    for (int id : next_level) {
      Grow& nd = all[id];
      children.push_back(nd.left);
      children.push_back(nd.right);
      if (nd.depth + 1 >= max_depth) { std::vector<Cell>().swap(nd.hist); continue; }     // the children are leaves: sums are given
      Grow &l = all[nd.left], &r = all[nd.right];
      Grow& small = (l.hi - l.lo) <= (r.hi - r.lo) ? l : r;
      small.hist.assign(cells, Cell{0, 0, 0, 0});
      small.counted = true;
      counted.push_back(&small == &l ? nd.left : nd.right);
      parents_of.push_back(id);
    }
    if (!counted.empty()) {
      // (3) gradients in row order for the rows that will be counted: chunks of every counted child, one run
      {
        std::vector<std::pair<long long, long long>> pieces;
        for (int c : counted)
          for (long long a = all[c].lo; a < all[c].hi; a += 16384) pieces.emplace_back(a, a + 16384 < all[c].hi ? a + 16384 : all[c].hi);
        for_each(pool, static_cast<long long>(pieces.size()), wide, [&](long long i) {
          for (long long k = pieces[i].first; k < pieces[i].second; ++k) { og[k] = g[idx[k]]; oh[k] = h[idx[k]]; }
        });
      }
      // (4) one (child, feature) pass per task
      const long long tasks = static_cast<long long>(counted.size()) * F;
      for_each(pool, tasks, wide, [&](long long t) { count_feature(all[counted[t / F]], static_cast<int>(t % F)); });
      // (5) the sibling takes what is left of the parent's histogram
      for_each(pool, static_cast<long long>(counted.size()), wide && counted.size() >= 4, [&](long long i) {
        Grow& parent = all[parents_of[i]];
        Grow& small = all[counted[i]];
        Grow& big = all[counted[i] == parent.left ? parent.right : parent.left];
        big.hist = std::move(parent.hist);
        for (size_t c = 0; c < cells; ++c) { big.hist[c].g -= small.hist[c].g; big.hist[c].h -= small.hist[c].h; big.hist[c].c -= small.hist[c].c; }
      });
    }
    level.swap(children);
  }
  // numbered depth first, left before right, like a recursive builder numbers them
  int n_nodes = 0;
  std::vector<std::pair<int, int>> stack;      // (node in the list, slot of the parent to patch or -1)
  stack.emplace_back(0, -1);
  while (!stack.empty()) {
    const auto [id, slot] = stack.back();
    stack.pop_back();
    const Grow& nd = all[id];
    if (n_nodes >= max_nodes) return -1;
    double* out = nodes + static_cast<size_t>(n_nodes) * 5;
    const double value = -nd.G / (nd.H + l2);
    out[0] = nd.feature; out[1] = nd.feature >= 0 ? nd.bin : 0; out[2] = -1; out[3] = -1; out[4] = value;
    if (slot >= 0) nodes[slot] = n_nodes;
    if (nd.feature >= 0) {
      stack.emplace_back(nd.right, n_nodes * 5 + 3);      // right is pushed first so that left is numbered first
      stack.emplace_back(nd.left, n_nodes * 5 + 2);
    } else if (leaf_out) {
      const float v = static_cast<float>(value);
      for (long long k = nd.lo; k < nd.hi; ++k) leaf_out[idx[k]] = v;
    }
    ++n_nodes;
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
