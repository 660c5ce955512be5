// Gradient histograms for tree learners on the host (reference: the hand-written histogram kernels
// behind tree/ and its forests: one pass over the rows of a node adds each row's gradient, hessian
// and count into the bin of every feature).
//
// bins: uint8 [rows_total][F] row-major; idx: the rows of the node (null = rows 0 .. n-1); out: double
// [3][F][nbins] = sums of g, sums of h, counts.  Rows are split evenly over the worker threads, each
// adds into a histogram of its own, and the partial histograms are summed in thread order, so the
// result does not depend on timing.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <memory>
#include <new>

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

// A node's histogram: cells that are NOT zeroed when they are made (the pass that counts a feature clears that
// feature's cells first, on the worker that counts it).
struct Hist {
  Cell* p = nullptr;
  Hist() = default;
  Hist(const Hist&) = delete;
  Hist& operator=(const Hist&) = delete;
  Hist(Hist&& o) noexcept : p(o.p) { o.p = nullptr; }
  Hist& operator=(Hist&& o) noexcept { if (this != &o) { release(); p = o.p; o.p = nullptr; } return *this; }
  ~Hist() { release(); }
  void make(size_t cells) { release(); p = static_cast<Cell*>(::operator new(cells * sizeof(Cell), std::align_val_t(32))); }
  void release() { if (p) ::operator delete(p, std::align_val_t(32)); p = nullptr; }
  bool empty() const { return p == nullptr; }
  Cell* data() { return p; }
  const Cell* data() const { return p; }
  Cell& operator[](size_t i) { return p[i]; }
};

// A node while the tree grows, level by level.
struct Grow {
  long long lo = 0, hi = 0;        // its rows are idx[lo .. hi)
  int depth = 0;
  uint64_t path = 1;               // 1 for the root, 2p / 2p + 1 for the children of p: seeds the feature draw
  int left = -1, right = -1;       // indices into the growing list, -1 for a leaf
  int feature = -1, bin = 0;
  double G = 0, H = 0, gain = 0, GL = 0, HL = 0;
  long long nl = 0;                // rows that go left
  std::vector<int> feats;          // the features drawn for this node (empty: all of them)
  Hist hist;                       // empty for a node that cannot split (depth limit): its sums are given
  bool counted = false;            // its histogram is counted from its rows (the smaller child); else parent - sibling
};

// One pass over the rows idx[lo .. hi) for one feature or for two at once: the cell of each row's bin takes
// (gradient, hessian, 1).  gh holds the two numbers of a row side by side, in row order.  Two features per pass
// halve the reads of the row numbers and the gradients, which is what a large node's pass waits for.  With AVX2
// the three additions are one 256-bit add on the padded cell.
__attribute__((target("avx2"))) void count_cells_avx2(const uint8_t* col, const uint8_t* col2, const int32_t* idx, const float* gh,
                                                       long long lo, long long hi, Cell* c, Cell* c2) {
  const __m256d one = _mm256_set_pd(0.0, 1.0, 0.0, 0.0);
  if (col2 == nullptr) {
    for (long long k = lo; k < hi; ++k) {
      double* cell = reinterpret_cast<double*>(c + col[idx[k]]);
      const __m128 pair = _mm_castpd_ps(_mm_load_sd(reinterpret_cast<const double*>(gh + 2 * k)));
      const __m256d inc = _mm256_add_pd(_mm256_insertf128_pd(_mm256_setzero_pd(), _mm_cvtps_pd(pair), 0), one);
      _mm256_store_pd(cell, _mm256_add_pd(_mm256_load_pd(cell), inc));
    }
    return;
  }
  for (long long k = lo; k < hi; ++k) {
    const int32_t r = idx[k];
    double* cell = reinterpret_cast<double*>(c + col[r]);
    double* cell2 = reinterpret_cast<double*>(c2 + col2[r]);
    const __m128 pair = _mm_castpd_ps(_mm_load_sd(reinterpret_cast<const double*>(gh + 2 * k)));
    const __m256d inc = _mm256_add_pd(_mm256_insertf128_pd(_mm256_setzero_pd(), _mm_cvtps_pd(pair), 0), one);
    _mm256_store_pd(cell, _mm256_add_pd(_mm256_load_pd(cell), inc));
    _mm256_store_pd(cell2, _mm256_add_pd(_mm256_load_pd(cell2), inc));
  }
}

void count_cells(const uint8_t* col, const uint8_t* col2, const int32_t* idx, const float* gh, long long lo, long long hi, Cell* c,
                 Cell* c2) {
  static const bool avx2 = __builtin_cpu_supports("avx2");
  if (avx2) {
    count_cells_avx2(col, col2, idx, gh, lo, hi, c, c2);
    return;
  }
  for (long long k = lo; k < hi; ++k) {
    const int32_t r = idx[k];
    Cell& cell = c[col[r]];
    cell.g += gh[2 * k];
    cell.h += gh[2 * k + 1];
    cell.c += 1.0;
    if (col2) {
      Cell& other = c2[col2[r]];
      other.g += gh[2 * k];
      other.h += gh[2 * k + 1];
      other.c += 1.0;
    }
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
// children are counted, one (child, feature pair) pass per task, each pass touching its two features' cells only,
// (5) the larger children take the parent's histogram minus the sibling's.  Every sum is made by one worker in
// row order, so the tree does not depend on the number of workers.
// The caller holds the pool's lock, or passes serial = true: then nothing is handed to the pool and several
// trees may grow at once, one per worker (a forest).
static int grow_tree(mimir_cpu::Pool& pool, const uint8_t* bins, long long total, int F, int32_t* idx, long long n, const float* g,
                     const float* h, int nbins, int max_depth, long long min_leaf, double min_gain, double l2, int colsample_k,
                     unsigned long long seed, double* nodes, int max_nodes, double* importance, float* leaf_out, bool serial,
                     double min_weight, const int32_t* allowed, int n_allowed) {
  if (F < 1 || nbins < 1 || nbins > 256 || n < 1 || max_nodes < 1 || max_depth < 0) return -1;
  // `allowed` (ascending feature numbers, or null for all) is what this tree may split on: below, features are
  // counted, drawn and compared by their place u in that list, and feat(u) is the feature itself
  if (allowed) {
    if (n_allowed < 1) return -1;
    for (int u = 0; u < n_allowed; ++u)
      if (allowed[u] < 0 || allowed[u] >= F || (u > 0 && allowed[u] <= allowed[u - 1])) return -1;
  }
  const int Fu = allowed ? n_allowed : F;
  auto feat = [&](int u) { return allowed ? static_cast<int>(allowed[u]) : u; };
  // With few features drawn per node (at most half of them, as forests do) a node counts the features it drew
  // and nothing else, and both children are counted: cheaper than counting every feature for the smaller child
  // and subtracting whole histograms, which small nodes deep in a tree cannot pay for.
  const bool sampled = colsample_k > 0 && colsample_k < Fu;
  const bool direct = sampled && colsample_k * 2 <= Fu;
  const int held = direct ? colsample_k : Fu;                      // features a node's histogram holds
  const size_t cells = static_cast<size_t>(held) * nbins;
  auto draw = [&](Grow& nd) {
    nd.feats.resize(Fu);
    for (int f = 0; f < Fu; ++f) nd.feats[f] = f;
    uint64_t rng = mix(seed ^ (nd.path * 0x9E3779B97F4A7C15ull));
    for (int k = 0; k < colsample_k; ++k) {
      rng = mix(rng + 0x9E3779B97F4A7C15ull);
      const int j = k + static_cast<int>(rng % static_cast<uint64_t>(Fu - k));
      const int t = nd.feats[k]; nd.feats[k] = nd.feats[j]; nd.feats[j] = t;
    }
    nd.feats.resize(colsample_k);
  };
  std::vector<Grow> all;
  all.reserve(static_cast<size_t>(max_nodes < 4096 ? max_nodes : 4096));
  std::vector<float> gh(2 * static_cast<size_t>(n));       // (gradient, hessian) of the rows in the order of idx
  std::vector<int32_t> scratch(n);
  const bool wide = !serial && n * static_cast<long long>(Fu) >= 65536;      // enough work to share at all
  // the workers stay awake while a shared tree grows, so even its small steps are worth handing out
  std::unique_ptr<mimir_cpu::Pool::Awake> awake(wide ? new mimir_cpu::Pool::Awake(pool) : nullptr);
  auto busy = [&](long long work) { return wide && work > 0; };

  auto gather = [&](long long lo, long long hi) {
    const long long chunk = 16384, count = (hi - lo + chunk - 1) / chunk;
    for_each(pool, count, busy(hi - lo), [&](long long c) {
      const long long a = lo + c * chunk, b = a + chunk < hi ? a + chunk : hi;
      for (long long k = a; k < b; ++k) { gh[2 * k] = g[idx[k]]; gh[2 * k + 1] = h[idx[k]]; }
    });
  };
  // held features 2 q and 2 q + 1 (the last pair of an odd count is one feature) of a node, cleared and counted
  const int pairs = (held + 1) / 2;
  auto count_pair = [&](Grow& nd, int q) {
    const int j = 2 * q;
    const bool two = j + 1 < held;
    const int f = feat(direct ? nd.feats[j] : j), f2 = !two ? 0 : feat(direct ? nd.feats[j + 1] : j + 1);
    Cell* c = nd.hist.data() + static_cast<size_t>(j) * nbins;
    memset(static_cast<void*>(c), 0, sizeof(Cell) * nbins * (two ? 2 : 1));
    count_cells(bins + static_cast<size_t>(f) * total, two ? bins + static_cast<size_t>(f2) * total : nullptr, idx, gh.data(), nd.lo,
                nd.hi, c, c + nbins);
  };

  all.emplace_back();
  all[0].lo = 0;
  all[0].hi = n;
  all[0].hist.make(cells);
  if (direct) draw(all[0]);
  gather(0, n);
  for_each(pool, pairs, busy(n * held), [&](long long q) { count_pair(all[0], static_cast<int>(q)); });
  {
    double G = 0, H = 0;
    for (int b = 0; b < nbins; ++b) { G += all[0].hist[b].g; H += all[0].hist[b].h; }      // every row falls in some bin of the first held feature
    all[0].G = G;
    all[0].H = H;
  }
  std::vector<int> level{0}, next_level;
  while (!level.empty()) {
    // (1) the best split of every node of the level that may split
    for_each(pool, static_cast<long long>(level.size()), level.size() >= 4 && busy(static_cast<long long>(level.size()) * held * nbins / 4), [&](long long li) {
      Grow& nd = all[level[li]];
      const long long cnt = nd.hi - nd.lo;
      if (nd.hist.empty() || nd.depth >= max_depth || cnt < 2 * min_leaf) return;
      if (sampled && !direct) draw(nd);
      const int nf = sampled ? colsample_k : Fu;
      const double parent_score = nd.G * nd.G / (nd.H + l2);
      double best_gain = -1, best_GL = 0, best_HL = 0, best_CL = 0;
      int best_f = -1, best_b = 0;
      for (int q = 0; q < nf; ++q) {
        const int f = sampled ? nd.feats[q] : q;
        const Cell* hc = nd.hist.data() + static_cast<size_t>(direct ? q : f) * nbins;
        double GL = 0, HL = 0, CL = 0;
        for (int b = 0; b < nbins; ++b) {
          if (hc[b].c == 0) continue;          // no row here: the same cut as the bin before
          GL += hc[b].g; HL += hc[b].h; CL += hc[b].c;
          const double CR = static_cast<double>(cnt) - CL;
          if (CL < static_cast<double>(min_leaf) || CR < static_cast<double>(min_leaf)) continue;
          const double GR = nd.G - GL, HR = nd.H - HL;
          if (HL < min_weight || HR < min_weight) continue;
          const double gain = GL * GL / (HL + l2) + GR * GR / (HR + l2) - parent_score;
          if (gain > best_gain || (gain == best_gain && best_f >= 0 && f < best_f)) {
            best_gain = gain; best_f = f; best_b = b; best_GL = GL; best_HL = HL; best_CL = CL;
          }
        }
      }
      if (best_f < 0 || !(best_gain > min_gain)) return;
      nd.feature = feat(best_f);
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
        all[id].hist.release();          // a leaf: its histogram is not needed again
        continue;
      }
      if (static_cast<int>(all.size()) + 2 > max_nodes) return -1;
      Grow p;
      p.lo = all[id].lo; p.hi = all[id].hi; p.depth = all[id].depth; p.path = all[id].path;
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
    const int workers = serial ? 1 : pool.size();
    long long level_rows = 0;
    for (int id : next_level) level_rows += all[id].hi - all[id].lo;
    auto split_rows = [&](Grow& nd) {
      const uint8_t* col = bins + static_cast<size_t>(nd.feature) * total;
      long long nl = 0, nr = 0;
      for (long long k = nd.lo; k < nd.hi; ++k) {
        const int32_t r = idx[k];
        const bool left = col[r] <= nd.bin;
        idx[nd.lo + nl] = r;          // both stores are made and one cursor moves: no branch to mispredict
        scratch[nd.lo + nr] = r;
        nl += left;
        nr += !left;
      }
      memcpy(idx + nd.lo + nl, scratch.data() + nd.lo, sizeof(int32_t) * nr);
    };
    if (wide && parents < workers) {
      std::vector<int> small_ones;
      for (int id : next_level)
        if (all[id].hi - all[id].lo < 32768) small_ones.push_back(id);
      long long small_rows = 0;
      for (int id : small_ones) small_rows += all[id].hi - all[id].lo;
      for_each(pool, static_cast<long long>(small_ones.size()), busy(small_rows), [&](long long i) { split_rows(all[small_ones[i]]); });
      for (int id : next_level) {
        Grow& nd = all[id];
        const uint8_t* col = bins + static_cast<size_t>(nd.feature) * total;
        const long long rows = nd.hi - nd.lo;
        if (rows < 32768) continue;
        const int chunks = workers;
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
            const int32_t r = idx[k];
            if (col[r] <= nd.bin) scratch[wl++] = r;
            else scratch[wr++] = r;
          }
        });
        for_each(pool, chunks, true, [&](long long part) {
          const long long a = nd.lo + part * per, b = a + per < nd.hi ? a + per : nd.hi;
          if (b > a) memcpy(idx + a, scratch.data() + a, sizeof(int32_t) * (b - a));
        });
      }
    } else {
      for_each(pool, parents, busy(level_rows), [&](long long pi) { split_rows(all[next_level[pi]]); });
    }
    // children that may split again need histograms: the smaller one is counted, the larger one is the
    // parent's minus it
    std::vector<int> counted, parents_of;
    std::vector<int> children;
    for (int id : next_level) {
      Grow& nd = all[id];
      children.push_back(nd.left);
      children.push_back(nd.right);
      if (nd.depth + 1 >= max_depth) { nd.hist.release(); continue; }     // the children are leaves: sums are given
      Grow &l = all[nd.left], &r = all[nd.right];
      if (direct) {
        nd.hist.release();
        for (int child : {nd.left, nd.right}) {
          Grow& ch = all[child];
          if (ch.hi - ch.lo < 2 * min_leaf || ch.hi - ch.lo < 2) continue;      // it cannot split: no histogram
          ch.hist.make(cells);
          ch.counted = true;
          draw(ch);
          counted.push_back(child);
        }
        continue;
      }
      Grow& small = (l.hi - l.lo) <= (r.hi - r.lo) ? l : r;
      small.hist.make(cells);
      small.counted = true;
      counted.push_back(&small == &l ? nd.left : nd.right);
      parents_of.push_back(id);
    }
    if (!counted.empty()) {
      // (3) gradients in row order for the rows that will be counted: chunks of every counted child, one run
      long long counted_rows = 0;
      {
        std::vector<std::pair<long long, long long>> pieces;
        for (int c : counted) {
          counted_rows += all[c].hi - all[c].lo;
          for (long long a = all[c].lo; a < all[c].hi; a += 16384) pieces.emplace_back(a, a + 16384 < all[c].hi ? a + 16384 : all[c].hi);
        }
        for_each(pool, static_cast<long long>(pieces.size()), busy(counted_rows), [&](long long i) {
          for (long long k = pieces[i].first; k < pieces[i].second; ++k) { gh[2 * k] = g[idx[k]]; gh[2 * k + 1] = h[idx[k]]; }
        });
      }
      // (4) one (child, feature pair) pass per task
      const long long tasks = static_cast<long long>(counted.size()) * pairs;
      for_each(pool, tasks, busy(counted_rows * held), [&](long long t) { count_pair(all[counted[t / pairs]], static_cast<int>(t % pairs)); });
      // (5) the sibling takes what is left of the parent's histogram
      for_each(pool, static_cast<long long>(parents_of.size()), parents_of.size() >= 4 && busy(static_cast<long long>(parents_of.size() * cells)), [&](long long i) {
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
  std::vector<int> leaves;
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
      leaves.push_back(id);
    }
    ++n_nodes;
  }
  // every row's answer: the leaves share the workers (a row belongs to one leaf, so no two tasks write one place)
  for_each(pool, static_cast<long long>(leaves.size()), busy(n), [&](long long i) {
    const Grow& nd = all[leaves[i]];
    const float v = static_cast<float>(-nd.G / (nd.H + l2));
    for (long long k = nd.lo; k < nd.hi; ++k) leaf_out[idx[k]] = v;
  });
  return n_nodes;
}

// bins: one COLUMN per feature, uint8 [F][total]; idx [n] holds row numbers in [0, total).
// leaf_out (float [total], may be null) receives the value of the leaf each grown-on row reached.
// min_weight: the smallest sum of hessians a child may hold; allowed [n_allowed]: the features (ascending) the
// tree may split on, or null for all.
MIMIR_CPU_API int mimir_cpu_grow_tree_answers(const uint8_t* colbins, long long total, int F, int64_t* idx, long long n, const float* g,
                                              const float* h, int nbins, int max_depth, long long min_leaf, double min_gain, double l2,
                                              int colsample_k, unsigned long long seed, double* nodes, int max_nodes,
                                              double* importance, float* leaf_out, double min_weight, const int32_t* allowed,
                                              int n_allowed) {
  if (total < 1 || total > INT32_MAX || n < 1) return -1;
  std::vector<int32_t> rows(n);          // row numbers as 32-bit values: half the bytes every pass reads
  for (long long k = 0; k < n; ++k) {
    if (idx[k] < 0 || idx[k] >= total) return -1;
    rows[k] = static_cast<int32_t>(idx[k]);
  }
  std::lock_guard<std::mutex> lk(mimir_cpu::pool_mutex());
  const int cnt = grow_tree(mimir_cpu::pool(), colbins, total, F, rows.data(), n, g, h, nbins, max_depth, min_leaf, min_gain, l2,
                            colsample_k, seed, nodes, max_nodes, importance, leaf_out, false, min_weight, allowed, n_allowed);
  for (long long k = 0; k < n; ++k) idx[k] = rows[k];
  return cnt;
}

// A forest: `trees` trees, each grown on its own list of rows (rows int64 [trees][n], numbers in [0, total),
// repeats allowed: bootstrap samples) with the gradients g, h [total] shared by all.  The trees share the workers,
// one whole tree per task, each grown serially: small nodes deep in a tree have too little work to split among
// threads, whole trees do.  seeds [trees]: the feature-draw seed of each tree.  nodes: double
// [trees][max_nodes][5]; counts: int [trees]; importance: double [trees][F] (zeroed here).  min_weight, allowed
// [trees][n_allowed]: as in mimir_cpu_boost.  Returns 0 or -1.
MIMIR_CPU_API int mimir_cpu_grow_forest(const uint8_t* colbins, long long total, int F, const int64_t* rows, long long n, int trees,
                                        const float* g, const float* h, int nbins, int max_depth, long long min_leaf, double min_gain,
                                        double l2, int colsample_k, const unsigned long long* seeds, double* nodes, int max_nodes,
                                        int* counts, double* importance, double min_weight, const int32_t* allowed, int n_allowed) {
  if (total < 1 || total > INT32_MAX || n < 1 || trees < 0) return -1;
  std::lock_guard<std::mutex> lk(mimir_cpu::pool_mutex());
  mimir_cpu::Pool& pool = mimir_cpu::pool();
  std::atomic<int> bad{0};
  for_each(pool, trees, trees > 1, [&](long long t) {
    std::vector<int32_t> idx(n);
    const int64_t* mine = rows + static_cast<size_t>(t) * n;
    for (long long k = 0; k < n; ++k) {
      if (mine[k] < 0 || mine[k] >= total) { bad.store(1); return; }
      idx[k] = static_cast<int32_t>(mine[k]);
    }
    double* imp = importance + static_cast<size_t>(t) * F;
    for (int f = 0; f < F; ++f) imp[f] = 0;
    const int cnt = grow_tree(pool, colbins, total, F, idx.data(), n, g, h, nbins, max_depth, min_leaf, min_gain, l2, colsample_k,
                              seeds ? seeds[t] : 0ull, nodes + static_cast<size_t>(t) * max_nodes * 5, max_nodes, imp, nullptr, true,
                              min_weight, allowed ? allowed + static_cast<size_t>(t) * n_allowed : nullptr, n_allowed);
    if (cnt <= 0) { bad.store(1); return; }
    counts[t] = cnt;
  });
  return bad.load() ? -1 : 0;
}

// `rounds` rounds of second-order boosting over all rows, without returning to the caller between trees: the
// workers stay awake from one tree to the next, and a round's gradients and score update are two passes here
// instead of a dozen tensor operations.  kind 0: squared error (g = score - y, h = 1); kind 1: logistic
// (p = sigmoid(score), g = p - y, h = max(p (1 - p), 1e-6)).  score [total] (float) is updated in place by
// lr * (the leaf each row reached).  seeds [rounds]: the feature-draw seed of each tree (read when colsample_k > 0).
// nodes: double [rounds][max_nodes][5]; counts: int [rounds]; importance: double [rounds][F] (zeroed here).
// min_weight: the smallest sum of hessians a child may hold; allowed: int32 [rounds][n_allowed], the features
// (ascending) each round's tree may split on, or null for all.  Returns the number of rounds done (all), or -1.
MIMIR_CPU_API int mimir_cpu_boost(const uint8_t* colbins, long long total, int F, const float* y, float* score, int kind, int rounds,
                                  double lr, int nbins, int max_depth, long long min_leaf, double min_gain, double l2, int colsample_k,
                                  const unsigned long long* seeds, double* nodes, int max_nodes, int* counts, double* importance,
                                  double min_weight, const int32_t* allowed, int n_allowed) {
  if (total < 1 || total > INT32_MAX || rounds < 0 || (kind != 0 && kind != 1)) return -1;
  std::lock_guard<std::mutex> lk(mimir_cpu::pool_mutex());
  mimir_cpu::Pool& pool = mimir_cpu::pool();
  mimir_cpu::Pool::Awake awake(pool);
  std::vector<float> g(total), h(total), leaf(total);
  std::vector<int32_t> idx(total);
  const long long chunk = 8192, chunks = (total + chunk - 1) / chunk;
  const bool wide = total >= 4 * chunk;
  const float step = static_cast<float>(lr);
  for (int r = 0; r < rounds; ++r) {
    for_each(pool, chunks, wide, [&](long long c) {
      const long long a = c * chunk, b = a + chunk < total ? a + chunk : total;
      for (long long k = a; k < b; ++k) idx[k] = static_cast<int32_t>(k);
      if (kind == 0) {
        for (long long k = a; k < b; ++k) { g[k] = score[k] - y[k]; h[k] = 1.0f; }
      } else {
        for (long long k = a; k < b; ++k) {
          const float p = 1.0f / (1.0f + std::exp(-score[k]));
          const float hh = p * (1.0f - p);
          g[k] = p - y[k];
          h[k] = hh < 1e-6f ? 1e-6f : hh;
        }
      }
    });
    double* imp = importance + static_cast<size_t>(r) * F;
    for (int f = 0; f < F; ++f) imp[f] = 0;
    const int cnt = grow_tree(pool, colbins, total, F, idx.data(), total, g.data(), h.data(), nbins, max_depth, min_leaf, min_gain, l2,
                              colsample_k, seeds ? seeds[r] : 0ull, nodes + static_cast<size_t>(r) * max_nodes * 5, max_nodes, imp,
                              leaf.data(), false, min_weight, allowed ? allowed + static_cast<size_t>(r) * n_allowed : nullptr, n_allowed);
    if (cnt <= 0) return -1;
    counts[r] = cnt;
    for_each(pool, chunks, wide, [&](long long c) {
      const long long a = c * chunk, b = a + chunk < total ? a + chunk : total;
      for (long long k = a; k < b; ++k) score[k] += step * leaf[k];
    });
  }
  return rounds;
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

// Softmax boosting over `classes` classes: as mimir_cpu_boost, but a round computes every row's class
// probabilities once from score [total][classes] and then grows one tree per class on
// g = p_c - (y == c), h = max(p_c (1 - p_c), 1e-6); the scores move after each tree, the probabilities of the round
// do not.  y: int64 [total] in [0, classes).  seeds [rounds][classes]; allowed [rounds][n_allowed] (one list per
// round, shared by its trees) or null.  nodes: double [rounds * classes][max_nodes][5]; counts: int
// [rounds * classes]; importance: double [rounds * classes][F].  Returns the rounds done, or -1.
MIMIR_CPU_API int mimir_cpu_boost_classes(const uint8_t* colbins, long long total, int F, const int64_t* y, float* score, int classes,
                                          int rounds, double lr, int nbins, int max_depth, long long min_leaf, double min_gain, double l2,
                                          int colsample_k, const unsigned long long* seeds, double* nodes, int max_nodes, int* counts,
                                          double* importance, double min_weight, const int32_t* allowed, int n_allowed) {
  if (total < 1 || total > INT32_MAX || rounds < 0 || classes < 2 || classes > 4096) return -1;
  for (long long k = 0; k < total; ++k)
    if (y[k] < 0 || y[k] >= classes) return -1;
  std::lock_guard<std::mutex> lk(mimir_cpu::pool_mutex());
  mimir_cpu::Pool& pool = mimir_cpu::pool();
  mimir_cpu::Pool::Awake awake(pool);
  std::vector<float> p(static_cast<size_t>(total) * classes), g(total), h(total), leaf(total);
  std::vector<int32_t> idx(total);
  const long long chunk = 4096, chunks = (total + chunk - 1) / chunk;
  const bool wide = total >= 4 * chunk;
  const float step = static_cast<float>(lr);
  for (int r = 0; r < rounds; ++r) {
    for_each(pool, chunks, wide, [&](long long c) {
      const long long a = c * chunk, b = a + chunk < total ? a + chunk : total;
      for (long long k = a; k < b; ++k) {
        const float* s = score + static_cast<size_t>(k) * classes;
        float* q = p.data() + static_cast<size_t>(k) * classes;
        float top = s[0];
        for (int c2 = 1; c2 < classes; ++c2) top = s[c2] > top ? s[c2] : top;
        float sum = 0.f;
        for (int c2 = 0; c2 < classes; ++c2) { q[c2] = std::exp(s[c2] - top); sum += q[c2]; }
        const float inv = 1.0f / sum;
        for (int c2 = 0; c2 < classes; ++c2) q[c2] *= inv;
      }
    });
    for (int cls = 0; cls < classes; ++cls) {
      const size_t t = static_cast<size_t>(r) * classes + cls;
      for_each(pool, chunks, wide, [&](long long c) {
        const long long a = c * chunk, b = a + chunk < total ? a + chunk : total;
        for (long long k = a; k < b; ++k) {
          const float pk = p[static_cast<size_t>(k) * classes + cls];
          const float hh = pk * (1.0f - pk);
          idx[k] = static_cast<int32_t>(k);
          g[k] = pk - (y[k] == cls ? 1.0f : 0.0f);
          h[k] = hh < 1e-6f ? 1e-6f : hh;
        }
      });
      double* imp = importance + t * F;
      for (int f = 0; f < F; ++f) imp[f] = 0;
      const int cnt = grow_tree(pool, colbins, total, F, idx.data(), total, g.data(), h.data(), nbins, max_depth, min_leaf, min_gain, l2,
                                colsample_k, seeds ? seeds[t] : 0ull, nodes + t * max_nodes * 5, max_nodes, imp, leaf.data(), false,
                                min_weight, allowed ? allowed + static_cast<size_t>(r) * n_allowed : nullptr, n_allowed);
      if (cnt <= 0) return -1;
      counts[t] = cnt;
      for_each(pool, chunks, wide, [&](long long c) {
        const long long a = c * chunk, b = a + chunk < total ? a + chunk : total;
        for (long long k = a; k < b; ++k) score[static_cast<size_t>(k) * classes + cls] += step * leaf[k];
      });
    }
  }
  return rounds;
}

namespace {

// the number of edges below x (NaN: n_edges): the first edge that is not below x, found without a branch the
// processor has to guess
inline int bin_of(const float* e, int n_edges, float x) {
  if (!(x == x) || n_edges == 0) return n_edges;
  const float* base = e;
  int len = n_edges;
  while (len > 1) {
    const int half = len / 2;
    base += base[half - 1] < x ? half : 0;
    len -= half;
  }
  return static_cast<int>(base - e) + (base[0] < x ? 1 : 0);
}

// sixteen values of one feature at a time: the same halving search in every lane, the probes fetched by a gather
__attribute__((target("avx512f,avx512bw"))) void bins_avx512(const float* e, int n_edges, const float* x, long long count, uint8_t* out) {
  long long k = 0;
  if (n_edges > 0) {
    for (; k + 16 <= count; k += 16) {
      const __m512 v = _mm512_loadu_ps(x + k);
      __m512i base = _mm512_setzero_si512();
      int len = n_edges;
      while (len > 1) {
        const int half = len / 2;
        const __m512 probe = _mm512_i32gather_ps(_mm512_add_epi32(base, _mm512_set1_epi32(half - 1)), e, 4);
        base = _mm512_mask_add_epi32(base, _mm512_cmp_ps_mask(probe, v, _CMP_LT_OQ), base, _mm512_set1_epi32(half));
        len -= half;
      }
      const __m512 probe = _mm512_i32gather_ps(base, e, 4);
      base = _mm512_mask_add_epi32(base, _mm512_cmp_ps_mask(probe, v, _CMP_LT_OQ), base, _mm512_set1_epi32(1));
      base = _mm512_mask_mov_epi32(base, _mm512_cmp_ps_mask(v, v, _CMP_UNORD_Q), _mm512_set1_epi32(n_edges));
      _mm_storeu_si128(reinterpret_cast<__m128i*>(out + k), _mm512_cvtepi32_epi8(base));
    }
  }
  for (; k < count; ++k) out[k] = static_cast<uint8_t>(bin_of(e, n_edges, x[k]));
}

}  // namespace

// Bins a table: X float [n][F] (row-major); edges float [F][n_edges], ascending per feature.  The bin of a value
// is the number of its feature's edges below it (NaN: n_edges, after every edge).  Written twice: rows uint8
// [n][F] (what prediction walks) and cols uint8 [F][n] (what the grower reads); either may be null.
// n_edges <= 255.  Chunks of rows share the workers; a chunk is turned to one column per feature first, so the
// search runs over sixteen neighbouring values of a feature at a time where the CPU has AVX-512.
MIMIR_CPU_API int mimir_cpu_bin_table(const float* X, long long n, int F, const float* edges, int n_edges, uint8_t* rows, uint8_t* cols) {
  if (n < 0 || F < 1 || n_edges < 0 || n_edges > 255) return -1;
  static const bool wide_lanes = __builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw");
  std::lock_guard<std::mutex> lk(mimir_cpu::pool_mutex());
  mimir_cpu::Pool& pool = mimir_cpu::pool();
  const long long chunk = 2048, chunks = (n + chunk - 1) / chunk;
  for_each(pool, chunks, n * F >= 65536, [&](long long c) {
    const long long a = c * chunk, b = a + chunk < n ? a + chunk : n, m = b - a;
    std::vector<float> xs(static_cast<size_t>(F) * m);
    std::vector<uint8_t> bs(static_cast<size_t>(F) * m);
    for (long long r = 0; r < m; ++r)
      for (int f = 0; f < F; ++f) xs[static_cast<size_t>(f) * m + r] = X[static_cast<size_t>(a + r) * F + f];
    for (int f = 0; f < F; ++f) {
      const float* e = edges + static_cast<size_t>(f) * n_edges;
      const float* x = xs.data() + static_cast<size_t>(f) * m;
      uint8_t* o = bs.data() + static_cast<size_t>(f) * m;
      if (wide_lanes) bins_avx512(e, n_edges, x, m, o);
      else
        for (long long r = 0; r < m; ++r) o[r] = static_cast<uint8_t>(bin_of(e, n_edges, x[r]));
      if (cols) memcpy(cols + static_cast<size_t>(f) * n + a, o, m);
    }
    if (rows)
      for (long long r = 0; r < m; ++r)
        for (int f = 0; f < F; ++f) rows[static_cast<size_t>(a + r) * F + f] = bs[static_cast<size_t>(f) * m + r];
  });
  return 0;
}

// out[r] = the sum over `trees` trees of the value of the leaf row r of `bins` (uint8 [n][F]) reaches.  The
// trees' node tables lie one after another in `nodes` (double [.][5], child numbers relative to the tree's
// first node); tree t owns nodes offsets[t] .. offsets[t + 1].  Sums are made in tree order in double.
MIMIR_CPU_API int mimir_cpu_trees_predict(const uint8_t* bins, int F, long long n, const double* nodes, const long long* offsets, int trees,
                                          float* out) {
  if (F < 1 || n < 0 || trees < 0) return -1;
  // the tables in a form a walk reads quickly, checked once: a child comes after its parent (so every walk
  // ends) and lies inside its tree, a feature inside the row
  struct Step { int32_t feature, bin, child[2]; double value; };
  std::vector<Step> steps(trees > 0 ? static_cast<size_t>(offsets[trees] - offsets[0]) : 0);
  for (int t = 0; t < trees; ++t) {
    const long long lo = offsets[t], count = offsets[t + 1] - lo;
    if (count <= 0 || lo - offsets[0] < 0) return -1;
    for (long long i = 0; i < count; ++i) {
      const double* nd = nodes + static_cast<size_t>(lo + i) * 5;
      Step& s = steps[static_cast<size_t>(lo - offsets[0] + i)];
      s.feature = static_cast<int32_t>(nd[0]);
      s.bin = static_cast<int32_t>(nd[1]);
      s.child[0] = static_cast<int32_t>(nd[2]);
      s.child[1] = static_cast<int32_t>(nd[3]);
      s.value = nd[4];
      if (s.feature >= F) return -1;
      if (s.feature >= 0 && (s.child[0] <= i || s.child[0] >= count || s.child[1] <= i || s.child[1] >= count)) return -1;
    }
  }
  std::lock_guard<std::mutex> lk(mimir_cpu::pool_mutex());
  mimir_cpu::Pool& pool = mimir_cpu::pool();
  const long long chunk = 1024, chunks = (n + chunk - 1) / chunk;
  for_each(pool, chunks, n * trees >= 65536, [&](long long c) {
    const long long a = c * chunk, b = a + chunk < n ? a + chunk : n;
    std::vector<double> sum(b - a, 0.0);
    for (int t = 0; t < trees; ++t) {
      const Step* tree = steps.data() + (offsets[t] - offsets[0]);
      for (long long r = a; r < b; ++r) {
        const uint8_t* row = bins + static_cast<size_t>(r) * F;
        const Step* s = tree;
        while (s->feature >= 0) s = tree + s->child[row[s->feature] > s->bin];
        sum[r - a] += s->value;
      }
    }
    for (long long r = a; r < b; ++r) out[r] = static_cast<float>(sum[r - a]);
  });
  return 0;
}

// Isolation trees: out[r] = the sum over `trees` trees of (the number of cuts row r of X (float [n][F]) passes
// before it reaches a leaf + that leaf's `extra`).  Node tables as in mimir_cpu_trees_predict, but a node is
// (feature, threshold, left, right, extra) and a row goes left when its value is below the threshold (a NaN
// goes right).  Returns 0, or -1 for a table that is not a tree.
MIMIR_CPU_API int mimir_cpu_paths_sum(const float* X, int F, long long n, const double* nodes, const long long* offsets, int trees,
                                      float* out) {
  if (F < 1 || n < 0 || trees < 0) return -1;
  struct Cut { int32_t feature, child[2]; float threshold; double extra; };
  std::vector<Cut> cuts(trees > 0 ? static_cast<size_t>(offsets[trees] - offsets[0]) : 0);
  for (int t = 0; t < trees; ++t) {
    const long long lo = offsets[t], count = offsets[t + 1] - lo;
    if (count <= 0 || lo - offsets[0] < 0) return -1;
    for (long long i = 0; i < count; ++i) {
      const double* nd = nodes + static_cast<size_t>(lo + i) * 5;
      Cut& c = cuts[static_cast<size_t>(lo - offsets[0] + i)];
      c.feature = static_cast<int32_t>(nd[0]);
      c.threshold = static_cast<float>(nd[1]);
      c.child[0] = static_cast<int32_t>(nd[2]);
      c.child[1] = static_cast<int32_t>(nd[3]);
      c.extra = nd[4];
      if (c.feature >= F) return -1;
      if (c.feature >= 0 && (c.child[0] <= i || c.child[0] >= count || c.child[1] <= i || c.child[1] >= count)) return -1;
    }
  }
  std::lock_guard<std::mutex> lk(mimir_cpu::pool_mutex());
  mimir_cpu::Pool& pool = mimir_cpu::pool();
  const long long chunk = 1024, chunks = (n + chunk - 1) / chunk;
  for_each(pool, chunks, n * trees >= 65536, [&](long long c) {
    const long long a = c * chunk, b = a + chunk < n ? a + chunk : n;
    std::vector<double> sum(b - a, 0.0);
    for (int t = 0; t < trees; ++t) {
      const Cut* tree = cuts.data() + (offsets[t] - offsets[0]);
      for (long long r = a; r < b; ++r) {
        const float* row = X + static_cast<size_t>(r) * F;
        const Cut* s = tree;
        int depth = 0;
        while (s->feature >= 0) {
          s = tree + s->child[row[s->feature] < s->threshold ? 0 : 1];
          ++depth;
        }
        sum[r - a] += depth + s->extra;
      }
    }
    for (long long r = a; r < b; ++r) out[r] = static_cast<float>(sum[r - a]);
  });
  return 0;
}
