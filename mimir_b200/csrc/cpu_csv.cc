// Numeric CSV bodies parsed on the host (reference: data/datasets CSV and CSVShards readers): the bytes of a file
// are cut at line ends into pieces, the pieces' lines are counted, and every piece is parsed by a worker into
// its rows of the output table.
#include <atomic>
#include <charconv>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <mutex>
#include <vector>

#include "cpu_pool.h"

#define MIMIR_CPU_API extern "C" __attribute__((visibility("default")))

namespace {

struct Piece { const char* lo; const char* hi; long long rows; };

inline bool blank(const char* a, const char* b) {
  for (; a < b; ++a)
    if (*a != ' ' && *a != '\t' && *a != '\r') return false;
  return true;
}

// the lines of [lo, hi) that hold something
long long count_lines(const char* lo, const char* hi) {
  long long n = 0;
  while (lo < hi) {
    const char* e = static_cast<const char*>(memchr(lo, '\n', hi - lo));
    if (!e) e = hi;
    if (!blank(lo, e)) ++n;
    lo = e + 1;
  }
  return n;
}

// one field [a, b) as a number; an empty field is NaN.  False when it is not a plain number.
bool field(const char* a, const char* b, double* out) {
  while (a < b && (*a == ' ' || *a == '\t')) ++a;
  while (b > a && (b[-1] == ' ' || b[-1] == '\t' || b[-1] == '\r')) --b;
  if (a == b) { *out = std::numeric_limits<double>::quiet_NaN(); return true; }
  if (*a == '+') ++a;
  const auto r = std::from_chars(a, b, *out);
  return r.ec == std::errc() && r.ptr == b;
}

}  // namespace

// The number of lines of buf [len] that hold something (a header line counts).
MIMIR_CPU_API long long mimir_cpu_csv_lines(const char* buf, long long len) { return len < 0 ? -1 : count_lines(buf, buf + len); }

// Parses the lines of buf [len] (comma-separated plain numbers, no quotes; an empty field is NaN; blank lines
// are skipped) into out: double [rows][cols], rows = mimir_cpu_csv_lines(buf, len).  Returns the rows written,
// or -(line number) - 1, counted over the lines that hold something, for the first line the worker that met it
// could not read (a field that is not a number, too few or too many fields): the caller then falls back to a
// general reader.
MIMIR_CPU_API long long mimir_cpu_csv_parse(const char* buf, long long len, int cols, double* out, long long rows) {
  if (len < 0 || cols < 1 || rows < 0) return -1;
  std::lock_guard<std::mutex> lk(mimir_cpu::pool_mutex());
  mimir_cpu::Pool& pool = mimir_cpu::pool();
  const int want = len >= (1 << 20) ? pool.size() * 4 : 1;
  std::vector<Piece> pieces;
  const char* end = buf + len;
  const char* lo = buf;
  for (int p = 0; p < want && lo < end; ++p) {
    const char* hi = p + 1 == want ? end : buf + len / want * (p + 1);
    if (hi < lo) hi = lo;
    if (hi < end) {
      const char* e = static_cast<const char*>(memchr(hi, '\n', end - hi));
      hi = e ? e + 1 : end;
    }
    pieces.push_back({lo, hi, 0});
    lo = hi;
  }
  std::atomic<long long> next{0};
  const long long n = static_cast<long long>(pieces.size());
  auto count = [&](int, int) {
    for (long long i = next.fetch_add(1); i < n; i = next.fetch_add(1)) pieces[i].rows = count_lines(pieces[i].lo, pieces[i].hi);
  };
  if (n > 1) pool.run_shared(count); else count(0, 1);
  std::vector<long long> first(n + 1, 0);
  for (long long i = 0; i < n; ++i) first[i + 1] = first[i] + pieces[i].rows;
  if (first[n] != rows) return -1;
  std::atomic<long long> bad{std::numeric_limits<long long>::max()};
  next.store(0);
  auto parse = [&](int, int) {
    for (long long i = next.fetch_add(1); i < n; i = next.fetch_add(1)) {
      long long row = first[i];
      const char* a = pieces[i].lo;
      while (a < pieces[i].hi) {
        const char* e = static_cast<const char*>(memchr(a, '\n', pieces[i].hi - a));
        if (!e) e = pieces[i].hi;
        if (!blank(a, e)) {
          double* dst = out + static_cast<size_t>(row) * cols;
          int c = 0;
          bool ok = true;
          const char* f = a;
          while (ok) {
            const char* comma = static_cast<const char*>(memchr(f, ',', e - f));
            const char* fe = comma ? comma : e;
            if (c >= cols || !field(f, fe, dst + c)) { ok = false; break; }
            ++c;
            if (!comma) break;
            f = comma + 1;
          }
          if (!ok || c != cols) {
            long long seen = bad.load();
            while (row < seen && !bad.compare_exchange_weak(seen, row)) {}
            break;
          }
          ++row;
        }
        a = e + 1;
      }
    }
  };
  if (n > 1) pool.run_shared(parse); else parse(0, 1);
  const long long b = bad.load();
  return b == std::numeric_limits<long long>::max() ? rows : -b - 1;
}
