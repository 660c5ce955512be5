// Segment reduction on the host (reference: tensor/segment.go, backend OpSegment): output row i
// combines the rows x[list[k]] for k in [offsets[i], offsets[i+1]), in the order of k, so the result
// is the same for any number of workers.  A sparse pattern's product, its transpose's product and the
// gather / scatter maps of a graph all are this one kernel with different lists.
#include <cstdint>
#include <cstring>
#include <mutex>

#include "cpu_pool.h"

#define MIMIR_CPU_API extern "C" __attribute__((visibility("default")))

namespace {

template <bool kMax>
void rows_range(const float* x, const int32_t* offsets, const int32_t* list, float* out, long long r0, long long r1,
                long long inner) {
  for (long long i = r0; i < r1; ++i) {
    float* o = out + i * inner;
    const int32_t a = offsets[i], b = offsets[i + 1];
    if (a >= b) {
      memset(o, 0, sizeof(float) * inner);
      continue;
    }
    memcpy(o, x + static_cast<long long>(list[a]) * inner, sizeof(float) * inner);
    for (int32_t k = a + 1; k < b; ++k) {
      const float* s = x + static_cast<long long>(list[k]) * inner;
      if (kMax) {
        // NaN propagates: (s > o) is false for a NaN s, so it is tested for by itself
        for (long long j = 0; j < inner; ++j) o[j] = (s[j] > o[j] || s[j] != s[j]) ? s[j] : o[j];
      } else {
        for (long long j = 0; j < inner; ++j) o[j] += s[j];
      }
    }
  }
}

}  // namespace

// x [n_in, inner] float32, offsets [n_out + 1], list [offsets[n_out]] with entries in [0, n_in);
// combine 0 = sum, 1 = max.  Returns 0, or -1 for arguments out of range (nothing is written then).
MIMIR_CPU_API int mimir_cpu_segment(const float* x, long long n_in, const int32_t* offsets, const int32_t* list,
                                    float* out, long long n_out, long long inner, int combine) {
  if (n_in < 0 || n_out < 0 || inner < 0 || (combine != 0 && combine != 1)) return -1;
  if (n_out == 0 || inner == 0) return 0;
  if (offsets[0] != 0) return -1;
  for (long long i = 0; i < n_out; ++i)
    if (offsets[i + 1] < offsets[i]) return -1;
  const long long entries = offsets[n_out];
  for (long long k = 0; k < entries; ++k)
    if (list[k] < 0 || list[k] >= n_in) return -1;
  auto range = [&](long long r0, long long r1) {
    if (combine == 1) rows_range<true>(x, offsets, list, out, r0, r1, inner);
    else rows_range<false>(x, offsets, list, out, r0, r1, inner);
  };
  const long long work = (entries + n_out) * inner;
  if (work < (1 << 15)) {
    range(0, n_out);
    return 0;
  }
  std::lock_guard<std::mutex> lk(mimir_cpu::pool_mutex());
  mimir_cpu::Pool& pool = mimir_cpu::pool();
  // rows are cut so that every part holds about the same number of entries
  pool.run([&](int part, int parts) {
    const long long lo = entries * part / parts, hi = entries * (part + 1) / parts;
    auto first_row_at = [&](long long e) {   // the first row whose entries start at or after e
      long long a = 0, b = n_out;
      while (a < b) {
        const long long m = (a + b) / 2;
        if (offsets[m] < e) a = m + 1; else b = m;
      }
      return a;
    };
    const long long r0 = part == 0 ? 0 : first_row_at(lo), r1 = part == parts - 1 ? n_out : first_row_at(hi);
    if (r0 < r1) range(r0, r1);
  });
  return 0;
}
