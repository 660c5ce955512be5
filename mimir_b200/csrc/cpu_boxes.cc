// Greedy non-maximum suppression on the host (reference: vision/boxes.go): boxes are visited by falling score
// and one is kept unless a kept box overlaps it by more than the threshold.  Each candidate is compared with
// the boxes kept so far, so no n x n table of overlaps is made.
#include <cstdint>
#include <vector>

#define MIMIR_CPU_API extern "C" __attribute__((visibility("default")))

// boxes: float [n][4] = x1, y1, x2, y2; order: int64 [n], the boxes by falling score; keep: int64 [n] receives
// the kept boxes in that order.  Returns how many were kept, or -1.
MIMIR_CPU_API long long mimir_cpu_nms(const float* boxes, const int64_t* order, long long n, float threshold, int64_t* keep) {
  if (n < 0) return -1;
  std::vector<float> kept;        // x1, y1, x2, y2, area of each kept box, side by side
  kept.reserve(256 * 5);
  long long count = 0;
  for (long long k = 0; k < n; ++k) {
    const int64_t i = order[k];
    if (i < 0 || i >= n) return -1;
    const float* b = boxes + static_cast<size_t>(i) * 4;
    const float w = b[2] - b[0], h = b[3] - b[1];
    const float area = (w > 0 ? w : 0) * (h > 0 ? h : 0);
    bool gone = false;
    for (size_t q = 0; q < kept.size(); q += 5) {
      const float x1 = b[0] > kept[q] ? b[0] : kept[q], y1 = b[1] > kept[q + 1] ? b[1] : kept[q + 1];
      const float x2 = b[2] < kept[q + 2] ? b[2] : kept[q + 2], y2 = b[3] < kept[q + 3] ? b[3] : kept[q + 3];
      const float iw = x2 - x1, ih = y2 - y1;
      if (iw <= 0 || ih <= 0) continue;
      const float inter = iw * ih, uni = area + kept[q + 4] - inter;
      if (inter / (uni > 1e-9f ? uni : 1e-9f) > threshold) { gone = true; break; }
    }
    if (gone) continue;
    kept.insert(kept.end(), {b[0], b[1], b[2], b[3], area});
    keep[count++] = i;
  }
  return count;
}
