// Host post-processing utilities of the vision layer (fastdeploy/vision/utils/nms.cc:24-145, sort_det_res.cc:20-75,
// utils.h:33-54): greedy hard NMS over score-sorted boxes, stable arg-sort by score, top-k indices. Plain C ABI.
#include <algorithm>
#include <cstdint>
#include <numeric>
#include <vector>

#include "fdb_cpu.h"

namespace {

inline float iou_xyxy(const float* a, const float* b) {
  const float x1 = std::max(a[0], b[0]), y1 = std::max(a[1], b[1]);
  const float x2 = std::min(a[2], b[2]), y2 = std::min(a[3], b[3]);
  const float inter = std::max(x2 - x1, 0.f) * std::max(y2 - y1, 0.f);
  const float ua = (a[2] - a[0]) * (a[3] - a[1]) + (b[2] - b[0]) * (b[3] - b[1]) - inter;
  return inter / std::max(ua, 1e-12f);
}

}  // namespace

// Indices of the n scores in descending order; equal scores keep their input order.
FDB_CPU_API void fdv_argsort_desc(const float* scores, long long n, long long* order) {
  std::iota(order, order + n, 0LL);
  std::stable_sort(order, order + n, [&](long long a, long long b) { return scores[a] > scores[b]; });
}

// Greedy hard NMS: boxes [n][4] as (x1, y1, x2, y2), visited in descending score order (stable); a box is dropped
// when its IoU with an already kept box exceeds iou_threshold. Writes the kept input indices, in visiting order, to
// keep (room for n) and returns how many there are; at most max_keep when max_keep > 0.
FDB_CPU_API long long fdv_hard_nms(const float* boxes, const float* scores, long long n, float iou_threshold,
                                   long long max_keep, long long* keep) {
  if (n <= 0) return 0;
  std::vector<long long> order(static_cast<size_t>(n));
  fdv_argsort_desc(scores, n, order.data());
  std::vector<uint8_t> dead(static_cast<size_t>(n), 0);
  long long kept = 0;
  for (long long i = 0; i < n; ++i) {
    if (dead[i]) continue;
    const float* bi = boxes + order[i] * 4;
    keep[kept++] = order[i];
    if (max_keep > 0 && kept >= max_keep) break;
    for (long long j = i + 1; j < n; ++j) {
      if (!dead[j] && iou_xyxy(bi, boxes + order[j] * 4) > iou_threshold) dead[j] = 1;
    }
  }
  return kept;
}

// The k largest scores' indices in descending order (ties: lower index first); returns min(k, n).
FDB_CPU_API long long fdv_topk(const float* scores, long long n, long long k, long long* out) {
  if (n <= 0 || k <= 0) return 0;
  k = std::min(k, n);
  std::vector<long long> order(static_cast<size_t>(n));
  std::iota(order.begin(), order.end(), 0LL);
  std::partial_sort(order.begin(), order.begin() + k, order.end(), [&](long long a, long long b) {
    return scores[a] > scores[b] || (scores[a] == scores[b] && a < b);
  });
  std::copy(order.begin(), order.begin() + k, out);
  return k;
}
