// Host-side builder of the blended-dataset index (no device code).
//
// Given the number of items to draw from each of n source datasets, emit (dataset, item) pairs so that after every
// step the dataset that lags furthest behind its target share comes next (ties: lowest dataset number).  Items of a
// dataset are emitted in order 0, 1, 2, ... (the sources are shuffled already).  Two stopping rules: the blend of
// src/scaling/core/data/blended_dataset.py:326-329 (the `blended_dataset_loop.sample` extension) runs until every
// dataset has reached its target, finished datasets dropping out of the choice (its tests expect as many items as
// the targets add up to); the Python loop of src/scaling/transformer/data/legacy_blended_dataset.py:214-229 stops
// when the first dataset reaches its target.  Computed with a heap in O(N log n) and exact integer comparisons
// instead of O(N n) floating-point argmin passes.
#include <cstdint>
#include <cstdio>
#include <queue>
#include <vector>

#include "common.cuh"

namespace {

struct Entry {
  int64_t sampled;
  int64_t target;
  int32_t dataset;
};
// a comes after b in the heap order when a's share sampled/target is larger, or equal with a larger dataset number
struct Later {
  bool operator()(const Entry& a, const Entry& b) const {
    const __int128 lhs = (__int128)a.sampled * b.target, rhs = (__int128)b.sampled * a.target;
    if (lhs != rhs) return lhs > rhs;
    return a.dataset > b.dataset;
  }
};

}  // namespace

// targets[n] > 0.  Writes int64 pairs (dataset, item) to `bin_path`; returns the number of pairs, or a negative
// value: -1 bad arguments, -2 the file cannot be written.
//   until_all != 0: go on until every dataset has reached its target; 0: stop at the first that does.
SB_API long sb200_blend_index_ex(const int64_t* targets, int n, const char* bin_path, int until_all) {
  if (!targets || n <= 0 || !bin_path) return -1;
  for (int i = 0; i < n; ++i)
    if (targets[i] <= 0) return -1;
  FILE* f = std::fopen(bin_path, "wb");
  if (!f) return -2;
  std::priority_queue<Entry, std::vector<Entry>, Later> heap;
  for (int i = 0; i < n; ++i) heap.push(Entry{0, targets[i], i});
  std::vector<int64_t> buffer;
  buffer.reserve(1 << 16);
  long count = 0;
  bool ok = true;
  while (!heap.empty()) {
    Entry e = heap.top();
    heap.pop();
    buffer.push_back(e.dataset);
    buffer.push_back(e.sampled);
    ++count;
    ++e.sampled;
    if (buffer.size() >= (1u << 16)) {
      ok = ok && std::fwrite(buffer.data(), sizeof(int64_t), buffer.size(), f) == buffer.size();
      buffer.clear();
    }
    if (e.sampled >= e.target) {
      if (!until_all) break;  // one dataset is exhausted: the blend ends here
      continue;               // this dataset is done, the others go on
    }
    heap.push(e);
  }
  if (!buffer.empty()) ok = ok && std::fwrite(buffer.data(), sizeof(int64_t), buffer.size(), f) == buffer.size();
  ok = (std::fclose(f) == 0) && ok;
  return ok ? count : -2;
}

// The first-exhausted rule under the earlier name.
SB_API long sb200_blend_index(const int64_t* targets, int n, const char* bin_path) {
  return sb200_blend_index_ex(targets, n, bin_path, 0);
}
