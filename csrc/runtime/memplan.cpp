// Arena planning by liveness: greedy first-fit placement of buffers with [first, last] lifetimes into one arena.
//
// Buffers are placed in program order.  A buffer may share addresses with any buffer whose lifetime does not overlap
// its own; among the gaps between the live buffers (sorted by offset) it takes the lowest one that fits.  This is the
// planner behind compiled plans (the reference's `AllocationPlanner`); the Python package carries the same algorithm
// and a parity test keeps the two identical.
#include <algorithm>
#include <cstdint>
#include <utility>
#include <vector>

#define API extern "C" __attribute__((visibility("default")))

// sizes / first / last: n entries (sizes already aligned by the caller).  skip[i] != 0 leaves buffer i out (graph
// inputs own their memory): its offset is reported as -1.  Returns the arena size (peak), or -1 on bad arguments.
API int64_t incin_memplan_first_fit(int64_t n, const int64_t* sizes, const int64_t* first, const int64_t* last,
                                    const uint8_t* skip, int64_t* offsets_out) {
  if (n < 0 || !sizes || !first || !last || !offsets_out) return -1;
  struct Placed {
    int64_t off, size, first, last;
  };
  std::vector<Placed> placed;
  placed.reserve(static_cast<size_t>(n));
  std::vector<std::pair<int64_t, int64_t>> busy;
  int64_t peak = 0;
  for (int64_t i = 0; i < n; ++i) {
    if (skip && skip[i]) {
      offsets_out[i] = -1;
      continue;
    }
    if (sizes[i] < 0 || last[i] < first[i]) return -1;
    busy.clear();
    for (const Placed& p : placed)
      if (!(p.last < first[i] || p.first > last[i])) busy.emplace_back(p.off, p.size);
    std::sort(busy.begin(), busy.end());
    int64_t off = 0;
    for (const auto& b : busy) {
      if (off + sizes[i] <= b.first) break;
      off = std::max(off, b.first + b.second);
    }
    offsets_out[i] = off;
    placed.push_back({off, sizes[i], first[i], last[i]});
    peak = std::max(peak, off + sizes[i]);
  }
  return peak;
}
