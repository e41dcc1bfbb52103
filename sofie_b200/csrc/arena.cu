// Lifetime-aware placement of pooled tensors in one device arena.
//
// Policy of the reference planner (OrganizeMemory, core/inc/SOFIE/utils/shared/MemoryPlanner.inc:47-132):
// walk the lifetimes in time order, releasing before allocating at equal times; an allocation
// takes the smallest free block that fits (lowest offset among equals) and splits it, or grows
// the arena at its end; a released block merges with free neighbours.  Sizes are rounded up to
// 256 bytes, the alignment the reference applies to every arena region (core/src/RModel_ALPAKA.cxx:25).
// Host-only code; it lives in the CUDA library because the emitted Session calls it at
// construction, next to the plan-creation calls.
#include <algorithm>
#include <map>

#include "common.cuh"

namespace {

struct Event {
  int64_t t;
  int kind;  // 0 release, 1 allocate
  int64_t idx;
};

class FreeList {
 public:
  // smallest block with size >= need, lowest offset among equals; -1 if none
  int64_t take(int64_t need) {
    auto best = blocks_.end();
    for (auto it = blocks_.begin(); it != blocks_.end(); ++it)
      if (it->second >= need && (best == blocks_.end() || it->second < best->second)) best = it;
    if (best == blocks_.end()) return -1;
    const int64_t off = best->first, size = best->second;
    blocks_.erase(best);
    if (size > need) blocks_[off + need] = size - need;
    return off;
  }
  void give(int64_t off, int64_t size) {
    auto it = blocks_.emplace(off, size).first;
    if (it != blocks_.begin()) {
      auto prev = std::prev(it);
      if (prev->first + prev->second == it->first) {
        prev->second += it->second;
        blocks_.erase(it);
        it = prev;
      }
    }
    auto next = std::next(it);
    if (next != blocks_.end() && it->first + it->second == next->first) {
      it->second += next->second;
      blocks_.erase(next);
    }
  }

 private:
  std::map<int64_t, int64_t> blocks_;  // offset -> size
};

}  // namespace

extern "C" int sofie_b200_plan_arena(const sofie_b200_tensor_life *lives, int64_t n, int64_t *offsets,
                                     int64_t *total_bytes) {
  using sb200::fail;
  if (n < 0 || (n > 0 && (!lives || !offsets)) || !total_bytes)
    return fail(SOFIE_B200_ERR_INVALID, "plan_arena: NULL argument");
  std::vector<Event> ev;
  ev.reserve((size_t)n * 2);
  for (int64_t i = 0; i < n; ++i) {
    if (!(lives[i].end > lives[i].begin))
      return fail(SOFIE_B200_ERR_INVALID, "plan_arena: tensor %lld must have end > begin", (long long)i);
    if (lives[i].size < 0) return fail(SOFIE_B200_ERR_INVALID, "plan_arena: tensor %lld has a negative size", (long long)i);
    ev.push_back({lives[i].end, 0, i});
    ev.push_back({lives[i].begin, 1, i});
  }
  std::stable_sort(ev.begin(), ev.end(), [](const Event &a, const Event &b) {
    if (a.t != b.t) return a.t < b.t;
    return a.kind < b.kind;
  });
  FreeList fl;
  int64_t total = 0;
  std::vector<int64_t> rounded((size_t)n);
  for (int64_t i = 0; i < n; ++i) rounded[i] = (lives[i].size + 255) / 256 * 256;
  for (const Event &e : ev) {
    if (e.kind == 0) {
      if (rounded[e.idx] > 0) fl.give(offsets[e.idx], rounded[e.idx]);
    } else {
      const int64_t need = rounded[e.idx];
      int64_t off = need > 0 ? fl.take(need) : total;
      if (off < 0) {
        off = total;
        total += need;
      }
      offsets[e.idx] = off;
    }
  }
  *total_bytes = total;
  return 0;
}
