// Lifetime-aware placement of pooled tensors in one arena (host code, header-only).
//
// One implementation serves both the code generator (RModel::GenerateGPU_B200 plans the arena of
// the Session it emits) and the runtime library (sofie_b200_plan_arena).  Policy of the reference
// planner OrganizeMemory (core/inc/SOFIE/utils/shared/MemoryPlanner.inc:47-132): walk the
// lifetimes in time order, releasing before allocating at equal times; an allocation takes the
// smallest free block that fits (lowest offset among equals) and splits it, else grows the arena
// at its end; a released block merges with free neighbours.  Sizes are rounded up to 256 bytes, the
// alignment the reference applies to every arena region (core/src/RModel_ALPAKA.cxx:25).
#pragma once
#include <algorithm>
#include <cstdint>
#include <map>
#include <stdexcept>
#include <vector>

namespace SOFIE_B200 {

struct TensorLifeInfo {
   int64_t begin;  // first operator step that writes the tensor
   int64_t end;    // one past the last step that reads it
   int64_t size;   // bytes
};

struct MemoryResult {
   int64_t total_bytes = 0;
   std::vector<int64_t> offsets;
   // free space inside the footprint at the moment it last grew (the reference snapshots the same two figures there,
   // MemoryPlanner.inc:119-126, and the emitted Session reports them and the fragmentation derived from them)
   int64_t total_free_bytes = 0;
   int64_t largest_free_block = 0;
};

constexpr int64_t kArenaAlignment = 256;

inline int64_t AlignUp(int64_t n, int64_t a = kArenaAlignment) { return (n + a - 1) / a * a; }
// AlignUp of "a * n + b" with n unknown until the Session is constructed: both parts are rounded, so the sum is aligned
// for every n (symbolicBase: the number that stands for n, a multiple of the alignment; 0 = no symbolic sizes)
inline int64_t AlignUpSymbolic(int64_t v, int64_t symbolicBase)
{
   if (symbolicBase <= 0 || v < symbolicBase / 2) return AlignUp(v);
   const int64_t a = (v + symbolicBase / 2) / symbolicBase, b = v - a * symbolicBase;
   return AlignUp(a) * symbolicBase + AlignUp(b < 0 ? 0 : b);
}

namespace memory_detail {

class FreeList {
public:
   // smallest block with size >= need, lowest offset among equals; -1 if none
   int64_t Take(int64_t need)
   {
      auto best = fBlocks.end();
      for (auto it = fBlocks.begin(); it != fBlocks.end(); ++it)
         if (it->second >= need && (best == fBlocks.end() || it->second < best->second))
            best = it;
      if (best == fBlocks.end())
         return -1;
      const int64_t off = best->first, size = best->second;
      fBlocks.erase(best);
      if (size > need)
         fBlocks[off + need] = size - need;
      return off;
   }
   void Give(int64_t off, int64_t size)
   {
      auto it = fBlocks.emplace(off, size).first;
      if (it != fBlocks.begin()) {
         auto prev = std::prev(it);
         if (prev->first + prev->second == it->first) {
            prev->second += it->second;
            fBlocks.erase(it);
            it = prev;
         }
      }
      auto next = std::next(it);
      if (next != fBlocks.end() && it->first + it->second == next->first) {
         it->second += next->second;
         fBlocks.erase(next);
      }
   }

   void Stats(int64_t &total, int64_t &largest) const
   {
      total = largest = 0;
      for (auto &b : fBlocks) { total += b.second; largest = std::max(largest, b.second); }
   }

private:
   std::map<int64_t, int64_t> fBlocks;  // offset -> size
};

struct Event {
   int64_t t;
   int kind;  // 0 release, 1 allocate
   int64_t idx;
};

}  // namespace memory_detail

inline MemoryResult OrganizeMemory(const std::vector<TensorLifeInfo> &tensors)
{
   using memory_detail::Event;
   std::vector<Event> ev;
   ev.reserve(tensors.size() * 2);
   for (size_t i = 0; i < tensors.size(); ++i) {
      if (!(tensors[i].end > tensors[i].begin))
         throw std::runtime_error("Each tensor must have end > begin.");
      if (tensors[i].size < 0)
         throw std::runtime_error("Tensor sizes must not be negative.");
      ev.push_back({tensors[i].end, 0, int64_t(i)});
      ev.push_back({tensors[i].begin, 1, int64_t(i)});
   }
   std::stable_sort(ev.begin(), ev.end(), [](const Event &a, const Event &b) {
      if (a.t != b.t)
         return a.t < b.t;
      return a.kind < b.kind;
   });
   MemoryResult res;
   res.offsets.assign(tensors.size(), 0);
   memory_detail::FreeList fl;
   for (const Event &e : ev) {
      const int64_t need = AlignUp(tensors[e.idx].size);
      if (e.kind == 0) {
         if (need > 0)
            fl.Give(res.offsets[e.idx], need);
      } else {
         int64_t off = need > 0 ? fl.Take(need) : res.total_bytes;
         if (off < 0) {
            off = res.total_bytes;
            res.total_bytes += need;
            fl.Stats(res.total_free_bytes, res.largest_free_block);
         }
         res.offsets[e.idx] = off;
      }
   }
   return res;
}

}  // namespace SOFIE_B200
