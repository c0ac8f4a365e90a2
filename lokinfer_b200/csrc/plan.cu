// Memory planner of the activation arena (host code; no device work): the counterpart, for one device and one program,
// of the reference's planner (src/compiler/plan_memory.cpp: liveness over the program, offsets into an arena;
// src/runtime/executable.cpp:732-815 allocates the arena once). The program here is the traced op sequence of a
// forward that forks into several streams, so "may still be in use" is decided with vector clocks and not with
// program order: tensor p blocks its byte range for a later allocation a unless every use of p happens-before a,
// i.e. unless last_use[p][s] <= alloc_clock[a][s] on every stream s (same stream, or separated by a join).
// Placement is greedy: allocations in program order, each at the lowest offset that is free of blocking tensors.
#include <algorithm>
#include <utility>
#include <vector>

#include "lkc_common.h"

// n tensors in allocation order, S streams. bytes[i]; pinned[i] != 0: never reused; alloc_clock[i * S + s]: the vector
// clock of the allocating stream when tensor i was allocated; last_use[i * S + s]: the largest count of stream s at
// which tensor i was used (its allocation included; 0 = never on that stream). align: power of two. Writes
// offsets[i] and *total (arena bytes). Returns 0, or non-zero with lkc_last_error() on bad arguments.
extern "C" LKC_API int lkc_plan_memory(int64_t n, int64_t num_streams, const int64_t* bytes, const int32_t* pinned,
                                       const int64_t* alloc_clock, const int64_t* last_use, int64_t align,
                                       int64_t* offsets, int64_t* total) {
  LKC_REQUIRE(n >= 0 && num_streams >= 1 && align >= 1 && (align & (align - 1)) == 0, "plan_memory: bad sizes");
  LKC_REQUIRE(n == 0 || (bytes && pinned && alloc_clock && last_use && offsets), "plan_memory: null array");
  LKC_REQUIRE(total, "plan_memory: null total");
  const int64_t S = num_streams;
  std::vector<int64_t> size(static_cast<size_t>(n));
  std::vector<std::pair<int64_t, int64_t>> busy;
  int64_t top = 0;
  for (int64_t i = 0; i < n; ++i) {
    LKC_REQUIRE(bytes[i] >= 0, "plan_memory: negative size");
    size[i] = (bytes[i] + align - 1) / align * align;
    busy.clear();
    for (int64_t p = 0; p < i; ++p) {
      bool before = pinned[p] == 0;
      for (int64_t s = 0; before && s < S; ++s) before = last_use[p * S + s] <= alloc_clock[i * S + s];
      if (!before) busy.emplace_back(offsets[p], offsets[p] + size[p]);
    }
    std::sort(busy.begin(), busy.end());
    int64_t off = 0;
    for (const auto& b : busy) {
      if (off + size[i] <= b.first) break;
      if (b.second > off) off = b.second;
    }
    offsets[i] = off;
    top = std::max(top, off + size[i]);
  }
  *total = top;
  return 0;
}
