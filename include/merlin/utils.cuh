// Small helpers client code uses next to the table (reference:
// include/merlin/utils.cuh:127-135, 338-342).
#pragma once

#include <cooperative_groups.h>

#include <cstddef>
#include <cstdint>

// Functors written for export_batch_if_v2 / erase_if_v2 / for_each name the
// tile type as cg::thread_block_tile<GroupSize>; the reference provides this
// alias at global scope (include/merlin/utils.cuh:30).
namespace cg = cooperative_groups;

namespace nv {
namespace merlin {

// The 64-bit Murmur3 finaliser the table addresses buckets with.
inline uint64_t Murmur3HashHost(const uint64_t& key) {
  uint64_t h = key;
  h = (h ^ (h >> 33)) * UINT64_C(0xff51afd7ed558ccd);
  h = (h ^ (h >> 33)) * UINT64_C(0xc4ceb9fe1a85ec53);
  return h ^ (h >> 33);
}

inline constexpr size_t KB(size_t n) { return n << 10; }
inline constexpr size_t MB(size_t n) { return n << 20; }
inline constexpr size_t GB(size_t n) { return n << 30; }

}  // namespace merlin
}  // namespace nv
