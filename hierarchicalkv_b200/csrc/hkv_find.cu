// Read-only lookups: find (values / pointers / missed-keys form) and contains.
//
// Replaces the reference's lookup kernels
//   include/merlin/core_kernels/lookup.cuh:119-378   (pipeline find)
//   include/merlin/core_kernels/lookup.cuh:873-925   (tile find)
//   include/merlin/core_kernels/lookup_ptr.cuh:26-152 (find*)
//   include/merlin/core_kernels/contains.cuh:46-214  (contains)
// with one warp kernel: 8-lane digest probe of 32 keys with every digest line
// and every first-candidate key load in flight at once, then a
// warp-cooperative streaming gather of the hit rows.
#include <cub/device/device_radix_sort.cuh>

#include <cstdlib>

#include "hkv_device.cuh"
#include "hkv_internal.h"

namespace hkv {

namespace {

constexpr int kFindBlock = 128;
#ifndef HKV_FIND_MIN_BLOCKS
#define HKV_FIND_MIN_BLOCKS 8
#endif
constexpr int kFindMinBlocks = HKV_FIND_MIN_BLOCKS;  // resident blocks per SM asked of the compiler
#ifndef HKV_FIND_LIGHT_MIN_BLOCKS
#define HKV_FIND_LIGHT_MIN_BLOCKS 8
#endif
// the forms that move no rows (find*, contains, the probe step of the hybrid find)
constexpr int kFindLightMinBlocks = HKV_FIND_LIGHT_MIN_BLOCKS;

// Probes the 32 keys of a warp.  Returns in the owner lane the global slot of
// its key, or kNoSlot.
__device__ __forceinline__ uint32_t warp_probe_readonly(const TableView& t, const ProbeLane& pl,
                                                        uint64_t key, bool valid,
                                                        const Address& a) {
  const uint32_t full = 0xFFFFFFFFu;
  const uint32_t my_bucket = static_cast<uint32_t>(a.bucket);
  uint4 dg[kPasses];
  uint32_t bkt[kPasses];
  bool act[kPasses];
#pragma unroll
  for (int j = 0; j < kPasses; ++j) {
    const uint32_t owner = pass_owner(j, pl.group);
    bkt[j] = __shfl_sync(full, my_bucket, owner);
    act[j] = __shfl_sync(full, valid ? 1u : 0u, owner) != 0u;
    dg[j] = make_uint4(0, 0, 0, 0);
    if (act[j]) {
      dg[j] = ld_meta_v4(t.digests + (uint64_t(bkt[j]) << 7) + pl.sub * 16u);
    }
  }
  uint32_t cand[kPasses];
  uint64_t first_key[kPasses];
#pragma unroll
  for (int j = 0; j < kPasses; ++j) {
    const uint32_t owner = pass_owner(j, pl.group);
    const uint32_t tgt = __shfl_sync(full, a.digest, owner);
    cand[j] = act[j] ? match16(dg[j], replicate4(tgt)) : 0u;
    first_key[j] = 0;
    if (cand[j]) {
      const uint32_t pos = pl.sub * 16u + (__ffs(cand[j]) - 1);
      first_key[j] = ld_meta_u64(key_ptr_in_line_bucket(t, bkt[j], pos));
    }
  }
  uint32_t my_slot = kNoSlot;
#pragma unroll
  for (int j = 0; j < kPasses; ++j) {
    const uint32_t owner = pass_owner(j, pl.group);
    const uint64_t want = __shfl_sync(full, key, owner);
    uint32_t hit_slot = kNoSlot;
    if (cand[j]) {
      uint32_t m = cand[j];
      uint32_t pos = pl.sub * 16u + (__ffs(m) - 1);
      if (first_key[j] == want) {
        hit_slot = (bkt[j] << 7) + pos;
      } else {
        m &= m - 1;
        while (m) {
          pos = pl.sub * 16u + (__ffs(m) - 1);
          m &= m - 1;
          if (ld_meta_u64(key_ptr_in_line_bucket(t, bkt[j], pos)) == want) {
            hit_slot = (bkt[j] << 7) + pos;
            break;
          }
        }
      }
    }
    const uint32_t votes = (__ballot_sync(full, hit_slot != kNoSlot) >> (pl.group * 8u)) & 0xFFu;
    const uint32_t src = votes ? (pl.group * 8u + (__ffs(votes) - 1)) : pl.lane;
    const uint32_t group_slot = __shfl_sync(full, hit_slot, src);
    // hand the result to the owner lane: owner of (j, g) is lane 4j + g
    const uint32_t got = __shfl_sync(full, group_slot, (pl.lane & 3u) * 8u);
    if ((pl.lane >> 2) == uint32_t(j)) my_slot = got;
  }
  return my_slot;
}

// FORM 0: values + founds (+scores)       (HashTable::find, merlin_hashtable.cuh:2464)
// FORM 1: value pointers + founds (+scores) (find*, merlin_hashtable.cuh:2729)
// FORM 2: values + missed keys/indices/size (merlin_hashtable.cuh:2600)
// FORM 3: founds only                     (contains, merlin_hashtable.cuh:2856)
// FORM 4: founds (+scores) and, per key, the place of its row and its batch
//         index: the first step of find on a table whose rows partly live in
//         host memory
template <int FORM, int VEC>
__global__ void __launch_bounds__(kFindBlock, (FORM == 1 || FORM == 3 || FORM == 4)
                                                  ? kFindLightMinBlocks
                                                  : kFindMinBlocks)
    find_kernel(const TableView t, const uint64_t* __restrict__ keys, const uint64_t n,
                uint8_t* __restrict__ values, void** __restrict__ ptrs, bool* __restrict__ founds,
                uint64_t* __restrict__ scores, uint64_t* __restrict__ missed_keys,
                int* __restrict__ missed_indices, int* __restrict__ missed_size,
                uint32_t* __restrict__ slot_out, uint32_t* __restrict__ index_out) {
  const ProbeLane pl = probe_lane();
  const uint64_t warp = (uint64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const uint64_t base = warp * 32u;
  if (base >= n) return;
  const uint64_t i = base + pl.lane;
  uint64_t key = 0;
  bool valid = false;
  if (i < n) {
    key = keys[i];
    valid = !is_reserved(t, key);
  }
  Address a{0, 0, 0};
  if (valid) a = locate_line(t, key);

  const uint32_t slot = warp_probe_readonly(t, pl, key, valid, a);
  const bool found = slot != kNoSlot;

  if (i < n) {
    if (FORM != 2) founds[i] = found;
    if (FORM == 1) ptrs[i] = found ? row_ptr(t, slot) : nullptr;
    if (FORM != 3 && scores != nullptr && found) scores[i] = *score_ptr(t, slot);
    if (FORM == 4) {
      // where the row lives (kNoSlot sorts behind every real place)
      slot_out[i] = found ? static_cast<uint32_t>(row_slot(t, slot)) : kNoSlot;
      index_out[i] = static_cast<uint32_t>(i);
    }
    // hybrid tables (they never run the VEC != 0 instantiations): hits per
    // bucket, sampled (every fourth key of a batch) to keep the atomics on the
    // hot buckets' counters cheap -- the promotion only ranks buckets
    if (VEC == 0 && FORM != 3 && found && t.bucket_heat != nullptr && (uint32_t(i) & 3u) == 0) {
      atomicAdd(t.bucket_heat + (slot >> 7), 1u);
    }
  }
  if (FORM == 2) {
    const bool missed = (i < n) && !found;
    const uint32_t mm = __ballot_sync(0xFFFFFFFFu, missed);
    if (mm) {
      int at = 0;
      if (pl.lane == 0) at = atomicAdd(missed_size, __popc(mm));
      at = __shfl_sync(0xFFFFFFFFu, at, 0);
      if (missed) {
        const int mine = at + __popc(mm & ((1u << pl.lane) - 1u));
        missed_keys[mine] = key;
        missed_indices[mine] = static_cast<int>(i);
      }
    }
  }
  if (FORM == 0 || FORM == 2) {
    if (values != nullptr) {
      warp_move_rows<0, VEC>(t, values + base * t.row_bytes, slot, pl.lane);
    }
  }
}

// find for the key-hash sharded table: this rank is the owner, the keys came
// from `world` source ranks (one inbox segment each), and every hit row goes
// directly to the source rank's result buffer over NVLink (plain peer stores)
// while the next buckets are being probed -- lookup and transfer are one kernel.
template <int VEC>
__global__ void __launch_bounds__(kFindBlock)
    find_routed_kernel(const TableView t, const uint32_t world,
                       const uint32_t first_segment, const uint64_t segment_capacity, const uint64_t* __restrict__ inbox_keys,
                       const uint32_t* __restrict__ inbox_origin,
                       const uint64_t* __restrict__ inbox_counts, const PeerPtrs out_values,
                       const PeerPtrs out_founds, const bool writers_fence) {
  // The key counts are only known on the device, so the grid covers every
  // segment's full capacity and blocks beyond a segment's count leave at once.
  const ProbeLane pl = probe_lane();
  // Consecutive blocks serve different source ranks (block b: the b % world-th
  // rank after this one), so at every moment an owner stores into all
  // requesters at once -- its own buffer included -- instead of saturating one
  // NVLink destination while its HBM idles, and no requester's ingress has all
  // owners converging on it.
  const uint32_t turn = blockIdx.x % world;
  uint32_t seg = turn + first_segment;
  seg = seg >= world ? seg - world : seg;
  const uint64_t base = uint64_t(blockIdx.x / world) * kFindBlock + (threadIdx.x & ~31u);
  const uint64_t count = inbox_counts[seg];
  if (base >= count) return;
  uint8_t* values_of = nullptr;
  uint8_t* founds_of = nullptr;
#pragma unroll
  for (int s = 0; s < kMaxPeers; ++s) {
    if (uint32_t(s) == seg) {
      values_of = static_cast<uint8_t*>(out_values.p[s]);
      founds_of = static_cast<uint8_t*>(out_founds.p[s]);
    }
  }
  const uint64_t in_seg = base + pl.lane;
  const bool present = in_seg < count;
  uint64_t key = 0;
  uint32_t origin = 0;
  bool valid = false;
  if (present) {
    key = inbox_keys[seg * segment_capacity + in_seg];
    origin = inbox_origin[seg * segment_capacity + in_seg];
    valid = !is_reserved(t, key);
  }
  Address a{0, 0, 0};
  if (valid) a = locate_line(t, key);
  const uint32_t slot = warp_probe_readonly(t, pl, key, valid, a);
  if (present) founds_of[origin] = slot != kNoSlot ? 1 : 0;
  warp_gather_rows_to<VEC>(t, values_of, origin, slot, pl.lane);
  // Rows and flags went to other GPUs; the barrier kernel that follows orders
  // them before its flags with a system-scope fence of its own.  The strict
  // form, in which every storing thread also fences its own stores before it
  // leaves, costs 14 % of the two-GPU lookup and is off unless asked for.
  if (writers_fence) __threadfence_system();
}

// find on a dual-bucket table (include/merlin/core_kernels/dual_bucket_lookup.cuh):
// the first bucket of every key is probed, then the second bucket of the keys
// that were not there.
__global__ void __launch_bounds__(kFindBlock)
    dual_find_kernel(const TableView t, const uint64_t* __restrict__ keys, const uint64_t n,
                     uint8_t* __restrict__ values, bool* __restrict__ founds,
                     uint64_t* __restrict__ scores) {
  const ProbeLane pl = probe_lane();
  const uint64_t warp = (uint64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const uint64_t base = warp * 32u;
  if (base >= n) return;
  const uint64_t i = base + pl.lane;
  uint64_t key = 0;
  bool valid = false;
  if (i < n) {
    key = keys[i];
    valid = !is_reserved(t, key);
  }
  DualAddress a{};
  if (valid) a = locate_dual(t, key);
  uint32_t slot = warp_probe_readonly(t, pl, key, valid, a.first);
  const bool again = valid && slot == kNoSlot;
  if (__ballot_sync(0xFFFFFFFFu, again)) {
    const uint32_t second = warp_probe_readonly(t, pl, key, again, a.second);
    if (again) slot = second;
  }
  const bool found = slot != kNoSlot;
  if (i < n) {
    founds[i] = found;
    if (scores != nullptr && found) scores[i] = *score_ptr(t, slot);
  }
  if (values != nullptr) warp_move_rows<0>(t, values + base * t.row_bytes, slot, pl.lane);
}

// Lookups on a table whose buckets are not one 128-byte digest line
// (max_bucket_size of 16 ... 1024 other than 128; the reference serves them
// with its tile kernels, include/merlin/core_kernels/lookup.cuh:873-925): one
// warp per key walks the bucket's digests four per lane and 128 per step,
// verifies the candidates' keys and copies the row with all 32 lanes.  Same
// forms as find_kernel.
template <int FORM>
__global__ void __launch_bounds__(kFindBlock)
    find_generic_kernel(const TableView t, const uint64_t* __restrict__ keys, const uint64_t n,
                        uint8_t* __restrict__ values, void** __restrict__ ptrs,
                        bool* __restrict__ founds, uint64_t* __restrict__ scores,
                        uint64_t* __restrict__ missed_keys, int* __restrict__ missed_indices,
                        int* __restrict__ missed_size) {
  const uint32_t lane = threadIdx.x & 31u;
  const uint64_t i = (uint64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (i >= n) return;
  const uint64_t key = keys[i];
  uint32_t slot = kNoSlot;
  if (!is_reserved(t, key)) {
    const Address a = locate(t, key);
    const uint64_t slot0 = a.bucket << t.bucket_shift;
    const uint32_t pattern = replicate4(a.digest);
    for (uint32_t first = 0; first < t.bucket_slots && slot == kNoSlot; first += 128u) {
      const uint32_t at = first + lane * 4u;
      uint32_t hit = kNoSlot;
      if (at < t.bucket_slots) {
        uint32_t m = match4(*reinterpret_cast<const uint32_t*>(t.digests + slot0 + at), pattern);
        while (m) {
          const uint32_t pos = at + (__ffs(m) - 1);
          m &= m - 1;
          if (ld_relaxed(key_ptr(t, slot0 + pos)) == key) {
            hit = uint32_t(slot0) + pos;
            break;
          }
        }
      }
      const uint32_t votes = __ballot_sync(0xFFFFFFFFu, hit != kNoSlot);
      if (votes) slot = __shfl_sync(0xFFFFFFFFu, hit, __ffs(votes) - 1);
    }
  }
  const bool found = slot != kNoSlot;
  if (lane == 0) {
    if (FORM != 2) founds[i] = found;
    if (FORM == 1) ptrs[i] = found ? row_ptr(t, slot) : nullptr;
    if (FORM != 3 && scores != nullptr && found) scores[i] = *score_ptr(t, slot);
    if (FORM != 3 && found && t.bucket_heat != nullptr && (uint32_t(i) & 3u) == 0) {
      atomicAdd(t.bucket_heat + (slot >> t.bucket_shift), 1u);
    }
    if (FORM == 2 && !found) {
      const int at = atomicAdd(missed_size, 1);
      missed_keys[at] = key;
      missed_indices[at] = static_cast<int>(i);
    }
  }
  if ((FORM == 0 || FORM == 2) && found && values != nullptr) {
    warp_copy_one_row<0>(t, values + i * t.row_bytes, row_ptr(t, slot), lane);
  }
}

template <int FORM>
void launch_form(const TableView& t, uint64_t n, const uint64_t* keys, void* values, void** ptrs,
                 bool* founds, uint64_t* scores, uint64_t* missed_keys, int* missed_indices,
                 int* missed_size, cudaStream_t stream) {
  if (n == 0) return;
  if (!line_buckets(t)) {
    const uint64_t blocks = (n * 32 + kFindBlock - 1) / kFindBlock;
    find_generic_kernel<FORM><<<static_cast<unsigned>(blocks), kFindBlock, 0, stream>>>(
        t, keys, n, static_cast<uint8_t*>(values), ptrs, founds, scores, missed_keys,
        missed_indices, missed_size);
    return;
  }
  const uint64_t warps = (n + 31) / 32;
  const uint64_t blocks = (warps * 32 + kFindBlock - 1) / kFindBlock;
  auto kernel = fast_rows(t) ? find_kernel<FORM, 16> : find_kernel<FORM, 0>;
  kernel<<<static_cast<unsigned>(blocks), kFindBlock, 0, stream>>>(
      t, keys, n, static_cast<uint8_t*>(values), ptrs, founds, scores, missed_keys, missed_indices,
      missed_size, nullptr, nullptr);
}

// Second step of the hybrid find: (slot, batch index) pairs sorted by slot.
// A warp takes 32 pairs and gathers their rows into the caller's buffer at
// the keys' own positions.  Sorted order makes the reads of host-resident
// rows walk host memory monotonically and puts repeated keys next to each
// other, which is what the host link and its address translation want (the
// reference sorts row addresses for the same reason,
// include/merlin_hashtable.cuh:2562-2572).
__global__ void __launch_bounds__(kFindBlock)
    gather_sorted_kernel(const TableView t, const uint64_t n,
                         const uint32_t* __restrict__ sorted_slot,
                         const uint32_t* __restrict__ sorted_index, uint8_t* __restrict__ values) {
  const uint32_t lane = threadIdx.x & 31u;
  const uint64_t i = ((uint64_t(blockIdx.x) * blockDim.x + threadIdx.x) & ~uint64_t(31)) + lane;
  if (i - lane >= n) return;
  uint32_t slot = kNoSlot, dest = 0;
  if (i < n) {
    slot = sorted_slot[i];
    dest = sorted_index[i];
  }
  if (__ballot_sync(0xFFFFFFFFu, slot != kNoSlot) == 0) return;
  warp_gather_rows_to<0, true>(t, values, dest, slot, lane);
}

// find on a table with rows in pinned host memory: probe, sort by slot, gather.
// Only the bits a row place can have are sorted (misses carry kNoSlot, whose
// low bits are all ones: they end up behind or among the last places, and the
// gather skips them by value).
int hybrid_sort_bits(const TableView& t) {
  int bits = 1;
  while (bits < 32 && (1ull << bits) < t.capacity) ++bits;
  return bits;
}

size_t hybrid_sort_temp_bytes(const TableView& t, uint64_t n) {
  size_t temp_bytes = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, temp_bytes, static_cast<uint32_t*>(nullptr),
                                  static_cast<uint32_t*>(nullptr), static_cast<uint32_t*>(nullptr),
                                  static_cast<uint32_t*>(nullptr), static_cast<int>(n), 0,
                                  hybrid_sort_bits(t));
  return temp_bytes;
}

bool launch_find_hybrid(const TableView& t, uint64_t n, const uint64_t* keys, void* values,
                        bool* founds, uint64_t* scores, cudaStream_t stream, void* scratch,
                        size_t scratch_bytes) {
  if (n < 4096 || n >= (1ull << 32) || scratch == nullptr || !line_buckets(t)) return false;
  const size_t arrays = ((n * sizeof(uint32_t)) + 255) & ~size_t(255);
  size_t temp_bytes = hybrid_sort_temp_bytes(t, n);
  if (4 * arrays + temp_bytes > scratch_bytes) return false;
  uint8_t* work = static_cast<uint8_t*>(scratch);
  uint32_t* slot = reinterpret_cast<uint32_t*>(work);
  uint32_t* index = reinterpret_cast<uint32_t*>(work + arrays);
  uint32_t* slot_sorted = reinterpret_cast<uint32_t*>(work + 2 * arrays);
  uint32_t* index_sorted = reinterpret_cast<uint32_t*>(work + 3 * arrays);
  const uint64_t blocks = (((n + 31) / 32) * 32 + kFindBlock - 1) / kFindBlock;
  find_kernel<4, 0><<<static_cast<unsigned>(blocks), kFindBlock, 0, stream>>>(
      t, keys, n, nullptr, nullptr, founds, scores, nullptr, nullptr, nullptr, slot, index);
  cub::DeviceRadixSort::SortPairs(work + 4 * arrays, temp_bytes, slot, slot_sorted, index,
                                  index_sorted, static_cast<int>(n), 0, hybrid_sort_bits(t), stream);
  gather_sorted_kernel<<<static_cast<unsigned>(blocks), kFindBlock, 0, stream>>>(
      t, n, slot_sorted, index_sorted, static_cast<uint8_t*>(values));
  return true;
}

}  // namespace

size_t find_workspace_bytes(const TableView& t, uint64_t n, const void* values) {
  if (t.hbm_slots == t.capacity || values == nullptr || n < 4096 || n >= (1ull << 32) ||
      !line_buckets(t)) {
    return 0;
  }
  const size_t arrays = ((n * sizeof(uint32_t)) + 255) & ~size_t(255);
  return 4 * arrays + hybrid_sort_temp_bytes(t, n);
}

void launch_find(const TableView& t, uint64_t n, const uint64_t* keys, void* values, bool* founds,
                 uint64_t* scores, cudaStream_t stream, void* work, size_t work_bytes) {
  if (t.hbm_slots < t.capacity && values != nullptr &&
      launch_find_hybrid(t, n, keys, values, founds, scores, stream, work, work_bytes)) {
    return;
  }
  launch_form<0>(t, n, keys, values, nullptr, founds, scores, nullptr, nullptr, nullptr, stream);
}

void launch_dual_find(const TableView& t, uint64_t n, const uint64_t* keys, void* values,
                      bool* founds, uint64_t* scores, cudaStream_t stream) {
  if (n == 0) return;
  const uint64_t blocks = (((n + 31) / 32) * 32 + kFindBlock - 1) / kFindBlock;
  dual_find_kernel<<<static_cast<unsigned>(blocks), kFindBlock, 0, stream>>>(
      t, keys, n, static_cast<uint8_t*>(values), founds, scores);
}

void launch_find_ptr(const TableView& t, uint64_t n, const uint64_t* keys, void** ptrs,
                     bool* founds, uint64_t* scores, cudaStream_t stream) {
  launch_form<1>(t, n, keys, nullptr, ptrs, founds, scores, nullptr, nullptr, nullptr, stream);
}

void launch_find_missed(const TableView& t, uint64_t n, const uint64_t* keys, void* values,
                        uint64_t* missed_keys, int* missed_indices, int* missed_size,
                        uint64_t* scores, cudaStream_t stream) {
  launch_form<2>(t, n, keys, values, nullptr, nullptr, scores, missed_keys, missed_indices,
                 missed_size, stream);
}

void launch_find_routed(const TableView& t, uint32_t world, uint32_t my_rank,
                        uint64_t segment_capacity,
                        const uint64_t* inbox_keys, const uint32_t* inbox_origin,
                        const uint64_t* inbox_counts, const PeerPtrs& out_values,
                        const PeerPtrs& out_founds, cudaStream_t stream) {
  if (segment_capacity == 0) return;
  // HKV_STRICT_PEER_ORDER=1 in the environment: every thread that stored rows
  // into a peer's buffer fences them at system scope before it exits
  static const bool writers_fence = [] {
    const char* e = std::getenv("HKV_STRICT_PEER_ORDER");
    return e != nullptr && e[0] == '1';
  }();
  const uint64_t per_segment = (segment_capacity + kFindBlock - 1) / kFindBlock;
  auto kernel = fast_rows(t) ? find_routed_kernel<16> : find_routed_kernel<0>;
  kernel<<<static_cast<unsigned>(per_segment * world), kFindBlock, 0, stream>>>(
      t, world, (my_rank + 1) % world, segment_capacity,
      inbox_keys, inbox_origin,
      inbox_counts, out_values, out_founds, writers_fence);
}

void launch_contains(const TableView& t, uint64_t n, const uint64_t* keys, bool* founds,
                     cudaStream_t stream) {
  launch_form<3>(t, n, keys, nullptr, nullptr, founds, nullptr, nullptr, nullptr, nullptr, stream);
}

}  // namespace hkv
