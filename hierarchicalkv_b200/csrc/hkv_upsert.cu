// Mutating operations: insert_or_assign, find_or_insert (value and pointer
// forms), insert_and_evict, accum_or_assign, assign / assign_scores /
// assign_values, find_and_update, lock_keys.
//
// Replaces the reference's
//   include/merlin/core_kernels/upsert.cuh:27-986            (insert_or_assign)
//   include/merlin/core_kernels/upsert_and_evict.cuh:27-1099 (insert_and_evict)
//   include/merlin/core_kernels/find_or_insert.cuh:27-1050   (find_or_insert)
//   include/merlin/core_kernels/find_ptr_or_insert.cuh:27-260
//   include/merlin/core_kernels/accum_or_assign.cuh:83-174
//   include/merlin/core_kernels/update*.cuh                  (assign family)
// and the score rules of kernel_utils.cuh:267-615.
//
// One warp serves 32 keys:
//   1. eight 8-lane digest probes, all digest lines and first-candidate
//      accesses in flight at once; a hit is locked by CAS key -> LOCKED;
//   2. a miss claims the first EMPTY slot from its start position by CAS;
//   3. digests / scores are written, rows move cooperatively and coalesced,
//      and the owner lanes publish their keys with a release store;
//   4. keys whose bucket is full: 8-lane groups scan the buckets' 128 scores
//      (1 KiB each, coalesced; warp REDUX for the 64-bit minimum), then all
//      owner lanes CAS their victims at the same time, then rows move and
//      keys are published; losers of a CAS go round again.
// Locks are never held across a wait: phases 1-3 contain no wait at all, and
// phase 4 polls a foreign lock (bounded) only while the warp holds nothing.
#include "hkv_device.cuh"
#include "hkv_internal.h"

namespace hkv {

namespace {

constexpr int kMutateBlock = 128;
#ifndef HKV_MUTATE_MIN_BLOCKS
#define HKV_MUTATE_MIN_BLOCKS 8
#endif
// Resident blocks per SM asked of the compiler.  The kernel is bound by memory
// latency: 8 blocks (64 registers, a few spilled values) measured 13 % faster
// than 5 blocks (96 registers, no spills) and faster than 10 or 12.
constexpr int kMutateMinBlocks = HKV_MUTATE_MIN_BLOCKS;
#ifndef HKV_MUTATE_LIGHT_MIN_BLOCKS
#define HKV_MUTATE_LIGHT_MIN_BLOCKS 8
#endif
constexpr int kMutateLightMinBlocks = HKV_MUTATE_LIGHT_MIN_BLOCKS;
constexpr uint32_t kEvictIterLimit = 1u << 16;  // iterations of the full-bucket loop per warp
constexpr uint32_t kHeldLockWaits = 1u << 12;   // polls (about a millisecond) before a lock counts as held

enum Result : uint32_t {
  kInitial = 0,
  kDuplicate = 1,         // key found and locked
  kOccupiedEmpty = 2,     // claimed an EMPTY slot
  kOccupiedReclaimed = 3, // claimed a RECLAIM tombstone via the score scan
  kEvict = 4,             // locked a victim
  kRefused = 5,           // incoming score below the bucket minimum
  kNeedEvict = 6,         // bucket has no free slot, goes to phase 3
  kMiss = 7,              // not found and the operation does not insert
  kFoundNoLock = 8,       // found, operation leaves the slot alone
  kDeferred = 9,          // left to the serialising kernel (accum_or_assign with repeats)
};

constexpr uint32_t kModeValid = 1u;
constexpr uint32_t kModeLockOnHit = 2u;
constexpr uint32_t kModeInsertOnMiss = 4u;

__device__ __forceinline__ bool op_inserts(int op) { return op <= kOpAccumOrAssign; }

__device__ __forceinline__ uint64_t epoch_hi(uint64_t e) { return e << 32; }
__device__ __forceinline__ uint64_t nano_lo() { return (global_nano() >> 20) & 0xFFFFFFFFull; }

// Score an incoming key competes with (kernel_utils.cuh desired_when_missed).
__device__ __forceinline__ uint64_t desired_score(int strategy, const uint64_t* scores,
                                                  uint64_t in_score, uint64_t epoch) {
  switch (strategy) {
    case kLru: return global_nano();
    case kLfu: return kMaxScore;
    case kEpochLru:
      if (epoch == kIgnoredEpoch && scores != nullptr) return in_score;
      return epoch_hi(epoch) | nano_lo();
    case kEpochLfu:
      if (epoch == kIgnoredEpoch) return in_score;
      return epoch_hi(epoch) | (in_score & 0xFFFFFFFFull);
    default: return in_score;
  }
}

// Score stored for a newly inserted key (update_with_digest, new_insert=true).
__device__ __forceinline__ uint64_t inserted_score(int strategy, uint64_t in_score,
                                                   uint64_t desired) {
  switch (strategy) {
    case kLru: return global_nano();
    case kLfu: return in_score;
    default: return desired;
  }
}

__device__ __forceinline__ uint64_t epoch_lfu_merge(uint64_t old_score, uint64_t add) {
  const uint64_t lo = old_score & 0xFFFFFFFFull;
  if (0xFFFFFFFFull - lo > (add & 0xFFFFFFFFull)) return lo + add;
  return (add & 0xFFFFFFFF00000000ull) | 0xFFFFFFFFull;
}

// Score stored when an upsert hits an existing key (update_with_digest,
// new_insert=false).  Returns false when the score is left untouched.
__device__ __forceinline__ bool hit_score_upsert(int strategy, const uint64_t* scores,
                                                 uint64_t in_score, uint64_t desired,
                                                 uint64_t old_score, uint64_t* out) {
  switch (strategy) {
    case kLru: *out = global_nano(); return true;
    case kLfu:
      if (scores == nullptr) return false;
      *out = in_score + old_score;
      return true;
    case kEpochLfu: *out = epoch_lfu_merge(old_score, desired); return true;
    default: *out = desired; return true;
  }
}

// Score stored by the assign family (update_without_missed).
__device__ __forceinline__ bool hit_score_assign(int strategy, const uint64_t* scores,
                                                 uint64_t in_score, uint64_t epoch,
                                                 uint64_t old_score, uint64_t* out) {
  switch (strategy) {
    case kLru: *out = global_nano(); return true;
    case kLfu:
      if (scores == nullptr) return false;
      *out = in_score + old_score;
      return true;
    case kEpochLru: *out = epoch_hi(epoch) | nano_lo(); return true;
    case kEpochLfu:
      if (scores == nullptr) return false;
      *out = epoch_lfu_merge(old_score, epoch_hi(epoch) | (in_score & 0xFFFFFFFFull));
      return true;
    default:
      if (scores == nullptr) return false;
      *out = in_score;
      return true;
  }
}

// Score scan of one bucket by the 8 lanes of a group.  In step q the lanes 0-3
// of the group read the scores of positions 16q .. 16q + 7 and the lanes 4-7
// those of positions 16q + 8 .. 16q + 15, 16 bytes (two scores) each: with
// separate planes a group reads 128 contiguous bytes per instruction, with
// shared lines the 64-byte score halves of two neighbouring lines.  A lane
// ends up with the 16 scores
//   s[2q + e] = score of bucket position scan_pos(sub, 2q + e).
__device__ __forceinline__ uint32_t scan_pos(uint32_t sub, uint32_t b) {
  return ((b & ~1u) + (sub >> 2)) * kLineSlots + (sub & 3u) * 2u + (b & 1u);
}

__device__ __forceinline__ void ld_scores16(const TableView& t, uint64_t bucket, uint32_t sub,
                                            uint64_t (&s)[16]) {
  // positions scan_pos(sub, 2q) for q = 0 .. 7 are 16 slots apart
  const uint64_t* mine = score_ptr(t, (bucket << 7) + scan_pos(sub, 0));
  const uint64_t step = 16u + (16u & t.line_mask);   // words between them
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    asm volatile("ld.relaxed.gpu.global.v2.u64 {%0,%1}, [%2];"
                 : "=l"(s[2 * q]), "=l"(s[2 * q + 1])
                 : "l"(mine + q * step)
                 : "memory");
  }
}

// Distance, in probe order from `start`, of the first set bit of a lane's
// 16-slot mask; 255 when the mask is empty.
__device__ __forceinline__ uint32_t first_from_start(uint32_t mask16, uint32_t sub,
                                                     uint32_t start) {
  const int rel = int(start) - int(sub * 16u);
  uint32_t hi;
  if (rel <= 0) {
    hi = mask16;
  } else if (rel >= 16) {
    hi = 0;
  } else {
    hi = mask16 & (0xFFFFu << rel);
  }
  const uint32_t lo = mask16 & ~hi;
  if (hi) return sub * 16u + (__ffs(hi) - 1) - start;
  if (lo) return sub * 16u + (__ffs(lo) - 1) + kBucketSlots - start;
  return 255u;
}

// Does the operation copy the batch row into a freshly claimed slot?
__device__ __forceinline__ constexpr bool op_writes_row_on_insert(int op) {
  return op == kOpInsertOrAssign || op == kOpFindOrInsert || op == kOpInsertAndEvict ||
         op == kOpAccumOrAssign;
}

// Minimum score of a full bucket and its first position, computed by the 8
// lanes of a group from the bucket's 1 KiB of scores.  Within a lane the
// positions grow with the index, so the first minimum in the lane is the one
// at the lowest position; across lanes the lowest position wins.
__device__ __forceinline__ void lane_min16(const uint64_t (&s)[16], uint64_t* ms, uint32_t* mp) {
  *ms = s[0];
  *mp = 0;
#pragma unroll
  for (int b = 1; b < 16; ++b) {
    if (s[b] < *ms) {
      *ms = s[b];
      *mp = b;
    }
  }
}

__device__ __forceinline__ void group_reduce_min(uint32_t gmask, uint32_t sub, uint64_t ms,
                                                 uint32_t mp, uint64_t* gmin, uint32_t* gpos) {
  const uint32_t hi = uint32_t(ms >> 32);
  const uint32_t ghi = __reduce_min_sync(gmask, hi);
  const uint32_t lo = hi == ghi ? uint32_t(ms) : 0xFFFFFFFFu;
  const uint32_t glo = __reduce_min_sync(gmask, lo);
  const uint32_t cand = (hi == ghi && lo == glo) ? scan_pos(sub, mp) : 255u;
  *gpos = __reduce_min_sync(gmask, cand);
  *gmin = (uint64_t(ghi) << 32) | glo;
}

__device__ __forceinline__ void group_min_score(const TableView& t, const ProbeLane& pl,
                                                uint32_t bucket, uint64_t* gmin, uint32_t* gpos) {
  uint64_t s[16];
  ld_scores16(t, bucket, pl.sub, s);
  uint64_t ms;
  uint32_t mp;
  lane_min16(s, &ms, &mp);
  group_reduce_min(group_mask(pl.group), pl.sub, ms, mp, gmin, gpos);
}

// One warp serves 32 keys.
//   phase 0  own key: hash, bucket, digest, incoming score, bucket fill
//   phase 1  all eight digest lines in flight, then all first candidates: a
//            locking operation CASes key -> LOCKED straight away (a digest
//            match is the key 255 times out of 256), a non-locking one loads
//   phase 2  per pass: confirm the hit or claim the first EMPTY slot (CAS)
//   phase 3  metadata, rows (warp-cooperative, coalesced) and publication of
//            everything locked so far -- no lock survives into phase 4
//   phase 4  keys whose bucket is full, in iterations of
//              A  8-lane groups scan the score lines (four buckets per round)
//              B  every owner lane runs its own lock chain at the same time:
//                 victim key load, CAS, score verification, digest + score
//              C  evicted rows leave, new rows arrive (whole warp, coalesced),
//                 keys are published
//            A lane that meets a LOCKED victim or loses a CAS tries again in
//            the next iteration; it polls the foreign lock (bounded) only
//            after step C, when the warp holds nothing.  The victim is always
//            the true current minimum, as in the reference (upsert.cuh:149-215).
//
// INDEXED is the routed form of the key-hash sharded table: the batch is one
// source rank's inbox segment, the number of keys is read from device memory
// and key i's row is row args.row_index[i] of the source rank's buffer.
// Resident blocks per SM asked of the compiler: the forms that move no rows
// can afford more of them, insert_and_evict (evicted rows, tickets) fewer.
__host__ __device__ constexpr int mutate_min_blocks(int op) {
  return op == kOpInsertAndEvict ? kMutateMinBlocks - 2
         : (op == kOpFindOrInsertPtr || op == kOpAssignScores || op == kOpFindAndUpdate ||
            op == kOpLockKeys || op == kOpErase)
             ? kMutateLightMinBlocks
             : kMutateMinBlocks;
}

// What the routed form knows about the tile a warp serves.
constexpr uint32_t kMaxRequests = 16;     // requests for one key in one call: one per rank
constexpr uint32_t kNoEntry = 0xFFFFFFFFu;
// The plan word of an inbox entry that serves its key: bits 0-4 the number of
// requests, 5-20 which of them accumulate, 21-25 the first that assigns
// (kMaxRequests: none), 26-57 where the later ranks' requests start in the
// list array, bit 63 set.  Zero: the entry does nothing.
constexpr uint32_t kPlanAccumShift = 5, kPlanAssignShift = 21, kPlanListShift = 26;
struct RoutedWarp {
  const RoutedArgs* r;
  uint32_t segment;                        // source rank of the tile's keys
  uint8_t* const* values_of;               // shared-memory copies of the ranks' buffers
  uint32_t (*requests)[kMutateBlock];      // per thread: its key's requests in turn order
};

// Turn of source rank `segment`: the owner applies rank first_segment first.
__device__ __forceinline__ uint32_t turn_of(const RoutedArgs& r, uint32_t segment) {
  return segment >= r.first_segment ? segment - r.first_segment
                                    : segment + r.world - r.first_segment;
}
__device__ __forceinline__ uint32_t segment_of(const RoutedArgs& r, uint32_t turn) {
  const uint32_t s = turn + r.first_segment;
  return s >= r.world ? s - r.world : s;
}

// accum_or_assign for the requests of each lane's key: requests `from` ..
// `count - 1` that `which` selects (bit q: request q) add their rank's row to
// the slot's, one after the other, in request order.  All lanes call it; a
// lane without a slot passes kNoSlot.  (One pass over the row with all
// requests' chunks in flight, as find_or_insert has it below, was built for
// the accumulation as well: it needs more registers than this kernel has and
// measured slower, 226 against 184 us for 2 x 156 k keys nobody shares, 309
// against 269 us for eight ranks sharing most keys.)
template <int VEC>
__device__ __forceinline__ void serve_accumulate(const TableView& t, const RoutedWarp* rw,
                                                 uint32_t slot, uint32_t from, uint32_t count,
                                                 uint32_t which, uint32_t lane) {
  const uint32_t most = __reduce_max_sync(0xFFFFFFFFu, slot != kNoSlot ? count : 0u);
  for (uint32_t q = 0; q < most; ++q) {
    const bool mine = slot != kNoSlot && q >= from && q < count && ((which >> q) & 1u);
    if (__ballot_sync(0xFFFFFFFFu, mine) == 0) continue;
    const uint32_t tag = mine ? rw->requests[q][threadIdx.x] : 0u;
    warp_move_rows<2, VEC, true>(t, nullptr, mine ? slot : kNoSlot, lane, tag, rw->values_of);
    __syncwarp();  // request q + 1 of a key sees what request q did to its row
  }
}

// find_or_insert for the requests of each lane's key, in ONE pass over the
// key's row, chunk by chunk, instead of one pass per request: a key that all
// ranks ask for costs one read of its row, not one per rank.  Per lane (key):
// `slot` (kNoSlot: nothing to do), `todo` (bit q: request q gets the row) and
// `first` (the request whose row is the source -- a new key, the row also goes
// into the table; kMaxRequests: the row stored in the table).  Requests are
// read from the warp's columns of rw->requests, rows are addressed as
// values_of[rank] + row * row_bytes with plain loads and stores (other GPUs'
// memory).
constexpr uint32_t kServeNothing = 0xFFFFFFFFu;
template <int V, bool PURE>
__device__ __forceinline__ void serve_gather_vec(const TableView& t, const RoutedWarp* rw,
                                                 uint32_t slot, uint32_t todo, uint32_t first,
                                                 uint32_t lane) {
  using T = typename VecType<V>::type;
  constexpr int U = 4;  // chunks in flight per lane
  const uint32_t cpr = t.chunks_per_row;
  const uint32_t total = cpr * 32u;
  const uint32_t column0 = threadIdx.x & ~31u;
  const bool idle = slot == kNoSlot || (todo == 0 && first == kMaxRequests);
  const uint32_t packed = idle ? kServeNothing : (todo & 0xFFFFu) | (first << 16);
  // the row of request `tag` (rank << 28 | row) at byte `off`
  auto request_row = [&](uint32_t tag, uint32_t off) -> uint8_t* {
    return rw->values_of[tag >> kRowTagShift] + uint64_t(tag & kRowTagMask) * t.row_bytes + off;
  };
  __syncwarp();  // the lanes read each other's columns of rw->requests
  for (uint32_t base = 0; base < total; base += 32u * U) {
    T cur[U];
    uint8_t* tab[U];
    uint32_t work[U], off[U], column[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t c = base + u * 32u + lane;
      const uint32_t r = row_of_chunk(t, c);
      const uint32_t s = __shfl_sync(0xFFFFFFFFu, slot, r & 31u);
      const uint32_t w = __shfl_sync(0xFFFFFFFFu, packed, r & 31u);
      work[u] = (c < total) ? w : kServeNothing;
      column[u] = column0 + (r & 31u);
      off[u] = (c - r * cpr) * V;
      const bool ok = work[u] != kServeNothing;
      const uint64_t rs = (ok && !PURE) ? row_slot(t, s) : s;
      tab[u] = !ok ? nullptr
                   : (PURE ? t.values_hbm + uint64_t(s) * t.row_bytes
                           : row_ptr_of_row_slot(t, rs)) + off[u];
      if (ok) {
        const uint32_t f = work[u] >> 16;
        if (f == kMaxRequests) {
          cur[u] = ld_table_row<T>(tab[u], !PURE && rs >= t.hbm_slots);
        } else {
          cur[u] = ld_peer(reinterpret_cast<const T*>(request_row(rw->requests[f][column[u]], off[u])));
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (work[u] == kServeNothing) continue;
      if ((work[u] >> 16) != kMaxRequests) st_stream(reinterpret_cast<T*>(tab[u]), cur[u]);
      uint32_t m = work[u] & 0xFFFFu;
      while (m != 0) {
        const uint32_t q = __ffs(m) - 1;
        m &= m - 1;
        *reinterpret_cast<T*>(request_row(rw->requests[q][column[u]], off[u])) = cur[u];
      }
    }
  }
  __syncwarp();
}

// VEC != 0: the access width is fixed at compile time and every row is in HBM
// at its slot's own place (the launcher picks the instantiation).
template <int VEC>
__device__ __forceinline__ void serve_gather(const TableView& t, const RoutedWarp* rw,
                                             uint32_t slot, uint32_t todo, uint32_t first,
                                             uint32_t lane) {
  if constexpr (VEC != 0) {
    serve_gather_vec<VEC, true>(t, rw, slot, todo, first, lane);
    return;
  }
  switch (t.vec_bytes) {
    case 16: serve_gather_vec<16, false>(t, rw, slot, todo, first, lane); break;
    case 8: serve_gather_vec<8, false>(t, rw, slot, todo, first, lane); break;
    case 4: serve_gather_vec<4, false>(t, rw, slot, todo, first, lane); break;
    case 2: serve_gather_vec<2, false>(t, rw, slot, todo, first, lane); break;
    default: serve_gather_vec<1, false>(t, rw, slot, todo, first, lane); break;
  }
}

template <int OP, int VEC, bool INDEXED>
__device__ __forceinline__ void mutate_warp(const TableView& t, const MutateArgs& args,
                                            const uint64_t base, const uint64_t n,
                                            const RoutedWarp* rw = nullptr) {
  const uint32_t full = 0xFFFFFFFFu;
  const ProbeLane pl = probe_lane();
  const uint64_t i = base + pl.lane;
  const int strategy = args.strategy;
  const uint32_t lane_lt = (1u << pl.lane) - 1u;

  // ---- phase 0 ------------------------------------------------------------
  uint64_t key = 0;
  uint64_t in_score = 0;
  uint64_t desired = 0;
  uint32_t mode = 0;
  uint32_t bucket_full = 0;  // the key's bucket has no EMPTY slot left (inserting operations)
  Address a{0, 0, 0};
  uint32_t my_row = 0;  // INDEXED: tag of the row this key is written from / read into
  // INDEXED: the requests for this key (this lane's own and those of the ranks
  // whose turn comes later): how many, which of them accumulate (bit r: request
  // r), and the first that assigns (kMaxRequests: none)
  uint32_t n_requests = 1, accumulating = 0, first_assign = kMaxRequests;
  uint8_t* const* const bases = INDEXED ? rw->values_of : nullptr;
  // Batches that may repeat a key (unique_key == false): this kernel only
  // serves keys it finds and can lock.  A key that meets a LOCKED candidate
  // slot (another occurrence may hold it) and every key that would have to be
  // inserted (two occurrences must not both insert it) is appended to
  // args.deferred_list for the serialising kernel that runs next.
  const bool tolerant = !INDEXED && args.deferred_list != nullptr;
  bool defer_me = false;
  uint8_t* const batch_rows = INDEXED ? nullptr : args.values + base * t.row_bytes;
  bool serves = true;  // INDEXED: this lane is the first in turn order to ask for its key
  if (INDEXED && i < n) {
    // This lane's inbox entry and what routed_resolve_kernel planned for it:
    // nothing (another rank's entry serves the key, or the key is reserved), or
    // the number of requests for the key, which of them accumulate, the first
    // that assigns, and where the requests of the later ranks are listed.  The
    // lane keeps the requests, in turn order, in its column of rw->requests as
    // rank << 28 | row.
    const RoutedArgs& r = *rw->r;
    const uint64_t entry = uint64_t(rw->segment) * r.segment_capacity + i;
    key = r.inbox_keys[entry];
    const uint64_t plan = r.plan[entry];
    serves = plan != 0;
    if (serves) {
      n_requests = uint32_t(plan) & 31u;
      accumulating = uint32_t(plan >> kPlanAccumShift) & 0xFFFFu;
      first_assign = uint32_t(plan >> kPlanAssignShift) & 31u;
      const uint32_t* later = r.lists + (uint32_t(plan >> kPlanListShift));
      rw->requests[0][threadIdx.x] = (rw->segment << kRowTagShift) | r.inbox_origin[entry];
      for (uint32_t q = 1; q < n_requests; ++q) rw->requests[q][threadIdx.x] = later[q - 1];
      // nobody reads the scratch set after the resolving pass: the one entry
      // that serves a key leaves the key's place empty for the next call
      const uint32_t at = r.set_slot[entry];
      r.set_keys[at] = t.empty_key;
      r.set_head[at] = kNoEntry;
    }
  }
  if (i < n) {
    if (!INDEXED) key = args.keys[i];
    if (!is_reserved(t, key) && serves) {
      mode = kModeValid;
      a = locate_line(t, key);
      if (args.scores != nullptr) in_score = args.scores[i];
      if (op_inserts(OP) || OP == kOpLockKeys) {
        desired = desired_score(strategy, args.scores, in_score, args.epoch);
      }
      if (INDEXED) {
        // insert_or_assign: the last rank's row is what stays; find_or_insert: the
        // first rank's row is inserted; accum_or_assign: the first assigning rank's
        my_row = rw->requests[OP == kOpInsertOrAssign ? n_requests - 1
                              : (OP == kOpAccumOrAssign && first_assign != kMaxRequests)
                                  ? first_assign
                                  : 0][threadIdx.x];
      }
      if (OP == kOpAccumOrAssign && INDEXED) {
        if (accumulating) mode |= kModeLockOnHit;
        if (first_assign != kMaxRequests) mode |= kModeInsertOnMiss;
      } else if (OP == kOpAccumOrAssign) {
        const bool is_accum = args.accum_flags[i];
        mode |= is_accum ? kModeLockOnHit : kModeInsertOnMiss;
        // a batch that may repeat keys: two occurrences of a new key must not
        // both insert it, so assigning keys go to the serialising kernel
        if (tolerant && !is_accum) {
          mode = 0;
          defer_me = true;
        }
      } else if (op_inserts(OP)) {
        mode |= kModeLockOnHit | kModeInsertOnMiss;
      } else {
        mode |= kModeLockOnHit;
      }
      // kept out of `mode`: the digest loads of phase 1 are issued on `mode`
      // and must not wait for this load
      if (op_inserts(OP)) bucket_full = t.bucket_sizes[a.bucket] >= kBucketSlots ? 1u : 0u;
    }
  }
  const uint32_t my_bucket = uint32_t(a.bucket);

  // ---- phase 1 ------------------------------------------------------------
  // masks[j]: low half = slots whose digest equals the key's, high half =
  // slots whose digest is the empty digest (this lane's 16 slots of pass j)
  __shared__ uint32_t sm_masks[kPasses][kMutateBlock];
  __shared__ uint64_t sm_first[kPasses][kMutateBlock];
  {
    uint32_t masks[kPasses];
    uint64_t first_key[kPasses];  // key observed at the first candidate slot
    uint4 dg[kPasses];
#pragma unroll
    for (int j = 0; j < kPasses; ++j) {
      const uint32_t owner = pass_owner(j, pl.group);
      const uint32_t b = __shfl_sync(full, my_bucket, owner);
      const uint32_t m = __shfl_sync(full, mode, owner);
      dg[j] = make_uint4(0, 0, 0, 0);
      if (m & kModeValid) dg[j] = ld_meta_v4(t.digests + (uint64_t(b) << 7) + pl.sub * 16u);
    }
#pragma unroll
    for (int j = 0; j < kPasses; ++j) {
      const uint32_t owner = pass_owner(j, pl.group);
      const uint32_t b = __shfl_sync(full, my_bucket, owner);
      const uint32_t m = __shfl_sync(full, mode, owner);
      const uint32_t tgt = __shfl_sync(full, a.digest, owner);
      const uint64_t want = __shfl_sync(full, key, owner);
      masks[j] = 0;
      first_key[j] = ~want;
      if (m & kModeValid) {
        const uint32_t cand = match16(dg[j], replicate4(tgt));
        masks[j] = cand | (match16(dg[j], t.empty_digest4) << 16);
        if (cand) {
          uint64_t* kp = key_ptr_in_line_bucket(t, b, pl.sub * 16u + (__ffs(cand) - 1));
          first_key[j] = (m & kModeLockOnHit) ? cas_relaxed(kp, want, t.locked_key)
                                              : ld_relaxed(kp);
          // with the score's sector on the way into L2 the score store that
          // follows the lock merges there instead of becoming a read-modify-write
          // in DRAM (shared lines: the sector is in the line the lock has just
          // opened; separate planes: a second random access, still cheaper)
          if (OP != kOpAssignValues && (m & kModeLockOnHit)) {
            prefetch_l2(score_ptr(t, (uint64_t(b) << 7) + pl.sub * 16u + (__ffs(cand) - 1)));
          }
        }
      }
    }
    // Parked in shared memory, the per-pass results can be walked by a rolled
    // loop: phase 2 is emitted once instead of eight times (26 KB less code in
    // a kernel that stalled on instruction fetch) and 24 registers are free.
#pragma unroll
    for (int j = 0; j < kPasses; ++j) {
      sm_masks[j][threadIdx.x] = masks[j];
      sm_first[j][threadIdx.x] = first_key[j];
    }
  }

  // ---- phase 2 ------------------------------------------------------------
  uint32_t my_result = kInitial;
  uint32_t my_slot = kNoSlot;
#pragma unroll 1
  for (int j = 0; j < kPasses; ++j) {
    const uint32_t mask_j = sm_masks[j][threadIdx.x];
    const uint64_t first_j = sm_first[j][threadIdx.x];
    const uint32_t gmask = group_mask(pl.group);
    const uint32_t owner = pass_owner(j, pl.group);
    const uint32_t pmode = __shfl_sync(full, mode, owner);
    const bool pfull = __shfl_sync(full, bucket_full, owner) != 0u;
    const uint32_t start = __shfl_sync(full, a.start, owner);
    const uint64_t want = __shfl_sync(full, key, owner);
    const uint64_t slot0 = uint64_t(__shfl_sync(full, my_bucket, owner)) << 7;
    const bool lock_on_hit = (pmode & kModeLockOnHit) != 0;
    uint32_t result = kInitial;
    uint32_t slot = kNoSlot;
    if (pmode & kModeValid) {
      uint32_t hit_pos = 255u;
      bool met_lock = false;  // a candidate slot was LOCKED: it may hold this very key
      uint32_t m = mask_j & 0xFFFFu;
      if (m) {
        uint32_t pos = pl.sub * 16u + (__ffs(m) - 1);
        if (first_j == want) {
          hit_pos = pos;
        } else {
          met_lock = first_j == t.locked_key;
          m &= m - 1;
          while (m) {
            pos = pl.sub * 16u + (__ffs(m) - 1);
            m &= m - 1;
            uint64_t* kp = key_ptr(t, slot0 + pos);
            const uint64_t seen = lock_on_hit ? cas_relaxed(kp, want, t.locked_key)
                                              : ld_relaxed(kp);
            if (seen == want) {
              hit_pos = pos;
              break;
            }
            met_lock |= seen == t.locked_key;
          }
        }
      }
      const uint32_t votes = __ballot_sync(gmask, hit_pos != 255u);
      if (votes) {
        const uint32_t src = __ffs(votes) - 1;
        const uint32_t pos = __shfl_sync(gmask, hit_pos, src);
        result = lock_on_hit ? kDuplicate : kFoundNoLock;
        slot = uint32_t(slot0) + pos;
      } else if (tolerant &&
                 (__ballot_sync(gmask, met_lock) != 0 || (pmode & kModeInsertOnMiss) != 0)) {
        result = kDeferred;
      } else if (!(pmode & kModeInsertOnMiss)) {
        result = kMiss;
      } else if (pfull) {
        result = kNeedEvict;
      } else {
        uint32_t em = mask_j >> 16;
        while (true) {
          const uint32_t d = first_from_start(em, pl.sub, start);
          const uint32_t gd = __reduce_min_sync(gmask, d);
          if (gd == 255u) {
            result = kNeedEvict;
            break;
          }
          const uint32_t pos = (start + gd) & (kBucketSlots - 1);
          bool won = false;
          if (d == gd) {
            won = cas_relaxed(key_ptr(t, slot0 + pos), t.empty_key, t.locked_key) == t.empty_key;
            prefetch_l2(score_ptr(t, slot0 + pos));
            em &= ~(1u << (pos & 15u));
          }
          if (__ballot_sync(gmask, won)) {
            result = kOccupiedEmpty;
            slot = uint32_t(slot0) + pos;
            break;
          }
        }
      }
    }
    __syncwarp();
    const uint32_t r = __shfl_sync(full, result, (pl.lane & 3u) * 8u);
    const uint32_t s = __shfl_sync(full, slot, (pl.lane & 3u) * 8u);
    if ((pl.lane >> 2) == uint32_t(j)) {
      my_result = r;
      my_slot = s;
    }
  }

  if (tolerant) {
    const uint32_t later = __ballot_sync(full, defer_me || my_result == kDeferred);
    if (later) {
      unsigned int first = 0;
      if (pl.lane == 0) first = atomicAdd(args.deferred_count, __popc(later));
      first = __shfl_sync(full, first, 0);
      if ((later >> pl.lane) & 1u) {
        args.deferred_list[first + __popc(later & lane_lt)] = static_cast<uint32_t>(i);
      }
    }
  }

  // ---- phase 3: everything locked so far is written and published ---------------
  // the locks above were taken with relaxed CAS so that they overlap; this is
  // their acquire
  fence_acquire();
  const bool keep_locked =
      (OP == kOpFindOrInsertPtr || OP == kOpLockKeys) && args.locked_key_ptrs != nullptr;
  {
    const bool holds_lock = my_result == kDuplicate || my_result == kOccupiedEmpty;
    if (my_result == kOccupiedEmpty) {
      st_u8_cg(t.digests + my_slot, a.digest);
      st_relaxed(score_ptr(t, my_slot), inserted_score(strategy, in_score, desired));
      atomicAdd(t.bucket_sizes + a.bucket, 1);
    }
    if (my_result == kDuplicate && OP != kOpAssignValues && OP != kOpErase) {
      const bool needs_old = strategy == kLfu || strategy == kEpochLfu ||
                             (OP == kOpFindAndUpdate && args.scores_out != nullptr);
      const uint64_t old_score = needs_old ? ld_relaxed(score_ptr(t, my_slot)) : 0;
      uint64_t ns = 0;
      bool write;
      if (op_inserts(OP) || OP == kOpLockKeys) {
        write = hit_score_upsert(strategy, args.scores, in_score, desired, old_score, &ns);
      } else {
        write = hit_score_assign(strategy, args.scores, in_score, args.epoch, old_score, &ns);
      }
      if (write) st_relaxed(score_ptr(t, my_slot), ns);
      if (OP == kOpFindAndUpdate && args.scores_out != nullptr) {
        args.scores_out[i] = write ? ns : old_score;
      }
    }
    if (OP == kOpInsertOrAssign || OP == kOpInsertAndEvict || OP == kOpAssign ||
        OP == kOpAssignValues) {
      warp_move_rows<1, VEC, INDEXED>(t, batch_rows, holds_lock ? my_slot : kNoSlot, pl.lane,
                                      my_row, bases);
    } else if (OP == kOpFindOrInsert) {
      if constexpr (INDEXED) {
        // a key that was there: its row goes to every rank that asked; a new key:
        // the first rank's row goes in and to the ranks whose turn comes later
        const bool fresh = my_result == kOccupiedEmpty;
        const uint32_t everyone = (1u << n_requests) - 1u;
        serve_gather<VEC>(t, rw, holds_lock ? my_slot : kNoSlot,
                               fresh ? (everyone & ~1u) : everyone, fresh ? 0u : kMaxRequests,
                               pl.lane);
      } else {
        warp_move_rows<0, VEC>(t, batch_rows, my_result == kDuplicate ? my_slot : kNoSlot, pl.lane);
        warp_move_rows<1, VEC>(t, batch_rows, my_result == kOccupiedEmpty ? my_slot : kNoSlot,
                               pl.lane);
      }
    } else if (OP == kOpAccumOrAssign && !INDEXED) {
      warp_move_rows<2, VEC, false>(t, batch_rows, my_result == kDuplicate ? my_slot : kNoSlot,
                                    pl.lane, my_row);
      warp_move_rows<1, VEC, false>(t, batch_rows,
                                    my_result == kOccupiedEmpty ? my_slot : kNoSlot, pl.lane,
                                    my_row);
    } else if constexpr (OP == kOpAccumOrAssign && INDEXED) {
      // a key that was there: every accumulating request adds, in turn order; a
      // new key: the first assigning request's row goes in (my_row), the
      // accumulating requests behind it add
      warp_move_rows<1, VEC, true>(t, batch_rows, my_result == kOccupiedEmpty ? my_slot : kNoSlot,
                                   pl.lane, my_row, bases);
      __syncwarp();
      serve_accumulate<VEC>(t, rw, holds_lock ? my_slot : kNoSlot,
                            my_result == kDuplicate ? 0u : first_assign + 1u, n_requests,
                            accumulating, pl.lane);
    }
    __syncwarp();
    if (OP == kOpErase) {
      // the slot becomes a tombstone: RECLAIM key, reclaim digest, score 0, size - 1
      // (include/merlin/core_kernels.cuh:680-734)
      if (my_result == kDuplicate) {
        st_u8_cg(t.digests + my_slot, t.reclaim_digest);
        st_relaxed(score_ptr(t, my_slot), 0);
        atomicSub(t.bucket_sizes + a.bucket, 1);
        st_release(key_ptr(t, my_slot), t.reclaim_key);
      }
    } else if (holds_lock && !keep_locked) {
      st_release(key_ptr(t, my_slot), key);
    }
  }

  // ---- phase 4: full buckets ----------------------------------------------------------
  if (op_inserts(OP)) {
    uint32_t pending = __ballot_sync(full, my_result == kNeedEvict);
    uint32_t iterations = 0;
    while (pending) {
      const bool mine = (pending >> pl.lane) & 1u;
#ifdef HKV_COUNT_ITERATIONS
      if (pl.lane == 0) {
        atomicAdd(t.status + 4, 1u);
        atomicAdd(t.status + 5, __popc(pending));
      }
#endif
      if (++iterations > kEvictIterLimit) {
        if (mine) {
          my_result = kRefused;
          atomicOr(t.status, kStatusRetryExhausted);
        }
        break;
      }
      // -- A: score scans, four buckets per round
      uint64_t my_min = kMaxScore;
      uint32_t my_pos = 255u;
      for (uint32_t scan = pending; scan != 0;) {
        const uint32_t k = __fns(scan, 0, pl.group + 1);
        const bool active = k != 0xFFFFFFFFu;
        const uint32_t e_bucket = __shfl_sync(full, my_bucket, active ? k : 0u);
        uint64_t gmin = kMaxScore;
        uint32_t gpos = 255u;
        if (active) group_min_score(t, pl, e_bucket, &gmin, &gpos);
        __syncwarp();
        const uint32_t rank = __popc(scan & lane_lt);
        const uint64_t rmin = __shfl_sync(full, gmin, (rank & 3u) * 8u);
        const uint32_t rpos = __shfl_sync(full, gpos, (rank & 3u) * 8u);
        if (((scan >> pl.lane) & 1u) && rank < 4u) {
          my_min = rmin;
          my_pos = rpos;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) scan &= scan - 1;  // (0 & -1) stays 0
      }
      // -- B: every owner lane runs its lock chain, nobody waits
      uint64_t victim = 0;
      uint64_t* wait_on = nullptr;
      bool placed = false;
      bool refused_now = false;
      if (mine) {
        const bool refuse =
            (OP == kOpFindOrInsertPtr) ? (desired <= my_min) : (desired < my_min);
        if (refuse) {
          refused_now = true;
          my_result = kRefused;
        } else {
          const uint32_t slot = (my_bucket << 7) + my_pos;
          uint64_t* kp = key_ptr(t, slot);
          // one round trip: swapping LOCKED in returns the victim; over a slot
          // that is already LOCKED the swap changes nothing
          victim = exch_acquire(kp, t.locked_key);
          if (victim == t.locked_key) {
            wait_on = kp;
          } else {
            uint64_t* sp = score_ptr(t, slot);
            if (ld_relaxed(sp) > my_min) {
              st_release(kp, victim);  // the slot was refreshed in between: scan again
            } else {
              placed = true;
              my_slot = slot;
              st_u8_cg(t.digests + slot, a.digest);
              st_relaxed(sp, inserted_score(strategy, in_score, desired));
              if (victim == t.empty_key || victim == t.reclaim_key) {
                my_result = kOccupiedReclaimed;
                atomicAdd(t.bucket_sizes + a.bucket, 1);
              } else {
                my_result = kEvict;
              }
            }
          }
        }
      }
      // -- C: rows and publication
      if (OP == kOpInsertAndEvict) {
        const uint32_t ev = __ballot_sync(full, placed && my_result == kEvict);
        const uint32_t rf = __ballot_sync(full, refused_now);
        if (ev | rf) {
          unsigned long long first = 0;
          if (pl.lane == 0) {
            first = atomicAdd(args.evicted_counter, (unsigned long long)(__popc(ev) + __popc(rf)));
          }
          first = __shfl_sync(full, first, 0);
          if ((ev >> pl.lane) & 1u) {
            const unsigned long long at = first + __popc(ev & lane_lt);
            __stcs(args.evicted_keys + at, victim);
            if (args.evicted_scores != nullptr) __stcs(args.evicted_scores + at, my_min);
          }
          if ((rf >> pl.lane) & 1u) {
            // a refused input leaves through the evicted arrays as well
            // (upsert_and_evict.cuh:189-194,244-246)
            const unsigned long long at = first + __popc(ev) + __popc(rf & lane_lt);
            __stcs(args.evicted_keys + at, key);
            if (args.evicted_scores != nullptr) __stcs(args.evicted_scores + at, desired);
          }
          if (ev) {
            // lane r carries the slot of the r-th evicting lane
            const uint32_t src = __fns(ev, 0, pl.lane + 1);
            const uint32_t s = __shfl_sync(full, my_slot, src & 31u);
            warp_move_rows<0, VEC>(t, args.evicted_values + first * t.row_bytes,
                              src == 0xFFFFFFFFu ? kNoSlot : s, pl.lane);
            __syncwarp();  // the old rows are out before the new ones come in
          }
          for (uint32_t left = rf, q = 0; left != 0; left &= left - 1, ++q) {
            const uint32_t src = __ffs(left) - 1;
            warp_copy_one_row<VEC>(t, args.evicted_values + (first + __popc(ev) + q) * t.row_bytes,
                              args.values + (base + src) * t.row_bytes, pl.lane);
          }
        }
      }
      if constexpr (INDEXED && OP == kOpFindOrInsert) {
        // the first rank's row goes in and to the ranks whose turn comes later
        serve_gather<VEC>(t, rw, placed ? my_slot : kNoSlot, ((1u << n_requests) - 1u) & ~1u,
                               0u, pl.lane);
      } else if (op_writes_row_on_insert(OP)) {
        warp_move_rows<1, VEC, INDEXED>(t, batch_rows, placed ? my_slot : kNoSlot, pl.lane,
                                        my_row, bases);
      }
      if constexpr (INDEXED && OP == kOpAccumOrAssign) {
        // the first assigning request's row went in; the accumulating ones behind it add
        __syncwarp();
        serve_accumulate<VEC>(t, rw, placed ? my_slot : kNoSlot, first_assign + 1u, n_requests,
                              accumulating, pl.lane);
      }
      __syncwarp();
      if (placed && !(OP == kOpFindOrInsertPtr && keep_locked)) st_release(key_ptr(t, my_slot), key);
      pending &= ~__ballot_sync(full, placed || refused_now);
      // the warp holds no lock now: lanes that met a foreign lock poll it (bounded)
      if (wait_on != nullptr) {
        bool freed = false;
        for (uint32_t spin = 0; spin < kSpinLimit && !freed; ++spin) {
          __nanosleep(spin < 64 ? 32 : 256);
          freed = ld_acquire(wait_on) != t.locked_key;
        }
        if (!freed) {
          my_result = kRefused;
          atomicOr(t.status, kStatusLockTimeout);
        }
      }
      pending &= ~__ballot_sync(full, mine && my_result == kRefused);
    }
  }

  if (OP == kOpFindOrInsertPtr || OP == kOpFindAndUpdate || OP == kOpLockKeys) {
    const bool has_slot = my_result == kDuplicate || my_result == kOccupiedEmpty ||
                          my_result == kOccupiedReclaimed || my_result == kEvict;
    if (i < n) {
      if (args.ptrs != nullptr) args.ptrs[i] = has_slot ? row_ptr(t, my_slot) : nullptr;
      if (args.founds != nullptr) args.founds[i] = my_result == kDuplicate;
      if (args.locked_key_ptrs != nullptr) {
        args.locked_key_ptrs[i] = has_slot ? key_ptr(t, my_slot) : nullptr;
      }
    }
  }
}

template <int OP, int VEC, bool INDEXED>
__global__ void __launch_bounds__(kMutateBlock, mutate_min_blocks(OP))
    mutate_kernel(const TableView t, const MutateArgs args) {
  static_assert(!INDEXED, "the routed form is mutate_routed_kernel");
  const uint64_t warp = (uint64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (warp * 32u < args.n) mutate_warp<OP, VEC, false>(t, args, warp * 32u, args.n);
}

// ---- the routed form ------------------------------------------------------------
//
// Tiles of 128 inbox entries of one segment; tile k belongs to the k % world-th
// rank in turn order, so a block reads from (and, for find_or_insert, writes
// to) all source ranks in rotation.  The key counts live in device memory: the
// grid is a fixed number of resident blocks that stride over the tiles.
__device__ __forceinline__ uint64_t routed_tiles(const RoutedArgs& r) {
  uint64_t most = 0;
  for (uint32_t s = 0; s < r.world; ++s) most = max(most, r.inbox_counts[s]);
  most = min(most, r.segment_capacity);
  return ((most + kMutateBlock - 1) / kMutateBlock) * r.world;
}

// Chains the requests for one key: every inbox entry enters its key into the
// scratch set (linear probing from the top bits of the key's hash, which the
// table's own addressing does not use) and pushes itself onto the key's chain.
__global__ void __launch_bounds__(kMutateBlock)
    routed_group_kernel(const TableView t, const RoutedArgs r) {
  const uint64_t tiles = routed_tiles(r);
  const uint32_t set_mask = (1u << r.set_bits) - 1u;
  for (uint64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    const uint32_t seg = segment_of(r, uint32_t(tile % r.world));
    const uint64_t i = (tile / r.world) * kMutateBlock + threadIdx.x;
    if (i >= r.inbox_counts[seg] || i >= r.segment_capacity) continue;
    const uint64_t entry = uint64_t(seg) * r.segment_capacity + i;
    const uint64_t key = r.inbox_keys[entry];
    if (is_reserved(t, key)) continue;
    uint32_t at = uint32_t(fmix64(key) >> (64 - r.set_bits));
    // the set has at least twice as many places as the inbox has entries
    for (uint32_t probe = 0; probe <= set_mask; ++probe, at = (at + 1u) & set_mask) {
      const uint64_t seen = atomicCAS(reinterpret_cast<unsigned long long*>(r.set_keys + at),
                                      (unsigned long long)t.empty_key, (unsigned long long)key);
      if (seen == t.empty_key || seen == key) break;
    }
    r.set_slot[entry] = at;
    r.next[entry] = atomicExch(r.set_head + at, uint32_t(entry));
  }
}

// Plans the serving pass, one thread per inbox entry: the entry whose rank comes
// first in turn order among all requests for its key serves the key; it sorts
// the chain by turn, reads the accumulate flags of accum_or_assign from the
// requesting ranks, and leaves the later ranks' requests as one contiguous run
// of the list array.  What the serving kernel then needs per entry is its plan
// word (coalesced) and, for keys several ranks asked for, that run: the chain
// walk with its dependent loads happens here, where nothing else waits for it.
__global__ void __launch_bounds__(kMutateBlock)
    routed_resolve_kernel(const TableView t, const RoutedArgs r, const bool with_flags) {
  const uint64_t tiles = routed_tiles(r);
  for (uint64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    const uint32_t seg = segment_of(r, uint32_t(tile % r.world));
    const uint64_t i = (tile / r.world) * kMutateBlock + threadIdx.x;
    if (i >= r.inbox_counts[seg] || i >= r.segment_capacity) continue;
    const uint64_t entry = uint64_t(seg) * r.segment_capacity + i;
    uint64_t plan = 0;
    if (!is_reserved(t, r.inbox_keys[entry])) {
      const uint32_t my_turn = turn_of(r, seg);
      uint32_t words[kMaxRequests];  // turn << 28 | row, sorted
      uint32_t n_requests = 0, hops = 0;
      bool serves = true;
      for (uint32_t e = r.set_head[r.set_slot[entry]];
           e != kNoEntry && hops < 4 * kMaxRequests && serves; e = r.next[e], ++hops) {
        const uint32_t turn = turn_of(r, uint32_t(e / r.segment_capacity));
        if (turn < my_turn || (turn == my_turn && e < entry)) serves = false;
        if (serves && n_requests < kMaxRequests) {
          const uint32_t word = (turn << kRowTagShift) | r.inbox_origin[e];
          uint32_t at = n_requests++;
          while (at > 0 && words[at - 1] > word) {
            words[at] = words[at - 1];
            --at;
          }
          words[at] = word;
        }
      }
      if (serves && n_requests > 0) {
        uint32_t accumulating = 0, first_assign = kMaxRequests;
        for (uint32_t q = 0; q < n_requests; ++q) {
          // rows are named by rank << 28 | row from here on
          const uint32_t rank = segment_of(r, words[q] >> kRowTagShift);
          const uint32_t row = words[q] & kRowTagMask;
          words[q] = (rank << kRowTagShift) | row;
          if (with_flags) {
            if (ld_peer(static_cast<const uint8_t*>(r.flags_of.p[rank]) + row)) accumulating |= 1u << q;
            else if (first_assign == kMaxRequests) first_assign = q;
          }
        }
        uint32_t list = 0;
        if (n_requests > 1) {
          list = atomicAdd(r.list_cursor, n_requests - 1);
          for (uint32_t q = 1; q < n_requests; ++q) r.lists[list + q - 1] = words[q];
        }
        plan = (1ull << 63) | n_requests | (uint64_t(accumulating) << kPlanAccumShift) |
               (uint64_t(first_assign) << kPlanAssignShift) | (uint64_t(list) << kPlanListShift);
      }
    }
    r.plan[entry] = plan;
  }
}

__global__ void __launch_bounds__(256)
    routed_fill_kernel(uint64_t* set_keys, uint32_t* set_head, uint64_t places, uint64_t empty_key) {
  for (uint64_t p = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; p < places;
       p += uint64_t(gridDim.x) * blockDim.x) {
    set_keys[p] = empty_key;
    set_head[p] = kNoEntry;
  }
}

// Serving the later ranks' requests and addressing rows by rank and index cost
// registers the local form does not need: fewer resident blocks per SM than
// its eight keep the routed form free of large spills (its pace is set by the
// peer-memory accesses anyway).  Measured per operation with both source
// ranks' buffers local, 2 x 156 k keys: find_or_insert 144 / 145 / 141 / 174 us
// at 4 / 5 / 6 / 8 blocks (eight ranks sharing most keys: 165 us at 4, 143 us
// at 6), accum_or_assign 211 / 223 / 184 us at 4 / 5 / 6, insert_or_assign
// 140 / 132 / 142 / 166 us at 4 / 5 / 6 / 8.
#ifdef HKV_ROUTED_MIN_BLOCKS
__host__ __device__ constexpr int routed_min_blocks(int) { return HKV_ROUTED_MIN_BLOCKS; }
#else
__host__ __device__ constexpr int routed_min_blocks(int op) {
  return op == kOpInsertOrAssign ? 5 : 6;
}
#endif

template <int OP, int VEC>
__global__ void __launch_bounds__(kMutateBlock, routed_min_blocks(OP))
    mutate_routed_kernel(const TableView t, const MutateArgs args, const RoutedArgs r) {
  static_assert(OP == kOpInsertOrAssign || OP == kOpFindOrInsert || OP == kOpAccumOrAssign,
                "the routed form exists for the three operations the sharded table routes");
  __shared__ uint8_t* sm_values[kMaxPeers];
  __shared__ uint32_t sm_requests[kMaxRequests][kMutateBlock];
  // a copy in shared memory: the warps reach the arguments through a pointer,
  // which would otherwise put the whole parameter block into local memory
  __shared__ RoutedArgs sm_r;
  if (threadIdx.x < kMaxPeers) {
    sm_values[threadIdx.x] = static_cast<uint8_t*>(r.values_of.p[threadIdx.x]);
  }
  if (threadIdx.x == 0) {
    sm_r.world = r.world;
    sm_r.first_segment = r.first_segment;
    sm_r.segment_capacity = r.segment_capacity;
    sm_r.inbox_keys = r.inbox_keys;
    sm_r.inbox_origin = r.inbox_origin;
    sm_r.inbox_counts = r.inbox_counts;
    sm_r.plan = r.plan;
    sm_r.lists = r.lists;
    sm_r.set_keys = r.set_keys;
    sm_r.set_head = r.set_head;
    sm_r.set_slot = r.set_slot;
    if (blockIdx.x == 0) *r.list_cursor = 0;  // the resolving pass is over
  }
  __syncthreads();
  const uint64_t tiles = routed_tiles(r);
  RoutedWarp rw{&sm_r, 0, sm_values, sm_requests};
  for (uint64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    rw.segment = segment_of(r, uint32_t(tile % r.world));
    const uint64_t base = (tile / r.world) * kMutateBlock + (threadIdx.x & ~31u);
    const uint64_t n = min(r.inbox_counts[rw.segment], r.segment_capacity);
    if (base < n) mutate_warp<OP, VEC, true>(t, args, base, n, &rw);
    __syncwarp();  // the warp's columns of the parked results and requests are reused
  }
  // Rows found by find_or_insert went to other GPUs, and the requesters overwrite
  // those buffers (the next operation's rows) as soon as the barrier that
  // follows lets them.  That barrier's own system-scope fence orders the stores
  // before its flags; this one, by the writers themselves, costs a few per
  // cent of the step and stays as a second line until the replay check of the
  // step, which failed at eight ranks on symmetric-memory workspaces, is
  // understood.
  __threadfence_system();
}

// ---- serialising kernel for batches that may repeat a key -------------------
//
// One warp walks its 32 keys one after the other and finishes each (lock,
// write, publish) before the next, reading the bucket's 128 keys directly
// (4 per lane) as the reference's tile kernels do
// (kernel_utils.cuh:675-898, upsert.cuh:1233-1305).  A LOCKED slot met during
// the scan is waited for (bounded), so a second occurrence of a key finds the
// first one's slot once it is published.
template <int OP>
__global__ void __launch_bounds__(kMutateBlock)
    mutate_serial_kernel(const TableView t, const MutateArgs args) {
  const uint32_t full = 0xFFFFFFFFu;
  const uint32_t lane = threadIdx.x & 31u;
  const uint64_t warp = (uint64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const uint64_t base = warp * 32u;
  // with an index list the kernel walks the listed batch positions only
  const uint64_t n = args.index_list != nullptr ? uint64_t(*args.index_count) : args.n;
  if (base >= n) return;
  const int strategy = args.strategy;
  const uint32_t count = uint32_t(min(uint64_t(32), n - base));

  for (uint32_t q = 0; q < count; ++q) {
    const uint64_t i = args.index_list != nullptr ? uint64_t(args.index_list[base + q]) : base + q;
    const uint64_t key = args.keys[i];
    if (is_reserved(t, key)) {
      if (lane == 0 &&
          (OP == kOpFindOrInsertPtr || OP == kOpFindAndUpdate || OP == kOpLockKeys)) {
        if (args.ptrs != nullptr) args.ptrs[i] = nullptr;
        if (args.founds != nullptr) args.founds[i] = false;
        if (args.locked_key_ptrs != nullptr) args.locked_key_ptrs[i] = nullptr;
      }
      continue;
    }
    const Address a = locate(t, key);
    const uint64_t in_score = args.scores != nullptr ? args.scores[i] : 0;
    const uint64_t desired = (op_inserts(OP) || OP == kOpLockKeys)
                                 ? desired_score(strategy, args.scores, in_score, args.epoch)
                                 : 0;
    const bool is_accum = OP == kOpAccumOrAssign ? args.accum_flags[i] : false;
    const bool lock_on_hit = OP == kOpAccumOrAssign ? is_accum : true;
    const bool insert_on_miss = OP == kOpAccumOrAssign ? !is_accum : op_inserts(OP);
    const uint64_t slot0 = a.bucket << t.bucket_shift;
    const uint32_t bucket_slots = t.bucket_slots;
    const uint32_t steps = (bucket_slots + 31u) >> 5;  // 32 slots per step, at most 32 steps

    uint32_t result = kInitial;
    uint32_t pos = 0;
    uint64_t victim = 0;
    uint64_t victim_score = 0;
    uint32_t attempts = 0;
    while (result == kInitial) {
      if (++attempts > kRescanLimit) {
        if (lane == 0) atomicOr(t.status, kStatusLockTimeout);
        result = kRefused;
        break;
      }
      // lane l looks at slots l, l + 32, l + 64, ... (bit c of the masks: step c)
      uint32_t eq = 0, locked = 0, empty = 0;
      for (uint32_t c = 0; c < steps; ++c) {
        const uint32_t at = c * 32u + lane;
        if (at < bucket_slots) {
          const uint64_t k = ld_acquire(key_ptr(t, slot0 + at));
          eq |= (k == key) ? (1u << c) : 0u;
          locked |= (k == t.locked_key) ? (1u << c) : 0u;
          empty |= (k == t.empty_key) ? (1u << c) : 0u;
        }
      }
      const uint32_t any_eq = __ballot_sync(full, eq != 0);
      if (any_eq) {
        const uint32_t src = __ffs(any_eq) - 1;
        const uint32_t p = __shfl_sync(full, (__ffs(eq) - 1) * 32 + lane, src);
        uint32_t ok = 1;
        if (lock_on_hit) {
          if (lane == src) ok = cas_acquire(key_ptr(t, slot0 + p), key, t.locked_key) == key ? 1u : 0u;
          ok = __shfl_sync(full, ok, src);
        }
        if (ok) {
          result = lock_on_hit ? kDuplicate : kFoundNoLock;
          pos = p;
        }
        continue;
      }
      // Somebody holds a slot of this bucket; it may be writing this very key.
      // A kernel holds a slot for microseconds, so the slot is waited for.  A
      // slot that stays locked (a key held through lock_keys or the pointer form
      // of find_or_insert) would starve the bucket: after kHeldLockWaits polls
      // a locked slot is passed over if its digest, stable by then, belongs to
      // another key.  A held slot with this key's own digest (one in 256)
      // cannot be told from this key and is waited for to the bound.
      if (__ballot_sync(full, locked != 0)) {
        bool may_be_mine = attempts <= kHeldLockWaits;
        for (uint32_t c = 0; c < steps && !may_be_mine; ++c) {
          if ((locked >> c) & 1u) {
            uint32_t d;
            asm volatile("ld.global.cg.u8 %0, [%1];" : "=r"(d) : "l"(t.digests + slot0 + c * 32u + lane));
            may_be_mine = d == a.digest || d == (t.empty_digest4 & 0xFFu) || d == t.reclaim_digest;
          }
        }
        if (__ballot_sync(full, may_be_mine)) {
          __nanosleep(128);
          continue;
        }
      }
      if (!insert_on_miss) {
        result = kMiss;
        break;
      }
      // first EMPTY slot in probe order from a.start
      uint32_t best = kNoSlot;
      for (uint32_t c = 0; c < steps; ++c) {
        if ((empty >> c) & 1u) {
          const uint32_t d = (c * 32u + lane - a.start) & (bucket_slots - 1u);
          best = min(best, d);
        }
      }
      const uint32_t gbest = __reduce_min_sync(full, best);
      if (gbest != kNoSlot) {
        const uint32_t p = (a.start + gbest) & (bucket_slots - 1u);
        uint32_t ok = 0;
        if (lane == 0) ok = cas_acquire(key_ptr(t, slot0 + p), t.empty_key, t.locked_key) == t.empty_key;
        ok = __shfl_sync(full, ok, 0);
        if (ok) {
          result = kOccupiedEmpty;
          pos = p;
        }
        continue;
      }
      // full bucket: minimum score, first position on ties
      uint64_t ms = kMaxScore;
      uint32_t mp = kNoSlot;
      for (uint32_t c = 0; c < steps; ++c) {
        const uint32_t at = c * 32u + lane;
        if (at < bucket_slots) {
          const uint64_t sc = ld_relaxed(score_ptr(t, slot0 + at));
          if (mp == kNoSlot || sc < ms) {
            ms = sc;
            mp = at;
          }
        }
      }
      // lanes beyond a small bucket hold no score: they take no part in the minimum
      const bool has = mp != kNoSlot;
      const uint32_t hi = has ? uint32_t(ms >> 32) : 0xFFFFFFFFu;
      const uint32_t ghi = __reduce_min_sync(full, hi);
      const uint32_t lo = (has && hi == ghi) ? uint32_t(ms) : 0xFFFFFFFFu;
      const uint32_t glo = __reduce_min_sync(full, lo);
      const uint32_t cp = (has && hi == ghi && lo == glo) ? mp : kNoSlot;
      const uint32_t gpos = __reduce_min_sync(full, cp);
      const uint64_t gmin = (uint64_t(ghi) << 32) | glo;
      const bool refuse = (OP == kOpFindOrInsertPtr) ? (desired <= gmin) : (desired < gmin);
      if (refuse) {
        result = kRefused;
        break;
      }
      uint32_t code = 0;
      if (lane == 0) {
        uint64_t* kp = key_ptr(t, slot0 + gpos);
        const uint64_t v = ld_relaxed(kp);
        if (v != t.locked_key && cas_acquire(kp, v, t.locked_key) == v) {
          if (ld_relaxed(score_ptr(t, slot0 + gpos)) > gmin) {
            st_release(kp, v);
          } else {
            victim = v;
            code = (v == t.empty_key || v == t.reclaim_key) ? 2 : 1;
          }
        }
      }
      code = __shfl_sync(full, code, 0);
      if (code) {
        result = code == 2 ? kOccupiedReclaimed : kEvict;
        pos = gpos;
        victim = __shfl_sync(full, victim, 0);
        victim_score = gmin;
      }
    }

    const uint32_t slot = uint32_t(slot0) + pos;
    const bool holds_lock = result == kDuplicate || result == kOccupiedEmpty ||
                            result == kOccupiedReclaimed || result == kEvict;
    const bool fresh = holds_lock && result != kDuplicate;
    uint8_t* batch_row = args.values != nullptr ? args.values + i * t.row_bytes : nullptr;

    if (OP == kOpInsertAndEvict && (result == kEvict || result == kRefused)) {
      unsigned long long ticket = 0;
      if (lane == 0) {
        ticket = atomicAdd(args.evicted_counter, 1ull);
        args.evicted_keys[ticket] = result == kEvict ? victim : key;
        if (args.evicted_scores != nullptr) {
          args.evicted_scores[ticket] = result == kEvict ? victim_score : desired;
        }
      }
      ticket = __shfl_sync(full, ticket, 0);
      const uint8_t* src = result == kEvict ? row_ptr(t, slot) : batch_row;
      uint8_t* dst = args.evicted_values + ticket * t.row_bytes;
      for (uint32_t c = lane; c < t.row_bytes / t.vec_bytes; c += 32) {
        for (uint32_t b = 0; b < t.vec_bytes; ++b) dst[c * t.vec_bytes + b] = src[c * t.vec_bytes + b];
      }
      __syncwarp();
    }

    if (holds_lock) {
      if (lane == 0) {
        if (fresh) {
          st_u8_cg(t.digests + slot, a.digest);
          st_relaxed(score_ptr(t, slot), inserted_score(strategy, in_score, desired));
          if (result != kEvict) atomicAdd(t.bucket_sizes + a.bucket, 1);
        } else if (OP != kOpAssignValues) {
          const uint64_t old_score = ld_relaxed(score_ptr(t, slot));
          uint64_t ns = 0;
          const bool write =
              (op_inserts(OP) || OP == kOpLockKeys)
                  ? hit_score_upsert(strategy, args.scores, in_score, desired, old_score, &ns)
                  : hit_score_assign(strategy, args.scores, in_score, args.epoch, old_score, &ns);
          if (write) st_relaxed(score_ptr(t, slot), ns);
          if (OP == kOpFindAndUpdate && args.scores_out != nullptr) {
            args.scores_out[i] = write ? ns : old_score;
          }
        }
      }
      uint8_t* row = row_ptr(t, slot);
      const uint32_t vec = t.vec_bytes;
      const uint32_t words = t.row_bytes / vec;
      const bool to_table = OP == kOpInsertOrAssign || OP == kOpInsertAndEvict ||
                            OP == kOpAssign || OP == kOpAssignValues ||
                            ((OP == kOpFindOrInsert || OP == kOpAccumOrAssign) && fresh);
      const bool from_table = OP == kOpFindOrInsert && !fresh;
      const bool accumulate = OP == kOpAccumOrAssign && !fresh;
      if (to_table || from_table) {
        uint8_t* dst = to_table ? row : batch_row;
        const uint8_t* src = to_table ? batch_row : row;
        if (vec == 16) {
          for (uint32_t c = lane; c < words; c += 32)
            reinterpret_cast<uint4*>(dst)[c] = reinterpret_cast<const uint4*>(src)[c];
        } else if (vec == 8) {
          for (uint32_t c = lane; c < words; c += 32)
            reinterpret_cast<uint2*>(dst)[c] = reinterpret_cast<const uint2*>(src)[c];
        } else if (vec == 4) {
          for (uint32_t c = lane; c < words; c += 32)
            reinterpret_cast<uint32_t*>(dst)[c] = reinterpret_cast<const uint32_t*>(src)[c];
        } else {
          for (uint32_t c = lane; c < t.row_bytes; c += 32) dst[c] = src[c];
        }
      } else if (accumulate) {
        warp_accumulate_row(row, batch_row, t.row_bytes, t.value_kind, lane);
      }
    }
    if (lane == 0 &&
        (OP == kOpFindOrInsertPtr || OP == kOpFindAndUpdate || OP == kOpLockKeys)) {
      if (args.ptrs != nullptr) args.ptrs[i] = holds_lock ? row_ptr(t, slot) : nullptr;
      if (args.founds != nullptr) args.founds[i] = result == kDuplicate;
      if (args.locked_key_ptrs != nullptr) {
        args.locked_key_ptrs[i] = holds_lock ? key_ptr(t, slot) : nullptr;
      }
    }
    __syncwarp();
    const bool keep_locked =
        (OP == kOpFindOrInsertPtr || OP == kOpLockKeys) && args.locked_key_ptrs != nullptr;
    if (holds_lock && !keep_locked && lane == 0) {
      __threadfence();
      st_release(key_ptr(t, slot0 + pos), key);
    }
    __syncwarp();
  }
}

__global__ void unlock_keys_kernel(const TableView t, uint64_t n, uint64_t** locked_key_ptrs,
                                   const uint64_t* keys, bool* success) {
  const uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  uint64_t* p = locked_key_ptrs[i];
  bool ok = false;
  if (p != nullptr) {
    // only a slot that is still locked is given back its key
    // (core_kernels.cuh:1181-1204)
    ok = cas_acquire(p, t.locked_key, keys[i]) == t.locked_key;
  }
  if (success != nullptr) success[i] = ok;
}

// erase on tables whose buckets are not one 128-byte digest line (the others
// run mutate_kernel<kOpErase>): one warp per key; tombstone = RECLAIM key,
// reclaim digest, score 0, size - 1 (core_kernels.cuh:680-734).
__global__ void __launch_bounds__(kMutateBlock)
    erase_kernel(const TableView t, uint64_t n, const uint64_t* keys) {
  const uint32_t lane = threadIdx.x & 31u;
  const uint64_t warp = (uint64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (warp >= n) return;
  const uint64_t key = keys[warp];
  if (is_reserved(t, key)) return;
  const Address a = locate(t, key);
  const uint64_t slot0 = a.bucket << t.bucket_shift;
  // four digests per lane, 128 slots per step
  for (uint32_t first = 0; first < t.bucket_slots; first += 128u) {
    const uint32_t at = first + lane * 4u;
    bool erased = false;
    if (at < t.bucket_slots) {
      const uint32_t d4 = *reinterpret_cast<const uint32_t*>(t.digests + slot0 + at);
      uint32_t m = match4(d4, replicate4(a.digest));
      while (m) {
        const uint32_t pos = at + (__ffs(m) - 1);
        m &= m - 1;
        if (cas_acquire(key_ptr(t, slot0 + pos), key, t.locked_key) == key) {
          st_u8_cg(t.digests + slot0 + pos, t.reclaim_digest);
          st_relaxed(score_ptr(t, slot0 + pos), 0);
          atomicSub(t.bucket_sizes + a.bucket, 1);
          st_release(key_ptr(t, slot0 + pos), t.reclaim_key);
          erased = true;
          break;
        }
      }
    }
    if (__any_sync(0xFFFFFFFFu, erased)) break;
  }
}

// ---- dual-bucket tables (TableMode::kMemory) ----------------------------------------
//
// insert_or_assign of unique keys on a table where a key may live in one of
// two buckets (include/merlin/core_kernels/dual_bucket_upsert.cuh:27-48):
//   0  the key is looked for in BOTH buckets before anything is claimed;
//   1  a new key goes to the emptier bucket (the first one on a tie), into the
//      first EMPTY slot from its start position there, else into the other;
//   2  with both buckets full the entry with the smallest score of the two
//      buckets (the first bucket on a tie) is evicted, unless the new score is
//      below it.
// One warp walks its 32 keys one after the other, reading both buckets' 128
// keys directly (4 per lane and bucket).
struct BucketScan {
  uint32_t eq;      // bit c: slot c * 32 + lane holds the key
  uint32_t locked;  // bit c: that slot is LOCKED
  uint32_t empty;   // bit c: that slot is EMPTY
};

__device__ __forceinline__ BucketScan scan_bucket_keys(const TableView& t, uint64_t slot0,
                                                       uint64_t key, uint32_t lane) {
  BucketScan r{0, 0, 0};
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint64_t k = ld_acquire(key_ptr(t, slot0 + c * 32 + lane));
    r.eq |= (k == key) ? (1u << c) : 0u;
    r.locked |= (k == t.locked_key) ? (1u << c) : 0u;
    r.empty |= (k == t.empty_key) ? (1u << c) : 0u;
  }
  return r;
}

// Distance from `start` to the first EMPTY slot of the scan (255: none).
__device__ __forceinline__ uint32_t first_empty_distance(const BucketScan& s, uint32_t start,
                                                         uint32_t lane) {
  uint32_t best = 255u;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    if ((s.empty >> c) & 1u) {
      best = min(best, (uint32_t(c) * 32u + lane - start) & (kBucketSlots - 1));
    }
  }
  return __reduce_min_sync(0xFFFFFFFFu, best);
}

// Minimum score of a bucket and its first position.
__device__ __forceinline__ void bucket_min_score(const TableView& t, uint64_t slot0, uint32_t lane,
                                                 uint64_t* gmin, uint32_t* gpos) {
  uint64_t ms = kMaxScore;
  uint32_t mp = 255u;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint64_t s = ld_relaxed(score_ptr(t, slot0 + c * 32 + lane));
    if (mp == 255u || s < ms) {
      ms = s;
      mp = c * 32 + lane;
    }
  }
  const uint32_t hi = uint32_t(ms >> 32);
  const uint32_t ghi = __reduce_min_sync(0xFFFFFFFFu, hi);
  const uint32_t lo = hi == ghi ? uint32_t(ms) : 0xFFFFFFFFu;
  const uint32_t glo = __reduce_min_sync(0xFFFFFFFFu, lo);
  const uint32_t cp = (hi == ghi && lo == glo) ? mp : 255u;
  *gpos = __reduce_min_sync(0xFFFFFFFFu, cp);
  *gmin = (uint64_t(ghi) << 32) | glo;
}

__global__ void __launch_bounds__(kMutateBlock)
    dual_upsert_kernel(const TableView t, const MutateArgs args) {
  const uint32_t full = 0xFFFFFFFFu;
  const uint32_t lane = threadIdx.x & 31u;
  const uint64_t warp = (uint64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const uint64_t base = warp * 32u;
  const uint64_t n = args.n;
  if (base >= n) return;
  const int strategy = args.strategy;
  const uint32_t count = uint32_t(min(uint64_t(32), n - base));

  for (uint32_t q = 0; q < count; ++q) {
    const uint64_t i = base + q;
    const uint64_t key = args.keys[i];
    if (is_reserved(t, key)) continue;
    const DualAddress a = locate_dual(t, key);
    const uint64_t in_score = args.scores != nullptr ? args.scores[i] : 0;
    const uint64_t desired = desired_score(strategy, args.scores, in_score, args.epoch);
    const uint64_t slot0[2] = {a.first.bucket << 7, a.second.bucket << 7};
    const uint32_t start[2] = {a.first.start, a.second.start};
    const uint64_t bucket[2] = {a.first.bucket, a.second.bucket};

    uint32_t result = kInitial;
    uint32_t which = 0, pos = 0;
    uint64_t victim = 0;
    uint32_t attempts = 0;
    while (result == kInitial) {
      if (++attempts > kRescanLimit) {
        if (lane == 0) atomicOr(t.status, kStatusLockTimeout);
        result = kRefused;
        break;
      }
      const BucketScan s0 = scan_bucket_keys(t, slot0[0], key, lane);
      const BucketScan s1 = scan_bucket_keys(t, slot0[1], key, lane);
      // phase 0: the key itself, in either bucket
      const uint32_t eq0 = __ballot_sync(full, s0.eq != 0);
      const uint32_t eq1 = __ballot_sync(full, s1.eq != 0);
      if (eq0 | eq1) {
        const uint32_t w = eq0 ? 0u : 1u;
        const uint32_t src = __ffs(eq0 ? eq0 : eq1) - 1;
        const uint32_t mine = (__ffs(w == 0 ? s0.eq : s1.eq) - 1) * 32 + lane;
        const uint32_t p = __shfl_sync(full, mine, src);
        uint32_t ok = 0;
        if (lane == src) ok = cas_acquire(key_ptr(t, slot0[w] + p), key, t.locked_key) == key;
        if (__shfl_sync(full, ok, src)) {
          result = kDuplicate;
          which = w;
          pos = p;
        }
        continue;
      }
      if (__ballot_sync(full, (s0.locked | s1.locked) != 0)) {
        __nanosleep(128);  // somebody is writing one of these buckets
        continue;
      }
      // phase 1: the emptier bucket first
      const int size0 = *reinterpret_cast<volatile int32_t*>(t.bucket_sizes + bucket[0]);
      const int size1 = *reinterpret_cast<volatile int32_t*>(t.bucket_sizes + bucket[1]);
      const uint32_t prefer = size0 <= size1 ? 0u : 1u;
      bool retry = false;
      for (uint32_t turn = 0; turn < 2 && result == kInitial && !retry; ++turn) {
        const uint32_t w = turn == 0 ? prefer : 1u - prefer;
        if ((w == 0 ? size0 : size1) >= kBucketSlots) continue;
        const uint32_t d = first_empty_distance(w == 0 ? s0 : s1, start[w], lane);
        if (d == 255u) continue;
        const uint32_t p = (start[w] + d) & (kBucketSlots - 1);
        uint32_t ok = 0;
        if (lane == 0) {
          ok = cas_acquire(key_ptr(t, slot0[w] + p), t.empty_key, t.locked_key) == t.empty_key;
        }
        if (__shfl_sync(full, ok, 0)) {
          result = kOccupiedEmpty;
          which = w;
          pos = p;
        } else {
          retry = true;  // lost the slot to another warp: look again
        }
      }
      if (result != kInitial || retry) continue;
      // phase 2: the smallest score of both buckets
      uint64_t min0, min1;
      uint32_t pos0, pos1;
      bucket_min_score(t, slot0[0], lane, &min0, &pos0);
      bucket_min_score(t, slot0[1], lane, &min1, &pos1);
      const uint32_t w = min0 <= min1 ? 0u : 1u;
      const uint64_t gmin = w == 0 ? min0 : min1;
      const uint32_t gpos = w == 0 ? pos0 : pos1;
      if (desired < gmin) {
        result = kRefused;
        break;
      }
      uint32_t code = 0;
      if (lane == 0) {
        uint64_t* kp = key_ptr(t, slot0[w] + gpos);
        const uint64_t v = ld_relaxed(kp);
        if (v != t.locked_key && cas_acquire(kp, v, t.locked_key) == v) {
          if (ld_relaxed(score_ptr(t, slot0[w] + gpos)) > gmin) {
            st_release(kp, v);  // refreshed in between: scan again
          } else {
            victim = v;
            code = (v == t.empty_key || v == t.reclaim_key) ? 2 : 1;
          }
        }
      }
      code = __shfl_sync(full, code, 0);
      if (code) {
        result = code == 2 ? kOccupiedReclaimed : kEvict;
        which = w;
        pos = gpos;
      }
    }
    if (result == kRefused || result == kInitial) continue;

    const uint32_t slot = uint32_t(slot0[which]) + pos;
    if (lane == 0) {
      if (result == kDuplicate) {
        const uint64_t old_score = ld_relaxed(score_ptr(t, slot));
        uint64_t ns = 0;
        if (hit_score_upsert(strategy, args.scores, in_score, desired, old_score, &ns)) {
          st_relaxed(score_ptr(t, slot), ns);
        }
      } else {
        st_u8_cg(t.digests + slot, a.first.digest);
        st_relaxed(score_ptr(t, slot), inserted_score(strategy, in_score, desired));
        if (result != kEvict) atomicAdd(t.bucket_sizes + bucket[which], 1);
      }
    }
    warp_copy_one_row<0>(t, row_ptr(t, slot), args.values + i * t.row_bytes, lane);
    __syncwarp();
    if (lane == 0) {
      __threadfence();
      st_release(key_ptr(t, slot), key);
    }
    __syncwarp();
  }
}

template <int OP>
void launch_fast(const TableView& t, const MutateArgs& args, uint64_t blocks, cudaStream_t stream) {
  auto kernel = fast_rows(t) ? mutate_kernel<OP, 16, false> : mutate_kernel<OP, 0, false>;
  kernel<<<static_cast<unsigned>(blocks), kMutateBlock, 0, stream>>>(t, args);
}

template <int OP>
void launch_op(const TableView& t, const MutateArgs& args, bool unique_key, cudaStream_t stream,
               void* scratch) {
  const uint64_t warps = (args.n + 31) / 32;
  const uint64_t blocks = (warps * 32 + kMutateBlock - 1) / kMutateBlock;
  if (!line_buckets(t)) {
    // buckets that are not one 128-byte digest line: the serialising kernel
    // walks buckets of any size (the reference's own fallback for them are its
    // tile kernels, e.g. include/merlin/core_kernels/upsert.cuh:1233-1305)
    mutate_serial_kernel<OP><<<static_cast<unsigned>(blocks), kMutateBlock, 0, stream>>>(t, args);
  } else if (unique_key) {
    launch_fast<OP>(t, args, blocks, stream);
  } else if (OP != kOpFindOrInsertPtr && OP != kOpLockKeys && args.n < (1ull << 32)) {
    // Repeated keys are allowed.  The fast kernel serves every key it finds
    // and can lock; keys that have to be inserted and keys whose slot another
    // occurrence held at that moment are listed and served by the serialising
    // kernel afterwards (an empty list costs one launch that exits at once).
    uint8_t* work = static_cast<uint8_t*>(scratch);
    if (work == nullptr) {
      mutate_serial_kernel<OP><<<static_cast<unsigned>(blocks), kMutateBlock, 0, stream>>>(t, args);
      return;
    }
    unsigned int* count = reinterpret_cast<unsigned int*>(work);
    uint32_t* list = reinterpret_cast<uint32_t*>(work + 256);
    cudaMemsetAsync(count, 0, sizeof(unsigned int), stream);
    MutateArgs fast = args;
    fast.deferred_list = list;
    fast.deferred_count = count;
    launch_fast<OP>(t, fast, blocks, stream);
    MutateArgs rest = args;
    rest.index_list = list;
    rest.index_count = count;
    mutate_serial_kernel<OP><<<static_cast<unsigned>(blocks), kMutateBlock, 0, stream>>>(t, rest);
  } else {
    mutate_serial_kernel<OP><<<static_cast<unsigned>(blocks), kMutateBlock, 0, stream>>>(t, args);
  }
}

}  // namespace

size_t mutate_workspace_bytes(int op, uint64_t n, bool unique_key) {
  if (unique_key || op == kOpFindOrInsertPtr || op == kOpLockKeys || n >= (1ull << 32)) return 0;
  return n * sizeof(uint32_t) + 256;   // counter | list of deferred batch positions
}

void launch_mutate(int op, const TableView& t, const MutateArgs& args, bool unique_key,
                   cudaStream_t stream, void* work) {
  if (args.n == 0) return;
  switch (op) {
    case kOpInsertOrAssign: launch_op<kOpInsertOrAssign>(t, args, unique_key, stream, work); break;
    case kOpFindOrInsert: launch_op<kOpFindOrInsert>(t, args, unique_key, stream, work); break;
    case kOpInsertAndEvict: launch_op<kOpInsertAndEvict>(t, args, unique_key, stream, work); break;
    case kOpFindOrInsertPtr: launch_op<kOpFindOrInsertPtr>(t, args, unique_key, stream, work); break;
    case kOpAccumOrAssign: launch_op<kOpAccumOrAssign>(t, args, unique_key, stream, work); break;
    case kOpAssign: launch_op<kOpAssign>(t, args, unique_key, stream, work); break;
    case kOpAssignScores: launch_op<kOpAssignScores>(t, args, unique_key, stream, work); break;
    case kOpAssignValues: launch_op<kOpAssignValues>(t, args, unique_key, stream, work); break;
    case kOpFindAndUpdate: launch_op<kOpFindAndUpdate>(t, args, unique_key, stream, work); break;
    case kOpLockKeys: launch_op<kOpLockKeys>(t, args, unique_key, stream, work); break;
    default: break;
  }
}

template <int OP>
void launch_routed_op(const TableView& t, const MutateArgs& args, const RoutedArgs& r,
                      cudaStream_t stream) {
  // the key counts are only known on the device: grids of resident blocks
  // stride over whatever arrived
  int device = 0, sms = 148;
  cudaGetDevice(&device);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  const uint64_t tiles = ((r.segment_capacity + kMutateBlock - 1) / kMutateBlock) * r.world;
  const uint64_t resident = uint64_t(sms) * routed_min_blocks(OP);
  const unsigned blocks = static_cast<unsigned>(tiles < resident ? tiles : resident);
  const unsigned scan_blocks = static_cast<unsigned>(tiles < uint64_t(sms) * 16 ? tiles : sms * 16);
  routed_group_kernel<<<scan_blocks, kMutateBlock, 0, stream>>>(t, r);
  routed_resolve_kernel<<<scan_blocks, kMutateBlock, 0, stream>>>(t, r, OP == kOpAccumOrAssign);
  auto kernel = fast_rows(t) ? mutate_routed_kernel<OP, 16> : mutate_routed_kernel<OP, 0>;
  kernel<<<blocks, kMutateBlock, 0, stream>>>(t, args, r);
}

size_t routed_workspace_bytes(uint32_t world, uint64_t segment_capacity) {
  const uint64_t entries = uint64_t(world) * segment_capacity;
  uint32_t bits = 10;
  while (bits < 31 && (1ull << bits) < 2 * entries) ++bits;
  const uint64_t places = 1ull << bits;
  return places * sizeof(uint64_t) + entries * sizeof(uint64_t) + places * sizeof(uint32_t) +
         3 * entries * sizeof(uint32_t) + 1024;
}

void prepare_routed_workspace(const TableView& t, RoutedArgs& r, void* work, bool fresh,
                              cudaStream_t stream) {
  const uint64_t entries = uint64_t(r.world) * r.segment_capacity;
  uint32_t bits = 10;
  while (bits < 31 && (1ull << bits) < 2 * entries) ++bits;
  const uint64_t places = 1ull << bits;
  uint8_t* at = static_cast<uint8_t*>(work);
  r.set_keys = reinterpret_cast<uint64_t*>(at);
  at += places * sizeof(uint64_t);
  r.plan = reinterpret_cast<uint64_t*>(at);
  at += entries * sizeof(uint64_t);
  r.set_head = reinterpret_cast<uint32_t*>(at);
  at += places * sizeof(uint32_t);
  r.next = reinterpret_cast<uint32_t*>(at);
  at += entries * sizeof(uint32_t);
  r.set_slot = reinterpret_cast<uint32_t*>(at);
  at += entries * sizeof(uint32_t);
  r.lists = reinterpret_cast<uint32_t*>(at);
  at += entries * sizeof(uint32_t);
  r.list_cursor = reinterpret_cast<uint32_t*>(at);
  r.set_bits = bits;
  if (fresh) {
    routed_fill_kernel<<<1184, 256, 0, stream>>>(r.set_keys, r.set_head, places, t.empty_key);
    cudaMemsetAsync(r.list_cursor, 0, sizeof(uint32_t), stream);
  }
}

void launch_mutate_routed(int op, const TableView& t, const MutateArgs& args, const RoutedArgs& r,
                          cudaStream_t stream) {
  if (r.segment_capacity == 0 || r.world == 0) return;
  switch (op) {
    case kOpInsertOrAssign: launch_routed_op<kOpInsertOrAssign>(t, args, r, stream); break;
    case kOpFindOrInsert: launch_routed_op<kOpFindOrInsert>(t, args, r, stream); break;
    case kOpAccumOrAssign: launch_routed_op<kOpAccumOrAssign>(t, args, r, stream); break;
    default: break;
  }
}

void launch_dual_upsert(const TableView& t, const MutateArgs& args, cudaStream_t stream) {
  if (args.n == 0) return;
  const uint64_t blocks = (((args.n + 31) / 32) * 32 + kMutateBlock - 1) / kMutateBlock;
  dual_upsert_kernel<<<static_cast<unsigned>(blocks), kMutateBlock, 0, stream>>>(t, args);
}

void launch_unlock_keys(const TableView& t, uint64_t n, uint64_t** locked_key_ptrs,
                        const uint64_t* keys, bool* success, cudaStream_t stream) {
  if (n == 0) return;
  unlock_keys_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(
      t, n, locked_key_ptrs, keys, success);
}

void launch_erase(const TableView& t, uint64_t n, const uint64_t* keys, cudaStream_t stream) {
  if (n == 0) return;
  if (line_buckets(t)) {
    // 32 keys per warp on the 8-lane digest probe, like every other keyed operation
    MutateArgs args;
    args.keys = keys;
    args.n = n;
    const uint64_t fast_blocks = (((n + 31) / 32) * 32 + kMutateBlock - 1) / kMutateBlock;
    launch_fast<kOpErase>(t, args, fast_blocks, stream);
    return;
  }
  const uint64_t blocks = (n * 32 + kMutateBlock - 1) / kMutateBlock;
  erase_kernel<<<static_cast<unsigned>(blocks), kMutateBlock, 0, stream>>>(t, n, keys);
}

}  // namespace hkv
