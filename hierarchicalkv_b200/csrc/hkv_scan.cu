// Whole-table scans: export_batch / export_batch_if, size_if, size, clear.
//
// Replaces the reference's
//   include/merlin/core_kernels.cuh:859-912   dump_kernel      (export_batch)
//   include/merlin/core_kernels.cuh:983-1041  dump_kernel_v2   (export_batch_if)
//   include/merlin/core_kernels.cuh:1116-1151 size_if_kernel
//   include/merlin/core_kernels.cuh:657-676   clear_kernel
//   include/merlin/core_kernels.cuh:1396-1423 SumOp            (size)
//   include/merlin/core_kernels.cuh:385-401, 531-590  double_capacity +
//                                             rehash_kernel_for_fast_mode (reserve)
//
// Export is a compacting scan: a block of 256 threads reads 256 consecutive
// slots (keys and scores are linear planes, so these are two fully coalesced
// 2 KiB reads), every warp ballots its survivors, the block takes ONE ticket
// range from the global counter, and each warp gathers its survivors' rows
// with the same coalesced row mover the lookups use.
#include "hkv_device.cuh"
#include "hkv_internal.h"

namespace hkv {

namespace {

constexpr int kScanBlock = 256;
constexpr int kScanWarps = kScanBlock / 32;

__device__ __forceinline__ bool keep(const TableView& t, int pred, uint64_t key, uint64_t score,
                                     uint64_t pattern, uint64_t threshold) {
  if (is_reserved(t, key)) return false;
  switch (pred) {
    case kPredAll: return true;
    case kPredScoreLess: return score < threshold;
    case kPredScoreGreaterEq: return score >= threshold;
    case kPredKeyMaskEq: return (key & threshold) == pattern;
    case kPredScoreGreater: return score > threshold;
    case kPredScoreLessEq: return score <= threshold;
    default: return false;
  }
}

__global__ void __launch_bounds__(kScanBlock)
    export_kernel(const TableView t, const int pred, const uint64_t pattern,
                  const uint64_t threshold, const uint64_t n, const uint64_t offset,
                  unsigned long long* __restrict__ d_counter, uint64_t* __restrict__ out_keys,
                  uint8_t* __restrict__ out_values, uint64_t* __restrict__ out_scores) {
  __shared__ uint32_t warp_count[kScanWarps];
  __shared__ unsigned long long block_base;
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t wid = threadIdx.x >> 5;
  const uint64_t tiles = (n + kScanBlock - 1) / kScanBlock;
  for (uint64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    const uint64_t rel = tile * kScanBlock + threadIdx.x;
    const uint64_t slot = offset + rel;
    uint64_t key = t.empty_key;
    uint64_t score = 0;
    bool live = false;
    if (rel < n) {
      key = __ldcs(key_ptr(t, slot));
      score = __ldcs(score_ptr(t, slot));
      live = keep(t, pred, key, score, pattern, threshold);
    }
    const uint32_t votes = __ballot_sync(0xFFFFFFFFu, live);
    if (lane == 0) warp_count[wid] = __popc(votes);
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t total = 0;
#pragma unroll
      for (int w = 0; w < kScanWarps; ++w) total += warp_count[w];
      block_base = total ? atomicAdd(d_counter, (unsigned long long)total) : 0ull;
    }
    __syncthreads();
    uint64_t at = block_base;
    for (uint32_t w = 0; w < wid; ++w) at += warp_count[w];
    __syncthreads();  // warp_count / block_base are rewritten by the next tile
    if (votes) {
      const uint32_t mine = __popc(votes & ((1u << lane) - 1u));
      if (live) {
        __stcs(out_keys + at + mine, key);
        if (out_scores != nullptr) __stcs(out_scores + at + mine, score);
      }
      if (out_values != nullptr) {
        // lane r carries the slot of the r-th survivor
        const uint32_t src = __fns(votes, 0, lane + 1);
        const uint32_t s = __shfl_sync(0xFFFFFFFFu, uint32_t(slot), src & 31u);
        warp_move_rows<0>(t, out_values + at * t.row_bytes, src == 0xFFFFFFFFu ? kNoSlot : s,
                          lane);
      }
    }
  }
}

__global__ void __launch_bounds__(kScanBlock)
    size_if_kernel(const TableView t, const int pred, const uint64_t pattern,
                   const uint64_t threshold, unsigned long long* __restrict__ d_counter) {
  unsigned long long local = 0;
  for (uint64_t slot = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; slot < t.capacity;
       slot += uint64_t(gridDim.x) * blockDim.x) {
    const uint64_t key = __ldcs(key_ptr(t, slot));
    const uint64_t score = __ldcs(score_ptr(t, slot));
    local += keep(t, pred, key, score, pattern, threshold) ? 1 : 0;
  }
  for (int o = 16; o > 0; o >>= 1) local += __shfl_down_sync(0xFFFFFFFFu, local, o);
  if ((threadIdx.x & 31u) == 0 && local) atomicAdd(d_counter, local);
}

// erase_if: every live slot the predicate selects becomes a tombstone (RECLAIM
// key, reclaim digest, score 0), as remove_kernel does
// (include/merlin/core_kernels.cuh:736-792).  Runs under the exclusive lock.
__global__ void __launch_bounds__(kScanBlock)
    erase_if_kernel(const TableView t, const int pred, const uint64_t pattern,
                    const uint64_t threshold, unsigned long long* __restrict__ d_counter) {
  unsigned long long local = 0;
  for (uint64_t slot = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; slot < t.capacity;
       slot += uint64_t(gridDim.x) * blockDim.x) {
    const uint64_t key = *key_ptr(t, slot);
    const uint64_t score = *score_ptr(t, slot);
    if (keep(t, pred, key, score, pattern, threshold)) {
      *key_ptr(t, slot) = t.reclaim_key;
      t.digests[slot] = static_cast<uint8_t>(t.reclaim_digest);
      *score_ptr(t, slot) = 0;
      atomicSub(t.bucket_sizes + (slot >> t.bucket_shift), 1);
      ++local;
    }
  }
  for (int o = 16; o > 0; o >>= 1) local += __shfl_down_sync(0xFFFFFFFFu, local, o);
  if ((threadIdx.x & 31u) == 0 && local) atomicAdd(d_counter, local);
}

__global__ void __launch_bounds__(kScanBlock)
    sum_sizes_kernel(const TableView t, const uint64_t buckets,
                     unsigned long long* __restrict__ d_total) {
  unsigned long long local = 0;
  for (uint64_t b = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; b < buckets;
       b += uint64_t(gridDim.x) * blockDim.x) {
    local += static_cast<unsigned long long>(t.bucket_sizes[b]);
  }
  for (int o = 16; o > 0; o >>= 1) local += __shfl_down_sync(0xFFFFFFFFu, local, o);
  if ((threadIdx.x & 31u) == 0 && local) atomicAdd(d_total, local);
}

__global__ void __launch_bounds__(kScanBlock) clear_kernel(const TableView t) {
  // one thread per 16 slots: a 16-byte digest store, 16 keys and 16 scores
  const uint64_t groups = t.capacity / 16;
  for (uint64_t g = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; g < groups;
       g += uint64_t(gridDim.x) * blockDim.x) {
    const uint32_t d = t.empty_digest4;
    reinterpret_cast<uint4*>(t.digests)[g] = make_uint4(d, d, d, d);
    // slots 16g .. 16g+15, two at a time (an even slot's words are 16-byte aligned
    // in both layouts)
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const uint64_t slot = g * 16 + 2 * q;
      *reinterpret_cast<ulonglong2*>(key_ptr(t, slot)) = make_ulonglong2(t.empty_key, t.empty_key);
      *reinterpret_cast<ulonglong2*>(score_ptr(t, slot)) = make_ulonglong2(0ull, 0ull);
    }
    // the thread that clears a bucket's first 16 slots also clears its size
    const uint64_t groups_per_bucket = t.bucket_slots / 16u;
    if (g % groups_per_bucket == 0) t.bucket_sizes[g / groups_per_bucket] = 0;
  }
}

// Doubling rehash.  `dst` has twice the buckets of `src` and was cleared.  With
// a power-of-two capacity a key of old bucket b lands in new bucket b or
// b + src.buckets, so one block owns one old bucket and both of its targets
// and no atomics are needed: thread i carries old slot i, the live keys of each
// side are ranked in slot order with ballots, and the new position is the rank
// (a compacted bucket; tombstones are dropped).  Lookups and inserts probe the
// whole digest line, so any position inside the bucket is valid.  Rows are then
// copied one per warp instruction group, coalesced.
// The block has max(32, bucket_slots) threads; thread i carries old slot i.
constexpr int kRehashMaxWarps = kMaxBucketSlots / 32;

__global__ void __launch_bounds__(kMaxBucketSlots)
    rehash_kernel(const TableView src, const TableView dst) {
  __shared__ uint32_t side_count[2][kRehashMaxWarps];
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t wid = threadIdx.x >> 5;
  const uint32_t warps = blockDim.x >> 5;
  const uint32_t below = (1u << lane) - 1u;
  for (uint64_t b = blockIdx.x; b < src.buckets; b += gridDim.x) {
    const bool in_bucket = threadIdx.x < src.bucket_slots;
    const uint64_t slot = b * src.bucket_slots + (in_bucket ? threadIdx.x : 0u);
    const uint64_t key = in_bucket ? *key_ptr(src, slot) : src.empty_key;
    const bool live = !is_reserved(src, key);
    const Address a = locate(dst, key);
    const bool high = live && a.bucket != b;
    const uint32_t votes_low = __ballot_sync(0xFFFFFFFFu, live && !high);
    const uint32_t votes_high = __ballot_sync(0xFFFFFFFFu, high);
    if (lane == 0) {
      side_count[0][wid] = __popc(votes_low);
      side_count[1][wid] = __popc(votes_high);
    }
    __syncthreads();
    uint32_t rank = __popc((high ? votes_high : votes_low) & below);
    for (uint32_t w = 0; w < wid; ++w) rank += side_count[high ? 1 : 0][w];
    uint64_t to = 0;
    if (live) {
      to = a.bucket * dst.bucket_slots + rank;
      *key_ptr(dst, to) = key;
      dst.digests[to] = static_cast<uint8_t>(a.digest);
      *score_ptr(dst, to) = *score_ptr(src, slot);
    }
    if (threadIdx.x < 2) {
      uint32_t total = 0;
      for (uint32_t w = 0; w < warps; ++w) total += side_count[threadIdx.x][w];
      dst.bucket_sizes[b + threadIdx.x * src.buckets] = static_cast<int32_t>(total);
    }
    // rows: the warp walks its live lanes; all 32 lanes copy one row together
    uint32_t todo = votes_low | votes_high;
    while (todo) {
      const uint32_t r = __ffs(todo) - 1;
      todo &= todo - 1;
      const uint64_t from_slot = __shfl_sync(0xFFFFFFFFu, slot, r);
      const uint64_t to_slot = __shfl_sync(0xFFFFFFFFu, to, r);
      const uint8_t* from_row = row_ptr(src, from_slot);
      uint8_t* to_row = row_ptr(dst, to_slot);
      if (src.vec_bytes == 16) {
        for (uint32_t off = lane * 16; off < src.row_bytes; off += 32 * 16) {
          *reinterpret_cast<uint4*>(to_row + off) = *reinterpret_cast<const uint4*>(from_row + off);
        }
      } else {
        for (uint32_t off = lane; off < src.row_bytes; off += 32) to_row[off] = from_row[off];
      }
    }
    __syncthreads();  // side_count is rewritten by the next bucket
  }
}

// ---- hybrid tables: which row block holds which bucket ------------------------
__global__ void __launch_bounds__(kScanBlock) identity_map_kernel(const TableView t) {
  for (uint64_t b = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; b < t.buckets;
       b += uint64_t(gridDim.x) * blockDim.x) {
    t.bucket_map[b] = static_cast<uint32_t>(b);
    t.bucket_heat[b] = 0;
  }
}

// Hit counters fade: what was hot before the previous promotion counts half.
__global__ void __launch_bounds__(kScanBlock) decay_heat_kernel(const TableView t) {
  for (uint64_t b = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; b < t.buckets;
       b += uint64_t(gridDim.x) * blockDim.x) {
    t.bucket_heat[b] >>= 1;
  }
}

// One block per pair (a, b) of buckets: the two buckets trade row blocks --
// the rows of each are copied to the other's place (16-byte chunks,
// coalesced; one of the two places is pinned host memory) and the map entries
// are exchanged.  Runs under the exclusive lock.
__global__ void __launch_bounds__(kScanBlock)
    swap_row_blocks_kernel(const TableView t, const uint32_t* __restrict__ pairs,
                           const uint64_t n_pairs) {
  const uint64_t block_bytes = uint64_t(t.bucket_slots) * t.row_bytes;
  for (uint64_t p = blockIdx.x; p < n_pairs; p += gridDim.x) {
    const uint32_t a = pairs[2 * p], b = pairs[2 * p + 1];
    const uint32_t place_a = t.bucket_map[a], place_b = t.bucket_map[b];
    uint8_t* rows_a = row_ptr_of_row_slot(t, uint64_t(place_a) << t.bucket_shift);
    uint8_t* rows_b = row_ptr_of_row_slot(t, uint64_t(place_b) << t.bucket_shift);
    if (t.row_bytes % 16 == 0) {
      for (uint64_t off = uint64_t(threadIdx.x) * 16; off < block_bytes;
           off += uint64_t(blockDim.x) * 16) {
        const uint4 x = *reinterpret_cast<const uint4*>(rows_a + off);
        const uint4 y = *reinterpret_cast<const uint4*>(rows_b + off);
        *reinterpret_cast<uint4*>(rows_a + off) = y;
        *reinterpret_cast<uint4*>(rows_b + off) = x;
      }
    } else {
      for (uint64_t off = threadIdx.x; off < block_bytes; off += blockDim.x) {
        const uint8_t x = rows_a[off], y = rows_b[off];
        rows_a[off] = y;
        rows_b[off] = x;
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      t.bucket_map[a] = place_b;
      t.bucket_map[b] = place_a;
    }
    __syncthreads();
  }
}

// 32-bit score arrays at the API boundary <-> the 64-bit scores the kernels use.
__global__ void __launch_bounds__(kScanBlock)
    widen_scores_kernel(const uint32_t* __restrict__ in, uint64_t* __restrict__ out, uint64_t n) {
  for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += uint64_t(gridDim.x) * blockDim.x) {
    out[i] = in[i];
  }
}

__global__ void __launch_bounds__(kScanBlock)
    narrow_scores_kernel(const uint64_t* __restrict__ in, uint32_t* __restrict__ out, uint64_t n) {
  for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += uint64_t(gridDim.x) * blockDim.x) {
    out[i] = static_cast<uint32_t>(in[i]);
  }
}

unsigned scan_grid(uint64_t items_per_block_pass, uint64_t items) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const uint64_t want = (items + items_per_block_pass - 1) / items_per_block_pass;
  const uint64_t cap = uint64_t(sms) * 8;  // 8 resident blocks of 256 threads per SM
  return static_cast<unsigned>(want < cap ? (want ? want : 1) : cap);
}

}  // namespace

void launch_export(const TableView& t, int pred, uint64_t pattern, uint64_t threshold, uint64_t n,
                   uint64_t offset, unsigned long long* d_counter, uint64_t* keys, void* values,
                   uint64_t* scores, cudaStream_t stream) {
  if (n == 0) return;
  export_kernel<<<scan_grid(kScanBlock, n), kScanBlock, 0, stream>>>(
      t, pred, pattern, threshold, n, offset, d_counter, keys, static_cast<uint8_t*>(values),
      scores);
}

void launch_size_if(const TableView& t, int pred, uint64_t pattern, uint64_t threshold,
                    unsigned long long* d_counter, cudaStream_t stream) {
  size_if_kernel<<<scan_grid(kScanBlock * 4, t.capacity), kScanBlock, 0, stream>>>(
      t, pred, pattern, threshold, d_counter);
}

void launch_erase_if(const TableView& t, int pred, uint64_t pattern, uint64_t threshold,
                     unsigned long long* d_counter, cudaStream_t stream) {
  erase_if_kernel<<<scan_grid(kScanBlock * 4, t.capacity), kScanBlock, 0, stream>>>(
      t, pred, pattern, threshold, d_counter);
}

void launch_clear(const TableView& t, cudaStream_t stream) {
  clear_kernel<<<scan_grid(kScanBlock, t.capacity / 16), kScanBlock, 0, stream>>>(t);
}

void launch_sum_sizes(const TableView& t, uint64_t buckets, unsigned long long* d_total,
                      cudaStream_t stream) {
  sum_sizes_kernel<<<scan_grid(kScanBlock * 4, buckets), kScanBlock, 0, stream>>>(t, buckets,
                                                                                  d_total);
}

void launch_identity_map(const TableView& t, cudaStream_t stream) {
  identity_map_kernel<<<scan_grid(kScanBlock * 4, t.buckets), kScanBlock, 0, stream>>>(t);
}

void launch_decay_heat(const TableView& t, cudaStream_t stream) {
  decay_heat_kernel<<<scan_grid(kScanBlock * 4, t.buckets), kScanBlock, 0, stream>>>(t);
}

void launch_swap_row_blocks(const TableView& t, const uint32_t* pairs, uint64_t n_pairs,
                            cudaStream_t stream) {
  if (n_pairs == 0) return;
  swap_row_blocks_kernel<<<scan_grid(1, n_pairs), kScanBlock, 0, stream>>>(t, pairs, n_pairs);
}

void launch_widen_scores(const uint32_t* in, uint64_t* out, uint64_t n, cudaStream_t stream) {
  if (n == 0) return;
  widen_scores_kernel<<<scan_grid(kScanBlock * 4, n), kScanBlock, 0, stream>>>(in, out, n);
}

void launch_narrow_scores(const uint64_t* in, uint32_t* out, uint64_t n, cudaStream_t stream) {
  if (n == 0) return;
  narrow_scores_kernel<<<scan_grid(kScanBlock * 4, n), kScanBlock, 0, stream>>>(in, out, n);
}

void launch_rehash(const TableView& src, const TableView& dst, cudaStream_t stream) {
  const unsigned threads = src.bucket_slots < 32u ? 32u : src.bucket_slots;
  rehash_kernel<<<scan_grid(1, src.buckets), threads, 0, stream>>>(src, dst);
}

}  // namespace hkv
