// Drop-in replacement of the reference's include/merlin_hashtable.cuh for the
// hash-table hot path: same namespace, class, enum, option and method names,
// same defaults, same exception types.  Every method is a thin call into the
// C ABI of libhkv_b200.so (include/hkv_b200.h), where the sm_100a kernels live.
//
//   #include "merlin_hashtable.cuh"
//   using Table = nv::merlin::HashTable<uint64_t, float, uint64_t,
//                                       nv::merlin::EvictStrategy::kLru>;
//   Table t;  nv::merlin::HashTableOptions o;  ...  t.init(o);
//   t.insert_or_assign(n, d_keys, d_values, nullptr, stream);
//
// Link with -lhkv_b200.  User-templated functors (export_batch_if<Pred>,
// export_batch_if_v2, size_if<Pred>, erase_if<Pred>, erase_if_v2, for_each)
// are evaluated by small kernels in this header over the table's planes
// (hkv_get_view); everything else runs inside the library.
//
// Differences a caller can observe are listed in the integration notes shipped
// with the library.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstddef>
#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <vector>

#include "hkv_b200.h"
#include "merlin/allocator.cuh"
#include "merlin/debug.hpp"
#include "merlin/types.cuh"
#include "merlin/utils.cuh"

namespace nv {
namespace merlin {

// merlin_hashtable.cuh:79-87 of the reference
struct EvictStrategy {
  enum EvictStrategyEnum {
    kLru = 0,
    kLfu = 1,
    kEpochLru = 2,
    kEpochLfu = 3,
    kCustomized = 4,
  };
};

// merlin_hashtable.cuh:95-98
enum class TableMode {
  kThroughput = 0,
  kMemory = 1,
};

// merlin/memory_pool.cuh:139-143 -- kept so option structs written for the
// reference still compile; this library has no workspace pool to configure.
struct MemoryPoolOptions {
  size_t max_stock = 4;
  size_t max_pending = 16;
};

// merlin_hashtable.cuh:103-136, field for field (plus slot_layout at the end)
struct HashTableOptions {
  size_t init_capacity = 0;
  size_t max_capacity = 0;
  size_t max_hbm_for_vectors = 0;
  size_t max_bucket_size = 128;
  size_t dim = 64;
  float max_load_factor = 0.5f;
  int block_size = 128;
  int io_block_size = 1024;
  int device_id = -1;
  bool io_by_cpu = false;
  bool use_constant_memory = false;
  int reserved_key_start_bit = 0;
  size_t num_of_buckets_per_alloc = 1;
  bool api_lock = true;
  TableMode table_mode = TableMode::kThroughput;
  MemoryPoolOptions device_memory_pool;
  MemoryPoolOptions host_memory_pool;
  // Not in the reference (hkv_slot_layout): 0 keeps keys and scores in separate
  // arrays, 1 puts the keys of 8 slots and their scores into one 128-byte line,
  // which makes updates of resident keys faster and lookups and evictions slower.
  int slot_layout = 0;
};

// merlin_hashtable.cuh:173-179
template <class K, class S>
using EraseIfPredict = bool (*)(const K& key, S& score, const K& pattern, const S& threshold);

namespace detail {

// Rethrows a failed C-ABI call as the exception type the reference throws.
inline void rethrow(int rc) {
  if (rc == HKV_OK) return;
  const std::string msg = hkv_last_error();
  switch (rc) {
    case HKV_ERR_MERLIN: throw MerlinException(msg);
    case HKV_ERR_CUDA: throw CudaException(msg);
    case HKV_ERR_INVALID_ARG: throw std::invalid_argument(msg);
    default: throw std::runtime_error(msg);
  }
}

// hkv_value_kind of V: the element types accum_or_assign can add.
template <class V>
constexpr uint32_t value_kind_of() {
  if (std::is_same<V, float>::value) return HKV_VALUE_F32;
  if (std::is_same<V, double>::value) return HKV_VALUE_F64;
  if (std::is_integral<V>::value && sizeof(V) == 4) return HKV_VALUE_I32;
  if (std::is_integral<V>::value && sizeof(V) == 8) return HKV_VALUE_I64;
  if (std::is_same<V, __half>::value) return HKV_VALUE_F16;
  if (std::is_same<V, __nv_bfloat16>::value) return HKV_VALUE_BF16;
  return HKV_VALUE_OPAQUE;
}

// BaseAllocator* -> hkv_allocator trampolines.
inline int alloc_trampoline(void* ctx, int type, void** ptr, size_t size, unsigned int flags) {
  try {
    static_cast<BaseAllocator*>(ctx)->alloc(static_cast<MemoryType>(type), ptr, size, flags);
    return 0;
  } catch (...) {
    return 1;
  }
}
inline int free_trampoline(void* ctx, int type, void* ptr) {
  try {
    static_cast<BaseAllocator*>(ctx)->free(static_cast<MemoryType>(type), ptr);
    return 0;
  } catch (...) {
    return 1;
  }
}

__device__ __forceinline__ bool view_is_reserved(const hkv_table_view& v, uint64_t key) {
  return (key & v.reserved_mask) == v.reserved_value;
}

__device__ __forceinline__ const uint8_t* view_row(const hkv_table_view& v, uint64_t slot) {
  if (v.bucket_map != nullptr) {
    const uint64_t b = v.max_bucket_size;
    slot = uint64_t(v.bucket_map[slot / b]) * b + slot % b;
  }
  return slot < v.hbm_slots ? v.values_hbm + slot * v.row_bytes
                            : v.values_host + (slot - v.hbm_slots) * v.row_bytes;
}

// One row, all 32 lanes: 16-byte chunks when the row size and both addresses
// allow it, else elements of `elem` bytes.
__device__ __forceinline__ void copy_row(uint8_t* dst, const uint8_t* src, uint64_t row_bytes,
                                         uint32_t lane, uint32_t elem) {
  if (((row_bytes | reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15u) == 0) {
    for (uint64_t b = uint64_t(lane) * 16; b < row_bytes; b += 32 * 16) {
      *reinterpret_cast<uint4*>(dst + b) = *reinterpret_cast<const uint4*>(src + b);
    }
  } else if (elem == 4) {
    for (uint64_t b = uint64_t(lane) * 4; b < row_bytes; b += 32 * 4) {
      *reinterpret_cast<uint32_t*>(dst + b) = *reinterpret_cast<const uint32_t*>(src + b);
    }
  } else {
    for (uint64_t b = lane; b < row_bytes; b += 32) dst[b] = src[b];
  }
}

// export_batch_if<PredFunctor>: one warp per 32 consecutive slots, ballot,
// one ticket range per warp, rows copied by the whole warp.
template <class K, class V, class S, template <typename, typename> class PredFunctor>
__global__ void export_if_kernel(const hkv_table_view v, const K pattern, const S threshold,
                                 const uint64_t n, const uint64_t offset, size_t* d_counter,
                                 K* out_keys, V* out_values, S* out_scores) {
  PredFunctor<K, S> pred;
  const uint32_t lane = threadIdx.x & 31u;
  const uint64_t warps = (uint64_t(gridDim.x) * blockDim.x) >> 5;
  const uint64_t tiles = (n + 31) / 32;
  for (uint64_t tile = (uint64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; tile < tiles;
       tile += warps) {
    const uint64_t rel = tile * 32 + lane;
    const uint64_t slot = offset + rel;
    K key = 0;
    S score = 0;
    bool live = false;
    if (rel < n) {
      key = static_cast<K>(v.keys[HKV_SLOT_WORD(v, slot)]);
      score = static_cast<S>(v.scores[HKV_SLOT_WORD(v, slot)]);
      live = !view_is_reserved(v, static_cast<uint64_t>(key)) && pred(key, score, pattern, threshold);
    }
    const uint32_t votes = __ballot_sync(0xFFFFFFFFu, live);
    if (votes == 0) continue;
    unsigned long long at = 0;
    if (lane == 0) {
      at = atomicAdd(reinterpret_cast<unsigned long long*>(d_counter),
                     static_cast<unsigned long long>(__popc(votes)));
    }
    at = __shfl_sync(0xFFFFFFFFu, at, 0);
    const uint32_t mine = __popc(votes & ((1u << lane) - 1u));
    if (live) {
      out_keys[at + mine] = key;
      if (out_scores != nullptr) out_scores[at + mine] = score;
    }
    if (out_values != nullptr) {
      uint32_t left = votes;
      uint32_t rank = 0;
      while (left) {
        const uint32_t src = __ffs(left) - 1;
        left &= left - 1;
        const uint8_t* row = view_row(v, offset + tile * 32 + src);
        uint8_t* dst = reinterpret_cast<uint8_t*>(out_values) + (at + rank) * v.row_bytes;
        copy_row(dst, row, v.row_bytes, lane, sizeof(V));
        ++rank;
      }
    }
  }
}

template <class K, class S, template <typename, typename> class PredFunctor>
__global__ void size_if_kernel(const hkv_table_view v, const K pattern, const S threshold,
                               size_t* d_counter) {
  PredFunctor<K, S> pred;
  unsigned long long local = 0;
  for (uint64_t slot = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; slot < v.capacity;
       slot += uint64_t(gridDim.x) * blockDim.x) {
    K key = static_cast<K>(v.keys[HKV_SLOT_WORD(v, slot)]);
    S score = static_cast<S>(v.scores[HKV_SLOT_WORD(v, slot)]);
    if (!view_is_reserved(v, static_cast<uint64_t>(key)) && pred(key, score, pattern, threshold)) {
      ++local;
    }
  }
  for (int o = 16; o > 0; o >>= 1) local += __shfl_down_sync(0xFFFFFFFFu, local, o);
  if ((threadIdx.x & 31u) == 0 && local) {
    atomicAdd(reinterpret_cast<unsigned long long*>(d_counter), local);
  }
}

// erase_if<PredFunctor>: selected slots become tombstones (RECLAIM key,
// reclaim digest, score 0).  Runs under the table's exclusive lock.
template <class K, class S, template <typename, typename> class PredFunctor>
__global__ void erase_if_kernel(const hkv_table_view v, const K pattern, const S threshold,
                                const uint8_t reclaim_digest, unsigned long long* d_counter) {
  PredFunctor<K, S> pred;
  unsigned long long local = 0;
  for (uint64_t slot = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; slot < v.capacity;
       slot += uint64_t(gridDim.x) * blockDim.x) {
    K key = static_cast<K>(v.keys[HKV_SLOT_WORD(v, slot)]);
    S score = static_cast<S>(v.scores[HKV_SLOT_WORD(v, slot)]);
    if (!view_is_reserved(v, static_cast<uint64_t>(key)) && pred(key, score, pattern, threshold)) {
      v.keys[HKV_SLOT_WORD(v, slot)] = v.reclaim_key;
      v.digests[slot] = reclaim_digest;
      v.scores[HKV_SLOT_WORD(v, slot)] = 0;
      atomicSub(v.bucket_sizes + slot / v.max_bucket_size, 1);
      ++local;
    }
  }
  for (int o = 16; o > 0; o >>= 1) local += __shfl_down_sync(0xFFFFFFFFu, local, o);
  if ((threadIdx.x & 31u) == 0 && local) atomicAdd(d_counter, local);
}

// ---- functors that see the value row and a cooperative tile ------------------
//
// export_batch_if_v2 / erase_if_v2 / for_each hand each slot's key, row and
// score to a functor together with a tile of GroupSize threads that hold
// GroupSize consecutive slots; the functor may exchange data inside the tile
// (merlin_hashtable.cuh:3306-3407, 3007-3053).  The tile width follows the
// reference: the widest of 32 / 16 / 8 that does not exceed dim and divides the
// number of slots scanned, else 1, so whole tiles enter and leave the loop
// together.
template <class Launch>
inline void dispatch_tile(uint64_t dim, uint64_t n, Launch&& launch) {
  if (dim >= 32 && n % 32 == 0) {
    launch(std::integral_constant<uint32_t, 32>{});
  } else if (dim >= 16 && n % 16 == 0) {
    launch(std::integral_constant<uint32_t, 16>{});
  } else if (dim >= 8 && n % 8 == 0) {
    launch(std::integral_constant<uint32_t, 8>{});
  } else {
    launch(std::integral_constant<uint32_t, 1>{});
  }
}

inline unsigned tile_scan_blocks(uint64_t n) {
  return static_cast<unsigned>(std::min<uint64_t>((n + 127) / 128, 148 * 16));
}

template <class K, class V, class S, class PredFunctor, uint32_t G>
__global__ void export_if_v2_kernel(const hkv_table_view v, PredFunctor pred, const uint64_t n,
                                    const uint64_t offset, size_t* d_counter, K* out_keys,
                                    V* out_values, S* out_scores) {
  cg::thread_block_tile<G> g = cg::tiled_partition<G>(cg::this_thread_block());
  const uint64_t dim = v.row_bytes / sizeof(V);
  for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += uint64_t(gridDim.x) * blockDim.x) {
    const uint64_t slot = offset + i;
    const K key = static_cast<K>(v.keys[HKV_SLOT_WORD(v, slot)]);
    const S score = static_cast<S>(v.scores[HKV_SLOT_WORD(v, slot)]);
    const V* value = reinterpret_cast<const V*>(view_row(v, slot));
    bool match = pred.template operator()<G>(key, value, score, g);
    match = match && !view_is_reserved(v, static_cast<uint64_t>(key));
    const uint32_t votes = g.ballot(match);
    if (votes == 0) continue;
    unsigned long long at = 0;
    if (g.thread_rank() == 0) {
      at = atomicAdd(reinterpret_cast<unsigned long long*>(d_counter),
                     static_cast<unsigned long long>(__popc(votes)));
    }
    at = g.shfl(at, 0);
    if (match) {
      const uint32_t mine = __popc(votes & ((1u << g.thread_rank()) - 1u));
      out_keys[at + mine] = key;
      if (out_scores != nullptr) out_scores[at + mine] = score;
    }
    uint32_t left = votes;
    while (left) {
      const uint32_t src = __ffs(left) - 1;
      left &= left - 1;
      const V* row = g.shfl(value, src);
      V* dst = out_values + at * dim;
      for (uint64_t j = g.thread_rank(); j < dim; j += G) dst[j] = row[j];
      ++at;
    }
  }
}

template <class K, class V, class S, class PredFunctor, uint32_t G>
__global__ void erase_if_v2_kernel(const hkv_table_view v, PredFunctor pred, const uint64_t n,
                                   const uint8_t reclaim_digest,
                                   unsigned long long* d_counter) {
  cg::thread_block_tile<G> g = cg::tiled_partition<G>(cg::this_thread_block());
  for (uint64_t slot = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; slot < n;
       slot += uint64_t(gridDim.x) * blockDim.x) {
    const K key = static_cast<K>(v.keys[HKV_SLOT_WORD(v, slot)]);
    const S score = static_cast<S>(v.scores[HKV_SLOT_WORD(v, slot)]);
    const V* value = reinterpret_cast<const V*>(view_row(v, slot));
    bool match = pred.template operator()<G>(key, value, score, g);
    match = match && !view_is_reserved(v, static_cast<uint64_t>(key));
    const uint32_t votes = g.ballot(match);
    if (g.thread_rank() == 0 && votes) {
      atomicAdd(d_counter, static_cast<unsigned long long>(__popc(votes)));
      // G divides the bucket size (a power of two >= 16): a tile never straddles two buckets
      atomicSub(v.bucket_sizes + slot / v.max_bucket_size, __popc(votes));
    }
    if (match) {
      v.keys[HKV_SLOT_WORD(v, slot)] = v.reclaim_key;
      v.digests[slot] = reclaim_digest;
      v.scores[HKV_SLOT_WORD(v, slot)] = 0;
    }
  }
}

template <class K, class V, class S, class ExecutionFunc, uint32_t G>
__global__ void for_each_kernel(const hkv_table_view v, ExecutionFunc f, const uint64_t n,
                                const uint64_t first) {
  cg::thread_block_tile<G> g = cg::tiled_partition<G>(cg::this_thread_block());
  for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += uint64_t(gridDim.x) * blockDim.x) {
    const uint64_t slot = first + i;
    const K key = static_cast<K>(v.keys[HKV_SLOT_WORD(v, slot)]);
    S* score = reinterpret_cast<S*>(v.scores + HKV_SLOT_WORD(v, slot));
    V* value = reinterpret_cast<V*>(const_cast<uint8_t*>(view_row(v, slot)));
    f.template operator()<G>(key, value, score, g);
  }
}

}  // namespace detail

// The pure-virtual interface, merlin_hashtable.cuh:187-885.
template <typename K, typename V, typename S = uint64_t>
class HashTableBase {
 public:
  using size_type = size_t;
  using key_type = K;
  using value_type = V;
  using score_type = S;
  using allocator_type = BaseAllocator;

  virtual ~HashTableBase() {}
  virtual void init(const HashTableOptions& options, allocator_type* allocator = nullptr) = 0;
  virtual void insert_or_assign(const size_type n, const key_type* keys, const value_type* values,
                                const score_type* scores = nullptr, cudaStream_t stream = 0,
                                bool unique_key = true, bool ignore_evict_strategy = false) = 0;
  virtual void insert_and_evict(const size_type n, const key_type* keys, const value_type* values,
                                const score_type* scores, key_type* evicted_keys,
                                value_type* evicted_values, score_type* evicted_scores,
                                size_type* d_evicted_counter, cudaStream_t stream = 0,
                                bool unique_key = true, bool ignore_evict_strategy = false) = 0;
  virtual size_type insert_and_evict(const size_type n, const key_type* keys,
                                     const value_type* values, const score_type* scores,
                                     key_type* evicted_keys, value_type* evicted_values,
                                     score_type* evicted_scores, cudaStream_t stream = 0,
                                     bool unique_key = true,
                                     bool ignore_evict_strategy = false) = 0;
  virtual void accum_or_assign(const size_type n, const key_type* keys,
                               const value_type* value_or_deltas, const bool* accum_or_assigns,
                               const score_type* scores = nullptr, cudaStream_t stream = 0,
                               bool ignore_evict_strategy = false) = 0;
  virtual void find_or_insert(const size_type n, const key_type* keys, value_type* values,
                              score_type* scores = nullptr, cudaStream_t stream = 0,
                              bool unique_key = true, bool ignore_evict_strategy = false) = 0;
  virtual void find_or_insert(const size_type n, const key_type* keys, value_type** values,
                              bool* founds, score_type* scores = nullptr, cudaStream_t stream = 0,
                              bool unique_key = true, bool ignore_evict_strategy = false,
                              key_type** locked_key_ptrs = nullptr) = 0;
  virtual void lock_keys(const size_type n, key_type const* keys, key_type** locked_key_ptrs,
                         bool* succeededs = nullptr, cudaStream_t stream = 0,
                         score_type const* scores = nullptr) = 0;
  virtual void unlock_keys(const size_type n, key_type** locked_key_ptrs, const key_type* keys,
                           bool* succeededs = nullptr, cudaStream_t stream = 0) = 0;
  virtual void assign(const size_type n, const key_type* keys, const value_type* values,
                      const score_type* scores = nullptr, cudaStream_t stream = 0,
                      bool unique_key = true) = 0;
  virtual void assign_scores(const size_type n, const key_type* keys,
                             const score_type* scores = nullptr, cudaStream_t stream = 0,
                             bool unique_key = true) = 0;
  virtual void assign(const size_type n, const key_type* keys, const score_type* scores = nullptr,
                      cudaStream_t stream = 0, bool unique_key = true) = 0;
  virtual void assign_values(const size_type n, const key_type* keys, const value_type* values,
                             cudaStream_t stream = 0, bool unique_key = true) = 0;
  virtual void find(const size_type n, const key_type* keys, value_type* values, bool* founds,
                    score_type* scores = nullptr, cudaStream_t stream = 0) const = 0;
  virtual void find(const size_type n, const key_type* keys, value_type* values,
                    key_type* missed_keys, int* missed_indices, int* missed_size,
                    score_type* scores = nullptr, cudaStream_t stream = 0) const = 0;
  virtual void find(const size_type n, const key_type* keys, value_type** values, bool* founds,
                    score_type* scores = nullptr, cudaStream_t stream = 0,
                    bool unique_key = true) const = 0;
  virtual void find_and_update(const size_type n, const key_type* keys, value_type** values,
                               bool* founds, score_type* scores = nullptr, cudaStream_t stream = 0,
                               bool unique_key = true) = 0;
  virtual void contains(const size_type n, const key_type* keys, bool* founds,
                        cudaStream_t stream = 0) const = 0;
  virtual void erase(const size_type n, const key_type* keys, cudaStream_t stream = 0) = 0;
  virtual void clear(cudaStream_t stream = 0) = 0;
  virtual void export_batch(size_type n, const size_type offset, size_type* d_counter,
                            key_type* keys, value_type* values, score_type* scores = nullptr,
                            cudaStream_t stream = 0) const = 0;
  virtual size_type export_batch(const size_type n, const size_type offset, key_type* keys,
                                 value_type* values, score_type* scores = nullptr,
                                 cudaStream_t stream = 0) const = 0;
  virtual bool empty(cudaStream_t stream = 0) const = 0;
  virtual size_type size(cudaStream_t stream = 0) const = 0;
  virtual size_type capacity() const = 0;
  virtual void reserve(const size_type new_capacity, cudaStream_t stream = 0) = 0;
  virtual float load_factor(cudaStream_t stream = 0) const = 0;
  virtual void set_max_capacity(size_type new_max_capacity) = 0;
  virtual size_type dim() const noexcept = 0;
  virtual size_type max_bucket_size() const noexcept = 0;
  virtual size_type bucket_count() const noexcept = 0;
  virtual size_type save(BaseKVFile<K, V, S>* file,
                         const size_t max_workspace_size = 1L * 1024 * 1024,
                         cudaStream_t stream = 0) const = 0;
  virtual size_type load(BaseKVFile<K, V, S>* file,
                         const size_t max_workspace_size = 1L * 1024 * 1024,
                         cudaStream_t stream = 0) = 0;
  virtual void set_global_epoch(const uint64_t epoch) = 0;
};

// merlin_hashtable.cuh:910-3892 of the reference.  ArchTag is accepted for
// source compatibility and ignored: the library is built for sm_100a only.
template <typename K, typename V, typename S = uint64_t, int Strategy = EvictStrategy::kLru,
          typename ArchTag = Sm80>
class HashTable : public HashTableBase<K, V, S> {
  static_assert(sizeof(K) == 8 && std::is_integral<K>::value,
                "The key_type must be int64_t or uint64_t.");
  static_assert(std::is_same<S, uint64_t>::value || std::is_same<S, uint32_t>::value,
                "The score_type must be uint64_t or uint32_t.");
  // merlin_hashtable.cuh:944-948: the epoch strategies pack epoch | score into 64 bits
  static_assert(!(std::is_same<S, uint32_t>::value && Strategy != EvictStrategy::kCustomized),
                "score_type uint32_t is only compatible with Customized; use uint64_t.");

 public:
  using size_type = size_t;
  using key_type = K;
  using value_type = V;
  using score_type = S;
  static constexpr int evict_strategy = Strategy;
  using allocator_type = BaseAllocator;

  HashTable() = default;
  HashTable(const HashTable&) = delete;
  HashTable& operator=(const HashTable&) = delete;
  HashTable(HashTable&&) = delete;
  HashTable& operator=(HashTable&&) = delete;

  ~HashTable() override {
    if (table_ != nullptr) hkv_table_destroy(table_);
  }

  void init(const HashTableOptions& options, allocator_type* allocator = nullptr) override {
    if (table_ != nullptr) return;
    options_ = options;
    hkv_options o{};
    o.init_capacity = options.init_capacity;
    o.max_capacity = options.max_capacity;
    o.max_hbm_for_vectors = options.max_hbm_for_vectors;
    o.max_bucket_size = options.max_bucket_size;
    o.dim = options.dim;
    o.max_load_factor = options.max_load_factor;
    o.block_size = options.block_size;
    o.io_block_size = options.io_block_size;
    o.device_id = options.device_id;
    o.io_by_cpu = options.io_by_cpu ? 1 : 0;
    o.use_constant_memory = options.use_constant_memory ? 1 : 0;
    o.reserved_key_start_bit = options.reserved_key_start_bit;
    o.num_of_buckets_per_alloc = options.num_of_buckets_per_alloc;
    o.api_lock = options.api_lock ? 1 : 0;
    o.table_mode = static_cast<int32_t>(options.table_mode);
    o.evict_strategy = Strategy;
    o.value_size = sizeof(V);
    o.value_kind = detail::value_kind_of<V>();
    o.slot_layout = static_cast<uint32_t>(options.slot_layout);
    o.score_size = sizeof(S);
    hkv_allocator bridge{allocator, detail::alloc_trampoline, detail::free_trampoline};
    detail::rethrow(hkv_table_create(&o, allocator ? &bridge : nullptr, &table_));
  }

  void insert_or_assign(const size_type n, const key_type* keys, const value_type* values,
                        const score_type* scores = nullptr, cudaStream_t stream = 0,
                        bool unique_key = true, bool ignore_evict_strategy = false) override {
    detail::rethrow(hkv_insert_or_assign(table_, n, u(keys), values, w(scores), stream, unique_key,
                                         ignore_evict_strategy));
  }

  void insert_and_evict(const size_type n, const key_type* keys, const value_type* values,
                        const score_type* scores, key_type* evicted_keys,
                        value_type* evicted_values, score_type* evicted_scores,
                        size_type* d_evicted_counter, cudaStream_t stream = 0,
                        bool unique_key = true, bool ignore_evict_strategy = false) override {
    detail::rethrow(hkv_insert_and_evict(table_, n, u(keys), values, w(scores), u(evicted_keys),
                                         evicted_values, w(evicted_scores),
                                         reinterpret_cast<uint64_t*>(d_evicted_counter), stream,
                                         unique_key, ignore_evict_strategy));
  }

  size_type insert_and_evict(const size_type n, const key_type* keys, const value_type* values,
                             const score_type* scores, key_type* evicted_keys,
                             value_type* evicted_values, score_type* evicted_scores,
                             cudaStream_t stream = 0, bool unique_key = true,
                             bool ignore_evict_strategy = false) override {
    uint64_t count = 0;
    detail::rethrow(hkv_insert_and_evict_count(table_, n, u(keys), values, w(scores), u(evicted_keys),
                                               evicted_values, w(evicted_scores), stream, unique_key,
                                               ignore_evict_strategy, &count));
    return count;
  }

  void accum_or_assign(const size_type n, const key_type* keys, const value_type* value_or_deltas,
                       const bool* accum_or_assigns, const score_type* scores = nullptr,
                       cudaStream_t stream = 0, bool ignore_evict_strategy = false) override {
    detail::rethrow(hkv_accum_or_assign(table_, n, u(keys), value_or_deltas, accum_or_assigns,
                                        w(scores), stream, ignore_evict_strategy));
  }

  void find_or_insert(const size_type n, const key_type* keys, value_type* values,
                      score_type* scores = nullptr, cudaStream_t stream = 0,
                      bool unique_key = true, bool ignore_evict_strategy = false) override {
    detail::rethrow(hkv_find_or_insert(table_, n, u(keys), values, w(scores), stream, unique_key,
                                       ignore_evict_strategy));
  }

  void find_or_insert(const size_type n, const key_type* keys, value_type** values, bool* founds,
                      score_type* scores = nullptr, cudaStream_t stream = 0,
                      bool unique_key = true, bool ignore_evict_strategy = false,
                      key_type** locked_key_ptrs = nullptr) override {
    detail::rethrow(hkv_find_or_insert_ptr(table_, n, u(keys), reinterpret_cast<void**>(values),
                                           founds, w(scores), stream, unique_key,
                                           ignore_evict_strategy,
                                           reinterpret_cast<uint64_t**>(locked_key_ptrs)));
  }

  void lock_keys(const size_type n, key_type const* keys, key_type** locked_key_ptrs,
                 bool* succeededs = nullptr, cudaStream_t stream = 0,
                 score_type const* scores = nullptr) override {
    detail::rethrow(hkv_lock_keys(table_, n, u(keys),
                                  reinterpret_cast<uint64_t**>(locked_key_ptrs), succeededs,
                                  stream, w(scores)));
  }

  void unlock_keys(const size_type n, key_type** locked_key_ptrs, const key_type* keys,
                   bool* succeededs = nullptr, cudaStream_t stream = 0) override {
    detail::rethrow(hkv_unlock_keys(table_, n, reinterpret_cast<uint64_t**>(locked_key_ptrs),
                                    u(keys), succeededs, stream));
  }

  void assign(const size_type n, const key_type* keys, const value_type* values,
              const score_type* scores = nullptr, cudaStream_t stream = 0,
              bool unique_key = true) override {
    detail::rethrow(hkv_assign(table_, n, u(keys), values, w(scores), stream, unique_key));
  }

  void assign_scores(const size_type n, const key_type* keys, const score_type* scores = nullptr,
                     cudaStream_t stream = 0, bool unique_key = true) override {
    detail::rethrow(hkv_assign_scores(table_, n, u(keys), w(scores), stream, unique_key));
  }

  // alias of assign_scores, merlin_hashtable.cuh:2278-2283
  void assign(const size_type n, const key_type* keys, const score_type* scores = nullptr,
              cudaStream_t stream = 0, bool unique_key = true) override {
    assign_scores(n, keys, scores, stream, unique_key);
  }

  void assign_values(const size_type n, const key_type* keys, const value_type* values,
                     cudaStream_t stream = 0, bool unique_key = true) override {
    detail::rethrow(hkv_assign_values(table_, n, u(keys), values, stream, unique_key));
  }

  void find(const size_type n, const key_type* keys, value_type* values, bool* founds,
            score_type* scores = nullptr, cudaStream_t stream = 0) const override {
    detail::rethrow(hkv_find(table_, n, u(keys), values, founds, w(scores), stream));
  }

  /**
   * @brief find for a batch that lives in host memory (not in the reference,
   * whose batch buffers must be GPU-accessible): the batch is staged through
   * the device in chunks whose copies and lookups overlap.  `keys`, `values`,
   * `founds` (and `scores`, 64-bit scores only) are host pointers, pinned for
   * asynchronous copies; they are complete once `stream` has passed the call.
   * Rows of keys that are not in the table are zero-filled.
   */
  void find_host(const size_type n, const key_type* keys, value_type* values, bool* founds,
                 score_type* scores = nullptr, cudaStream_t stream = 0) const {
    detail::rethrow(hkv_find_host(table_, n, u(keys), values, founds, w(scores), stream));
  }

  void find(const size_type n, const key_type* keys, value_type* values, key_type* missed_keys,
            int* missed_indices, int* missed_size, score_type* scores = nullptr,
            cudaStream_t stream = 0) const override {
    detail::rethrow(hkv_find_missed(table_, n, u(keys), values, u(missed_keys), missed_indices,
                                    missed_size, w(scores), stream));
  }

  void find(const size_type n, const key_type* keys, value_type** values, bool* founds,
            score_type* scores = nullptr, cudaStream_t stream = 0,
            bool unique_key = true) const override {
    detail::rethrow(hkv_find_ptr(table_, n, u(keys), reinterpret_cast<void**>(values), founds,
                                 w(scores), stream, unique_key));
  }

  void find_and_update(const size_type n, const key_type* keys, value_type** values, bool* founds,
                       score_type* scores = nullptr, cudaStream_t stream = 0,
                       bool unique_key = true) override {
    detail::rethrow(hkv_find_and_update(table_, n, u(keys), reinterpret_cast<void**>(values),
                                        founds, w(scores), stream, unique_key));
  }

  void contains(const size_type n, const key_type* keys, bool* founds,
                cudaStream_t stream = 0) const override {
    detail::rethrow(hkv_contains(table_, n, u(keys), founds, stream));
  }

  void erase(const size_type n, const key_type* keys, cudaStream_t stream = 0) override {
    detail::rethrow(hkv_erase(table_, n, u(keys), stream));
  }

  void clear(cudaStream_t stream = 0) override { detail::rethrow(hkv_clear(table_, stream)); }

  void export_batch(size_type n, const size_type offset, size_type* d_counter, key_type* keys,
                    value_type* values, score_type* scores = nullptr,
                    cudaStream_t stream = 0) const override {
    detail::rethrow(hkv_export_batch(table_, n, offset, reinterpret_cast<uint64_t*>(d_counter),
                                     u(keys), values, w(scores), stream));
  }

  size_type export_batch(const size_type n, const size_type offset, key_type* keys,
                         value_type* values, score_type* scores = nullptr,
                         cudaStream_t stream = 0) const override {
    uint64_t count = 0;
    detail::rethrow(
        hkv_export_batch_count(table_, n, offset, u(keys), values, w(scores), stream, &count));
    return count;
  }

  // export_batch_if<PredFunctor>, merlin_hashtable.cuh:3193-3276.  The functor
  // is the reference's: PredFunctor<K,S>()(key, score, pattern, threshold).
  template <template <typename, typename> class PredFunctor>
  void export_batch_if(const key_type& pattern, const score_type& threshold, size_type n,
                       const size_type offset, size_type* d_counter, key_type* keys,
                       value_type* values, score_type* scores = nullptr,
                       cudaStream_t stream = 0) const {
    detail::rethrow(hkv_external_begin(table_, 0, stream));
    hkv_table_view v{};
    hkv_get_view(table_, &v);  // after the lock: a doubling replaces the planes
    cudaError_t err = cudaMemsetAsync(d_counter, 0, sizeof(size_type), stream);
    if (err == cudaSuccess && offset < v.capacity) {
      n = std::min<size_type>(v.capacity - offset, n);
      if (n > 0) {
        const unsigned blocks = static_cast<unsigned>(std::min<size_type>((n + 255) / 256, 148 * 8));
        detail::export_if_kernel<K, V, S, PredFunctor><<<blocks, 256, 0, stream>>>(
            v, pattern, threshold, n, offset, d_counter, keys, values, scores);
        err = cudaGetLastError();
      }
    }
    detail::rethrow(hkv_external_end(table_, 0, stream));
    CUDA_CHECK(err);
  }

  // size_if<PredFunctor>, merlin_hashtable.cuh:3459-3476
  template <template <typename, typename> class PredFunctor>
  void size_if(const key_type& pattern, const score_type& threshold, size_type* d_counter,
               cudaStream_t stream = 0) const {
    detail::rethrow(hkv_external_begin(table_, 0, stream));
    hkv_table_view v{};
    hkv_get_view(table_, &v);  // after the lock: a doubling replaces the planes
    cudaError_t err = cudaMemsetAsync(d_counter, 0, sizeof(size_type), stream);
    if (err == cudaSuccess) {
      detail::size_if_kernel<K, S, PredFunctor>
          <<<148 * 8, 256, 0, stream>>>(v, pattern, threshold, d_counter);
      err = cudaGetLastError();
    }
    detail::rethrow(hkv_external_end(table_, 0, stream));
    CUDA_CHECK(err);
  }

  // erase_if<PredFunctor>, merlin_hashtable.cuh:2964-2996: returns the number
  // of erased keys (synchronises the stream).
  template <template <typename, typename> class PredFunctor>
  size_type erase_if(const key_type& pattern, const score_type& threshold,
                     cudaStream_t stream = 0) {
    unsigned long long* d_count = nullptr;
    CUDA_CHECK(cudaMallocAsync(reinterpret_cast<void**>(&d_count), sizeof(*d_count), stream));
    detail::rethrow(hkv_external_begin(table_, 2, stream));
    hkv_table_view v{};
    hkv_get_view(table_, &v);  // after the lock: a doubling replaces the planes
    cudaError_t err = cudaMemsetAsync(d_count, 0, sizeof(*d_count), stream);
    if (err == cudaSuccess) {
      const uint8_t reclaim_digest =
          static_cast<uint8_t>(Murmur3HashHost(v.reclaim_key) >> 32);
      detail::erase_if_kernel<K, S, PredFunctor>
          <<<148 * 8, 256, 0, stream>>>(v, pattern, threshold, reclaim_digest, d_count);
      err = cudaGetLastError();
    }
    detail::rethrow(hkv_external_end(table_, 2, stream));
    unsigned long long count = 0;
    if (err == cudaSuccess) {
      err = cudaMemcpyAsync(&count, d_count, sizeof(count), cudaMemcpyDeviceToHost, stream);
    }
    if (err == cudaSuccess) err = cudaStreamSynchronize(stream);
    cudaFreeAsync(d_count, stream);
    CUDA_CHECK(err);
    return count;
  }

  // export_batch_if_v2<PredFunctor>, merlin_hashtable.cuh:3306-3347.  The
  // functor is the reference's: pred.operator()<GroupSize>(key, value, score,
  // tile).  Reserved keys (empty slots, tombstones) are never exported.
  template <typename PredFunctor>
  void export_batch_if_v2(PredFunctor& pred, size_type n, const size_type offset,
                          size_type* d_counter, key_type* keys, value_type* values,
                          score_type* scores = nullptr, cudaStream_t stream = 0) const {
    detail::rethrow(hkv_external_begin(table_, 0, stream));
    hkv_table_view v{};
    int rc = hkv_get_view(table_, &v);
    cudaError_t err = cudaMemsetAsync(d_counter, 0, sizeof(size_type), stream);
    if (rc == HKV_OK && err == cudaSuccess && offset < v.capacity) {
      n = std::min<size_type>(v.capacity - offset, n);
      if (n > 0) {
        detail::dispatch_tile(options_.dim, n, [&](auto tile) {
          detail::export_if_v2_kernel<K, V, S, PredFunctor, decltype(tile)::value>
              <<<detail::tile_scan_blocks(n), 128, 0, stream>>>(v, pred, n, offset, d_counter,
                                                               keys, values, scores);
        });
        err = cudaGetLastError();
      }
    }
    detail::rethrow(hkv_external_end(table_, 0, stream));
    detail::rethrow(rc);
    CUDA_CHECK(err);
  }

  // erase_if_v2<PredFunctor>, merlin_hashtable.cuh:3007-3053: returns the
  // number of erased keys (synchronises the stream).
  template <typename PredFunctor>
  size_type erase_if_v2(PredFunctor& pred, cudaStream_t stream = 0) {
    unsigned long long* d_count = nullptr;
    CUDA_CHECK(cudaMallocAsync(reinterpret_cast<void**>(&d_count), sizeof(*d_count), stream));
    detail::rethrow(hkv_external_begin(table_, 2, stream));
    hkv_table_view v{};
    int rc = hkv_get_view(table_, &v);
    cudaError_t err = cudaMemsetAsync(d_count, 0, sizeof(*d_count), stream);
    if (rc == HKV_OK && err == cudaSuccess) {
      const uint8_t reclaim_digest = static_cast<uint8_t>(Murmur3HashHost(v.reclaim_key) >> 32);
      const uint64_t n = v.capacity;
      // a tile must not straddle two buckets: its size is capped by the bucket size
      detail::dispatch_tile(std::min<uint64_t>(options_.dim, v.max_bucket_size), n, [&](auto tile) {
        detail::erase_if_v2_kernel<K, V, S, PredFunctor, decltype(tile)::value>
            <<<detail::tile_scan_blocks(n), 128, 0, stream>>>(v, pred, n, reclaim_digest, d_count);
      });
      err = cudaGetLastError();
    }
    detail::rethrow(hkv_external_end(table_, 2, stream));
    unsigned long long count = 0;
    if (err == cudaSuccess) {
      err = cudaMemcpyAsync(&count, d_count, sizeof(count), cudaMemcpyDeviceToHost, stream);
    }
    if (err == cudaSuccess) err = cudaStreamSynchronize(stream);
    cudaFreeAsync(d_count, stream);
    detail::rethrow(rc);
    CUDA_CHECK(err);
    return count;
  }

  // for_each<ExecutionFunc>, merlin_hashtable.cuh:3371-3407: applies
  // f.operator()<GroupSize>(key, value*, score*, tile) to every slot of
  // [first, last), occupied or not, under the exclusive lock.
  template <typename ExecutionFunc>
  void for_each(const size_type first, const size_type last, ExecutionFunc& f,
                cudaStream_t stream = 0) {
    detail::rethrow(hkv_external_begin(table_, 2, stream));
    hkv_table_view v{};
    int rc = hkv_get_view(table_, &v);
    cudaError_t err = cudaSuccess;
    if (rc == HKV_OK && first < v.capacity && last <= v.capacity && first < last) {
      const uint64_t n = last - first;
      detail::dispatch_tile(options_.dim, n, [&](auto tile) {
        detail::for_each_kernel<K, V, S, ExecutionFunc, decltype(tile)::value>
            <<<detail::tile_scan_blocks(n), 128, 0, stream>>>(v, f, n, first);
      });
      err = cudaGetLastError();
    }
    detail::rethrow(hkv_external_end(table_, 2, stream));
    detail::rethrow(rc);
    CUDA_CHECK(err);
  }

  bool empty(cudaStream_t stream = 0) const override { return size(stream) == 0; }

  size_type size(cudaStream_t stream = 0) const override {
    uint64_t s = 0;
    detail::rethrow(hkv_size(table_, stream, &s));
    return s;
  }

  size_type capacity() const override { return hkv_capacity(table_); }

  void reserve(const size_type new_capacity, cudaStream_t stream = 0) override {
    detail::rethrow(hkv_reserve(table_, new_capacity, stream));
  }

  // Not in the reference: on a hybrid table, moves the rows of the buckets
  // that lookups hit most into HBM (hkv_promote_hot_buckets).  Returns the
  // number of buckets moved in.
  size_type promote_hot_buckets(cudaStream_t stream = 0) {
    uint64_t promoted = 0;
    detail::rethrow(hkv_promote_hot_buckets(table_, stream, &promoted));
    return promoted;
  }

  float load_factor(cudaStream_t stream = 0) const override {
    float lf = 0.f;
    detail::rethrow(hkv_load_factor(table_, stream, &lf));
    return lf;
  }

  void set_max_capacity(size_type new_max_capacity) override {
    // merlin_hashtable.cuh:3561-3579
    detail::rethrow(hkv_set_max_capacity(table_, new_max_capacity));
    if (new_max_capacity >= capacity()) options_.max_capacity = new_max_capacity;
  }

  size_type dim() const noexcept override { return options_.dim; }
  size_type max_bucket_size() const noexcept override { return options_.max_bucket_size; }
  size_type bucket_count() const noexcept override { return hkv_bucket_count(table_); }

  // save, merlin_hashtable.cuh:3615-3689: the table is walked in chunks that
  // fit max_workspace_size; each chunk is exported, copied to the host and
  // handed to file->write.
  size_type save(BaseKVFile<K, V, S>* file, const size_t max_workspace_size = 1L * 1024 * 1024,
                 cudaStream_t stream = 0) const override {
    const size_type tuple_size = sizeof(K) + sizeof(S) + sizeof(V) * dim();
    MERLIN_CHECK(max_workspace_size >= tuple_size,
                 "[HierarchicalKV] max_workspace_size is smaller than a single "
                 "`key + scoredata + value` tuple! Please set a larger value!");
    const size_type total = capacity();
    const size_type n = std::min(max_workspace_size / tuple_size, total);
    Workspace ws(n, dim());
    size_type written = 0;
    for (size_type at = 0; at < total; at += n) {
      const size_type count =
          export_batch(std::min(total - at, n), at, ws.d_keys, ws.d_values, ws.d_scores, stream);
      if (count == 0) continue;
      CUDA_CHECK(cudaMemcpyAsync(ws.h_keys.data(), ws.d_keys, sizeof(K) * count,
                                 cudaMemcpyDeviceToHost, stream));
      CUDA_CHECK(cudaMemcpyAsync(ws.h_scores.data(), ws.d_scores, sizeof(S) * count,
                                 cudaMemcpyDeviceToHost, stream));
      CUDA_CHECK(cudaMemcpyAsync(ws.h_values.data(), ws.d_values, sizeof(V) * dim() * count,
                                 cudaMemcpyDeviceToHost, stream));
      CUDA_CHECK(cudaStreamSynchronize(stream));
      file->write(count, dim(), ws.h_keys.data(), ws.h_values.data(), ws.h_scores.data());
      written += count;
    }
    return written;
  }

  // load, merlin_hashtable.cuh:3702-3758: chunks are read from the file and
  // inserted with their stored scores, whatever the table's strategy.
  size_type load(BaseKVFile<K, V, S>* file, const size_t max_workspace_size = 1L * 1024 * 1024,
                 cudaStream_t stream = 0) override {
    const size_type tuple_size = sizeof(K) + sizeof(S) + sizeof(V) * dim();
    MERLIN_CHECK(max_workspace_size >= tuple_size,
                 "[HierarchicalKV] max_workspace_size is smaller than a single "
                 "`key + score + value` tuple! Please set a larger value!");
    const size_type n = max_workspace_size / tuple_size;
    Workspace ws(n, dim());
    size_type loaded = 0;
    while (true) {
      const size_type count =
          file->read(n, dim(), ws.h_keys.data(), ws.h_values.data(), ws.h_scores.data());
      if (count == 0) break;
      CUDA_CHECK(cudaMemcpyAsync(ws.d_keys, ws.h_keys.data(), sizeof(K) * count,
                                 cudaMemcpyHostToDevice, stream));
      CUDA_CHECK(cudaMemcpyAsync(ws.d_scores, ws.h_scores.data(), sizeof(S) * count,
                                 cudaMemcpyHostToDevice, stream));
      CUDA_CHECK(cudaMemcpyAsync(ws.d_values, ws.h_values.data(), sizeof(V) * dim() * count,
                                 cudaMemcpyHostToDevice, stream));
      insert_or_assign(count, ws.d_keys, ws.d_values, ws.d_scores, stream, true, true);
      CUDA_CHECK(cudaStreamSynchronize(stream));
      loaded += count;
      if (count < n) break;
    }
    return loaded;
  }

  void set_global_epoch(const uint64_t epoch) override {
    detail::rethrow(hkv_set_global_epoch(table_, epoch));
  }

  // Not part of the reference: the library handle, for callers that mix the
  // class with direct C-ABI calls.
  hkv_table* native_handle() const noexcept { return table_; }

 private:
  static const uint64_t* u(const K* p) { return reinterpret_cast<const uint64_t*>(p); }
  static uint64_t* u(K* p) { return reinterpret_cast<uint64_t*>(p); }
  // score arrays cross the ABI as they are: hkv_options.score_size tells the
  // library whether they hold 64-bit or 32-bit scores
  static const uint64_t* w(const S* p) { return reinterpret_cast<const uint64_t*>(p); }
  static uint64_t* w(S* p) { return reinterpret_cast<uint64_t*>(p); }

  struct Workspace {
    K* d_keys = nullptr;
    V* d_values = nullptr;
    S* d_scores = nullptr;
    std::vector<K> h_keys;
    std::vector<V> h_values;
    std::vector<S> h_scores;
    Workspace(size_t n, size_t dim) : h_keys(n), h_values(n * dim), h_scores(n) {
      CUDA_CHECK(cudaMalloc(&d_keys, sizeof(K) * n));
      CUDA_CHECK(cudaMalloc(&d_scores, sizeof(S) * n));
      CUDA_CHECK(cudaMalloc(&d_values, sizeof(V) * n * dim));
    }
    ~Workspace() {
      cudaFree(d_keys);
      cudaFree(d_scores);
      cudaFree(d_values);
    }
  };

  HashTableOptions options_;
  mutable hkv_table* table_ = nullptr;
};

}  // namespace merlin
}  // namespace nv
