// TEST INFRASTRUCTURE ONLY -- never linked into, loaded by or called from the
// product library.
//
// Thin C-ABI shim around the *unmodified* reference headers
// (include/merlin_hashtable.cuh of NVIDIA-Merlin/HierarchicalKV).  It is
// compiled from the reference sources where they lie (see oracle/Makefile),
// one shared object per eviction strategy (-DREF_STRATEGY=0..4), with hidden
// visibility so that the reference's nv::merlin symbols never meet the
// product's.  The parity tests and the reference arm of the benchmark drive
// both libraries with the same seeded batches.
//
// K = uint64_t, V = float, S = uint64_t, as in the reference benchmark
// (benchmark/merlin_hashtable_benchmark.cc.cu:492).
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <exception>
#include <memory>
#include <string>

#include "merlin_hashtable.cuh"
#include "merlin_localfile.hpp"

#ifndef REF_STRATEGY
#define REF_STRATEGY 0
#endif

#define REF_API extern "C" __attribute__((visibility("default")))

namespace {

using K = uint64_t;
using V = float;
using S = uint64_t;
using Table = nv::merlin::HashTable<K, V, S, REF_STRATEGY>;

thread_local std::string g_err;

template <class K_, class S_>
struct PredScoreLess {
  __forceinline__ __device__ bool operator()(const K_& key, S_& score,
                                             const K_& pattern,
                                             const S_& threshold) {
    return score < threshold;
  }
};

template <class K_, class S_>
struct PredScoreGreaterEq {
  __forceinline__ __device__ bool operator()(const K_& key, S_& score,
                                             const K_& pattern,
                                             const S_& threshold) {
    return score >= threshold;
  }
};

template <class K_, class S_>
struct PredKeyMask {
  __forceinline__ __device__ bool operator()(const K_& key, S_& score,
                                             const K_& pattern,
                                             const S_& threshold) {
    return (key & static_cast<K_>(threshold)) == pattern;
  }
};

// Device-side probes of the reference's own arithmetic, for golden vectors.
__global__ void probe_constants_kernel(uint64_t* out) {
  out[0] = nv::merlin::EMPTY_KEY;
  out[1] = nv::merlin::RECLAIM_KEY;
  out[2] = nv::merlin::LOCKED_KEY;
  out[3] = nv::merlin::empty_digest<uint64_t>();
  out[4] = nv::merlin::reclaim_digest<uint64_t>();
}

__global__ void probe_keys_kernel(uint64_t n, const uint64_t* keys, uint64_t* hashes,
                                  uint8_t* digests, bool* reserved) {
  const uint64_t i = blockIdx.x * uint64_t(blockDim.x) + threadIdx.x;
  if (i >= n) return;
  hashes[i] = nv::merlin::Murmur3HashDevice(keys[i]);
  digests[i] = nv::merlin::get_digest<uint64_t>(keys[i]);
  reserved[i] = nv::merlin::IS_RESERVED_KEY<uint64_t>(keys[i]);
}

template <class F>
int guarded(F&& f) {
  try {
    f();
    return 0;
  } catch (const std::exception& e) {
    g_err = e.what();
    return 1;
  } catch (...) {
    g_err = "unknown exception";
    return 1;
  }
}

}  // namespace

REF_API const char* ref_last_error() { return g_err.c_str(); }
REF_API int ref_strategy() { return REF_STRATEGY; }

REF_API int ref_create(uint64_t init_capacity, uint64_t max_capacity,
                       uint64_t max_hbm_for_vectors, uint64_t dim,
                       uint64_t max_bucket_size, int reserved_key_start_bit,
                       int api_lock, void** out) {
  return guarded([&] {
    nv::merlin::HashTableOptions o;
    o.init_capacity = init_capacity;
    o.max_capacity = max_capacity;
    o.max_hbm_for_vectors = max_hbm_for_vectors;
    o.dim = dim;
    o.max_bucket_size = max_bucket_size;
    o.reserved_key_start_bit = reserved_key_start_bit;
    o.api_lock = api_lock != 0;
    // One allocation for all buckets instead of one per bucket.  The reference
    // places whole allocations in HBM while max_hbm_for_vectors lasts
    // (include/merlin/core_kernels.cuh:204-232), so a table whose rows only
    // partly fit gets allocations small enough for the HBM share to be used.
    size_t buckets = 1;
    while (buckets * 2 * max_bucket_size <= init_capacity) buckets *= 2;
    const uint64_t row_bytes = dim * sizeof(V);
    while (buckets > 1 && max_hbm_for_vectors > 0 &&
           max_hbm_for_vectors < init_capacity * row_bytes &&
           buckets * max_bucket_size * row_bytes > max_hbm_for_vectors) {
      buckets /= 2;
    }
    o.num_of_buckets_per_alloc = buckets;
    auto* t = new Table();
    try {
      t->init(o);
    } catch (...) {
      delete t;
      throw;
    }
    *out = t;
  });
}

// A table that may grow: init_capacity * 2 <= max_capacity, and the insert-like
// calls double it while the estimated load is above max_load_factor.
REF_API int ref_create_growable(uint64_t init_capacity, uint64_t max_capacity,
                                uint64_t max_hbm_for_vectors, uint64_t dim,
                                float max_load_factor, void** out) {
  return guarded([&] {
    nv::merlin::HashTableOptions o;
    o.init_capacity = init_capacity;
    o.max_capacity = max_capacity;
    o.max_hbm_for_vectors = max_hbm_for_vectors;
    o.dim = dim;
    o.max_load_factor = max_load_factor;
    size_t buckets = 1;
    while (buckets * 2 * o.max_bucket_size <= init_capacity) buckets *= 2;
    o.num_of_buckets_per_alloc = buckets;
    auto* t = new Table();
    try {
      t->init(o);
    } catch (...) {
      delete t;
      throw;
    }
    *out = t;
  });
}

// TableMode::kMemory: dual-bucket table (insert_or_assign of unique keys and find).
REF_API int ref_create_memory_mode(uint64_t capacity, uint64_t dim, void** out) {
  return guarded([&] {
    nv::merlin::HashTableOptions o;
    o.init_capacity = capacity;
    o.max_capacity = capacity;
    o.max_hbm_for_vectors = 0;
    o.dim = dim;
    o.table_mode = nv::merlin::TableMode::kMemory;
    size_t buckets = 1;
    while (buckets * 2 * o.max_bucket_size <= capacity) buckets *= 2;
    o.num_of_buckets_per_alloc = buckets;
    auto* t = new Table();
    try {
      t->init(o);
    } catch (...) {
      delete t;
      throw;
    }
    *out = t;
  });
}

REF_API int ref_reserve(void* t, uint64_t new_capacity, cudaStream_t stream) {
  return guarded([&] { static_cast<Table*>(t)->reserve(new_capacity, stream); });
}

// 0 ok, 1 the reference threw std::invalid_argument, -1 anything else
REF_API int ref_set_max_capacity(void* t, uint64_t new_max_capacity) {
  try {
    static_cast<Table*>(t)->set_max_capacity(new_max_capacity);
    return 0;
  } catch (const std::invalid_argument& e) {
    g_err = e.what();
    return 1;
  } catch (const std::exception& e) {
    g_err = e.what();
    return -1;
  }
}

// save / load through the reference's own LocalKVFile
// (include/merlin_localfile.hpp:44-158): <prefix>.keys / .values / .scores.
REF_API int ref_save(void* t, const char* prefix, uint64_t max_workspace_size,
                     cudaStream_t stream, uint64_t* saved) {
  return guarded([&] {
    nv::merlin::LocalKVFile<K, V, S> file;
    const std::string p(prefix);
    if (!file.open(p + ".keys", p + ".values", p + ".scores", "wb")) {
      throw std::runtime_error("cannot open " + p + ".* for writing");
    }
    *saved = static_cast<Table*>(t)->save(&file, max_workspace_size, stream);
    file.close();
  });
}

REF_API int ref_load(void* t, const char* prefix, uint64_t max_workspace_size,
                     cudaStream_t stream, uint64_t* loaded) {
  return guarded([&] {
    nv::merlin::LocalKVFile<K, V, S> file;
    const std::string p(prefix);
    if (!file.open(p + ".keys", p + ".values", p + ".scores", "rb")) {
      throw std::runtime_error("cannot open " + p + ".* for reading");
    }
    *loaded = static_cast<Table*>(t)->load(&file, max_workspace_size, stream);
    file.close();
  });
}

REF_API int ref_destroy(void* t) {
  return guarded([&] { delete static_cast<Table*>(t); });
}

REF_API int ref_set_global_epoch(void* t, uint64_t epoch) {
  return guarded([&] { static_cast<Table*>(t)->set_global_epoch(epoch); });
}

REF_API int ref_insert_or_assign(void* t, uint64_t n, const K* keys,
                                 const V* values, const S* scores,
                                 cudaStream_t stream, int unique_key) {
  return guarded([&] {
    static_cast<Table*>(t)->insert_or_assign(n, keys, values, scores, stream,
                                             unique_key != 0);
  });
}

REF_API int ref_insert_and_evict(void* t, uint64_t n, const K* keys,
                                 const V* values, const S* scores,
                                 K* evicted_keys, V* evicted_values,
                                 S* evicted_scores, uint64_t* d_evicted_counter,
                                 cudaStream_t stream, int unique_key) {
  return guarded([&] {
    static_cast<Table*>(t)->insert_and_evict(
        n, keys, values, scores, evicted_keys, evicted_values, evicted_scores,
        reinterpret_cast<size_t*>(d_evicted_counter), stream, unique_key != 0);
  });
}

REF_API int ref_accum_or_assign(void* t, uint64_t n, const K* keys,
                                const V* value_or_deltas,
                                const bool* accum_or_assigns, const S* scores,
                                cudaStream_t stream) {
  return guarded([&] {
    static_cast<Table*>(t)->accum_or_assign(n, keys, value_or_deltas,
                                            accum_or_assigns, scores, stream);
  });
}

REF_API int ref_find_or_insert(void* t, uint64_t n, const K* keys, V* values,
                               S* scores, cudaStream_t stream, int unique_key) {
  return guarded([&] {
    static_cast<Table*>(t)->find_or_insert(n, keys, values, scores, stream,
                                           unique_key != 0);
  });
}

REF_API int ref_find_or_insert_ptr(void* t, uint64_t n, const K* keys,
                                   V** values, bool* founds, S* scores,
                                   cudaStream_t stream, int unique_key) {
  return guarded([&] {
    static_cast<Table*>(t)->find_or_insert(n, keys, values, founds, scores,
                                           stream, unique_key != 0);
  });
}

REF_API int ref_assign(void* t, uint64_t n, const K* keys, const V* values,
                       const S* scores, cudaStream_t stream, int unique_key) {
  return guarded([&] {
    static_cast<Table*>(t)->assign(n, keys, values, scores, stream,
                                   unique_key != 0);
  });
}

REF_API int ref_assign_scores(void* t, uint64_t n, const K* keys,
                              const S* scores, cudaStream_t stream,
                              int unique_key) {
  return guarded([&] {
    static_cast<Table*>(t)->assign_scores(n, keys, scores, stream,
                                          unique_key != 0);
  });
}

REF_API int ref_find(void* t, uint64_t n, const K* keys, V* values,
                     bool* founds, S* scores, cudaStream_t stream) {
  return guarded([&] {
    static_cast<const Table*>(t)->find(n, keys, values, founds, scores, stream);
  });
}

REF_API int ref_find_missed(void* t, uint64_t n, const K* keys, V* values,
                            K* missed_keys, int* missed_indices,
                            int* missed_size, S* scores, cudaStream_t stream) {
  return guarded([&] {
    static_cast<const Table*>(t)->find(n, keys, values, missed_keys,
                                       missed_indices, missed_size, scores,
                                       stream);
  });
}

REF_API int ref_find_ptr(void* t, uint64_t n, const K* keys, V** values,
                         bool* founds, S* scores, cudaStream_t stream,
                         int unique_key) {
  return guarded([&] {
    static_cast<const Table*>(t)->find(n, keys, values, founds, scores, stream,
                                       unique_key != 0);
  });
}

REF_API int ref_contains(void* t, uint64_t n, const K* keys, bool* founds,
                         cudaStream_t stream) {
  return guarded(
      [&] { static_cast<const Table*>(t)->contains(n, keys, founds, stream); });
}

REF_API int ref_erase(void* t, uint64_t n, const K* keys, cudaStream_t stream) {
  return guarded([&] { static_cast<Table*>(t)->erase(n, keys, stream); });
}

REF_API int ref_export_batch(void* t, uint64_t n, uint64_t offset,
                             uint64_t* d_counter, K* keys, V* values, S* scores,
                             cudaStream_t stream) {
  return guarded([&] {
    static_cast<const Table*>(t)->export_batch(
        n, offset, reinterpret_cast<size_t*>(d_counter), keys, values, scores,
        stream);
  });
}

// pred: 0 = score < threshold, 1 = score >= threshold,
//       2 = (key & threshold) == pattern.
REF_API int ref_export_batch_if(void* t, int pred, uint64_t pattern,
                                uint64_t threshold, uint64_t n, uint64_t offset,
                                uint64_t* d_counter, K* keys, V* values,
                                S* scores, cudaStream_t stream) {
  return guarded([&] {
    const Table* tb = static_cast<const Table*>(t);
    size_t* c = reinterpret_cast<size_t*>(d_counter);
    switch (pred) {
      case 0:
        tb->export_batch_if<PredScoreLess>(pattern, threshold, n, offset, c,
                                           keys, values, scores, stream);
        break;
      case 1:
        tb->export_batch_if<PredScoreGreaterEq>(pattern, threshold, n, offset,
                                                c, keys, values, scores, stream);
        break;
      case 2:
        tb->export_batch_if<PredKeyMask>(pattern, threshold, n, offset, c, keys,
                                         values, scores, stream);
        break;
      default:
        throw std::invalid_argument("unknown predicate");
    }
  });
}

REF_API int ref_size(void* t, cudaStream_t stream, uint64_t* out) {
  return guarded([&] { *out = static_cast<const Table*>(t)->size(stream); });
}

REF_API int ref_capacity(void* t, uint64_t* out) {
  return guarded([&] { *out = static_cast<const Table*>(t)->capacity(); });
}

REF_API int ref_bucket_count(void* t, uint64_t* out) {
  return guarded([&] { *out = static_cast<const Table*>(t)->bucket_count(); });
}

REF_API int ref_load_factor(void* t, cudaStream_t stream, float* out) {
  return guarded(
      [&] { *out = static_cast<const Table*>(t)->load_factor(stream); });
}

REF_API int ref_clear(void* t, cudaStream_t stream) {
  return guarded([&] { static_cast<Table*>(t)->clear(stream); });
}

// out[0..4] = EMPTY_KEY, RECLAIM_KEY, LOCKED_KEY, empty digest, reclaim digest
// as the reference's device code sees them after init_reserved_keys(bit).
REF_API int ref_probe_reserved(int reserved_key_start_bit, uint64_t* d_out5) {
  return guarded([&] {
    // init_reserved_keys leaves the defaults in place for bit 0
    // (include/merlin/types.cuh:81-85), so a fresh process is assumed there.
    CUDA_CHECK(nv::merlin::init_reserved_keys(reserved_key_start_bit));
    probe_constants_kernel<<<1, 1>>>(d_out5);
    CUDA_CHECK(cudaDeviceSynchronize());
  });
}

REF_API int ref_probe_keys(uint64_t n, const uint64_t* d_keys, uint64_t* d_hashes,
                           uint8_t* d_digests, bool* d_reserved) {
  return guarded([&] {
    probe_keys_kernel<<<unsigned((n + 255) / 256), 256>>>(n, d_keys, d_hashes, d_digests,
                                                          d_reserved);
    CUDA_CHECK(cudaDeviceSynchronize());
  });
}
