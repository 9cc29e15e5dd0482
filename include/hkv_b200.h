/*
 * hkv_b200 -- C ABI of the B200-native HierarchicalKV hash-table hot path.
 *
 * Every entry point takes plain pointers and sizes.  Batch buffers (keys,
 * values, scores, flags, counters) must be GPU-accessible (device memory or
 * mapped pinned host memory), exactly as the reference requires of its
 * callers (include/merlin_hashtable.cuh:216-221).  All operations enqueue on
 * the caller's stream and return without synchronising, except those that
 * return a count to the host.
 *
 * Each declaration names the reference interface it replaces, by the file's
 * path inside NVIDIA-Merlin/HierarchicalKV.  The drop-in C++ class
 * nv::merlin::HashTable<K,V,S,Strategy> in include/merlin_hashtable.cuh is a
 * thin wrapper over these functions.
 *
 * Key type: 64-bit (uint64_t or int64_t bit pattern).  Score type: uint64_t
 * (uint32_t with the Customized strategy, see hkv_options.score_size).  Value
 * rows are opaque bytes of `dim * value_size` except in hkv_accum_or_assign,
 * which adds elements of the type hkv_options.value_kind names.
 */
#ifndef HKV_B200_H_
#define HKV_B200_H_

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HKV_API __attribute__((visibility("default")))

typedef struct hkv_table hkv_table;
typedef void* hkv_stream; /* cudaStream_t */

/* Return codes.  The C++ wrapper rethrows them as the reference's exception
 * types (include/merlin/debug.hpp:27-72). */
typedef enum hkv_status {
  HKV_OK = 0,
  HKV_ERR_MERLIN = 1,      /* nv::merlin::MerlinException (MERLIN_CHECK failed) */
  HKV_ERR_CUDA = 2,        /* nv::merlin::CudaException   (CUDA_CHECK failed)   */
  HKV_ERR_RUNTIME = 3,     /* std::runtime_error                                 */
  HKV_ERR_INVALID_ARG = 4, /* std::invalid_argument                              */
  HKV_ERR_UNSUPPORTED = 5  /* feature of the reference outside this library      */
} hkv_status;

/* EvictStrategy::EvictStrategyEnum, include/merlin_hashtable.cuh:79-87 */
typedef enum hkv_evict_strategy {
  HKV_LRU = 0,
  HKV_LFU = 1,
  HKV_EPOCH_LRU = 2,
  HKV_EPOCH_LFU = 3,
  HKV_CUSTOMIZED = 4
} hkv_evict_strategy;

/* MemoryType, include/merlin/allocator.cuh:27-31 */
typedef enum hkv_memory_type { HKV_MEM_DEVICE = 0, HKV_MEM_PINNED = 1, HKV_MEM_HOST = 2 } hkv_memory_type;

/* BaseAllocator bridged to C, include/merlin/allocator.cuh:37-59.  Borrowed,
 * never owned.  A null hkv_allocator* selects cudaMalloc / cudaHostAlloc. */
typedef struct hkv_allocator {
  void* ctx;
  int (*alloc)(void* ctx, int memory_type, void** ptr, size_t size, unsigned int pinned_flags);
  int (*free)(void* ctx, int memory_type, void* ptr);
} hkv_allocator;

/* HashTableOptions, include/merlin_hashtable.cuh:103-136, field for field,
 * followed by what the class template carries as template parameters. */
typedef struct hkv_options {
  uint64_t init_capacity;
  uint64_t max_capacity;
  uint64_t max_hbm_for_vectors; /* bytes; 0 puts every value row in pinned host memory */
  uint64_t max_bucket_size;     /* a power of two, 16 ... 1024; 128 runs the tuned kernels */
  uint64_t dim;
  float max_load_factor;
  int32_t block_size;
  int32_t io_block_size;
  int32_t device_id; /* -1: current device */
  int32_t io_by_cpu; /* must be 0 */
  int32_t use_constant_memory;
  int32_t reserved_key_start_bit; /* 0..62 */
  uint64_t num_of_buckets_per_alloc;
  int32_t api_lock;
  int32_t table_mode; /* 0 kThroughput; 1 kMemory: dual-bucket table (insert_or_assign of unique
                         keys, find and the whole-table scans only, as in the reference) */
  /* template parameters of HashTable<K,V,S,Strategy> */
  int32_t evict_strategy; /* hkv_evict_strategy */
  uint32_t value_size;    /* sizeof(V) */
  uint32_t score_size;    /* sizeof(S): 8, or 4 with HKV_CUSTOMIZED; with 4 every `scores` array of
                             this header holds uint32 values (the pointer type stays uint64_t*) */
  uint32_t value_kind;    /* hkv_value_kind: what accum_or_assign adds */
  /* Not in the reference.  Where a slot's key and score live (hkv_slot_layout):
   * HKV_SLOT_PLANES, the default, keeps an array of keys and an array of
   * scores; HKV_SLOT_LINES puts the keys of 8 consecutive slots and their 8
   * scores into one 128-byte line, so the score store every update makes lands
   * in the line its lock has just opened.  Measured on B200 (64 Mi slots, dim
   * 64): lines make updates of resident keys and inserts into free slots about
   * a quarter faster, evicting inserts a sixth slower, find 4 % and contains /
   * find* 12 % slower.  Results are identical. */
  uint32_t slot_layout;
} hkv_options;

typedef enum hkv_slot_layout { HKV_SLOT_PLANES = 0, HKV_SLOT_LINES = 1 } hkv_slot_layout;

/* Element type of V.  Rows are opaque bytes to every operation except
 * accum_or_assign, which adds elements as V's operator+= does in the reference
 * (include/merlin/core_kernels/accum_or_assign.cuh:139-172). */
typedef enum hkv_value_kind {
  HKV_VALUE_OPAQUE = 0, /* accum_or_assign: float32 when sizeof(V) == 4, else rejected */
  HKV_VALUE_F32 = 1,
  HKV_VALUE_F64 = 2,
  HKV_VALUE_I32 = 3,
  HKV_VALUE_I64 = 4,
  HKV_VALUE_F16 = 5,
  HKV_VALUE_BF16 = 6
} hkv_value_kind;

/* Predicates that cross the ABI by number (export_batch_if / size_if /
 * erase_if with the functors the reference's tests and benchmarks use). */
typedef enum hkv_predicate {
  HKV_PRED_ALL = 0,
  HKV_PRED_SCORE_LESS = 1,       /* score <  threshold */
  HKV_PRED_SCORE_GREATER_EQ = 2, /* score >= threshold */
  HKV_PRED_KEY_MASK_EQ = 3,      /* (key & threshold) == pattern */
  HKV_PRED_SCORE_GREATER = 4,    /* score >  threshold */
  HKV_PRED_SCORE_LESS_EQ = 5     /* score <= threshold */
} hkv_predicate;

/* Raw view of the table's planes for header-side kernels that evaluate a
 * user-templated functor (export_batch_if<PredFunctor>, for_each).  Valid
 * until the table is destroyed. */
#define HKV_SLOT_WORD(view, slot) \
  ((uint64_t)(slot) + (((uint64_t)(slot) & ~(uint64_t)7) & (view).slot_word_mask))
typedef struct hkv_table_view {
  uint8_t* digests;      /* [buckets][max_bucket_size] */
  /* Index both arrays with HKV_SLOT_WORD(view, slot), never with the slot itself:
   * with HKV_SLOT_LINES a 128-byte line holds the keys of 8 consecutive slots
   * followed by their 8 scores (scores == keys + 8 then). */
  uint64_t* keys;        /* key of slot s:   keys[HKV_SLOT_WORD(view, s)]   */
  uint64_t* scores;      /* score of slot s: scores[HKV_SLOT_WORD(view, s)] */
  uint8_t* values_hbm;   /* rows of row slots [0, hbm_slots) */
  uint8_t* values_host;  /* rows of row slots [hbm_slots, capacity), mapped pinned */
  int32_t* bucket_sizes; /* [buckets] */
  uint32_t* bucket_map;  /* null, or [buckets]: with B = max_bucket_size the row of slot s is
                            row slot bucket_map[s / B] * B + s % B (hybrid tables) */
  uint64_t buckets;
  uint64_t capacity;
  uint64_t hbm_slots;
  uint64_t row_bytes;
  uint64_t empty_key, reclaim_key, locked_key;
  uint64_t reserved_mask, reserved_value; /* reserved iff (key & mask) == value */
  uint64_t max_bucket_size; /* slots per bucket: bucket of slot s is s / max_bucket_size */
  uint64_t slot_word_mask;  /* all ones with HKV_SLOT_LINES, else 0 (HKV_SLOT_WORD) */
} hkv_table_view;

/* Message of the last failing call on this thread. */
HKV_API const char* hkv_last_error(void);

/* HashTable::init, include/merlin_hashtable.cuh:984-1089 (create_table,
 * include/merlin/core_kernels.cuh:327-381) and ~HashTable 960-970. */
HKV_API int hkv_table_create(const hkv_options* options, const hkv_allocator* allocator,
                             hkv_table** out);
HKV_API int hkv_table_destroy(hkv_table* table);

/* HashTable::insert_or_assign, include/merlin_hashtable.cuh:1125-1305 */
HKV_API int hkv_insert_or_assign(hkv_table* table, uint64_t n, const uint64_t* keys,
                                 const void* values, const uint64_t* scores, hkv_stream stream,
                                 int unique_key, int ignore_evict_strategy);

/* HashTable::insert_and_evict, include/merlin_hashtable.cuh:1351-1473; the
 * caller zeroes *d_evicted_counter. */
HKV_API int hkv_insert_and_evict(hkv_table* table, uint64_t n, const uint64_t* keys,
                                 const void* values, const uint64_t* scores,
                                 uint64_t* evicted_keys, void* evicted_values,
                                 uint64_t* evicted_scores, uint64_t* d_evicted_counter,
                                 hkv_stream stream, int unique_key, int ignore_evict_strategy);
/* count-returning overload, include/merlin_hashtable.cuh:1518-1546
 * (synchronises the stream) */
HKV_API int hkv_insert_and_evict_count(hkv_table* table, uint64_t n, const uint64_t* keys,
                                       const void* values, const uint64_t* scores,
                                       uint64_t* evicted_keys, void* evicted_values,
                                       uint64_t* evicted_scores, hkv_stream stream, int unique_key,
                                       int ignore_evict_strategy, uint64_t* evicted_count);

/* HashTable::accum_or_assign, include/merlin_hashtable.cuh:1589-1680.  Adds
 * elements of hkv_options.value_kind.  A batch may repeat keys, as in the
 * reference (the call has no unique_key argument there). */
HKV_API int hkv_accum_or_assign(hkv_table* table, uint64_t n, const uint64_t* keys,
                                const void* value_or_deltas, const bool* accum_or_assigns,
                                const uint64_t* scores, hkv_stream stream,
                                int ignore_evict_strategy);

/* HashTable::find_or_insert (values in/out), include/merlin_hashtable.cuh:1699-1857 */
HKV_API int hkv_find_or_insert(hkv_table* table, uint64_t n, const uint64_t* keys, void* values,
                               uint64_t* scores, hkv_stream stream, int unique_key,
                               int ignore_evict_strategy);

/* HashTable::find_or_insert (pointer form), include/merlin_hashtable.cuh:1883-1965;
 * with locked_key_ptrs the keys stay locked until hkv_unlock_keys. */
HKV_API int hkv_find_or_insert_ptr(hkv_table* table, uint64_t n, const uint64_t* keys,
                                   void** values, bool* founds, uint64_t* scores,
                                   hkv_stream stream, int unique_key, int ignore_evict_strategy,
                                   uint64_t** locked_key_ptrs);

/* HashTable::lock_keys / unlock_keys, include/merlin_hashtable.cuh:1982-2044 */
HKV_API int hkv_lock_keys(hkv_table* table, uint64_t n, const uint64_t* keys,
                          uint64_t** locked_key_ptrs, bool* success, hkv_stream stream,
                          const uint64_t* scores);
HKV_API int hkv_unlock_keys(hkv_table* table, uint64_t n, uint64_t** locked_key_ptrs,
                            const uint64_t* keys, bool* success, hkv_stream stream);

/* HashTable::assign, include/merlin_hashtable.cuh:2071-2205 */
HKV_API int hkv_assign(hkv_table* table, uint64_t n, const uint64_t* keys, const void* values,
                       const uint64_t* scores, hkv_stream stream, int unique_key);
/* HashTable::assign_scores, include/merlin_hashtable.cuh:2228-2283 */
HKV_API int hkv_assign_scores(hkv_table* table, uint64_t n, const uint64_t* keys,
                              const uint64_t* scores, hkv_stream stream, int unique_key);
/* HashTable::assign_values, include/merlin_hashtable.cuh:2299-2444 */
HKV_API int hkv_assign_values(hkv_table* table, uint64_t n, const uint64_t* keys,
                              const void* values, hkv_stream stream, int unique_key);

/* HashTable::find, include/merlin_hashtable.cuh:2464-2577 */
HKV_API int hkv_find(hkv_table* table, uint64_t n, const uint64_t* keys, void* values,
                     bool* founds, uint64_t* scores, hkv_stream stream);
/* HashTable::find, include/merlin_hashtable.cuh:2464-2577, for batches that live in HOST memory
 * (the reference wants every batch buffer GPU-accessible, include/merlin_hashtable.cuh:216-221, and
 * leaves the staging to the caller).  The batch is cut into chunks of about 32 MiB of rows that
 * alternate over two internal streams and two sets of staging buffers: key copy, lookup and row
 * copy of neighbouring chunks overlap, so the call runs at the rate of the host link.  All of it
 * is ordered after what `stream` holds at the call and before what is queued on `stream`
 * afterwards; the host buffers are complete once `stream` has reached that point.  Pinned
 * host memory gives asynchronous copies, pageable memory works but blocks per chunk.  Rows of keys
 * that are not in the table come back as zero bytes (hkv_find leaves them untouched).  Scores
 * (optional) for tables with 64-bit scores.  Calls on one table take turns.  Not for use
 * inside a stream capture. */
HKV_API int hkv_find_host(hkv_table* table, uint64_t n, const uint64_t* host_keys,
                          void* host_values, bool* host_founds, uint64_t* host_scores,
                          hkv_stream stream);
/* HashTable::find (missed-keys form), include/merlin_hashtable.cuh:2600-2705 */
HKV_API int hkv_find_missed(hkv_table* table, uint64_t n, const uint64_t* keys, void* values,
                            uint64_t* missed_keys, int* missed_indices, int* missed_size,
                            uint64_t* scores, hkv_stream stream);
/* HashTable::find (pointer form, "find*"), include/merlin_hashtable.cuh:2729-2787 */
HKV_API int hkv_find_ptr(hkv_table* table, uint64_t n, const uint64_t* keys, void** values,
                         bool* founds, uint64_t* scores, hkv_stream stream, int unique_key);
/* HashTable::find_and_update, include/merlin_hashtable.cuh:2811-2843 */
HKV_API int hkv_find_and_update(hkv_table* table, uint64_t n, const uint64_t* keys, void** values,
                                bool* founds, uint64_t* scores, hkv_stream stream, int unique_key);
/* HashTable::contains, include/merlin_hashtable.cuh:2856-2894 */
HKV_API int hkv_contains(hkv_table* table, uint64_t n, const uint64_t* keys, bool* founds,
                         hkv_stream stream);

/* HashTable::erase, include/merlin_hashtable.cuh:2904-2930 */
HKV_API int hkv_erase(hkv_table* table, uint64_t n, const uint64_t* keys, hkv_stream stream);
/* HashTable::erase_if<PredFunctor>, include/merlin_hashtable.cuh:2964-2996, for
 * the built-in predicates; returns the number of erased keys (synchronises). */
HKV_API int hkv_erase_if(hkv_table* table, int predicate, uint64_t pattern, uint64_t threshold,
                         hkv_stream stream, uint64_t* erased);
/* HashTable::clear, include/merlin_hashtable.cuh:3059-3073 */
HKV_API int hkv_clear(hkv_table* table, hkv_stream stream);

/* HashTable::export_batch, include/merlin_hashtable.cuh:3099-3147; n and
 * offset count slots; *d_counter is zeroed by the call. */
HKV_API int hkv_export_batch(hkv_table* table, uint64_t n, uint64_t offset, uint64_t* d_counter,
                             uint64_t* keys, void* values, uint64_t* scores, hkv_stream stream);
/* count-returning overload, include/merlin_hashtable.cuh:3131-3147 (synchronises) */
HKV_API int hkv_export_batch_count(hkv_table* table, uint64_t n, uint64_t offset, uint64_t* keys,
                                   void* values, uint64_t* scores, hkv_stream stream,
                                   uint64_t* count);
/* HashTable::export_batch_if<PredFunctor>, include/merlin_hashtable.cuh:3193-3276,
 * for the built-in predicates */
HKV_API int hkv_export_batch_if(hkv_table* table, int predicate, uint64_t pattern,
                                uint64_t threshold, uint64_t n, uint64_t offset,
                                uint64_t* d_counter, uint64_t* keys, void* values,
                                uint64_t* scores, hkv_stream stream);
/* HashTable::size_if<PredFunctor>, include/merlin_hashtable.cuh:3459-3476 */
HKV_API int hkv_size_if(hkv_table* table, int predicate, uint64_t pattern, uint64_t threshold,
                        uint64_t* d_counter, hkv_stream stream);

/* HashTable::size / empty / load_factor / capacity / bucket_count / dim /
 * max_bucket_size, include/merlin_hashtable.cuh:3416-3451,3487,3551-3553,3586-3602 */
HKV_API int hkv_size(hkv_table* table, hkv_stream stream, uint64_t* size);
HKV_API int hkv_load_factor(hkv_table* table, hkv_stream stream, float* load_factor);
HKV_API uint64_t hkv_capacity(const hkv_table* table);
HKV_API uint64_t hkv_bucket_count(const hkv_table* table);
HKV_API uint64_t hkv_dim(const hkv_table* table);
HKV_API uint64_t hkv_max_bucket_size(const hkv_table* table);

/* No counterpart in the reference.  hkv_size for callers that must not
 * allocate: processes whose set-up phase is over and whose memory budget is
 * fixed (serving loops, plug-ins inside a host application that owns every
 * allocation, monitoring threads that must not cause the device-wide
 * synchronisation an allocation implies).  The partial sums live in a fixed
 * array inside the library image instead of scratch memory obtained at run
 * time, so the call obtains no device memory: no cudaMalloc / cudaFree, no
 * stream-ordered allocation, no library routine that allocates on the device.
 * (Host side, two small things remain: with api_lock on, the first call that
 * uses a new stream makes the table's lock create one CUDA event for that
 * stream, and a failing call builds its error message as a string.)  Limits
 * and rules:
 *   - tables of at most 4,194,304 buckets (2^29 slots); larger ones are
 *     rejected with HKV_ERR_INVALID_ARG -- use hkv_size for them;
 *   - every GPU that loads the library holds the array (about 32 KiB) until
 *     the process exits;
 *   - the first call on a device resolves the array's device address; make
 *     that first call before any stream capture begins;
 *   - all calls share the array: calls that overlap on one GPU (two streams,
 *     two threads) race and must be serialised by the caller.
 * Synchronises the stream, like hkv_size.  The message of a failure is
 * returned by hkv_size_no_alloc_last_error. */
HKV_API int hkv_size_no_alloc(hkv_table* table, hkv_stream stream, uint64_t* size);
HKV_API const char* hkv_size_no_alloc_last_error(void);

/* HashTable::set_global_epoch, include/merlin_hashtable.cuh:3760 */
HKV_API int hkv_set_global_epoch(hkv_table* table, uint64_t epoch);

/* HashTable::reserve, include/merlin_hashtable.cuh:3503-3545.  Doubles the
 * capacity (rehashing every entry) until it reaches new_capacity or the next
 * doubling would pass max_capacity; a request above max_capacity is ignored.
 * The insert-like calls grow the same way before they run, while the load
 * estimated from the first 1024 buckets plus the batch is above
 * max_load_factor (include/merlin_hashtable.cuh:1151-1154, 3796-3828).  Only
 * tables created with init_capacity * 2 <= max_capacity grow.  Synchronises
 * the device; row and key pointers handed out before are invalid afterwards. */
HKV_API int hkv_reserve(hkv_table* table, uint64_t new_capacity, hkv_stream stream);

/* HashTable::set_max_capacity, include/merlin_hashtable.cuh:3561-3579.
 * HKV_ERR_INVALID_ARG (std::invalid_argument in the reference) unless
 * new_max_capacity is a power of two; ignored when below the capacity. */
HKV_API int hkv_set_max_capacity(hkv_table* table, uint64_t new_max_capacity);

/* Hybrid tables (rows partly in HBM, partly in pinned host memory): moves the
 * rows of the host-resident buckets with the most lookup hits since the last
 * call into HBM, in exchange for the coldest HBM-resident buckets, and halves
 * the hit counters.  *promoted receives the number of buckets moved in (0 for
 * a table that is not hybrid).  Exclusive like clear; synchronises the stream.
 * Row pointers handed out before are invalid afterwards.  No counterpart in the
 * reference, whose README lists a warm-up of hot rows as planned. */
HKV_API int hkv_promote_hot_buckets(hkv_table* table, hkv_stream stream, uint64_t* promoted);

/* Planes of the table for header-side functor kernels.  No counterpart in
 * the reference, whose templated kernels live in the class itself.  The planes
 * are replaced when the table doubles (hkv_reserve, growth on the insert
 * path): fetch the view between hkv_external_begin and hkv_external_end. */
HKV_API int hkv_get_view(const hkv_table* table, hkv_table_view* view);

/* Bracket a kernel the CALLER launches on `stream` over hkv_get_view's planes
 * so that it takes part in the table's reader (0) / updater (1) / inserter
 * (2) exclusion, as the reference's lock guards do around its templated
 * kernels (include/merlin/group_lock.cuh:168-337).  begin orders the stream
 * after conflicting operations; end must follow the launch on the same host
 * thread.  Both are no-ops when api_lock is off. */
HKV_API int hkv_external_begin(hkv_table* table, int group, hkv_stream stream);
HKV_API int hkv_external_end(hkv_table* table, int group, hkv_stream stream);

/* ---- key-hash sharding across GPUs ------------------------------------------
 * No counterpart in the reference, which is a single-GPU library: its users
 * shard by hand, one table per GPU.  owner(key) = Murmur3(key) % world, the
 * hash being the table's own (include/merlin/utils.cuh:137-145).  The helpers
 * below are pure device work on the caller's stream; the exchange between
 * ranks (NCCL all-to-all) is done by the caller. */

/* Groups a batch by owner rank.  d_counts[world] receives the keys per owner,
 * d_offsets[world] their exclusive prefix sum, grouped_keys[n] the keys owner
 * by owner, origin[n] the batch index each grouped key came from.
 * d_cursors[world] is scratch.  All pointers are device memory. */
HKV_API int hkv_shard_partition(uint64_t n, const uint64_t* keys, uint32_t world,
                                uint64_t* d_counts, uint64_t* d_offsets, uint64_t* d_cursors,
                                uint64_t* grouped_keys, uint32_t* origin, hkv_stream stream);
/* dst[i] = src[index[i]] for rows of row_bytes bytes */
HKV_API int hkv_shard_gather_rows(uint64_t n, uint64_t row_bytes, const void* src_rows,
                                  const uint32_t* index, void* dst_rows, hkv_stream stream);
/* dst[index[i]] = src[i]; rows whose index is 0xFFFFFFFF are skipped */
HKV_API int hkv_shard_scatter_rows(uint64_t n, uint64_t row_bytes, const void* src_rows,
                                   const uint32_t* index, void* dst_rows, hkv_stream stream);
HKV_API const char* hkv_shard_last_error(void);

/* Peer buffers of the ranks of one node: p[r] is rank r's buffer, mapped into
 * this process (CUDA IPC / symmetric memory).  At most 16 ranks. */
typedef struct hkv_peer_ptrs {
  void* p[16];
} hkv_peer_ptrs;

/* Fused routing, no counterpart in the reference.  Every rank owns an inbox
 * of `world` segments of `segment_capacity` entries: keys (uint64), origins
 * (uint32) and one count per segment (uint64).  This call groups the batch by
 * owner and stores each key and its batch index directly into segment
 * `my_rank` of the owner's inbox over NVLink, then the counts.  d_cursors is
 * world x uint64 of local scratch. */
HKV_API int hkv_shard_route_keys_p2p(uint64_t n, const uint64_t* keys, uint32_t world,
                                     uint32_t my_rank, uint64_t segment_capacity,
                                     const hkv_peer_ptrs* inbox_keys,
                                     const hkv_peer_ptrs* inbox_origin,
                                     const hkv_peer_ptrs* inbox_counts, uint64_t* d_cursors,
                                     hkv_stream stream);
/* Barrier of the node's ranks on `stream` over peer flags (uint32[16] per
 * rank, zero-initialised; `epoch` grows by one per call on every rank).  The
 * wait is bounded by max_polls; a time-out sets bit 0 of *d_status instead
 * of hanging. */
HKV_API int hkv_shard_barrier(uint32_t world, uint32_t my_rank, const hkv_peer_ptrs* flags,
                              uint32_t epoch, uint32_t* d_status, uint32_t max_polls,
                              hkv_stream stream);
/* HashTable::find (include/merlin_hashtable.cuh:2464-2577) for the owner side
 * of the sharded table: looks up every key of this rank's inbox and stores
 * hit rows and found flags straight into the requesting rank's result buffers
 * (out_values->p[s], out_founds->p[s], indexed by the key's origin). */
HKV_API int hkv_find_routed(hkv_table* table, uint32_t world, uint32_t my_rank,
                            uint64_t segment_capacity,
                            const uint64_t* inbox_keys, const uint32_t* inbox_origin,
                            const uint64_t* inbox_counts, const hkv_peer_ptrs* out_values,
                            const hkv_peer_ptrs* out_founds, hkv_stream stream);

/* insert_or_assign (op 0), find_or_insert (op 1) and accum_or_assign (op 2)
 * (include/merlin_hashtable.cuh:1125, 1699, 1589) for the owner side of the
 * sharded table, on the same inbox as hkv_find_routed.  Key i of segment s
 * owns row inbox_origin[i] of values->p[s], the requesting rank's batch buffer,
 * which the kernels read (new rows, deltas) and write (rows found by
 * find_or_insert) in place over NVLink; accum_flags->p[s] is that rank's
 * accum_or_assigns array, indexed like the rows (op 2 only).  The segments are
 * applied one after the other, starting with rank my_rank + 1 and wrapping, so
 * a key requested by several ranks behaves as if those ranks had called the
 * table in that order.  Scores cannot be routed: the table's strategy must be
 * kLru or kEpochLru. */
#define HKV_ROUTED_INSERT_OR_ASSIGN 0
#define HKV_ROUTED_FIND_OR_INSERT 1
#define HKV_ROUTED_ACCUM_OR_ASSIGN 2
HKV_API int hkv_upsert_routed(hkv_table* table, int op, uint32_t world, uint32_t my_rank,
                              uint64_t segment_capacity, const uint64_t* inbox_keys,
                              const uint32_t* inbox_origin, const uint64_t* inbox_counts,
                              const hkv_peer_ptrs* values, const hkv_peer_ptrs* accum_flags,
                              hkv_stream stream);

/* ---- the sharded table's host side -----------------------------------------
 * No counterpart in the reference.  One hkv_sharded per rank (one rank per GPU;
 * ranks are processes, or threads of one process) wraps that rank's sub-table
 * and its peer workspaces ("lanes": inbox of routed keys, barrier flags, batch /
 * result buffers; allocated here with cudaMalloc and shared over CUDA IPC, or
 * supplied by the caller -- hkv_sharded_create_external).
 * Set-up, once:
 *   1. every rank: hkv_sharded_create;
 *   2. ranks in different processes exchange hkv_sharded_ipc_handle of every
 *      lane by any means they have (files, sockets, MPI, torch.distributed) and
 *      call hkv_sharded_connect_ipc; threads of one process pass each other
 *      hkv_sharded_workspace pointers, enable peer access and call
 *      hkv_sharded_connect_pointers;
 *   3. a barrier of the caller's own before the first operation (every rank's
 *      workspace must be connected and its flags still zero).
 * Every rank then makes the same sequence of calls.  The device-side barriers
 * are bounded by max_polls: a rank that never arrives sets bit 0 of the lane's
 * status word instead of hanging the others. */
typedef struct hkv_sharded hkv_sharded;
typedef struct hkv_ipc_handle {
  unsigned char bytes[64]; /* a cudaIpcMemHandle_t */
} hkv_ipc_handle;

HKV_API int hkv_sharded_create(hkv_table* table, uint32_t world, uint32_t rank,
                               uint64_t max_batch, uint32_t lanes, hkv_sharded** out);
/* The same with workspaces the caller supplies: workspaces[lanes], each
 * hkv_sharded_workspace_bytes of device memory on the table's GPU that every
 * rank can map (CUDA virtual-memory allocations shared through file
 * descriptors or fabric handles, a framework's symmetric memory, ...).  The
 * library clears them, never frees them and cannot export them
 * (hkv_sharded_ipc_handle fails): the caller maps its peers' workspaces itself
 * and passes the addresses to hkv_sharded_connect_pointers. */
HKV_API int hkv_sharded_workspace_bytes(hkv_table* table, uint32_t world, uint64_t max_batch,
                                        uint64_t* bytes);
HKV_API int hkv_sharded_create_external(hkv_table* table, uint32_t world, uint32_t rank,
                                        uint64_t max_batch, uint32_t lanes,
                                        void* const* workspaces, hkv_sharded** out);
HKV_API int hkv_sharded_destroy(hkv_sharded* sharded);
HKV_API uint32_t hkv_sharded_lanes(const hkv_sharded* sharded);
HKV_API uint64_t hkv_sharded_max_batch(const hkv_sharded* sharded);
HKV_API int hkv_sharded_ipc_handle(hkv_sharded* sharded, uint32_t lane, hkv_ipc_handle* handle);
/* handles[world]: every rank's handle of this lane (this rank's own is ignored) */
HKV_API int hkv_sharded_connect_ipc(hkv_sharded* sharded, uint32_t lane,
                                    const hkv_ipc_handle* handles);
HKV_API void* hkv_sharded_workspace(hkv_sharded* sharded, uint32_t lane);
/* bases[world]: every rank's hkv_sharded_workspace of this lane, valid in this process */
HKV_API int hkv_sharded_connect_pointers(hkv_sharded* sharded, uint32_t lane, void* const* bases);
/* This rank's buffers of a lane: rows (max_batch x row bytes) are the results
 * of find and the batch rows of the updates, flags (max_batch) the found flags
 * of find and the accum_or_assigns of accum_or_assign. */
HKV_API int hkv_sharded_buffers(hkv_sharded* sharded, uint32_t lane, void** rows, bool** flags);
/* HashTable::find over all shards (include/merlin_hashtable.cuh:2464 per shard):
 * keys are routed to their owners, every owner looks up what arrived and stores
 * hit rows and found flags into the requesters' buffers of `lane`, row i for
 * key i.  Rows of misses keep their previous content.  Enqueued on `stream`. */
HKV_API int hkv_sharded_find(hkv_sharded* sharded, uint32_t lane, uint64_t n, const uint64_t* keys,
                             uint32_t max_polls, hkv_stream stream);
/* The same on the next lane's own streams (routing and barriers at high
 * priority), so that the routing of batch k + 1 overlaps the lookup of batch
 * k: returns at once with the lane it used; hkv_sharded_wait makes a stream
 * wait for that lane's results.  Issue batch k + 1 before waiting for batch k. */
HKV_API int hkv_sharded_find_async(hkv_sharded* sharded, uint64_t n, const uint64_t* keys,
                                   uint32_t max_polls, hkv_stream stream, uint32_t* lane_used);
HKV_API int hkv_sharded_wait(hkv_sharded* sharded, uint32_t lane, hkv_stream stream);
/* insert_or_assign / find_or_insert / accum_or_assign over all shards
 * (op: HKV_ROUTED_*; include/merlin_hashtable.cuh:1125, 1699, 1589 per shard).
 * The batch rows are the first n rows of lane 0's buffers (accum_or_assign: its
 * flags too); find_or_insert writes the stored rows of the hits back into
 * them.  A key several ranks send is applied as if those ranks had called the
 * table one after the other, starting with rank owner + 1 and wrapping.
 * reuse_route != 0: `keys` are the keys of the previous hkv_sharded_upsert call
 * on every rank (the update that follows a find_or_insert of the same batch);
 * the inboxes still hold them and the routing is skipped. */
HKV_API int hkv_sharded_upsert(hkv_sharded* sharded, int op, uint64_t n, const uint64_t* keys,
                               int reuse_route, uint32_t max_polls, hkv_stream stream);
/* bit 0: a peer barrier of this lane timed out.  Synchronises the stream. */
HKV_API int hkv_sharded_status(hkv_sharded* sharded, uint32_t lane, hkv_stream stream,
                               uint32_t* status);
HKV_API const char* hkv_sharded_last_error(void);

/* hkv_accum_or_assign for batches the caller guarantees to hold each key once
 * (the sharded table de-duplicates before routing): one launch of the probe
 * kernel the other insert-like operations use, without the second pass that
 * serves repeated and newly inserted keys one after the other.  The reference
 * has a single, key-scanning tile kernel here
 * (include/merlin/core_kernels/accum_or_assign.cuh:83-174). */
HKV_API int hkv_accum_or_assign_unique(hkv_table* table, uint64_t n, const uint64_t* keys,
                                       const void* value_or_deltas, const bool* accum_or_assigns,
                                       const uint64_t* scores, hkv_stream stream,
                                       int ignore_evict_strategy);

/* Device status word: bit 0 a bounded slot wait ran out, bit 1 eviction
 * retries ran out.  Reading it synchronises the stream; it is cleared by the
 * read.  (The reference spins without bound in these places:
 * include/merlin/core_kernels/kernel_utils.cuh:853-855, upsert.cuh:149.) */
HKV_API int hkv_device_status(hkv_table* table, hkv_stream stream, uint32_t* status);

#ifdef __cplusplus
}
#endif

#endif /* HKV_B200_H_ */
