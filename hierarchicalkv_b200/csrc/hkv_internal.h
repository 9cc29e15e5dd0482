// Launchers shared between the kernel translation units and the C-ABI layer.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "hkv_device.cuh"

namespace hkv {

// Operations served by the mutating kernel (hkv_upsert.cu).
enum MutateOp : int {
  kOpInsertOrAssign = 0,   // HashTable::insert_or_assign
  kOpFindOrInsert = 1,     // HashTable::find_or_insert (values in/out)
  kOpInsertAndEvict = 2,   // HashTable::insert_and_evict
  kOpFindOrInsertPtr = 3,  // HashTable::find_or_insert (pointer form)
  kOpAccumOrAssign = 4,    // HashTable::accum_or_assign
  kOpAssign = 5,           // HashTable::assign (values + scores)
  kOpAssignScores = 6,     // HashTable::assign_scores
  kOpAssignValues = 7,     // HashTable::assign_values
  kOpFindAndUpdate = 8,    // HashTable::find_and_update
  kOpLockKeys = 9,         // HashTable::lock_keys
  kOpErase = 10,           // HashTable::erase
};

struct MutateArgs {
  const uint64_t* keys = nullptr;
  uint64_t n = 0;
  uint8_t* values = nullptr;          // batch rows (read, or read/write)
  const uint64_t* scores = nullptr;   // input scores, may be null
  uint64_t* scores_out = nullptr;     // find_and_update: scores returned
  void** ptrs = nullptr;              // pointer forms: row addresses out
  bool* founds = nullptr;             // pointer forms: hit flags out
  uint64_t** locked_key_ptrs = nullptr;  // keys left locked when non-null
  const bool* accum_flags = nullptr;
  uint64_t* evicted_keys = nullptr;
  uint8_t* evicted_values = nullptr;
  uint64_t* evicted_scores = nullptr;
  unsigned long long* evicted_counter = nullptr;
  int strategy = kLru;
  uint64_t epoch = kIgnoredEpoch;
  // Routed form (launch_mutate_routed): the keys are one source rank's segment
  // of the owner's inbox; key i's row is row row_index[i] of `values` (the
  // source rank's buffer, possibly peer memory), its accumulate flag is
  // accum_flags[row_index[i]], and the number of keys is read on the device.
  const uint32_t* row_index = nullptr;
  const uint64_t* n_device = nullptr;
  // accum_or_assign on batches that may repeat a key: the fast kernel handles
  // every accumulating key whose slot it can lock and appends the batch index
  // of the others (assigning keys, and keys whose slot another occurrence holds
  // at that moment) to deferred_list; the serialising kernel then walks that
  // list (index_list / index_count).
  uint32_t* deferred_list = nullptr;
  unsigned int* deferred_count = nullptr;
  const uint32_t* index_list = nullptr;
  const unsigned int* index_count = nullptr;
};

// `work` / `work_bytes`: scratch for the sort of the hybrid find
// (find_workspace_bytes; null: the one-kernel form runs instead).
void launch_find(const TableView& t, uint64_t n, const uint64_t* keys, void* values, bool* founds,
                 uint64_t* scores, cudaStream_t stream, void* work = nullptr, size_t work_bytes = 0);
// Scratch find needs for n keys on this table: 0 unless rows live in host memory.
size_t find_workspace_bytes(const TableView& t, uint64_t n, const void* values);
void launch_find_ptr(const TableView& t, uint64_t n, const uint64_t* keys, void** ptrs,
                     bool* founds, uint64_t* scores, cudaStream_t stream);
void launch_find_missed(const TableView& t, uint64_t n, const uint64_t* keys, void* values,
                        uint64_t* missed_keys, int* missed_indices, int* missed_size,
                        uint64_t* scores, cudaStream_t stream);
void launch_contains(const TableView& t, uint64_t n, const uint64_t* keys, bool* founds,
                     cudaStream_t stream);

// Dual-bucket tables (TableMode::kMemory): find and insert_or_assign of unique keys.
void launch_dual_find(const TableView& t, uint64_t n, const uint64_t* keys, void* values,
                      bool* founds, uint64_t* scores, cudaStream_t stream);
void launch_dual_upsert(const TableView& t, const MutateArgs& args, cudaStream_t stream);

// Peer buffers of the sharded table, one pointer per rank (world <= kMaxPeers).
constexpr int kMaxPeers = 16;
struct PeerPtrs {
  void* p[kMaxPeers];
};

// find over an inbox of keys that arrived from `world` source ranks: segment s
// holds inbox_counts[s] keys and, for each, the row index it came from in the
// source's batch.  Hit rows and found flags are stored straight into the
// source rank's result buffers.
void launch_find_routed(const TableView& t, uint32_t world, uint32_t my_rank,
                        uint64_t segment_capacity,
                        const uint64_t* inbox_keys, const uint32_t* inbox_origin,
                        const uint64_t* inbox_counts, const PeerPtrs& out_values,
                        const PeerPtrs& out_founds, cudaStream_t stream);

// unique_key == false selects the serialising kernel that tolerates repeated
// keys inside one batch.
// `work`: scratch of mutate_workspace_bytes(op, n, unique_key) bytes for the
// list of keys the fast kernel leaves to the serialising one (null: batches
// that may repeat keys run on the serialising kernel alone).
void launch_mutate(int op, const TableView& t, const MutateArgs& args, bool unique_key,
                   cudaStream_t stream, void* work = nullptr);
size_t mutate_workspace_bytes(int op, uint64_t n, bool unique_key);

// insert_or_assign / find_or_insert / accum_or_assign over the inbox segments
// of a key-hash sharded table (segment s: the keys source rank s sent, each
// with the row it has in that rank's batch buffer).  A key that several ranks
// sent is applied as if those ranks had called the table one after the other
// in the order first_segment, first_segment + 1, ... (wrapping): the requests
// for one key are chained in a scratch hash table first, the first rank in
// that order serves the key in the warp-parallel kernel and applies the other
// ranks' requests behind its own while it holds the slot.
struct RoutedArgs {
  uint32_t world = 0;
  uint32_t first_segment = 0;
  uint64_t segment_capacity = 0;       // a multiple of 32, at most 2^28
  const uint64_t* inbox_keys = nullptr;
  const uint32_t* inbox_origin = nullptr;
  const uint64_t* inbox_counts = nullptr;
  PeerPtrs values_of{};                // each source rank's batch rows
  PeerPtrs flags_of{};                 // accum_or_assign: each source rank's flags
  // grouping scratch (routed_workspace_bytes): an open-addressing set of the
  // inbox's keys, the head of each key's request chain, and per inbox entry
  // the next request for the same key and the set slot of its key; then what
  // the resolving pass leaves for the serving pass: a plan word per entry and
  // the later ranks' requests of every key as runs of a list array
  uint64_t* set_keys = nullptr;
  uint32_t* set_head = nullptr;
  uint32_t* next = nullptr;
  uint32_t* set_slot = nullptr;
  uint32_t set_bits = 0;               // log2 of the set's size
  uint64_t* plan = nullptr;
  uint32_t* lists = nullptr;
  uint32_t* list_cursor = nullptr;     // zero between calls
};
size_t routed_workspace_bytes(uint32_t world, uint64_t segment_capacity);
// Carves `work` into the scratch arrays of `r`; `fresh`: the memory is new and
// is put into the all-empty state the calls leave behind.
void prepare_routed_workspace(const TableView& t, RoutedArgs& r, void* work, bool fresh,
                              cudaStream_t stream);
void launch_mutate_routed(int op, const TableView& t, const MutateArgs& args, const RoutedArgs& r,
                          cudaStream_t stream);

void launch_unlock_keys(const TableView& t, uint64_t n, uint64_t** locked_key_ptrs,
                        const uint64_t* keys, bool* success, cudaStream_t stream);

void launch_erase(const TableView& t, uint64_t n, const uint64_t* keys, cudaStream_t stream);

// Predicates of export_batch_if / size_if that cross the C ABI by number.
enum Predicate : int {
  kPredAll = 0,             // every live slot (export_batch)
  kPredScoreLess = 1,       // score <  threshold
  kPredScoreGreaterEq = 2,  // score >= threshold
  kPredKeyMaskEq = 3,       // (key & threshold) == pattern
  kPredScoreGreater = 4,    // score >  threshold
  kPredScoreLessEq = 5,     // score <= threshold
};

void launch_export(const TableView& t, int pred, uint64_t pattern, uint64_t threshold, uint64_t n,
                   uint64_t offset, unsigned long long* d_counter, uint64_t* keys, void* values,
                   uint64_t* scores, cudaStream_t stream);
void launch_size_if(const TableView& t, int pred, uint64_t pattern, uint64_t threshold,
                    unsigned long long* d_counter, cudaStream_t stream);
void launch_erase_if(const TableView& t, int pred, uint64_t pattern, uint64_t threshold,
                     unsigned long long* d_counter, cudaStream_t stream);
void launch_clear(const TableView& t, cudaStream_t stream);
// Sum of the sizes of the first `buckets` buckets.
void launch_sum_sizes(const TableView& t, uint64_t buckets, unsigned long long* d_total,
                      cudaStream_t stream);
// Hybrid tables: bucket b keeps its rows in row block bucket_map[b].
void launch_identity_map(const TableView& t, cudaStream_t stream);
void launch_decay_heat(const TableView& t, cudaStream_t stream);
// pairs[2p], pairs[2p+1]: buckets that trade row blocks (each bucket at most once).
void launch_swap_row_blocks(const TableView& t, const uint32_t* pairs, uint64_t n_pairs,
                            cudaStream_t stream);
// uint32 score arrays of the API boundary (sizeof(S) == 4) to and from uint64.
void launch_widen_scores(const uint32_t* in, uint64_t* out, uint64_t n, cudaStream_t stream);
void launch_narrow_scores(const uint64_t* in, uint32_t* out, uint64_t n, cudaStream_t stream);
// Moves every live entry of `src` into the cleared table `dst`, which must have
// exactly twice the buckets and a power-of-two capacity.
void launch_rehash(const TableView& src, const TableView& dst, cudaStream_t stream);

}  // namespace hkv
