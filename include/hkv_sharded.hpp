// nv::merlin::ShardedHashTable -- the key-hash sharded table for C++ callers.
//
// The reference is a single-GPU library; its users shard by hand with one
// HashTable per GPU.  This class is that pattern over the library's fused
// peer-memory path: one object per rank (one rank per GPU), owner(key) =
// Murmur3(key) % world, every batch routed over NVLink with the library's own
// kernels -- keys into the owners' inboxes, rows and flags back into the
// requesters' buffers -- without NCCL and without host synchronisation.
//
//   HashTable<K, V, S, EvictStrategy::kLru> local;   local.init(options);
//   ShardedHashTable<K, V, S, EvictStrategy::kLru> table(&local, world, rank, max_batch, lanes);
//   // ranks in different processes exchange table.ipc_handle(lane) and call
//   // table.connect(lane, all_handles); then a barrier of their own
//   table.find(n, d_keys, stream);                    // results in table.rows(0) / table.flags(0)
//   table.find_or_insert(n, d_keys, stream);          // batch rows in table.rows(0), in and out
//   table.accum_or_assign(n, d_keys, stream, true);   // deltas in table.rows(0), flags in table.flags(0)
//
// Every rank makes the same sequence of calls.  The updates need a strategy
// without caller-supplied scores (kLru, kEpochLru).
#pragma once

#include <cstdint>
#include <vector>

#include "hkv_b200.h"
#include "merlin_hashtable.cuh"

namespace nv {
namespace merlin {

template <class K, class V, class S = uint64_t, int Strategy = EvictStrategy::kLru>
class ShardedHashTable {
 public:
  static_assert(sizeof(K) == 8, "keys are 64-bit");
  using Local = HashTable<K, V, S, Strategy>;

  ShardedHashTable(Local* local, uint32_t world, uint32_t rank, uint64_t max_batch,
                   uint32_t lanes = 1, uint32_t max_polls = 50000000u)
      : local_(local), max_polls_(max_polls) {
    if (hkv_sharded_create(local->native_handle(), world, rank, max_batch, lanes, &s_) != HKV_OK) {
      throw MerlinException(hkv_sharded_last_error());
    }
  }
  // The same over workspaces the caller allocated (one per lane, each
  // workspace_bytes() of device memory every rank can map: CUDA virtual-memory
  // allocations shared through file descriptors or fabric handles, a
  // framework's symmetric memory); connect them with connect(lane, pointers).
  ShardedHashTable(Local* local, uint32_t world, uint32_t rank, uint64_t max_batch,
                   const std::vector<void*>& workspaces, uint32_t max_polls = 50000000u)
      : local_(local), max_polls_(max_polls) {
    if (hkv_sharded_create_external(local->native_handle(), world, rank, max_batch,
                                    static_cast<uint32_t>(workspaces.size()), workspaces.data(),
                                    &s_) != HKV_OK) {
      throw MerlinException(hkv_sharded_last_error());
    }
  }
  static uint64_t workspace_bytes(Local* local, uint32_t world, uint64_t max_batch) {
    uint64_t bytes = 0;
    if (hkv_sharded_workspace_bytes(local->native_handle(), world, max_batch, &bytes) != HKV_OK) {
      throw MerlinException(hkv_sharded_last_error());
    }
    return bytes;
  }
  ShardedHashTable(const ShardedHashTable&) = delete;
  ShardedHashTable& operator=(const ShardedHashTable&) = delete;
  ~ShardedHashTable() { hkv_sharded_destroy(s_); }

  hkv_sharded* native_handle() { return s_; }
  uint32_t lanes() const { return hkv_sharded_lanes(s_); }
  uint64_t max_batch() const { return hkv_sharded_max_batch(s_); }

  // set-up: what the other ranks need to reach this rank's workspace ...
  hkv_ipc_handle ipc_handle(uint32_t lane) {
    hkv_ipc_handle h;
    check(hkv_sharded_ipc_handle(s_, lane, &h));
    return h;
  }
  // ... and the handles of all ranks (index = rank), from other processes
  void connect(uint32_t lane, const std::vector<hkv_ipc_handle>& handles) {
    check(hkv_sharded_connect_ipc(s_, lane, handles.data()));
  }
  // ranks that are threads of one process share plain pointers instead
  void* workspace(uint32_t lane) { return hkv_sharded_workspace(s_, lane); }
  void connect(uint32_t lane, const std::vector<void*>& bases) {
    check(hkv_sharded_connect_pointers(s_, lane, bases.data()));
  }

  // this rank's batch / result rows and flags of a lane (device memory)
  V* rows(uint32_t lane = 0) {
    void* p = nullptr;
    check(hkv_sharded_buffers(s_, lane, &p, nullptr));
    return static_cast<V*>(p);
  }
  bool* flags(uint32_t lane = 0) {
    bool* p = nullptr;
    check(hkv_sharded_buffers(s_, lane, nullptr, &p));
    return p;
  }

  void find(uint64_t n, const K* keys, cudaStream_t stream = 0, uint32_t lane = 0) {
    check(hkv_sharded_find(s_, lane, n, reinterpret_cast<const uint64_t*>(keys), max_polls_, stream));
  }
  // returns the lane whose buffers will hold the results; wait(lane, stream) orders a stream after them
  uint32_t find_async(uint64_t n, const K* keys, cudaStream_t stream = 0) {
    uint32_t lane = 0;
    check(hkv_sharded_find_async(s_, n, reinterpret_cast<const uint64_t*>(keys), max_polls_, stream,
                                 &lane));
    return lane;
  }
  void wait(uint32_t lane, cudaStream_t stream = 0) { check(hkv_sharded_wait(s_, lane, stream)); }

  void insert_or_assign(uint64_t n, const K* keys, cudaStream_t stream = 0) {
    upsert(HKV_ROUTED_INSERT_OR_ASSIGN, n, keys, stream, false);
  }
  void find_or_insert(uint64_t n, const K* keys, cudaStream_t stream = 0) {
    upsert(HKV_ROUTED_FIND_OR_INSERT, n, keys, stream, false);
  }
  // same_keys_as_previous_update: the keys are those of the update every rank made just before
  void accum_or_assign(uint64_t n, const K* keys, cudaStream_t stream = 0,
                       bool same_keys_as_previous_update = false) {
    upsert(HKV_ROUTED_ACCUM_OR_ASSIGN, n, keys, stream, same_keys_as_previous_update);
  }

  // 0, or bit 0 set after a peer barrier timed out (synchronises the stream)
  uint32_t status(uint32_t lane = 0, cudaStream_t stream = 0) {
    uint32_t st = 0;
    check(hkv_sharded_status(s_, lane, stream, &st));
    return st;
  }

  Local* local() { return local_; }

 private:
  void upsert(int op, uint64_t n, const K* keys, cudaStream_t stream, bool reuse) {
    check(hkv_sharded_upsert(s_, op, n, reinterpret_cast<const uint64_t*>(keys), reuse ? 1 : 0,
                             max_polls_, stream));
  }
  static void check(int rc) {
    if (rc != HKV_OK) throw MerlinException(hkv_sharded_last_error());
  }

  Local* local_;
  hkv_sharded* s_ = nullptr;
  uint32_t max_polls_;
};

}  // namespace merlin
}  // namespace nv
