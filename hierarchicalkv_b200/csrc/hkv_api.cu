// C-ABI layer: table life cycle, option checks, the stream-ordered group lock
// and one thin function per operation of include/hkv_b200.h.
//
// Host logic follows the reference's HashTable methods
// (include/merlin_hashtable.cuh: init 984-1089, check_evict_strategy 3832-3861,
// export clamp 3206-3212, size 3424-3451) and create_table
// (include/merlin/core_kernels.cuh:327-381).
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/hkv_b200.h"
#include "hkv_device.cuh"
#include "hkv_internal.h"

namespace {

thread_local std::string g_last_error;

struct HkvError {
  int code;
  std::string msg;
};

#define HKV_CUDA(call)                                                                   \
  do {                                                                                   \
    cudaError_t e_ = (call);                                                             \
    if (e_ != cudaSuccess) {                                                             \
      throw HkvError{HKV_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(e_)};  \
    }                                                                                    \
  } while (0)

#define HKV_CHECK(cond, msg)                               \
  do {                                                     \
    if (!(cond)) throw HkvError{HKV_ERR_MERLIN, (msg)};    \
  } while (0)

// ---- stream-ordered group lock ----------------------------------------------
//
// The reference serialises readers / updaters / inserters with a host+device
// mutex: every acquire launches a one-thread kernel and synchronises a side
// stream, every release is another one-thread kernel
// (include/merlin/group_lock.cuh:57-337, core_kernels/group_lock_kernels.cuh).
// Here the same exclusion (readers share, updaters share, inserters are alone)
// is expressed as stream dependencies: an operation makes ITS stream wait on
// the completion events of the incompatible operations enqueued before it on
// OTHER streams, and leaves an event behind for later ones.  Nothing blocks on
// the host and no extra kernel runs; operations on one stream are ordered by
// the stream itself.
enum Group : int { kReader = 0, kUpdater = 1, kInserter = 2 };

class StreamGroupLock {
 public:
  ~StreamGroupLock() {
    for (auto& e : entries_) cudaEventDestroy(e.event);
  }

  // Held from acquire() to release() by the enqueueing host thread.
  void acquire(Group g, cudaStream_t stream) {
    mu_.lock();
    for (auto& e : entries_) {
      if (!e.pending || e.stream == stream) continue;
      const bool compatible = (e.group == g) && g != kInserter;
      if (compatible) continue;
      if (cudaEventQuery(e.event) == cudaSuccess) {
        e.pending = false;
        continue;
      }
      cudaStreamWaitEvent(stream, e.event, 0);
    }
    if (g == kInserter) {
      // everything enqueued before is now ordered before this operation
      for (auto& e : entries_) {
        if (e.stream != stream) e.pending = false;
      }
    }
  }

  void release(Group g, cudaStream_t stream) {
    Entry* slot = nullptr;
    for (auto& e : entries_) {
      if (e.stream == stream && e.group == g) {
        slot = &e;
        break;
      }
    }
    if (slot == nullptr) {
      for (auto& e : entries_) {
        if (!e.pending) {
          slot = &e;
          break;
        }
      }
    }
    if (slot == nullptr) {
      Entry e{};
      if (cudaEventCreateWithFlags(&e.event, cudaEventDisableTiming) != cudaSuccess) {
        mu_.unlock();
        throw HkvError{HKV_ERR_CUDA, "cudaEventCreateWithFlags failed in the group lock"};
      }
      entries_.push_back(e);
      slot = &entries_.back();
    }
    slot->stream = stream;
    slot->group = g;
    slot->pending = true;
    cudaEventRecord(slot->event, stream);
    mu_.unlock();
  }

  void abandon() { mu_.unlock(); }

 private:
  struct Entry {
    cudaEvent_t event;
    cudaStream_t stream;
    Group group;
    bool pending;
  };
  std::mutex mu_;
  std::vector<Entry> entries_;
};

}  // namespace

struct hkv_table {
  hkv_options opt{};
  hkv::TableView view{};
  hkv_allocator alloc{};
  bool own_allocator = true;
  std::atomic<uint64_t> global_epoch{hkv::kIgnoredEpoch};
  // counters for size / count overloads: an allocation of their own, so that a
  // doubling of the table in the middle of a call does not move them.  Readers
  // on different streams overlap, so every call that returns a count leases a
  // counter of its own (CounterLease) until its stream has been synchronised.
  unsigned long long* d_scratch = nullptr;
  std::mutex counter_mu;
  std::condition_variable counter_cv;
  uint64_t counter_free = ~0ull;  // bit k set: counter k is free
  StreamGroupLock lock;
  // Scratch the operations reuse instead of allocating per call: [0] the
  // deferred-key list of batches that may repeat keys and the sort buffers of
  // the hybrid find, [1] and [2] widened copies of 32-bit score arrays, [3]
  // the request chains of the routed updates (kept in its all-empty state
  // between calls, so it has a workspace of its own).
  struct Workspace {
    std::mutex mu;
    void* ptr = nullptr;
    size_t bytes = 0;
    cudaStream_t stream = nullptr;   // stream of the last user
    cudaEvent_t done = nullptr;      // end of the last user's work
    bool used = false;
  } workspace[4];
  // shape of the last routed update: another shape lays the scratch out anew
  uint32_t routed_world = 0;
  uint64_t routed_segment_capacity = 0;
  int device = 0;
  void* meta_block = nullptr;  // digests + slot lines (keys, scores) + sizes + status
  void* host_rows = nullptr;   // host address of the pinned value rows
  // reserve() and the automatic growth of the insert-like calls stop once the
  // capacity cannot double below max_capacity
  // (reach_max_capacity_, include/merlin_hashtable.cuh:1064, 3508-3538)
  std::atomic<bool> reach_max_capacity{true};
  // hkv_find_host: two sets of device staging buffers and the two streams that
  // alternate over the chunks of a host-resident batch; created on first use
  struct HostStage {
    std::mutex mu;
    cudaStream_t stream[2] = {nullptr, nullptr};
    cudaEvent_t done[2] = {nullptr, nullptr};
    cudaEvent_t start = nullptr;
    uint64_t chunk = 0;        // keys per chunk
    uint8_t* block = nullptr;  // one allocation, carved below
    uint64_t* keys[2] = {nullptr, nullptr};
    uint8_t* rows[2] = {nullptr, nullptr};
    uint64_t* scores[2] = {nullptr, nullptr};
    bool* founds[2] = {nullptr, nullptr};
  } stage;
};

namespace {

int default_alloc(void*, int type, void** ptr, size_t size, unsigned int flags) {
  switch (type) {
    case HKV_MEM_DEVICE: return cudaMalloc(ptr, size);
    case HKV_MEM_PINNED: return cudaHostAlloc(ptr, size, flags);
    default:
      *ptr = std::malloc(size);
      return *ptr ? 0 : int(cudaErrorMemoryAllocation);
  }
}

int default_free(void*, int type, void* ptr) {
  switch (type) {
    case HKV_MEM_DEVICE: return cudaFree(ptr);
    case HKV_MEM_PINNED: return cudaFreeHost(ptr);
    default: std::free(ptr); return 0;
  }
}

struct DeviceGuard {
  int prev = -1;
  explicit DeviceGuard(int dev) {
    cudaGetDevice(&prev);
    if (prev != dev) cudaSetDevice(dev);
    else prev = -1;
  }
  ~DeviceGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

// One of the table's 64 device counters, held by one call from its memset to
// the end of the stream synchronisation that reads it back.  A 65th concurrent
// call waits for a counter to come back.
constexpr int kCounters = 64;
class CounterLease {
 public:
  explicit CounterLease(hkv_table* t) : t_(t) {
    std::unique_lock<std::mutex> hold(t->counter_mu);
    t->counter_cv.wait(hold, [&] { return t->counter_free != 0; });
    index_ = __builtin_ctzll(t->counter_free);
    t->counter_free &= ~(1ull << index_);
  }
  CounterLease(const CounterLease&) = delete;
  CounterLease& operator=(const CounterLease&) = delete;
  ~CounterLease() {
    {
      std::lock_guard<std::mutex> hold(t_->counter_mu);
      t_->counter_free |= 1ull << index_;
    }
    t_->counter_cv.notify_one();
  }
  unsigned long long* get() const { return t_->d_scratch + index_; }

 private:
  hkv_table* t_;
  int index_;
};

// Scratch memory for the work one call enqueues on `stream`.  The table's
// workspace serves it when the previous user ran on the same stream (stream
// order protects the memory) or has finished; it grows on demand and is never
// returned before the table is destroyed.  A call that finds the workspace
// busy on another stream (concurrent readers) gets a stream-ordered allocation
// of its own instead.  The host mutex is held while the call enqueues.
class WorkspaceLease {
 public:
  WorkspaceLease(hkv_table* t, int which, size_t bytes, cudaStream_t stream)
      : t_(t), ws_(t->workspace[which]), stream_(stream) {
    if (bytes == 0) return;
    ws_.mu.lock();
    locked_ = true;
    const bool busy_elsewhere =
        ws_.used && ws_.stream != stream && cudaEventQuery(ws_.done) != cudaSuccess;
    if (busy_elsewhere) {
      ws_.mu.unlock();
      locked_ = false;
      if (cudaMallocAsync(&own_, bytes, stream) != cudaSuccess) {
        cudaGetLastError();
        own_ = nullptr;   // the caller falls back to its scratch-free form
      }
      fresh_ = true;
      return;
    }
    if (bytes > ws_.bytes) {
      if (ws_.ptr != nullptr) {
        if (ws_.used) cudaEventSynchronize(ws_.done);
        t->alloc.free(t->alloc.ctx, HKV_MEM_DEVICE, ws_.ptr);
        ws_.ptr = nullptr;
        ws_.bytes = 0;
      }
      const size_t want = bytes + bytes / 2 + 4096;
      void* p = nullptr;
      if (t->alloc.alloc(t->alloc.ctx, HKV_MEM_DEVICE, &p, want, 0) != 0 || p == nullptr) {
        cudaGetLastError();
        ws_.mu.unlock();
        locked_ = false;
        return;
      }
      ws_.ptr = p;
      ws_.bytes = want;
      fresh_ = true;
    }
    if (ws_.done == nullptr &&
        cudaEventCreateWithFlags(&ws_.done, cudaEventDisableTiming) != cudaSuccess) {
      cudaGetLastError();
      ws_.mu.unlock();
      locked_ = false;
      return;
    }
    shared_ = ws_.ptr;
  }
  WorkspaceLease(const WorkspaceLease&) = delete;
  WorkspaceLease& operator=(const WorkspaceLease&) = delete;
  ~WorkspaceLease() {
    if (own_ != nullptr) cudaFreeAsync(own_, stream_);
    if (locked_) {
      if (shared_ != nullptr) {
        ws_.stream = stream_;
        ws_.used = true;
        cudaEventRecord(ws_.done, stream_);
      }
      ws_.mu.unlock();
    }
  }
  void* get() const { return own_ != nullptr ? own_ : shared_; }
  // the memory was obtained by this lease: nothing an earlier call left is in it
  bool fresh() const { return fresh_; }

 private:
  hkv_table* t_;
  hkv_table::Workspace& ws_;
  bool fresh_ = false;
  cudaStream_t stream_;
  void* own_ = nullptr;
  void* shared_ = nullptr;
  bool locked_ = false;
};

struct LockScope {
  hkv_table* t;
  Group g;
  cudaStream_t s;
  bool held;
  LockScope(hkv_table* table, Group group, cudaStream_t stream)
      : t(table), g(group), s(stream), held(table->opt.api_lock != 0) {
    if (held) t->lock.acquire(g, s);
  }
  // Called after the kernels were enqueued.
  void done() {
    if (held) {
      held = false;
      t->lock.release(g, s);
    }
  }
  ~LockScope() {
    if (held) t->lock.abandon();
  }
};

template <class F>
int guarded(F&& f) {
  try {
    f();
    return HKV_OK;
  } catch (const HkvError& e) {
    g_last_error = e.msg;
    return e.code;
  } catch (const std::bad_alloc&) {
    g_last_error = "out of host memory";
    return HKV_ERR_RUNTIME;
  } catch (const std::exception& e) {
    g_last_error = e.what();
    return HKV_ERR_RUNTIME;
  }
}

void check_launch() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    throw HkvError{HKV_ERR_CUDA, std::string("kernel launch: ") + cudaGetErrorString(e)};
  }
}

uint32_t widest_vec(uint64_t row_bytes) {
  for (uint32_t v = 16; v > 1; v >>= 1) {
    if (row_bytes % v == 0) return v;
  }
  return 1;
}

// View whose row access width also respects the alignment of the caller's
// batch buffers.
hkv::TableView view_for(const hkv_table* t, const void* a, const void* b = nullptr) {
  hkv::TableView v = t->view;
  uint32_t vec = v.vec_bytes;
  auto lower = [&](const void* p) {
    if (p == nullptr) return;
    while (vec > 1 && (reinterpret_cast<uintptr_t>(p) % vec) != 0) vec >>= 1;
  };
  lower(a);
  lower(b);
  if (vec != v.vec_bytes) {
    v.vec_bytes = vec;
    v.chunks_per_row = v.row_bytes / vec;
    int shift = -1;
    if ((v.chunks_per_row & (v.chunks_per_row - 1)) == 0) {
      shift = 0;
      while ((1u << shift) < v.chunks_per_row) ++shift;
    }
    v.chunks_per_row_shift = shift;
    v.chunks_per_row_magic = hkv::chunks_per_row_magic_of(v.chunks_per_row);
  }
  return v;
}

// sizeof(S) == 4 (only with kCustomized, include/merlin_hashtable.cuh:939-949
// of the reference): the caller's score arrays hold uint32 while the kernels
// work on uint64.  An array is widened into a stream-ordered temporary before
// the kernels run; an output array is narrowed back afterwards (it was widened
// first so that entries the kernels leave alone keep their value).  With
// 64-bit scores this is the caller's pointer and nothing else.
class Scores {
 public:
  // `which`: the workspace the widened copy lives in (1, or 2 for a call's
  // second score array)
  Scores(hkv_table* t, const uint64_t* user, uint64_t n, hkv_stream stream, bool is_output,
         int which = 1)
      : user_(const_cast<uint64_t*>(user)),
        n_(n),
        stream_(static_cast<cudaStream_t>(stream)),
        output_(is_output),
        exceptions_(std::uncaught_exceptions()),
        guard_(t->device),
        lease_(t, which, (user == nullptr || n == 0 || t->opt.score_size == 8) ? 0 : n * sizeof(uint64_t),
               static_cast<cudaStream_t>(stream)) {
    if (user == nullptr || n == 0 || t->opt.score_size == 8) return;
    wide_ = static_cast<uint64_t*>(lease_.get());
    if (wide_ == nullptr) {
      throw HkvError{HKV_ERR_CUDA, "out of device memory for the widened score array"};
    }
    hkv::launch_widen_scores(reinterpret_cast<const uint32_t*>(user), wide_, n, stream_);
  }
  Scores(const Scores&) = delete;
  Scores& operator=(const Scores&) = delete;
  ~Scores() {
    if (wide_ == nullptr) return;
    if (output_ && std::uncaught_exceptions() == exceptions_) {
      hkv::launch_narrow_scores(wide_, reinterpret_cast<uint32_t*>(user_), n_, stream_);
    }
  }
  uint64_t* get() const { return wide_ != nullptr ? wide_ : user_; }

 private:
  uint64_t* user_;
  uint64_t* wide_ = nullptr;
  uint64_t n_;
  cudaStream_t stream_;
  bool output_;
  int exceptions_;
  DeviceGuard guard_;      // the lease allocates on the table's device
  WorkspaceLease lease_;   // released after the narrowing pass was enqueued
};

// Dual-bucket tables serve insert_or_assign and find and the whole-table scans;
// everything else that addresses a bucket by key is refused, in the reference's
// words where it has some (include/merlin_hashtable.cuh:1361, 1596, 1704, 2232, 2303, 2859,
// 2905, 3504).
void refuse_in_memory_mode(const hkv_table* t, const char* what) {
  if (t->opt.table_mode == 1) {
    throw HkvError{HKV_ERR_MERLIN, std::string("[MEMORY_MODE] ") + what +
                                       "() is not supported in dual-bucket mode."};
  }
}

// accum_or_assign adds elements of V (include/merlin/core_kernels/accum_or_assign.cuh:139-172):
// the element type must be known and a row chunk must hold whole elements.
void check_accum_type(const hkv_table* t, const void* batch) {
  static const uint32_t size_of_kind[] = {4, 4, 8, 4, 8, 2, 2};
  const uint32_t kind = t->view.value_kind;
  HKV_CHECK(kind <= hkv::kValueBF16 && t->opt.value_size == size_of_kind[kind],
            "accum_or_assign needs a float32, float64, int32, int64, float16 or bfloat16 value type "
            "(hkv_options.value_kind).");
  HKV_CHECK(view_for(t, batch).vec_bytes >= t->opt.value_size,
            "accum_or_assign needs value_or_deltas aligned to the element size.");
}

// check_evict_strategy, include/merlin_hashtable.cuh:3832-3861
void check_strategy(const hkv_table* t, int strategy, const uint64_t* scores) {
  if (strategy == HKV_LRU || strategy == HKV_EPOCH_LRU) {
    HKV_CHECK(scores == nullptr,
              "the scores should not be specified when running on LRU or Epoch LRU mode.");
  }
  if (strategy == HKV_LFU || strategy == HKV_EPOCH_LFU) {
    HKV_CHECK(scores != nullptr,
              "the scores should be specified when running on LFU or Epoch LFU mode.");
  }
  if (strategy == HKV_CUSTOMIZED) {
    HKV_CHECK(scores != nullptr, "the scores should be specified when running on customized mode.");
  }
  if (strategy == HKV_EPOCH_LRU || strategy == HKV_EPOCH_LFU) {
    HKV_CHECK(t->global_epoch.load() != hkv::kIgnoredEpoch,
              "the global_epoch is invalid and should be assigned by calling `set_global_epoch` "
              "when running on Epoch LRU or Epoch LFU mode.");
  }
}

hkv::MutateArgs base_args(hkv_table* t, uint64_t n, const uint64_t* keys, const void* values,
                          const uint64_t* scores, bool ignore_strategy) {
  hkv::MutateArgs a;
  a.keys = keys;
  a.n = n;
  a.values = static_cast<uint8_t*>(const_cast<void*>(values));
  a.scores = scores;
  // ignore_evict_strategy re-dispatches as kCustomized with the epoch ignored
  // (include/merlin_hashtable.cuh:1131-1133)
  a.strategy = ignore_strategy ? int(HKV_CUSTOMIZED) : t->opt.evict_strategy;
  a.epoch = t->global_epoch.load();
  return a;
}

// The planes of one table size: a metadata block (digests | slot lines of keys
// and scores | bucket sizes | status) and the value rows, whole buckets in HBM while
// max_hbm_for_vectors lasts and the rest in mapped pinned host memory (a static
// split by bucket index, as include/merlin/core_kernels.cuh:204-232 does per
// slice).
struct Planes {
  void* meta_block = nullptr;
  void* values_hbm = nullptr;
  void* host_rows = nullptr;
};

void free_planes(hkv_table* t, Planes& p) {
  if (p.meta_block) t->alloc.free(t->alloc.ctx, HKV_MEM_DEVICE, p.meta_block);
  if (p.values_hbm) t->alloc.free(t->alloc.ctx, HKV_MEM_DEVICE, p.values_hbm);
  if (p.host_rows) t->alloc.free(t->alloc.ctx, HKV_MEM_PINNED, p.host_rows);
  p = Planes{};
}

// Fills the size-dependent fields of `v` (the others are taken as they are)
// and clears the new table on `stream`.
void allocate_planes(hkv_table* t, uint64_t buckets, hkv::TableView& v, Planes& p,
                     cudaStream_t stream) {
  const uint64_t capacity = buckets * v.bucket_slots;
  HKV_CHECK(capacity <= (1ull << 31), "capacity above 2^31 slots is not supported.");
  const uint64_t row_bytes = v.row_bytes;
  v.buckets = buckets;
  v.capacity = capacity;
  v.capacity_pow2 = (capacity & (capacity - 1)) == 0 ? 1u : 0u;
  try {
    auto align256 = [](uint64_t x) { return (x + 255) & ~255ull; };
    const uint64_t off_digests = 0;
    const uint64_t off_lines = align256(off_digests + capacity);
    const uint64_t off_sizes = align256(off_lines + capacity * 16);
    const uint64_t off_status = align256(off_sizes + buckets * 4);
    uint64_t hbm_buckets = t->opt.max_hbm_for_vectors / (row_bytes * v.bucket_slots);
    if (hbm_buckets > buckets) hbm_buckets = buckets;
    // a table with rows on both sides gets a bucket map and hit counters
    const bool mapped = hbm_buckets > 0 && hbm_buckets < buckets;
    const uint64_t off_map = align256(off_status + 256);
    const uint64_t off_heat = align256(off_map + (mapped ? buckets * 4 : 0));
    const uint64_t meta_bytes = mapped ? align256(off_heat + buckets * 4) : off_status + 256;
    if (t->alloc.alloc(t->alloc.ctx, HKV_MEM_DEVICE, &p.meta_block, meta_bytes, 0) != 0 ||
        p.meta_block == nullptr) {
      cudaGetLastError();
      throw HkvError{HKV_ERR_CUDA, "device allocation of the table metadata failed"};
    }
    uint8_t* mb = static_cast<uint8_t*>(p.meta_block);
    v.digests = mb + off_digests;
    // keys | scores, or lines of 8 keys + 8 scores: the same 16 bytes per slot
    v.key_words = reinterpret_cast<uint64_t*>(mb + off_lines);
    v.score_words = v.line_mask ? v.key_words + hkv::kLineSlots : v.key_words + capacity;
    v.bucket_sizes = reinterpret_cast<int32_t*>(mb + off_sizes);
    v.status = reinterpret_cast<uint32_t*>(mb + off_status);
    HKV_CUDA(cudaMemsetAsync(mb + off_status, 0, 256, stream));
    v.bucket_map = mapped ? reinterpret_cast<uint32_t*>(mb + off_map) : nullptr;
    v.bucket_heat = mapped ? reinterpret_cast<uint32_t*>(mb + off_heat) : nullptr;

    v.hbm_slots = hbm_buckets * v.bucket_slots;
    v.values_hbm = nullptr;
    v.values_host = nullptr;
    if (v.hbm_slots > 0) {
      if (t->alloc.alloc(t->alloc.ctx, HKV_MEM_DEVICE, &p.values_hbm, v.hbm_slots * row_bytes,
                         0) != 0 ||
          p.values_hbm == nullptr) {
        cudaGetLastError();
        throw HkvError{HKV_ERR_CUDA, "device allocation of the value rows failed"};
      }
      v.values_hbm = static_cast<uint8_t*>(p.values_hbm);
    }
    if (v.hbm_slots < capacity) {
      const uint64_t bytes = (capacity - v.hbm_slots) * row_bytes;
      if (t->alloc.alloc(t->alloc.ctx, HKV_MEM_PINNED, &p.host_rows, bytes,
                         cudaHostAllocMapped | cudaHostAllocPortable) != 0 ||
          p.host_rows == nullptr) {
        cudaGetLastError();
        throw HkvError{HKV_ERR_CUDA, "pinned host allocation of the value rows failed"};
      }
      void* dp = nullptr;
      HKV_CUDA(cudaHostGetDevicePointer(&dp, p.host_rows, 0));
      v.values_host = static_cast<uint8_t*>(dp);
    }
    hkv::launch_clear(v, stream);
    if (mapped) hkv::launch_identity_map(v, stream);
    check_launch();
  } catch (...) {
    free_planes(t, p);
    throw;
  }
}

// Hot buckets of a hybrid table move into HBM: the host-resident buckets with
// the most lookup hits since the last call trade row blocks with the coldest
// HBM-resident ones, as long as the bucket moving in was hit more than twice
// as often as the one moving out.  The
// choice is made on the host from the hit counters; the rows move in one kernel.
uint64_t promote_hot_buckets(hkv_table* t, cudaStream_t s) {
  const hkv::TableView& v = t->view;
  if (v.bucket_map == nullptr) return 0;
  LockScope ls(t, kInserter, s);
  const uint64_t buckets = v.buckets;
  const uint32_t hbm_blocks = static_cast<uint32_t>(v.hbm_slots / v.bucket_slots);
  std::vector<uint32_t> map(buckets), heat(buckets);
  HKV_CUDA(cudaMemcpyAsync(map.data(), v.bucket_map, buckets * 4, cudaMemcpyDeviceToHost, s));
  HKV_CUDA(cudaMemcpyAsync(heat.data(), v.bucket_heat, buckets * 4, cudaMemcpyDeviceToHost, s));
  HKV_CUDA(cudaStreamSynchronize(s));
  std::vector<uint32_t> in_hbm, in_host;
  for (uint64_t b = 0; b < buckets; ++b) {
    (map[b] < hbm_blocks ? in_hbm : in_host).push_back(static_cast<uint32_t>(b));
  }
  std::sort(in_hbm.begin(), in_hbm.end(),
            [&](uint32_t a, uint32_t b) { return heat[a] != heat[b] ? heat[a] < heat[b] : a < b; });
  std::sort(in_host.begin(), in_host.end(),
            [&](uint32_t a, uint32_t b) { return heat[a] != heat[b] ? heat[a] > heat[b] : a < b; });
  std::vector<uint32_t> pairs;
  for (size_t i = 0; i < in_hbm.size() && i < in_host.size(); ++i) {
    // a move costs two row blocks over the host link: it has to pay
    if (uint64_t(heat[in_host[i]]) < 2ull * heat[in_hbm[i]] + 8) break;
    pairs.push_back(in_host[i]);
    pairs.push_back(in_hbm[i]);
  }
  const uint64_t n_pairs = pairs.size() / 2;
  if (n_pairs > 0) {
    uint32_t* d_pairs = nullptr;
    HKV_CUDA(cudaMallocAsync(reinterpret_cast<void**>(&d_pairs), pairs.size() * 4, s));
    cudaMemcpyAsync(d_pairs, pairs.data(), pairs.size() * 4, cudaMemcpyHostToDevice, s);
    hkv::launch_swap_row_blocks(v, d_pairs, n_pairs, s);
    cudaFreeAsync(d_pairs, s);
    // `pairs` is pageable host memory: the copy above has been staged when it returns
  }
  hkv::launch_decay_heat(v, s);
  ls.done();
  check_launch();
  return n_pairs;
}

// fast_load_factor, include/merlin_hashtable.cuh:3796-3828: the load the table
// would have after `delta` more keys, estimated from the first 1024 buckets.
float fast_load_factor(hkv_table* t, uint64_t delta, cudaStream_t s) {
  CounterLease lease(t);
  unsigned long long* ctr = lease.get();
  uint64_t sampled = 0, capacity = 0;
  {
    LockScope ls(t, kReader, s);
    sampled = t->view.buckets < 1024 ? t->view.buckets : 1024;
    capacity = t->view.capacity;
    HKV_CUDA(cudaMemsetAsync(ctr, 0, sizeof(*ctr), s));
    hkv::launch_sum_sizes(t->view, sampled, ctr, s);
    ls.done();
  }
  check_launch();
  unsigned long long h = 0;
  HKV_CUDA(cudaMemcpyAsync(&h, ctr, sizeof(h), cudaMemcpyDeviceToHost, s));
  HKV_CUDA(cudaStreamSynchronize(s));
  return static_cast<float>((delta * 1.0) / (capacity * 1.0) +
                            (h * 1.0) / (t->view.bucket_slots * sampled * 1.0));
}

// reserve, include/merlin_hashtable.cuh:3503-3545.  Each doubling builds the
// planes of the larger table, moves the live entries over and frees the old
// planes: pointers into the table handed out earlier (find / find_or_insert
// pointer forms, lock_keys) are invalid afterwards, as in the reference.
void reserve(hkv_table* t, uint64_t new_capacity, cudaStream_t s) {
  if (t->reach_max_capacity.load() || new_capacity > t->opt.max_capacity) {
    t->reach_max_capacity.store(t->view.capacity * 2 > t->opt.max_capacity);
    return;
  }
  LockScope ls(t, kInserter, s);
  HKV_CUDA(cudaDeviceSynchronize());
  while (t->view.capacity < new_capacity && t->view.capacity * 2 <= t->opt.max_capacity) {
    hkv::TableView grown = t->view;
    Planes fresh;
    allocate_planes(t, t->view.buckets * 2, grown, fresh, s);
    hkv::launch_rehash(t->view, grown, s);
    // the status word moves with the table
    cudaMemcpyAsync(grown.status, t->view.status, 64, cudaMemcpyDeviceToDevice, s);
    if (cudaStreamSynchronize(s) != cudaSuccess || cudaGetLastError() != cudaSuccess) {
      free_planes(t, fresh);
      throw HkvError{HKV_ERR_CUDA, "rehash into the doubled table failed"};
    }
    Planes old;
    old.meta_block = t->meta_block;
    old.values_hbm = t->view.values_hbm;
    old.host_rows = t->host_rows;
    t->view = grown;
    t->meta_block = fresh.meta_block;
    t->host_rows = fresh.host_rows;
    free_planes(t, old);
  }
  t->reach_max_capacity.store(t->view.capacity * 2 > t->opt.max_capacity);
  ls.done();
  check_launch();
}

// `batch_a` / `batch_b` are the caller's row buffers; their alignment bounds
// the row access width of the view the kernel gets.
void mutate(hkv_table* t, int op, hkv::MutateArgs& args, const void* batch_a, const void* batch_b,
            Group g, bool unique_key, cudaStream_t stream) {
  DeviceGuard dg(t->device);
  if (op <= hkv::kOpAccumOrAssign) {
    // the insert-like calls grow the table first
    // (include/merlin_hashtable.cuh:1151-1154, 1369-1372, 1604-1607, 1712-1715, 1898-1901)
    while (!t->reach_max_capacity.load() &&
           fast_load_factor(t, args.n, stream) > t->opt.max_load_factor) {
      reserve(t, t->view.capacity * 2, stream);
    }
  }
  WorkspaceLease work(t, 0, hkv::mutate_workspace_bytes(op, args.n, unique_key), stream);
  LockScope ls(t, g, stream);
  hkv::launch_mutate(op, view_for(t, batch_a, batch_b), args, unique_key, stream, work.get());
  ls.done();
  check_launch();
}

}  // namespace

extern "C" {

const char* hkv_last_error(void) { return g_last_error.c_str(); }

int hkv_table_create(const hkv_options* options, const hkv_allocator* allocator, hkv_table** out) {
  return guarded([&] {
    if (options == nullptr || out == nullptr) {
      throw HkvError{HKV_ERR_INVALID_ARG, "options and out must not be null"};
    }
    const hkv_options& o = *options;
    HKV_CHECK(o.table_mode == 0 || o.table_mode == 1, "options.table_mode should be 0 or 1.");
    if (o.table_mode == 1) {
      // include/merlin_hashtable.cuh:991-1015
      HKV_CHECK(o.init_capacity == o.max_capacity,
                "[MEMORY_MODE] init_capacity must equal max_capacity. Auto-rehash is not "
                "supported in dual-bucket mode.");
      HKV_CHECK(o.max_hbm_for_vectors == 0,
                "[MEMORY_MODE] Only pure HBM (fast mode) is supported. Set max_hbm_for_vectors = 0.");
      HKV_CHECK(o.dim * uint64_t(o.value_size) <= 224 * sizeof(float),
                "[MEMORY_MODE] dim * sizeof(V) must not exceed 896 bytes (i.e. dim <= 224 for "
                "float).");
      HKV_CHECK(o.max_bucket_size != 0 && o.init_capacity / o.max_bucket_size >= 2,
                "[MEMORY_MODE] capacity must provide at least 2 buckets (capacity >= 2 * "
                "max_bucket_size).");
    }
    HKV_CHECK(o.reserved_key_start_bit >= 0 && o.reserved_key_start_bit <= 62,
              "options.reserved_key_start_bit should >= 0 and <= 62.");
    HKV_CHECK(o.max_bucket_size != 0 && (o.max_bucket_size & (o.max_bucket_size - 1)) == 0,
              "Bucket size should be the pow of 2");
    // the reference takes any power of two whose key and score lines are
    // 128-byte aligned (include/merlin_hashtable.cuh:1032-1048); here a bucket
    // holds 16 to 1024 slots, and dual-bucket tables keep the default 128
    HKV_CHECK(o.max_bucket_size >= 16 && o.max_bucket_size <= hkv::kMaxBucketSlots,
              "max_bucket_size should be a power of two between 16 and 1024.");
    HKV_CHECK(o.table_mode == 0 || o.max_bucket_size == uint64_t(hkv::kBucketSlots),
              "[MEMORY_MODE] dual-bucket tables need max_bucket_size == 128.");
    HKV_CHECK(o.num_of_buckets_per_alloc != 0 &&
                  (o.num_of_buckets_per_alloc & (o.num_of_buckets_per_alloc - 1)) == 0,
              "Then `num_of_buckets_per_alloc` should be the pow of 2");
    HKV_CHECK(o.init_capacity >= o.num_of_buckets_per_alloc * o.max_bucket_size,
              "Then `num_of_buckets_per_alloc` must be equal or less than initial required "
              "buckets number");
    HKV_CHECK(!(o.io_by_cpu && o.max_hbm_for_vectors != 0),
              "[HierarchicalKV] `io_by_cpu` should not be true when `max_hbm_for_vectors` is "
              "not 0!");
    HKV_CHECK(!o.io_by_cpu, "`io_by_cpu` is not part of this library.");
    HKV_CHECK(o.score_size == 8 || o.score_size == 4, "The score_type must be uint64_t or uint32_t.");
    HKV_CHECK(o.score_size == 8 || o.evict_strategy == HKV_CUSTOMIZED,
              "score_type uint32_t is only compatible with Customized; use uint64_t.");
    HKV_CHECK(o.evict_strategy >= HKV_LRU && o.evict_strategy <= HKV_CUSTOMIZED,
              "unknown evict strategy");
    HKV_CHECK(o.dim > 0 && o.value_size > 0, "dim and value_size must be positive");
    HKV_CHECK(o.slot_layout == HKV_SLOT_PLANES || o.slot_layout == HKV_SLOT_LINES,
              "hkv_options.slot_layout should be HKV_SLOT_PLANES or HKV_SLOT_LINES.");

    auto* t = new hkv_table();
    try {
      t->opt = o;
      if (allocator != nullptr) {
        t->alloc = *allocator;
        t->own_allocator = false;
      } else {
        t->alloc = hkv_allocator{nullptr, default_alloc, default_free};
      }
      if (o.device_id >= 0) {
        HKV_CUDA(cudaSetDevice(o.device_id));
        t->device = o.device_id;
      } else {
        HKV_CUDA(cudaGetDevice(&t->device));
        t->opt.device_id = t->device;
      }

      // create_table, include/merlin/core_kernels.cuh:336-356
      const uint64_t max_size = o.init_capacity > o.max_capacity ? o.init_capacity : o.max_capacity;
      uint64_t buckets;
      if (o.init_capacity * 2 > max_size) {
        buckets = 1 + (max_size - 1) / o.max_bucket_size;
      } else {
        buckets = 1;
        while (buckets * o.max_bucket_size < o.init_capacity) buckets *= 2;
      }
      const uint64_t row_bytes = o.dim * uint64_t(o.value_size);
      HKV_CHECK(row_bytes < (1ull << 24), "value rows above 16 MiB are not supported.");
      t->reach_max_capacity.store(o.init_capacity * 2 > o.max_capacity || o.table_mode == 1);

      hkv::TableView& v = t->view;
      v.line_mask = o.slot_layout == HKV_SLOT_LINES ? ~uint64_t(0) : 0;
      v.bucket_slots = uint32_t(o.max_bucket_size);
      v.bucket_shift = 0;
      while ((1u << v.bucket_shift) < v.bucket_slots) ++v.bucket_shift;
      v.row_bytes = uint32_t(row_bytes);
      v.vec_bytes = widest_vec(row_bytes);
      v.chunks_per_row = uint32_t(row_bytes / v.vec_bytes);
      v.chunks_per_row_shift = -1;
      if ((v.chunks_per_row & (v.chunks_per_row - 1)) == 0) {
        int s = 0;
        while ((1u << s) < v.chunks_per_row) ++s;
        v.chunks_per_row_shift = s;
      }
      v.chunks_per_row_magic = hkv::chunks_per_row_magic_of(v.chunks_per_row);
      HKV_CHECK(o.value_kind <= hkv::kValueBF16, "hkv_options.value_kind out of range.");
      v.value_kind = o.value_kind;
      // reserved keys, include/merlin/types.cuh:80-109
      const int bit = o.reserved_key_start_bit;
      if (bit == 0) {
        v.empty_key = 0xFFFFFFFFFFFFFFFFull;
        v.reclaim_key = 0xFFFFFFFFFFFFFFFEull;
        v.locked_key = 0xFFFFFFFFFFFFFFFDull;
        v.reserved_mask = 0xFFFFFFFFFFFFFFFCull;
        v.reserved_value = 0xFFFFFFFFFFFFFFFCull;
      } else {
        const uint64_t m1 = ~(3ull << bit);
        const uint64_t m2 = m1 & ~1ull;
        v.reserved_mask = m1;
        v.reserved_value = m2;
        v.empty_key = m2 | (3ull << bit);
        v.reclaim_key = (~(1ull << bit)) & ~1ull;
        v.locked_key = v.empty_key & ~(2ull << bit);
      }
      // digest byte: bits 32-39 of the hash, bits 56-63 on a dual-bucket table
      // (include/merlin/core_kernels/dual_bucket_utils.cuh:47-65)
      const int digest_shift = o.table_mode == 1 ? 56 : 32;
      const uint32_t ed = uint32_t(hkv::fmix64(v.empty_key) >> digest_shift) & 0xFFu;
      v.empty_digest4 = ed * 0x01010101u;
      v.reclaim_digest = uint32_t(hkv::fmix64(v.reclaim_key) >> digest_shift) & 0xFFu;

      Planes planes;
      allocate_planes(t, buckets, v, planes, nullptr);
      t->meta_block = planes.meta_block;
      t->host_rows = planes.host_rows;
      void* scratch = nullptr;
      if (t->alloc.alloc(t->alloc.ctx, HKV_MEM_DEVICE, &scratch, kCounters * 8, 0) != 0 ||
          scratch == nullptr) {
        cudaGetLastError();
        throw HkvError{HKV_ERR_CUDA, "device allocation of the counters failed"};
      }
      t->d_scratch = static_cast<unsigned long long*>(scratch);
      HKV_CUDA(cudaMemset(scratch, 0, kCounters * 8));
      HKV_CUDA(cudaDeviceSynchronize());
    } catch (...) {
      hkv_table_destroy(t);
      throw;
    }
    *out = t;
  });
}

int hkv_table_destroy(hkv_table* t) {
  if (t == nullptr) return HKV_OK;
  return guarded([&] {
    DeviceGuard dg(t->device);
    cudaDeviceSynchronize();
    if (t->meta_block) t->alloc.free(t->alloc.ctx, HKV_MEM_DEVICE, t->meta_block);
    if (t->d_scratch) t->alloc.free(t->alloc.ctx, HKV_MEM_DEVICE, t->d_scratch);
    if (t->view.values_hbm) t->alloc.free(t->alloc.ctx, HKV_MEM_DEVICE, t->view.values_hbm);
    if (t->host_rows) t->alloc.free(t->alloc.ctx, HKV_MEM_PINNED, t->host_rows);
    if (t->stage.block) t->alloc.free(t->alloc.ctx, HKV_MEM_DEVICE, t->stage.block);
    for (auto& w : t->workspace) {
      if (w.ptr) t->alloc.free(t->alloc.ctx, HKV_MEM_DEVICE, w.ptr);
      if (w.done) cudaEventDestroy(w.done);
    }
    for (int i = 0; i < 2; ++i) {
      if (t->stage.stream[i]) cudaStreamDestroy(t->stage.stream[i]);
      if (t->stage.done[i]) cudaEventDestroy(t->stage.done[i]);
    }
    if (t->stage.start) cudaEventDestroy(t->stage.start);
    delete t;
  });
}

int hkv_insert_or_assign(hkv_table* t, uint64_t n, const uint64_t* keys, const void* values,
                         const uint64_t* scores, hkv_stream stream, int unique_key,
                         int ignore_evict_strategy) {
  return guarded([&] {
    if (n == 0) return;
    Scores scores_w(t, scores, n, stream, false);
    if (!ignore_evict_strategy) check_strategy(t, t->opt.evict_strategy, scores);
    hkv::MutateArgs a = base_args(t, n, keys, values, scores_w.get(), ignore_evict_strategy != 0);
    if (ignore_evict_strategy) a.epoch = hkv::kIgnoredEpoch;
    if (t->opt.table_mode == 1) {
      // include/merlin_hashtable.cuh:1165-1170
      HKV_CHECK(unique_key != 0,
                "[MEMORY_MODE] insert_or_assign requires unique_key=true in dual-bucket mode.");
      DeviceGuard dg(t->device);
      cudaStream_t s = static_cast<cudaStream_t>(stream);
      LockScope ls(t, kInserter, s);
      hkv::launch_dual_upsert(t->view, a, s);
      ls.done();
      check_launch();
      return;
    }
    mutate(t, hkv::kOpInsertOrAssign, a, values, nullptr, kInserter, unique_key != 0,
           static_cast<cudaStream_t>(stream));
  });
}

int hkv_insert_and_evict(hkv_table* t, uint64_t n, const uint64_t* keys, const void* values,
                         const uint64_t* scores, uint64_t* evicted_keys, void* evicted_values,
                         uint64_t* evicted_scores, uint64_t* d_evicted_counter, hkv_stream stream,
                         int unique_key, int ignore_evict_strategy) {
  return guarded([&] {
    refuse_in_memory_mode(t, "insert_and_evict");
    if (n == 0) return;
    Scores scores_w(t, scores, n, stream, false);
    Scores evicted_scores_w(t, evicted_scores, n, stream, true, 2);
    if (t->view.hbm_slots < t->view.capacity) {
      // include/merlin_hashtable.cuh:1384-1386
      throw HkvError{HKV_ERR_RUNTIME, "Only allow insert_and_evict in pure HBM mode."};
    }
    if (!ignore_evict_strategy) check_strategy(t, t->opt.evict_strategy, scores);
    hkv::MutateArgs a = base_args(t, n, keys, values, scores_w.get(), ignore_evict_strategy != 0);
    if (ignore_evict_strategy) a.epoch = hkv::kIgnoredEpoch;
    a.evicted_keys = evicted_keys;
    a.evicted_values = static_cast<uint8_t*>(evicted_values);
    a.evicted_scores = evicted_scores_w.get();
    a.evicted_counter = reinterpret_cast<unsigned long long*>(d_evicted_counter);
    mutate(t, hkv::kOpInsertAndEvict, a, values, evicted_values, kInserter,
           unique_key != 0, static_cast<cudaStream_t>(stream));
  });
}

int hkv_insert_and_evict_count(hkv_table* t, uint64_t n, const uint64_t* keys, const void* values,
                               const uint64_t* scores, uint64_t* evicted_keys,
                               void* evicted_values, uint64_t* evicted_scores, hkv_stream stream,
                               int unique_key, int ignore_evict_strategy,
                               uint64_t* evicted_count) {
  return guarded([&] {
    *evicted_count = 0;
    if (n == 0) return;
    DeviceGuard dg(t->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    CounterLease lease(t);
    unsigned long long* ctr = lease.get();
    HKV_CUDA(cudaMemsetAsync(ctr, 0, sizeof(*ctr), s));
    int rc = hkv_insert_and_evict(t, n, keys, values, scores, evicted_keys, evicted_values,
                                  evicted_scores, reinterpret_cast<uint64_t*>(ctr), stream,
                                  unique_key, ignore_evict_strategy);
    if (rc != HKV_OK) throw HkvError{rc, g_last_error};
    unsigned long long h = 0;
    HKV_CUDA(cudaMemcpyAsync(&h, ctr, sizeof(h), cudaMemcpyDeviceToHost, s));
    HKV_CUDA(cudaStreamSynchronize(s));
    *evicted_count = h;
  });
}

int hkv_accum_or_assign(hkv_table* t, uint64_t n, const uint64_t* keys,
                        const void* value_or_deltas, const bool* accum_or_assigns,
                        const uint64_t* scores, hkv_stream stream, int ignore_evict_strategy) {
  return guarded([&] {
    refuse_in_memory_mode(t, "accum_or_assign");
    if (n == 0) return;
    Scores scores_w(t, scores, n, stream, false);
    check_accum_type(t, value_or_deltas);
    if (!ignore_evict_strategy) check_strategy(t, t->opt.evict_strategy, scores);
    hkv::MutateArgs a = base_args(t, n, keys, value_or_deltas, scores_w.get(), ignore_evict_strategy != 0);
    if (ignore_evict_strategy) a.epoch = hkv::kIgnoredEpoch;
    a.accum_flags = accum_or_assigns;
    // the reference has no unique_key argument here and always runs its
    // duplicate-tolerant tile kernel (include/merlin_hashtable.cuh:1618-1631)
    mutate(t, hkv::kOpAccumOrAssign, a, value_or_deltas, nullptr, kInserter, false,
           static_cast<cudaStream_t>(stream));
  });
}

int hkv_accum_or_assign_unique(hkv_table* t, uint64_t n, const uint64_t* keys,
                               const void* value_or_deltas, const bool* accum_or_assigns,
                               const uint64_t* scores, hkv_stream stream,
                               int ignore_evict_strategy) {
  return guarded([&] {
    refuse_in_memory_mode(t, "accum_or_assign");
    if (n == 0) return;
    Scores scores_w(t, scores, n, stream, false);
    check_accum_type(t, value_or_deltas);
    if (!ignore_evict_strategy) check_strategy(t, t->opt.evict_strategy, scores);
    hkv::MutateArgs a = base_args(t, n, keys, value_or_deltas, scores_w.get(), ignore_evict_strategy != 0);
    if (ignore_evict_strategy) a.epoch = hkv::kIgnoredEpoch;
    a.accum_flags = accum_or_assigns;
    mutate(t, hkv::kOpAccumOrAssign, a, value_or_deltas, nullptr, kInserter, true,
           static_cast<cudaStream_t>(stream));
  });
}

int hkv_find_or_insert(hkv_table* t, uint64_t n, const uint64_t* keys, void* values,
                       uint64_t* scores, hkv_stream stream, int unique_key,
                       int ignore_evict_strategy) {
  return guarded([&] {
    refuse_in_memory_mode(t, "find_or_insert");
    if (n == 0) return;
    Scores scores_w(t, scores, n, stream, false);
    if (!ignore_evict_strategy) check_strategy(t, t->opt.evict_strategy, scores);
    hkv::MutateArgs a = base_args(t, n, keys, values, scores_w.get(), ignore_evict_strategy != 0);
    if (ignore_evict_strategy) a.epoch = hkv::kIgnoredEpoch;
    mutate(t, hkv::kOpFindOrInsert, a, values, nullptr, kInserter, unique_key != 0,
           static_cast<cudaStream_t>(stream));
  });
}

int hkv_find_or_insert_ptr(hkv_table* t, uint64_t n, const uint64_t* keys, void** values,
                           bool* founds, uint64_t* scores, hkv_stream stream, int unique_key,
                           int ignore_evict_strategy, uint64_t** locked_key_ptrs) {
  return guarded([&] {
    refuse_in_memory_mode(t, "find_or_insert");
    if (n == 0) return;
    Scores scores_w(t, scores, n, stream, false);
    if (!ignore_evict_strategy) check_strategy(t, t->opt.evict_strategy, scores);
    hkv::MutateArgs a = base_args(t, n, keys, nullptr, scores_w.get(), ignore_evict_strategy != 0);
    if (ignore_evict_strategy) a.epoch = hkv::kIgnoredEpoch;
    a.ptrs = values;
    a.founds = founds;
    a.locked_key_ptrs = locked_key_ptrs;
    mutate(t, hkv::kOpFindOrInsertPtr, a, nullptr, nullptr, kInserter, unique_key != 0,
           static_cast<cudaStream_t>(stream));
  });
}

int hkv_lock_keys(hkv_table* t, uint64_t n, const uint64_t* keys, uint64_t** locked_key_ptrs,
                  bool* success, hkv_stream stream, const uint64_t* scores) {
  return guarded([&] {
    refuse_in_memory_mode(t, "lock_keys");
    if (n == 0) return;
    Scores scores_w(t, scores, n, stream, false);
    if (locked_key_ptrs == nullptr) {
      throw HkvError{HKV_ERR_INVALID_ARG, "locked_key_ptrs must not be null"};
    }
    hkv::MutateArgs a = base_args(t, n, keys, nullptr, scores_w.get(), false);
    a.founds = success;
    a.locked_key_ptrs = locked_key_ptrs;
    mutate(t, hkv::kOpLockKeys, a, nullptr, nullptr, kInserter, true,
           static_cast<cudaStream_t>(stream));
  });
}

int hkv_unlock_keys(hkv_table* t, uint64_t n, uint64_t** locked_key_ptrs, const uint64_t* keys,
                    bool* success, hkv_stream stream) {
  return guarded([&] {
    if (n == 0) return;
    DeviceGuard dg(t->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    LockScope ls(t, kInserter, s);
    hkv::launch_unlock_keys(t->view, n, locked_key_ptrs, keys, success, s);
    ls.done();
    check_launch();
  });
}

int hkv_assign(hkv_table* t, uint64_t n, const uint64_t* keys, const void* values,
               const uint64_t* scores, hkv_stream stream, int unique_key) {
  return guarded([&] {
    refuse_in_memory_mode(t, "assign");
    if (n == 0) return;
    Scores scores_w(t, scores, n, stream, false);
    check_strategy(t, t->opt.evict_strategy, scores);
    hkv::MutateArgs a = base_args(t, n, keys, values, scores_w.get(), false);
    mutate(t, hkv::kOpAssign, a, values, nullptr, kUpdater, unique_key != 0,
           static_cast<cudaStream_t>(stream));
  });
}

int hkv_assign_scores(hkv_table* t, uint64_t n, const uint64_t* keys, const uint64_t* scores,
                      hkv_stream stream, int unique_key) {
  return guarded([&] {
    refuse_in_memory_mode(t, "assign_scores");
    if (n == 0) return;
    Scores scores_w(t, scores, n, stream, false);
    check_strategy(t, t->opt.evict_strategy, scores);
    hkv::MutateArgs a = base_args(t, n, keys, nullptr, scores_w.get(), false);
    mutate(t, hkv::kOpAssignScores, a, nullptr, nullptr, kUpdater, unique_key != 0,
           static_cast<cudaStream_t>(stream));
  });
}

int hkv_assign_values(hkv_table* t, uint64_t n, const uint64_t* keys, const void* values,
                      hkv_stream stream, int unique_key) {
  return guarded([&] {
    refuse_in_memory_mode(t, "assign_values");
    if (n == 0) return;
    hkv::MutateArgs a = base_args(t, n, keys, values, nullptr, false);
    mutate(t, hkv::kOpAssignValues, a, values, nullptr, kUpdater, unique_key != 0,
           static_cast<cudaStream_t>(stream));
  });
}

int hkv_find(hkv_table* t, uint64_t n, const uint64_t* keys, void* values, bool* founds,
             uint64_t* scores, hkv_stream stream) {
  return guarded([&] {
    if (n == 0) return;
    Scores scores_w(t, scores, n, stream, true);
    DeviceGuard dg(t->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t work_bytes =
        t->opt.table_mode == 1 ? 0 : hkv::find_workspace_bytes(t->view, n, values);
    WorkspaceLease work(t, 0, work_bytes, s);
    LockScope ls(t, kReader, s);
    if (t->opt.table_mode == 1) {
      hkv::launch_dual_find(view_for(t, values), n, keys, values, founds, scores_w.get(), s);
    } else {
      hkv::launch_find(view_for(t, values), n, keys, values, founds, scores_w.get(), s,
                       work.get(), work_bytes);
    }
    ls.done();
    check_launch();
  });
}

namespace {

// Creates the staging state of hkv_find_host on first use.  A chunk carries
// about 32 MiB of rows: large enough for the copy engines to run at the rate of
// the host link, small enough that the first rows leave after a few dozen
// microseconds of lookup.
void prepare_stage(hkv_table* t) {
  hkv_table::HostStage& st = t->stage;
  if (st.block != nullptr) return;
  const uint64_t row_bytes = t->view.row_bytes;
  uint64_t chunk = (32ull << 20) / (row_bytes ? row_bytes : 1);
  chunk = chunk > (1ull << 17) ? (1ull << 17) : chunk;
  chunk = chunk < 4096 ? 4096 : chunk;
  chunk &= ~uint64_t(255);
  auto up = [](uint64_t x) { return (x + 255) / 256 * 256; };
  const uint64_t per_set = up(chunk * 8) + up(chunk * row_bytes) + up(chunk * 8) + up(chunk);
  void* block = nullptr;
  if (t->alloc.alloc(t->alloc.ctx, HKV_MEM_DEVICE, &block, 2 * per_set, 0) != 0 || block == nullptr) {
    cudaGetLastError();
    throw HkvError{HKV_ERR_CUDA, "hkv_find_host: out of device memory for the staging buffers"};
  }
  for (int i = 0; i < 2; ++i) {
    HKV_CUDA(cudaStreamCreateWithFlags(&st.stream[i], cudaStreamNonBlocking));
    HKV_CUDA(cudaEventCreateWithFlags(&st.done[i], cudaEventDisableTiming));
    uint8_t* at = static_cast<uint8_t*>(block) + i * per_set;
    st.keys[i] = reinterpret_cast<uint64_t*>(at);
    at += up(chunk * 8);
    st.rows[i] = at;
    at += up(chunk * row_bytes);
    st.scores[i] = reinterpret_cast<uint64_t*>(at);
    at += up(chunk * 8);
    st.founds[i] = reinterpret_cast<bool*>(at);
  }
  HKV_CUDA(cudaEventCreateWithFlags(&st.start, cudaEventDisableTiming));
  st.chunk = chunk;
  st.block = static_cast<uint8_t*>(block);
}

}  // namespace

int hkv_find_host(hkv_table* t, uint64_t n, const uint64_t* host_keys, void* host_values,
                  bool* host_founds, uint64_t* host_scores, hkv_stream stream) {
  return guarded([&] {
    if (n == 0) return;
    HKV_CHECK(host_keys != nullptr && host_values != nullptr && host_founds != nullptr,
              "hkv_find_host: keys, values and founds must not be null");
    HKV_CHECK(host_scores == nullptr || t->opt.score_size == 8,
              "hkv_find_host: scores are returned for 64-bit scores only");
    DeviceGuard dg(t->device);
    cudaStream_t user = static_cast<cudaStream_t>(stream);
    hkv_table::HostStage& st = t->stage;
    std::lock_guard<std::mutex> hold(st.mu);   // one batch at a time owns the staging buffers
    prepare_stage(t);
    const uint64_t row_bytes = t->view.row_bytes;
    // everything below starts after what the caller queued before the call ...
    HKV_CUDA(cudaEventRecord(st.start, user));
    for (int i = 0; i < 2; ++i) HKV_CUDA(cudaStreamWaitEvent(st.stream[i], st.start, 0));
    uint64_t c = 0;
    for (uint64_t off = 0; off < n; off += st.chunk, ++c) {
      const int b = static_cast<int>(c & 1);
      const uint64_t m = n - off < st.chunk ? n - off : st.chunk;
      cudaStream_t cs = st.stream[b];
      // keys in, lookup, rows out: on the chunk's stream; the other stream does
      // the same for the neighbouring chunk, so one chunk's lookup and key copy
      // run under the other's row copy and the host link never idles
      HKV_CUDA(cudaMemcpyAsync(st.keys[b], host_keys + off, m * 8, cudaMemcpyHostToDevice, cs));
      HKV_CUDA(cudaMemsetAsync(st.rows[b], 0, m * row_bytes, cs));   // rows of misses: zero
      const int rc = hkv_find(t, m, st.keys[b], st.rows[b], st.founds[b],
                              host_scores ? st.scores[b] : nullptr, cs);
      if (rc != HKV_OK) throw HkvError{rc, g_last_error};
      // flags and scores leave first and the rows last: a small copy queued
      // behind the rows would wait for the NEXT chunk's rows on the shared
      // copy engine, and this stream's next chunk would wait with it
      HKV_CUDA(cudaMemcpyAsync(host_founds + off, st.founds[b], m, cudaMemcpyDeviceToHost, cs));
      if (host_scores) {
        HKV_CUDA(cudaMemcpyAsync(host_scores + off, st.scores[b], m * 8, cudaMemcpyDeviceToHost,
                                 cs));
      }
      HKV_CUDA(cudaMemcpyAsync(static_cast<uint8_t*>(host_values) + off * row_bytes, st.rows[b],
                               m * row_bytes, cudaMemcpyDeviceToHost, cs));
    }
    // ... and what the caller queues after it starts when both streams are done
    for (int i = 0; i < 2; ++i) {
      HKV_CUDA(cudaEventRecord(st.done[i], st.stream[i]));
      HKV_CUDA(cudaStreamWaitEvent(user, st.done[i], 0));
    }
  });
}

int hkv_find_missed(hkv_table* t, uint64_t n, const uint64_t* keys, void* values,
                    uint64_t* missed_keys, int* missed_indices, int* missed_size, uint64_t* scores,
                    hkv_stream stream) {
  return guarded([&] {
    refuse_in_memory_mode(t, "find");
    if (n == 0) return;
    Scores scores_w(t, scores, n, stream, true);
    DeviceGuard dg(t->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    HKV_CUDA(cudaMemsetAsync(missed_size, 0, sizeof(int), s));
    LockScope ls(t, kReader, s);
    hkv::launch_find_missed(view_for(t, values), n, keys, values, missed_keys, missed_indices,
                            missed_size, scores_w.get(), s);
    ls.done();
    check_launch();
  });
}

int hkv_find_ptr(hkv_table* t, uint64_t n, const uint64_t* keys, void** values, bool* founds,
                 uint64_t* scores, hkv_stream stream, int /*unique_key*/) {
  return guarded([&] {
    refuse_in_memory_mode(t, "find");
    if (n == 0) return;
    Scores scores_w(t, scores, n, stream, true);
    DeviceGuard dg(t->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    LockScope ls(t, kReader, s);
    hkv::launch_find_ptr(t->view, n, keys, values, founds, scores_w.get(), s);
    ls.done();
    check_launch();
  });
}

int hkv_find_and_update(hkv_table* t, uint64_t n, const uint64_t* keys, void** values,
                        bool* founds, uint64_t* scores, hkv_stream stream, int unique_key) {
  return guarded([&] {
    refuse_in_memory_mode(t, "find_and_update");
    if (n == 0) return;
    Scores scores_w(t, scores, n, stream, true);
    // scores are an input here for the strategies that take them and are
    // overwritten with the stored score
    hkv::MutateArgs a = base_args(t, n, keys, nullptr, scores_w.get(), false);
    a.scores_out = scores_w.get();
    a.ptrs = values;
    a.founds = founds;
    mutate(t, hkv::kOpFindAndUpdate, a, nullptr, nullptr, kUpdater, unique_key != 0,
           static_cast<cudaStream_t>(stream));
  });
}

int hkv_find_routed(hkv_table* t, uint32_t world, uint32_t my_rank, uint64_t segment_capacity,
                    const uint64_t* inbox_keys, const uint32_t* inbox_origin,
                    const uint64_t* inbox_counts, const hkv_peer_ptrs* out_values,
                    const hkv_peer_ptrs* out_founds, hkv_stream stream) {
  return guarded([&] {
    refuse_in_memory_mode(t, "find");
    if (world == 0 || world > hkv::kMaxPeers || my_rank >= world) {
      throw HkvError{HKV_ERR_INVALID_ARG, "world size must be between 1 and 16"};
    }
    if (!hkv::line_buckets(t->view)) {
      throw HkvError{HKV_ERR_UNSUPPORTED, "the routed form needs max_bucket_size == 128"};
    }
    DeviceGuard dg(t->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    hkv::PeerPtrs ov{}, of{};
    for (uint32_t r = 0; r < world; ++r) {
      ov.p[r] = out_values->p[r];
      of.p[r] = out_founds->p[r];
    }
    LockScope ls(t, kReader, s);
    hkv::launch_find_routed(t->view, world, my_rank, segment_capacity, inbox_keys, inbox_origin,
                            inbox_counts, ov, of, s);
    ls.done();
    check_launch();
  });
}

int hkv_upsert_routed(hkv_table* t, int op, uint32_t world, uint32_t my_rank,
                      uint64_t segment_capacity, const uint64_t* inbox_keys,
                      const uint32_t* inbox_origin, const uint64_t* inbox_counts,
                      const hkv_peer_ptrs* values, const hkv_peer_ptrs* accum_flags,
                      hkv_stream stream) {
  return guarded([&] {
    refuse_in_memory_mode(t, "insert_or_assign");
    if (world == 0 || world > hkv::kMaxPeers || my_rank >= world) {
      throw HkvError{HKV_ERR_INVALID_ARG, "world size must be between 1 and 16"};
    }
    int kernel_op;
    switch (op) {
      case HKV_ROUTED_INSERT_OR_ASSIGN: kernel_op = hkv::kOpInsertOrAssign; break;
      case HKV_ROUTED_FIND_OR_INSERT: kernel_op = hkv::kOpFindOrInsert; break;
      case HKV_ROUTED_ACCUM_OR_ASSIGN: kernel_op = hkv::kOpAccumOrAssign; break;
      default: throw HkvError{HKV_ERR_INVALID_ARG, "op must be 0, 1 or 2"};
    }
    if (op == HKV_ROUTED_ACCUM_OR_ASSIGN && accum_flags == nullptr) {
      throw HkvError{HKV_ERR_INVALID_ARG, "accum_or_assign needs the ranks' flag arrays"};
    }
    if (op == HKV_ROUTED_ACCUM_OR_ASSIGN) check_accum_type(t, nullptr);
    if (segment_capacity % 32 != 0) {
      throw HkvError{HKV_ERR_INVALID_ARG, "segment_capacity must be a multiple of 32"};
    }
    check_strategy(t, t->opt.evict_strategy, nullptr);  // only the score-free strategies pass
    if (t->view.hbm_slots < t->view.capacity || !t->reach_max_capacity.load() ||
        !hkv::line_buckets(t->view)) {
      throw HkvError{HKV_ERR_UNSUPPORTED,
                     "the routed form needs a pure-HBM table of fixed capacity with "
                     "max_bucket_size == 128"};
    }
    DeviceGuard dg(t->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    hkv::PeerPtrs pv{}, pf{};
    for (uint32_t r = 0; r < world; ++r) {
      pv.p[r] = values->p[r];
      pf.p[r] = accum_flags != nullptr ? accum_flags->p[r] : nullptr;
    }
    if (segment_capacity > (1ull << hkv::kRowTagShift)) {
      throw HkvError{HKV_ERR_INVALID_ARG, "segment_capacity above 2^28 keys"};
    }
    hkv::MutateArgs a = base_args(t, 0, nullptr, nullptr, nullptr, false);
    hkv::RoutedArgs r;
    r.world = world;
    r.first_segment = (my_rank + 1) % world;
    r.segment_capacity = segment_capacity;
    r.inbox_keys = inbox_keys;
    r.inbox_origin = inbox_origin;
    r.inbox_counts = inbox_counts;
    r.values_of = pv;
    r.flags_of = pf;
    WorkspaceLease work(t, 3, hkv::routed_workspace_bytes(world, segment_capacity), s);
    if (work.get() == nullptr) {
      throw HkvError{HKV_ERR_CUDA, "out of device memory for the request chains of the routed update"};
    }
    const bool same_shape =
        t->routed_world == world && t->routed_segment_capacity == segment_capacity;
    t->routed_world = world;
    t->routed_segment_capacity = segment_capacity;
    hkv::prepare_routed_workspace(t->view, r, work.get(), work.fresh() || !same_shape, s);
    LockScope ls(t, kInserter, s);
    hkv::launch_mutate_routed(kernel_op, t->view, a, r, s);
    ls.done();
    check_launch();
  });
}

int hkv_contains(hkv_table* t, uint64_t n, const uint64_t* keys, bool* founds, hkv_stream stream) {
  return guarded([&] {
    refuse_in_memory_mode(t, "contains");
    if (n == 0) return;
    DeviceGuard dg(t->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    LockScope ls(t, kReader, s);
    hkv::launch_contains(t->view, n, keys, founds, s);
    ls.done();
    check_launch();
  });
}

int hkv_erase(hkv_table* t, uint64_t n, const uint64_t* keys, hkv_stream stream) {
  return guarded([&] {
    refuse_in_memory_mode(t, "erase");
    if (n == 0) return;
    DeviceGuard dg(t->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    LockScope ls(t, kInserter, s);
    hkv::launch_erase(t->view, n, keys, s);
    ls.done();
    check_launch();
  });
}

int hkv_erase_if(hkv_table* t, int predicate, uint64_t pattern, uint64_t threshold,
                 hkv_stream stream, uint64_t* erased) {
  return guarded([&] {
    DeviceGuard dg(t->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (predicate < HKV_PRED_ALL || predicate > HKV_PRED_SCORE_LESS_EQ) {
      throw HkvError{HKV_ERR_INVALID_ARG, "unknown predicate"};
    }
    CounterLease lease(t);
    unsigned long long* ctr = lease.get();
    {
      LockScope ls(t, kInserter, s);
      HKV_CUDA(cudaMemsetAsync(ctr, 0, sizeof(*ctr), s));
      hkv::launch_erase_if(t->view, predicate, pattern, threshold, ctr, s);
      ls.done();
    }
    check_launch();
    unsigned long long h = 0;
    HKV_CUDA(cudaMemcpyAsync(&h, ctr, sizeof(h), cudaMemcpyDeviceToHost, s));
    HKV_CUDA(cudaStreamSynchronize(s));
    if (erased != nullptr) *erased = h;
  });
}

int hkv_clear(hkv_table* t, hkv_stream stream) {
  return guarded([&] {
    DeviceGuard dg(t->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    LockScope ls(t, kInserter, s);
    hkv::launch_clear(t->view, s);
    ls.done();
    check_launch();
  });
}

int hkv_export_batch_if(hkv_table* t, int predicate, uint64_t pattern, uint64_t threshold,
                        uint64_t n, uint64_t offset, uint64_t* d_counter, uint64_t* keys,
                        void* values, uint64_t* scores, hkv_stream stream) {
  return guarded([&] {
    DeviceGuard dg(t->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (predicate < HKV_PRED_ALL || predicate > HKV_PRED_SCORE_LESS_EQ) {
      throw HkvError{HKV_ERR_INVALID_ARG, "unknown predicate"};
    }
    // The window is clamped before anything is sized by it: "export everything"
    // callers pass a huge n.  The capacity read here can only be smaller than
    // the one the kernel sees (tables never shrink).
    {
      const uint64_t capacity = t->view.capacity;
      n = offset < capacity ? (n < capacity - offset ? n : capacity - offset) : 0;
    }
    Scores scores_w(t, scores, n, stream, true);
    LockScope ls(t, kReader, s);
    HKV_CUDA(cudaMemsetAsync(d_counter, 0, sizeof(uint64_t), s));
    if (n > 0 && offset < t->view.capacity) {
      hkv::launch_export(view_for(t, values), predicate, pattern, threshold, n, offset,
                         reinterpret_cast<unsigned long long*>(d_counter), keys, values, scores_w.get(),
                         s);
    }
    ls.done();
    check_launch();
  });
}

int hkv_export_batch(hkv_table* t, uint64_t n, uint64_t offset, uint64_t* d_counter,
                     uint64_t* keys, void* values, uint64_t* scores, hkv_stream stream) {
  return hkv_export_batch_if(t, HKV_PRED_ALL, 0, 0, n, offset, d_counter, keys, values, scores,
                             stream);
}

int hkv_export_batch_count(hkv_table* t, uint64_t n, uint64_t offset, uint64_t* keys,
                           void* values, uint64_t* scores, hkv_stream stream, uint64_t* count) {
  return guarded([&] {
    DeviceGuard dg(t->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    CounterLease lease(t);
    unsigned long long* ctr = lease.get();
    int rc = hkv_export_batch(t, n, offset, reinterpret_cast<uint64_t*>(ctr), keys, values,
                              scores, stream);
    if (rc != HKV_OK) throw HkvError{rc, g_last_error};
    unsigned long long h = 0;
    HKV_CUDA(cudaMemcpyAsync(&h, ctr, sizeof(h), cudaMemcpyDeviceToHost, s));
    HKV_CUDA(cudaStreamSynchronize(s));
    *count = h;
  });
}

int hkv_size_if(hkv_table* t, int predicate, uint64_t pattern, uint64_t threshold,
                uint64_t* d_counter, hkv_stream stream) {
  return guarded([&] {
    DeviceGuard dg(t->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (predicate < HKV_PRED_ALL || predicate > HKV_PRED_SCORE_LESS_EQ) {
      throw HkvError{HKV_ERR_INVALID_ARG, "unknown predicate"};
    }
    LockScope ls(t, kReader, s);
    HKV_CUDA(cudaMemsetAsync(d_counter, 0, sizeof(uint64_t), s));
    hkv::launch_size_if(t->view, predicate, pattern, threshold,
                        reinterpret_cast<unsigned long long*>(d_counter), s);
    ls.done();
    check_launch();
  });
}

int hkv_size(hkv_table* t, hkv_stream stream, uint64_t* size) {
  return guarded([&] {
    DeviceGuard dg(t->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    CounterLease lease(t);
    unsigned long long* ctr = lease.get();
    {
      LockScope ls(t, kReader, s);
      HKV_CUDA(cudaMemsetAsync(ctr, 0, sizeof(*ctr), s));
      hkv::launch_sum_sizes(t->view, t->view.buckets, ctr, s);
      ls.done();
    }
    check_launch();
    unsigned long long h = 0;
    HKV_CUDA(cudaMemcpyAsync(&h, ctr, sizeof(h), cudaMemcpyDeviceToHost, s));
    HKV_CUDA(cudaStreamSynchronize(s));
    *size = h;
  });
}

int hkv_load_factor(hkv_table* t, hkv_stream stream, float* load_factor) {
  uint64_t sz = 0;
  int rc = hkv_size(t, stream, &sz);
  if (rc != HKV_OK) return rc;
  *load_factor = static_cast<float>((sz * 1.0) / (t->view.capacity * 1.0));
  return HKV_OK;
}

uint64_t hkv_capacity(const hkv_table* t) { return t->view.capacity; }
uint64_t hkv_bucket_count(const hkv_table* t) { return t->view.buckets; }
uint64_t hkv_dim(const hkv_table* t) { return t->opt.dim; }
uint64_t hkv_max_bucket_size(const hkv_table* t) { return t->opt.max_bucket_size; }

int hkv_set_global_epoch(hkv_table* t, uint64_t epoch) {
  t->global_epoch.store(epoch);
  return HKV_OK;
}

int hkv_reserve(hkv_table* t, uint64_t new_capacity, hkv_stream stream) {
  return guarded([&] {
    refuse_in_memory_mode(t, "reserve");
    DeviceGuard dg(t->device);
    reserve(t, new_capacity, static_cast<cudaStream_t>(stream));
  });
}

int hkv_set_max_capacity(hkv_table* t, uint64_t new_max_capacity) {
  return guarded([&] {
    // set_max_capacity, include/merlin_hashtable.cuh:3561-3579
    if (new_max_capacity == 0 || (new_max_capacity & (new_max_capacity - 1)) != 0) {
      throw HkvError{HKV_ERR_INVALID_ARG, "None power-of-2 new_max_capacity is not supported."};
    }
    LockScope ls(t, kInserter, nullptr);
    if (new_max_capacity >= t->view.capacity) {
      t->reach_max_capacity.store(false);
      t->opt.max_capacity = new_max_capacity;
    }
    ls.done();
  });
}

int hkv_promote_hot_buckets(hkv_table* t, hkv_stream stream, uint64_t* promoted) {
  return guarded([&] {
    DeviceGuard dg(t->device);
    const uint64_t n = promote_hot_buckets(t, static_cast<cudaStream_t>(stream));
    if (promoted != nullptr) *promoted = n;
  });
}

int hkv_get_view(const hkv_table* t, hkv_table_view* view) {
  return guarded([&] {
    const hkv::TableView& v = t->view;
    view->digests = v.digests;
    view->keys = v.key_words;
    view->scores = v.score_words;
    view->slot_word_mask = v.line_mask;
    view->values_hbm = v.values_hbm;
    view->values_host = v.values_host;
    view->bucket_sizes = v.bucket_sizes;
    view->buckets = v.buckets;
    view->capacity = v.capacity;
    view->hbm_slots = v.hbm_slots;
    view->bucket_map = v.bucket_map;
    view->row_bytes = v.row_bytes;
    view->max_bucket_size = v.bucket_slots;
    view->empty_key = v.empty_key;
    view->reclaim_key = v.reclaim_key;
    view->locked_key = v.locked_key;
    view->reserved_mask = v.reserved_mask;
    view->reserved_value = v.reserved_value;
  });
}

int hkv_external_begin(hkv_table* t, int group, hkv_stream stream) {
  return guarded([&] {
    if (group < kReader || group > kInserter) {
      throw HkvError{HKV_ERR_INVALID_ARG, "group must be 0 (reader), 1 (updater) or 2 (inserter)"};
    }
    if (t->opt.api_lock) t->lock.acquire(static_cast<Group>(group), static_cast<cudaStream_t>(stream));
  });
}

int hkv_external_end(hkv_table* t, int group, hkv_stream stream) {
  return guarded([&] {
    if (group < kReader || group > kInserter) {
      throw HkvError{HKV_ERR_INVALID_ARG, "group must be 0 (reader), 1 (updater) or 2 (inserter)"};
    }
    if (t->opt.api_lock) t->lock.release(static_cast<Group>(group), static_cast<cudaStream_t>(stream));
  });
}

int hkv_device_status(hkv_table* t, hkv_stream stream, uint32_t* status) {
  return guarded([&] {
    DeviceGuard dg(t->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    uint32_t h = 0;
    HKV_CUDA(cudaMemcpyAsync(&h, t->view.status, sizeof(h), cudaMemcpyDeviceToHost, s));
    HKV_CUDA(cudaMemsetAsync(t->view.status, 0, sizeof(uint32_t), s));
    HKV_CUDA(cudaStreamSynchronize(s));
    *status = h;
  });
}

}  // extern "C"
