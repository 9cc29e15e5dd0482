// Host side of the key-hash sharded table: one process (or thread) per GPU,
// every rank owns one sub-table and a workspace the other ranks of the node can
// store into -- its inbox of routed keys and its batch / result buffers.  This
// file allocates the workspaces, maps the peers' workspaces (CUDA IPC between
// processes, plain peer pointers inside one process), keeps the barrier epochs
// and strings the device steps together:
//
//   find      route keys into the owners' inboxes | barrier | every owner looks
//             up what arrived and stores hit rows and flags into the
//             requesters' buffers | barrier
//   update    the same routing and barriers around insert_or_assign /
//             find_or_insert / accum_or_assign of the routed form
//
// No NCCL call, no host synchronisation.  The reference is a single-GPU library
// and has no counterpart; its users shard by hand, one table per GPU.
#include <cuda_runtime.h>

#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "../../include/hkv_b200.h"

namespace {

thread_local std::string g_sharded_error;

int fail(int code, const std::string& msg) {
  g_sharded_error = msg;
  return code;
}

constexpr uint32_t kMaxRanks = 16;

uint64_t up256(uint64_t x) { return (x + 255) / 256 * 256; }

// One workspace.  All ranks lay theirs out the same way, so a peer's arrays are
// its base address plus the same offsets.
struct Lane {
  uint8_t* local = nullptr;             // this rank's workspace
  bool owns_local = false;              // ... from cudaMalloc here (else the caller's memory)
  void* base[kMaxRanks] = {};           // every rank's workspace as this process sees it
  bool opened[kMaxRanks] = {};          // base[r] came from cudaIpcOpenMemHandle
  uint64_t* scratch = nullptr;          // [0,16): routing cursors; [16]: barrier status
  uint32_t epoch = 0;
  bool connected = false;
  cudaStream_t hi = nullptr, lo = nullptr;  // streams of the asynchronous form
  cudaEvent_t ready = nullptr, routed = nullptr, served = nullptr, done = nullptr;
};

}  // namespace

struct hkv_sharded {
  hkv_table* table = nullptr;
  uint32_t world = 1, rank = 0;
  uint64_t max_batch = 0, row_bytes = 0, bytes = 0;
  uint64_t off_keys = 0, off_origin = 0, off_counts = 0, off_flags = 0, off_founds = 0,
           off_values = 0;
  int device = 0;
  uint32_t next_lane = 0;
  std::vector<Lane> lanes;
};

namespace {

hkv_peer_ptrs peers_at(const Lane& l, uint32_t world, uint64_t offset) {
  hkv_peer_ptrs p{};
  for (uint32_t r = 0; r < world; ++r) p.p[r] = static_cast<uint8_t*>(l.base[r]) + offset;
  return p;
}

struct DeviceScope {
  int prev = -1;
  explicit DeviceScope(int dev) {
    cudaGetDevice(&prev);
    if (prev != dev) cudaSetDevice(dev);
    else prev = -1;
  }
  ~DeviceScope() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

// Offsets of the arrays inside a workspace (needs world, max_batch, row_bytes).
void lay_out(hkv_sharded* s) {
  uint64_t at = 0;
  s->off_keys = at;
  at = up256(at + uint64_t(s->world) * s->max_batch * 8);
  s->off_origin = at;
  at = up256(at + uint64_t(s->world) * s->max_batch * 4);
  s->off_counts = at;
  at = up256(at + kMaxRanks * 8);
  s->off_flags = at;
  at = up256(at + kMaxRanks * 4);
  s->off_founds = at;
  at = up256(at + s->max_batch);
  s->off_values = at;
  at = up256(at + s->max_batch * s->row_bytes);
  s->bytes = at;
}

int check_lane(const hkv_sharded* s, uint32_t lane, bool connected) {
  if (s == nullptr) return fail(HKV_ERR_INVALID_ARG, "null sharded table");
  if (lane >= s->lanes.size()) return fail(HKV_ERR_INVALID_ARG, "no such lane");
  if (connected && !s->lanes[lane].connected) {
    return fail(HKV_ERR_RUNTIME, "the lane is not connected to its peers yet");
  }
  return HKV_OK;
}

int route(hkv_sharded* s, Lane& l, uint64_t n, const uint64_t* keys, cudaStream_t stream) {
  if (n > s->max_batch) return fail(HKV_ERR_INVALID_ARG, "batch larger than the workspace");
  const hkv_peer_ptrs k = peers_at(l, s->world, s->off_keys);
  const hkv_peer_ptrs o = peers_at(l, s->world, s->off_origin);
  const hkv_peer_ptrs c = peers_at(l, s->world, s->off_counts);
  if (hkv_shard_route_keys_p2p(n, keys, s->world, s->rank, s->max_batch, &k, &o, &c, l.scratch,
                               stream) != HKV_OK) {
    return fail(HKV_ERR_CUDA, hkv_shard_last_error());
  }
  return HKV_OK;
}

int barrier(hkv_sharded* s, Lane& l, uint32_t max_polls, cudaStream_t stream) {
  const hkv_peer_ptrs f = peers_at(l, s->world, s->off_flags);
  l.epoch += 1;
  if (hkv_shard_barrier(s->world, s->rank, &f, l.epoch,
                        reinterpret_cast<uint32_t*>(l.scratch + 16), max_polls,
                        stream) != HKV_OK) {
    return fail(HKV_ERR_CUDA, hkv_shard_last_error());
  }
  return HKV_OK;
}

int lookup(hkv_sharded* s, Lane& l, cudaStream_t stream) {
  const hkv_peer_ptrs v = peers_at(l, s->world, s->off_values);
  const hkv_peer_ptrs f = peers_at(l, s->world, s->off_founds);
  const int rc = hkv_find_routed(
      s->table, s->world, s->rank, s->max_batch,
      reinterpret_cast<const uint64_t*>(l.local + s->off_keys),
      reinterpret_cast<const uint32_t*>(l.local + s->off_origin),
      reinterpret_cast<const uint64_t*>(l.local + s->off_counts), &v, &f, stream);
  if (rc != HKV_OK) return fail(rc, hkv_last_error());
  return HKV_OK;
}

}  // namespace

extern "C" {

const char* hkv_sharded_last_error(void) { return g_sharded_error.c_str(); }

int hkv_sharded_create(hkv_table* table, uint32_t world, uint32_t rank, uint64_t max_batch,
                       uint32_t lanes, hkv_sharded** out) {
  return hkv_sharded_create_external(table, world, rank, max_batch, lanes, nullptr, out);
}

int hkv_sharded_workspace_bytes(hkv_table* table, uint32_t world, uint64_t max_batch,
                                uint64_t* bytes) {
  if (table == nullptr || bytes == nullptr) return fail(HKV_ERR_INVALID_ARG, "null argument");
  if (world == 0 || world > kMaxRanks) {
    return fail(HKV_ERR_INVALID_ARG, "world size must be between 1 and 16");
  }
  hkv_table_view view{};
  if (hkv_get_view(table, &view) != HKV_OK) return fail(HKV_ERR_RUNTIME, hkv_last_error());
  hkv_sharded layout;
  layout.world = world;
  layout.max_batch = (max_batch + 31) / 32 * 32;
  layout.row_bytes = view.row_bytes;
  lay_out(&layout);
  *bytes = layout.bytes;
  return HKV_OK;
}

int hkv_sharded_create_external(hkv_table* table, uint32_t world, uint32_t rank,
                                uint64_t max_batch, uint32_t lanes, void* const* workspaces,
                                hkv_sharded** out) {
  if (table == nullptr || out == nullptr) {
    return fail(HKV_ERR_INVALID_ARG, "table and out must not be null");
  }
  if (world == 0 || world > kMaxRanks || rank >= world) {
    return fail(HKV_ERR_INVALID_ARG, "world size must be between 1 and 16");
  }
  if (lanes == 0 || lanes > 8) return fail(HKV_ERR_INVALID_ARG, "between 1 and 8 lanes");
  hkv_table_view view{};
  if (hkv_get_view(table, &view) != HKV_OK) return fail(HKV_ERR_RUNTIME, hkv_last_error());
  cudaPointerAttributes attr{};
  if (cudaPointerGetAttributes(&attr, view.bucket_sizes) != cudaSuccess) {
    cudaGetLastError();
    return fail(HKV_ERR_CUDA, "cannot tell which device owns the table");
  }
  hkv_sharded* s = new (std::nothrow) hkv_sharded();
  if (s == nullptr) return fail(HKV_ERR_RUNTIME, "out of host memory");
  s->table = table;
  s->world = world;
  s->rank = rank;
  s->device = attr.device;
  s->max_batch = (max_batch + 31) / 32 * 32;  // inbox segments hold whole warps of keys
  s->row_bytes = view.row_bytes;
  lay_out(s);
  DeviceScope scope(s->device);
  s->lanes.resize(lanes);
  for (uint32_t i = 0; i < lanes; ++i) {
    Lane& l = s->lanes[i];
    int least = 0, greatest = 0;
    cudaDeviceGetStreamPriorityRange(&least, &greatest);
    if (workspaces != nullptr) {
      if (workspaces[i] == nullptr) {
        hkv_sharded_destroy(s);
        return fail(HKV_ERR_INVALID_ARG, "null workspace");
      }
      l.local = static_cast<uint8_t*>(workspaces[i]);
    } else if (cudaMalloc(reinterpret_cast<void**>(&l.local), s->bytes) == cudaSuccess) {
      l.owns_local = true;
    } else {
      l.local = nullptr;
    }
    if (l.local == nullptr ||
        cudaMalloc(reinterpret_cast<void**>(&l.scratch), 32 * sizeof(uint64_t)) != cudaSuccess ||
        cudaMemset(l.local, 0, s->bytes) != cudaSuccess ||
        cudaMemset(l.scratch, 0, 32 * sizeof(uint64_t)) != cudaSuccess ||
        // routing and barriers of the next batch must not queue behind the
        // blocks of the previous batch's lookup: they run at higher priority
        cudaStreamCreateWithPriority(&l.hi, cudaStreamNonBlocking, greatest) != cudaSuccess ||
        cudaStreamCreateWithPriority(&l.lo, cudaStreamNonBlocking, least) != cudaSuccess ||
        cudaEventCreateWithFlags(&l.ready, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&l.routed, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&l.served, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&l.done, cudaEventDisableTiming) != cudaSuccess) {
      cudaGetLastError();
      hkv_sharded_destroy(s);
      return fail(HKV_ERR_CUDA, "out of device memory for the peer workspace");
    }
    l.base[rank] = l.local;
    if (world == 1) l.connected = true;
  }
  if (cudaDeviceSynchronize() != cudaSuccess) {
    cudaGetLastError();
    hkv_sharded_destroy(s);
    return fail(HKV_ERR_CUDA, "clearing the peer workspace failed");
  }
  *out = s;
  return HKV_OK;
}

int hkv_sharded_destroy(hkv_sharded* s) {
  if (s == nullptr) return HKV_OK;
  DeviceScope scope(s->device);
  cudaDeviceSynchronize();
  for (Lane& l : s->lanes) {
    for (uint32_t r = 0; r < s->world; ++r) {
      if (l.opened[r]) cudaIpcCloseMemHandle(l.base[r]);
    }
    if (l.local && l.owns_local) cudaFree(l.local);
    if (l.scratch) cudaFree(l.scratch);
    if (l.hi) cudaStreamDestroy(l.hi);
    if (l.lo) cudaStreamDestroy(l.lo);
    for (cudaEvent_t e : {l.ready, l.routed, l.served, l.done}) {
      if (e) cudaEventDestroy(e);
    }
  }
  cudaGetLastError();
  delete s;
  return HKV_OK;
}

uint32_t hkv_sharded_lanes(const hkv_sharded* s) { return s ? uint32_t(s->lanes.size()) : 0; }
uint64_t hkv_sharded_max_batch(const hkv_sharded* s) { return s ? s->max_batch : 0; }

int hkv_sharded_ipc_handle(hkv_sharded* s, uint32_t lane, hkv_ipc_handle* handle) {
  if (int rc = check_lane(s, lane, false)) return rc;
  static_assert(sizeof(cudaIpcMemHandle_t) <= sizeof(hkv_ipc_handle), "handle size");
  if (!s->lanes[lane].owns_local) {
    return fail(HKV_ERR_RUNTIME, "the caller supplied this workspace and shares it by its own means");
  }
  DeviceScope scope(s->device);
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, s->lanes[lane].local) != cudaSuccess) {
    const std::string why = cudaGetErrorString(cudaGetLastError());
    return fail(HKV_ERR_CUDA, "cudaIpcGetMemHandle: " + why);
  }
  std::memset(handle, 0, sizeof(*handle));
  std::memcpy(handle, &h, sizeof(h));
  return HKV_OK;
}

int hkv_sharded_connect_ipc(hkv_sharded* s, uint32_t lane, const hkv_ipc_handle* handles) {
  if (int rc = check_lane(s, lane, false)) return rc;
  DeviceScope scope(s->device);
  Lane& l = s->lanes[lane];
  for (uint32_t r = 0; r < s->world; ++r) {
    if (r == s->rank || l.base[r] != nullptr) continue;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, &handles[r], sizeof(h));
    void* p = nullptr;
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
      const std::string why = cudaGetErrorString(cudaGetLastError());
      return fail(HKV_ERR_CUDA, "cudaIpcOpenMemHandle of rank " + std::to_string(r) + ": " + why);
    }
    l.base[r] = p;
    l.opened[r] = true;
  }
  l.connected = true;
  return HKV_OK;
}

int hkv_sharded_connect_pointers(hkv_sharded* s, uint32_t lane, void* const* bases) {
  if (int rc = check_lane(s, lane, false)) return rc;
  Lane& l = s->lanes[lane];
  for (uint32_t r = 0; r < s->world; ++r) {
    if (r == s->rank) continue;
    if (bases[r] == nullptr) return fail(HKV_ERR_INVALID_ARG, "null peer workspace");
    l.base[r] = bases[r];
  }
  l.connected = true;
  return HKV_OK;
}

void* hkv_sharded_workspace(hkv_sharded* s, uint32_t lane) {
  return (s && lane < s->lanes.size()) ? s->lanes[lane].local : nullptr;
}

int hkv_sharded_buffers(hkv_sharded* s, uint32_t lane, void** rows, bool** flags) {
  if (int rc = check_lane(s, lane, false)) return rc;
  Lane& l = s->lanes[lane];
  if (rows) *rows = l.local + s->off_values;
  if (flags) *flags = reinterpret_cast<bool*>(l.local + s->off_founds);
  return HKV_OK;
}

int hkv_sharded_find(hkv_sharded* s, uint32_t lane, uint64_t n, const uint64_t* keys,
                     uint32_t max_polls, hkv_stream stream) {
  if (int rc = check_lane(s, lane, true)) return rc;
  DeviceScope scope(s->device);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Lane& l = s->lanes[lane];
  if (int rc = route(s, l, n, keys, st)) return rc;
  if (int rc = barrier(s, l, max_polls, st)) return rc;
  if (int rc = lookup(s, l, st)) return rc;
  return barrier(s, l, max_polls, st);
}

int hkv_sharded_find_async(hkv_sharded* s, uint64_t n, const uint64_t* keys, uint32_t max_polls,
                           hkv_stream stream, uint32_t* lane_used) {
  if (s == nullptr || lane_used == nullptr) return fail(HKV_ERR_INVALID_ARG, "null argument");
  const uint32_t lane = s->next_lane;
  if (int rc = check_lane(s, lane, true)) return rc;
  s->next_lane = (lane + 1) % uint32_t(s->lanes.size());
  DeviceScope scope(s->device);
  cudaStream_t user = static_cast<cudaStream_t>(stream);
  Lane& l = s->lanes[lane];
  // the lane starts after what the caller queued before this call (the
  // producer of `keys`, the consumer of the lane's previous results)
  cudaEventRecord(l.ready, user);
  cudaStreamWaitEvent(l.hi, l.ready, 0);
  if (int rc = route(s, l, n, keys, l.hi)) return rc;
  if (int rc = barrier(s, l, max_polls, l.hi)) return rc;
  cudaEventRecord(l.routed, l.hi);
  cudaStreamWaitEvent(l.lo, l.routed, 0);
  if (int rc = lookup(s, l, l.lo)) return rc;
  cudaEventRecord(l.served, l.lo);
  cudaStreamWaitEvent(l.hi, l.served, 0);
  if (int rc = barrier(s, l, max_polls, l.hi)) return rc;
  cudaEventRecord(l.done, l.hi);
  *lane_used = lane;
  if (cudaGetLastError() != cudaSuccess) return fail(HKV_ERR_CUDA, "enqueueing the lane failed");
  return HKV_OK;
}

int hkv_sharded_wait(hkv_sharded* s, uint32_t lane, hkv_stream stream) {
  if (int rc = check_lane(s, lane, true)) return rc;
  DeviceScope scope(s->device);
  if (cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), s->lanes[lane].done, 0) !=
      cudaSuccess) {
    return fail(HKV_ERR_CUDA, cudaGetErrorString(cudaGetLastError()));
  }
  return HKV_OK;
}

int hkv_sharded_upsert(hkv_sharded* s, int op, uint64_t n, const uint64_t* keys, int reuse_route,
                       uint32_t max_polls, hkv_stream stream) {
  if (int rc = check_lane(s, 0, true)) return rc;
  DeviceScope scope(s->device);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Lane& l = s->lanes[0];
  if (!reuse_route) {
    if (int rc = route(s, l, n, keys, st)) return rc;
  }
  if (int rc = barrier(s, l, max_polls, st)) return rc;
  const hkv_peer_ptrs v = peers_at(l, s->world, s->off_values);
  const hkv_peer_ptrs f = peers_at(l, s->world, s->off_founds);
  const int rc = hkv_upsert_routed(
      s->table, op, s->world, s->rank, s->max_batch,
      reinterpret_cast<const uint64_t*>(l.local + s->off_keys),
      reinterpret_cast<const uint32_t*>(l.local + s->off_origin),
      reinterpret_cast<const uint64_t*>(l.local + s->off_counts), &v, &f, st);
  if (rc != HKV_OK) return fail(rc, hkv_last_error());
  return barrier(s, l, max_polls, st);
}

int hkv_sharded_status(hkv_sharded* s, uint32_t lane, hkv_stream stream, uint32_t* status) {
  if (int rc = check_lane(s, lane, false)) return rc;
  DeviceScope scope(s->device);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint32_t h = 0;
  if (cudaMemcpyAsync(&h, s->lanes[lane].scratch + 16, sizeof(h), cudaMemcpyDeviceToHost, st) !=
          cudaSuccess ||
      cudaStreamSynchronize(st) != cudaSuccess) {
    return fail(HKV_ERR_CUDA, cudaGetErrorString(cudaGetLastError()));
  }
  *status = h;
  return HKV_OK;
}

}  // extern "C"
