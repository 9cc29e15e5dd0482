// Routing helpers of the key-hash sharded table: owner = Murmur3(key) % world.
// The reference is a single-GPU library and has nothing like this; the
// sharding rule is the one its users apply by hand (one table per GPU).
//
//   partition   groups a batch of keys by owner rank (counts, offsets, the
//               grouped keys and, for every grouped position, the index the
//               key had in the caller's batch)
//   gather / scatter rows by index, to put rows that came back from the
//               owners into the caller's order (and flags, as 1-byte rows)
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../../include/hkv_b200.h"
#include "hkv_device.cuh"

namespace {

constexpr int kBlock = 256;
constexpr uint32_t kMaxWorld = 64;

__device__ __forceinline__ uint32_t owner_of(uint64_t key, uint32_t world) {
  return static_cast<uint32_t>(hkv::fmix64(key) % world);
}

__global__ void __launch_bounds__(kBlock)
    count_kernel(const uint64_t* __restrict__ keys, uint64_t n, uint32_t world,
                 unsigned long long* __restrict__ counts) {
  __shared__ uint32_t local[kMaxWorld];
  if (threadIdx.x < kMaxWorld) local[threadIdx.x] = 0;
  __syncthreads();
  for (uint64_t i = uint64_t(blockIdx.x) * kBlock + threadIdx.x; i < n;
       i += uint64_t(gridDim.x) * kBlock) {
    atomicAdd(&local[owner_of(keys[i], world)], 1u);
  }
  __syncthreads();
  if (threadIdx.x < world && local[threadIdx.x]) {
    atomicAdd(&counts[threadIdx.x], (unsigned long long)local[threadIdx.x]);
  }
}

// offsets = exclusive prefix sum of counts; cursors start at the offsets
__global__ void offsets_kernel(const unsigned long long* counts, uint32_t world,
                               unsigned long long* offsets, unsigned long long* cursors) {
  if (threadIdx.x == 0) {
    unsigned long long at = 0;
    for (uint32_t r = 0; r < world; ++r) {
      offsets[r] = at;
      cursors[r] = at;
      at += counts[r];
    }
  }
}

__global__ void __launch_bounds__(kBlock)
    place_kernel(const uint64_t* __restrict__ keys, uint64_t n, uint32_t world,
                 unsigned long long* __restrict__ cursors, uint64_t* __restrict__ grouped_keys,
                 uint32_t* __restrict__ origin) {
  __shared__ uint32_t local[kMaxWorld];
  __shared__ unsigned long long base[kMaxWorld];
  // every block takes whole tiles of kBlock keys so that one reservation per
  // owner and tile is enough
  const uint64_t tiles = (n + kBlock - 1) / kBlock;
  for (uint64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    if (threadIdx.x < kMaxWorld) local[threadIdx.x] = 0;
    __syncthreads();
    const uint64_t i = tile * kBlock + threadIdx.x;
    uint64_t key = 0;
    uint32_t owner = 0, rank = 0;
    if (i < n) {
      key = keys[i];
      owner = owner_of(key, world);
      rank = atomicAdd(&local[owner], 1u);
    }
    __syncthreads();
    if (threadIdx.x < world && local[threadIdx.x]) {
      base[threadIdx.x] = atomicAdd(&cursors[threadIdx.x], (unsigned long long)local[threadIdx.x]);
    }
    __syncthreads();
    if (i < n) {
      const unsigned long long at = base[owner] + rank;
      grouped_keys[at] = key;
      origin[at] = static_cast<uint32_t>(i);
    }
    __syncthreads();
  }
}

struct Peers {
  void* p[16];
};

// Groups a batch by owner and stores every key, with the index it has in the
// batch, straight into the owner rank's inbox (segment `my_rank` of it).  A
// block regroups a tile of 1024 keys by owner in shared memory first, so the
// peer stores that follow are runs of consecutive addresses per owner (about
// 1 KiB of keys per owner and tile at 8 ranks) instead of single 8-byte
// writes scattered over all peers.
constexpr int kRouteKeysPerThread = 4;
constexpr int kRouteTile = kBlock * kRouteKeysPerThread;

__global__ void __launch_bounds__(kBlock)
    route_p2p_kernel(const uint64_t* __restrict__ keys, uint64_t n, uint32_t world,
                     uint32_t my_rank, uint64_t segment_capacity,
                     unsigned long long* __restrict__ cursors, const Peers inbox_keys,
                     const Peers inbox_origin) {
  __shared__ uint32_t local[kMaxWorld];
  __shared__ uint32_t start[kMaxWorld];
  __shared__ unsigned long long base[kMaxWorld];
  __shared__ uint64_t tile_keys[kRouteTile];
  __shared__ uint32_t tile_origin[kRouteTile];
  __shared__ uint8_t tile_owner[kRouteTile];
  __shared__ uint64_t* dst_keys[16];
  __shared__ uint32_t* dst_origin[16];
  if (threadIdx.x < 16) {
    dst_keys[threadIdx.x] = static_cast<uint64_t*>(inbox_keys.p[threadIdx.x]);
    dst_origin[threadIdx.x] = static_cast<uint32_t*>(inbox_origin.p[threadIdx.x]);
  }
  const uint64_t tiles = (n + kRouteTile - 1) / kRouteTile;
  for (uint64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    if (threadIdx.x < kMaxWorld) local[threadIdx.x] = 0;
    __syncthreads();
    uint64_t key[kRouteKeysPerThread];
    uint32_t owner[kRouteKeysPerThread], rank[kRouteKeysPerThread];
#pragma unroll
    for (int q = 0; q < kRouteKeysPerThread; ++q) {
      const uint64_t i = tile * kRouteTile + q * kBlock + threadIdx.x;
      key[q] = 0;
      owner[q] = 0;
      rank[q] = 0;
      const bool have = i < n;
      if (have) {
        key[q] = keys[i];
        owner[q] = owner_of(key[q], world);
      }
      // one shared-memory atomic per owner and warp, not per key: with few
      // ranks all keys of a tile would otherwise queue on a handful of counters
      const uint32_t same = __match_any_sync(0xFFFFFFFFu, have ? owner[q] : kMaxWorld);
      if (have) {
        const uint32_t lane = threadIdx.x & 31u;
        const uint32_t leader = __ffs(same) - 1;
        uint32_t first = 0;
        if (lane == leader) first = atomicAdd(&local[owner[q]], uint32_t(__popc(same)));
        first = __shfl_sync(same, first, leader);
        rank[q] = first + __popc(same & ((1u << lane) - 1u));
      }
    }
    __syncthreads();
    if (threadIdx.x < world && local[threadIdx.x]) {
      base[threadIdx.x] = atomicAdd(&cursors[threadIdx.x], (unsigned long long)local[threadIdx.x]);
    }
    if (threadIdx.x == 0) {
      uint32_t at = 0;
      for (uint32_t r = 0; r < world; ++r) {
        start[r] = at;
        at += local[r];
      }
    }
    __syncthreads();
#pragma unroll
    for (int q = 0; q < kRouteKeysPerThread; ++q) {
      const uint64_t i = tile * kRouteTile + q * kBlock + threadIdx.x;
      if (i < n) {
        const uint32_t pos = start[owner[q]] + rank[q];
        tile_keys[pos] = key[q];
        tile_origin[pos] = static_cast<uint32_t>(i);
        tile_owner[pos] = static_cast<uint8_t>(owner[q]);
      }
    }
    __syncthreads();
    const uint32_t in_tile =
        static_cast<uint32_t>(min(uint64_t(kRouteTile), n - tile * kRouteTile));
#pragma unroll
    for (int q = 0; q < kRouteKeysPerThread; ++q) {
      const uint32_t j = q * kBlock + threadIdx.x;
      if (j < in_tile) {
        const uint32_t o = tile_owner[j];
        const unsigned long long at =
            uint64_t(my_rank) * segment_capacity + base[o] + (j - start[o]);
        dst_keys[o][at] = tile_keys[j];
        dst_origin[o][at] = tile_origin[j];
      }
    }
    __syncthreads();
  }
}

// Tells every owner how many keys this rank put into its inbox.
__global__ void publish_counts_kernel(const unsigned long long* cursors, uint32_t world,
                                      uint32_t my_rank, const Peers inbox_counts) {
  if (threadIdx.x < world) {
    static_cast<unsigned long long*>(inbox_counts.p[threadIdx.x])[my_rank] = cursors[threadIdx.x];
  }
}

// Barrier between the ranks of one node over peer memory.  Thread p raises
// this rank's flag at peer p to `epoch` (system-scope release) and waits until
// peer p has raised its flag here (system-scope acquire).  The wait is bounded:
// when it runs out the kernel records kBarrierTimeout in *status and returns.
constexpr uint32_t kBarrierTimeout = 1u;
__global__ void barrier_kernel(uint32_t world, uint32_t my_rank, const Peers flags,
                               uint32_t epoch, uint32_t* status, uint32_t max_polls) {
  const uint32_t p = threadIdx.x;
  if (p >= world) return;
  uint32_t* theirs = static_cast<uint32_t*>(flags.p[p]) + my_rank;
  uint32_t* mine = static_cast<uint32_t*>(flags.p[my_rank]) + p;
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
  bool arrived = false;
  for (uint32_t poll = 0; poll < max_polls; ++poll) {
    uint32_t seen;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
    // epochs only grow; a wrapped difference keeps the comparison valid
    if (int32_t(seen - epoch) >= 0) {
      arrived = true;
      break;
    }
    __nanosleep(200);
  }
  if (!arrived) atomicOr(status, kBarrierTimeout);
  __threadfence_system();
}

// MODE 0: dst[i] = src[index[i]]   MODE 1: dst[index[i]] = src[i]
template <int VEC, int MODE>
__global__ void __launch_bounds__(kBlock)
    move_rows_kernel(uint64_t n, uint32_t chunks_per_row, const uint8_t* __restrict__ src,
                     const uint32_t* __restrict__ index, uint8_t* __restrict__ dst) {
  using T = typename hkv::VecType<VEC>::type;
  const uint64_t total = n * chunks_per_row;
  for (uint64_t c = uint64_t(blockIdx.x) * kBlock + threadIdx.x; c < total;
       c += uint64_t(gridDim.x) * kBlock) {
    const uint64_t row = c / chunks_per_row;
    const uint32_t off = static_cast<uint32_t>(c - row * chunks_per_row);
    const uint64_t other = index[row];
    if (MODE == 1 && other == 0xFFFFFFFFull) continue;  // "skip this row"
    const uint64_t s = (MODE == 0 ? other : row) * chunks_per_row + off;
    const uint64_t d = (MODE == 0 ? row : other) * chunks_per_row + off;
    reinterpret_cast<T*>(dst)[d] = reinterpret_cast<const T*>(src)[s];
  }
}

thread_local std::string g_shard_error;

int shard_fail(int code, const std::string& msg) {
  g_shard_error = msg;
  return code;
}

unsigned grid_for(uint64_t items) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const uint64_t want = (items + kBlock - 1) / kBlock;
  const uint64_t cap = uint64_t(sms) * 8;
  return static_cast<unsigned>(want < cap ? (want ? want : 1) : cap);
}

template <int MODE>
int move_rows(uint64_t n, uint64_t row_bytes, const void* src, const uint32_t* index, void* dst,
              cudaStream_t s) {
  if (n == 0 || row_bytes == 0) return HKV_OK;
  uint32_t vec = 16;
  while (vec > 1 && (row_bytes % vec != 0 || reinterpret_cast<uintptr_t>(src) % vec != 0 ||
                     reinterpret_cast<uintptr_t>(dst) % vec != 0)) {
    vec >>= 1;
  }
  const uint32_t cpr = static_cast<uint32_t>(row_bytes / vec);
  const unsigned grid = grid_for(n * cpr);
  const uint8_t* sp = static_cast<const uint8_t*>(src);
  uint8_t* dp = static_cast<uint8_t*>(dst);
  switch (vec) {
    case 16: move_rows_kernel<16, MODE><<<grid, kBlock, 0, s>>>(n, cpr, sp, index, dp); break;
    case 8: move_rows_kernel<8, MODE><<<grid, kBlock, 0, s>>>(n, cpr, sp, index, dp); break;
    case 4: move_rows_kernel<4, MODE><<<grid, kBlock, 0, s>>>(n, cpr, sp, index, dp); break;
    case 2: move_rows_kernel<2, MODE><<<grid, kBlock, 0, s>>>(n, cpr, sp, index, dp); break;
    default: move_rows_kernel<1, MODE><<<grid, kBlock, 0, s>>>(n, cpr, sp, index, dp); break;
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return shard_fail(HKV_ERR_CUDA, cudaGetErrorString(e));
  return HKV_OK;
}

}  // namespace

extern "C" {

const char* hkv_shard_last_error(void) { return g_shard_error.c_str(); }

int hkv_shard_partition(uint64_t n, const uint64_t* keys, uint32_t world, uint64_t* d_counts,
                        uint64_t* d_offsets, uint64_t* d_cursors, uint64_t* grouped_keys,
                        uint32_t* origin, hkv_stream stream) {
  if (world == 0 || world > kMaxWorld) {
    return shard_fail(HKV_ERR_INVALID_ARG, "world size must be between 1 and 64");
  }
  if (n >= (1ull << 32)) return shard_fail(HKV_ERR_INVALID_ARG, "batches above 2^32 keys");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(d_counts, 0, sizeof(uint64_t) * world, s);
  if (e != cudaSuccess) return shard_fail(HKV_ERR_CUDA, cudaGetErrorString(e));
  auto* counts = reinterpret_cast<unsigned long long*>(d_counts);
  auto* offsets = reinterpret_cast<unsigned long long*>(d_offsets);
  auto* cursors = reinterpret_cast<unsigned long long*>(d_cursors);
  if (n > 0) count_kernel<<<grid_for(n), kBlock, 0, s>>>(keys, n, world, counts);
  offsets_kernel<<<1, 32, 0, s>>>(counts, world, offsets, cursors);
  if (n > 0) place_kernel<<<grid_for(n), kBlock, 0, s>>>(keys, n, world, cursors, grouped_keys, origin);
  e = cudaGetLastError();
  if (e != cudaSuccess) return shard_fail(HKV_ERR_CUDA, cudaGetErrorString(e));
  return HKV_OK;
}

int hkv_shard_route_keys_p2p(uint64_t n, const uint64_t* keys, uint32_t world, uint32_t my_rank,
                             uint64_t segment_capacity, const hkv_peer_ptrs* inbox_keys,
                             const hkv_peer_ptrs* inbox_origin, const hkv_peer_ptrs* inbox_counts,
                             uint64_t* d_cursors, hkv_stream stream) {
  if (world == 0 || world > 16 || my_rank >= world) {
    return shard_fail(HKV_ERR_INVALID_ARG, "world size must be between 1 and 16");
  }
  if (n > segment_capacity || n >= (1ull << 32)) {
    return shard_fail(HKV_ERR_INVALID_ARG, "batch larger than an inbox segment");
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  Peers k{}, o{}, c{};
  for (uint32_t r = 0; r < world; ++r) {
    k.p[r] = inbox_keys->p[r];
    o.p[r] = inbox_origin->p[r];
    c.p[r] = inbox_counts->p[r];
  }
  cudaError_t e = cudaMemsetAsync(d_cursors, 0, sizeof(uint64_t) * world, s);
  if (e != cudaSuccess) return shard_fail(HKV_ERR_CUDA, cudaGetErrorString(e));
  auto* cursors = reinterpret_cast<unsigned long long*>(d_cursors);
  if (n > 0) {
    route_p2p_kernel<<<grid_for((n + kRouteKeysPerThread - 1) / kRouteKeysPerThread), kBlock, 0,
                       s>>>(keys, n, world, my_rank, segment_capacity, cursors, k, o);
  }
  publish_counts_kernel<<<1, 32, 0, s>>>(cursors, world, my_rank, c);
  e = cudaGetLastError();
  if (e != cudaSuccess) return shard_fail(HKV_ERR_CUDA, cudaGetErrorString(e));
  return HKV_OK;
}

int hkv_shard_barrier(uint32_t world, uint32_t my_rank, const hkv_peer_ptrs* flags, uint32_t epoch,
                      uint32_t* d_status, uint32_t max_polls, hkv_stream stream) {
  if (world == 0 || world > 16 || my_rank >= world) {
    return shard_fail(HKV_ERR_INVALID_ARG, "world size must be between 1 and 16");
  }
  Peers f{};
  for (uint32_t r = 0; r < world; ++r) f.p[r] = flags->p[r];
  barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(world, my_rank, f, epoch,
                                                                  d_status, max_polls);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return shard_fail(HKV_ERR_CUDA, cudaGetErrorString(e));
  return HKV_OK;
}

int hkv_shard_gather_rows(uint64_t n, uint64_t row_bytes, const void* src_rows,
                          const uint32_t* index, void* dst_rows, hkv_stream stream) {
  return move_rows<0>(n, row_bytes, src_rows, index, dst_rows, static_cast<cudaStream_t>(stream));
}

int hkv_shard_scatter_rows(uint64_t n, uint64_t row_bytes, const void* src_rows,
                           const uint32_t* index, void* dst_rows, hkv_stream stream) {
  return move_rows<1>(n, row_bytes, src_rows, index, dst_rows, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
