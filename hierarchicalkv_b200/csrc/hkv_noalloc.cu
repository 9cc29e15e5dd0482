// hkv_size_no_alloc: the table's size computed without allocating anything.
//
// Who this is for: code that runs after a process has finished its set-up
// phase and is no longer allowed to allocate -- a serving loop with a memory
// budget fixed at start-up, a plug-in whose host application owns every
// allocation, a monitoring thread that must not trigger the implicit
// device-wide synchronisation cudaMalloc and cudaFree bring with them.  The
// regular hkv_size keeps its partial result in scratch memory that belongs to
// the table; this variant keeps its partial sums in a fixed array that is part
// of the library image, so the call itself never asks CUDA (or any library
// that allocates, torch included) for device memory.  On the host side the
// table's API lock may create one CUDA event the first time it sees a stream,
// and a failing call builds its error message as a std::string.
//
// The price is a fixed ceiling: the array has room for one partial sum per
// 1024 buckets of a table with at most kNoAllocMaxBuckets buckets.  Every GPU
// that loads the library carries the array (32 KiB + 256 B) until the process
// exits.
#include <cuda_runtime.h>

#include <mutex>
#include <string>

#include "../../include/hkv_b200.h"

namespace {

constexpr int kBucketsPerBlock = 1024;
constexpr int kNoAllocMaxBlocks = 4096;
constexpr unsigned long long kNoAllocMaxBuckets =
    (unsigned long long)kBucketsPerBlock * kNoAllocMaxBlocks;  // 4,194,304 buckets = 2^29 slots
constexpr int kMaxDevices = 64;

// [0, kNoAllocMaxBlocks): one partial sum per block; [kNoAllocMaxBlocks]: total.
// Nothing in it has to start at zero: each call writes every element it later
// reads.  All calls share it, so two calls that overlap on the GPU race.
static __device__ __align__(256) unsigned long long g_size_scratch[kNoAllocMaxBlocks + 32];

// In host code `g_size_scratch` is only a handle; the device address is
// fetched once per device, with that device current.
unsigned long long* g_scratch_addr[kMaxDevices] = {};
std::mutex g_setup_mutex;

thread_local std::string g_noalloc_error;

__global__ void __launch_bounds__(256)
    size_partials_kernel(const int32_t* __restrict__ bucket_sizes, unsigned long long buckets,
                         unsigned long long* __restrict__ partials) {
  __shared__ unsigned long long warp_sums[8];
  const unsigned long long first = (unsigned long long)blockIdx.x * kBucketsPerBlock;
  unsigned long long local = 0;
  for (int k = threadIdx.x; k < kBucketsPerBlock; k += 256) {
    const unsigned long long b = first + k;
    if (b < buckets) local += (unsigned long long)bucket_sizes[b];
  }
  for (int o = 16; o > 0; o >>= 1) local += __shfl_down_sync(0xFFFFFFFFu, local, o);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = local;
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long total = 0;
    for (int w = 0; w < 8; ++w) total += warp_sums[w];
    partials[blockIdx.x] = total;
  }
}

__global__ void __launch_bounds__(256)
    size_total_kernel(const unsigned long long* __restrict__ partials, int blocks,
                      unsigned long long* __restrict__ total_out) {
  __shared__ unsigned long long warp_sums[8];
  unsigned long long local = 0;
  for (int k = threadIdx.x; k < blocks; k += 256) local += partials[k];
  for (int o = 16; o > 0; o >>= 1) local += __shfl_down_sync(0xFFFFFFFFu, local, o);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = local;
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long total = 0;
    for (int w = 0; w < 8; ++w) total += warp_sums[w];
    *total_out = total;
  }
}

int fail(int code, const std::string& msg) {
  g_noalloc_error = msg;
  return code;
}

}  // namespace

extern "C" {

const char* hkv_size_no_alloc_last_error(void) { return g_noalloc_error.c_str(); }

int hkv_size_no_alloc(hkv_table* table, hkv_stream stream, uint64_t* size) {
  if (table == nullptr || size == nullptr) {
    return fail(HKV_ERR_INVALID_ARG, "hkv_size_no_alloc: table and size must not be null");
  }
  // The reader lock comes first: a doubling of the table on another thread
  // replaces (and frees) the planes the view points at, and it cannot run
  // between hkv_external_begin and hkv_external_end.
  if (hkv_external_begin(table, 0, stream) != HKV_OK) {
    return fail(HKV_ERR_RUNTIME, "hkv_size_no_alloc: cannot join the table's readers");
  }
  int rc = HKV_OK;
  int previous = -1;
  int device = -1;
  unsigned long long* scratch = nullptr;
  hkv_table_view view{};
  if (hkv_get_view(table, &view) != HKV_OK) {
    rc = fail(HKV_ERR_RUNTIME, "hkv_size_no_alloc: cannot read the table's view");
  } else if (view.buckets > kNoAllocMaxBuckets) {
    rc = fail(HKV_ERR_INVALID_ARG,
              "hkv_size_no_alloc: the table has " + std::to_string(view.buckets) +
                  " buckets, the fixed scratch array serves at most " +
                  std::to_string(kNoAllocMaxBuckets) + "; use hkv_size");
  }
  cudaError_t e = cudaSuccess;
  if (rc == HKV_OK) {
    cudaPointerAttributes attr{};
    e = cudaPointerGetAttributes(&attr, view.bucket_sizes);
    if (e != cudaSuccess || attr.device < 0 || attr.device >= kMaxDevices) {
      cudaGetLastError();
      rc = fail(HKV_ERR_CUDA, "hkv_size_no_alloc: cannot tell which device owns the table");
    } else {
      device = attr.device;
      cudaGetDevice(&previous);
      if (previous != device) cudaSetDevice(device);
    }
  }
  if (rc == HKV_OK) {
    // first call on this device: resolve the array's device address
    std::lock_guard<std::mutex> guard(g_setup_mutex);
    if (g_scratch_addr[device] == nullptr) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_size_scratch);
      if (e != cudaSuccess || p == nullptr) {
        cudaGetLastError();
        rc = fail(HKV_ERR_CUDA, std::string("hkv_size_no_alloc: cudaGetSymbolAddress: ") +
                                    cudaGetErrorString(e));
      } else {
        g_scratch_addr[device] = static_cast<unsigned long long*>(p);
      }
    }
    scratch = g_scratch_addr[device];
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (rc == HKV_OK) {
    const int blocks = static_cast<int>((view.buckets + kBucketsPerBlock - 1) / kBucketsPerBlock);
    size_partials_kernel<<<blocks, 256, 0, s>>>(view.bucket_sizes, view.buckets, scratch);
    size_total_kernel<<<1, 256, 0, s>>>(scratch, blocks, scratch + kNoAllocMaxBlocks);
    e = cudaGetLastError();
    if (e != cudaSuccess) {
      rc = fail(HKV_ERR_CUDA, std::string("hkv_size_no_alloc: launch: ") + cudaGetErrorString(e));
    }
  }
  // every path leaves the readers again; the kernels above are ordered before
  // whatever an inserter enqueues afterwards
  if (hkv_external_end(table, 0, stream) != HKV_OK && rc == HKV_OK) {
    rc = fail(HKV_ERR_RUNTIME, "hkv_size_no_alloc: cannot leave the table's readers");
  }
  if (rc == HKV_OK) {
    unsigned long long host_total = 0;
    e = cudaMemcpyAsync(&host_total, scratch + kNoAllocMaxBlocks, sizeof(host_total),
                        cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) {
      rc = fail(HKV_ERR_CUDA, std::string("hkv_size_no_alloc: ") + cudaGetErrorString(e));
    } else {
      *size = host_total;
    }
  }
  if (previous >= 0 && previous != device) cudaSetDevice(previous);
  return rc;
}

}  // extern "C"
