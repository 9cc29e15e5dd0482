// Allocator interface of the drop-in boundary (reference:
// include/merlin/allocator.cuh:27-59).  HashTable::init borrows a
// BaseAllocator*; the table's storage is requested through it.
#pragma once

#include <cuda_runtime.h>

#include <cstdlib>

#include "debug.hpp"

namespace nv {
namespace merlin {

enum MemoryType {
  Device,   // HBM
  Pinned,   // pinned (optionally mapped) host memory
  Host,     // pageable host memory
  Managed,  // unused
};

class BaseAllocator {
 public:
  BaseAllocator() = default;
  virtual ~BaseAllocator() = default;
  BaseAllocator(const BaseAllocator&) = delete;
  BaseAllocator& operator=(const BaseAllocator&) = delete;
  BaseAllocator(BaseAllocator&&) = delete;
  BaseAllocator& operator=(BaseAllocator&&) = delete;

  virtual void alloc(const MemoryType type, void** ptr, size_t size,
                     unsigned int pinned_flags = cudaHostAllocDefault) = 0;
  virtual void alloc_async(const MemoryType type, void** ptr, size_t size,
                           cudaStream_t stream) = 0;
  virtual void free(const MemoryType type, void* ptr) = 0;
  virtual void free_async(const MemoryType type, void* ptr, cudaStream_t stream) = 0;
};

class DefaultAllocator : public virtual BaseAllocator {
 public:
  DefaultAllocator() = default;
  ~DefaultAllocator() override = default;

  void alloc(const MemoryType type, void** ptr, size_t size,
             unsigned int pinned_flags = cudaHostAllocDefault) override {
    if (type == MemoryType::Device) {
      CUDA_CHECK(cudaMalloc(ptr, size));
    } else if (type == MemoryType::Pinned) {
      CUDA_CHECK(cudaHostAlloc(ptr, size, pinned_flags));
    } else {
      *ptr = std::malloc(size);
      MERLIN_CHECK(*ptr != nullptr, "host allocation failed");
    }
  }

  void alloc_async(const MemoryType type, void** ptr, size_t size, cudaStream_t stream) override {
    if (type == MemoryType::Device) {
      CUDA_CHECK(cudaMallocAsync(ptr, size, stream));
    } else {
      MERLIN_CHECK(false, "[DefaultAllocator] only device memory can be allocated asynchronously");
    }
  }

  void free(const MemoryType type, void* ptr) override {
    if (ptr == nullptr) return;
    if (type == MemoryType::Device) {
      CUDA_CHECK(cudaFree(ptr));
    } else if (type == MemoryType::Pinned) {
      CUDA_CHECK(cudaFreeHost(ptr));
    } else {
      std::free(ptr);
    }
  }

  void free_async(const MemoryType type, void* ptr, cudaStream_t stream) override {
    if (ptr == nullptr) return;
    if (type == MemoryType::Device) {
      CUDA_CHECK(cudaFreeAsync(ptr, stream));
    } else {
      MERLIN_CHECK(false, "[DefaultAllocator] only device memory can be freed asynchronously");
    }
  }
};

}  // namespace merlin
}  // namespace nv
