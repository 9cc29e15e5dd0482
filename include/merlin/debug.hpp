// Error convention of the drop-in boundary: the two exception types and the
// two check macros client code of nv::merlin::HashTable relies on
// (reference: include/merlin/debug.hpp:27-72).
#pragma once

#include <cuda_runtime_api.h>

#include <stdexcept>
#include <string>

namespace nv {
namespace merlin {

class CudaException : public std::runtime_error {
 public:
  explicit CudaException(const std::string& what) : std::runtime_error(what) {}
};

class MerlinException : public std::runtime_error {
 public:
  explicit MerlinException(const std::string& what) : std::runtime_error(what) {}
};

namespace detail {

inline std::string where(const char* file, int line) {
  return std::string(file) + ':' + std::to_string(line) + ": ";
}

inline void throw_if_cuda_failed(cudaError_t status, const char* file, int line) {
  if (status == cudaSuccess) return;
  throw CudaException(where(file, line) + "CUDA error " + cudaGetErrorName(status) + " (#" +
                      std::to_string(static_cast<int>(status)) + "): " +
                      cudaGetErrorString(status));
}

inline void throw_unless(bool ok, const std::string& message, const char* file, int line) {
  if (ok) return;
  throw MerlinException(where(file, line) + "HierarchicalKV error " + message);
}

}  // namespace detail
}  // namespace merlin
}  // namespace nv

#ifndef CUDA_CHECK
#define CUDA_CHECK(status) \
  ::nv::merlin::detail::throw_if_cuda_failed((status), __FILE__, __LINE__)
#endif

#ifndef MERLIN_CHECK
#define MERLIN_CHECK(condition, message) \
  ::nv::merlin::detail::throw_unless((condition), (message), __FILE__, __LINE__)
#endif
