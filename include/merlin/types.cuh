// Types client code of nv::merlin::HashTable names directly: the reserved
// key constants, the file interface of save/load and the architecture tags
// (reference: include/merlin/types.cuh:47-66, 242-281, 300-330).  The
// table's storage structs are private to the library and not declared here.
#pragma once

#include <cstddef>
#include <cstdint>

namespace nv {
namespace merlin {

constexpr uint64_t DEFAULT_EMPTY_KEY = UINT64_C(0xFFFFFFFFFFFFFFFF);
constexpr uint64_t DEFAULT_RECLAIM_KEY = UINT64_C(0xFFFFFFFFFFFFFFFE);
constexpr uint64_t DEFAULT_LOCKED_KEY = UINT64_C(0xFFFFFFFFFFFFFFFD);
constexpr uint64_t DEFAULT_RESERVED_KEY_MASK = UINT64_C(0xFFFFFFFFFFFFFFFC);
constexpr uint64_t MAX_SCORE = UINT64_C(0xFFFFFFFFFFFFFFFF);
constexpr uint64_t EMPTY_SCORE = UINT64_C(0);
constexpr uint64_t IGNORED_GLOBAL_EPOCH = UINT64_C(0xFFFFFFFFFFFFFFFF);
constexpr int MAX_RESERVED_KEY_BIT = 62;

// Abstract key/value/score file used by HashTable::save and ::load.
template <class K, class V, class S>
class BaseKVFile {
 public:
  virtual ~BaseKVFile() {}
  // Fills the buffers with up to n tuples; returns how many were read.
  virtual size_t read(const size_t n, const size_t dim, K* keys, V* vectors, S* scores) = 0;
  // Appends n tuples; returns how many were written.
  virtual size_t write(const size_t n, const size_t dim, const K* keys, const V* vectors,
                       const S* scores) = 0;
};

// Architecture tags.  The reference uses them to pick A100/V100 tuning
// thresholds; this library is built for sm_100a only and ignores the tag.
struct Sm70 {
  static constexpr int kComputeCapability = 70;
};
struct Sm80 {
  static constexpr int kComputeCapability = 80;
};
struct Sm90 {
  static constexpr int kComputeCapability = 90;
};
struct Sm100 {
  static constexpr int kComputeCapability = 100;
};

}  // namespace merlin
}  // namespace nv
