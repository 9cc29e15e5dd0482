// TEST INFRASTRUCTURE ONLY.
//
// Host-only program over the reference's own headers: prints, as JSON, the
// values the reference's HOST functions compute, so the CPU oracle can be
// pinned without a GPU:
//   * Murmur3HashHost (include/merlin/utils.cuh:127-135) for a fixed key list;
//   * the EMPTY key init_reserved_keys derives for reserved_key_start_bit
//     0..62 (include/merlin/types.cuh:80-96, read back from EMPTY_KEY_CPU; the
//     copy to __constant__ memory that follows needs a GPU and is allowed to
//     fail here).
// Built by `make -C oracle ref`; its output is committed as
// tests/golden/host_pins.json.
#include <cstdint>
#include <cstdio>

#include "merlin/types.cuh"
#include "merlin/utils.cuh"

int main() {
  const uint64_t keys[] = {0ull,
                           1ull,
                           2ull,
                           42ull,
                           127ull,
                           128ull,
                           0xFFFFFFFFull,
                           0x100000000ull,
                           0x0123456789ABCDEFull,
                           0xDEADBEEFCAFEBABEull,
                           0x8000000000000000ull,
                           0xFFFFFFFFFFFFFFFBull,
                           0xFFFFFFFFFFFFFFFCull,
                           0xFFFFFFFFFFFFFFFDull,
                           0xFFFFFFFFFFFFFFFEull,
                           0xFFFFFFFFFFFFFFFFull};
  std::printf("{\n  \"murmur3_host\": {");
  const int nk = int(sizeof(keys) / sizeof(keys[0]));
  for (int i = 0; i < nk; ++i) {
    std::printf("%s\"%llu\": \"%llu\"", i ? ", " : "", (unsigned long long)keys[i],
                (unsigned long long)nv::merlin::Murmur3HashHost(keys[i]));
  }
  std::printf("},\n  \"empty_key_by_start_bit\": [");
  for (int bit = 0; bit <= 62; ++bit) {
    nv::merlin::EMPTY_KEY_CPU = nv::merlin::DEFAULT_EMPTY_KEY;
    try {
      nv::merlin::init_reserved_keys(bit);
    } catch (...) {
      // no GPU: the host-side value was stored before the device copy
    }
    std::printf("%s\"%llu\"", bit ? ", " : "", (unsigned long long)nv::merlin::EMPTY_KEY_CPU);
  }
  std::printf("]\n}\n");
  return 0;
}
