// Checkpoint tool for the cross-implementation test of save / load
// (tests/test_checkpoint_gpu.py): a client of the drop-in header that
//   save <prefix> <capacity> <dim> <n> <seed> <score_bytes>
//       fills a Customized table with n seeded keys and saves it with
//       LocalKVFile to <prefix>.keys / .values / .scores
//   load <prefix> <capacity> <dim> <out_prefix> <score_bytes>
//       loads those three files into an empty table and writes the table's
//       export to <out_prefix>.keys / .values / .scores the same way
// The file format is the reference's: three raw little-endian arrays, no
// header (include/merlin_localfile.hpp:44-158 of the reference).
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "merlin_hashtable.cuh"
#include "merlin_localfile.hpp"

using namespace nv::merlin;

static uint64_t mix(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

template <class S>
int run(int argc, char** argv) {
  using Table = HashTable<uint64_t, float, S, EvictStrategy::kCustomized>;
  const std::string mode = argv[1];
  const std::string prefix = argv[2];
  const size_t capacity = strtoull(argv[3], nullptr, 10);
  const size_t dim = strtoull(argv[4], nullptr, 10);
  HashTableOptions o;
  o.init_capacity = capacity;
  o.max_capacity = capacity;
  o.max_hbm_for_vectors = size_t(1) << 30;
  o.dim = dim;
  Table table;
  table.init(o);
  LocalKVFile<uint64_t, float, S> file;
  if (mode == "save") {
    const size_t n = strtoull(argv[5], nullptr, 10);
    const uint64_t seed = strtoull(argv[6], nullptr, 10);
    std::vector<uint64_t> keys(n);
    std::vector<S> scores(n);
    std::vector<float> values(n * dim);
    for (size_t i = 0; i < n; ++i) {
      keys[i] = mix(seed * 1000003ull + i) >> 2;   // never a reserved key
      scores[i] = static_cast<S>(1000 + i);
      for (size_t j = 0; j < dim; ++j) values[i * dim + j] = float(keys[i] % 1000003ull) + float(j);
    }
    uint64_t* d_keys;
    S* d_scores;
    float* d_values;
    cudaMalloc(&d_keys, n * 8);
    cudaMalloc(&d_scores, n * sizeof(S));
    cudaMalloc(&d_values, n * dim * 4);
    cudaMemcpy(d_keys, keys.data(), n * 8, cudaMemcpyHostToDevice);
    cudaMemcpy(d_scores, scores.data(), n * sizeof(S), cudaMemcpyHostToDevice);
    cudaMemcpy(d_values, values.data(), n * dim * 4, cudaMemcpyHostToDevice);
    table.insert_or_assign(n, d_keys, d_values, d_scores);
    cudaDeviceSynchronize();
    if (!file.open(prefix + ".keys", prefix + ".values", prefix + ".scores", "wb")) return 2;
    // a small workspace: the table is written in many chunks
    const size_t saved = table.save(&file, 64 * 1024);
    file.close();
    printf("saved %zu of %zu\n", saved, table.size());
    return saved == table.size() ? 0 : 3;
  }
  if (mode == "load") {
    const std::string out = argv[5];
    if (!file.open(prefix + ".keys", prefix + ".values", prefix + ".scores", "rb")) return 2;
    const size_t loaded = table.load(&file, 48 * 1024);
    file.close();
    LocalKVFile<uint64_t, float, S> dump;
    if (!dump.open(out + ".keys", out + ".values", out + ".scores", "wb")) return 2;
    const size_t saved = table.save(&dump);
    dump.close();
    printf("loaded %zu, table holds %zu, exported %zu\n", loaded, table.size(), saved);
    return saved == table.size() ? 0 : 3;
  }
  return 1;
}

int main(int argc, char** argv) {
  if (argc < 7) {
    fprintf(stderr, "usage: ckpt_tool save|load <prefix> <capacity> <dim> ... <score_bytes>\n");
    return 1;
  }
  const int score_bytes = atoi(argv[argc - 1]);
  try {
    return score_bytes == 4 ? run<uint32_t>(argc, argv) : run<uint64_t>(argc, argv);
  } catch (const std::exception& e) {
    fprintf(stderr, "ckpt_tool: %s\n", e.what());
    return 4;
  }
}
