// Two (or more) processes, one per GPU, drive nv::merlin::ShardedHashTable --
// the C++ host of the key-hash sharded table -- and check every result against
// what one global table would hold.  The processes exchange the CUDA IPC
// handles of their workspaces through files in a directory the launcher
// (tests/test_sharded_cpp_gpu.py) gives them.
//
//   sharded_test <rank> <world> <exchange dir>
//
// Checked, bit for bit:
//   * insert_or_assign of every rank's own keys, then find of ALL ranks' keys
//     on every rank (pipelined over two lanes as well);
//   * find_or_insert of new keys that every rank sends with a row of its own:
//     the row of rank owner + 1 is stored and everybody gets it back;
//   * accum_or_assign of per-rank deltas for those keys: the stored row is
//     ((row + delta of rank owner + 1) + delta of rank owner + 2) + ... in fp32;
//   * the barrier status word stays 0.
#include <unistd.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <memory>
#include <string>
#include <vector>

#include "hkv_sharded.hpp"

using namespace nv::merlin;
using K = uint64_t;
using V = float;
using Table = HashTable<K, V, uint64_t, EvictStrategy::kLru>;
using Sharded = ShardedHashTable<K, V, uint64_t, EvictStrategy::kLru>;

#define REQUIRE(cond)                                                        \
  do {                                                                       \
    if (!(cond)) {                                                           \
      fprintf(stderr, "rank %d: FAILED %s (line %d)\n", g_rank, #cond, __LINE__); \
      exit(1);                                                               \
    }                                                                        \
  } while (0)

static int g_rank = 0;
constexpr int kDim = 8;

static uint64_t mix(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return (z ^ (z >> 31)) >> 2;   // never a reserved key
}
static uint64_t fmix64(uint64_t k) {
  k ^= k >> 33; k *= 0xff51afd7ed558ccdull; k ^= k >> 33; k *= 0xc4ceb9fe1a85ec53ull; k ^= k >> 33;
  return k;
}
// column j of the row rank r supplies for `key` in phase `what`
static float cell(uint64_t key, int r, int what, int j) {
  return float((key >> 7) % 1000) * 0.25f + float(r) * 16.0f + float(what) * 1024.0f + float(j);
}
static float delta(uint64_t key, int r, int j) {
  return (float((key >> 3) % 97) + 1.0f) * 0.001f * float(r + 1) + float(j) * 0.0001f;
}

static void file_barrier(const std::string& dir, const std::string& tag, int rank, int world) {
  { std::ofstream f(dir + "/" + tag + "." + std::to_string(rank)); f << "x"; }
  for (int r = 0; r < world; ++r) {
    const std::string p = dir + "/" + tag + "." + std::to_string(r);
    for (int tries = 0; access(p.c_str(), F_OK) != 0; ++tries) {
      if (tries > 60000) { fprintf(stderr, "rank %d: peer %d never arrived at %s\n", rank, r, tag.c_str()); exit(2); }
      usleep(1000);
    }
  }
}

int main(int argc, char** argv) {
  if (argc < 4) { fprintf(stderr, "usage: sharded_test <rank> <world> <dir>\n"); return 1; }
  const int rank = g_rank = atoi(argv[1]), world = atoi(argv[2]);
  const std::string dir = argv[3];
  CUDA_CHECK(cudaSetDevice(rank));
  HashTableOptions o;
  o.init_capacity = o.max_capacity = 128 * 512;
  o.max_hbm_for_vectors = size_t(1) << 30;
  o.dim = kDim;
  Table local;
  local.init(o);
  const uint64_t per = 4000, shared = 1500, max_batch = per * world + shared;
  // "external" (one rank): the caller allocates the workspaces and the
  // library adopts them instead of allocating and exporting its own
  const bool external = argc > 4 && std::string(argv[4]) == "external";
  std::vector<void*> own_workspaces;
  if (external) {
    REQUIRE(world == 1);
    const uint64_t bytes = Sharded::workspace_bytes(&local, world, max_batch);
    REQUIRE(bytes > max_batch * kDim * sizeof(V));
    for (int lane = 0; lane < 2; ++lane) {
      void* w = nullptr;
      CUDA_CHECK(cudaMalloc(&w, bytes));
      own_workspaces.push_back(w);
    }
  }
  std::unique_ptr<Sharded> table_owner(external
                                           ? new Sharded(&local, world, rank, max_batch, own_workspaces)
                                           : new Sharded(&local, world, rank, max_batch, 2));
  Sharded& table = *table_owner;
  if (external) {
    hkv_ipc_handle none;
    REQUIRE(hkv_sharded_ipc_handle(table.native_handle(), 0, &none) != HKV_OK);  // not the library's to export
    REQUIRE(table.rows(0) != nullptr && table.lanes() == 2);
  }

  // exchange the workspaces' IPC handles through files
  for (uint32_t lane = 0; !external && lane < table.lanes(); ++lane) {
    const hkv_ipc_handle h = table.ipc_handle(lane);
    std::ofstream f(dir + "/handle." + std::to_string(lane) + "." + std::to_string(rank) + ".tmp", std::ios::binary);
    f.write(reinterpret_cast<const char*>(&h), sizeof(h));
    f.close();
    rename((dir + "/handle." + std::to_string(lane) + "." + std::to_string(rank) + ".tmp").c_str(),
           (dir + "/handle." + std::to_string(lane) + "." + std::to_string(rank)).c_str());
  }
  file_barrier(dir, "handles", rank, world);
  for (uint32_t lane = 0; !external && lane < table.lanes(); ++lane) {
    std::vector<hkv_ipc_handle> all(world);
    for (int r = 0; r < world; ++r) {
      std::ifstream f(dir + "/handle." + std::to_string(lane) + "." + std::to_string(r), std::ios::binary);
      f.read(reinterpret_cast<char*>(&all[r]), sizeof(hkv_ipc_handle));
      REQUIRE(f.gcount() == sizeof(hkv_ipc_handle));
    }
    table.connect(lane, all);
  }
  file_barrier(dir, "connected", rank, world);

  auto own_key = [&](int r, uint64_t i) { return mix(uint64_t(r) * 1000003ull + i); };
  K* d_keys;
  CUDA_CHECK(cudaMalloc(&d_keys, max_batch * sizeof(K)));
  std::vector<K> h_keys(max_batch);
  std::vector<V> h_rows(max_batch * kDim);
  std::vector<char> h_flags(max_batch);
  auto upload_keys = [&](uint64_t n) { CUDA_CHECK(cudaMemcpy(d_keys, h_keys.data(), n * sizeof(K), cudaMemcpyHostToDevice)); };
  auto upload_rows = [&](uint64_t n) { CUDA_CHECK(cudaMemcpy(table.rows(0), h_rows.data(), n * kDim * sizeof(V), cudaMemcpyHostToDevice)); };
  auto download = [&](uint32_t lane, uint64_t n) {
    CUDA_CHECK(cudaMemcpy(h_rows.data(), table.rows(lane), n * kDim * sizeof(V), cudaMemcpyDeviceToHost));
    CUDA_CHECK(cudaMemcpy(h_flags.data(), table.flags(lane), n, cudaMemcpyDeviceToHost));
  };

  // 1. every rank inserts its own keys
  for (uint64_t i = 0; i < per; ++i) {
    h_keys[i] = own_key(rank, i);
    for (int j = 0; j < kDim; ++j) h_rows[i * kDim + j] = cell(h_keys[i], rank, 0, j);
  }
  upload_keys(per);
  upload_rows(per);
  table.insert_or_assign(per, d_keys);
  CUDA_CHECK(cudaDeviceSynchronize());
  file_barrier(dir, "inserted", rank, world);

  // 2. every rank looks up all ranks' keys and some that nobody inserted
  uint64_t n = 0;
  for (int r = 0; r < world; ++r)
    for (uint64_t i = 0; i < per; ++i) h_keys[n++] = own_key(r, i);
  for (uint64_t i = 0; i < shared; ++i) h_keys[n++] = mix(900000007ull + i);
  upload_keys(n);
  CUDA_CHECK(cudaMemset(table.rows(0), 0xFF, n * kDim * sizeof(V)));
  table.find(n, d_keys);
  CUDA_CHECK(cudaDeviceSynchronize());
  download(0, n);
  for (uint64_t i = 0; i < n; ++i) {
    const bool want = i < per * world;
    REQUIRE(bool(h_flags[i]) == want);
    if (want)
      for (int j = 0; j < kDim; ++j) REQUIRE(h_rows[i * kDim + j] == cell(h_keys[i], int(i / per), 0, j));
  }
  // the same lookups pipelined over both lanes: batch k + 1 is issued before batch k is waited for
  uint32_t used[4];
  for (int b = 0; b < 4; ++b) {
    used[b] = table.find_async(n - 64 * b, d_keys + 64 * b);
    if (b > 0) {
      table.wait(used[b - 1]);
      CUDA_CHECK(cudaStreamSynchronize(0));
      download(used[b - 1], n - 64 * (b - 1));
      for (uint64_t i = 0; i + 64 * (b - 1) < per * world; i += 37) {
        REQUIRE(h_flags[i]);
        REQUIRE(h_rows[i * kDim + 3] == cell(h_keys[i + 64 * (b - 1)], int((i + 64 * (b - 1)) / per), 0, 3));
      }
    }
  }
  table.wait(used[3]);
  CUDA_CHECK(cudaDeviceSynchronize());
  file_barrier(dir, "found", rank, world);

  // 3. find_or_insert: new keys every rank sends, each with a row of its own
  for (uint64_t i = 0; i < shared; ++i) {
    h_keys[i] = mix(900000007ull + i);
    for (int j = 0; j < kDim; ++j) h_rows[i * kDim + j] = cell(h_keys[i], rank, 1, j);
  }
  upload_keys(shared);
  upload_rows(shared);
  table.find_or_insert(shared, d_keys);
  CUDA_CHECK(cudaDeviceSynchronize());
  download(0, shared);
  std::vector<V> expect(shared * kDim);
  for (uint64_t i = 0; i < shared; ++i) {
    const int first = int((fmix64(h_keys[i]) % uint64_t(world) + 1) % uint64_t(world));
    for (int j = 0; j < kDim; ++j) {
      expect[i * kDim + j] = cell(h_keys[i], first, 1, j);
      REQUIRE(h_rows[i * kDim + j] == expect[i * kDim + j]);
    }
  }
  file_barrier(dir, "inserted2", rank, world);

  // 4. accum_or_assign of per-rank deltas for the same keys (routing reused)
  for (uint64_t i = 0; i < shared; ++i)
    for (int j = 0; j < kDim; ++j) h_rows[i * kDim + j] = delta(h_keys[i], rank, j);
  upload_rows(shared);
  CUDA_CHECK(cudaMemset(table.flags(0), 1, shared));
  table.accum_or_assign(shared, d_keys, 0, true);
  CUDA_CHECK(cudaDeviceSynchronize());
  file_barrier(dir, "accumulated", rank, world);
  table.find(shared, d_keys);
  CUDA_CHECK(cudaDeviceSynchronize());
  download(0, shared);
  for (uint64_t i = 0; i < shared; ++i) {
    const int owner = int(fmix64(h_keys[i]) % uint64_t(world));
    REQUIRE(h_flags[i]);
    for (int j = 0; j < kDim; ++j) {
      volatile float v = expect[i * kDim + j];
      for (int t = 1; t <= world; ++t) v = v + delta(h_keys[i], (owner + t) % world, j);
      REQUIRE(h_rows[i * kDim + j] == v);
    }
  }
  REQUIRE(table.status(0) == 0 && table.status(1) == 0);
  file_barrier(dir, "done", rank, world);
  table_owner.reset();  // the library never frees workspaces it did not allocate
  for (void* w : own_workspaces) CUDA_CHECK(cudaFree(w));
  printf("rank %d PASS\n", rank);
  return 0;
}
