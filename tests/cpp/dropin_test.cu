// A client of nv::merlin::HashTable written against the reference's API,
// compiled against THIS repository's include/merlin_hashtable.cuh.  The checks
// restate invariants of the reference's own tests:
//   * value[j] == float(key * 0.00001), score == key      tests/test_util.cuh:155-166
//   * size arithmetic around insert / erase / clear, export count == size
//                                                        tests/merlin_hashtable_test.cc.cu:242-344,388-392
//   * insert_and_evict conservation                      tests/insert_and_evict_test.cc.cu:87-153
//   * export_batch_if with a user functor                tests/export_batch_if_test.cc.cu:129-300
//   * save / load round trip                             tests/save_and_load_test.cc.cu:31-105
// Prints PASS and exits 0 when every check holds.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <memory>
#include <numeric>
#include <set>
#include <string>
#include <vector>

#include "merlin_hashtable.cuh"
#include "merlin_localfile.hpp"

using K = uint64_t;
using V = float;
using S = uint64_t;
using nv::merlin::EvictStrategy;
using nv::merlin::HashTableOptions;

#define EXPECT(cond)                                                        \
  do {                                                                      \
    if (!(cond)) {                                                          \
      std::printf("FAIL %s:%d: %s\n", __FILE__, __LINE__, #cond);           \
      std::exit(1);                                                         \
    }                                                                       \
  } while (0)

template <class K_, class S_>
struct ScoreBelow {
  __forceinline__ __device__ bool operator()(const K_& key, S_& score, const K_& pattern,
                                             const S_& threshold) {
    return score < threshold;
  }
};

// Functors of the forms export_batch_if_v2 / erase_if_v2 / for_each take
// (tests/export_batch_if_test.cc.cu:34-130 of the reference shows the shapes).
// ScoreBelowAndRowIntact checks the score alone, then lets the tile verify the
// selected rows together: every element must equal float(key * 1e-5).
template <class K_, class V_, class S_>
struct ScoreBelowAndRowIntact {
  S_ threshold;
  int dim;
  template <int GroupSize>
  __forceinline__ __device__ bool operator()(const K_& key, const V_* value, const S_& score,
                                             cg::thread_block_tile<GroupSize>& g) {
    bool keep = score < threshold;
    for (int r = 0; r < GroupSize; ++r) {
      const bool r_keep = g.shfl(keep, r);
      if (!r_keep) continue;
      const V_* row = g.shfl(value, r);
      const V_ want = static_cast<V_>(g.shfl(key, r) * 0.00001);
      bool bad = false;
      for (int j = g.thread_rank(); j < dim; j += GroupSize) bad |= row[j] != want;
      if (g.any(bad) && g.thread_rank() == r) keep = false;
    }
    return keep;
  }
};

// for_each body: rows of keys with score < threshold are negated by the tile
// and their score is raised by one.
template <class K_, class V_, class S_>
struct NegateRowsBelow {
  S_ threshold;
  int dim;
  template <int GroupSize>
  __forceinline__ __device__ void operator()(const K_& key, V_* value, S_* score,
                                             cg::thread_block_tile<GroupSize>& g) {
    // empty slots and tombstones are visited too
    const bool hit = (key & 0xFFFFFFFFFFFFFFFCull) != 0xFFFFFFFFFFFFFFFCull && *score < threshold;
    for (int r = 0; r < GroupSize; ++r) {
      if (!g.shfl(hit, r)) continue;
      V_* row = g.shfl(value, r);
      for (int j = g.thread_rank(); j < dim; j += GroupSize) row[j] = -row[j];
    }
    if (hit) *score += 1;
  }
};

template <class T>
struct DeviceBuffer {
  T* p = nullptr;
  size_t n = 0;
  explicit DeviceBuffer(size_t count) : n(count) { CUDA_CHECK(cudaMalloc(&p, sizeof(T) * count)); }
  ~DeviceBuffer() { cudaFree(p); }
  void upload(const std::vector<T>& h) {
    CUDA_CHECK(cudaMemcpy(p, h.data(), sizeof(T) * h.size(), cudaMemcpyHostToDevice));
  }
  std::vector<T> download(size_t count) const {
    std::vector<T> h(count);
    CUDA_CHECK(cudaMemcpy(h.data(), p, sizeof(T) * count, cudaMemcpyDeviceToHost));
    return h;
  }
};

static uint64_t mix(uint64_t x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

static void make_batch(uint64_t first, size_t n, size_t dim, std::vector<K>& keys,
                       std::vector<V>& values, std::vector<S>& scores) {
  keys.resize(n);
  scores.resize(n);
  values.resize(n * dim);
  for (size_t i = 0; i < n; ++i) {
    keys[i] = mix(first + i) >> 8;  // never a reserved key
    scores[i] = keys[i];
    for (size_t j = 0; j < dim; ++j) values[i * dim + j] = static_cast<float>(keys[i] * 0.00001);
  }
}

static void test_basic() {
  constexpr size_t kDim = 16, kCap = 128 * 1024, kN = 32 * 1024;
  using Table = nv::merlin::HashTable<K, V, S, EvictStrategy::kCustomized>;
  HashTableOptions opt;
  opt.init_capacity = opt.max_capacity = kCap;
  opt.max_hbm_for_vectors = nv::merlin::GB(1);
  opt.dim = kDim;
  std::unique_ptr<Table> table = std::make_unique<Table>();
  table->init(opt);
  EXPECT(table->capacity() == kCap);
  EXPECT(table->bucket_count() == kCap / 128);
  EXPECT(table->dim() == kDim);
  EXPECT(table->max_bucket_size() == 128);
  EXPECT(table->empty());

  std::vector<K> hk;
  std::vector<V> hv;
  std::vector<S> hs;
  make_batch(1, kN, kDim, hk, hv, hs);
  DeviceBuffer<K> dk(kN);
  DeviceBuffer<V> dv(kN * kDim);
  DeviceBuffer<S> ds(kN);
  DeviceBuffer<uint8_t> df(kN);
  dk.upload(hk);
  dv.upload(hv);
  ds.upload(hs);
  cudaStream_t stream;
  CUDA_CHECK(cudaStreamCreate(&stream));

  table->insert_or_assign(kN, dk.p, dv.p, ds.p, stream);
  EXPECT(table->size(stream) == kN);
  EXPECT(std::abs(table->load_factor(stream) - float(kN) / kCap) < 1e-6f);

  DeviceBuffer<V> out_v(kN * kDim);
  DeviceBuffer<S> out_s(kN);
  CUDA_CHECK(cudaMemset(out_v.p, 0, sizeof(V) * kN * kDim));
  table->find(kN, dk.p, out_v.p, reinterpret_cast<bool*>(df.p), out_s.p, stream);
  CUDA_CHECK(cudaStreamSynchronize(stream));
  auto f = df.download(kN);
  auto v = out_v.download(kN * kDim);
  auto s = out_s.download(kN);
  for (size_t i = 0; i < kN; ++i) {
    EXPECT(f[i]);
    EXPECT(s[i] == hk[i]);
    for (size_t j = 0; j < kDim; ++j) EXPECT(v[i * kDim + j] == static_cast<float>(hk[i] * 0.00001));
  }

  // erase half, sizes halve; erased keys are missed
  table->erase(kN / 2, dk.p, stream);
  EXPECT(table->size(stream) == kN / 2);
  table->find(kN, dk.p, out_v.p, reinterpret_cast<bool*>(df.p), out_s.p, stream);
  CUDA_CHECK(cudaStreamSynchronize(stream));
  f = df.download(kN);
  for (size_t i = 0; i < kN; ++i) EXPECT(f[i] == (i >= kN / 2));

  // export count == size, every exported tuple keeps value == key * 1e-5
  DeviceBuffer<K> ek(kCap);
  DeviceBuffer<V> ev(kCap * kDim);
  DeviceBuffer<S> es(kCap);
  const size_t exported = table->export_batch(table->capacity(), 0, ek.p, ev.p, es.p, stream);
  EXPECT(exported == kN / 2);
  auto xk = ek.download(exported);
  auto xv = ev.download(exported * kDim);
  auto xs = es.download(exported);
  std::set<K> seen;
  for (size_t i = 0; i < exported; ++i) {
    EXPECT(seen.insert(xk[i]).second);
    EXPECT(xs[i] == xk[i]);
    EXPECT(xv[i * kDim] == static_cast<float>(xk[i] * 0.00001));
  }

  // export_batch_if with a user functor; count equals size_if
  DeviceBuffer<size_t> dc(1);
  const S threshold = hk[kN / 2 + 5000];
  table->export_batch_if<ScoreBelow>(K(0), threshold, table->capacity(), 0, dc.p, ek.p, ev.p, es.p,
                                     stream);
  CUDA_CHECK(cudaStreamSynchronize(stream));
  const size_t matched = dc.download(1)[0];
  table->size_if<ScoreBelow>(K(0), threshold, dc.p, stream);
  CUDA_CHECK(cudaStreamSynchronize(stream));
  EXPECT(matched == dc.download(1)[0]);
  size_t want = 0;
  for (size_t i = kN / 2; i < kN; ++i) want += hs[i] < threshold ? 1 : 0;
  EXPECT(matched == want);
  xk = ek.download(matched);
  xs = es.download(matched);
  xv = ev.download(matched * kDim);
  for (size_t i = 0; i < matched; ++i) {
    EXPECT(xs[i] < threshold);
    EXPECT(xv[i * kDim + kDim - 1] == static_cast<float>(xk[i] * 0.00001));
  }

  // erase_if with the same functor removes exactly those keys; a second pass finds none
  {
    std::unique_ptr<Table> victim = std::make_unique<Table>();
    victim->init(opt);
    victim->insert_or_assign(kN, dk.p, dv.p, ds.p, stream);
    size_t below = 0;
    for (size_t i = 0; i < kN; ++i) below += hs[i] < threshold ? 1 : 0;
    EXPECT(victim->erase_if<ScoreBelow>(K(0), threshold, stream) == below);
    EXPECT(victim->size(stream) == kN - below);
    EXPECT(victim->erase_if<ScoreBelow>(K(0), threshold, stream) == 0);
  }

  // save / load round trip through LocalKVFile
  {
    nv::merlin::LocalKVFile<K, V, S> file;
    const std::string base = "/tmp/hkv_dropin_";
    EXPECT(file.open(base + "keys", base + "values", base + "scores", "wb"));
    EXPECT(table->save(&file, 1 << 20, stream) == kN / 2);
    file.close();
    std::unique_ptr<Table> copy = std::make_unique<Table>();
    copy->init(opt);
    EXPECT(file.open(base + "keys", base + "values", base + "scores", "rb"));
    EXPECT(copy->load(&file, 1 << 20, stream) == kN / 2);
    file.close();
    EXPECT(copy->size(stream) == kN / 2);
    copy->find(kN, dk.p, out_v.p, reinterpret_cast<bool*>(df.p), out_s.p, stream);
    CUDA_CHECK(cudaStreamSynchronize(stream));
    f = df.download(kN);
    s = out_s.download(kN);
    v = out_v.download(kN * kDim);
    for (size_t i = kN / 2; i < kN; ++i) {
      EXPECT(f[i] && s[i] == hk[i]);
      EXPECT(v[i * kDim + 3] == static_cast<float>(hk[i] * 0.00001));
    }
  }

  table->clear(stream);
  EXPECT(table->size(stream) == 0);
  EXPECT(table->empty(stream));
  CUDA_CHECK(cudaStreamDestroy(stream));
  std::printf("basic ok\n");
}

// n_evicted + size == inserted; the union of {table, evicted} holds every
// input key exactly once with its own value.
static void test_insert_and_evict_conservation() {
  constexpr size_t kDim = 8, kCap = 64 * 128, kN = 4096, kRounds = 6;
  using Table = nv::merlin::HashTable<K, V, S, EvictStrategy::kLru>;
  HashTableOptions opt;
  opt.init_capacity = opt.max_capacity = kCap;
  opt.max_hbm_for_vectors = nv::merlin::GB(1);
  opt.dim = kDim;
  Table table;
  table.init(opt);
  DeviceBuffer<K> dk(kN), ek(kN);
  DeviceBuffer<V> dv(kN * kDim), ev(kN * kDim);
  DeviceBuffer<S> es(kN);
  std::map<K, float> evicted;
  size_t inserted = 0;
  for (size_t r = 0; r < kRounds; ++r) {
    std::vector<K> hk;
    std::vector<V> hv;
    std::vector<S> hs;
    make_batch(1000000 + r * kN, kN, kDim, hk, hv, hs);
    dk.upload(hk);
    dv.upload(hv);
    const size_t n_evicted =
        table.insert_and_evict(kN, dk.p, dv.p, nullptr, ek.p, ev.p, es.p, cudaStream_t(0));
    inserted += kN;
    auto xk = ek.download(n_evicted);
    auto xv = ev.download(n_evicted * kDim);
    for (size_t i = 0; i < n_evicted; ++i) {
      EXPECT(evicted.emplace(xk[i], xv[i * kDim]).second);
      EXPECT(xv[i * kDim + kDim - 1] == static_cast<float>(xk[i] * 0.00001));
    }
    EXPECT(evicted.size() + table.size() == inserted);
  }
  EXPECT(table.size() == kCap);  // overfilled: every bucket is full
  DeviceBuffer<K> all_k(kCap);
  DeviceBuffer<V> all_v(kCap * kDim);
  const size_t live = table.export_batch(kCap, 0, all_k.p, all_v.p, nullptr, cudaStream_t(0));
  auto lk = all_k.download(live);
  for (K k : lk) EXPECT(evicted.count(k) == 0);
  EXPECT(live + evicted.size() == inserted);
  std::printf("insert_and_evict conservation ok (%zu evicted)\n", evicted.size());
}

static void test_errors() {
  using Table = nv::merlin::HashTable<K, V, S, EvictStrategy::kLfu>;
  HashTableOptions opt;
  opt.init_capacity = opt.max_capacity = 1024;
  opt.max_hbm_for_vectors = nv::merlin::MB(16);
  opt.dim = 4;
  opt.reserved_key_start_bit = 63;
  Table bad;
  bool threw = false;
  try {
    bad.init(opt);
  } catch (const nv::merlin::MerlinException&) {
    threw = true;
  }
  EXPECT(threw);
  opt.reserved_key_start_bit = 0;
  Table t;
  t.init(opt);
  DeviceBuffer<K> dk(8);
  DeviceBuffer<V> dv(32);
  threw = false;
  try {
    t.insert_or_assign(8, dk.p, dv.p, nullptr);  // Lfu needs scores
  } catch (const nv::merlin::MerlinException&) {
    threw = true;
  }
  EXPECT(threw);
  t.insert_or_assign(0, nullptr, nullptr, nullptr);  // n == 0 is a no-op
  std::printf("errors ok\n");
}

// tests/merlin_hashtable_test.cc.cu:1080-1222 (test_rehash): the table doubles
// on the insert path and by reserve(); entries keep their rows and scores.
static void test_rehash() {
  constexpr size_t kDim = 8, kInit = 1024, kMax = 8 * kInit, kN = 700;
  using Table = nv::merlin::HashTable<K, V, S, EvictStrategy::kCustomized>;
  HashTableOptions opt;
  opt.init_capacity = kInit;
  opt.max_capacity = kMax;
  opt.max_hbm_for_vectors = nv::merlin::GB(1);
  opt.dim = kDim;
  opt.max_load_factor = 0.5f;
  Table table;
  table.init(opt);
  std::vector<K> hk;
  std::vector<V> hv;
  std::vector<S> hs;
  make_batch(777, kN, kDim, hk, hv, hs);
  DeviceBuffer<K> dk(kN);
  DeviceBuffer<V> dv(kN * kDim);
  DeviceBuffer<S> ds(kN);
  DeviceBuffer<bool> df(kN);
  dk.upload(hk);
  dv.upload(hv);
  ds.upload(hs);
  table.insert_or_assign(kN, dk.p, dv.p, ds.p);
  EXPECT(table.capacity() == 2 * kInit);  // 700 / 1024 is above 0.5
  EXPECT(table.size() == kN);
  table.reserve(kMax);
  EXPECT(table.capacity() == kMax);
  table.reserve(2 * kMax);                 // above max_capacity: ignored
  EXPECT(table.capacity() == kMax);
  bool threw = false;
  try {
    table.set_max_capacity(3 * kMax);
  } catch (const std::invalid_argument&) {
    threw = true;
  }
  EXPECT(threw);
  table.set_max_capacity(2 * kMax);
  table.reserve(2 * kMax);
  EXPECT(table.capacity() == 2 * kMax);
  EXPECT(table.size() == kN);
  CUDA_CHECK(cudaMemset(dv.p, 0, sizeof(V) * kN * kDim));
  CUDA_CHECK(cudaMemset(ds.p, 0, sizeof(S) * kN));
  table.find(kN, dk.p, dv.p, df.p, ds.p);
  CUDA_CHECK(cudaDeviceSynchronize());
  std::vector<V> gv = dv.download(kN * kDim);
  std::vector<S> gs = ds.download(kN);
  std::vector<uint8_t> gf(kN);
  CUDA_CHECK(cudaMemcpy(gf.data(), df.p, kN, cudaMemcpyDeviceToHost));
  for (size_t i = 0; i < kN; ++i) {
    EXPECT(gf[i] == 1);
    EXPECT(gs[i] == hs[i]);
    for (size_t j = 0; j < kDim; ++j) EXPECT(gv[i * kDim + j] == hv[i * kDim + j]);
  }
  std::printf("rehash ok\n");
}

// export_batch_if_v2, erase_if_v2 and for_each with functors that use the
// value row and the cooperative tile; dim 16 and dim 4 select tiles of 16 and
// of 1 thread.
template <size_t kDim>
static void test_tile_functors() {
  constexpr size_t kCap = 64 * 1024, kN = 24 * 1024;
  using Table = nv::merlin::HashTable<K, V, S, EvictStrategy::kCustomized>;
  HashTableOptions opt;
  opt.init_capacity = opt.max_capacity = kCap;
  opt.max_hbm_for_vectors = nv::merlin::GB(1);
  opt.dim = kDim;
  Table table;
  table.init(opt);
  std::vector<K> hk;
  std::vector<V> hv;
  std::vector<S> hs;
  make_batch(31337, kN, kDim, hk, hv, hs);
  // damage every 7th row: the predicate must drop those
  for (size_t i = 0; i < kN; i += 7) hv[i * kDim + (i % kDim)] *= -1.0f;
  DeviceBuffer<K> dk(kN);
  DeviceBuffer<V> dv(kN * kDim);
  DeviceBuffer<S> ds(kN);
  dk.upload(hk);
  dv.upload(hv);
  ds.upload(hs);
  table.insert_or_assign(kN, dk.p, dv.p, ds.p);
  EXPECT(table.size() == kN);

  std::vector<S> sorted = hs;
  std::sort(sorted.begin(), sorted.end());
  const S threshold = sorted[kN / 3];
  std::set<K> want;
  for (size_t i = 0; i < kN; ++i) {
    if (hs[i] < threshold && i % 7 != 0) want.insert(hk[i]);
  }

  DeviceBuffer<size_t> dc(1);
  DeviceBuffer<K> ek(kCap);
  DeviceBuffer<V> ev(kCap * kDim);
  DeviceBuffer<S> es(kCap);
  ScoreBelowAndRowIntact<K, V, S> pred{threshold, int(kDim)};
  table.export_batch_if_v2(pred, table.capacity(), 0, dc.p, ek.p, ev.p, es.p);
  CUDA_CHECK(cudaDeviceSynchronize());
  const size_t got = dc.download(1)[0];
  EXPECT(got == want.size());
  auto xk = ek.download(got);
  auto xv = ev.download(got * kDim);
  auto xs = es.download(got);
  for (size_t i = 0; i < got; ++i) {
    EXPECT(want.count(xk[i]) == 1);
    EXPECT(xs[i] == xk[i]);
    for (size_t j = 0; j < kDim; ++j) EXPECT(xv[i * kDim + j] == static_cast<float>(xk[i] * 0.00001));
  }
  // a window that is not a multiple of 8 runs with tiles of one thread
  table.export_batch_if_v2(pred, table.capacity() - 3, 1, dc.p, ek.p, ev.p, es.p);
  CUDA_CHECK(cudaDeviceSynchronize());
  EXPECT(dc.download(1)[0] <= got && dc.download(1)[0] + 3 >= got);

  // for_each: negate the selected rows, bump their scores
  NegateRowsBelow<K, V, S> body{threshold, int(kDim)};
  table.for_each(0, table.capacity(), body);
  DeviceBuffer<bool> df(kN);
  table.find(kN, dk.p, dv.p, df.p, ds.p);
  CUDA_CHECK(cudaDeviceSynchronize());
  auto fv = dv.download(kN * kDim);
  auto fs = ds.download(kN);
  for (size_t i = 0; i < kN; ++i) {
    const bool hit = hs[i] < threshold;
    EXPECT(fs[i] == hs[i] + (hit ? 1 : 0));
    for (size_t j = 0; j < kDim; ++j) {
      EXPECT(fv[i * kDim + j] == (hit ? -hv[i * kDim + j] : hv[i * kDim + j]));
    }
  }
  // put the rows back, then erase with the tile predicate
  table.for_each(0, table.capacity(), body);   // scores are now +1 or +2, rows of hits restored
  ScoreBelowAndRowIntact<K, V, S> erase_pred{threshold + 2, int(kDim)};
  size_t want_erased = 0;
  std::vector<uint8_t> erased(kN, 0);
  for (size_t i = 0; i < kN; ++i) {
    // the second for_each saw score+1 < threshold for all but the keys just below it
    const S after = hs[i] + (hs[i] < threshold ? 1 : 0) + (hs[i] + 1 < threshold ? 1 : 0);
    const bool twice = hs[i] < threshold && hs[i] + 1 < threshold;
    const bool once = hs[i] < threshold && !twice;
    const bool intact = (i % 7 != 0) && !once;   // negated once: no longer key * 1e-5
    erased[i] = after < threshold + 2 && intact;
    want_erased += erased[i];
  }
  EXPECT(table.erase_if_v2(erase_pred) == want_erased);
  EXPECT(table.size() == kN - want_erased);
  dk.upload(hk);
  table.find(kN, dk.p, dv.p, df.p, ds.p);
  CUDA_CHECK(cudaDeviceSynchronize());
  std::vector<uint8_t> gf(kN);
  CUDA_CHECK(cudaMemcpy(gf.data(), df.p, kN, cudaMemcpyDeviceToHost));
  for (size_t i = 0; i < kN; ++i) EXPECT(gf[i] == (erased[i] ? 0 : 1));
  EXPECT(table.erase_if_v2(erase_pred) == 0);
  std::printf("tile functors ok (dim %zu)\n", kDim);
}

// S = uint32_t (Customized only): 32-bit score arrays in and out.
static void test_uint32_scores() {
  constexpr size_t kDim = 4, kCap = 8 * 1024, kN = 4096;
  using Table = nv::merlin::HashTable<K, V, uint32_t, EvictStrategy::kCustomized>;
  HashTableOptions opt;
  opt.init_capacity = opt.max_capacity = kCap;
  opt.max_hbm_for_vectors = nv::merlin::GB(1);
  opt.dim = kDim;
  Table table;
  table.init(opt);
  std::vector<K> hk;
  std::vector<V> hv;
  std::vector<S> unused;
  make_batch(4242, kN, kDim, hk, hv, unused);
  std::vector<uint32_t> hs(kN);
  for (size_t i = 0; i < kN; ++i) hs[i] = 0x80000000u + static_cast<uint32_t>(i);
  DeviceBuffer<K> dk(kN);
  DeviceBuffer<V> dv(kN * kDim);
  DeviceBuffer<uint32_t> ds(kN);
  DeviceBuffer<bool> df(kN);
  dk.upload(hk);
  dv.upload(hv);
  ds.upload(hs);
  table.insert_or_assign(kN, dk.p, dv.p, ds.p);
  EXPECT(table.size() == kN);
  CUDA_CHECK(cudaMemset(ds.p, 0, sizeof(uint32_t) * kN));
  table.find(kN, dk.p, dv.p, df.p, ds.p);
  CUDA_CHECK(cudaDeviceSynchronize());
  auto gs = ds.download(kN);
  for (size_t i = 0; i < kN; ++i) EXPECT(gs[i] == hs[i]);
  DeviceBuffer<K> ek(kCap);
  DeviceBuffer<V> ev(kCap * kDim);
  DeviceBuffer<uint32_t> es(kCap);
  const size_t exported = table.export_batch(table.capacity(), 0, ek.p, ev.p, es.p);
  EXPECT(exported == kN);
  auto xs = es.download(exported);
  for (size_t i = 0; i < exported; ++i) EXPECT(xs[i] >= 0x80000000u && xs[i] < 0x80000000u + kN);
  std::printf("uint32 scores ok\n");
}

int main() {
  test_uint32_scores();
  test_rehash();
  test_tile_functors<16>();
  test_tile_functors<4>();
  test_errors();
  test_basic();
  test_insert_and_evict_conservation();
  std::printf("PASS\n");
  return 0;
}
