// Device-side building blocks shared by every kernel of the table:
// addressing, reserved keys, slot atomics, the 8-lane bucket probe and the
// warp-cooperative row copy.
//
// Storage is flat structure-of-arrays (one allocation per plane):
//   digests      [buckets][128]  u8    one 128-byte line per bucket
//   keys, scores [buckets][128]  u64   the key doubles as the slot lock; two
//                                       layouts, chosen when the table is made:
//       planes (default)  one array of keys, one of scores
//       lines             16 lines of 128 bytes per bucket, line l holding the
//                         keys of slots 8l .. 8l+7 and behind them the scores
//                         of the same slots
//   values       [buckets*128][row_bytes]   HBM part, then pinned-host part
//   bucket_sizes [buckets]       i32
//
// What the two layouts trade (measured on B200, 64 Mi-slot table, 1 Mi-key
// batches).  Every operation that locks a slot also writes its score.  With
// separate planes that 8-byte store goes into a 32-byte sector that is not in
// L2: a read-modify-write in DRAM at a random address, as expensive as the
// whole 256-byte row write (73 us of a 239 us update of present keys).  With
// the score in the line the lock's compare-and-swap has just opened, and a
// prefetch of its sector issued with the compare-and-swap, the store merges in
// L2 and the line is written back once: updates of present keys and inserts
// into free slots run a quarter faster (insert_or_assign of present keys 3.96
// -> 4.95 B-KV/s).  The price: a bucket's 128 scores are the second halves of
// 16 lines instead of 8 whole lines, which makes every eviction's score scan
// dearer (inserts that all evict 1.81 -> 1.55 B-KV/s), and the keys a lookup
// verifies are spread over twice the address range (find 8.2 -> 7.9, contains
// 20.3 -> 17.9 B-KV/s).  Tables that mostly update resident keys want lines,
// tables that mostly look up or churn want planes.
//
// Semantics follow the reference (NVIDIA-Merlin/HierarchicalKV):
//   hash / bucket / start / digest  include/merlin/utils.cuh:137-145,
//                                   include/merlin/core_kernels/kernel_utils.cuh:72-103,638-643
//   reserved keys                   include/merlin/types.cuh:47-109
//   key-as-lock slot protocol       include/merlin/core_kernels/upsert.cuh:89-110,199-232
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace hkv {

// Slots per bucket of the tables the warp-parallel kernels serve (one digest
// line).  Tables created with another max_bucket_size run the bucket-size
// generic kernels (find_generic_kernel, mutate_serial_kernel).
constexpr int kBucketSlots = 128;
constexpr uint32_t kMaxBucketSlots = 1024;
constexpr int kGroupLanes = 8;           // lanes that probe one bucket
constexpr int kKeysPerPass = 4;          // buckets probed per warp instruction
constexpr int kPasses = 8;               // passes to cover a warp's 32 keys
constexpr uint32_t kNoSlot = 0xFFFFFFFFu;
constexpr uint32_t kRowTagShift = 28;              // routed form: row tag = rank << 28 | row
constexpr uint32_t kRowTagMask = (1u << kRowTagShift) - 1u;
constexpr uint64_t kMaxScore = 0xFFFFFFFFFFFFFFFFull;
constexpr uint64_t kIgnoredEpoch = 0xFFFFFFFFFFFFFFFFull;
constexpr uint32_t kSpinLimit = 1u << 22;    // polls of one slot before a wait gives up (about a second)
constexpr uint32_t kRescanLimit = 1u << 20;  // bucket rescans of the serialising kernels (about a second)

// Bits of the per-table device status word.
constexpr uint32_t kStatusLockTimeout = 1u;   // a bounded slot wait ran out
constexpr uint32_t kStatusRetryExhausted = 2u;  // eviction retries ran out

enum Strategy : int {
  kLru = 0,
  kLfu = 1,
  kEpochLru = 2,
  kEpochLfu = 3,
  kCustomized = 4,
};

// Kernel-parameter view of a table.  Reserved keys travel with the view (not
// in __constant__ memory) so tables with different reserved_key_start_bit can
// live side by side in one process.
// Element types accum_or_assign can add (the reference adds with V's own
// operator+=, include/merlin/core_kernels/accum_or_assign.cuh:139-172).
enum ValueKind : uint32_t {
  kValueOpaque = 0,  // rows are bytes; float32 is assumed when sizeof(V) == 4
  kValueF32 = 1,
  kValueF64 = 2,
  kValueI32 = 3,
  kValueI64 = 4,
  kValueF16 = 5,
  kValueBF16 = 6,
};

struct TableView {
  uint8_t* digests;
  uint64_t* key_words;    // keys and scores: see key_ptr / score_ptr
  uint64_t* score_words;
  uint64_t line_mask;     // ~0: keys and scores share 128-byte lines; 0: separate planes
  uint8_t* values_hbm;    // rows of row slots [0, hbm_slots)
  uint8_t* values_host;   // rows of row slots [hbm_slots, capacity), pinned+mapped
  // Hybrid tables only (else null): bucket b keeps its 128 rows in row block
  // bucket_map[b] (blocks below hbm_slots / 128 are in HBM), so hot buckets
  // can trade places with cold ones; bucket_heat[b] counts the hits lookups
  // found in bucket b since the last promotion.
  uint32_t* bucket_map;
  uint32_t* bucket_heat;
  int32_t* bucket_sizes;
  uint32_t* status;       // device status word (kStatus* bits)
  uint64_t buckets;
  uint64_t capacity;      // buckets * bucket_slots
  uint32_t bucket_slots;  // slots per bucket: a power of two, 16 ... 1024 (128 by default)
  uint32_t bucket_shift;  // log2(bucket_slots)
  uint64_t hbm_slots;
  uint32_t row_bytes;     // dim * sizeof(V)
  uint32_t vec_bytes;     // widest power-of-two access usable on a row
  uint32_t chunks_per_row;        // row_bytes / vec_bytes
  int32_t chunks_per_row_shift;   // log2(chunks_per_row) or -1
  uint32_t chunks_per_row_magic;  // floor(2^32 / chunks_per_row) + 1 (when not a power of two)
  uint32_t capacity_pow2;         // 1 when capacity is a power of two
  uint32_t value_kind;            // element type of a row, used by accum_or_assign only (ValueKind)
  uint64_t empty_key;
  uint64_t reclaim_key;
  uint64_t locked_key;
  uint64_t reserved_mask;   // (key & reserved_mask) == reserved_value
  uint64_t reserved_value;
  uint32_t empty_digest4;   // empty digest replicated in 4 bytes
  uint32_t reclaim_digest;
};

__host__ __device__ __forceinline__ uint64_t fmix64(uint64_t k) {
  k ^= k >> 33;
  k *= 0xff51afd7ed558ccdull;
  k ^= k >> 33;
  k *= 0xc4ceb9fe1a85ec53ull;
  k ^= k >> 33;
  return k;
}

__device__ __forceinline__ bool is_reserved(const TableView& t, uint64_t key) {
  return (key & t.reserved_mask) == t.reserved_value;
}

__device__ __forceinline__ uint64_t global_nano() {
  uint64_t v;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(v));
  return v;
}

struct Address {
  uint64_t bucket;
  uint32_t start;   // probe start slot inside the bucket
  uint32_t digest;  // 8-bit digest
};

__device__ __forceinline__ Address locate(const TableView& t, uint64_t key) {
  const uint64_t h = fmix64(key);
  const uint64_t g = t.capacity_pow2 ? (h & (t.capacity - 1)) : (h % t.capacity);
  Address a;
  a.bucket = g >> t.bucket_shift;
  a.start = static_cast<uint32_t>(g) & (t.bucket_slots - 1u);
  a.digest = static_cast<uint32_t>(h >> 32) & 0xFFu;
  return a;
}

// The same for the kernels that only serve 128-slot buckets: constant shifts.
__device__ __forceinline__ Address locate_line(const TableView& t, uint64_t key) {
  const uint64_t h = fmix64(key);
  const uint64_t g = t.capacity_pow2 ? (h & (t.capacity - 1)) : (h % t.capacity);
  Address a;
  a.bucket = g >> 7;
  a.start = static_cast<uint32_t>(g) & (kBucketSlots - 1);
  a.digest = static_cast<uint32_t>(h >> 32) & 0xFFu;
  return a;
}

// Dual-bucket addressing (TableMode::kMemory of the reference,
// include/merlin/core_kernels/dual_bucket_utils.cuh:31-65): a key may live in
// one of two buckets, chosen from the low and the high half of its hash; the
// digest is the top byte of the hash.
struct DualAddress {
  Address first;   // bucket from the low 32 bits
  Address second;  // bucket from the high 32 bits, never the same bucket
};

__host__ __device__ __forceinline__ uint32_t dual_digest(uint64_t hashed) {
  return static_cast<uint32_t>(hashed >> 56);
}

__device__ __forceinline__ DualAddress locate_dual(const TableView& t, uint64_t key) {
  const uint64_t h = fmix64(key);
  const uint32_t lo = static_cast<uint32_t>(h);
  const uint32_t hi = static_cast<uint32_t>(h >> 32);
  DualAddress d;
  d.first.bucket = lo % t.buckets;
  d.second.bucket = hi % t.buckets;
  if (d.second.bucket == d.first.bucket) d.second.bucket = (d.second.bucket + 1) % t.buckets;
  d.first.start = static_cast<uint32_t>(lo % t.capacity) & (kBucketSlots - 1);
  d.second.start = static_cast<uint32_t>(hi % t.capacity) & (kBucketSlots - 1);
  d.first.digest = d.second.digest = dual_digest(h);
  return d;
}

// Key and score of a slot.  Planes: word `slot` of the key array and of the
// score array.  Lines: line slot / 8 holds 16 words, 0-7 the keys of its 8
// slots and 8-15 their scores; score_words points 8 words behind key_words.
constexpr uint32_t kLineSlots = 8;
__host__ __device__ __forceinline__ uint64_t slot_word(const TableView& t, uint64_t slot) {
  return slot + ((slot & ~uint64_t(7)) & t.line_mask);
}
__host__ __device__ __forceinline__ uint64_t* key_ptr(const TableView& t, uint64_t slot) {
  return t.key_words + slot_word(t, slot);
}
__host__ __device__ __forceinline__ uint64_t* score_ptr(const TableView& t, uint64_t slot) {
  return t.score_words + slot_word(t, slot);
}
// Key at position pos of 128-slot bucket b.
__device__ __forceinline__ uint64_t* key_ptr_in_line_bucket(const TableView& t, uint32_t bucket,
                                                            uint32_t pos) {
  return key_ptr(t, (uint64_t(bucket) << 7) + pos);
}

// Host side: may the kernels specialised for 16-byte chunks of pure-HBM rows run?
inline bool fast_rows(const TableView& t) {
  return t.vec_bytes == 16 && t.hbm_slots == t.capacity && t.bucket_map == nullptr;
}

// Host side: do the kernels built around the 128-byte digest line serve this table?
inline bool line_buckets(const TableView& t) { return t.bucket_slots == uint32_t(kBucketSlots); }

// Where slot's row lives: the slot itself, or its place in the row block the
// bucket map assigns to the slot's bucket.
__device__ __forceinline__ uint64_t row_slot(const TableView& t, uint64_t slot) {
  if (t.bucket_map == nullptr) return slot;
  return (uint64_t(t.bucket_map[slot >> t.bucket_shift]) << t.bucket_shift) |
         (slot & (t.bucket_slots - 1u));
}

__device__ __forceinline__ uint8_t* row_ptr_of_row_slot(const TableView& t, uint64_t rs) {
  return rs < t.hbm_slots ? t.values_hbm + rs * t.row_bytes
                          : t.values_host + (rs - t.hbm_slots) * t.row_bytes;
}

__device__ __forceinline__ uint8_t* row_ptr(const TableView& t, uint64_t slot) {
  return row_ptr_of_row_slot(t, row_slot(t, slot));
}

// ---- slot atomics (64-bit keys and scores, device scope) -------------------

__device__ __forceinline__ uint64_t ld_relaxed(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ uint64_t ld_acquire(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_relaxed(uint64_t* p, uint64_t v) {
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__device__ __forceinline__ void st_release(uint64_t* p, uint64_t v) {
  asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// Returns the value observed; the swap happened iff it equals `expected`.
__device__ __forceinline__ uint64_t cas_acquire(uint64_t* p, uint64_t expected,
                                                uint64_t desired) {
  uint64_t old;
  asm volatile("atom.acquire.gpu.global.cas.b64 %0, [%1], %2, %3;"
               : "=l"(old)
               : "l"(p), "l"(expected), "l"(desired)
               : "memory");
  return old;
}

// Swaps `desired` in and returns what was there.
__device__ __forceinline__ uint64_t exch_acquire(uint64_t* p, uint64_t desired) {
  uint64_t old;
  asm volatile("atom.acquire.gpu.global.exch.b64 %0, [%1], %2;"
               : "=l"(old)
               : "l"(p), "l"(desired)
               : "memory");
  return old;
}

// Relaxed CAS: several of them can be in flight at once.  A thread that took a
// lock this way issues one acquire fence (fence_acquire) before it touches what
// the lock protects -- atomic followed by fence is the acquire pattern.
__device__ __forceinline__ uint64_t cas_relaxed(uint64_t* p, uint64_t expected,
                                                uint64_t desired) {
  uint64_t old;
  asm volatile("atom.relaxed.gpu.global.cas.b64 %0, [%1], %2, %3;"
               : "=l"(old)
               : "l"(p), "l"(expected), "l"(desired)
               : "memory");
  return old;
}

// Asks L2 for the 32-byte sector around p without waiting for it.
__device__ __forceinline__ void prefetch_l2(const void* p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

__device__ __forceinline__ void fence_acquire() {
  asm volatile("fence.acq_rel.gpu;" ::: "memory");
}

__device__ __forceinline__ void st_u8_cg(uint8_t* p, uint32_t v) {
  asm volatile("st.global.cg.u8 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Loads with an L2 cache policy.  Digest lines and key lines are reused by
// later batches and are asked to stay in L2 (evict_last); value rows are
// touched once per batch and stream through (__ldcs / __stcs, evict_first).
__device__ __forceinline__ uint64_t policy_keep() {
  uint64_t p;
  asm("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}

#ifndef HKV_DIGEST_HINT
#define HKV_DIGEST_HINT 1
#endif
#ifndef HKV_KEY_HINT
#define HKV_KEY_HINT 1
#endif
__device__ __forceinline__ uint4 ld_meta_v4(const void* p) {
  uint4 v;
#if HKV_DIGEST_HINT
  asm volatile("ld.global.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p), "l"(policy_keep())
               : "memory");
#else
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
#endif
  return v;
}

__device__ __forceinline__ uint64_t ld_meta_u64(const uint64_t* p) {
  uint64_t v;
#if HKV_KEY_HINT
  asm volatile("ld.global.L1::no_allocate.L2::cache_hint.u64 %0, [%1], %2;"
               : "=l"(v)
               : "l"(p), "l"(policy_keep())
               : "memory");
#else
  asm volatile("ld.global.L1::no_allocate.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
#endif
  return v;
}

template <int VEC>
struct VecType;
template <>
struct VecType<16> { using type = uint4; };
template <>
struct VecType<8> { using type = uint2; };
template <>
struct VecType<4> { using type = uint32_t; };
template <>
struct VecType<2> { using type = uint16_t; };
template <>
struct VecType<1> { using type = uint8_t; };

template <class T>
__device__ __forceinline__ T ld_stream(const T* p) {
  return __ldcs(p);
}
template <class T>
__device__ __forceinline__ void st_stream(T* p, const T& v) {
  __stcs(p, v);
}
// A load from a buffer that may be another GPU's memory and that its owner
// rewrites between this GPU's launches: never served from L1 (ld.global.cv
// fetches again whatever the cache holds).
template <class T>
__device__ __forceinline__ T ld_peer(const T* p) {
  return __ldcv(p);
}
// __ldcs/__stcs have no 1- and 2-byte unsigned overloads for every toolkit;
// narrow rows are rare, plain accesses are enough for them.
template <>
__device__ __forceinline__ uint16_t ld_stream<uint16_t>(const uint16_t* p) {
  return *p;
}
template <>
__device__ __forceinline__ void st_stream<uint16_t>(uint16_t* p, const uint16_t& v) {
  *p = v;
}
template <>
__device__ __forceinline__ uint8_t ld_stream<uint8_t>(const uint8_t* p) {
  return *p;
}
template <>
__device__ __forceinline__ void st_stream<uint8_t>(uint8_t* p, const uint8_t& v) {
  *p = v;
}

// A chunk of a value row read for the caller.  Rows in HBM are touched once
// per batch and stream through L2 (evict-first).  Rows in pinned host memory
// cross the host link, which is two orders of magnitude slower than HBM: they
// are read with the default cache policy so that the hot rows of a skewed
// query stream, and rows asked for twice in one batch, are served from L2
// instead of the link.  (Measured on the Zipf(1.05) workload: evict-first
// loads 0.17, default loads 0.22 B-KV/s; loads carrying an explicit L2 cache
// hint were split into small link requests and fell to 0.06.)
template <class T>
__device__ __forceinline__ T ld_table_row(const uint8_t* p, bool in_host_memory) {
  if (in_host_memory) return *reinterpret_cast<const T*>(p);  // default policy: may stay in L2
  return ld_stream(reinterpret_cast<const T*>(p));
}

// ---- digest matching -------------------------------------------------------

// 4-bit mask, bit i set when byte i of `word` equals the byte replicated in
// `pattern4`.
__device__ __forceinline__ uint32_t match4(uint32_t word, uint32_t pattern4) {
  const uint32_t eq = __vcmpeq4(word, pattern4) & 0x01010101u;
  return (eq * 0x01020408u) >> 24;
}

// 16-bit mask over the 16 digests a lane holds.
__device__ __forceinline__ uint32_t match16(const uint4& d, uint32_t pattern4) {
  return match4(d.x, pattern4) | (match4(d.y, pattern4) << 4) |
         (match4(d.z, pattern4) << 8) | (match4(d.w, pattern4) << 12);
}

__device__ __forceinline__ uint32_t replicate4(uint32_t byte) {
  return byte * 0x01010101u;
}

// Row of chunk c (c / chunks_per_row) without an integer division: a shift for
// power-of-two rows, otherwise a multiply by the rounded-up reciprocal, which
// can only overshoot by one.
__host__ __device__ __forceinline__ uint32_t chunks_per_row_magic_of(uint32_t cpr) {
  return cpr > 1 ? uint32_t((uint64_t(1) << 32) / cpr) + 1u : 0u;
}

__device__ __forceinline__ uint32_t row_of_chunk(const TableView& t, uint32_t c) {
  if (t.chunks_per_row_shift >= 0) return c >> t.chunks_per_row_shift;
  uint32_t r = __umulhi(c, t.chunks_per_row_magic);
  if (r * t.chunks_per_row > c) --r;
  return r;
}

// row += delta for one row, all 32 lanes, in the row's own element type.  The
// float32 case does not come here: it is folded into the chunked row mover.
__device__ __forceinline__ void warp_accumulate_row(uint8_t* row, const uint8_t* delta,
                                                    uint32_t row_bytes, uint32_t kind,
                                                    uint32_t lane) {
  switch (kind) {
    case kValueF64:
      for (uint32_t e = lane; e < row_bytes / 8; e += 32)
        reinterpret_cast<double*>(row)[e] += reinterpret_cast<const double*>(delta)[e];
      break;
    case kValueI64:
      for (uint32_t e = lane; e < row_bytes / 8; e += 32)
        reinterpret_cast<uint64_t*>(row)[e] += reinterpret_cast<const uint64_t*>(delta)[e];
      break;
    case kValueI32:
      for (uint32_t e = lane; e < row_bytes / 4; e += 32)
        reinterpret_cast<uint32_t*>(row)[e] += reinterpret_cast<const uint32_t*>(delta)[e];
      break;
    case kValueF16:
      for (uint32_t e = lane; e < row_bytes / 2; e += 32)
        reinterpret_cast<__half*>(row)[e] =
            __hadd(reinterpret_cast<__half*>(row)[e], reinterpret_cast<const __half*>(delta)[e]);
      break;
    case kValueBF16:
      for (uint32_t e = lane; e < row_bytes / 2; e += 32)
        reinterpret_cast<__nv_bfloat16*>(row)[e] =
            __hadd(reinterpret_cast<__nv_bfloat16*>(row)[e],
                   reinterpret_cast<const __nv_bfloat16*>(delta)[e]);
      break;
    default:
      for (uint32_t e = lane; e < row_bytes / 4; e += 32)
        reinterpret_cast<float*>(row)[e] += reinterpret_cast<const float*>(delta)[e];
      break;
  }
}

// ---- warp-cooperative row copy --------------------------------------------
//
// A warp owns up to 32 consecutive rows of a batch buffer (`batch_rows` points
// at the first).  Lane r holds in `slot` the table slot paired with batch row
// r, or kNoSlot when that row takes no part.  All 32 lanes move 16-byte (or
// narrower) chunks: chunk c belongs to row c / chunks_per_row, so the batch
// side is one contiguous, fully coalesced stream and the table side is one
// contiguous segment per row.
//
// MODE 0: table -> batch (gather)   MODE 1: batch -> table (scatter)
// MODE 2: table += batch, float32 elements (needs VEC % 4 == 0); the other
//         element types go through warp_accumulate_rows
//
// INDEXED (the routed form of the sharded table): the batch rows are not the
// warp's 32 consecutive rows.  Lane r holds in `row_index` a row tag: bits
// 28-31 name the source rank, bits 0-27 the row in that rank's batch buffer,
// whose address is bases[rank].  Those buffers may be other GPUs' memory and
// are accessed with plain loads and stores.
//
// PURE: every row is in HBM at its slot's own place (no host rows, no bucket
// map), which the launcher checks before it picks such an instantiation.
template <int VEC, int MODE, bool INDEXED = false, bool PURE = false>
__device__ __forceinline__ void warp_move_rows_vec(const TableView& t, uint8_t* batch_rows,
                                                   uint32_t slot, uint32_t lane,
                                                   uint32_t row_index = 0,
                                                   uint8_t* const* bases = nullptr) {
  using T = typename VecType<VEC>::type;
  // Chunks in flight per lane.  Accumulation holds two values per chunk (the
  // delta and the stored chunk: both are loaded before anything is written, so
  // the stored chunks of a pass arrive together instead of one after the
  // other) and the routed form keeps a second address per chunk: four instead
  // of eight for those, two where both apply (the routed accumulation then
  // runs six blocks per SM instead of five: 208 -> 184 us for 2 x 156 k keys).
  constexpr int U = (VEC == 16 && MODE != 2 && !INDEXED) ? 8 : (MODE == 2 && INDEXED) ? 2 : 4;
  const uint32_t cpr = t.chunks_per_row;
  const uint32_t total = cpr * 32u;
  for (uint32_t base = 0; base < total; base += 32u * U) {
    T regs[U];
    T stored[MODE == 2 ? U : 1];
    uint8_t* tab[U];
    uint8_t* bat[U];
    bool ok[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t c = base + u * 32u + lane;
      const uint32_t r = row_of_chunk(t, c);
      const uint32_t s = __shfl_sync(0xFFFFFFFFu, slot, r & 31u);
      ok[u] = (c < total) && (s != kNoSlot);
      const uint32_t off = (c - r * cpr) * VEC;
      const uint64_t rs = (ok[u] && !PURE) ? row_slot(t, s) : s;
      tab[u] = !ok[u] ? nullptr
                      : (PURE ? t.values_hbm + uint64_t(s) * t.row_bytes
                              : row_ptr_of_row_slot(t, rs)) + off;
      if (INDEXED) {
        const uint32_t at = __shfl_sync(0xFFFFFFFFu, row_index, r & 31u);
        bat[u] = bases[at >> kRowTagShift] + uint64_t(at & kRowTagMask) * t.row_bytes + off;
      }
      if (ok[u]) {
        if (MODE == 0) {
          regs[u] = ld_table_row<T>(tab[u], !PURE && rs >= t.hbm_slots);
        } else if (INDEXED) {
          regs[u] = ld_peer(reinterpret_cast<const T*>(bat[u]));
        } else {
          regs[u] = ld_stream(reinterpret_cast<const T*>(batch_rows + size_t(c) * VEC));
        }
        if (MODE == 2) stored[MODE == 2 ? u : 0] = *reinterpret_cast<const T*>(tab[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t c = base + u * 32u + lane;
      if (ok[u]) {
        if (MODE == 0) {
          if (INDEXED) {
            *reinterpret_cast<T*>(bat[u]) = regs[u];
          } else {
            st_stream(reinterpret_cast<T*>(batch_rows + size_t(c) * VEC), regs[u]);
          }
        } else if (MODE == 1) {
          st_stream(reinterpret_cast<T*>(tab[u]), regs[u]);
        } else {
          if constexpr (VEC % 4 == 0) {
            T cur = stored[MODE == 2 ? u : 0];
            float* a = reinterpret_cast<float*>(&cur);
            const float* b = reinterpret_cast<const float*>(&regs[u]);
#pragma unroll
            for (int e = 0; e < VEC / 4; ++e) a[e] += b[e];
            *reinterpret_cast<T*>(tab[u]) = cur;
          }
        }
      }
    }
  }
}

// Gather variant whose destination is not a contiguous batch: lane r holds the
// table slot of row r (or kNoSlot) and the row index `dest_row` it goes to in
// `dest_base` (possibly another GPU's memory, written with plain stores).
// ROW_SLOTS: `slot` already names the place of the row (row_slot()), not the
// table slot.
template <int VEC, bool ROW_SLOTS = false, bool PURE = false>
__device__ __forceinline__ void warp_gather_rows_to_vec(const TableView& t, uint8_t* dest_base,
                                                        uint32_t dest_row, uint32_t slot,
                                                        uint32_t lane) {
  using T = typename VecType<VEC>::type;
  constexpr int U = (VEC == 16) ? 8 : 4;
  const uint32_t cpr = t.chunks_per_row;
  const uint32_t total = cpr * 32u;
  for (uint32_t base = 0; base < total; base += 32u * U) {
    T regs[U];
    uint32_t drow[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t c = base + u * 32u + lane;
      const uint32_t r = row_of_chunk(t, c);
      const uint32_t s = __shfl_sync(0xFFFFFFFFu, slot, r & 31u);
      const uint32_t d = __shfl_sync(0xFFFFFFFFu, dest_row, r & 31u);
      drow[u] = kNoSlot;
      if (c < total && s != kNoSlot) {
        const uint8_t* row = PURE ? t.values_hbm + uint64_t(s) * t.row_bytes
                                  : (ROW_SLOTS ? row_ptr_of_row_slot(t, s) : row_ptr(t, s));
        regs[u] = ld_stream(reinterpret_cast<const T*>(row + (c - r * cpr) * VEC));
        drow[u] = d;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (drow[u] != kNoSlot) {
        const uint32_t c = base + u * 32u + lane;
        const uint32_t r = row_of_chunk(t, c);
        *reinterpret_cast<T*>(dest_base + uint64_t(drow[u]) * t.row_bytes + (c - r * cpr) * VEC) =
            regs[u];
      }
    }
  }
}

template <int VEC = 0, bool ROW_SLOTS = false>
__device__ __forceinline__ void warp_gather_rows_to(const TableView& t, uint8_t* dest_base,
                                                    uint32_t dest_row, uint32_t slot,
                                                    uint32_t lane) {
  if constexpr (VEC != 0) {
    warp_gather_rows_to_vec<VEC, ROW_SLOTS, true>(t, dest_base, dest_row, slot, lane);
    return;
  }
  switch (t.vec_bytes) {
    case 16: warp_gather_rows_to_vec<16, ROW_SLOTS>(t, dest_base, dest_row, slot, lane); break;
    case 8: warp_gather_rows_to_vec<8, ROW_SLOTS>(t, dest_base, dest_row, slot, lane); break;
    case 4: warp_gather_rows_to_vec<4, ROW_SLOTS>(t, dest_base, dest_row, slot, lane); break;
    case 2: warp_gather_rows_to_vec<2, ROW_SLOTS>(t, dest_base, dest_row, slot, lane); break;
    default: warp_gather_rows_to_vec<1, ROW_SLOTS>(t, dest_base, dest_row, slot, lane); break;
  }
}

// VEC != 0 fixes the access width at compile time and promises a pure-HBM
// table (the launcher picks the instantiation: t.vec_bytes == VEC and no host
// rows), which keeps the four other unrolled copy loops, the bucket map and
// the host-memory cases out of the hot kernels' instruction footprint.
template <int MODE, int VEC = 0, bool INDEXED = false>
__device__ __forceinline__ void warp_move_rows(const TableView& t, uint8_t* batch_rows,
                                               uint32_t slot, uint32_t lane,
                                               uint32_t row_index = 0,
                                               uint8_t* const* bases = nullptr) {
  if constexpr (MODE == 2) {
    if (t.value_kind > kValueF32) {
      // the rarer element types: one row after the other, all lanes on one row
      uint32_t todo = __ballot_sync(0xFFFFFFFFu, slot != kNoSlot);
      while (todo) {
        const uint32_t r = __ffs(todo) - 1;
        todo &= todo - 1;
        const uint32_t s = __shfl_sync(0xFFFFFFFFu, slot, r);
        const uint32_t at = INDEXED ? __shfl_sync(0xFFFFFFFFu, row_index, r) : r;
        const uint8_t* delta = INDEXED ? bases[at >> kRowTagShift] +
                                             uint64_t(at & kRowTagMask) * t.row_bytes
                                       : batch_rows + uint64_t(at) * t.row_bytes;
        warp_accumulate_row(row_ptr(t, s), delta, t.row_bytes, t.value_kind, lane);
      }
      return;
    }
  }
  if constexpr (VEC != 0) {
    // the fixed-width instantiations serve pure-HBM tables only
    warp_move_rows_vec<VEC, MODE, INDEXED, true>(t, batch_rows, slot, lane, row_index, bases);
    return;
  }
  // vec_bytes is warp-uniform; the host lowers it when a batch pointer is
  // less aligned than the rows.
  switch (t.vec_bytes) {
    case 16: warp_move_rows_vec<16, MODE, INDEXED>(t, batch_rows, slot, lane, row_index, bases); break;
    case 8: warp_move_rows_vec<8, MODE, INDEXED>(t, batch_rows, slot, lane, row_index, bases); break;
    case 4: warp_move_rows_vec<4, MODE, INDEXED>(t, batch_rows, slot, lane, row_index, bases); break;
    case 2: warp_move_rows_vec<2, MODE, INDEXED>(t, batch_rows, slot, lane, row_index, bases); break;
    default: warp_move_rows_vec<1, MODE, INDEXED>(t, batch_rows, slot, lane, row_index, bases); break;
  }
}

// Copies one row with all 32 lanes (used for the few rows that do not follow
// the warp's batch order, e.g. refused inputs leaving through the evicted
// arrays).
template <int VEC = 0>
__device__ __forceinline__ void warp_copy_one_row(const TableView& t, uint8_t* dst,
                                                  const uint8_t* src, uint32_t lane) {
  const uint32_t vec = VEC != 0 ? uint32_t(VEC) : t.vec_bytes;
  const uint32_t cpr = t.chunks_per_row;
  if (vec == 16) {
    for (uint32_t c = lane; c < cpr; c += 32)
      reinterpret_cast<uint4*>(dst)[c] = reinterpret_cast<const uint4*>(src)[c];
  } else if (vec == 8) {
    for (uint32_t c = lane; c < cpr; c += 32)
      reinterpret_cast<uint2*>(dst)[c] = reinterpret_cast<const uint2*>(src)[c];
  } else if (vec == 4) {
    for (uint32_t c = lane; c < cpr; c += 32)
      reinterpret_cast<uint32_t*>(dst)[c] = reinterpret_cast<const uint32_t*>(src)[c];
  } else if (vec == 2) {
    for (uint32_t c = lane; c < cpr; c += 32)
      reinterpret_cast<uint16_t*>(dst)[c] = reinterpret_cast<const uint16_t*>(src)[c];
  } else {
    for (uint32_t c = lane; c < cpr; c += 32) dst[c] = src[c];
  }
}

// ---- the 8-lane bucket probe ----------------------------------------------
//
// One warp serves 32 keys.  Lane l owns key l.  The probe runs in 8 passes; in
// pass j the four 8-lane groups g = lane >> 3 look at keys 4j + g.  A group
// loads its bucket's 128-byte digest line as 8 x 16 bytes (one fully used
// cache line per group, four lines per warp instruction), so a lane holds 16
// digests of slots [16*sub, 16*sub + 16), sub = lane & 7.

struct ProbeLane {
  uint32_t sub;    // lane & 7
  uint32_t group;  // lane >> 3
  uint32_t lane;
};

__device__ __forceinline__ ProbeLane probe_lane() {
  ProbeLane p;
  p.lane = threadIdx.x & 31u;
  p.sub = p.lane & 7u;
  p.group = p.lane >> 3;
  return p;
}

// Owner lane of the key a group looks at in pass j.
__device__ __forceinline__ uint32_t pass_owner(uint32_t j, uint32_t group) {
  return j * kKeysPerPass + group;
}

// Mask of the 8 lanes of this lane's group.
__device__ __forceinline__ uint32_t group_mask(uint32_t group) {
  return 0xFFu << (group * 8u);
}

}  // namespace hkv
