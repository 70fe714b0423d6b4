// Shared device helpers for the sm_100a exact radix top-k indexer:
// order-preserving key map, 64-bit composite (key, ~index), block scans and
// the kernel parameter block.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ff {

constexpr int kThreads = 512;          // threads per CTA for every kernel here
constexpr int kWarps = kThreads / 32;
constexpr int kMaxK = 2048;            // largest supported k
constexpr int kSortCap = 4096;         // survivors the finishing sort can take
constexpr int kCandCap = 4096;         // per-CTA compacted threshold-bin candidates
constexpr int kMaxBins = 8192;         // first-level digit: top 13 key bits
constexpr int kFirstBits = 13;
constexpr int kFirstShift = 32 - kFirstBits;   // key >> kFirstShift is the first digit
constexpr int kFinishBins = 4096;      // bins of the finishing counting sort
constexpr int kMaxCluster = 16;
constexpr int kNumLevels = 6;          // 13+10+9 key bits, 11+11+10 index bits

// Digit layout over the 64-bit composite (key << 32 | ~index).
__host__ __device__ constexpr int level_shift(int l) {
  return l == 0 ? 51 : l == 1 ? 41 : l == 2 ? 32 : l == 3 ? 21 : l == 4 ? 10 : 0;
}
__host__ __device__ constexpr int level_bits(int l) {
  return l == 0 ? 13 : l == 1 ? 10 : l == 2 ? 9 : l == 3 ? 11 : l == 4 ? 11 : 10;
}

// Order-preserving fp32 -> uint32 map: a > b  <=>  key(a) > key(b), with
// -0.0 and +0.0 mapped to the same key and every NaN mapped to the top key
// (the order torch.sort(descending=True) uses).  The reference defines the
// same bit trick as convert_to_uint32 (topk_indexer_radix.cu:236-239) but
// never uses it; its live key is floor(x) (topk_indexer_radix.cu:228-231).
__host__ __device__ __forceinline__ uint32_t key_of_bits(uint32_t u) {
  const uint32_t a = u & 0x7fffffffu;
  if (a == 0u) u = 0u;
  uint32_t k = u ^ (static_cast<uint32_t>(static_cast<int32_t>(u) >> 31) | 0x80000000u);
  if (a > 0x7f800000u) k = 0xffffffffu;
  return k;
}
__device__ __forceinline__ uint32_t key_of(float x) { return key_of_bits(__float_as_uint(x)); }

// Inverse of key_of (up to the -0.0 / NaN canonicalisation).
__host__ __device__ __forceinline__ uint32_t bits_of_key(uint32_t k) {
  return (k & 0x80000000u) ? (k ^ 0x80000000u) : ~k;
}

__device__ __forceinline__ uint64_t make_comp(uint32_t key, int32_t idx) {
  return (static_cast<uint64_t>(key) << 32) | static_cast<uint32_t>(~static_cast<uint32_t>(idx));
}
__device__ __forceinline__ int32_t comp_index(uint64_t c) {
  return static_cast<int32_t>(~static_cast<uint32_t>(c));
}
__device__ __forceinline__ uint32_t comp_key(uint64_t c) { return static_cast<uint32_t>(c >> 32); }

// Score element types.  A row is always cut into 16-byte units (4 fp32 or 8 sixteen-bit scores);
// a 16-bit score is widened to fp32 exactly, so keys, threshold compares and results are those of
// the fp32 row holding the same values (the reference is fp32 only and leaves a half-precision
// value type commented out, topk_indexer_radix.cu:563-564).
template <typename T>
struct Elem;
template <>
struct Elem<float> {
  static constexpr int kPerUnit = 4;
  static constexpr int kLog2Bytes = 2;
  static __device__ __forceinline__ float to_float(float x) { return x; }
  static __device__ __forceinline__ float from_bits16(uint32_t) { return 0.f; }
};
template <>
struct Elem<__nv_bfloat16> {
  static constexpr int kPerUnit = 8;
  static constexpr int kLog2Bytes = 1;
  static __device__ __forceinline__ float from_bits16(uint32_t b) { return __uint_as_float(b << 16); }
  static __device__ __forceinline__ float to_float(__nv_bfloat16 x) { return from_bits16(__bfloat16_as_ushort(x)); }
};
template <>
struct Elem<__half> {
  static constexpr int kPerUnit = 8;
  static constexpr int kLog2Bytes = 1;
  static __device__ __forceinline__ float from_bits16(uint32_t b) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(b)));
  }
  static __device__ __forceinline__ float to_float(__half x) { return __half2float(x); }
};

constexpr int kMaxPeers = 16;
struct PeerPtrs {
  uint32_t* base[kMaxPeers];   // each rank's exchange allocation as mapped in this process
};

struct TopkParams {
  const float* scores;         // [B, row_stride]; bf16 / fp16 rows are passed through this pointer too (the
                               // kernel instantiation knows the element type); row_stride counts elements
  int64_t row_stride;
  const int32_t* lengths;      // [B] (global lengths in context-parallel mode)
  const int32_t* row_starts;   // [B] or null
  const int32_t* idx_map;      // merge mode: explicit index per position (same addressing as scores)
  int32_t seg_len;             // merge mode: position i lives at (i / seg_len) * seg_stride + i % seg_len
  int64_t seg_stride;
  int32_t* out_idx;            // [B, k]
  int64_t* out_idx64;          // [B, k] 64-bit indices instead of out_idx when non-null
  float* out_val;              // [B, k] or null
  int32_t B;
  int32_t k;
  int64_t L_width;
  int64_t shard_offset;        // context-parallel: first global column of this shard
  int32_t fixed_len;           // >= 0: every row has this many positions (merge mode)
  int32_t epilogue;            // FF_EPILOGUE_*
  const int32_t* table;        // page table
  int64_t table_stride;
  const int32_t* cu_seqlens_q; // prefill row -> request map, or null
  int32_t n_table_rows;
  const int32_t* offsets;      // [B] ragged offsets
  int32_t* status;             // optional soft-error word
  const float* hint_in;        // [B] or null: a guess of a value between each row's k-th and 4096-th largest (NaN: none)
  float* hint_out;             // [B] or null: receives such a value for this call's rows (may alias hint_in)
  unsigned char* handover;     // or null: per row kHandoverRowBytes {count, readers, pad to 64 B, uint64 entries[kSortCap]}:
                               // the producer of the scores has already listed every score not below hint_in[row]
  int32_t self_seed;           // 1: a row split over clusters that has no guess makes its own (see seed_own_guess)
  int32_t groups;              // clusters per row (> 1 needs workspace and a cooperative launch)
  uint32_t* workspace;         // zero-filled global scratch, kWsRowWords words per row
  PeerPtrs push_peers;         // context-parallel send: results go to these exchange buffers
  int32_t push_world;          // > 0 switches the push on
  int32_t push_rank;
  int64_t push_slot_words;
  int64_t push_ctrl_offset;    // words from an exchange buffer's start to its control words
  int32_t push_fused;          // 1: the same launch also waits for the peers and merges (single-kernel step)
  int32_t push_sx;             // 1: the step first tries the exchange of survivors (needs push_fused)
  int64_t push_sx_offset;      // words from an exchange buffer's start to its survivor-exchange regions
  int32_t push_prefix;         // candidates per row sent to the peers right away (the first push_prefix of the k);
                               // the rest stay in this rank's own slot until a merge finds that it needs them
  int32_t block_base;          // first CTA of this rank's part of the grid (0 except when several ranks are
  int32_t grid_ctas;           // played by ONE launch on one GPU), and the number of CTAs of that part
  unsigned long long* trace;   // optional stage stamps, [grid CTAs][kTraceSlots] (debug aid)
};

constexpr int kTraceSlots = 40;
constexpr int kHandoverRowBytes = 64 + kSortCap * 8;   // FF_TOPK_HANDOVER_ROW_BYTES

// Stage stamp for the per-CTA timeline: SM cycle counter, thread 0 only.
#define FF_TRACE(p, slot)                                                                 \
  do {                                                                                    \
    if ((p).trace != nullptr && threadIdx.x == 0)                                         \
      (p).trace[static_cast<size_t>(blockIdx.x) * ff::kTraceSlots + (slot)] = clock64();  \
  } while (0)

// Bounds-checked build (-DFF_BOUNDS_CHECK): every data-dependent index into a shared or global
// work array is tested first; an index outside its array sets FF_STATUS_BOUNDS (32) and the number
// of the place in bits 8.. of the status word, and the access is skipped: nothing traps and the
// kernel runs on to its end (its result is then not to be trusted).  It stands in for a memory
// checker on machines where none can be run (the reference's counterpart is a static lint,
// tools/kernel_lint.py:58-163).  In the normal build the test compiles to nothing.
#ifdef FF_BOUNDS_CHECK
__device__ __forceinline__ bool index_in_range(int32_t* status, long long idx, long long n, int place) {
  if (idx >= 0 && idx < n) return true;
  if (status != nullptr) atomicOr(status, 32 | (place << 8));
  return false;
}
#define FF_IN_RANGE(p, idx, n, place) ff::index_in_range((p).status, static_cast<long long>(idx), static_cast<long long>(n), (place))
#else
#define FF_IN_RANGE(p, idx, n, place) true
#endif

// Exclusive suffix sum over the CTA: returns the sum of `v` over all threads
// with a higher thread index; `total` receives the CTA-wide sum.
__device__ __forceinline__ int block_suffix_exclusive(int v, int* warp_tot, int& total) {
  const int lane = threadIdx.x & 31;
  const int wid = threadIdx.x >> 5;
  int s = v;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int t = __shfl_down_sync(0xffffffffu, s, off);
    if (lane + off < 32) s += t;
  }
  if (lane == 0) warp_tot[wid] = s;
  __syncthreads();
  int higher = 0, tot = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) {
    const int x = warp_tot[w];
    tot += x;
    if (w > wid) higher += x;
  }
  total = tot;
  __syncthreads();
  return s - v + higher;
}

}  // namespace ff
