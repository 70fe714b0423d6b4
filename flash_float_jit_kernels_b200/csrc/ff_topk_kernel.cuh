// One thread-block cluster per row: exact radix select on the 64-bit composite
// (monotone fp32 key, ~index) followed by a counting-sort finish.
//
// Role in the reference: replaces topk_kernel<TopK> / fast_topk_split_kv_cuda_tl
// (jit_kernel/csrc/topk_indexer/topk_indexer_radix.cu:554-997) and the
// single-CTA topk_kernel_small_k (jit_kernel/csrc/topk_indexer/top_small_k.cuh:84-348).
// Differences by design: keys are the full order-preserving 32-bit map (any
// fp32 input, not only [0,256)); the first digit is 13 bits; the CTA's chunk is
// streamed through a ring of shared-memory tiles by bulk asynchronous copies and
// stays resident for the second sweep when it fits; per-CTA histograms are
// merged as a reduce-scatter over distributed shared memory followed by a
// cluster-wide suffix scan over unequal slices; nothing is ever dropped (a CTA
// whose threshold-bin candidates do not fit its buffer re-sweeps its chunk
// instead); ties are broken toward the lowest index by continuing the radix
// select into the index bits; the output is in canonical order.
//
// Stages per row (S = cluster barrier; plain CTA barriers when the cluster is 1 CTA):
//   sweep 1   13-bit histogram of the CTA's chunk, tiles arriving by cp.async.bulk
//   S  merge  each CTA sums its slice of bins from every peer's histogram (DSMEM loads)
//      scan   suffix scan of the slice; slice totals to every peer (DSMEM stores)
//   S  find   the CTA whose slice holds the crossing publishes (digit, above, count)
//   S  sweep 2  float compare x >= value(digit) on the tiles; hits -> local stage buffer
//      gather   stage buffer copied into EVERY peer's survivor list (DSMEM stores)
//   S  finish   counting sort on an adaptive linear digit + exact rank inside buckets,
//               ranking shared out over the cluster; first k written to global memory
// When more than kSortCap elements sit at or above the threshold digit, further
// digit levels run on the threshold bin's candidates before the finish.
#pragma once

#include <cooperative_groups.h>
#include <type_traits>

#include "ff_cp_exchange.cuh"
#include "ff_topk_common.cuh"

namespace ff {

namespace cg = cooperative_groups;

// Dynamic shared memory layout (bytes).
constexpr int kSmemHist = 0;                                   // uint32[kMaxBins]
constexpr int kSmemStage = kSmemHist + kMaxBins * 4;           // uint64[kSortCap]; merged slice aliases its head
constexpr int kSmemSort = kSmemStage + kSortCap * 8;           // uint64[kSortCap] survivor list (every CTA)
constexpr int kSmemRing = kSmemSort + kSortCap * 8;            // ring of score tiles; work lists in the finish
constexpr int kSmemCand = kSmemRing;                           // uint64[kCandCap]: deeper levels only, after the ring's last use
// One bulk copy costs about 0.3 us on top of its transfer time and an SM runs
// them one after the other (measured), so tiles are as large as shared memory allows.
#ifndef FF_TOPK_TILE_UNITS
#define FF_TOPK_TILE_UNITS 4096
#endif
constexpr int kTileUnits = FF_TOPK_TILE_UNITS;                 // 16-byte units per tile (64 KiB); a build-time knob for A/B runs
constexpr int kTileBytes = kTileUnits * 16;
static_assert(kTileUnits % kThreads == 0 && kTileUnits / kThreads <= 8, "a thread reads at most 8 units of a tile");
constexpr int kStages = 2;                                     // tiles in the ring (128 KiB)
constexpr int kMinStages = kStages;
constexpr int kMaxStages = kStages;
constexpr int kWaitLimit = 1 << 22;                            // bounded mbarrier polling

// The ring's region also holds the finish's work arrays (106 KiB) and the context-parallel merge's
// staged runs (up to 128 KiB), so it never shrinks below 128 KiB whatever the tile size.
constexpr int kMinRingBytes = 128 * 1024;
__host__ __device__ constexpr int smem_bytes_for(int stages) {
  return kSmemRing + (stages * kTileBytes > kMinRingBytes ? stages * kTileBytes : kMinRingBytes);
}

// ---- distributed shared memory primitives (PTX) ------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
// Address of the same shared-memory location in CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t dsmem_addr(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ uint32_t dsmem_ld_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void dsmem_st_u32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void dsmem_st_u64(uint32_t addr, uint64_t v) {
  asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(addr), "l"(v) : "memory");
}
__device__ __forceinline__ uint32_t dsmem_atomic_add_u32(uint32_t addr, uint32_t v) {
  uint32_t old;
  asm volatile("atom.shared::cluster.add.u32 %0, [%1], %2;" : "=r"(old) : "r"(addr), "r"(v) : "memory");
  return old;
}

// ---- bulk asynchronous copies global -> shared, completion on an mbarrier -----
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
// Polls until the phase with the given parity has completed; gives up after
// kWaitLimit polls and reports false so the caller can flag the launch.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (int i = 0; i < kWaitLimit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

// Geometry of one row as seen by one CTA of the cluster.  The row is cut into
// 16-byte units on absolute addresses so interior units load whole even
// when row_starts or an odd row stride misaligns the window.
template <typename T>
struct Chunk {
  const T* abase;         // 16-byte aligned, abase + mis == first element of the window
  const int32_t* imap;    // merge mode: index plane, addressed like the value plane
  int seg_len;            // merge mode: position i -> (i / seg_len) * seg_stride + i % seg_len
  int64_t seg_stride;
  int pb, pe;             // merge mode: this CTA's positions [pb, pe)
  int mis;                // window position 0 sits in lane `mis` of unit 0
  int len;                // positions in the window
  int fb, fe;             // this CTA's fully valid units [fb, fe)
  bool head, tail;        // this CTA owns the partial first / last unit
  int tail_unit;
};

__device__ __forceinline__ int64_t seg_addr(int i, int seg_len, int64_t seg_stride) {
  const int seg = i / seg_len;
  return static_cast<int64_t>(seg) * seg_stride + (i - seg * seg_len);
}

template <typename T>
__device__ __forceinline__ Chunk<T> make_chunk(const T* row, const int32_t* imap, int len, int C,
                                               int rank, int seg_len, int64_t seg_stride) {
  constexpr int kPU = Elem<T>::kPerUnit;
  Chunk<T> c;
  c.mis = static_cast<int>((reinterpret_cast<uintptr_t>(row) >> Elem<T>::kLog2Bytes) & (kPU - 1));
  c.abase = row - c.mis;
  c.imap = imap;
  c.len = len;
  c.seg_len = seg_len > 0 ? seg_len : 1;
  c.seg_stride = seg_stride;
  {
    const int pper = (len + C - 1) / C;
    c.pb = min(len, rank * pper);
    c.pe = min(len, c.pb + pper);
  }
  const int U = static_cast<int>((static_cast<int64_t>(len) + c.mis + (kPU - 1)) / kPU);
  const bool head_partial = c.mis != 0;
  const bool tail_partial = ((len + c.mis) & (kPU - 1)) != 0;
  const int full_begin = head_partial ? 1 : 0;
  const int full_end = tail_partial ? U - 1 : U;
  const int per = (U + C - 1) / C;
  const int ub = min(U, rank * per);
  const int ue = min(U, ub + per);
  c.fb = max(ub, full_begin);
  c.fe = min(ue, full_end);
  if (c.fe < c.fb) c.fe = c.fb;
  c.head = head_partial && ub == 0 && ue > 0;
  c.tail_unit = U - 1;
  c.tail = tail_partial && !(U - 1 == 0 && head_partial) && ub <= U - 1 && U - 1 < ue;
  return c;
}

// The (at most one) element of a partial first / last unit this thread owns:
// returns its window position or -1, value in x.  Scalar load of a valid lane only.
template <typename T>
__device__ __forceinline__ int partial_element(const Chunk<T>& c, float& x) {
  constexpr int kPU = Elem<T>::kPerUnit;
  int pos = -1;
  if (threadIdx.x < kPU && c.head) {
    pos = static_cast<int>(threadIdx.x) - c.mis;
    if (pos >= 0 && pos < c.len) x = Elem<T>::to_float(c.abase[threadIdx.x]); else pos = -1;
  }
  if (threadIdx.x >= 32 && threadIdx.x < 32 + kPU && c.tail) {
    const int l = static_cast<int>(threadIdx.x) - 32;
    pos = kPU * c.tail_unit - c.mis + l;
    if (pos >= 0 && pos < c.len) x = Elem<T>::to_float(c.abase[kPU * c.tail_unit + l]); else pos = -1;
  }
  return pos;
}

// One 16-byte unit as floats: v[0 .. kPerUnit).
template <typename T>
__device__ __forceinline__ void unpack_unit(const uint4& w, float (&v)[Elem<T>::kPerUnit]) {
  if constexpr (Elem<T>::kPerUnit == 4) {
    v[0] = __uint_as_float(w.x);
    v[1] = __uint_as_float(w.y);
    v[2] = __uint_as_float(w.z);
    v[3] = __uint_as_float(w.w);
  } else {
    const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = Elem<T>::from_bits16(ws[i] & 0xffffu);
      v[2 * i + 1] = Elem<T>::from_bits16(ws[i] >> 16);
    }
  }
}

// Generic (cold) sweep with direct global loads: calls f(x, index) for every
// valid position of the chunk whose raw value passes pre(x).  Used in merge mode
// and on the rare paths (deeper digit levels over a chunk that did not fit the
// candidate buffer).  In merge mode f receives index -1 for ignored entries and
// pre is not applied.
template <bool HAS_MAP, typename T, typename Pre, typename F>
__device__ __forceinline__ void for_each_in_chunk(const Chunk<T>& c, Pre&& pre, F&& f) {
  constexpr int kPU = Elem<T>::kPerUnit;
  if constexpr (HAS_MAP) {
    const T* vals = c.abase + c.mis;
    for (int i = c.pb + threadIdx.x; i < c.pe; i += kThreads) {
      const int64_t a = seg_addr(i, c.seg_len, c.seg_stride);
      f(Elem<T>::to_float(vals[a]), c.imap[a]);
    }
    return;
  }
  const uint4* p4 = reinterpret_cast<const uint4*>(c.abase);
#pragma unroll 1
  for (int u = c.fb + threadIdx.x; u < c.fe; u += kThreads) {
    float v[kPU];
    unpack_unit<T>(__ldg(p4 + u), v);
    const int pos = kPU * u - c.mis;
#pragma unroll
    for (int e = 0; e < kPU; ++e)
      if (pre(v[e])) f(v[e], pos + e);
  }
  float x = 0.f;
  const int pos = partial_element(c, x);
  if (pos >= 0 && pre(x)) f(x, pos);
}

// ---- the hot sweeps: tiles of the chunk stream through a shared-memory ring ----
struct TileStream {
  const float4* src;   // global address of unit fb (16-byte aligned)
  uint32_t ring;       // shared address of the ring
  uint32_t bars;       // shared address of the per-stage "full" mbarriers (8 bytes each)
  uint32_t ebars;      // shared address of the per-stage "empty" mbarriers
  int n_units;         // fe - fb
  int n_tiles;
  bool timed_out;
  // ring bookkeeping, mirrored by every thread (only thread 0 issues copies)
  // (two stages, kept in scalars so that nothing is indexed dynamically)
  int held0, held1;        // tile in each stage, -1 when empty
  int fills0, fills1;      // copies issued into the stage so far
  int fidx0, fidx1;        // index of the copy that brought the held tile (its "full" phase)
  bool arrived0, arrived1; // the held tile's copy has been waited for
  int cons0, cons1;        // "all warps are done with the stage" completions so far
  int passes;              // sweeps done; odd sweeps run in reverse to start on the resident tiles
};
static_assert(kStages == 2, "the ring bookkeeping is written for two stages");

__device__ __forceinline__ int tile_units(const TileStream& s, int t) {
  return min(kTileUnits, s.n_units - t * kTileUnits);
}
__device__ __forceinline__ void issue_tile(const TileStream& s, int t) {
  const int stage = t & 1;
  const uint32_t bytes = static_cast<uint32_t>(tile_units(s, t)) * 16u;
  const uint32_t bar = s.bars + 8u * stage;
  mbar_expect_tx(bar, bytes);
  bulk_load(s.ring + static_cast<uint32_t>(stage) * kTileBytes, s.src + static_cast<size_t>(t) * kTileUnits,
            bytes, bar);
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void stream_init(TileStream& s) {
  s.held0 = s.held1 = -1;
  s.fills0 = s.fills1 = 0;
  s.fidx0 = s.fidx1 = 0;
  s.arrived0 = s.arrived1 = false;
  s.cons0 = s.cons1 = 0;
  s.passes = 0;
  s.timed_out = false;
}

// Puts tile t into its stage (t & 1); every thread records it, thread 0 issues the copy.
__device__ __forceinline__ void stream_fetch(TileStream& s, int t) {
  if (t & 1) {
    s.held1 = t;
    s.fidx1 = s.fills1++;
    s.arrived1 = false;
  } else {
    s.held0 = t;
    s.fidx0 = s.fills0++;
    s.arrived0 = false;
  }
  if (threadIdx.x == 0) issue_tile(s, t);
}

// One sweep over the chunk's tiles; process(tile, t, units) is called by every
// thread once per tile with the tile's shared-memory address.  Sweeps alternate
// direction so that each one starts on the tiles the previous one left in the
// ring; a chunk of at most kStages tiles is copied once and stays resident for
// all later sweeps.  While a tile is processed the next one is in flight: a stage
// is refilled, without any CTA-wide barrier, as soon as every warp has arrived
// on its "empty" mbarrier (one bulk copy at a time is all an SM sustains).
template <typename F>
__device__ __forceinline__ void stream_pass(TileStream& s, F&& process) {
  const int n = s.n_tiles;
  const bool refill = n > kStages;
  const bool reverse = (s.passes & 1) != 0;
  s.passes += 1;
  if (refill || s.held0 < 0) __syncthreads();   // every thread has left the previous sweep before a stage is overwritten
  for (int i = 0; i < min(n, kStages); ++i) {
    const int t = reverse ? n - 1 - i : i;
    if (((t & 1) ? s.held1 : s.held0) != t) stream_fetch(s, t);
  }
#pragma unroll 1
  for (int i = 0; i < n; ++i) {
    const int t = reverse ? n - 1 - i : i;
    const int stage = t & 1;
    if (refill && i >= 1 && i + 1 < n) {
      // the stage used one step ago gets the tile of the next step
      const int prev = stage ^ 1;
      if (threadIdx.x == 0) {
        const int done = (prev ? s.cons1 : s.cons0) - 1;
        if (!mbar_wait(s.ebars + 8u * prev, static_cast<uint32_t>(done & 1))) s.timed_out = true;
      }
      stream_fetch(s, reverse ? t - 1 : t + 1);
    }
    if (!(stage ? s.arrived1 : s.arrived0)) {
      const int fidx = stage ? s.fidx1 : s.fidx0;
      if (!mbar_wait(s.bars + 8u * stage, static_cast<uint32_t>(fidx & 1))) s.timed_out = true;
      if (stage) s.arrived1 = true; else s.arrived0 = true;
    }
    process(s.ring + static_cast<uint32_t>(stage) * kTileBytes, t, tile_units(s, t));
    if (refill) {
      __syncwarp();
      if ((threadIdx.x & 31) == 0) mbar_arrive(s.ebars + 8u * stage);
      if (stage) s.cons1 += 1; else s.cons0 += 1;
    }
  }
}

__device__ __forceinline__ uint4 lds_u4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
// One score of a tile in shared memory: element e of unit lu.
template <typename T>
__device__ __forceinline__ float lds_score(uint32_t tile, int lu, int e) {
  if constexpr (Elem<T>::kPerUnit == 4) {
    float x;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(x) : "r"(tile + 16u * static_cast<uint32_t>(lu) + 4u * e));
    return x;
  } else {
    unsigned short b;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(b) : "r"(tile + 16u * static_cast<uint32_t>(lu) + 2u * e));
    return Elem<T>::from_bits16(b);
  }
}

// A thread's hit mask over its units of one tile: one bit per score, 32 or 64 of them.
template <typename T>
struct HitMask {
  using type = uint32_t;
};
template <>
struct HitMask<__nv_bfloat16> {
  using type = unsigned long long;
};
template <>
struct HitMask<__half> {
  using type = unsigned long long;
};
__device__ __forceinline__ int hit_count(uint32_t m) { return __popc(m); }
__device__ __forceinline__ int hit_count(unsigned long long m) { return __popcll(m); }
__device__ __forceinline__ int first_hit(uint32_t m) { return __ffs(m) - 1; }
__device__ __forceinline__ int first_hit(unsigned long long m) { return __ffsll(static_cast<long long>(m)) - 1; }

// The scores of this thread's units of a tile that are not below vmin, as a bit mask
// (bit j * kPerUnit + e: element e of unit threadIdx.x + j * kThreads).
template <typename T>
__device__ __forceinline__ typename HitMask<T>::type tile_hits(uint32_t tile, int units, float vmin) {
  constexpr int kPU = Elem<T>::kPerUnit;
  using Mask = typename HitMask<T>::type;
  Mask hits = 0;
#pragma unroll
  for (int j = 0; j < kTileUnits / kThreads; ++j) {
    const int lu = static_cast<int>(threadIdx.x) + j * kThreads;
    if (lu < units) {
      float v[kPU];
      unpack_unit<T>(lds_u4(tile + 16u * static_cast<uint32_t>(lu)), v);
      uint32_t h = 0u;
#pragma unroll
      for (int e = 0; e < kPU; ++e) h |= (!(v[e] < vmin) ? 1u : 0u) << e;
      hits |= static_cast<Mask>(h) << (kPU * j);
    }
  }
  return hits;
}

// Raw 13-bit digit of a score: sign | exponent | top 4 mantissa bits of x + 0.0f.
// The add maps -0.0 to +0.0 and every NaN to the canonical 0x7fffffff, so the
// digit needs no further special cases; raw_of_bin() translates between this
// sign-magnitude order and the monotone bin order when the histogram is read.
__device__ __forceinline__ uint32_t raw_digit(float x) { return __float_as_uint(__fadd_rn(x, 0.0f)) >> kFirstShift; }
__device__ __forceinline__ int raw_of_bin(int m) { return m ^ ((m & (kMaxBins >> 1)) ? (kMaxBins >> 1) : (kMaxBins - 1)); }
// the same translation for groups of bins (n groups, n a power of two)
__device__ __forceinline__ int raw_of_group(int m, int n) { return m ^ ((m & (n >> 1)) ? (n >> 1) : (n - 1)); }

// Key and composite of one element; ignored merge entries (index < 0) map to 0.
template <bool HAS_MAP>
__device__ __forceinline__ uint64_t comp_of(float x, int32_t idx) {
  if (HAS_MAP && idx < 0) return 0ull;
  return make_comp(key_of(x), idx);
}

struct ClusterShared {
  int slice_tot[kMaxCluster];
  int res[4];        // threshold digit, count above it, count in it, coarse bin (two-step merge)
  uint32_t coarse[256];   // this CTA's histogram summed in groups of 32 bins, raw order (read by peers)
  int warp_tot[kWarps];
  int stage_count;
  int sort_count;
  int cand_count;
  int push_base;
  int small_count;   // (spare)
  int flag;          // row-barrier result / last-CTA flag
  int big_count;     // elements of large buckets queued in the finish
  uint32_t fin_red[5];   // finish: max / min key, max / min index half, differing key bits of the survivors
  unsigned long long bars[kMaxStages + 1];
  unsigned long long ebars[kMaxStages + 1];
};

// Appends v to list[] with one shared atomic per group of converged lanes.
__device__ __forceinline__ void push_aggregated(uint64_t* list, int* counter, int cap, uint64_t v) {
  const unsigned mask = __activemask();
  const int lane = threadIdx.x & 31;
  const int leader = __ffs(mask) - 1;
  int base = 0;
  if (lane == leader) base = atomicAdd(counter, __popc(mask));
  base = __shfl_sync(mask, base, leader);
  const int pos = base + __popc(mask & ((1u << lane) - 1u));
  if (pos < cap) list[pos] = v;
}

// Everything the per-element classification of one digit level needs.  The
// classification is deliberately NOT inlined: it is the rare path of a sweep and
// one copy keeps the kernel's instruction footprint small.
struct LevelCtx {
  uint64_t Pn;        // candidates have (comp >> shift) == Pn
  uint64_t Pmax;      // this level's winners have Pn < (comp >> shift) <= Pmax
  int shift;
  int nshift;         // next level's digit: (comp >> nshift) & nmask
  uint32_t nmask;
  bool final_level;   // candidates are survivors too
  bool compact;       // copy candidates into the CTA's candidate buffer
  uint32_t* hist;
  uint64_t* stage;
  uint64_t* cand;
  ClusterShared* sh;
};

__device__ __noinline__ void classify_comp(const LevelCtx* c, uint64_t comp) {
  const uint64_t hi = comp >> c->shift;
  if (hi == c->Pn) {
    if (c->final_level) {
      push_aggregated(c->stage, &c->sh->stage_count, kSortCap, comp);
    } else {
      atomicAdd(&c->hist[static_cast<uint32_t>(comp >> c->nshift) & c->nmask], 1u);
      if (c->compact) push_aggregated(c->cand, &c->sh->cand_count, kCandCap, comp);
    }
  } else if (hi > c->Pn && hi <= c->Pmax) {
    push_aggregated(c->stage, &c->sh->stage_count, kSortCap, comp);
  }
}

template <bool HAS_MAP>
__device__ __noinline__ void classify_value(const LevelCtx* c, float x, int32_t idx) {
  classify_comp(c, comp_of<HAS_MAP>(x, idx));
}

// Second sweep over one tile: every value not below vmin is a hit; the hits'
// composites are appended to list[0, cap).  A warp tests its values (32 or 64 per lane)
// with float compares and votes once.  Only a warp that saw a hit assigns list
// slots: the per-lane hit counts are prefix-summed with one ballot per bit plane,
// one lane does the single shared atomic, and each lane then
// walks its own hit bits, re-reading the value from the tile.
template <typename T>
__device__ __forceinline__ void collect_tile(uint32_t tile, int units, int first_unit, int mis, float vmin,
                                             uint64_t* list, int cap, int* counter) {
  constexpr int kPU = Elem<T>::kPerUnit;
  constexpr int kPlanes = kPU == 4 ? 6 : 7;   // counts up to 32 or 64
  const int lane = threadIdx.x & 31;
  auto hits = tile_hits<T>(tile, units, vmin);
  if (__any_sync(0xffffffffu, hits != 0)) {
    const uint32_t n = static_cast<uint32_t>(hit_count(hits));
    const uint32_t lt = (1u << lane) - 1u;
    int before = 0, total = 0;
#pragma unroll
    for (int b = 0; b < kPlanes; ++b) {
      const uint32_t plane = __ballot_sync(0xffffffffu, n & (1u << b));
      before += __popc(plane & lt) << b;
      total += __popc(plane) << b;
    }
    int base = 0;
    if (lane == 0) base = atomicAdd(counter, total);
    base = __shfl_sync(0xffffffffu, base, 0);
    int pos = base + before;
    while (hits != 0) {
      const int e = first_hit(hits);
      hits &= hits - 1;
      const int lu = static_cast<int>(threadIdx.x) + (e / kPU) * kThreads;
      const float x = lds_score<T>(tile, lu, e & (kPU - 1));
      if (pos < cap) list[pos] = make_comp(key_of(x), kPU * (first_unit + lu) - mis + (e & (kPU - 1)));
      ++pos;
    }
  }
}

// Like collect_tile, but every value not below vmin is handed to on_hit(x, position)
// instead of being stored: used by the sweeps of the second digit level, where a
// hit is either counted in the next histogram or stored after an exact test.
template <typename T, typename F>
__device__ __forceinline__ void scan_tile(uint32_t tile, int units, int first_unit, int mis, float vmin,
                                          F&& on_hit) {
  constexpr int kPU = Elem<T>::kPerUnit;
  auto hits = tile_hits<T>(tile, units, vmin);
  while (hits != 0) {
    const int e = first_hit(hits);
    hits &= hits - 1;
    const int lu = static_cast<int>(threadIdx.x) + (e / kPU) * kThreads;
    on_hit(lds_score<T>(tile, lu, e & (kPU - 1)), kPU * (first_unit + lu) - mis + (e & (kPU - 1)));
  }
}

// ---- rows split over several clusters: global scratch and row-wide barriers ----
// Per-row scratch in global memory (all zero between launches; the kernel
// leaves it zeroed).  Word offsets:
//   [0, 6)   arrivals at the histogram barrier of digit level 0..5
//   [6]      arrivals at the survivor barrier      [7] CTAs that are done
//   [8]      survivors appended so far
//   [10,11]  hinted attempt: one 64-bit word, low half survivors appended, high half CTAs that have reserved
//   [64, 320) first digit level only: the row's histogram summed in groups of 32 bins
//   [320, 320 + 6 * 8192)        one 8192-bin global histogram per digit level
//   [320 + 6 * 8192, + 2 * 4096) survivor list (4096 x 64-bit composites), then a second one for a hinted
//                                attempt.  Both are zero between launches: an entry is valid once it is
//                                non-zero (no composite is zero), so readers need no barrier after the writes
//   then 64 words                a row that seeds its own threshold guess: one 64-bit accumulator of the
//                                CTAs' estimates (sum of keys, CTAs with an estimate, CTAs reported)
constexpr int kWsCoarseWord = 64;            // 256 coarse bins (sums of 32 first-level bins) of the row
constexpr int kWsHeaderWords = 64 + 256;
constexpr int kWsHistWords = kNumLevels * kMaxBins;
constexpr int kWsListWords = 2 * kSortCap;     // one survivor list (64-bit composites)
constexpr int kWsSeedWord = kWsHeaderWords + kWsHistWords + 2 * kWsListWords;   // 64-bit accumulator of the CTAs' own threshold estimates
constexpr int kWsSeedWords = 64;
static_assert(kWsSeedWord % 2 == 0, "the accumulator is a 64-bit word");
constexpr int kWsRowWords = kWsSeedWord + kWsSeedWords;
constexpr int kSpinLimit = 1 << 21;   // bounded polling of a row barrier (about a second)

// All `expected` CTAs of a row meet here (they are co-resident: cooperative
// launch).  Thread 0 publishes this CTA's earlier global writes and polls the
// arrival counter; returns false if the poll limit ran out.
__device__ __forceinline__ bool row_barrier(uint32_t* counter, uint32_t expected, int* flag) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(counter, 1u);
    int ok = 0;
    for (int i = 0; i < kSpinLimit; ++i) {
      uint32_t v;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
      if (v >= expected) {
        ok = 1;
        break;
      }
    }
    *flag = ok;
  }
  __syncthreads();
  return *flag != 0;
}

// Copies the first n entries of a global survivor list into shared memory.  The list is zero
// between launches and no composite is zero, so an entry is valid as soon as it is non-zero:
// each thread polls its own entries (bounded), and no barrier or fence follows the writers.
__device__ __forceinline__ bool load_list_validated(const uint64_t* glist, int n, uint64_t* dst) {
  // all of a thread's entries are requested before the first one is looked at (the list has at
  // most kSortCap entries: kSortCap / kThreads per thread); only missing ones are polled again
  constexpr int kPer = kSortCap / kThreads;
  unsigned long long v[kPer];
#pragma unroll
  for (int j = 0; j < kPer; ++j) {
    const int i = static_cast<int>(threadIdx.x) + j * kThreads;
    v[j] = 1ull;
    if (i < n) asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v[j]) : "l"(glist + i));
  }
  bool ok = true;
#pragma unroll
  for (int j = 0; j < kPer; ++j) {
    const int i = static_cast<int>(threadIdx.x) + j * kThreads;
    if (i < n) {
      for (int spin = 0; v[j] == 0ull && spin < kSpinLimit; ++spin)
        asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v[j]) : "l"(glist + i) : "memory");
      if (v[j] == 0ull) ok = false;
      dst[i] = v[j];
    }
  }
  return ok;
}

// Cluster-wide histogram merge (reduce-scatter over distributed shared memory)
// and suffix scan over the per-CTA slices.  On return every CTA's sh.res holds
// the digit t with  #(digit > t) < r <= #(digit >= t), and those two counts.
// raw0: the histogram is indexed by raw_digit() (first level of the fast path).
// `merged` must not alias `hist`; with a single CTA the histogram is scanned in place.
__device__ __forceinline__ void merge_and_scan(cg::cluster_group& cluster, int C, int rank,
                                               uint32_t* hist, uint32_t* merged, int nbins, int r,
                                               bool raw0, ClusterShared& sh, const TopkParams& p, bool tr,
                                               int G, uint32_t* ws, int level, bool& timed_out,
                                               int counted = -1) {
  // counted: how many elements the histograms of the whole row hold at this level (first level: the
  // row's length), or -1 if not known
  const int tid = threadIdx.x;
  int slice_n = nbins / C;
  int slice_base = rank * slice_n;
  const bool wide_slice = slice_n >= kThreads;   // every thread owns whole bins of the slice
  if (C > 1 && !wide_slice) {
    for (int i = tid; i < slice_n; i += kThreads) merged[i] = 0u;
  }
  if (tid == 0) sh.res[0] = -1;
  if (C > 1) cluster.sync(); else __syncthreads();   // every CTA's local histogram is complete
  if (tr) FF_TRACE(p, 26);
  if (C > 1) {
    // nbins loads per CTA in total, all issued before the first use.
    const uint32_t hist_local = smem_addr(hist);
    const int n_iter = nbins / kThreads;   // 16 for 8192 bins, 2 for 1024, 1 for 512, 4 for 2048
    uint32_t v[kMaxBins / kThreads];
    if (wide_slice) {
      // load j = m * C + c: bin (tid + m * kThreads) of my slice from peer c; the C loads of a bin
      // sit next to each other in v[], so a log-step reduction with static indices sums them
      int log2c = 0;
      while ((1 << log2c) < C) ++log2c;
#pragma unroll
      for (int j = 0; j < kMaxBins / kThreads; ++j) {
        if (j < n_iter) {
          int b = slice_base + tid + (j >> log2c) * kThreads;
          if (raw0) b = raw_of_bin(b);
          v[j] = dsmem_ld_u32(dsmem_addr(hist_local + 4u * static_cast<uint32_t>(b), j & (C - 1)));
        } else {
          v[j] = 0u;
        }
      }
#pragma unroll
      for (int step = 1; step < kMaxCluster; step <<= 1) {
        if (step < C) {
#pragma unroll
          for (int j = 0; j < kMaxBins / kThreads; j += 2 * step) v[j] += v[j + step];
        }
      }
#pragma unroll
      for (int j = 0; j < kMaxBins / kThreads; ++j) {
        if (j < n_iter && (j & (C - 1)) == 0) merged[tid + (j >> log2c) * kThreads] = v[j];
      }
    } else {
      // narrow slices (later digit levels): flat index -> (peer, bin of my slice), summed with shared atomics
#pragma unroll
      for (int j = 0; j < kMaxBins / kThreads; ++j) {
        if (j < n_iter) {
          const int flat = tid + j * kThreads;
          const int peer = flat / slice_n;
          int b = slice_base + (flat - peer * slice_n);
          if (raw0) b = raw_of_bin(b);
          v[j] = dsmem_ld_u32(dsmem_addr(hist_local + 4u * static_cast<uint32_t>(b), peer));
        }
      }
#pragma unroll
      for (int j = 0; j < kMaxBins / kThreads; ++j) {
        if (j < n_iter) {
          const int flat = tid + j * kThreads;
          if (v[j] != 0u) atomicAdd(&merged[flat % slice_n], v[j]);
        }
      }
    }
    __syncthreads();
  }
  if (tr) FF_TRACE(p, 27);
  // slice value i: merged[i], or (single CTA) the histogram itself in monotone order
  bool from_merged = C > 1;
  auto slice_at = [&](int i) -> int {
    if (from_merged) return static_cast<int>(merged[i]);
    return static_cast<int>(hist[raw0 ? raw_of_bin(i) : i]);
  };
  if (G > 1) {
    // Cross-cluster step: the cluster's merged slices are added into the row's
    // global histogram (L2 atomics carry only the G-way part of the merge), all
    // CTAs of the row meet, and every CTA reads the whole histogram back.
    uint32_t* gh = ws + kWsHeaderWords + level * kMaxBins;
    for (int i = tid; i < slice_n; i += kThreads) {
      const int v = slice_at(i);
      if (v != 0) atomicAdd(&gh[slice_base + i], static_cast<uint32_t>(v));
    }
    // first level: also a coarse view (groups of 32 bins), so that after the barrier a CTA reads
    // 256 + 32 words instead of the whole histogram
    const bool two_step = level == 0 && nbins == kMaxBins;
    const bool self_counting = two_step && counted >= 0;
    if (self_counting) {
      // No arrival counter: every CTA orders its fine-bin additions before its coarse sums, and the
      // coarse sums of the row add up to `counted` exactly when every CTA's have landed.
      __threadfence();
      __syncthreads();
    }
    if (two_step) {
      const int lane = tid & 31;
      // release side of the hand-over: the lane that publishes a coarse sum fences first, after the
      // CTA barrier that ordered every thread's fine-bin additions before it
      if (self_counting && lane == 0) __threadfence();
      for (int g = tid >> 5; g < slice_n / 32; g += kWarps) {
        const uint32_t sum = __reduce_add_sync(0xffffffffu, static_cast<uint32_t>(slice_at(32 * g + lane)));
        if (lane == 0 && sum != 0u) atomicAdd(ws + kWsCoarseWord + slice_base / 32 + g, sum);
      }
    }
    if (!self_counting) {
      if (!row_barrier(ws + level, static_cast<uint32_t>(G * C), &sh.flag)) timed_out = true;
    }
    if (two_step) {
      int val = 0, total = 0, excl = 0;
      if (self_counting) {
        // the poll is the coarse scan itself: read, sum, repeat until the sum is complete (bounded)
        bool complete = false;
        for (int spin = 0; spin < (kSpinLimit >> 6) && !complete; ++spin) {
          uint32_t w = 0u;
          // acquire: a complete coarse sum makes the fine bins added before it visible (the CTA
          // barriers of the scan below carry that on to the lanes that read the fine bins)
          if (tid < 256) asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(w) : "l"(ws + kWsCoarseWord + tid) : "memory");
          val = static_cast<int>(w);
          excl = block_suffix_exclusive(val, sh.warp_tot, total);
          complete = total == counted;
        }
        if (!complete) timed_out = true;
      } else {
        val = tid < 256 ? static_cast<int>(__ldcg(ws + kWsCoarseWord + tid)) : 0;
        excl = block_suffix_exclusive(val, sh.warp_tot, total);
      }
      if (tid < 256 && excl < r && r <= excl + val) {
        sh.res[3] = tid;
        sh.res[1] = excl;
      }
      __syncthreads();
      if (total < r) return;   // no crossing: res[0] stays -1 for every CTA of the row
      const int cbin = sh.res[3];
      const int above_c = sh.res[1];
      __syncthreads();
      if (tid < 32) {
        const int cnt = static_cast<int>(__ldcg(&gh[cbin * 32 + tid]));
        int incl = cnt;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
          const int t = __shfl_down_sync(0xffffffffu, incl, off);
          if (tid + off < 32) incl += t;
        }
        const int above = above_c + incl - cnt;
        if (above < r && r <= above + cnt) {
          sh.res[1] = above;
          sh.res[2] = cnt;
          sh.res[0] = cbin * 32 + tid;
        }
      }
      __syncthreads();
      return;
    }
    for (int i = tid; i < nbins; i += kThreads) merged[i] = __ldcg(&gh[i]);
    __syncthreads();
    from_merged = true;
    slice_n = nbins;
    slice_base = 0;
  }
  const bool publish_remote = C > 1 && G == 1;
  const int per = slice_n >= kThreads ? slice_n / kThreads : 1;
  const int first = tid * per;
  int local = 0;
  if (first < slice_n) {
    // a thread's `per` consecutive bins are read in a rotated order (the sum does not care)
    // so that the lanes of a warp hit distinct banks
    const int rot = per <= 32 ? (tid & 31) / (32 / per) : 0;
    for (int e = 0; e < per; ++e) local += slice_at(first + ((e + rot) & (per - 1)));
  }
  int total;
  const int excl = block_suffix_exclusive(local, sh.warp_tot, total);
  if (tr) FF_TRACE(p, 28);
  if (publish_remote) {
    if (tid < C) dsmem_st_u32(dsmem_addr(smem_addr(&sh.slice_tot[rank]), tid), static_cast<uint32_t>(total));
    cluster.sync();  // slice totals of every CTA have arrived
  }
  if (tr) FF_TRACE(p, 29);
  int above_slice = 0;
  if (publish_remote) {
    for (int c = rank + 1; c < C; ++c) above_slice += sh.slice_tot[c];
  }
  // only the one thread whose bins hold the crossing walks them
  if (first < slice_n && above_slice + excl < r && r <= above_slice + excl + local) {
    int running = above_slice + excl;
    for (int e = per - 1; e >= 0; --e) {
      const int cnt = slice_at(first + e);
      const int next = running;
      running += cnt;
      if (next < r && r <= running) {
        if (publish_remote) {
          for (int c = 0; c < C; ++c) {
            const uint32_t a = dsmem_addr(smem_addr(&sh.res[0]), c);
            dsmem_st_u32(a + 4, static_cast<uint32_t>(next));
            dsmem_st_u32(a + 8, static_cast<uint32_t>(cnt));
            dsmem_st_u32(a, static_cast<uint32_t>(slice_base + first + e));
          }
        } else {
          sh.res[1] = next;
          sh.res[2] = cnt;
          sh.res[0] = slice_base + first + e;
        }
      }
    }
  }
  if (tr) FF_TRACE(p, 30);
  if (publish_remote) cluster.sync(); else __syncthreads();   // the threshold triple has arrived everywhere
}

// First-digit merge for a row inside ONE cluster, without any exchange of partial
// results: after a single cluster barrier every CTA (1) reads a 256-bin coarse view
// (sums of 32 bins) of every peer's histogram over DSMEM and finds the coarse bin
// that holds the crossing, then (2) reads that coarse bin's 32 fine bins from every
// peer and finds the threshold digit.  Every CTA computes the same triple, so the
// two cluster barriers and the slice-total / result stores of merge_and_scan are
// not needed, and a CTA issues 8 + 1 remote loads per thread instead of 16.
// `scratch` needs 512 + 32 * C words.  The peers' histograms must stay untouched
// until the next cluster barrier.
__device__ __forceinline__ void merge_two_step(cg::cluster_group& cluster, int C, uint32_t* hist,
                                               uint32_t* scratch, int r, ClusterShared& sh,
                                               const TopkParams& p) {
  constexpr int kCoarse = 256;
  constexpr int kFinePer = kMaxBins / kCoarse;   // 32
  static_assert(kFinePer == 32 && kThreads == 2 * kCoarse, "layout of the two-step merge");
  const int tid = threadIdx.x;
  uint32_t* gcoarse = scratch;         // [2][256] sums over one half of the peers each
  uint32_t* gfine = scratch + 512;     // [C][32]
  {
    // local coarse sums: 16 consecutive words per thread, read in a rotated order (distinct banks)
    const int rot = (tid & 31) >> 1;
    uint32_t sum = 0;
#pragma unroll
    for (int e = 0; e < 16; ++e) sum += hist[16 * tid + ((e + rot) & 15)];
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    if ((tid & 1) == 0) sh.coarse[tid >> 1] = sum;
  }
  if (tid == 0) sh.res[0] = -1;
  cluster.sync();   // every CTA's histogram and coarse sums are complete
  FF_TRACE(p, 26);
  {
    const int g = tid & (kCoarse - 1);
    const int half = tid >> 8;
    const int per_half = C >> 1;
    const uint32_t a = smem_addr(&sh.coarse[g]);
    uint32_t v[kMaxCluster / 2];
#pragma unroll
    for (int j = 0; j < kMaxCluster / 2; ++j) v[j] = j < per_half ? dsmem_ld_u32(dsmem_addr(a, half * per_half + j)) : 0u;
    uint32_t sum = 0;
#pragma unroll
    for (int j = 0; j < kMaxCluster / 2; ++j) sum += v[j];
    gcoarse[half * kCoarse + g] = sum;
  }
  __syncthreads();
  FF_TRACE(p, 27);
  int val = 0;
  if (tid < kCoarse) {
    const int g = raw_of_group(tid, kCoarse);   // coarse bins in monotone order
    val = static_cast<int>(gcoarse[g] + gcoarse[kCoarse + g]);
  }
  int total;
  const int excl = block_suffix_exclusive(val, sh.warp_tot, total);
  if (tid < kCoarse && excl < r && r <= excl + val) {
    sh.res[3] = tid;
    sh.res[1] = excl;
  }
  __syncthreads();
  FF_TRACE(p, 28);
  if (total < r) return;   // no crossing: res[0] stays -1 (uniform over the cluster)
  const int cbin = sh.res[3];
  const int above_c = sh.res[1];
  if (tid < kFinePer * C) {
    const int f = tid & (kFinePer - 1);
    const int peer = tid >> 5;
    const int b = raw_of_bin(cbin * kFinePer + f);
    gfine[tid] = dsmem_ld_u32(dsmem_addr(smem_addr(hist) + 4u * static_cast<uint32_t>(b), peer));
  }
  __syncthreads();
  FF_TRACE(p, 29);
  if (tid < 32) {
    int cnt = 0;
    for (int c = 0; c < C; ++c) cnt += static_cast<int>(gfine[c * kFinePer + tid]);
    int incl = cnt;   // inclusive suffix sum over the lanes (higher lane = larger values)
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int t = __shfl_down_sync(0xffffffffu, incl, off);
      if (tid + off < 32) incl += t;
    }
    const int above = above_c + incl - cnt;
    if (above < r && r <= above + cnt) {
      sh.res[1] = above;
      sh.res[2] = cnt;
      sh.res[0] = cbin * kFinePer + tid;
    }
  }
  __syncthreads();
  FF_TRACE(p, 30);
}

// Context-parallel exchange of survivors: regions of one (step parity, sending rank, row).
constexpr int kSxRegions = 128;                 // one per CTA of the sending rank's row (unused ones are sent empty)
constexpr int kSxCap = 64;                      // entries per region
constexpr int kSxRegionWords = 4 + 4 * kSxCap;  // header {count | flags, step, guess key, step} + 16-byte entries
constexpr uint32_t kSxFallbackFlag = 1u << 16;

// ---- a row seeds its own threshold guess ----------------------------------------------------
// A threshold guess (a score between the row's k-th and 4096-th largest) lets the row be selected in
// one sweep without histogram, merge or second sweep.  When the caller has none and the row is
// spread over many CTAs, the row makes one: every CTA estimates, from the first tile of its own
// chunk, the score that about `target` scores of the whole row reach; the CTAs add their
// estimates into one word of the row's global scratch, and all take the mean.  If the
// guess does not fit, the row falls back to the histogram path like after any other guess, so
// the result stays exact; only rows whose chunks look alike (no trend along the row) profit.
//
// The estimate of one CTA: each of its threads keeps the largest of the few scores it reads (g of
// them); with p = target / length, a thread's largest reaches the wanted score v with probability
// q = 1 - (1 - p)^g, so about rho = threads * q of them do, and the rho-th largest of the threads'
// maxima estimates v.  The CTA's 32 largest maxima come out of a bitonic sort inside every warp
// and four rounds of pairwise bitonic merges that keep the upper 32.
struct SeedPlan {
  bool use;        // uniform over all CTAs of the row
  float p;         // target / length
  int n_use;       // 16-byte units of a CTA's first tile that it looks at
};
// Row-level decision, from quantities every CTA of the row computes alike.
// len_for_p: the length the target count refers to (the whole row's in a context-parallel step,
// where `len` is the shard's).
__device__ __forceinline__ SeedPlan seed_plan(int len, int mis, int per_unit, int n_share, int k, int len_for_p = 0,
                                              int ranks = 1) {
  SeedPlan sp;
  sp.use = false;
  // hint_target_rank(k) for one rank.  Several ranks' guesses side by side: the list must hold k
  // entries not below the LARGEST guess, which sits a standard deviation or two above the rest, so
  // aim half-way between k and the list's capacity.
  const int target = ranks > 1 ? min(k + (k >> 1), kSortCap - (kSortCap >> 3))
                               : min(k + (k >> 2) + 64, kSortCap - (kSortCap >> 3));
  if (len_for_p <= 0) len_for_p = len;
  sp.p = static_cast<float>(target) / static_cast<float>(len_for_p);
  sp.n_use = 0;
  if (n_share > kThreads || len_for_p < 4 * target) return sp;   // (the accumulator's counters hold up to 1023)
  const int U = static_cast<int>((static_cast<int64_t>(len) + mis + per_unit - 1) / per_unit);
  const int per = (U + n_share - 1) / n_share;          // units per CTA, as make_chunk cuts them
  int n0 = min(per, kTileUnits);                        // units of a CTA's first tile
  if (n0 < 64) return sp;
  auto rho_of = [&](int units) {
    const int lanes = min(kThreads, units);
    const float g = static_cast<float>(per_unit) * static_cast<float>(units) / static_cast<float>(lanes);
    return static_cast<float>(lanes) * (1.f - __expf(g * log1pf(-sp.p)));
  };
  float rho = rho_of(n0);
  if ((rho < 4.5f || rho * static_cast<float>(n_share) * static_cast<float>(ranks) < 400.f) && per > kTileUnits) {
    // a very long row (few of a tile's scores reach the target), or a row on few CTAs (too few
    // hits in all for a steady mean): look at the first TWO tiles, which lie side by side in the ring
    n0 = min(per, 2 * kTileUnits);
    rho = rho_of(n0);
  }
  if (rho > 26.f) {
    // more hits than the kept 32 can show: look at a part of the tile only (a multiple of the
    // thread count, so that every thread reads the same number of units)
    n0 = max(kThreads, (static_cast<int>(static_cast<float>(n0) * 24.f / rho) / kThreads) * kThreads);
    rho = rho_of(n0);
  }
  sp.n_use = n0;
  // a usable order statistic inside the kept 32, and enough hits over the row for a steady mean
  // (relative noise of the row's survivor count about 1.25 / sqrt(hits): 6 % at 400 hits, against a
  // window of -22 % .. +56 % around the target)
  // In a context-parallel step the `ranks` guesses are used side by side (every rank's own
  // for its own shard), so the row's count averages over all of them; a single rank's guess may be
  // noisier (it only shifts the largest guess, which the final check allows for).
  const float hits = rho * static_cast<float>(n_share);
  sp.use = rho >= 3.f && rho <= 30.f && hits * static_cast<float>(ranks) >= 400.f && hits >= 100.f;
  return sp;
}

// Brings the part of the chunk the plan wants looked at into the ring (its first tile; the second
// one too for very long rows) and returns how many 16-byte units of it are there.  `ring_busy`:
// threads may still be reading the ring (a barrier is needed before it is overwritten).
__device__ __forceinline__ int seed_sample_ready(TileStream& ts, const SeedPlan& sp, bool ring_busy) {
  if (ts.n_tiles <= 0) return 0;
  const bool two = sp.n_use > kTileUnits && ts.n_tiles > 1;
  const bool need0 = ts.held0 != 0, need1 = two && ts.held1 != 1;
  if (ring_busy && (need0 || need1)) __syncthreads();
  if (need0) stream_fetch(ts, 0);
  if (need1) stream_fetch(ts, 1);
  if (!ts.arrived0) {
    if (!mbar_wait(ts.bars, static_cast<uint32_t>(ts.fidx0 & 1))) ts.timed_out = true;
    ts.arrived0 = true;
  }
  int n = tile_units(ts, 0);
  if (two) {
    if (!ts.arrived1) {
      if (!mbar_wait(ts.bars + 8u, static_cast<uint32_t>(ts.fidx1 & 1))) ts.timed_out = true;
      ts.arrived1 = true;
    }
    n += tile_units(ts, 1);
  }
  return min(n, sp.n_use);
}

struct SeedResult {
  float guess;
  int code;   // 1: a guess, 0: none, 2: none and a bounded wait ran out
};
// tile0: shared address of the chunk's first tile (landed; the second one behind it when n0 exceeds a
// tile), n0: the 16-byte units to look at.
template <typename T>
// tr: this CTA's trace slots or nullptr; slots 5, 6, 7 get the GLOBAL timer (ns, comparable between
// SMs, unlike the cycle stamps of the other slots) when the sample has landed, when this CTA's
// estimate goes out, and when all CTAs' estimates are in.
__device__ __noinline__ SeedResult seed_own_guess(uint32_t tile0, int n0, int* flag, uint32_t* scratch, uint32_t* ws,
                                                  float p_frac, int n_share, int my_share,
                                                  unsigned long long* tr = nullptr) {
  constexpr int kPU = Elem<T>::kPerUnit;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int w = tid >> 5;
  uint32_t* sorted = scratch + 32;       // [kWarps][32] (scratch[0]: the result, handed to all threads)
  SeedResult res;
  res.guess = 0.f;
  res.code = 0;
  if (tr != nullptr && tid == 0) tr[5] = global_ns();
  // Where in the CTA's sorted maxima the estimate is read (depends on the sample's size only, so
  // it is worked out here, off the chain sample -> sort -> estimate).
  // The (i+1)-th largest maximum has i + 1 maxima at or above it; the MEAN over the CTAs of the
  // score at a random such count sits where the count is about half a step smaller (the tail
  // is convex), so the estimate is read at the fractional position rho - 0.5 (0-based),
  // between two neighbours of the sorted list, which also removes the rounding of rho.
  const int lanes = min(kThreads, n0);
  float pos = 0.f;
  if (lanes >= 32) {
    const float g = static_cast<float>(kPU) * static_cast<float>(n0) / static_cast<float>(lanes);
    const float rho = static_cast<float>(lanes) * (1.f - __expf(g * log1pf(-p_frac)));
    pos = fminf(fmaxf(rho - 0.5f, 0.f), 30.99f);
  }
  // ---- largest score per thread over the first tile of the chunk ----
  uint32_t mkey = 0u;
  if (n0 > 0) {
    float m = __uint_as_float(0xff800000u);
    bool any = false;
#pragma unroll
    for (int j = 0; j < 2 * kTileUnits / kThreads; ++j) {   // (the ring's two stages are contiguous)
      const int lu = tid + j * kThreads;
      if (lu < n0) {
        float v[kPU];
        unpack_unit<T>(lds_u4(tile0 + 16u * static_cast<uint32_t>(lu)), v);
#pragma unroll
        for (int e = 0; e < kPU; ++e) m = fmaxf(m, v[e]);   // (NaN scores are left out of the estimate)
        any = true;
      }
    }
    if (any) mkey = key_of(m);
  }
  // ---- the CTA's 32 largest thread maxima, descending ----
#pragma unroll
  for (int k2 = 2; k2 <= 32; k2 <<= 1) {
#pragma unroll
    for (int j = k2 >> 1; j > 0; j >>= 1) {
      const uint32_t o = __shfl_xor_sync(0xffffffffu, mkey, j);
      const bool keep_max = ((lane & j) == 0) == ((lane & k2) == 0);
      mkey = keep_max ? max(mkey, o) : min(mkey, o);
    }
  }
  sorted[w * 32 + lane] = mkey;
  __syncthreads();
#pragma unroll 1
  for (int stride = 1; stride < kWarps; stride <<= 1) {
    if ((w & (2 * stride - 1)) == 0) {
      // upper 32 of two descending lists: pair element i of one with element 31 - i of the other, keep
      // the larger (a bitonic sequence), and sort it again with one bitonic merge
      uint32_t v = max(mkey, sorted[(w + stride) * 32 + 31 - lane]);
#pragma unroll
      for (int j = 16; j > 0; j >>= 1) {
        const uint32_t o = __shfl_xor_sync(0xffffffffu, v, j);
        v = ((lane & j) == 0) ? max(v, o) : min(v, o);
      }
      mkey = v;
      sorted[w * 32 + lane] = v;
    }
    __syncthreads();
  }
  // ---- this CTA's estimate: the rho-th largest thread maximum, added to the row's accumulator ----
  // One 64-bit word per row collects all estimates: bits 0..43 the sum of the estimates' keys, bits
  // 44..53 how many CTAs gave one, bits 54..63 how many CTAs have reported at all.  One atomic
  // per CTA adds all three, so a reader sees them consistently, and one thread per CTA polls the
  // single word until every CTA has reported (many threads polling many words cost several
  // microseconds here: the pollers crowd out the writers in L2).
  unsigned long long* acc = reinterpret_cast<unsigned long long*>(ws + kWsSeedWord);
  if (tid == 0) {
    unsigned long long add = 1ull << 54;
    if (lanes >= 32) {
      const int i0 = static_cast<int>(pos);
      const uint32_t k0 = sorted[i0], k1 = sorted[i0 + 1];
      uint32_t key = k0;
      if (k1 != 0u && k1 <= k0) key = k0 - static_cast<uint32_t>((pos - static_cast<float>(i0)) * static_cast<float>(k0 - k1));
      // (keys above +inf's are NaN patterns, key 0 means too few threads had a score: no estimate)
      if (key != 0u && key <= 0xff800000u) add |= (1ull << 44) | key;
    }
    if (tr != nullptr) tr[6] = global_ns();
    atomicAdd(acc, add);
    unsigned long long v = 0ull;
    int spin = 0;
    for (; spin < kSpinLimit; ++spin) {
      asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(acc) : "memory");
      if (static_cast<int>(v >> 54) >= n_share) break;
    }
    if (tr != nullptr) tr[7] = global_ns();
    const int valid = static_cast<int>((v >> 44) & 1023ull);
    // the mean of the keys (keys are close to linear in the score over so narrow a range)
    uint32_t mean = 0u;
    if (spin < kSpinLimit && 2 * valid >= n_share) mean = static_cast<uint32_t>((v & ((1ull << 44) - 1ull)) / static_cast<unsigned long long>(valid));
    *flag = spin < kSpinLimit ? 1 : 0;
    scratch[0] = mean;
  }
  __syncthreads();
  const uint32_t mean = scratch[0];
  const bool ok = *flag != 0;
  __syncthreads();
  if (!ok) res.code = 2;
  if (ok && mean != 0u) {
    res.guess = __uint_as_float(bits_of_key(mean));
    res.code = 1;
  }
  return res;
}

// How many scores the next call's guess should let through: between k (fewer is a miss) and
// kSortCap (more is a miss), nearer to k because the finish costs grow with the square of it.
__device__ __forceinline__ int hint_target_rank(int k) { return min(k + (k >> 2) + 64, kSortCap - (kSortCap >> 3)); }

// Context-parallel send: the step of this launch and where its entries go in a peer's buffer.
struct PushCtx {
  int64_t off;     // words from a peer's base to this rank's slot of this step's parity
  uint32_t step;
};

// Writes output slot j of `row` from a window-relative index (or -1) and key.
// In push mode (context-parallel send) the slot is not written locally at all: the (value,
// global index) pair goes straight into this rank's slot of every peer's receive buffer.

template <bool PUSH, bool VALUES = true>
__device__ __forceinline__ void emit(const TopkParams& p, const PushCtx& push, int row, int j, int32_t idx,
                                     uint32_t key, bool is_map, int table_row) {
  if (PUSH) {
    // one self-validating 16-byte entry per peer: {value bits, step, global index, step}
    const uint32_t vbits = idx < 0 ? kNoCandidateBits : bits_of_key(key);
    const uint32_t gidx = idx < 0 ? 0xffffffffu : static_cast<uint32_t>(idx + p.shard_offset);
    const size_t at = push.off + 4 * (static_cast<size_t>(row) * p.k + j);
    // This rank's own slot gets every candidate; the peers get the first push_prefix of the run
    // now, and the rest only if a merge finds that the prefixes do not hold the whole top-k.
    st_entry(p.push_peers.base[p.push_rank] + at, vbits, gidx, push.step);
    if (j < p.push_prefix) {
      for (int q = 0; q < p.push_world; ++q)
        if (q != p.push_rank) st_entry(p.push_peers.base[q] + at, vbits, gidx, push.step);
    }
    return;
  }
  int32_t o;
  if (idx < 0) {
    o = -1;
  } else if (p.epilogue == 1) {
    o = p.table[static_cast<int64_t>(table_row) * p.table_stride + idx];
  } else if (p.epilogue == 2) {
    o = idx + p.offsets[row];
  } else {
    o = is_map ? idx : static_cast<int32_t>(idx + p.shard_offset);
  }
  if (!FF_IN_RANGE(p, j, p.k, 9) || !FF_IN_RANGE(p, row, p.B, 10)) return;
  if (p.out_idx64 != nullptr) p.out_idx64[static_cast<int64_t>(row) * p.k + j] = o;
  else p.out_idx[static_cast<int64_t>(row) * p.k + j] = o;
  if (VALUES && p.out_val != nullptr) {
    p.out_val[static_cast<int64_t>(row) * p.k + j] =
        idx < 0 ? __uint_as_float(0xff800000u) : __uint_as_float(bits_of_key(key));
  }
}

// Smallest float whose key is >= key_lo (clamped to +inf where key_lo lies in
// the NaN range): x passes the pre-filter iff !(x < value), which keeps NaN.
__device__ __forceinline__ float prefilter_value(uint32_t key_lo) {
  if (key_lo > 0xff800000u) key_lo = 0xff800000u;
  return __uint_as_float(bits_of_key(key_lo));
}

// MODE selects what is compiled in besides the plain select, so that the plain kernel
// carries no code of the others: kModeHinted = threshold guesses (hint_in / hint_out),
// kModePush = context-parallel send (and single-kernel step); the two are bits and combine.
constexpr int kModePlain = 0;
constexpr int kModeHinted = 1;
constexpr int kModePush = 2;
constexpr int kModePushHinted = kModePush | kModeHinted;
constexpr int kModeSx = 4;   // with kModePushHinted: also the context-parallel exchange of survivors
constexpr int kModePushHintedSx = kModePushHinted | kModeSx;

// Returns true when the row's output has been written by the survivor exchange of a
// context-parallel step (then the caller has no runs to merge).
template <bool HAS_MAP, int MODE, typename T>
__device__ __forceinline__ bool topk_row_body(const TopkParams& p, unsigned char* smem, ClusterShared& sh,
                                              const PushCtx& push) {
  static_assert(!HAS_MAP || Elem<T>::kPerUnit == 4, "merge mode selects among fp32 candidates");
  constexpr int kPU = Elem<T>::kPerUnit;
  constexpr bool kPush = (MODE & kModePush) != 0;
  constexpr bool kHinted = (MODE & kModeHinted) != 0;
  constexpr bool kSx = (MODE & kModeSx) != 0;
  uint32_t* hist = reinterpret_cast<uint32_t*>(smem + kSmemHist);
  uint64_t* stage = reinterpret_cast<uint64_t*>(smem + kSmemStage);
  uint32_t* merged = reinterpret_cast<uint32_t*>(smem + kSmemStage);
  uint64_t* sortbuf = reinterpret_cast<uint64_t*>(smem + kSmemSort);
  uint64_t* cand = reinterpret_cast<uint64_t*>(smem + kSmemCand);

  cg::cluster_group cluster = cg::this_cluster();
  const int C = static_cast<int>(cluster.num_blocks());
  const int rank = static_cast<int>(cluster.block_rank());
  const int G = HAS_MAP ? 1 : max(p.groups, 1);       // clusters per row
  const int bid = static_cast<int>(blockIdx.x) - p.block_base;
  const int row = bid / (C * G);
  const int group = (bid / C) % G;
  const int n_share = C * G;                           // CTAs working on this row
  const int my_share = group * C + rank;
  uint32_t* ws = G > 1 ? p.workspace + static_cast<size_t>(row) * kWsRowWords : nullptr;
  const int tid = threadIdx.x;
  const int k = p.k;

  // ---- row geometry (uniform over the cluster) ---------------------------
  const int rs = p.row_starts != nullptr ? p.row_starts[row] : 0;
  const int glen = p.lengths != nullptr ? p.lengths[row] : 0;
  int len;
  if (p.fixed_len >= 0) {
    len = p.fixed_len;
  } else {
    int64_t l = static_cast<int64_t>(glen) - p.shard_offset;
    const int64_t room = p.L_width - rs;
    if (l > room) l = room;
    if (l < 0) l = 0;
    len = static_cast<int>(l);
  }
  const T* rowp = reinterpret_cast<const T*>(p.scores) + static_cast<int64_t>(row) * p.row_stride + rs;
  const int32_t* imap =
      HAS_MAP ? p.idx_map + static_cast<int64_t>(row) * p.row_stride + rs : nullptr;

  int table_row = row;
  if (p.epilogue == 1 && p.cu_seqlens_q != nullptr) {
    // prefill: request r with cu_seqlens_q[r] <= row < cu_seqlens_q[r+1]
    int lo = 0, hi = p.n_table_rows;  // invariant: cu[lo] <= row
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (p.cu_seqlens_q[mid] <= row) lo = mid; else hi = mid;
    }
    table_row = lo;
  }

  // ---- short rows: nothing to select --------------------------------------
  const bool identity = HAS_MAP ? (glen <= k) : (len <= k);
  const bool is_short = identity || len <= k;
  auto short_row_path = [&]() {
    if (my_share != 0) return;
    if (kHinted && !HAS_MAP && p.handover != nullptr && tid == 0) {
      // nobody reads this row's hand-over list in this launch: leave its header zeroed for the next producer
      uint32_t* hdr = reinterpret_cast<uint32_t*>(p.handover + static_cast<int64_t>(row) * kHandoverRowBytes);
      hdr[0] = 0u;
      hdr[1] = 0u;
    }
    if (kHinted && !HAS_MAP && p.hint_out != nullptr && tid == 0) p.hint_out[row] = __uint_as_float(0x7fffffffu);   // no guess
    if (!HAS_MAP && p.out_val != nullptr) {
      // Context-parallel shard shorter than k: every position is a candidate, but the
      // merge expects the run in canonical order, so rank the few elements by counting.
      for (int j = tid; j < len; j += kThreads) stage[j] = make_comp(key_of(Elem<T>::to_float(rowp[j])), j);
      __syncthreads();
      for (int j = tid; j < k; j += kThreads) {
        if (j >= len) {
          emit<kPush>(p, push, row, j, -1, 0u, false, table_row);
          continue;
        }
        const uint64_t c = stage[j];
        int pos = 0;
        for (int q = 0; q < len; ++q) pos += stage[q] > c ? 1 : 0;
        emit<kPush>(p, push, row, pos, comp_index(c), comp_key(c), false, table_row);
      }
      return;
    }
    for (int j = tid; j < k; j += kThreads) {
      if (HAS_MAP && !identity) {
        // no more candidates than k slots: pass them through in position order
        const int64_t a = j < len ? seg_addr(j, p.seg_len, p.seg_stride) : 0;
        const int32_t idx = j < len ? imap[a] : -1;
        emit<kPush>(p, push, row, j, idx, j < len ? key_of(Elem<T>::to_float(rowp[a])) : 0u, true, table_row);
      } else {
        const int n = HAS_MAP ? glen : len;
        const bool v = j < n;
        uint32_t key = 0u;
        if (v && !HAS_MAP && p.out_val != nullptr) key = key_of(Elem<T>::to_float(rowp[j]));
        emit<kPush>(p, push, row, j, v ? j : -1, key, HAS_MAP, table_row);
      }
    }
    return;
  };
  // A context-parallel step whose ranks exchange survivors (below) needs every rank, also one whose
  // shard is short, to take part in the exchange.
  const bool sx_try = kSx && kPush && kHinted && !HAS_MAP && p.push_sx != 0 && p.push_fused != 0 && glen > k;
  if (is_short && !sx_try) {
    short_row_path();
    return false;
  }

  const Chunk<T> chunk = make_chunk<T>(rowp, imap, len, n_share, my_share, p.seg_len, p.seg_stride);
  FF_TRACE(p, 0);
  if (p.trace != nullptr && tid == 0) p.trace[static_cast<size_t>(blockIdx.x) * kTraceSlots + 8] = global_ns();
  bool hinted_done_sx = false;   // set by the survivor exchange of a context-parallel step
  int expected_total_sx = 0;

  TileStream ts;
  ts.src = reinterpret_cast<const float4*>(chunk.abase) + chunk.fb;
  ts.ring = smem_addr(smem + kSmemRing);
  ts.bars = smem_addr(&sh.bars[0]);
  ts.ebars = smem_addr(&sh.ebars[0]);
  ts.n_units = chunk.fe - chunk.fb;
  ts.n_tiles = (ts.n_units + kTileUnits - 1) / kTileUnits;
  stream_init(ts);
  if (tid == 0) {
    sh.stage_count = 0;
    sh.sort_count = 0;
    sh.cand_count = 0;
    sh.small_count = 0;
    sh.fin_red[0] = 0u;
    sh.fin_red[1] = 0xffffffffu;
    sh.fin_red[2] = 0u;
    sh.fin_red[3] = 0xffffffffu;
    sh.fin_red[4] = 0u;
    if (!HAS_MAP) {
      for (int s = 0; s < kStages; ++s) {
        mbar_init(ts.bars + 8u * s, 1u);
        mbar_init(ts.ebars + 8u * s, kWarps);
      }
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
  }

  // ---- context-parallel step by exchange of survivors ----------------------------------------
  // Instead of ranking its own candidates, sending the sorted run and merging runs, every rank
  // makes a guess of the score that about 1.25 k + 64 scores of the WHOLE row reach (from its own
  // shard: seed_own_guess with p = target / global length), collects what its shard holds at or
  // above it, and every CTA stores its few survivors straight into a region of its own in every
  // rank's buffer (header {count, flags, guess} + entries, all self-validating with the step).
  // Every CTA of every rank then reads all regions in the same order, so all hold the same list of
  // about 1.25 k survivors and finish it exactly like a one-GPU row whose guess fitted: no local
  // ranking before the exchange, no run merge after it.  The list holds the row's whole top-k if at
  // least k of its entries are not below the LARGEST of the ranks' guesses (what a rank did not send
  // is below its own guess).  Otherwise (a rank without a guess, too many survivors in one CTA, too
  // few or too many in all) every rank sees the same evidence and all fall back to the exchange of
  // sorted runs.  A rank whose shard is small sends all of it (guess "none").
  bool sx_done = false;
  if constexpr (kSx && kPush && kHinted && !HAS_MAP) {
    if (sx_try) {
      __syncthreads();   // the set-up above (counters, mbarriers) is visible to every thread
      const int world = p.push_world;
      const uint32_t step = push.step;
      bool fallback = n_share > kSxRegions;
      uint32_t hkey = 0u;
      int n_mine = 0;
      if (!fallback && len <= kSxCap * n_share) {
        // small shard: CTA c sends elements [c * cap, (c + 1) * cap)
        const int b0 = my_share * kSxCap;
        n_mine = min(max(len - b0, 0), kSxCap);
        if (tid < n_mine) stage[tid] = make_comp(key_of(Elem<T>::to_float(rowp[b0 + tid])), b0 + tid);
      } else if (!fallback) {
        const SeedPlan sp = seed_plan(len, chunk.mis, kPU, n_share, k, glen, world);
        if (!sp.use || G <= 1) {
          fallback = true;
        } else {
          const int n0 = seed_sample_ready(ts, sp, false);
          const SeedResult sr = seed_own_guess<T>(ts.ring, n0, &sh.flag, hist, ws, sp.p, n_share, my_share);
          if (sr.code == 2) ts.timed_out = true;
          FF_TRACE(p, 21);
          if (sr.code != 1) {
            fallback = true;
          } else {
            const float guess = sr.guess;
            hkey = key_of(guess);
            stream_pass(ts, [&](uint32_t tile, int tt, int units) {
              collect_tile<T>(tile, units, chunk.fb + tt * kTileUnits, chunk.mis, guess, stage, kSortCap, &sh.stage_count);
            });
            float x = 0.f;
            const int pos = partial_element(chunk, x);
            if (pos >= 0 && !(x < guess)) {
              const int slot = atomicAdd(&sh.stage_count, 1);
              if (slot < kSortCap) stage[slot] = make_comp(key_of(x), pos);
            }
            __syncthreads();
            n_mine = sh.stage_count;
            if (n_mine > kSxCap) {   // a crowded chunk: this protocol is not for such rows
              fallback = true;
              n_mine = 0;
            }
          }
        }
      }
      __syncthreads();
      FF_TRACE(p, 3);
      // ---- send: entries and header of this CTA's region to every rank (own rank included) ----
      auto region_in = [&](uint32_t* base, int src_rank, int c) {
        return base + p.push_sx_offset +
               ((((static_cast<size_t>(step & 1u) * world + src_rank) * p.B + row) * kSxRegions) + c) * kSxRegionWords;
      };
      if (my_share < kSxRegions) {
        for (int i = tid; i < world * n_mine; i += kThreads) {
          const int q = i / n_mine, e = i - q * n_mine;
          const uint64_t c = stage[e];
          st_entry(region_in(p.push_peers.base[q], p.push_rank, my_share) + 4 + 4 * e, bits_of_key(comp_key(c)),
                   static_cast<uint32_t>(comp_index(c) + p.shard_offset), step);
        }
        const uint32_t head = static_cast<uint32_t>(n_mine) | (fallback ? kSxFallbackFlag : 0u);
        if (tid < world) st_entry(region_in(p.push_peers.base[tid], p.push_rank, my_share), head, hkey, step);
        if (my_share == 0) {   // the regions no CTA of this launch owns: empty, same flags
          const int spare = kSxRegions - min(n_share, kSxRegions);
          for (int i = tid; i < world * spare; i += kThreads)
            st_entry(region_in(p.push_peers.base[i / spare], p.push_rank, n_share + i % spare),
                     fallback ? kSxFallbackFlag : 0u, 0u, step);
        }
      }
      // ---- receive: all regions of all ranks, in region order, into the survivor list ----
      uint32_t* pre = hist;                      // [world * kSxRegions + 1] entries before each region
      const int R = world * kSxRegions;
      const int J = (R + kThreads - 1) / kThreads;   // consecutive regions per thread (at most 4)
      const unsigned long long t0 = global_ns();
      bool sx_ok = true;
      uint32_t cnt[4] = {0u, 0u, 0u, 0u};
      uint32_t hmax = 0u, any_flag = 0u;
      {
        uint4 h[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int rr = tid * J + j;
          if (j < J && rr < R)
            h[j] = ld_entry_pair(region_in(p.push_peers.base[p.push_rank], rr / kSxRegions, rr % kSxRegions));
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int rr = tid * J + j;
          if (j < J && rr < R) {
            const uint32_t* reg = region_in(p.push_peers.base[p.push_rank], rr / kSxRegions, rr % kSxRegions);
            const uint2 hd = await_entry_pair(reg, h[j], step, t0, sx_ok);
            const uint32_t head = hd.x, hk = hd.y;
            if (sx_ok) {
              cnt[j] = head & 0xffffu;
              any_flag |= head & kSxFallbackFlag;
              hmax = max(hmax, hk);
            } else {
              any_flag |= kSxFallbackFlag;
            }
          }
        }
      }
      int total = 0;
      const int mine_sum = static_cast<int>(cnt[0] + cnt[1] + cnt[2] + cnt[3]);
      const int after = block_suffix_exclusive(mine_sum, sh.warp_tot, total);   // entries of the regions after mine
      {
        int before = total - after - mine_sum;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int rr = tid * J + j;
          if (j < J && rr < R) {
            pre[rr] = static_cast<uint32_t>(before);
            before += static_cast<int>(cnt[j]);
          }
        }
        if (tid == 0) pre[R] = static_cast<uint32_t>(total);
      }
      hmax = __reduce_max_sync(0xffffffffu, hmax);
      if ((tid & 31) == 0) sh.warp_tot[tid >> 5] = static_cast<int>(hmax);   // (the scan is done with warp_tot)
      const bool flagged = __syncthreads_or(any_flag != 0u ? 1 : 0) != 0;
#pragma unroll
      for (int wi = 0; wi < kWarps; ++wi) hmax = max(hmax, static_cast<uint32_t>(sh.warp_tot[wi]));
      FF_TRACE(p, 38);
      bool good = !flagged && total >= k && total <= kSortCap;
      int not_below = 0;
      if (good) {
        // every thread copies the entries of its own regions to their places in the list, eight
        // entries (sixteen loads) in flight at a time
        constexpr int kBatch = 8;
#pragma unroll 1
        for (int j = 0; j < J; ++j) {
          const int rr = tid * J + j;
          if (rr >= R) break;
          const int n_r = static_cast<int>(j == 0 ? cnt[0] : j == 1 ? cnt[1] : j == 2 ? cnt[2] : cnt[3]);
          const uint32_t* reg = region_in(p.push_peers.base[p.push_rank], rr / kSxRegions, rr % kSxRegions) + 4;
          const int at = static_cast<int>(pre[rr]);
#pragma unroll 1
          for (int e0 = 0; e0 < n_r; e0 += kBatch) {
            uint4 ev[kBatch];
#pragma unroll
            for (int u = 0; u < kBatch; ++u)
              if (e0 + u < n_r) ev[u] = ld_entry_pair(reg + 4 * (e0 + u));
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
              if (e0 + u < n_r) {
                const uint2 en = await_entry_pair(reg + 4 * (e0 + u), ev[u], step, t0, sx_ok);
                const uint32_t key = key_of_bits(en.x);
                sortbuf[at + e0 + u] = make_comp(key, static_cast<int32_t>(en.y));
                not_below += key >= hmax ? 1 : 0;
              }
            }
          }
        }
        if (tid == 0) sh.cand_count = 0;
        __syncthreads();
        not_below = __reduce_add_sync(0xffffffffu, not_below);
        if ((tid & 31) == 0 && not_below != 0) atomicAdd(&sh.cand_count, not_below);
        good = __syncthreads_and(sx_ok ? 1 : 0) != 0;
        good = good && sh.cand_count >= k;   // what no rank sent is below the largest guess, and k entries are not
        __syncthreads();
      }
      if (!sx_ok) ts.timed_out = true;
      FF_TRACE(p, 39);
      if (tid == 0) {
        sh.stage_count = 0;
        sh.cand_count = 0;
      }
      if (good) {
        sx_done = true;
        hinted_done_sx = true;
        expected_total_sx = total;
        if (my_share == 0 && tid == 0) sh.sort_count = total;
      } else {
        if (p.status != nullptr && tid == 0 && my_share == 0) atomicOr(p.status, 64);
        if (is_short) {
          __syncthreads();
          short_row_path();
          return false;
        }
      }
      __syncthreads();
    }
  }
  // Writes output slot `pos`: to the peers' slots in a context-parallel send, straight to the
  // output (the index is global already) after an exchange of survivors, else to the output.
  auto put = [&](int pos, int32_t idx, uint32_t key) {
    if (kPush && sx_done) emit<false, false>(p, push, row, pos, idx, key, true, table_row);
    else emit<kPush>(p, push, row, pos, idx, key, HAS_MAP, table_row);
  };

  int r = k;                // survivors still to be taken from the current candidate set
  uint64_t P = 0;           // digits fixed so far (value of comp >> shift of the last level)
  bool src_is_cand = false; // candidates live in `cand` instead of the chunk
  int cand_n = 0;
  bool ok = true;
  int expected_total = expected_total_sx;
  int levels_used = 0;
  uint64_t floor_comp = 0;  // no survivor's composite is below this

  // Stores this CTA's n_true staged survivors (the first kSortCap of them are in `stage`)
  // where every CTA working on the row will find them: one atomic reserves a block of slots
  // (the same in every copy of the list), coalesced stores fill it.  Inside one cluster the
  // list is all-gathered into EVERY peer over DSMEM, so each CTA ends up with the full list and
  // can take a share of the finishing work without further exchange; rows split over clusters
  // keep it in global scratch (count word `gcount`).
  auto gather_stage = [&](int n_true, bool hinted_attempt) {
    const int n_stage = min(n_true, kSortCap);
    if (G > 1 && (n_true > 0 || hinted_attempt)) {
      if (tid == 0) {
        if (hinted_attempt) {   // survivors and "this CTA has reserved" in one atomic: readers see both or neither
          const unsigned long long old = atomicAdd(reinterpret_cast<unsigned long long*>(ws + 10),
                                                   static_cast<unsigned long long>(n_true) | (1ull << 32));
          sh.push_base = static_cast<int>(static_cast<uint32_t>(old));
        } else {
          sh.push_base = static_cast<int>(atomicAdd(ws + 8, static_cast<uint32_t>(n_true)));
        }
      }
      __syncthreads();
      uint64_t* gsurv = reinterpret_cast<uint64_t*>(ws + kWsHeaderWords + kWsHistWords + (hinted_attempt ? kWsListWords : 0));
      const int base = sh.push_base;
      for (int i = tid; i < n_stage; i += kThreads) {
        if (base + i < kSortCap) gsurv[base + i] = stage[i];
      }
    } else if (n_true > 0) {
      if (C == 1) {
        const int base = sh.sort_count;
        __syncthreads();
        for (int i = tid; i < n_stage; i += kThreads) {
          if (base + i < kSortCap) sortbuf[base + i] = stage[i];
        }
        if (tid == 0) sh.sort_count = base + n_true;
      } else {
        if (tid == 0) {
          sh.push_base = static_cast<int>(dsmem_atomic_add_u32(
              dsmem_addr(smem_addr(&sh.sort_count), 0), static_cast<uint32_t>(n_true)));
        }
        __syncthreads();
        const int base = sh.push_base;
        const uint32_t sort_local = smem_addr(sortbuf);
        for (int j = tid; j < n_stage * C; j += kThreads) {
          const int c = j / n_stage;
          const int i = j - c * n_stage;
          if (base + i < kSortCap)
            dsmem_st_u64(dsmem_addr(sort_local + 8u * static_cast<uint32_t>(base + i), c), stage[i]);
        }
      }
    }
    __syncthreads();
  };

  // ---- hinted attempt: one sweep, no histogram ------------------------------
  // The caller's guess h of a value between the row's k-th and 4096-th largest: everything
  // not below h is collected in one sweep; if that is between k and 4096 elements the row is
  // finished from them directly.  Otherwise (a miss, reported as FF_STATUS_HINT_MISSED) the
  // row starts over on the histogram path below; the result is exact either way.
  // (see "Last use of the scratch" below)
  constexpr int kScratchThread = 96;
  uint32_t counted_out_before = 0u;
  int n_plain_to_clear = 0;
  bool hinted_done = hinted_done_sx;
  int hinted_total = 0;     // entries a hinted attempt left in its global list (rows split over clusters)
  float hint = 0.f;
  bool use_hint = false;
  if (kHinted && !HAS_MAP && p.hint_in != nullptr) {
    hint = p.hint_in[row];
    use_hint = hint == hint;   // NaN: no guess
  }
  __syncthreads();
  if (kHinted && !HAS_MAP && p.handover != nullptr) {
    // Hand-over from the kernel that produced the scores: it has already listed every score of
    // the row that is not below the guess (composites, in arrival order) and counted them.  If
    // the count fits, every CTA of the row copies the list and goes straight to the finish: no
    // score is read at all.  If it does not fit (or there was no guess), the count says so
    // exactly, so the row skips the sweep with the guess and selects from the scores.
    uint32_t* hdr = reinterpret_cast<uint32_t*>(p.handover + static_cast<int64_t>(row) * kHandoverRowBytes);
    uint32_t readers_before = 0u;
    if (tid == 0) {
      sh.push_base = static_cast<int>(__ldcg(hdr));
      __threadfence();                               // the count is read before this CTA counts itself as a reader
      readers_before = atomicAdd(hdr + 1, 1u);       // (looked at below, after the copy: its round trip overlaps)
    }
    __syncthreads();
    const int listed = sh.push_base;
    if (use_hint && listed >= k && listed <= kSortCap) {
      const unsigned long long* list = reinterpret_cast<const unsigned long long*>(hdr + 16);
      for (int i = tid; i < listed; i += kThreads) sortbuf[i] = __ldcg(list + i);
      hinted_done = true;
      expected_total = listed;
      floor_comp = static_cast<uint64_t>(key_of(hint)) << 32;
      if (my_share == 0 && tid == 0) sh.sort_count = listed;
    } else if (use_hint) {
      if (p.status != nullptr && tid == 0 && my_share == 0) atomicOr(p.status, 8);
    }
    use_hint = false;
    // the reader that counts itself last leaves the header zeroed for the next producer launch
    if (tid == 0 && readers_before == static_cast<uint32_t>(n_share) - 1u) {
      hdr[0] = 0u;
      hdr[1] = 0u;
    }
    __syncthreads();
  }
  bool self_seeded = false;
  if (kHinted && !HAS_MAP && p.self_seed != 0 && G > 1 && !use_hint && !hinted_done && p.handover == nullptr && !sx_try) {
    const SeedPlan sp = seed_plan(len, chunk.mis, kPU, n_share, k);
    if (sp.use) {
      // the chunk's first tile or two (they stay in the ring for the sweep that follows)
      const int n0 = seed_sample_ready(ts, sp, true);
      const SeedResult sr = seed_own_guess<T>(
          ts.ring, n0, &sh.flag, hist, ws, sp.p, n_share, my_share,
          p.trace != nullptr ? p.trace + static_cast<size_t>(blockIdx.x) * kTraceSlots : nullptr);
      if (sr.code == 2) ts.timed_out = true;
      if (sr.code == 1) {
        hint = sr.guess;
        use_hint = true;
        self_seeded = true;
      }
      FF_TRACE(p, 21);
    }
  }
  if (kHinted && use_hint) {
    stream_pass(ts, [&](uint32_t tile, int tt, int units) {
      collect_tile<T>(tile, units, chunk.fb + tt * kTileUnits, chunk.mis, hint, stage, kSortCap, &sh.stage_count);
    });
    {
      float x = 0.f;
      const int pos = partial_element(chunk, x);
      if (pos >= 0 && !(x < hint)) {
        const int slot = atomicAdd(&sh.stage_count, 1);
        if (slot < kSortCap) stage[slot] = make_comp(key_of(x), pos);
      }
    }
    __syncthreads();
    FF_TRACE(p, 3);
    gather_stage(sh.stage_count, true);
    FF_TRACE(p, 4);
    int total;
    if (G > 1) {
      // every CTA of the row has reserved when the word's high half reaches n_share; its low half is then the total
      if (tid == 0) {
        unsigned long long v = 0ull;
        int spin = 0;
        for (; spin < kSpinLimit; ++spin) {
          asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(ws + 10) : "memory");
          if (static_cast<uint32_t>(v >> 32) >= static_cast<uint32_t>(n_share)) break;
        }
        sh.flag = spin < kSpinLimit ? 1 : 0;
        sh.push_base = static_cast<int>(static_cast<uint32_t>(v));
      }
      __syncthreads();
      if (!sh.flag) ts.timed_out = true;
      total = sh.push_base;
    } else if (C > 1) {
      cluster.sync();
      total = static_cast<int>(dsmem_ld_u32(dsmem_addr(smem_addr(&sh.sort_count), 0)));
    } else {
      total = sh.sort_count;
    }
    hinted_total = G > 1 ? min(total, kSortCap) : 0;
    if (total >= k && total <= kSortCap) {
      hinted_done = true;
      expected_total = total;
      floor_comp = static_cast<uint64_t>(key_of(hint)) << 32;
      if (G > 1) {
        const uint64_t* gsurv = reinterpret_cast<const uint64_t*>(ws + kWsHeaderWords + kWsHistWords + kWsListWords);
        if (!load_list_validated(gsurv, total, sortbuf)) ts.timed_out = true;
        if (my_share == 0 && tid == 0) sh.sort_count = total;
      }
    } else {
      // a caller's guess that did not fit is reported; the row's own guess is its own business
      if (!self_seeded && p.status != nullptr && tid == 0 && my_share == 0) atomicOr(p.status, 8);
      if (C > 1 && G == 1) cluster.sync();   // every CTA has read the count before it is cleared
      if (tid == 0) sh.sort_count = 0;
    }
    if (tid == 0) sh.stage_count = 0;
    __syncthreads();
  }

  if (!hinted_done) {
  // ---- level 0: 13-bit histogram of the whole chunk -----------------------
  for (int i = tid; i < kMaxBins; i += kThreads) hist[i] = 0u;
  __syncthreads();
  if (HAS_MAP) {
    for_each_in_chunk<true, T>(
        chunk, [](float) { return true; },
        [&](float x, int32_t idx) { atomicAdd(&hist[(idx < 0 ? 0u : key_of(x)) >> kFirstShift], 1u); });
  } else {
    stream_pass(ts, [&](uint32_t tile, int, int units) {
#pragma unroll
      for (int j = 0; j < kTileUnits / kThreads; ++j) {
        const int lu = tid + j * kThreads;
        if (lu < units) {
          float v[kPU];
          unpack_unit<T>(lds_u4(tile + 16u * static_cast<uint32_t>(lu)), v);
#pragma unroll
          for (int e = 0; e < kPU; ++e) {
            const uint32_t d = raw_digit(v[e]);
            if (FF_IN_RANGE(p, d, kMaxBins, 1)) atomicAdd(&hist[d], 1u);
          }
        }
      }
    });
    float x = 0.f;
    if (partial_element(chunk, x) >= 0 && FF_IN_RANGE(p, raw_digit(x), kMaxBins, 2)) atomicAdd(&hist[raw_digit(x)], 1u);
  }
  __syncthreads();
  FF_TRACE(p, 1);

#pragma unroll 1
  for (int level = 0; level < kNumLevels; ++level) {
    const int bits = level_bits(level);
    const int shift = level_shift(level);
    const bool raw0 = !HAS_MAP && level == 0;
    const bool two_step = raw0 && G == 1 && C > 1;
    if (two_step) {
      merge_two_step(cluster, C, hist, merged, r, sh, p);
    } else {
      merge_and_scan(cluster, C, rank, hist, merged, 1 << bits, r, raw0, sh, p, level == 0, G, ws, level,
                     ts.timed_out, (level == 0 && !HAS_MAP) ? len : -1);
    }
    levels_used = level + 1;
    FF_TRACE(p, 2 + 3 * level);
    const int t = sh.res[0];
    const int above = sh.res[1];
    const int m = sh.res[2];
    if (t < 0) {
      ok = false;
      break;
    }
    const int total = (k - r) + above + m;
    const bool final_level = total <= kSortCap || level == kNumLevels - 1;
    const uint64_t Pn = (level == 0 ? 0ull : (P << bits)) | static_cast<uint64_t>(t);
    const uint64_t Pmax = Pn | ((1ull << bits) - 1ull);
    const int local_m = static_cast<int>(hist[raw0 ? raw_of_bin(t) : t]);
    const bool compact = !final_level && !src_is_cand && local_m <= kCandCap;
    const int nshift = final_level ? 0 : level_shift(level + 1);
    const uint32_t nmask = final_level ? 0u : ((1u << level_bits(level + 1)) - 1u);
    __syncthreads();
    if (!final_level) {
      if (two_step) cluster.sync();   // peers may still be reading this histogram (no barrier ended the merge)
      for (int i = tid; i < (1 << level_bits(level + 1)); i += kThreads) hist[i] = 0u;
    }
    __syncthreads();

    LevelCtx ctx;
    ctx.Pn = Pn;
    ctx.Pmax = Pmax;
    ctx.shift = shift;
    ctx.nshift = nshift;
    ctx.nmask = nmask;
    ctx.final_level = final_level;
    ctx.compact = compact;
    ctx.hist = hist;
    ctx.stage = stage;
    ctx.cand = cand;
    ctx.sh = &sh;
    // At level 0 "digit >= t" is exactly "value >= value(t << 19)" (unless t lies in
    // the NaN range), so the chunk is swept with float compares only.
    bool swept = false;
    if (!HAS_MAP && level == 0 && final_level && (static_cast<uint32_t>(t) << kFirstShift) <= 0xff800000u) {
      const float vmin = prefilter_value(static_cast<uint32_t>(t) << kFirstShift);
      stream_pass(ts, [&](uint32_t tile, int tt, int units) {
        collect_tile<T>(tile, units, chunk.fb + tt * kTileUnits, chunk.mis, vmin, stage, kSortCap, &sh.stage_count);
      });
      float x = 0.f;
      const int pos = partial_element(chunk, x);
      if (pos >= 0 && !(x < vmin)) {
        const int slot = atomicAdd(&sh.stage_count, 1);
        if (slot < kSortCap) stage[slot] = make_comp(key_of(x), pos);
      }
      swept = true;
    } else if (!HAS_MAP && !src_is_cand && level == 0 && !final_level &&
               (static_cast<uint32_t>(t) << kFirstShift) <= 0xff800000u) {
      // Too many elements at or above the threshold bin for the finish: winners
      // (bin > t) go to the stage buffer, the bin's own elements are only counted
      // in the histogram of the next 10 key bits; the chunk is swept once more
      // when that digit's threshold is known.
      const float vmin = prefilter_value(static_cast<uint32_t>(t) << kFirstShift);
      auto on_hit = [&](float x, int pos) {
        const uint32_t key = key_of(x);
        if ((key >> kFirstShift) > static_cast<uint32_t>(t)) {
          push_aggregated(stage, &sh.stage_count, kSortCap, make_comp(key, pos));
        } else {
          atomicAdd(&hist[(key >> (kFirstShift - 10)) & 1023u], 1u);
        }
      };
      stream_pass(ts, [&](uint32_t tile, int tt, int units) {
        scan_tile<T>(tile, units, chunk.fb + tt * kTileUnits, chunk.mis, vmin, on_hit);
      });
      float x = 0.f;
      const int pos = partial_element(chunk, x);
      if (pos >= 0 && !(x < vmin)) on_hit(x, pos);
      ctx.compact = false;
      swept = true;
    } else if (!HAS_MAP && !src_is_cand && level == 1 && final_level) {
      // Second digit resolved: survivors are the elements of bin P whose next 10
      // bits are >= t, i.e. 23-bit key prefix in [Pn, Pmax]; float pre-filter on the
      // lower bound, exact test on the key.
      const uint32_t key_lo = static_cast<uint32_t>(Pn) << (kFirstShift - 10);
      const float vmin = prefilter_value(key_lo);
      auto on_hit = [&](float x, int pos) {
        const uint32_t key = key_of(x);
        const uint32_t pre = key >> (kFirstShift - 10);
        if (pre >= static_cast<uint32_t>(Pn) && pre <= static_cast<uint32_t>(Pmax))
          push_aggregated(stage, &sh.stage_count, kSortCap, make_comp(key, pos));
      };
      stream_pass(ts, [&](uint32_t tile, int tt, int units) {
        scan_tile<T>(tile, units, chunk.fb + tt * kTileUnits, chunk.mis, vmin, on_hit);
      });
      float x = 0.f;
      const int pos = partial_element(chunk, x);
      if (pos >= 0 && !(x < vmin)) on_hit(x, pos);
      swept = true;
    }
    if (swept) {
      // nothing left to do for this level
    } else if (src_is_cand) {
      for (int i = tid; i < cand_n; i += kThreads) classify_comp(&ctx, cand[i]);
    } else {
      // Everything of interest has composite >= Pn << shift, i.e. value >= vmin.
      const float vmin = prefilter_value(static_cast<uint32_t>((Pn << shift) >> 32));
      for_each_in_chunk<HAS_MAP, T>(
          chunk, [vmin](float x) { return !(x < vmin); },
          [&](float x, int32_t idx) { classify_value<HAS_MAP>(&ctx, x, idx); });
    }
    __syncthreads();
    FF_TRACE(p, 3 + 3 * level);

    gather_stage(min(sh.stage_count, kSortCap), false);
    FF_TRACE(p, 4 + 3 * level);
    if (tid == 0) sh.stage_count = 0;
    if (ctx.compact && !src_is_cand) {
      src_is_cand = true;
      cand_n = min(sh.cand_count, kCandCap);
    }
    if (final_level) {
      expected_total = total;
      floor_comp = Pn << shift;
      break;
    }
    r -= above;
    P = Pn;
  }
  }   // !hinted_done

  if (G > 1) {
    const int n_load = (!hinted_done && ok) ? min(expected_total, kSortCap) : 0;
    if (!hinted_done) {
      // no barrier: the histogram told every CTA how many survivors to expect, and entries validate themselves
      const uint64_t* gsurv = reinterpret_cast<const uint64_t*>(ws + kWsHeaderWords + kWsHistWords);
      if (!load_list_validated(gsurv, n_load, sortbuf)) ts.timed_out = true;
      __syncthreads();
      if (my_share == 0 && tid == 0) sh.sort_count = static_cast<int>(__ldcg(ws + 8));   // all of them have been reserved by now
    }
    __syncthreads();
    // Last use of the scratch: this CTA counts itself out; the CTA that does so last zeroes the
    // scratch for the next launch.  The atomic is issued here and its result looked at only when
    // the row is finished (leave_scratch below), so its round trip is off the critical path.
    n_plain_to_clear = hinted_done ? 0 : (ok ? n_load : kSortCap);
    if (tid == kScratchThread) {
      __threadfence();
      counted_out_before = atomicAdd(ws + 7, 1u);
    }
  } else if (C > 1) {
    if (!hinted_done) cluster.sync();   // every survivor has landed in every CTA's list
  } else {
    __syncthreads();
  }
  FF_TRACE(p, 20);

  auto leave_scratch = [&]() {
    if (G <= 1) return;
    if (tid == kScratchThread) sh.flag = counted_out_before == static_cast<uint32_t>(n_share - 1) ? 1 : 0;
    __syncthreads();
    if (sh.flag) {
      for (int i = tid; i < kWsHeaderWords + levels_used * kMaxBins; i += kThreads) ws[i] = 0u;
      // the lists must read as empty for the next launch (a failed select may have left any number of entries)
      uint32_t* lists = ws + kWsHeaderWords + kWsHistWords;
      for (int i = tid; i < 2 * n_plain_to_clear; i += kThreads) lists[i] = 0u;
      for (int i = tid; i < 2 * hinted_total; i += kThreads) lists[kWsListWords + i] = 0u;
      if (kHinted && p.self_seed != 0) {
        if (tid < 2) ws[kWsSeedWord + tid] = 0u;
      }
    }
  };
  if (ts.timed_out && p.status != nullptr && tid == 0) atomicOr(p.status, 2);
  if (!ok) {
    if (p.status != nullptr && tid == 0 && my_share == 0) atomicOr(p.status, 4);
    if (kHinted && !HAS_MAP && p.hint_out != nullptr && tid == 0 && my_share == 0) p.hint_out[row] = __uint_as_float(0x7fffffffu);
    if (my_share == 0) {
      for (int j = tid; j < k; j += kThreads) emit<kPush>(p, push, row, j, -1, 0u, HAS_MAP, table_row);
    }
    leave_scratch();
    return false;
  }
  const int n_surv = min(expected_total, kSortCap);
  const int hint_rank = min(n_surv, hint_target_rank(k)) - 1;
  if (my_share == 0 && tid == 0 && sh.sort_count != expected_total && p.status != nullptr)
    atomicOr(p.status, 1);

  // ---- finish, many CTAs on the row: rank by direct counting ------------------
  // With n CTAs on the row, CTA s owns the survivors i = s, s + n, ...  When that is at most 32
  // of them (rows split over many clusters), the CTA's threads simply count the
  // survivors above it in this CTA's copy of the list: no histogram, scan or scatter.
  if (n_surv <= 32 * n_share) {
    // Register blocking: a group of 64 lanes (two warps) holds up to four owned survivors per lane
    // (as many as the eight groups need to cover what a CTA owns) and streams the list once for
    // all of them, so shared memory is read less often than it is compared.
    uint32_t* cnt_arr = reinterpret_cast<uint32_t*>(smem + kSmemRing + 1024);   // [32] ranks
    if (tid < 32) cnt_arr[tid] = 0u;
    const int grp = tid >> 6, l64 = tid & 63;
    const int owned_max = (n_surv + n_share - 1) / n_share;   // <= 32
    auto count_pass = [&](auto per_group) {
      constexpr int EC = decltype(per_group)::value;
      uint64_t own[EC];
      int part[EC];
#pragma unroll
      for (int e = 0; e < EC; ++e) {
        const int idx = my_share + (grp * EC + e) * n_share;
        own[e] = idx < n_surv ? sortbuf[idx] : ~0ull;
        part[e] = 0;
      }
      __syncthreads();
#pragma unroll 2
      for (int q = l64; q < n_surv; q += 64) {
        const uint64_t o = sortbuf[q];
#pragma unroll
        for (int e = 0; e < EC; ++e) part[e] += o > own[e] ? 1 : 0;
      }
#pragma unroll
      for (int e = 0; e < EC; ++e) {
        const int v = __reduce_add_sync(0xffffffffu, part[e]);
        if ((tid & 31) == 0 && v != 0) atomicAdd(&cnt_arr[grp * EC + e], static_cast<uint32_t>(v));
      }
    };
    if (owned_max <= 8) count_pass(std::integral_constant<int, 1>{});
    else if (owned_max <= 16) count_pass(std::integral_constant<int, 2>{});
    else if (owned_max <= 24) count_pass(std::integral_constant<int, 3>{});
    else count_pass(std::integral_constant<int, 4>{});
    __syncthreads();
    // threads 0..31 finish one owned survivor each
    const int i = my_share + tid * n_share;
    const bool valid = tid < 32 && i < n_surv;
    const uint64_t c = valid ? sortbuf[i] : ~0ull;
    const int cnt = valid ? static_cast<int>(cnt_arr[tid]) : 0;
    if (valid && cnt < k) put(cnt, c == 0ull ? -1 : comp_index(c), comp_key(c));
    if (kHinted && !HAS_MAP && p.hint_out != nullptr) {
      // Next call's guess: the score of rank min(n_surv, target) - 1 (hint_target_rank), written by its owner.  With fewer
      // than `target` survivors that is the smallest one; its owner then extrapolates linearly below
      // it with the owned survivor whose rank is nearest to n_surv/2 (ranks of the others are not known here).
      uint32_t* mid = reinterpret_cast<uint32_t*>(smem + kSmemRing);   // [32][3]: |rank - n_surv/2|, value bits, rank
      if (tid < 32) {
        mid[3 * tid] = valid ? static_cast<uint32_t>(abs(cnt - (n_surv >> 1))) : 0x7fffffffu;
        mid[3 * tid + 1] = bits_of_key(comp_key(c));
        mid[3 * tid + 2] = static_cast<uint32_t>(cnt);
      }
      __syncthreads();
      if (valid && cnt == hint_rank) {
        const float va = __uint_as_float(bits_of_key(comp_key(c)));
        float guess = va;
        const int want = hint_target_rank(k);
        if (n_surv < want) {
          int best = 0;
          for (int g = 1; g < 32; ++g)
            if (mid[3 * g] < mid[3 * best]) best = g;
          const float vm = __uint_as_float(mid[3 * best + 1]);
          const int gap = hint_rank - static_cast<int>(mid[3 * best + 2]);   // ranks between the two
          if (mid[3 * best] < static_cast<uint32_t>(n_surv >> 2) && gap > 0) {
            const float lower = va - (vm - va) * (static_cast<float>(want - n_surv) / static_cast<float>(gap));
            if (lower == lower && fabsf(lower) <= 3.0e38f) guess = lower;
          }
        }
        p.hint_out[row] = guess;
      }
    }
    FF_TRACE(p, 25);
    leave_scratch();
    return sx_done;
  }

  // ---- finish: rank the n_surv survivors and write the first k ------------------
  // A counting sort on an adaptive digit of at most 4096 bins (bin_of below; any
  // monotone bin map keeps the result exact).  Every CTA builds the same
  // buckets from its copy of the survivor list.  The exact rank inside a bucket
  // is found by counting: the thread that owns a survivor walks its bucket, and the
  // survivors are shared out over the CTAs of the row by list index.  The loops are
  // deliberately not unrolled: this code runs once per row and its instruction
  // footprint costs more than its trip counts (measured more than once).
  uint32_t* E = reinterpret_cast<uint32_t*>(smem + kSmemRing);                     // #(bin > b), padded index
  uint64_t* bucketed = stage;
  uint32_t* fh = reinterpret_cast<uint32_t*>(smem + kSmemRing + 20 * 1024);                   // bucket sizes, padded index
  uint16_t* at_arr = reinterpret_cast<uint16_t*>(smem + kSmemRing + 40 * 1024);     // slot of survivor i
  uint16_t* bin_arr = reinterpret_cast<uint16_t*>(smem + kSmemRing + 48 * 1024);    // padded bin of survivor i (worked out once)
  auto pad = [](uint32_t b) { return b + (b >> 3); };   // 8 consecutive bins per thread -> distinct banks
  constexpr int kPadBins = kFinishBins + kFinishBins / 8;
  // bounds of the survivors' composites: exact on the key half, and exact on the
  // index half too when every key is equal (then only the indices separate them)
  uint32_t hmax = 0u, hmin = 0xffffffffu, lmax = 0u, lmin = 0xffffffffu;
  uint32_t kdiff = 0u;   // the key bits in which survivors differ (against the first one's key)
  const uint32_t kref = static_cast<uint32_t>(sortbuf[0] >> 32);
#pragma unroll 1
  for (int i = tid; i < n_surv; i += kThreads) {
    const uint64_t c = sortbuf[i];
    hmax = max(hmax, static_cast<uint32_t>(c >> 32));
    hmin = min(hmin, static_cast<uint32_t>(c >> 32));
    lmax = max(lmax, static_cast<uint32_t>(c));
    lmin = min(lmin, static_cast<uint32_t>(c));
    kdiff |= static_cast<uint32_t>(c >> 32) ^ kref;
  }
  hmax = __reduce_max_sync(0xffffffffu, hmax);
  hmin = __reduce_min_sync(0xffffffffu, hmin);
  lmax = __reduce_max_sync(0xffffffffu, lmax);
  lmin = __reduce_min_sync(0xffffffffu, lmin);
  kdiff = __reduce_or_sync(0xffffffffu, kdiff);
  // one shared atomic per warp and quantity (set up when the CTA started), not a second pass over per-warp partials
  if ((tid & 31) == 0) {
    atomicMax(&sh.fin_red[0], hmax);
    atomicMin(&sh.fin_red[1], hmin);
    atomicMax(&sh.fin_red[2], lmax);
    atomicMin(&sh.fin_red[3], lmin);
    atomicOr(&sh.fin_red[4], kdiff);
  }
#pragma unroll 1
  for (int i = tid; i < kPadBins; i += kThreads) fh[i] = 0u;
  if (tid == 0) sh.big_count = 0;
  __syncthreads();
  hmax = sh.fin_red[0];
  hmin = sh.fin_red[1];
  lmax = sh.fin_red[2];
  lmin = sh.fin_red[3];
  kdiff = sh.fin_red[4];
  // The bin of a survivor is a monotone function of its composite that wastes no bits on what the
  // survivors have in common: the key is taken relative to the smallest key and without the low
  // bits in which no two keys differ (scores rounded to bf16, or quantised otherwise, leave 16
  // or more of them), the index half relative to its smallest value and at its own width; the two
  // are joined and the top 12 bits of the result are the bin.  So a row whose survivors share few
  // distinct scores (heavy ties) still spreads over the bins, by index, and a row whose scores are
  // all different spreads by score as before.
  const int ktz = kdiff == 0u ? 0 : __ffs(static_cast<int>(kdiff)) - 1;         // low key bits that never differ
  const int lbits = lmax == lmin ? 0 : 32 - __clz(static_cast<int>(lmax - lmin));  // width of the index half
  const uint32_t kspan = (hmax - hmin) >> ktz;
  const int nbits = (kspan == 0u ? 0 : 32 - __clz(static_cast<int>(kspan))) + lbits;
  constexpr int kBinBits = 12;
  static_assert((1 << kBinBits) == kFinishBins && kFinishBins + kFinishBins / 8 <= 5 * 1024, "bins, and room for two padded arrays of them");
  const int bshift = nbits > kBinBits ? nbits - kBinBits : 0;
  auto bin_of = [&](uint64_t c) -> uint32_t {
    const uint64_t joined = (static_cast<uint64_t>((static_cast<uint32_t>(c >> 32) - hmin) >> ktz) << lbits) |
                            (static_cast<uint32_t>(c) - lmin);
    return static_cast<uint32_t>(joined >> bshift);
  };
  // arrival order inside the bin doubles as the scatter offset
#pragma unroll 1
  for (int i = tid; i < n_surv; i += kThreads) {
    const uint32_t b = bin_of(sortbuf[i]);
    bin_arr[i] = static_cast<uint16_t>(pad(b));
    if (FF_IN_RANGE(p, b, kFinishBins, 3)) at_arr[i] = static_cast<uint16_t>(atomicAdd(&fh[pad(b)], 1u));
  }
  __syncthreads();
  FF_TRACE(p, 22);
  {
    constexpr int per = kFinishBins / kThreads;
    int local = 0;
#pragma unroll
    for (int q = 0; q < per; ++q) local += static_cast<int>(fh[pad(tid * per + q)]);
    int total;
    int running = block_suffix_exclusive(local, sh.warp_tot, total);
#pragma unroll
    for (int q = per - 1; q >= 0; --q) {
      const uint32_t b = pad(tid * per + q);
      E[b] = static_cast<uint32_t>(running);
      running += static_cast<int>(fh[b]);
    }
  }
  __syncthreads();
  FF_TRACE(p, 23);
#pragma unroll 1
  for (int i = tid; i < n_surv; i += kThreads) {
    const uint64_t c = sortbuf[i];
    const uint32_t b = bin_arr[i];
    const uint32_t at = E[b] + at_arr[i];
    at_arr[i] = static_cast<uint16_t>(at);
    if (FF_IN_RANGE(p, at, kSortCap, 4)) bucketed[at] = c;
  }
  __syncthreads();
  FF_TRACE(p, 24);
  // The survivor list has the same order in every CTA (the bucketed array does
  // not: atomics), so the ranking work is shared out by list index: CTA number s of the
  // n CTAs working on the row owns the survivors i with i % n == s.  An owner thread ranks its
  // survivor inside its bucket itself (buckets of up to kUnitBucket entries: a short loop, no
  // queue, no atomics) and writes the output slot at once; survivors of larger buckets (many
  // equal keys next to a far outlier) are queued and scanned by a whole warp each.
  constexpr uint32_t kUnitBucket = 32u;
  uint16_t* big_list = reinterpret_cast<uint16_t*>(smem + kSmemRing + 98 * 1024);   // slots, <= kSortCap
#pragma unroll 1
  for (int i = tid * n_share + my_share; i < n_surv; i += kThreads * n_share) {
    const uint64_t c = sortbuf[i];
    const uint32_t b = bin_arr[i];
    const int b0 = static_cast<int>(E[b]);
    if (b0 >= k) continue;
    const uint32_t n_b = fh[b];
    if (n_b <= kUnitBucket) {
      const int me = at_arr[i];
      const int q1 = b0 + static_cast<int>(n_b);
      int cnt = 0;
#pragma unroll 4
      for (int q = b0; q < q1; ++q) {
        const uint64_t o = bucketed[q];
        cnt += (o > c || (o == c && q < me)) ? 1 : 0;
      }
      const int pos = b0 + cnt;
      if (pos < k) put(pos, c == 0ull ? -1 : comp_index(c), comp_key(c));
    } else {
      const int slot = atomicAdd(&sh.big_count, 1);
      if (FF_IN_RANGE(p, slot, kSortCap, 6)) big_list[slot] = at_arr[i];
    }
  }
  __syncthreads();
  FF_TRACE(p, 31);
  {
    const int n_big = sh.big_count;
    const int lane = tid & 31;
#pragma unroll 1
    for (int d = tid >> 5; d < n_big; d += kWarps) {   // uniform per warp
      const int me = big_list[d];
      const uint64_t c = bucketed[me];
      const uint32_t b = pad(bin_of(c));
      const int b0 = static_cast<int>(E[b]);
      const int q1 = b0 + static_cast<int>(fh[b]);
      uint32_t cnt = 0;
#pragma unroll 2
      for (int q = b0 + lane; q < q1; q += 32) {
        const uint64_t o = bucketed[q];
        cnt += (o > c || (o == c && q < me)) ? 1u : 0u;
      }
      cnt = __reduce_add_sync(0xffffffffu, cnt);
      const int pos = b0 + static_cast<int>(cnt);
      if (lane == 0 && pos < k) put(pos, c == 0ull ? -1 : comp_index(c), comp_key(c));
    }
  }
  // Next call's guess: a score of rank hint_target_rank(k), so that about that many elements (between k and
  // 4096) pass it on similar data.  With at least that many survivors it is the lower edge of the bucket
  // that holds that rank; with fewer it is extrapolated linearly below the smallest survivor
  // from the ranks n_surv/2 and n_surv.  Two lanes of the row's first CTA each find one bucket by a
  // binary search over the buckets' suffix counts (the same in every CTA).
  if (kHinted && !HAS_MAP && p.hint_out != nullptr && my_share == 0 && tid < 32) {
    const int want = hint_target_rank(k);
    const int rank_a = min(n_surv, want) - 1;
    const int rank_m = n_surv >> 1;
    const int rank_mine = (tid & 1) ? rank_m : rank_a;
    int b_lo = 0, b_hi = kFinishBins - 1;   // largest bucket b with #(bins >= b) > rank
#pragma unroll 1
    while (b_lo < b_hi) {
      const int mid = (b_lo + b_hi + 1) >> 1;
      const uint32_t pm = pad(static_cast<uint32_t>(mid));
      if (static_cast<int>(E[pm] + fh[pm]) > rank_mine) b_lo = mid; else b_hi = mid - 1;
    }
    // lower edge of that bucket, as a key (the index half of the joined value is dropped)
    const uint32_t edge_key = hmin + (static_cast<uint32_t>((static_cast<uint64_t>(b_lo) << bshift) >> lbits) << ktz);
    const float v_mine = __uint_as_float(bits_of_key(edge_key));
    const float va = __shfl_sync(0xffffffffu, v_mine, 0);
    const float vm = __shfl_sync(0xffffffffu, v_mine, 1);
    if (tid == 0) {
      float guess = va;
      if (n_surv < want && rank_a > rank_m) {
        const float lower = va - (vm - va) * (static_cast<float>(want - 1 - rank_a) / static_cast<float>(rank_a - rank_m));
        if (lower == lower && fabsf(lower) <= 3.0e38f) guess = lower;   // finite
      }
      p.hint_out[row] = guess;
    }
  }
  FF_TRACE(p, 25);
  leave_scratch();
  return sx_done;
}

// One CTA's whole job for one rank: the row body, and in context-parallel send mode the step
// counter and (single-kernel step) the merge of the row's candidates from all ranks.
template <bool HAS_MAP, int MODE, typename T>
__device__ __forceinline__ void topk_cta(const TopkParams& p, unsigned char* smem, ClusterShared& sh) {
  constexpr bool kPush = (MODE & kModePush) != 0;
  // Context-parallel send: this launch also delivers its result to the peers.  The step number is
  // read from device memory (graph replays), the slot it selects is fixed for the whole launch.
  PushCtx push;
  push.off = 0;
  push.step = 0u;
  uint32_t* ctrl = nullptr;
  if (kPush && !HAS_MAP && p.push_world > 0) {
    ctrl = p.push_peers.base[p.push_rank] + p.push_ctrl_offset;
    push.step = *reinterpret_cast<volatile uint32_t*>(ctrl + kEpochWord) + 1u;
    push.off = (static_cast<int64_t>(push.step & 1u) * p.push_world + p.push_rank) * p.push_slot_words;
  }
  const bool written = topk_row_body<HAS_MAP, MODE, T>(p, smem, sh, push);
  if (kPush && !HAS_MAP && p.push_world > 0) {
    FF_TRACE(p, 32);
    // Every CTA read the step long ago; the one that counts itself last advances the counter.
    // The atomic is issued here and its result is looked at only after the merge below, so its
    // round trip overlaps the merge instead of delaying it.
    uint32_t counted_before = 0u;
    if (threadIdx.x == 32) counted_before = atomicAdd(ctrl + kPushDoneWord, 1u);
    if (p.push_fused != 0 && !written) {
      // Single-kernel step: merge this row's candidates right here.  All CTAs of the launch are
      // resident at once (cooperative launch), so a CTA that polls cannot keep a CTA that has
      // yet to store its entries from running.
      //
      // Round 1 works on the PREFIXES: the first S = push_prefix candidates of every rank's run,
      // which is all the peers were sent.  The row's first CTAs share those world x S candidates
      // out (at least one per thread); each stages all prefix keys in shared memory, polling
      // every entry until it carries this step, and ranks its share by binary searches.  The
      // prefixes hold the row's whole top-k exactly when, for every rank, the LAST candidate of
      // its prefix is not among the first k of the merged prefixes (then nothing behind it can
      // be either).  Every merging CTA of every rank checks that itself on the same keys, so all
      // reach the same verdict without talking to each other.
      // Round 2 (rare: most winners in few shards): every rank's merging CTAs send the rest of
      // their own run to the peers, and the merge is redone on the full runs.
      cg::cluster_group cluster = cg::this_cluster();
      const int C = static_cast<int>(cluster.num_blocks());
      const int G = max(p.groups, 1);
      const int bid = static_cast<int>(blockIdx.x) - p.block_base;
      const int row = bid / (C * G);
      const int n_share = C * G;
      const int my_share = (bid / C) % G * C + static_cast<int>(cluster.block_rank());
      const int k = p.k;
      const int world = p.push_world;
      const int S = min(max(p.push_prefix, 1), k);
      const int glen = p.lengths[row];
      const int n_cand = world * S;
      // kMergePer candidates per merging CTA (one per thread of its first warps): ranking costs
      // issue slots, so it is spread thin over many CTAs rather than packed into a few
      constexpr int kMergePer = 128;
      int per = (n_cand + n_share - 1) / n_share;
      if (per < kMergePer) per = kMergePer;
      const int n_merge = (n_cand + per - 1) / per;   // CTAs of the row that merge
      const int begin = my_share * per;
      int32_t* out_row = p.out_idx + static_cast<int64_t>(row) * k;
      if (glen <= k) {   // short row: identity order, as everywhere else
        if (my_share == 0)
          for (int j = threadIdx.x; j < k; j += kThreads) out_row[j] = j < glen ? j : -1;
      } else if (begin < n_cand) {
        RunSource src;
        src.base = p.push_peers.base[p.push_rank] + static_cast<int64_t>(push.step & 1u) * world * p.push_slot_words;
        src.slot_words = p.push_slot_words;
        src.row_words = 4 * static_cast<int64_t>(row) * k;
        uint32_t* run_keys = reinterpret_cast<uint32_t*>(smem + kSmemRing);   // [world][S] or [world][k], at most 128 KiB
        __syncthreads();   // the ring region is free in the whole CTA
        FF_TRACE(p, 36);
        const int log_sp = log2_ceil(S);
        bool ok = stage_run_keys(src, world, S, log_sp, push.step, run_keys);
        FF_TRACE(p, 33);
        const int end = min(n_cand, begin + per);
        const bool one_each = per <= kThreads - 32;   // one candidate per thread; the last warp checks the heads meanwhile
        const int c = one_each ? begin + static_cast<int>(threadIdx.x) : 0;
        int rank;
        const bool short_of =
            rank_share_and_check_heads(run_keys, world, S, log_sp, k, c, one_each ? end : 0, S < k, rank);
        FF_TRACE(p, 37);
        const bool enough = S >= k || __syncthreads_or(short_of ? 1 : 0) == 0;
        FF_TRACE(p, 34);
        if (enough) {
          if (one_each) ok = write_winner(src, S, c, rank, k, push.step, global_ns(), out_row) && ok;
          else ok = rank_and_write(src, run_keys, world, k, S, log_sp, push.step, begin, end, out_row) && ok;
        }
        if (!enough) {
          // the rest of this rank's run: from its own slot to every peer, shared out over the merging CTAs
          const unsigned long long t0 = global_ns();
          for (int j = S + my_share * kThreads + static_cast<int>(threadIdx.x); j < k; j += n_merge * kThreads) {
            const uint32_t* ve = src.value_entry(p.push_rank, j);
            const uint32_t vbits = await_entry(ve, ld_entry(ve), push.step, t0, ok);
            const uint32_t gidx = await_entry(ve + 2, ld_entry(ve + 2), push.step, t0, ok);
            if (ok) {
              const size_t at = push.off + 4 * (static_cast<size_t>(row) * k + j);
              for (int q = 0; q < world; ++q)
                if (q != p.push_rank) st_entry(p.push_peers.base[q] + at, vbits, gidx, push.step);
            }
          }
          __syncthreads();   // the prefix keys are not needed any more
          const int log_k = log2_ceil(k);
          ok = stage_run_keys(src, world, k, log_k, push.step, run_keys) && ok;
          const int all = world * k;
          const int slice = (all + n_merge - 1) / n_merge;
          ok = rank_and_write(src, run_keys, world, k, k, log_k, push.step, my_share * slice,
                              min(all, (my_share + 1) * slice), out_row) && ok;
          if (p.status != nullptr && threadIdx.x == 0 && my_share == 0) atomicOr(p.status, 16);
        }
        FF_TRACE(p, 35);
        if (!ok && p.status != nullptr) atomicOr(p.status, 2);
      }
    }
    if (threadIdx.x == 32 && counted_before == static_cast<uint32_t>(p.grid_ctas) - 1u) {
      ctrl[kPushDoneWord] = 0u;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(ctrl + kEpochWord) = push.step;
    }
  }
}

template <bool HAS_MAP, int MODE, typename T = float>
__global__ void __launch_bounds__(kThreads, 1) topk_cluster_kernel(const TopkParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ ClusterShared sh;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  topk_cta<HAS_MAP, MODE, T>(p, smem, sh);
}

// Several ranks of a context-parallel step played by ONE cooperative launch on one GPU (for
// tests on a box with fewer GPUs than ranks: kernels that wait for one another must never be
// separate launches on one device).  Rank r owns the CTAs [r * ctas_per_rank, (r + 1) * ctas_per_rank).
constexpr int kMaxEmulatedRanks = 8;
struct EmulatedRanks {
  TopkParams rank[kMaxEmulatedRanks];
  int32_t ctas_per_rank;
};
template <int MODE>
__global__ void __launch_bounds__(kThreads, 1) topk_emulated_ranks_kernel(const __grid_constant__ EmulatedRanks e) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ ClusterShared sh;
  topk_cta<false, MODE, float>(e.rank[blockIdx.x / e.ctas_per_rank], smem, sh);
}

}  // namespace ff
