// One thread-block cluster per row: exact radix select on the 64-bit composite
// (monotone fp32 key, ~index) followed by a finishing sort of the survivors.
//
// Role in the reference: replaces topk_kernel<TopK> / fast_topk_split_kv_cuda_tl
// (jit_kernel/csrc/topk_indexer/topk_indexer_radix.cu:554-997) and the
// single-CTA topk_kernel_small_k (jit_kernel/csrc/topk_indexer/top_small_k.cuh:84-348).
// Differences by design: keys are the full order-preserving 32-bit map (any
// fp32 input, not only [0,256)); the first digit is 12 bits; per-CTA histograms
// are merged as a reduce-scatter over distributed shared memory followed by a
// cluster-wide suffix scan over unequal slices; nothing is ever dropped (a CTA
// whose threshold-bin candidates do not fit its buffer re-sweeps its chunk
// instead); ties are broken toward the lowest index by continuing the radix
// select into the index bits; the output is in canonical order.
#pragma once

#include <cooperative_groups.h>

#include "ff_topk_common.cuh"

namespace ff {

namespace cg = cooperative_groups;

// Dynamic shared memory layout (bytes).
constexpr int kSmemHist = 0;                                   // uint32[kMaxBins]
constexpr int kSmemStage = kSmemHist + kMaxBins * 4;           // uint64[kSortCap]; merged slice aliases its head
constexpr int kSmemSort = kSmemStage + kSortCap * 8;           // uint64[kSortCap] (used on cluster rank 0)
constexpr int kSmemCand = kSmemSort + kSortCap * 8;            // uint64[kCandCap]
constexpr int kSmemBytes = kSmemCand + kCandCap * 8;

// Geometry of one row as seen by one CTA of the cluster.  The row is cut into
// 16-byte units on absolute addresses so interior units load as float4 even
// when row_starts or an odd row stride misaligns the window.
struct Chunk {
  const float* abase;     // 16-byte aligned, abase + mis == first element of the window
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

__device__ __forceinline__ Chunk make_chunk(const float* row, const int32_t* imap, int len, int C,
                                            int rank, int seg_len, int64_t seg_stride) {
  Chunk c;
  c.mis = static_cast<int>((reinterpret_cast<uintptr_t>(row) >> 2) & 3);
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
  const int U = static_cast<int>((static_cast<int64_t>(len) + c.mis + 3) >> 2);
  const bool head_partial = c.mis != 0;
  const bool tail_partial = ((len + c.mis) & 3) != 0;
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

// Calls f(key, index) once for every valid position of this CTA's chunk.
template <bool HAS_MAP, typename F>
__device__ __forceinline__ void for_each_in_chunk(const Chunk& c, F&& f) {
  if (HAS_MAP) {
    // Merge mode: a few thousand (value, index) pairs in rank-strided segments.
    const float* vals = c.abase + c.mis;
    for (int i = c.pb + threadIdx.x; i < c.pe; i += kThreads) {
      const int64_t a = seg_addr(i, c.seg_len, c.seg_stride);
      const int32_t idx = c.imap[a];
      if (idx < 0) {
        f(0u, -1);
      } else {
        f(key_of(vals[a]), idx);
      }
    }
    return;
  }
  const float4* p4 = reinterpret_cast<const float4*>(c.abase);
  auto one = [&](float x, int pos) { f(key_of(x), pos); };
  auto unit = [&](const float4& v, int u) {
    const int pos = 4 * u - c.mis;
    one(v.x, pos);
    one(v.y, pos + 1);
    one(v.z, pos + 2);
    one(v.w, pos + 3);
  };
  int u = c.fb + threadIdx.x;
  for (; u + 3 * kThreads < c.fe; u += 4 * kThreads) {
    const float4 v0 = __ldg(p4 + u);
    const float4 v1 = __ldg(p4 + u + kThreads);
    const float4 v2 = __ldg(p4 + u + 2 * kThreads);
    const float4 v3 = __ldg(p4 + u + 3 * kThreads);
    unit(v0, u);
    unit(v1, u + kThreads);
    unit(v2, u + 2 * kThreads);
    unit(v3, u + 3 * kThreads);
  }
  for (; u < c.fe; u += kThreads) {
    const float4 v = __ldg(p4 + u);
    unit(v, u);
  }
  // Partial first / last unit: scalar loads of the valid lanes only.
  if (threadIdx.x < 4 && c.head) {
    const int pos = static_cast<int>(threadIdx.x) - c.mis;
    if (pos >= 0 && pos < c.len) one(c.abase[threadIdx.x], pos);
  }
  if (threadIdx.x >= 32 && threadIdx.x < 36 && c.tail) {
    const int lane = static_cast<int>(threadIdx.x) - 32;
    const int pos = 4 * c.tail_unit - c.mis + lane;
    if (pos >= 0 && pos < c.len) one(c.abase[4 * c.tail_unit + lane], pos);
  }
}

struct ClusterShared {
  int slice_tot[kMaxCluster];
  int res[4];        // threshold digit, count above it, count in it, (unused)
  int warp_tot[kWarps];
  int stage_count;
  int sort_count;
  int cand_count;
  int push_base;
  int table_row;
};

// Cluster-wide histogram merge (reduce-scatter over distributed shared memory)
// and suffix scan over the per-CTA slices.  On return every CTA's sh.res holds
// the digit t with  #(digit > t) < r <= #(digit >= t), and those two counts.
__device__ __forceinline__ void merge_and_scan(cg::cluster_group& cluster, int C, int rank,
                                               uint32_t* hist, uint32_t* merged, int nbins, int r,
                                               ClusterShared& sh) {
  const int tid = threadIdx.x;
  cluster.sync();  // every CTA's local histogram is complete and visible
  const int slice_n = nbins / C;
  const int slice_base = rank * slice_n;
  for (int i = tid; i < slice_n; i += kThreads) {
    uint32_t s = 0;
    for (int c = 0; c < C; ++c) s += cluster.map_shared_rank(hist, c)[slice_base + i];
    merged[i] = s;
  }
  if (tid == 0) sh.res[0] = -1;
  __syncthreads();
  const int per = slice_n >= kThreads ? slice_n / kThreads : 1;
  const int first = tid * per;
  int local = 0;
  if (first < slice_n) {
    for (int e = 0; e < per; ++e) local += static_cast<int>(merged[first + e]);
  }
  int total;
  const int excl = block_suffix_exclusive(local, sh.warp_tot, total);
  if (tid < C) cluster.map_shared_rank(sh.slice_tot, tid)[rank] = total;
  cluster.sync();  // slice totals of every CTA have arrived
  int above_slice = 0;
  for (int c = rank + 1; c < C; ++c) above_slice += sh.slice_tot[c];
  if (first < slice_n) {
    int running = above_slice + excl;
    for (int e = per - 1; e >= 0; --e) {
      const int cnt = static_cast<int>(merged[first + e]);
      const int next = running;
      running += cnt;
      if (next < r && r <= running) {
        for (int c = 0; c < C; ++c) {
          int* rr = cluster.map_shared_rank(sh.res, c);
          rr[1] = next;
          rr[2] = cnt;
          rr[0] = slice_base + first + e;
        }
      }
    }
  }
  cluster.sync();  // the threshold triple has arrived everywhere
}

// Descending bitonic sort of buf[0, n) (n a power of two) in shared memory.
__device__ __forceinline__ void bitonic_sort_desc(uint64_t* buf, int n) {
  for (int size = 2; size <= n; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      __syncthreads();
      for (int q = threadIdx.x; q < (n >> 1); q += kThreads) {
        const int i = 2 * q - (q & (stride - 1));
        const int j = i + stride;
        const uint64_t a = buf[i];
        const uint64_t b = buf[j];
        const bool desc = (i & size) == 0;
        if ((a < b) == desc) {
          buf[i] = b;
          buf[j] = a;
        }
      }
    }
  }
  __syncthreads();
}

// Writes output slot j of `row` from a window-relative index (or -1) and key.
__device__ __forceinline__ void emit(const TopkParams& p, int row, int j, int32_t idx, uint32_t key,
                                     bool is_map, int table_row) {
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
  p.out_idx[static_cast<int64_t>(row) * p.k + j] = o;
  if (p.out_val != nullptr) {
    p.out_val[static_cast<int64_t>(row) * p.k + j] =
        idx < 0 ? __uint_as_float(0xff800000u) : __uint_as_float(bits_of_key(key));
  }
}

template <bool HAS_MAP>
__global__ void __launch_bounds__(kThreads) topk_cluster_kernel(const TopkParams p) {
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ ClusterShared sh;
  uint32_t* hist = reinterpret_cast<uint32_t*>(smem + kSmemHist);
  uint64_t* stage = reinterpret_cast<uint64_t*>(smem + kSmemStage);
  uint32_t* merged = reinterpret_cast<uint32_t*>(smem + kSmemStage);
  uint64_t* sortbuf = reinterpret_cast<uint64_t*>(smem + kSmemSort);
  uint64_t* cand = reinterpret_cast<uint64_t*>(smem + kSmemCand);

  cg::cluster_group cluster = cg::this_cluster();
  const int C = static_cast<int>(cluster.num_blocks());
  const int rank = static_cast<int>(cluster.block_rank());
  const int row = static_cast<int>(blockIdx.x) / C;
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
  const float* rowp = p.scores + static_cast<int64_t>(row) * p.row_stride + rs;
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
  if (identity || len <= k) {
    if (rank != 0) return;
    for (int j = tid; j < k; j += kThreads) {
      if (HAS_MAP && !identity) {
        // no more candidates than k slots: pass them through in position order
        const int64_t a = j < len ? seg_addr(j, p.seg_len, p.seg_stride) : 0;
        const int32_t idx = j < len ? imap[a] : -1;
        emit(p, row, j, idx, j < len ? key_of(rowp[a]) : 0u, true, table_row);
      } else {
        const int n = HAS_MAP ? glen : len;
        const bool v = j < n;
        uint32_t key = 0u;
        if (v && !HAS_MAP && p.out_val != nullptr) key = key_of(rowp[j]);
        emit(p, row, j, v ? j : -1, key, HAS_MAP, table_row);
      }
    }
    return;
  }

  const Chunk chunk = make_chunk(rowp, imap, len, C, rank, p.seg_len, p.seg_stride);

  // ---- level 0: 12-bit histogram of the whole chunk -----------------------
  for (int i = tid; i < kMaxBins; i += kThreads) hist[i] = 0u;
  if (tid == 0) {
    sh.stage_count = 0;
    sh.sort_count = 0;
    sh.cand_count = 0;
  }
  __syncthreads();
  for_each_in_chunk<HAS_MAP>(chunk, [&](uint32_t key, int32_t) { atomicAdd(&hist[key >> 20], 1u); });

  int r = k;                // survivors still to be taken from the current candidate set
  uint64_t P = 0;           // digits fixed so far (value of comp >> shift of the last level)
  bool src_is_cand = false; // candidates live in `cand` instead of the chunk
  int cand_n = 0;
  bool ok = true;
  int expected_total = 0;

  for (int level = 0; level < kNumLevels; ++level) {
    const int bits = level_bits(level);
    const int shift = level_shift(level);
    merge_and_scan(cluster, C, rank, hist, merged, 1 << bits, r, sh);
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
    const int local_m = static_cast<int>(hist[t]);
    const bool compact = !final_level && !src_is_cand && local_m <= kCandCap;
    const int nshift = final_level ? 0 : level_shift(level + 1);
    const uint32_t nmask = final_level ? 0u : ((1u << level_bits(level + 1)) - 1u);
    __syncthreads();
    if (!final_level) {
      for (int i = tid; i < (1 << level_bits(level + 1)); i += kThreads) hist[i] = 0u;
    }
    __syncthreads();

    auto classify = [&](uint64_t comp) {
      const uint64_t hi = comp >> shift;
      if (hi == Pn) {
        if (final_level) {
          const int pos = atomicAdd(&sh.stage_count, 1);
          if (pos < kSortCap) stage[pos] = comp;
        } else {
          atomicAdd(&hist[static_cast<uint32_t>(comp >> nshift) & nmask], 1u);
          if (compact) {
            const int pos = atomicAdd(&sh.cand_count, 1);
            if (pos < kCandCap) cand[pos] = comp;
          }
        }
      } else if (hi > Pn && hi <= Pmax) {
        const int pos = atomicAdd(&sh.stage_count, 1);
        if (pos < kSortCap) stage[pos] = comp;
      }
    };
    if (src_is_cand) {
      for (int i = tid; i < cand_n; i += kThreads) classify(cand[i]);
    } else {
      for_each_in_chunk<HAS_MAP>(chunk,
                                 [&](uint32_t key, int32_t idx) { classify(make_comp(key, idx)); });
    }
    __syncthreads();

    // Move this CTA's survivors into rank 0's sort buffer: one remote atomic
    // reserves a contiguous block, then coalesced remote stores fill it.
    const int n_stage = min(sh.stage_count, kSortCap);
    if (n_stage > 0) {
      if (tid == 0) sh.push_base = atomicAdd(&cluster.map_shared_rank(&sh, 0)->sort_count, n_stage);
      __syncthreads();
      uint64_t* dst = cluster.map_shared_rank(sortbuf, 0);
      const int base = sh.push_base;
      for (int i = tid; i < n_stage; i += kThreads) {
        if (base + i < kSortCap) dst[base + i] = stage[i];
      }
    }
    __syncthreads();
    if (tid == 0) sh.stage_count = 0;
    if (compact) {
      src_is_cand = true;
      cand_n = min(sh.cand_count, kCandCap);
    }
    if (final_level) {
      expected_total = total;
      break;
    }
    r -= above;
    P = Pn;
  }

  cluster.sync();  // every survivor has landed in rank 0's sort buffer
  if (rank != 0) return;

  // ---- finishing sort on the cluster's first CTA --------------------------
  int T = ok ? min(sh.sort_count, kSortCap) : 0;
  if (ok && T != expected_total && p.status != nullptr && tid == 0)
    atomicOr(p.status, 1);
  if (!ok && p.status != nullptr && tid == 0) atomicOr(p.status, 4);
  int n = 32;
  while (n < T) n <<= 1;
  for (int i = T + tid; i < n; i += kThreads) sortbuf[i] = 0ull;
  bitonic_sort_desc(sortbuf, n);
  for (int j = tid; j < k; j += kThreads) {
    const uint64_t c = j < T ? sortbuf[j] : 0ull;
    emit(p, row, j, c == 0ull ? -1 : comp_index(c), comp_key(c), HAS_MAP, table_row);
  }
}

}  // namespace ff
