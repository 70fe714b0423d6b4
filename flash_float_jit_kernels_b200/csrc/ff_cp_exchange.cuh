// Context-parallel candidate exchange over peer memory (NVLink / NVSwitch).
//
// Every rank owns one allocation holding, for two alternating steps ("parities"),
// a receive slot per rank.  A slot holds one 16-byte entry per (row, position):
// {value bits, step, global index, step}.  The shard-local select kernel stores
// each of its k candidates per row straight into EVERY peer's slot as it ranks
// them, one 16-byte store per candidate and peer (the link carries one packet
// per store, so fewer and wider stores matter at 8 ranks).  Each half is one
// 64-bit word (payload low, step high) and a 64-bit access is single-copy
// atomic, so the step number inside each half is its own "valid" mark: the
// receiver polls a half until it carries the current step (bounded wait).  No fence, no flag, no collective library call; the
// receiver reads local memory only.
// The reference has no multi-GPU path; semantics follow fast_topk_v3
// (jit_kernel/topk_indexer.py:109) on the unsharded row.
//
// Two parities suffice: a rank can only be one step ahead of a peer, because its
// merge of step s needs that peer's entries of step s, which the peer stores
// after its own merge of step s-1 on the same stream.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "ff_topk_common.cuh"

namespace ff {

constexpr unsigned long long kPeerWaitNs = 1000000000ull;   // bounded wait for a peer's entries: one second

// Control words behind the receive slots.  The step number lives in device
// memory so that a captured CUDA graph can be replayed: every CTA of a step's
// select kernel reads step = counter + 1 when it starts and counts itself in
// kPushDoneWord once it has; the CTA that counts last advances the counter (no
// CTA of the launch reads it again).  A merge kernel launched after the select
// reads the advanced counter back.
constexpr int kEpochWord = 0;
constexpr int kPushDoneWord = 1;
constexpr int kCtrlWords = 64;

// A slot position that holds no candidate carries this value pattern (a NaN the select
// never emits: it writes NaN as 0x7fffffff); the merge turns it into key 0, below every real key.
constexpr uint32_t kNoCandidateBits = 0xffffffffu;
__device__ __forceinline__ uint32_t run_key_of_bits(uint32_t bits) {
  return bits == kNoCandidateBits ? 0u : key_of_bits(bits);
}

// An entry is two 64-bit words, {value bits | step << 32} and {global index | step << 32}.  A 64-bit
// scalar access is single-copy atomic in the PTX memory model, so a reader that sees the current
// step in a word's high half also sees that word's payload: each word validates itself.
__device__ __forceinline__ void st_entry(uint32_t* entry, uint32_t value_bits, uint32_t gidx, uint32_t step) {
  const unsigned long long hi = static_cast<unsigned long long>(step) << 32;
  asm volatile("st.volatile.global.v2.u64 [%0], {%1, %2};" ::"l"(entry), "l"(hi | value_bits), "l"(hi | gidx)
               : "memory");
}
__device__ __forceinline__ uint2 ld_entry(const uint32_t* entry) {
  unsigned long long w;
  asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(w) : "l"(entry) : "memory");
  return make_uint2(static_cast<uint32_t>(w), static_cast<uint32_t>(w >> 32));
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Polls the entry until it carries `step`; gives up (ok = false, payload = no candidate) when
// more than kPeerWaitNs have passed since t0.
__device__ __forceinline__ uint32_t await_entry(const uint32_t* entry, uint2 first, uint32_t step,
                                                unsigned long long t0, bool& ok) {
  uint2 e = first;
  while (e.y != step) {
    if (global_ns() - t0 > kPeerWaitNs) {
      ok = false;
      return kNoCandidateBits;
    }
    e = ld_entry(entry);
  }
  return e.x;
}

// Where the receive slots of one step and one row are.
struct RunSource {
  const uint32_t* base;   // this rank's receive area of the step's parity: [world][slot_words]
  int64_t slot_words;     // per rank: 4 words per (row, position)
  int64_t row_words;      // 4 * row * k
  __device__ __forceinline__ const uint32_t* value_entry(int q, int j) const {   // the {value bits, step} half
    return base + q * slot_words + row_words + 4 * j;
  }
  __device__ __forceinline__ const uint32_t* index_entry(int q, int j) const {   // the {global index, step} half
    return base + q * slot_words + row_words + 4 * j + 2;
  }
};

// Waits for the value entries of the first S candidates of every rank's run of the row and stages
// their monotone keys in run_keys[world][S] (shared memory).  Sixteen entries per thread are in
// flight at a time (every round of loads costs a trip to L2 or memory).  Returns false
// (uniformly) if an entry did not arrive in time.
__device__ __forceinline__ bool stage_run_keys(const RunSource& src, int world, int k, int S, uint32_t step,
                                               uint32_t* run_keys) {
  constexpr int kInFlight = 16;
  (void)k;
  const int n_cand = world * S;
  const int nthreads = static_cast<int>(blockDim.x);
  const unsigned long long t0 = global_ns();
  bool ok = true;
  for (int i0 = threadIdx.x; i0 < n_cand; i0 += kInFlight * nthreads) {
    uint2 e[kInFlight];
#pragma unroll
    for (int u = 0; u < kInFlight; ++u) {
      const int i = i0 + u * nthreads;
      if (i < n_cand) {
        const int q = i / S;
        e[u] = ld_entry(src.value_entry(q, i - q * S));
      }
    }
#pragma unroll
    for (int u = 0; u < kInFlight; ++u) {
      const int i = i0 + u * nthreads;
      if (i < n_cand) {
        uint32_t bits = e[u].x;
        if (e[u].y != step) {   // not there yet: poll (rare once the peers are in step)
          const int q = i / S;
          bits = await_entry(src.value_entry(q, i - q * S), e[u], step, t0, ok);
        }
        run_keys[i] = run_key_of_bits(bits);
      }
    }
  }
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

// Global rank of candidate j (key `key`) of run `run` among `world` runs of S keys each, all
// in shared memory in descending order with key 0 in unused tail positions.  Every rank's run
// is in canonical order (value desc, index asc) and the shards are contiguous in rank order, so
//   rank = j + sum over q < run of #(key_q >= key) + sum over q > run of #(key_q > key),
// each term one binary search.
__device__ __forceinline__ int rank_among_runs(const uint32_t* run_keys, int world, int S, int run, int j,
                                               uint32_t key) {
  int rank = j;
  for (int q = 0; q < world; ++q) {
    if (q == run) continue;
    const uint32_t* keys = run_keys + q * S;
    int lo = 0, hi = S;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      const uint32_t kq = keys[mid];
      const bool before = q < run ? kq >= key : kq > key;
      if (before) lo = mid + 1; else hi = mid;
    }
    rank += lo;
  }
  return rank;
}

// Whether the first k of the merged prefixes (run_keys[world][S], S < k) are the first k of the
// merged full runs: true exactly when no run's LAST prefix candidate ranks among the first k
// (everything behind it in its run is below it, so it cannot rank there either).  An unused
// last position (key 0) means that run was sent whole.  One thread per run checks; the answer
// is uniform over the CTA (and over every CTA and rank that stages the same keys).
__device__ __forceinline__ bool prefixes_suffice(const uint32_t* run_keys, int world, int S, int k) {
  bool short_of = false;
  if (static_cast<int>(threadIdx.x) < world) {
    const int q = threadIdx.x;
    const uint32_t key = run_keys[q * S + S - 1];
    short_of = key != 0u && rank_among_runs(run_keys, world, S, q, S - 1, key) < k;
  }
  return __syncthreads_or(short_of ? 1 : 0) == 0;
}

// Ranks candidates [begin, end) of the row's world x S staged ones and writes each winner's global
// index straight to its output position.  run_keys must be staged.  Returns false if an index
// entry did not arrive in time (thread-local).
__device__ __forceinline__ bool rank_and_write(const RunSource& src, const uint32_t* run_keys, int world, int k, int S,
                                               uint32_t step, int begin, int end, int32_t* out_row) {
  const unsigned long long t0 = global_ns();
  bool ok = true;
  for (int c = begin + threadIdx.x; c < end; c += blockDim.x) {
    const uint32_t key = run_keys[c];
    if (key == 0u) continue;   // no candidate here
    const int run = c / S;
    const int j = c - run * S;
    const uint32_t* ie = src.index_entry(run, j);
    const uint2 first = ld_entry(ie);
    const int rank = rank_among_runs(run_keys, world, S, run, j, key);
    if (rank >= k) continue;   // (its index entry need not be waited for)
    const uint32_t gidx = await_entry(ie, first, step, t0, ok);
    if (ok) out_row[rank] = static_cast<int32_t>(gidx);
  }
  return ok;
}

// Merge-select as a launch of its own (after the select kernel on the same stream): used when
// the select's CTAs cannot all be resident at once, and by tests that play several ranks on one
// GPU.  grid = (ceil(world * k / 1024), B); dynamic shared memory world * k * 4 bytes.
struct CpMergeParams {
  const uint32_t* recv_even;   // receive area of even steps: [world][slot_words]
  int64_t parity_words;        // words to the area of odd steps
  int64_t slot_words;
  const uint32_t* ctrl;        // control words (step counter)
  const int32_t* lengths;      // global row lengths
  int32_t* out_idx;            // [B, k]
  int32_t* status;
  int world, B, k;
};

__global__ void __launch_bounds__(1024) cp_merge_sorted_kernel(const CpMergeParams p) {
  extern __shared__ uint32_t run_keys[];   // [world][k] monotone keys of this row's runs
  const int row = blockIdx.y;
  const uint32_t step = p.ctrl[kEpochWord];   // advanced by this step's select kernel
  const int k = p.k;
  const int glen = p.lengths[row];
  if (glen <= k) {   // short row: identity order, as everywhere else
    if (blockIdx.x == 0) {
      for (int j = threadIdx.x; j < k; j += blockDim.x) p.out_idx[static_cast<int64_t>(row) * k + j] = j < glen ? j : -1;
    }
    return;
  }
  RunSource src;
  src.base = p.recv_even + static_cast<int64_t>(step & 1u) * p.parity_words;
  src.slot_words = p.slot_words;
  src.row_words = 4 * static_cast<int64_t>(row) * k;
  bool ok = stage_run_keys(src, p.world, k, k, step, run_keys);   // the send launch delivered whole runs
  const int begin = blockIdx.x * blockDim.x;
  const int end = min(p.world * k, begin + static_cast<int>(blockDim.x));
  ok = rank_and_write(src, run_keys, p.world, k, k, step, begin, end, p.out_idx + static_cast<int64_t>(row) * k) && ok;
  if (!ok && p.status != nullptr) atomicOr(p.status, 2);
}

}  // namespace ff
