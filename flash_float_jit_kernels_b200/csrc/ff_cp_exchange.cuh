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
// Both words of an entry with one 16-byte request: {payload0, step0, payload1, step1}.  The two
// halves are validated separately (each 64-bit half is written whole).
__device__ __forceinline__ uint4 ld_entry_pair(const uint32_t* entry) {
  unsigned long long a, b;
  asm volatile("ld.volatile.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(entry) : "memory");
  return make_uint4(static_cast<uint32_t>(a), static_cast<uint32_t>(a >> 32), static_cast<uint32_t>(b),
                    static_cast<uint32_t>(b >> 32));
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Polls the entry until it carries `step`; gives up (ok = false, payload = no candidate) when
// more than kPeerWaitNs have passed since t0.
// Polls both halves of an entry until each carries `step`, pausing between polls so that many
// waiting threads do not keep the writers out of the memory system; gives up like await_entry.
__device__ __forceinline__ uint2 await_entry_pair(const uint32_t* entry, uint4 first, uint32_t step,
                                                  unsigned long long t0, bool& ok) {
  uint4 e = first;
  while (e.y != step || e.w != step) {
    if (global_ns() - t0 > kPeerWaitNs) {
      ok = false;
      return make_uint2(kNoCandidateBits, 0xffffffffu);
    }
    __nanosleep(100);
    e = ld_entry_pair(entry);
  }
  return make_uint2(e.x, e.z);
}
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

// Staged runs live in shared memory as run_keys[world][Sp]: Sp = 2^log_sp is the staged length S
// rounded up to a power of two, positions [S, Sp) hold key 0 (below every real key), so that the
// searches below take fixed power-of-two steps without range checks.
__device__ __forceinline__ int log2_ceil(int n) {
  int l = 0;
  while ((1 << l) < n) ++l;
  return l;
}

// Waits for the value entries of the first S candidates of every rank's run of the row and stages
// their monotone keys in run_keys[world][Sp] (shared memory).  Sixteen entries per thread are in
// flight at a time (every round of loads costs a trip to L2 or memory).  Returns false
// (uniformly) if an entry did not arrive in time.
__device__ __forceinline__ bool stage_run_keys(const RunSource& src, int world, int S, int log_sp, uint32_t step,
                                               uint32_t* run_keys) {
  constexpr int kInFlight = 16;
  const int n_slots = world << log_sp;
  const int sp_mask = (1 << log_sp) - 1;
  const int nthreads = static_cast<int>(blockDim.x);
  const unsigned long long t0 = global_ns();
  bool ok = true;
  for (int i0 = threadIdx.x; i0 < n_slots; i0 += kInFlight * nthreads) {
    uint2 e[kInFlight];
#pragma unroll
    for (int u = 0; u < kInFlight; ++u) {
      const int i = i0 + u * nthreads;
      if (i < n_slots && (i & sp_mask) < S) e[u] = ld_entry(src.value_entry(i >> log_sp, i & sp_mask));
    }
#pragma unroll
    for (int u = 0; u < kInFlight; ++u) {
      const int i = i0 + u * nthreads;
      if (i < n_slots) {
        uint32_t k = 0u;
        if ((i & sp_mask) < S) {
          uint32_t bits = e[u].x;
          if (e[u].y != step)   // not there yet: poll (rare once the peers are in step)
            bits = await_entry(src.value_entry(i >> log_sp, i & sp_mask), e[u], step, t0, ok);
          k = run_key_of_bits(bits);
        }
        run_keys[i] = k;
      }
    }
  }
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
  uint32_t v;
  asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}

// Global rank of candidate j (key `key`) of run `run` among the staged runs.  Every rank's run
// is in canonical order (value desc, index asc) and the shards are contiguous in rank order, so
//   rank = j + sum over q < run of #(key_q >= key) + sum over q > run of #(key_q > key).
// Each term is a binary search; the searches of all runs advance in lockstep, loads first, so
// that one independent shared-memory load per run is in flight instead of one dependent load at a
// time (measured on B200, 8 runs of 512 keys: 0.4 us against 2.9 us for one search after the
// other).  W >= world is a compile-time bound that keeps the per-run state in registers.
template <int W, int LOG>
__device__ __noinline__ int rank_among_runs_w(uint32_t base, int world, int log_sp_rt, int run, int j, uint32_t key) {
  // LOG >= 0: log_sp is the compile-time LOG and the level loop is unrolled (the common shapes;
  // unrolled it measured 0.37 us for 8 runs of 512 keys, as a loop 1.5 us); LOG < 0: any log_sp.
  const int log_sp = LOG >= 0 ? LOG : log_sp_rt;
  // Keys of run q that come before `key`: those > key, and for q < run also those == key (ties go
  // to the lower shard): kq > bound[q] with bound = key - 1 for q < run (key >= 1 for every real
  // candidate) and key for q > run.  The own run and the slots q >= world get the largest bound, so
  // nothing of theirs counts; a slot q >= world probes run 0's keys, so that every address is inside
  // the staged runs.  at[q] is the byte address of the last key of run q known to come before `key`
  // (one element before the run when there is none yet).
  uint32_t bound[W], at[W];
  auto origin = [&](int q) { return base + (static_cast<uint32_t>(q < world ? q : 0) << (log_sp + 2)) - 4u; };
#pragma unroll
  for (int q = 0; q < W; ++q) {
    at[q] = origin(q);
    bound[q] = (q >= world || q == run) ? 0xffffffffu : (q < run ? key - 1u : key);
  }
  // steps Sp/2, ..., 1 find min(count, Sp - 1); the last round (l = -1) probes the one element
  // after it, which decides between Sp - 1 and Sp and adds nothing otherwise
  auto level = [&](int l) {
    const uint32_t stepb = l >= 0 ? (4u << l) : 4u;
    uint32_t kq[W];
#pragma unroll
    for (int q = 0; q < W; ++q) kq[q] = lds_u32(at[q] + stepb);
#pragma unroll
    for (int q = 0; q < W; ++q) at[q] += kq[q] > bound[q] ? stepb : 0u;
  };
  if constexpr (LOG >= 0) {
#pragma unroll
    for (int l = LOG - 1; l >= -1; --l) level(l);
  } else {
#pragma unroll 1
    for (int l = log_sp - 1; l >= -1; --l) level(l);
  }
  int rank = j;
#pragma unroll
  for (int q = 0; q < W; ++q) rank += static_cast<int>((at[q] - origin(q)) >> 2);
  return rank;
}

// The staged shapes of a step with the default head length and k = 2048 (2 ranks: whole runs of
// 2048; 4 ranks: heads of 1024; 8 ranks: heads of 512) take the unrolled searches.
__device__ __forceinline__ int rank_among_runs(const uint32_t* run_keys, int world, int log_sp, int run, int j,
                                               uint32_t key) {
  const uint32_t base = static_cast<uint32_t>(__cvta_generic_to_shared(run_keys));
  if (world <= 2)
    return log_sp == 11 ? rank_among_runs_w<2, 11>(base, world, log_sp, run, j, key)
                        : rank_among_runs_w<2, -1>(base, world, log_sp, run, j, key);
  if (world <= 4)
    return log_sp == 10 ? rank_among_runs_w<4, 10>(base, world, log_sp, run, j, key)
                        : rank_among_runs_w<4, -1>(base, world, log_sp, run, j, key);
  if (world <= 8)
    return log_sp == 9 ? rank_among_runs_w<8, 9>(base, world, log_sp, run, j, key)
                       : rank_among_runs_w<8, -1>(base, world, log_sp, run, j, key);
  return rank_among_runs_w<kMaxPeers, -1>(base, world, log_sp, run, j, key);
}

// Ranks this thread's candidate c = run * S + j (if c < end and it is a real candidate) among the
// staged runs and, meanwhile, lets `world` otherwise idle threads (the CTA's last warp) rank the
// LAST staged candidate of every run.  The first k of the merged heads (S < k keys per run) are the
// first k of the merged full runs exactly when none of those last candidates ranks among the first k
// (everything behind it in its run is below it, so it cannot rank there either); an unused last
// position (key 0) means that run was sent whole.  Returns this thread's part of that verdict
// (true: a last candidate ranks among the first k); the caller ORs it over the CTA, and every CTA
// and rank that stages the same keys gets the same answer.  `rank_out` gets this thread's
// candidate's rank, or k if it has none.  Threads [0, kThreads - 32) may hold candidates.
__device__ __forceinline__ bool rank_share_and_check_heads(const uint32_t* run_keys, int world, int S, int log_sp, int k,
                                                           int c, int end, bool check, int& rank_out) {
  const int tid = threadIdx.x;
  bool short_of = false;
  rank_out = k;
  int run = 0, j = 0;
  uint32_t key = 0u;
  if (c < end) {
    run = c / S;
    j = c - run * S;
    key = run_keys[(run << log_sp) + j];
  } else if (check && tid >= kThreads - 32 && tid - (kThreads - 32) < world) {
    run = tid - (kThreads - 32);
    j = S - 1;
    key = run_keys[(run << log_sp) + j];
  }
  if (key != 0u) {
    const int r = rank_among_runs(run_keys, world, log_sp, run, j, key);
    if (c < end) rank_out = r; else short_of = r < k;
  }
  return short_of;
}

// Writes the winner's global index (rank < k) to its output position once its index entry has arrived.
__device__ __forceinline__ bool write_winner(const RunSource& src, int S, int c, int rank, int k, uint32_t step,
                                             unsigned long long t0, int32_t* out_row) {
  bool ok = true;
  if (rank < k) {
    const int run = c / S;
    const uint32_t* ie = src.index_entry(run, c - run * S);
    const uint32_t gidx = await_entry(ie, ld_entry(ie), step, t0, ok);
    if (ok) out_row[rank] = static_cast<int32_t>(gidx);
  }
  return ok;
}

// Ranks candidates [begin, end) of the row's world x S staged ones (c = run * S + j) and writes each
// winner's global index straight to its output position (any number of candidates per thread; no
// head check).  run_keys must be staged.  Returns false if an index entry did not arrive in time
// (thread-local).
__device__ __forceinline__ bool rank_and_write(const RunSource& src, const uint32_t* run_keys, int world, int k, int S,
                                               int log_sp, uint32_t step, int begin, int end, int32_t* out_row) {
  const unsigned long long t0 = global_ns();
  bool ok = true;
  for (int c = begin + threadIdx.x; c < end; c += blockDim.x) {
    const int run = c / S;
    const int j = c - run * S;
    const uint32_t key = run_keys[(run << log_sp) + j];
    if (key == 0u) continue;   // no candidate here
    const int rank = rank_among_runs(run_keys, world, log_sp, run, j, key);
    ok = write_winner(src, S, c, rank, k, step, t0, out_row) && ok;
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
  const int log_sp = log2_ceil(k);
  bool ok = stage_run_keys(src, p.world, k, log_sp, step, run_keys);   // the send launch delivered whole runs
  const int begin = blockIdx.x * blockDim.x;
  const int end = min(p.world * k, begin + static_cast<int>(blockDim.x));
  ok = rank_and_write(src, run_keys, p.world, k, k, log_sp, step, begin, end,
                      p.out_idx + static_cast<int64_t>(row) * k) && ok;
  if (!ok && p.status != nullptr) atomicOr(p.status, 2);
}

}  // namespace ff
