// Context-parallel candidate exchange over peer memory (NVLink / NVSwitch).
//
// Every rank owns one allocation holding, for two alternating steps ("parities"),
// a receive slot per rank and a flag per rank.  The shard-local select kernel
// stores the rank's k candidates per row straight into EVERY peer's receive slot
// with plain global stores as it ranks them; its last CTA fences at system scope
// and raises the rank's flag in every peer's memory; the merge kernel on
// each rank polls its own (local) flags with a bounded wait and then reads the
// candidates from local memory only.  No collective library call, no multicast.
// The reference has no multi-GPU path; semantics follow fast_topk_v3
// (jit_kernel/topk_indexer.py:109) on the unsharded row.
//
// Two parities suffice: a rank can only be one step ahead of a peer, because its
// merge of step s needs that peer's push of step s, which the peer issues after
// its own merge of step s-1 on the same stream.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "ff_topk_common.cuh"

namespace ff {

constexpr unsigned long long kPeerWaitNs = 1000000000ull;   // bounded wait for a peer's flag: one second

// The step number lives in device memory (word kEpochWord after the flags) so
// that a captured CUDA graph can be replayed.  The select kernel of a step reads
// step = counter + 1 when it starts, stores its candidates into the slot (step
// parity, rank) of every peer as it ranks them, and the CTA that finishes last in
// the whole launch (a done-count next to the counter) raises this rank's flag in
// every peer to `step` and advances the counter (ff_topk_kernel.cuh).  The merge
// kernel of the same step, a later launch on the same stream, reads it back.
constexpr int kEpochWord = 2 * kMaxPeers;
constexpr int kPushDoneWord = kEpochWord + 1;

// Polls `n` flags until each has reached `epoch`; returns false if a second passed.
__device__ __forceinline__ bool wait_for_peers(const uint32_t* flags, int n, uint32_t epoch) {
  bool ok = true;
  if (static_cast<int>(threadIdx.x) < n) {
    unsigned long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (;;) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + threadIdx.x) : "memory");
      if (static_cast<int32_t>(v - epoch) >= 0) break;
      unsigned long long t1;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
      if (t1 - t0 > kPeerWaitNs) {
        ok = false;
        break;
      }
    }
  }
  return __syncthreads_and(ok ? 1 : 0) != 0;
}

// Merge-select for the exchange path.  Every rank's block is a run already in
// canonical order (value desc, index asc) and the shards are contiguous in rank
// order, so the global rank of candidate j of run p is
//   j + sum over q < p of #(key_q >= key) + sum over q > p of #(key_q > key),
// each term one binary search on the keys of run q.  One thread per candidate
// writes its index straight to its output slot; nothing is sorted or staged.
struct CpMergeParams {
  const uint32_t* recv_even;   // receive buffer of even steps: [world][slot_words]
  int64_t parity_stride;       // words to the buffer of odd steps
  int64_t slot_words;          // per rank: value plane [B*k], index plane [B*k]
  const uint32_t* flags;       // [2][kMaxPeers] flags, then the step counter
  const int32_t* lengths;      // global row lengths
  int32_t* out_idx;            // [B, k]
  int32_t* status;
  int world, B, k;
};

__global__ void __launch_bounds__(1024) cp_merge_sorted_kernel(const CpMergeParams p) {
  extern __shared__ uint32_t run_keys[];   // [world][k] monotone keys of this row's runs
  __shared__ int n_valid[kMaxPeers];
  const int row = blockIdx.y;
  const uint32_t step = p.flags[kEpochWord];
  const int parity = static_cast<int>(step & 1u);
  if (!wait_for_peers(p.flags + parity * kMaxPeers, p.world, step) && p.status != nullptr && threadIdx.x == 0)
    atomicOr(p.status, 2);
  const int k = p.k;
  const int glen = p.lengths[row];
  if (glen <= k) {   // short row: identity order, as everywhere else
    if (blockIdx.x == 0) {
      for (int j = threadIdx.x; j < k; j += blockDim.x) p.out_idx[static_cast<int64_t>(row) * k + j] = j < glen ? j : -1;
    }
    return;
  }
  const uint32_t* base = p.recv_even + parity * p.parity_stride;
  const size_t plane = static_cast<size_t>(p.B) * k;
  auto idx_of = [&](int q, int j) {
    return static_cast<int32_t>(base[static_cast<size_t>(q) * p.slot_words + plane + static_cast<size_t>(row) * k + j]);
  };
  // stage the keys of all runs in shared memory: the binary searches then never leave the SM
  for (int i = threadIdx.x; i < p.world * k; i += blockDim.x) {
    const int q = i / k;
    run_keys[i] = key_of_bits(base[static_cast<size_t>(q) * p.slot_words + static_cast<size_t>(row) * k + (i - q * k)]);
  }
  if (static_cast<int>(threadIdx.x) < p.world) {   // valid entries of run q: unused slots (index -1) sit at its tail
    const int q = threadIdx.x;
    int lo = 0, hi = k;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (idx_of(q, mid) >= 0) lo = mid + 1; else hi = mid;
    }
    n_valid[q] = lo;
  }
  __syncthreads();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= p.world * k) return;
  const int run = c / k;
  const int j = c - run * k;
  if (j >= n_valid[run]) return;
  const uint32_t key = run_keys[c];
  int rank = j;
  for (int q = 0; q < p.world; ++q) {
    if (q == run) continue;
    const uint32_t* keys = run_keys + q * k;
    int lo = 0, hi = n_valid[q];
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      const uint32_t kq = keys[mid];
      const bool before = q < run ? kq >= key : kq > key;
      if (before) lo = mid + 1; else hi = mid;
    }
    rank += lo;
  }
  if (rank < k) p.out_idx[static_cast<int64_t>(row) * k + rank] = idx_of(run, j);
}

}  // namespace ff
