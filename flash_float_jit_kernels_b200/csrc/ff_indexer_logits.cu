// Lightning-indexer logits for sm_100a: the step that produces the scores the
// top-k indexer selects from,
//     s[b, j] = sum_h w[b, h] * relu( q[b, h, :] . k[b, j, :] ),
// 64 heads, head_dim 128, q and K in fp8 e4m3, fp32 accumulation.  The reference
// has no such kernel; the shape is the one its README gives for the indexer
// (README.md:28) and the benchmark's ragged decode batch is generated this way.
//
// One CTA works on one row b and a strided share of its 128-key tiles:
//   * four producer warps copy a tile of K (128 keys x 128 bytes) into shared
//     memory with 16-byte cp.async, writing the 128-byte-swizzled K-major layout
//     the tensor core reads (16-byte chunk c of key r goes to chunk c ^ (r & 7));
//     rows past the row's length are zero-filled, nothing outside K is read;
//   * one thread issues four tcgen05.mma (kind::f8f6f4, M = 128 keys, N = 64
//     heads, K = 32 per instruction) per tile into one of two accumulator
//     buffers in tensor memory (128 lanes x 64 fp32 columns each);
//   * four epilogue warps read their 32 lanes (one key per thread, its 64 head
//     dot products) with tcgen05.ld, apply relu, weight and sum over the heads with
//     fused multiply-adds (four interleaved partial sums), and store one score per key.
// Stages are handed over with mbarriers; every wait is bounded and sets a status
// bit instead of spinning for ever.
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdio>
#include <mutex>

#include "../../include/ff_indexer_logits.h"

namespace ffl {

constexpr int kHeads = 64;
constexpr int kDim = 128;          // bytes per key and per head (fp8)
constexpr int kTileKeys = 128;
constexpr int kStages = 6;         // K tiles in flight
constexpr int kTileBytes = kTileKeys * kDim;   // 16 KiB
constexpr int kQBytes = kHeads * kDim;         // 8 KiB
constexpr int kEpilogueWarps = 4;
constexpr int kMmaWarp = 4;
constexpr int kProducerWarp0 = 5;
constexpr int kProducerWarps = 4;
constexpr int kProducerThreads = kProducerWarps * 32;
constexpr int kThreads = (kProducerWarp0 + kProducerWarps) * 32;   // 288
constexpr int kTmemCols = 128;     // two accumulator buffers of 64 columns
constexpr int kWaitLimit = 1 << 20;   // polls of one bounded wait; the first wait that runs out ends all others early

// shared memory: [q 8 KiB][kStages x 16 KiB K tiles], 1024-byte aligned (swizzle atom)
constexpr int kSmemQ = 0;
constexpr int kSmemK = kQBytes;
constexpr int kSmemBytes = kQBytes + kStages * kTileBytes + 1024;   // + alignment slack

struct Params {
  const uint8_t* q;       // [B, 64, 128] e4m3
  const uint8_t* k;       // [B, k_row_stride] bytes, key j of row b at k + b * k_row_stride + j * 128
  int64_t k_row_stride;   // bytes
  const float* w;         // [B, 64]
  const int32_t* lengths; // [B]
  float* scores;          // [B, score_stride]
  int64_t score_stride;   // elements
  int32_t L_width;
  int32_t tiles_per_cta;  // target share of a CTA, in 128-key tiles
  int32_t* status;
  const float* hint;      // [B] threshold guesses or null: scores not below hint[b] also go to the hand-over list
  unsigned char* handover;   // per row FF_HANDOVER_ROW_BYTES: {count, readers, pad, uint64 entries[4096]}
};

constexpr int kHandoverCap = 4096;       // entries per row (the select's survivor capacity)
constexpr int kHandoverWarpBuf = 64;     // composites an epilogue warp collects in one of its two buffers

// Order-preserving fp32 -> uint32 map, the same as the select's (-0.0 == +0.0, NaN on top).
__device__ __forceinline__ uint32_t monotone_key(float x) {
  uint32_t u = __float_as_uint(x);
  const uint32_t a = u & 0x7fffffffu;
  if (a == 0u) u = 0u;
  uint32_t k = u ^ (static_cast<uint32_t>(static_cast<int32_t>(u) >> 31) | 0x80000000u);
  if (a > 0x7f800000u) k = 0xffffffffu;
  return k;
}

// An epilogue warp moves collected composites into the row's hand-over list at the slots it
// reserved (two stores per lane); what does not fit the list is dropped (the count tells the select).
__device__ __forceinline__ void store_handover(unsigned char* row_base, const unsigned long long* buf, int n,
                                               uint32_t base, int lane) {
  unsigned long long* list = reinterpret_cast<unsigned long long*>(row_base + 64);
  for (int i = lane; i < n; i += 32)
    if (base + i < static_cast<uint32_t>(kHandoverCap)) list[base + i] = buf[i];
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Bounded wait: gives up after kWaitLimit polls, or as soon as another wait of this CTA has
// given up (*gave_up != 0), and then records that itself.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* gave_up) {
  for (int i = 0; i < kWaitLimit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
    if ((i & 255) == 255 && *gave_up != 0) break;
  }
  *gave_up = 1;
  return false;
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done != 0;
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void fence_async_proxy() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Copies `rows` (a multiple of kProducerThreads / 8) rows of 128 bytes from global memory into the
// 128-byte-swizzled layout at `dst` with all producer threads: thread pt takes chunk pt & 7 of
// rows (pt >> 3) + (kProducerThreads / 8) * j.  The row step is a multiple of 8, so the swizzle term
// (row & 7) is the same for all of a thread's rows and both addresses advance by a constant.
// Rows at or beyond rows_valid are zero-filled and not read.
template <int kRows>
__device__ __forceinline__ void copy_rows_swizzled(uint32_t dst, const uint8_t* src, int pt, int rows_valid) {
  constexpr int kRowStep = kProducerThreads / 8;
  static_assert(kRowStep % 8 == 0 && kRows % kRowStep == 0, "producer thread count must keep (row & 7) fixed per thread");
  const int r0 = pt >> 3, ch = pt & 7;
  const uint32_t d0 = dst + r0 * kDim + ((ch ^ (r0 & 7)) << 4);
  const uint8_t* s0 = src + r0 * kDim + ch * 16;
  if (rows_valid >= kRows) {
#pragma unroll
    for (int j = 0; j < kRows / kRowStep; ++j) cp_async_16(d0 + j * kRowStep * kDim, s0 + j * kRowStep * kDim, 16u);
  } else {
#pragma unroll
    for (int j = 0; j < kRows / kRowStep; ++j) {
      const bool valid = r0 + j * kRowStep < rows_valid;
      cp_async_16(d0 + j * kRowStep * kDim, valid ? s0 + j * kRowStep * kDim : src, valid ? 16u : 0u);
    }
  }
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows at a
// 128-byte pitch, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr & 0x3ffffu) >> 4);    // start address, bits [0,14)
  d |= static_cast<uint64_t>(1) << 16;                    // leading byte offset (unused with one swizzle atom along K)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;            // stride byte offset: 8 rows x 128 bytes
  d |= static_cast<uint64_t>(1) << 46;                    // descriptor version for this architecture
  d |= static_cast<uint64_t>(2) << 61;                    // layout type: 128-byte swizzle
  return d;
}
// Instruction descriptor: e4m3 x e4m3 -> f32, both operands K-major, M = 128, N = 64.
constexpr uint32_t kInstrDesc = (1u << 4) | (0u << 7) | (0u << 10) | (0u << 15) | (0u << 16) |
                                (static_cast<uint32_t>(kHeads >> 3) << 17) | (static_cast<uint32_t>(kTileKeys >> 4) << 24);

__device__ __forceinline__ void mma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(kInstrDesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 consecutive fp32 columns of this thread's lane (issue only: tmem_ld_wait() before use).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// One key's score from its 64 head dot products (this thread's tensor-memory lane):
// relu, weight, and four interleaved partial sums (head h goes to sum h & 3) combined as
// (s0 + s1) + (s2 + s3): four short dependent chains instead of one of 64.  The checker
// (oracle/oracle_topk.c) sums in the same order.
__device__ __forceinline__ float score_of_lane(uint32_t taddr, const float* w) {
  float lo[32], hi[32];
  tmem_ld32(taddr, lo);
  tmem_ld32(taddr + 32, hi);
  tmem_ld_wait();
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int h = 0; h < 32; ++h) acc[h & 3] = fmaf(w[h], fmaxf(lo[h], 0.f), acc[h & 3]);
#pragma unroll
  for (int h = 0; h < 32; ++h) acc[h & 3] = fmaf(w[32 + h], fmaxf(hi[h], 0.f), acc[h & 3]);
  return (acc[0] + acc[1]) + (acc[2] + acc[3]);
}

struct Shared {
  unsigned long long full[kStages];    // K tile landed (producer threads arrive)
  unsigned long long empty[kStages];   // K tile consumed (tcgen05.commit arrives)
  unsigned long long qfull;            // q landed
  unsigned long long tfull[2];         // accumulator buffer complete (tcgen05.commit arrives)
  unsigned long long tempty[2];        // accumulator buffer read out (epilogue threads arrive)
  uint32_t tmem_base;
  int timed_out;
  float w[kHeads];
  unsigned long long handover[kEpilogueWarps][2][kHandoverWarpBuf];   // per epilogue warp: survivors not yet in the list
};

__global__ void __launch_bounds__(kThreads, 2) indexer_logits_kernel(const Params p) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ Shared sh;
  // A kernel launched behind this one with programmatic stream serialization (the select does that
  // on request) may be set up while this one runs; it waits for this grid's completion by itself.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;   // swizzle atoms need 1024-byte alignment
  const uint32_t q_s = smem_base + kSmemQ;
  const uint32_t k_s = smem_base + kSmemK;
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int row = blockIdx.y;
  int len = p.lengths[row];
  if (len > p.L_width) len = p.L_width;
  if (len < 0) len = 0;
  const int n_tiles_row = (len + kTileKeys - 1) / kTileKeys;
  // Ragged batches: a row uses as many of the grid's CTAs as give each about p.tiles_per_cta
  // tiles (the lengths live on the device, so the grid is sized for the longest possible row
  // and the CTAs a short row does not need leave at once).  CTA x of the n_ctas works on tiles
  // x, x + n_ctas, ...
  int n_ctas = (n_tiles_row + p.tiles_per_cta - 1) / p.tiles_per_cta;
  if (n_ctas > static_cast<int>(gridDim.x)) n_ctas = static_cast<int>(gridDim.x);
  const int cta = static_cast<int>(blockIdx.x);
  const int my_tiles = cta < n_ctas ? (n_tiles_row - cta + n_ctas - 1) / n_ctas : 0;
  if (my_tiles == 0) return;   // uniform over the CTA, before any barrier or allocation

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&sh.full[s]), kProducerThreads);
      mbar_init(smem_u32(&sh.empty[s]), 1);
    }
    mbar_init(smem_u32(&sh.qfull), kProducerThreads);
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&sh.tfull[b]), 1);
      mbar_init(smem_u32(&sh.tempty[b]), kEpilogueWarps * 32);
    }
    sh.timed_out = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (tid < kHeads) sh.w[tid] = p.w[static_cast<int64_t>(row) * kHeads + tid];
  if (warp == kMmaWarp) {   // one warp allocates the tensor memory columns
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh.tmem_base)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh.tmem_base;

  if (warp >= kProducerWarp0) {
    // ---------------- producers ----------------
    const int pt = tid - kProducerWarp0 * 32;
    const uint8_t* qrow = p.q + static_cast<int64_t>(row) * kQBytes;
    copy_rows_swizzled<kHeads>(q_s, qrow, pt, kHeads);
    cp_async_commit();
    cp_async_wait<0>();
    fence_async_proxy();
    mbar_arrive(smem_u32(&sh.qfull));
    const uint8_t* krow = p.k + static_cast<int64_t>(row) * p.k_row_stride;
    // tile i of this CTA goes to stage i % kStages; its copies are waited for kStages - 1 tiles later
    for (int i = 0; i < my_tiles + kStages - 1; ++i) {
      if (i < my_tiles) {
        const int stage = i % kStages;
        if (i >= kStages) {   // the stage's previous tile must have been consumed
          (void)mbar_wait(smem_u32(&sh.empty[stage]), static_cast<uint32_t>((i / kStages - 1) & 1), &sh.timed_out);
        }
        const int key0 = (cta + i * n_ctas) * kTileKeys;
        copy_rows_swizzled<kTileKeys>(k_s + stage * kTileBytes, krow + static_cast<int64_t>(key0) * kDim, pt,
                                      len - key0);   // zero-fill past the end
      }
      cp_async_commit();   // an empty group keeps the group count in step with i
      const int done = i - (kStages - 1);
      if (done >= 0) {
        cp_async_wait<kStages - 1>();   // tile `done` of this thread has landed
        fence_async_proxy();
        mbar_arrive(smem_u32(&sh.full[done % kStages]));
      }
    }
  } else if (warp == kMmaWarp) {
    // ---------------- tensor-core issue (one thread) ----------------
    if (lane == 0) {
      (void)mbar_wait(smem_u32(&sh.qfull), 0u, &sh.timed_out);
      for (int i = 0; i < my_tiles; ++i) {
        const int stage = i % kStages;
        const int buf = i & 1;
        if (i >= 2) {   // the accumulator buffer's previous tile must have been read out
          (void)mbar_wait(smem_u32(&sh.tempty[buf]), static_cast<uint32_t>((i / 2 - 1) & 1), &sh.timed_out);
        }
        (void)mbar_wait(smem_u32(&sh.full[stage]), static_cast<uint32_t>((i / kStages) & 1), &sh.timed_out);
        tc_fence_after();
        const uint32_t a_addr = k_s + stage * kTileBytes;
#pragma unroll
        for (int ks = 0; ks < kDim / 32; ++ks) {   // 32 bytes of K per instruction, inside the swizzle atom
          mma_f8(tmem + buf * kHeads, smem_desc(a_addr + ks * 32), smem_desc(q_s + ks * 32), ks > 0 ? 1u : 0u);
        }
        mma_commit(smem_u32(&sh.empty[stage]));   // the K tile may be overwritten once these MMAs are done
        mma_commit(smem_u32(&sh.tfull[buf]));     // ... and the accumulator is complete
      }
    }
  } else {
    // ---------------- epilogue: thread = key (tensor memory lane) ----------------
    const int key_in_tile = warp * 32 + lane;
    float* out_row = p.scores + static_cast<int64_t>(row) * p.score_stride;
    // hand-over to the select: scores not below the row's threshold guess are collected per warp
    float hint = __uint_as_float(0x7fffffffu);   // NaN: no guess, nothing is handed over
    if (p.hint != nullptr && p.handover != nullptr) hint = p.hint[row];
    const bool hand_over = hint == hint;
    unsigned char* row_base = p.handover + static_cast<int64_t>(row) * FF_HANDOVER_ROW_BYTES;
    // Two buffers per warp.  When the one being filled may not hold another tile's hits, lane 0
    // reserves list slots for it with one global atomic and the warp switches to the other buffer;
    // the reserved position is looked at a tile later, when the full buffer is stored, so the
    // atomic's round trip overlaps the next tile instead of stalling the epilogue (the accumulator
    // buffers give the epilogue only one tile of slack).
    int cur = 0, n_cur = 0;          // uniform over the warp
    int n_pending = 0;               // entries of the other buffer whose slots are reserved but not stored
    uint32_t pending_base = 0u;      // lane 0: result of that reservation
    for (int i = 0; i < my_tiles; ++i) {
      const int buf = i & 1;
      (void)mbar_wait(smem_u32(&sh.tfull[buf]), static_cast<uint32_t>((i / 2) & 1), &sh.timed_out);
      tc_fence_after();
      const uint32_t taddr = tmem + (static_cast<uint32_t>(warp * 32) << 16) + buf * kHeads;
      const float s = score_of_lane(taddr, sh.w);
      tc_fence_before();
      mbar_arrive(smem_u32(&sh.tempty[buf]));
      const int key = (cta + i * n_ctas) * kTileKeys + key_in_tile;
      if (key < p.L_width) out_row[key] = key < len ? s : __uint_as_float(0xff800000u);
      if (hand_over) {
        if (n_pending > 0) {   // last tile's reservation has long arrived
          store_handover(row_base, sh.handover[warp][cur ^ 1], n_pending, __shfl_sync(0xffffffffu, pending_base, 0), lane);
          n_pending = 0;
        }
        const bool hit = key < len && !(s < hint);
        const uint32_t votes = __ballot_sync(0xffffffffu, hit);
        if (votes != 0u) {
          if (hit)
            sh.handover[warp][cur][n_cur + __popc(votes & ((1u << lane) - 1u))] =
                (static_cast<unsigned long long>(monotone_key(s)) << 32) | static_cast<uint32_t>(~static_cast<uint32_t>(key));
          n_cur += __popc(votes);
          if (n_cur > kHandoverWarpBuf - 32) {   // the next tile might not fit: reserve list slots, switch buffers
            __syncwarp();
            if (lane == 0) pending_base = atomicAdd(reinterpret_cast<uint32_t*>(row_base), static_cast<uint32_t>(n_cur));
            n_pending = n_cur;
            cur ^= 1;
            n_cur = 0;
          }
        }
      }
    }
    if (hand_over) {
      __syncwarp();
      if (n_pending > 0)
        store_handover(row_base, sh.handover[warp][cur ^ 1], n_pending, __shfl_sync(0xffffffffu, pending_base, 0), lane);
      if (n_cur > 0) {
        uint32_t base = 0u;
        if (lane == 0) base = atomicAdd(reinterpret_cast<uint32_t*>(row_base), static_cast<uint32_t>(n_cur));
        store_handover(row_base, sh.handover[warp][cur], n_cur, __shfl_sync(0xffffffffu, base, 0), lane);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
  if (tid == 0 && sh.timed_out && p.status != nullptr) atomicOr(p.status, 2);
}


// ---- persistent variant ---------------------------------------------------------
// The grid is two CTAs per SM whatever the batch; the work is cut into units of
// kUnitTiles consecutive 128-key tiles of one row, numbered row by row (a prefix sum
// over the rows' unit counts, computed by every CTA from the device-side lengths), and
// CTA c takes units c, c + grid, c + 2 grid, ...  Barriers, tensor memory and the
// pipeline state are set up once per CTA and run on across units; q is double buffered
// (the next unit's q lands while the current unit's tiles are multiplied).
constexpr int kUnitTiles = 8;
constexpr int kPStages = 5;
constexpr int kMaxRowsPersistent = 1024;
constexpr int kPSmemQ = 0;                       // two q buffers
constexpr int kPSmemK = 2 * kQBytes;
constexpr int kPSmemBytes = 2 * kQBytes + kPStages * kTileBytes + 1024;

struct PShared {
  unsigned long long full[kPStages];
  unsigned long long empty[kPStages];
  unsigned long long qfull[2];
  unsigned long long qempty[2];
  unsigned long long tfull[2];
  unsigned long long tempty[2];
  uint32_t tmem_base;
  int timed_out;
  float w[kHeads];                       // head weights of the unit the epilogue is working on
  int prefix[kMaxRowsPersistent + 1];    // units before row b
};

// One unit of work and the position inside it; every role walks the same sequence.
struct UnitCursor {
  int u;        // unit number (global), advanced by the grid size
  int n;        // how many units this CTA has started before this one
  int row, len, tile0, ntile;
  int i;        // tile inside the unit
  int t;        // tiles this CTA has passed before this one (drives stages and phases)
};

__device__ __forceinline__ int clamp_len(const Params& p, int row) {
  int len = p.lengths[row];
  if (len > p.L_width) len = p.L_width;
  return len < 0 ? 0 : len;
}

__device__ __forceinline__ void cursor_load_unit(UnitCursor& c, const Params& p, const int* prefix, int B) {
  int lo = 0, hi = B;   // last row with prefix[row] <= u
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (prefix[mid] <= c.u) lo = mid; else hi = mid;
  }
  c.row = lo;
  c.len = clamp_len(p, lo);
  const int tiles_row = (c.len + kTileKeys - 1) / kTileKeys;
  c.tile0 = (c.u - prefix[lo]) * kUnitTiles;
  c.ntile = min(kUnitTiles, tiles_row - c.tile0);
  c.i = 0;
}
// Moves to the next tile; returns false when the CTA's units are used up.
__device__ __forceinline__ bool cursor_next(UnitCursor& c, const Params& p, const int* prefix, int B, int total_units,
                                            int stride) {
  c.t += 1;
  c.i += 1;
  if (c.i < c.ntile) return true;
  c.u += stride;
  c.n += 1;
  if (c.u >= total_units) return false;
  cursor_load_unit(c, p, prefix, B);
  return true;
}

__global__ void __launch_bounds__(kThreads, 2) indexer_logits_persistent_kernel(const Params p, const int B) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ PShared sh;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_s = smem_base + kPSmemQ;
  const uint32_t k_s = smem_base + kPSmemK;
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  // units per row -> exclusive prefix (one warp: each lane sums a contiguous run of rows)
  for (int b = tid; b < B; b += kThreads) {
    const int tiles = (clamp_len(p, b) + kTileKeys - 1) / kTileKeys;
    sh.prefix[b + 1] = (tiles + kUnitTiles - 1) / kUnitTiles;
  }
  if (tid == 0) {
    sh.prefix[0] = 0;
    for (int s = 0; s < kPStages; ++s) {
      mbar_init(smem_u32(&sh.full[s]), kProducerThreads);
      mbar_init(smem_u32(&sh.empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&sh.qfull[b]), kProducerThreads);
      mbar_init(smem_u32(&sh.qempty[b]), 1);
      mbar_init(smem_u32(&sh.tfull[b]), 1);
      mbar_init(smem_u32(&sh.tempty[b]), kEpilogueWarps * 32);
    }
    sh.timed_out = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (warp == 0) {
    const int per = (B + 31) / 32;
    const int b0 = lane * per;
    int sum = 0;
    for (int j = 0; j < per; ++j)
      if (b0 + j < B) sum += sh.prefix[b0 + j + 1];
    int incl = sum;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += v;
    }
    int running = incl - sum;
    for (int j = 0; j < per; ++j) {
      if (b0 + j < B) {
        running += sh.prefix[b0 + j + 1];
        sh.prefix[b0 + j + 1] = running;
      }
    }
  }
  __syncthreads();
  const int total_units = sh.prefix[B];
  const int stride = static_cast<int>(gridDim.x);
  if (static_cast<int>(blockIdx.x) >= total_units) return;   // uniform, before the allocation

  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh.tmem_base)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh.tmem_base;

  UnitCursor c;
  c.u = static_cast<int>(blockIdx.x);
  c.n = 0;
  c.t = 0;
  cursor_load_unit(c, p, sh.prefix, B);

  if (warp >= kProducerWarp0) {
    // ---------------- producers ----------------
    const int pt = tid - kProducerWarp0 * 32;
    // Every tile is one copy group.  A tile is announced (its "full" barrier, and with a unit's
    // first tile the unit's q) once its group has landed: normally when kPStages tiles are
    // outstanding, the oldest is waited for; at the end, and before a wait that the tensor-core
    // thread can only satisfy after seeing tiles still unannounced, everything outstanding is.
    UnitCursor d = c;          // the next tile to announce
    bool more = true;          // c points at a tile to issue
    int lag = 0;               // tiles issued and not yet announced
    auto announce_one = [&]() {
      if (d.i == 0) mbar_arrive(smem_u32(&sh.qfull[d.n & 1]));
      mbar_arrive(smem_u32(&sh.full[d.t % kPStages]));
      lag -= 1;
      (void)cursor_next(d, p, sh.prefix, B, total_units, stride);
    };
    auto announce_all = [&]() {
      cp_async_wait<0>();
      fence_async_proxy();
      while (lag > 0) announce_one();
    };
    while (more) {
      const int stage = c.t % kPStages;
      if (c.t >= kPStages)
        (void)mbar_wait(smem_u32(&sh.empty[stage]), static_cast<uint32_t>((c.t / kPStages - 1) & 1), &sh.timed_out);
      if (c.i == 0) {   // first tile of a unit: its q goes into the same copy group
        const int qb = c.n & 1;
        if (c.n >= 2) {
          // The buffer's previous unit (n - 2) must be multiplied.  After a short unit n - 1 some of
          // its tiles may still be unannounced: announce them before waiting.
          const uint32_t bar = smem_u32(&sh.qempty[qb]);
          const uint32_t parity = static_cast<uint32_t>((c.n / 2 - 1) & 1);
          if (!mbar_test(bar, parity)) {
            announce_all();
            (void)mbar_wait(bar, parity, &sh.timed_out);
          }
        }
        const uint8_t* qrow = p.q + static_cast<int64_t>(c.row) * kQBytes;
        copy_rows_swizzled<kHeads>(q_s + qb * kQBytes, qrow, pt, kHeads);
      }
      const uint8_t* krow = p.k + static_cast<int64_t>(c.row) * p.k_row_stride;
      const int key0 = (c.tile0 + c.i) * kTileKeys;
      copy_rows_swizzled<kTileKeys>(k_s + stage * kTileBytes, krow + static_cast<int64_t>(key0) * kDim, pt,
                                    c.len - key0);
      cp_async_commit();
      lag += 1;
      more = cursor_next(c, p, sh.prefix, B, total_units, stride);
      if (lag == kPStages) {
        cp_async_wait<kPStages - 1>();   // the oldest of the kPStages outstanding groups has landed
        fence_async_proxy();
        announce_one();
      }
    }
    announce_all();
  } else if (warp == kMmaWarp) {
    // ---------------- tensor-core issue (one thread) ----------------
    if (lane == 0) {
      bool more = true;
      while (more) {
        const int stage = c.t % kPStages;
        const int buf = c.t & 1;
        const int qb = c.n & 1;
        if (c.i == 0) (void)mbar_wait(smem_u32(&sh.qfull[qb]), static_cast<uint32_t>((c.n / 2) & 1), &sh.timed_out);
        if (c.t >= 2) (void)mbar_wait(smem_u32(&sh.tempty[buf]), static_cast<uint32_t>((c.t / 2 - 1) & 1), &sh.timed_out);
        (void)mbar_wait(smem_u32(&sh.full[stage]), static_cast<uint32_t>((c.t / kPStages) & 1), &sh.timed_out);
        tc_fence_after();
        const uint32_t a_addr = k_s + stage * kTileBytes;
        const uint32_t b_addr = q_s + qb * kQBytes;
#pragma unroll
        for (int ks = 0; ks < kDim / 32; ++ks)
          mma_f8(tmem + buf * kHeads, smem_desc(a_addr + ks * 32), smem_desc(b_addr + ks * 32), ks > 0 ? 1u : 0u);
        mma_commit(smem_u32(&sh.empty[stage]));
        mma_commit(smem_u32(&sh.tfull[buf]));
        if (c.i == c.ntile - 1) mma_commit(smem_u32(&sh.qempty[qb]));   // the unit's q buffer is free after these MMAs
        more = cursor_next(c, p, sh.prefix, B, total_units, stride);
      }
    }
  } else {
    // ---------------- epilogue: thread = key (tensor memory lane) ----------------
    const int key_in_tile = warp * 32 + lane;
    float w_next = p.w[static_cast<int64_t>(c.row) * kHeads + (tid & (kHeads - 1))];
    bool more = true;
    while (more) {
      if (c.i == 0) {
        // hand the head weights of this unit's row to all epilogue threads; the next unit's are fetched early
        asm volatile("bar.sync 1, 128;" ::: "memory");   // everyone is done with the previous unit's weights
        if (tid < kHeads) sh.w[tid] = w_next;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const int u_next = c.u + stride;
        if (u_next < total_units) {
          UnitCursor peek = c;
          peek.u = u_next;
          cursor_load_unit(peek, p, sh.prefix, B);
          w_next = p.w[static_cast<int64_t>(peek.row) * kHeads + (tid & (kHeads - 1))];
        }
      }
      const int buf = c.t & 1;
      (void)mbar_wait(smem_u32(&sh.tfull[buf]), static_cast<uint32_t>((c.t / 2) & 1), &sh.timed_out);
      tc_fence_after();
      const uint32_t taddr = tmem + (static_cast<uint32_t>(warp * 32) << 16) + buf * kHeads;
      const float s = score_of_lane(taddr, sh.w);
      tc_fence_before();
      mbar_arrive(smem_u32(&sh.tempty[buf]));
      const int key = (c.tile0 + c.i) * kTileKeys + key_in_tile;
      if (key < p.L_width)
        p.scores[static_cast<int64_t>(c.row) * p.score_stride + key] = key < c.len ? s : __uint_as_float(0xff800000u);
      more = cursor_next(c, p, sh.prefix, B, total_units, stride);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
  if (tid == 0 && sh.timed_out && p.status != nullptr) atomicOr(p.status, 2);
}

}  // namespace ffl

namespace {
thread_local char g_err[256] = "";
int fail(int code, const char* msg) {
  snprintf(g_err, sizeof(g_err), "%s", msg);
  return code;
}
int fail_cuda(cudaError_t e, const char* where) {
  snprintf(g_err, sizeof(g_err), "%s: %s", where, cudaGetErrorString(e));
  return static_cast<int>(e);
}
constexpr int kMaxDevices = 64;
std::once_flag g_once[kMaxDevices];
int g_rc[kMaxDevices];
std::atomic<int64_t> g_launches{0};
void init_device(int device) {
  cudaError_t e = cudaFuncSetAttribute(ffl::indexer_logits_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       ffl::kSmemBytes);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(ffl::indexer_logits_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             ffl::kPSmemBytes);
  g_rc[device] = static_cast<int>(e);
}
}  // namespace

extern "C" {

const char* ff_indexer_last_error_string(void) { return g_err; }
int64_t ff_indexer_launch_count(void) { return g_launches.load(); }

int ff_indexer_logits_launch(const void* q_e4m3, const void* k_e4m3, int64_t k_row_stride_bytes, const float* w,
                             const int32_t* lengths, float* scores, int64_t score_stride, int32_t B,
                             int32_t L_width, int32_t ctas_per_row, int32_t* status, void* stream) {
  return ff_indexer_logits_launch_handover(q_e4m3, k_e4m3, k_row_stride_bytes, w, lengths, scores, score_stride, B,
                                           L_width, ctas_per_row, nullptr, nullptr, status, stream);
}

int ff_indexer_logits_launch_handover(const void* q_e4m3, const void* k_e4m3, int64_t k_row_stride_bytes,
                                      const float* w, const int32_t* lengths, float* scores, int64_t score_stride,
                                      int32_t B, int32_t L_width, int32_t ctas_per_row, const float* hint,
                                      void* handover, int32_t* status, void* stream) {
  if (B < 0 || L_width < 0) return fail(-2, "negative B or L_width");
  if ((hint == nullptr) != (handover == nullptr)) return fail(-3, "hint and handover go together");
  if (handover != nullptr && ((reinterpret_cast<uintptr_t>(handover) & 63u) != 0 || ctas_per_row < 0))
    return fail(-2, "the hand-over list must be 64-byte aligned and needs the default kernel (ctas_per_row >= 0)");
  if (B == 0 || L_width == 0) return 0;
  if (q_e4m3 == nullptr || k_e4m3 == nullptr || w == nullptr || lengths == nullptr || scores == nullptr)
    return fail(-3, "q, k, w, lengths and scores must not be NULL");
  if ((reinterpret_cast<uintptr_t>(q_e4m3) & 15u) != 0 || (reinterpret_cast<uintptr_t>(k_e4m3) & 15u) != 0 ||
      (k_row_stride_bytes & 15) != 0)
    return fail(-2, "q, k and the K row stride must be 16-byte aligned");
  if (k_row_stride_bytes < static_cast<int64_t>(L_width) * ffl::kDim || score_stride < L_width)
    return fail(-2, "row strides are smaller than the row");
  if (B > 65535) return fail(-6, "B exceeds 65535 rows per launch");
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return fail_cuda(e, "cudaGetDevice");
  if (device < 0 || device >= kMaxDevices) return fail(-2, "device ordinal out of range");
  std::call_once(g_once[device], init_device, device);
  if (g_rc[device] != 0) return fail_cuda(static_cast<cudaError_t>(g_rc[device]), "cudaFuncSetAttribute");
  const int tiles = (L_width + ffl::kTileKeys - 1) / ffl::kTileKeys;
  ffl::Params p;
  p.q = static_cast<const uint8_t*>(q_e4m3);
  p.k = static_cast<const uint8_t*>(k_e4m3);
  p.k_row_stride = k_row_stride_bytes;
  p.w = w;
  p.lengths = lengths;
  p.scores = scores;
  p.score_stride = score_stride;
  p.L_width = L_width;
  p.tiles_per_cta = 0;
  p.status = status;
  p.hint = hint;
  p.handover = static_cast<unsigned char*>(handover);
  if (ctas_per_row < 0) {
    // The persistent kernel, two CTAs per SM, units of 8 tiles dealt out round robin.  Measured a few
    // per cent slower than shares of 32 tiles per CTA (below), which is therefore the default.
    if (B > ffl::kMaxRowsPersistent) return fail(-6, "the persistent kernel takes at most 1024 rows");
    int sms = 148;
    (void)cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const int64_t max_units = static_cast<int64_t>(B) * ((tiles + ffl::kUnitTiles - 1) / ffl::kUnitTiles);
    const int grid = static_cast<int>(max_units < 2 * sms ? max_units : 2 * sms);
    ffl::indexer_logits_persistent_kernel<<<grid, ffl::kThreads, ffl::kPSmemBytes, static_cast<cudaStream_t>(stream)>>>(p, B);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail_cuda(e, "indexer_logits_persistent_kernel");
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return 0;
  }
  // Default (ctas_per_row == 0): every row is cut into shares of about 32 tiles (512 KiB of K), but
  // into at least so many that the batch has about four CTAs per SM when every row is full, so that
  // small batches still fill the device.  ctas_per_row > 0 fixes the number of CTAs of a full row.
  int per_row = ctas_per_row;
  int tiles_per_cta = 32;
  if (per_row <= 0) {
    int sms = 148;
    (void)cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    const int want_ctas = (4 * sms + B - 1) / B;             // per row
    if (tiles_per_cta * want_ctas > tiles) tiles_per_cta = (tiles + want_ctas - 1) / want_ctas;
    if (tiles_per_cta < 1) tiles_per_cta = 1;
    per_row = (tiles + tiles_per_cta - 1) / tiles_per_cta;
  } else {
    tiles_per_cta = (tiles + per_row - 1) / per_row;
  }
  if (per_row > tiles) per_row = tiles;
  if (per_row < 1) per_row = 1;
  if (per_row > 65535) return fail(-6, "too many CTAs per row");
  p.tiles_per_cta = tiles_per_cta;
  ffl::indexer_logits_kernel<<<dim3(per_row, B, 1), ffl::kThreads, ffl::kSmemBytes, static_cast<cudaStream_t>(stream)>>>(p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail_cuda(e, "indexer_logits_kernel");
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return 0;
}

}  // extern "C"
