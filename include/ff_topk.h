/*
 * ff_topk.h -- C ABI of the B200 (sm_100a) exact radix top-k indexer.
 *
 * Every entry point takes plain device pointers and sizes (no torch / DLPack
 * types) so it can be bound from ctypes, cgo, JNI or a TVM-FFI shim alike.
 * All launches are asynchronous on the caller's stream, never synchronise the
 * host, never allocate, and never read `lengths` on the host, so a call can be
 * captured into a CUDA graph.
 *
 * Selection rule (all entry points): row i is the window
 *   scores[i*row_stride + row_starts[i] ... + lengths[i])
 * and the result is the first k positions of that window under the total order
 * (value descending, index ascending); -0.0 == +0.0, NaN sorts above +inf.
 * Indices are window-relative int32.  When lengths[i] <= k the result is
 * 0,1,...,lengths[i]-1 followed by -1 (the reference's short-row behaviour,
 * jit_kernel/csrc/topk_indexer/topk_indexer_radix.cu:180-191).
 *
 * Return value: 0 on success, a negative FF_ERR_* for an argument error, a
 * positive cudaError_t for a CUDA runtime error.  ff_last_error_string()
 * describes the last non-zero return on the calling thread.
 */
#ifndef FF_TOPK_H_
#define FF_TOPK_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FF_OK 0
#define FF_ERR_BAD_K (-1)         /* k outside [1, FF_TOPK_MAX_K] */
#define FF_ERR_BAD_SHAPE (-2)     /* B < 0, L_width < 0, strides inconsistent */
#define FF_ERR_NULL (-3)          /* a required pointer is NULL */
#define FF_ERR_WORKSPACE (-4)     /* workspace too small or misaligned */
#define FF_ERR_BAD_CLUSTER (-5)   /* cluster-size override not in {0,1,2,4,8,16} */
#define FF_ERR_TOO_LARGE (-6)     /* size beyond a documented maximum */

#define FF_TOPK_MAX_K 2048

/* Device-side soft-error bits OR-ed into the optional `status` word. */
#define FF_STATUS_COUNT_MISMATCH 1 /* gathered survivors != histogram count   */
#define FF_STATUS_WAIT_TIMEOUT 2   /* a bounded cross-cluster wait ran out    */
#define FF_STATUS_NO_THRESHOLD 4   /* no threshold digit found (corrupt hist) */
#define FF_STATUS_HINT_MISSED 8    /* information, not an error: a threshold guess did not fit */
#define FF_STATUS_CP_SECOND_ROUND 16 /* information, not an error: a context-parallel step needed the ranks' whole
                                        candidate runs, not only their first part (winners crowded into few shards) */

#define FF_STATUS_CP_SX_FALLBACK 64 /* information, not an error: a context-parallel step's exchange of survivors
                                       did not apply (a rank without a guess, a crowded chunk, too few or too
                                       many survivors) and the step exchanged sorted runs instead */
#define FF_STATUS_BOUNDS 32 /* only in the build with -DFF_BOUNDS_CHECK: an index fell outside its work array (the access
                               was skipped; bits 8.. name the place); the result of that launch is not to be trusted */

/* Output epilogue applied to each selected window-relative index `p`
 * (reference: topk_indexer_radix.cu:1000-1124, the fused page-table
 * transforms). */
#define FF_EPILOGUE_INDEX 0       /* out = p                                  */
#define FF_EPILOGUE_PAGE_TABLE 1  /* out = table[table_row(i)*table_stride+p] */
#define FF_EPILOGUE_ADD_OFFSET 2  /* out = p + offsets[i]                     */

/* One-time per-device set-up: kernel attributes (dynamic shared memory,
 * non-portable 16-CTA clusters) and occupancy queries.  Idempotent and
 * thread-safe; ff_topk_launch calls it lazily for the current device.
 * Replaces the per-call cudaFuncSetAttribute of launch_topk_kernel
 * (topk_indexer_radix.cu:1195-1233). */
int ff_topk_init(int device);

/* Bytes of caller-owned scratch ff_topk_launch can use for (B, L_width, k).
 * The workspace must be 256-byte aligned, zero-filled once before first use
 * (the kernels leave it zeroed), and must not be shared by launches that can
 * overlap on the GPU.  Returns 0 when no scratch is used (short rows or large
 * batches).  Scratch is optional: without it (NULL / too small) long rows are
 * handled by one cluster instead of being split over several. */
size_t ff_topk_workspace_bytes(int32_t B, int64_t L_width, int32_t k);

/* The fast_topk_v3 hot path.  Replaces the TVM-FFI symbol `fast_topk`
 * (topk_indexer_radix.cu:1285-1387) and the pybind `fast_topk`
 * (topk_indexer_radix.cu:1391-1547).
 *   scores      [B, L_width] fp32, unit inner stride, row stride `row_stride` elements
 *   lengths     [B] int32
 *   row_starts  [B] int32 or NULL
 *   out_idx     [B, k] int32, contiguous; every slot is written
 *   status      optional device int32 (NULL to ignore); soft-error bits are OR-ed in
 *   stream      cudaStream_t
 */
int ff_topk_launch(const float* scores, int64_t row_stride, const int32_t* lengths,
                   const int32_t* row_starts, int32_t* out_idx, int32_t B, int64_t L_width,
                   int32_t k, void* workspace, size_t workspace_bytes, int32_t* status,
                   void* stream);

/* Same result as ff_topk_launch, for callers that cannot hand over scratch
 * memory.  (No counterpart in the reference.)  Some hosts of this library may
 * not allocate device memory at all: an operator plugged into a runtime that
 * owns every buffer and gives a plugin only its inputs and outputs, a serving
 * loop whose memory pool is frozen after warm-up, or code running where a
 * cudaMalloc would stall the whole device.  Without a workspace ff_topk_launch
 * still works but handles a long row with a single cluster; this entry point
 * keeps the fast path (a long row split over several clusters) by using scratch
 * built into the library: a zero-initialised __device__ array of
 * FF_TOPK_STATIC_MAX_ROWS * 263,680 bytes (about 1030 KiB) that every GPU
 * loading the library holds until the process exits.
 *   - B > FF_TOPK_STATIC_MAX_ROWS is rejected with FF_ERR_TOO_LARGE.
 *   - It calls no cudaMalloc / cudaFree and no allocating library routine; it
 *     enqueues one kernel on `stream`, preceded by one cudaMemsetAsync when the
 *     rows are long enough to use the scratch (the array keeps the previous
 *     call's contents and its counters must start at zero).
 *   - The first call on each device resolves the array's device address
 *     (cudaGetSymbolAddress, with that device current); make that first call
 *     before starting any stream capture.  Only a successful look-up is kept:
 *     if it fails, the call returns the error and the next call tries again.
 *   - All calls on one GPU share the one array: two calls that can overlap on
 *     the GPU (different streams) race on it and give wrong results. */
#define FF_TOPK_STATIC_MAX_ROWS 4
int ff_topk_launch_static(const float* scores, int64_t row_stride, const int32_t* lengths,
                          const int32_t* row_starts, int32_t* out_idx, int32_t B, int64_t L_width,
                          int32_t k, int32_t* status, void* stream);

/* ff_topk_launch_hinted for scores whose producer has already listed the survivors (no reference
 * counterpart; the "producer fused with the first pass" step, whose shape the reference's README
 * names, README.md:28).  `handover` is the buffer ff_indexer_logits_launch_handover
 * (include/ff_indexer_logits.h) filled in the launch before this one on the same stream, with the
 * guesses hint_in: per row FF_TOPK_HANDOVER_ROW_BYTES holding {uint32 count, uint32 readers, pad to
 * 64 bytes, uint64 composites[4096]} of every score not below hint_in[row].  A row whose count is
 * between k and 4096 is ranked from its list alone: no score is read.  Any other row (no guess, or a
 * guess that let through too few or too many: FF_STATUS_HINT_MISSED) is selected from `scores` as
 * by ff_topk_launch; the result is exact either way.  Every header that was read is left zeroed for
 * the producer's next launch; hint_out receives the next guesses (may alias hint_in). */
#define FF_TOPK_HANDOVER_ROW_BYTES (64 + 4096 * 8)
int ff_topk_launch_handover(const float* scores, int64_t row_stride, const int32_t* lengths,
                            const int32_t* row_starts, int32_t* out_idx, int32_t B, int64_t L_width, int32_t k,
                            const float* hint_in, float* hint_out, void* handover, void* workspace,
                            size_t workspace_bytes, int32_t* status, void* stream);

/* ff_topk_launch for other score and index types (no reference counterpart: the reference is fp32
 * with int32 indices only and leaves a half-precision value type commented out,
 * topk_indexer_radix.cu:563-564).  score_dtype says what `scores` points to; row_stride counts
 * elements of that type.  A 16-bit score is widened to fp32 exactly, so the result is the one
 * ff_topk_launch gives for the fp32 row with the same values, while half the bytes are read.
 * index_bits = 64 makes out_idx an int64_t [B, k] array (the layout torch.topk returns), else 32.
 * hint_in / hint_out as in ff_topk_launch_hinted (both may be NULL). */
#define FF_DTYPE_F32 0
#define FF_DTYPE_BF16 1
#define FF_DTYPE_F16 2
int ff_topk_launch_typed(const void* scores, int32_t score_dtype, int64_t row_stride, const int32_t* lengths,
                         const int32_t* row_starts, void* out_idx, int32_t index_bits, int32_t B, int64_t L_width,
                         int32_t k, const float* hint_in, float* hint_out, void* workspace, size_t workspace_bytes,
                         int32_t* status, void* stream);

/* ff_topk_launch with a threshold guess per row (no reference counterpart: the
 * reference only discusses reusing the previous decode step's threshold,
 * README.md:100-106).  hint_in[i] is a guess of a value between row i's k-th and
 * 4096-th largest score (NaN = no guess for that row; hint_in may be NULL).  With
 * a guess the row is swept ONCE: everything not below the guess is collected and,
 * if that is between k and 4096 elements, ranked directly: no histogram, no merge
 * of histograms, no second sweep.  If the guess does not fit, the row starts over
 * on the normal path and FF_STATUS_HINT_MISSED is OR-ed into `status`; the result
 * is exact and identical to ff_topk_launch's either way.  hint_out[i] (may be NULL,
 * may alias hint_in) receives a score of rank about 1.25 k of row i (NaN for rows with
 * no more than k positions): a good guess for the next call on similar data, e.g. the
 * next decode step of the same sequences.  Device pointers, float32 [B]. */
int ff_topk_launch_hinted(const float* scores, int64_t row_stride, const int32_t* lengths,
                          const int32_t* row_starts, int32_t* out_idx, int32_t B, int64_t L_width,
                          int32_t k, const float* hint_in, float* hint_out, void* workspace,
                          size_t workspace_bytes, int32_t* status, void* stream);

/* Fused top-k + page-table gather / ragged offset.  Replaces
 * fast_topk_transform_fused and fast_topk_transform_ragged_fused
 * (topk_indexer_radix.cu:1549-1639).
 *   epilogue = FF_EPILOGUE_PAGE_TABLE: `table` is [n_table_rows, table_stride]
 *     int32; row i uses table row i when cu_seqlens_q is NULL (decode), else the
 *     request r with cu_seqlens_q[r] <= i < cu_seqlens_q[r+1] (prefill).
 *   epilogue = FF_EPILOGUE_ADD_OFFSET: `offsets` is [B] int32.
 */
int ff_topk_transform_launch(const float* scores, int64_t row_stride, const int32_t* lengths,
                             const int32_t* row_starts, int32_t* out, int32_t B,
                             int64_t L_width, int32_t k, int32_t epilogue,
                             const int32_t* table, int64_t table_stride,
                             const int32_t* cu_seqlens_q, int32_t n_table_rows,
                             const int32_t* offsets, void* workspace, size_t workspace_bytes,
                             int32_t* status, void* stream);

/* Context-parallel mode, step 1 (no reference counterpart: the reference has
 * no multi-GPU path; semantics follow fast_topk_v3 on the unsharded row).
 * This rank holds columns [shard_offset, shard_offset + L_width) of every row.
 * `lengths` are the GLOBAL row lengths; the shard's valid length is
 * clamp(lengths[i] - shard_offset, 0, L_width).  Emits the shard's top-k as
 * (value, global index) pairs in canonical order; unused slots get
 * (-inf, -1). */
int ff_topk_cp_local(const float* scores, int64_t row_stride, const int32_t* lengths,
                     int32_t* cand_idx, float* cand_val, int32_t B, int64_t L_width,
                     int32_t k, int64_t shard_offset, void* workspace, size_t workspace_bytes,
                     int32_t* status, void* stream);

/* Context-parallel mode, step 2: exact merge-select of the all-gathered
 * candidates.  Rank p's block of row i is
 *   cand_val[p*rank_stride + i*k ... + k),  cand_idx likewise
 * (so both planes of an all-gathered [P][2][B][k] buffer can be passed with
 * rank_stride = 2*B*k); entries with index < 0 are ignored.  `lengths` are the
 * global row lengths (rows with lengths[i] <= k get the short-row identity
 * result).  out_idx is [B, k] global indices in canonical order. */
int ff_topk_cp_merge(const float* cand_val, const int32_t* cand_idx, int32_t n_ranks,
                     int64_t rank_stride, const int32_t* lengths, int32_t* out_idx, int32_t B,
                     int32_t k, void* workspace, size_t workspace_bytes, int32_t* status,
                     void* stream);

/* ---- Context-parallel mode with the exchange fused over peer memory --------
 * (No reference counterpart.)  Instead of a collective library call, each rank
 * stores its candidates straight into every peer's receive buffer over NVLink as
 * self-validating 16-byte entries {value bits, step, global index, step}; the merge polls its own (local)
 * entries until they carry the current step (bounded to one second,
 * FF_STATUS_WAIT_TIMEOUT on expiry).  No fence, flag or collective call.
 *
 *   ff_cp_exchange_create      allocates this rank's buffers (cudaMalloc) for a fixed (world, B, k)
 *   ff_cp_exchange_ipc_handle  64-byte cudaIpcMemHandle_t of that allocation, to be sent to the peers
 *   ff_cp_exchange_open_peers  maps the peers' allocations from `n` = world handles (rank-major, 64 B each)
 *   ff_cp_exchange_set_peer    in-process alternative: give peer p's base pointer directly
 *   ff_topk_cp_send            shard-local select whose epilogue stores into all peers (1 launch)
 *   ff_topk_cp_recv_merge      wait for all peers' entries of the current step + merge (1 launch)
 *   ff_topk_cp_step            the whole step as ONE launch (select, store to peers, poll, merge) when
 *                              all CTAs of the launch can be resident at once; else send + recv_merge.
 *                              With FF_TOPK_CP_SX=1 in the environment (off by default: it measured slower
 *                              than what follows) and without caller's guesses the one-launch form first
 *                              tries an exchange of SURVIVORS: every rank guesses, from its own shard, the score that about
 *                              1.25 k + 64 scores of the whole row reach, every CTA stores the few scores of
 *                              its chunk that reach it into a region of its own in every rank's buffer, and
 *                              every rank finishes the same list of survivors like a one-GPU row (no local
 *                              ranking, no run merge; exact: the list is checked to hold k entries not below
 *                              the largest of the ranks' guesses).  Where that does not apply
 *                              (FF_STATUS_CP_SX_FALLBACK) the step exchanges sorted runs:
 *                              In the one-launch form with more than two ranks a rank first sends only the
 *                              head of its run (2k/world candidates per row, at least 256; FF_TOPK_CP_PREFIX
 *                              overrides): the heads hold the row's whole top-k unless some head is used up
 *                              entirely, which every rank detects on the same data; then all ranks send the
 *                              rest and merge the whole runs (FF_STATUS_CP_SECOND_ROUND, exact either way)
 *   ff_topk_cp_send_hinted / ff_topk_cp_step_hinted
 *                              the same with threshold guesses for the shard-local select: hint_in /
 *                              hint_out are [B] floats of THIS rank's shard, with the meaning and the
 *                              miss behaviour (FF_STATUS_HINT_MISSED, result still exact) of
 *                              ff_topk_launch_hinted; either may be NULL
 * Every rank must call the step functions the same number of times in the same
 * order; a rank may run at most one step ahead of its peers (two alternating
 * receive buffers).  out_idx is [B, k] global indices, identical on all ranks. */
int ff_cp_exchange_create(int32_t world, int32_t rank, int32_t B, int32_t k, void** handle_out);
int64_t ff_cp_exchange_bytes(void* handle);
void* ff_cp_exchange_base(void* handle);
int ff_cp_exchange_ipc_handle(void* handle, void* out64);
int ff_cp_exchange_open_peers(void* handle, const void* handles, int32_t n);
int ff_cp_exchange_set_peer(void* handle, int32_t peer, void* peer_base);
int ff_cp_exchange_destroy(void* handle);
int ff_topk_cp_send(void* handle, const float* scores, int64_t row_stride, const int32_t* lengths,
                    int64_t L_width, int64_t shard_offset, void* workspace, size_t workspace_bytes,
                    int32_t* status, void* stream);
int ff_topk_cp_recv_merge(void* handle, const int32_t* lengths, int32_t* out_idx, int32_t* status,
                          void* stream);
int ff_topk_cp_step(void* handle, const float* scores, int64_t row_stride, const int32_t* lengths,
                    int32_t* out_idx, int64_t L_width, int64_t shard_offset, void* workspace,
                    size_t workspace_bytes, int32_t* status, void* stream);
int ff_topk_cp_send_hinted(void* handle, const float* scores, int64_t row_stride, const int32_t* lengths,
                           int64_t L_width, int64_t shard_offset, const float* hint_in, float* hint_out,
                           void* workspace, size_t workspace_bytes, int32_t* status, void* stream);
int ff_topk_cp_step_hinted(void* handle, const float* scores, int64_t row_stride, const int32_t* lengths,
                           int32_t* out_idx, int64_t L_width, int64_t shard_offset, const float* hint_in,
                           float* hint_out, void* workspace, size_t workspace_bytes, int32_t* status,
                           void* stream);

/* Test hook (no reference counterpart): n_ranks <= 8 ranks of a context-parallel step played by ONE
 * cooperative launch on the current GPU, for boxes with fewer GPUs than ranks (kernels that wait for
 * one another must not be separate launches on one device).  handles[r] is rank r's exchange (peers set
 * with ff_cp_exchange_set_peer), scores[r] / L_width[r] / shard_offset[r] its shard, out_idx[r] its
 * [B, k] result, hints[r] (array or entries may be NULL) its [B] threshold guesses, read and updated,
 * workspaces[r] its zero-filled scratch of workspace_bytes each (may be NULL).  All shards must get the
 * same launch shape.  Same kernel code and protocol as ff_topk_cp_step_hinted on real ranks. */
int ff_topk_cp_step_emulated_ranks(int32_t n_ranks, void* const* handles, const float* const* scores,
                                   int64_t row_stride, const int32_t* lengths, int32_t* const* out_idx,
                                   const int64_t* L_width, const int64_t* shard_offset, float* const* hints,
                                   void* const* workspaces, size_t workspace_bytes, int32_t* status, void* stream);

/* Test / tuning hook: force the thread-block-cluster size per row
 * (0 = automatic policy, else 1, 2, 4, 8 or 16).  Process-wide. */
int ff_topk_set_cluster_override(int32_t cluster_size);

/* Debug aid: when non-NULL, every CTA of every later launch writes its stage
 * time stamps (SM cycle counter) to device_buffer[cta * 40 + slot] (uint64).
 * The buffer must hold 40 words per CTA of the largest launch.  Process-wide;
 * pass NULL to switch tracing off.  Plays the role of the reference's
 * SMALL_K_PROFILE clock64 brackets (top_small_k.cuh:39-41,132-135). */
int ff_topk_set_trace_buffer(void* device_buffer);

/* Test / tuning hook: clusters per row (0 = automatic, 1 = never split a row,
 * 2..64 = split every row with enough workspace over that many clusters of the
 * current cluster size, clamped to what can be co-resident).  Process-wide. */
int ff_topk_set_groups_override(int32_t groups);

/* Rows that are split over several clusters and come without a threshold guess make their own
 * (every CTA estimates, from its own chunk, a score that about 1.25 k of the row's scores reach;
 * the mean of the estimates is tried like a caller's guess, with the same fall-back, so results
 * are exact either way).  It pays on rows whose parts look alike and costs a few microseconds on
 * rows with a strong trend along the row.  on = 0 switches it off, 1 on, -1 back to the default
 * (on, unless the environment holds FF_TOPK_SELF_SEED=0).  Process-wide.  No reference counterpart
 * (the reference finds its threshold from histograms only, topk_indexer_radix.cu:637-672). */
int ff_topk_set_self_seed(int32_t on);

/* Every select is launched with programmatic stream serialization: the hardware may set the launch
 * up while the kernel before it on the stream is still running, and the select waits for that
 * kernel's completion itself (griddepcontrol.wait is its first instruction, so it reads nothing
 * early); its own first instructions also let a launch behind it, if made the same way, be set up
 * early.  Back-to-back calls in a CUDA graph lose 0.2-0.6 us of launch latency each; results do not
 * change.  on = 0 switches it off (plain stream order), 1 on, -1 back to the default (on, unless
 * the environment holds FF_TOPK_PDL=0).  Process-wide.  No reference counterpart (the reference
 * launches with the cluster attribute only, topk_indexer_radix.cu:1195-1233). */
int ff_topk_set_programmatic_launch(int32_t on);

/* The cluster size the automatic policy picks for (B, L_width, k) on the
 * current device (after overrides) when a row stays inside ONE cluster (no
 * workspace).  For the shape of an actual launch use ff_topk_policy_launch_shape. */
int32_t ff_topk_policy_cluster_size(int32_t B, int64_t L_width, int32_t k);

/* The launch shape ff_topk_launch (hinted == 0) or ff_topk_launch_hinted
 * (hinted != 0) uses for (B, L_width, k) on the current device: out2[0] = CTAs
 * per cluster, out2[1] = clusters per row (more than one only with workspace of
 * ff_topk_workspace_bytes; pass has_workspace = 0 for a call without).  The
 * grid is B * out2[0] * out2[1] CTAs.  Plays the role of reading the reference's
 * split policy off its launcher (topk_indexer_radix.cu:1309-1321). */
int ff_topk_policy_launch_shape(int32_t B, int64_t L_width, int32_t k, int32_t has_workspace, int32_t hinted,
                                int32_t* out2);

/* Number of kernel launches issued through this library since load
 * (all threads); used by the benchmark's launch accounting. */
int64_t ff_topk_launch_count(void);

const char* ff_last_error_string(void);

/* Library ABI version; bumped when a signature changes. */
int32_t ff_topk_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* FF_TOPK_H_ */
