/* C ABI of the lightning-indexer logit producer for sm_100a (libff_indexer.so).
 *
 * No reference counterpart: the reference repository has no kernel for the step
 * that produces the scores its top-k indexer consumes; the operation and its
 * shapes are the ones its README names for the indexer (README.md:28) and the
 * ones the ragged decode benchmark configuration is generated with:
 *
 *     scores[b, j] = sum over h < 64 of  w[b, h] * relu( q[b, h, :] . k[b, j, :] )
 *
 * with head_dim 128, q and k in fp8 e4m3 (one byte per element), products and
 * sums in fp32; heads summed with fused multiply-adds into four interleaved partial sums
 * (head h into sum h & 3) that are combined as (s0 + s1) + (s2 + s3).
 * Positions j >= lengths[b] inside a processed 128-key tile receive -inf;
 * tiles that start at or beyond lengths[b] are left untouched.
 *
 * All pointers are device pointers; the call enqueues one kernel on `stream`,
 * never synchronises and allocates nothing.  Return value: 0 = ok, negative =
 * argument error, positive = cudaError_t.  `status` (optional device int32)
 * receives bit 2 if a bounded wait inside the kernel ran out.
 */
#ifndef FF_INDEXER_LOGITS_H_
#define FF_INDEXER_LOGITS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FF_INDEXER_HEADS 64
#define FF_INDEXER_HEAD_DIM 128

/* q_e4m3: [B, 64, 128] bytes, contiguous, 16-byte aligned.
 * k_e4m3: key j of row b at k_e4m3 + b * k_row_stride_bytes + j * 128 (16-byte aligned stride).
 * w: [B, 64] float32.  lengths: [B] int32.  scores: [B, score_stride] float32, score_stride >= L_width.
 * ctas_per_row: 0 = automatic (shares of about 32 tiles of 128 keys per CTA, sized from each row's
 * length on the device); > 0 = that many CTAs for a full row; < 0 = the persistent variant (two CTAs
 * per SM walk units of 8 tiles round robin; at most 1024 rows). */
int ff_indexer_logits_launch(const void* q_e4m3, const void* k_e4m3, int64_t k_row_stride_bytes,
                             const float* w, const int32_t* lengths, float* scores,
                             int64_t score_stride, int32_t B, int32_t L_width, int32_t ctas_per_row,
                             int32_t* status, void* stream);

/* The same launch, which also hands the top-k select its survivors (no reference counterpart).
 * hint: [B] float32 threshold guesses as ff_topk_launch_hinted carries them from step to step
 * (NaN = no guess for that row).  Every score of row b that is not below hint[b] is, besides being
 * written to `scores`, appended as a 64-bit composite (monotone key << 32 | ~index) to row b's
 * hand-over list: handover + b * FF_HANDOVER_ROW_BYTES holds {uint32 count, uint32 readers, pad to
 * 64 bytes, uint64 entries[4096]}; the count keeps counting past 4096, entries beyond are dropped.
 * The counts must be zero when the launch starts (the buffer is zero-filled once by the caller;
 * ff_topk_launch_handover leaves every count it has read at zero again).  With the list the select
 * reads no score at all when the guess fits; when it does not, it falls back to the scores.
 * Only the default kernel (ctas_per_row >= 0) takes a hand-over. */
#define FF_HANDOVER_ROW_BYTES (64 + 4096 * 8)
int ff_indexer_logits_launch_handover(const void* q_e4m3, const void* k_e4m3, int64_t k_row_stride_bytes,
                                      const float* w, const int32_t* lengths, float* scores,
                                      int64_t score_stride, int32_t B, int32_t L_width, int32_t ctas_per_row,
                                      const float* hint, void* handover, int32_t* status, void* stream);

int64_t ff_indexer_launch_count(void);
const char* ff_indexer_last_error_string(void);

#ifdef __cplusplus
}
#endif
#endif /* FF_INDEXER_LOGITS_H_ */
