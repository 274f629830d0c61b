/*
 * TEST INFRASTRUCTURE -- not part of the product.
 *
 * CPU restatement, in plain C, of the reference's attention path: the
 * single-head operator, the dense mask builders, the patch group-id helpers
 * and the host decision functions. Every function names the reference
 * file:line it follows. It exists so that the CUDA path can be checked on a
 * machine where the reference tree is not present; where the reference tree
 * is present, oracle/Makefile also compiles the reference's own object code
 * (oracle/_ref/libblt_ref.so) and the test-suite pins this restatement
 * against it bit for bit.
 *
 * Only tests, the smoke check and the benchmark's CPU-baseline leg may load
 * this library. Nothing under the package directory calls it.
 */
#ifndef FBLT_ATTN_ORACLE_H
#define FBLT_ATTN_ORACLE_H

#include <stddef.h>
#include <stdint.h>
#include "../include/fblt_attn.h"

/* ops/attn_core_cpu.c:16-57 with ops/vecmath_cpu.c:6-14 and :16-53. */
void oracle_attention_head(const fblt_head_args *a);

/*
 * Runs n independent head jobs on `nthreads` threads. The reference operator
 * is single-threaded; independent (sequence, head) units are spread over a
 * pool without touching the per-unit arithmetic. A job whose weights_out and
 * scores_scratch are both NULL gets a per-thread scratch. Returns seconds of
 * wall time spent inside the pool.
 */
double oracle_run_heads(const fblt_head_args *jobs, size_t n, int nthreads);

/* ops/mask_builder_cpu.c:21-95. Returns the number of query rows with no
 * allowed key (the reference aborts when that is non-zero). */
size_t oracle_build_mask(size_t nq, size_t nk, size_t window, const size_t *doc_boundaries, size_t num_docs,
                         const size_t *q_groups, const size_t *k_groups, int bidirectional, int is_causal,
                         size_t causal_offset, float *out);

/* ops/mask_builder_cpu.c:97-154. mode 0 = TRAIN, 1 = INFER. */
size_t oracle_block_diffusion_mask(int mode, size_t S, size_t N, size_t B, const size_t *block_starts,
                                   size_t num_blocks, float *out);

/* infer/kv_cache.c:225-236: rows of the incremental decoder's self mask. */
void oracle_decode_self_mask(size_t n, size_t base, size_t window, float *out);
/* infer/kv_cache.c:206-218 and :243-249: rows of its cross mask. */
void oracle_decode_cross_mask(const fblt_patch_info *patches, size_t num_patches, size_t k, size_t n, size_t base,
                              int trailing_closed, float *out);

/* ops/patch_pool_cpu.c:98-112. Returns 0, or 1 when the patches do not tile. */
int oracle_patch_group_ids(const fblt_patch_info *patches, size_t num_patches, size_t seq_len, size_t *q_groups,
                           size_t *k_groups);
/* ops/patch_pool_cpu.c:114-131. */
size_t oracle_decoder_latent_at(const fblt_patch_info *patches, size_t num_patches, size_t pos);
/* ops/patch_pool_cpu.c:133-142. */
void oracle_expand_group_ids(const size_t *in, size_t n, size_t k, size_t *out);

/* infer/self_speculation.c:21-31 (same rule as infer/block_generation.c:83-92). */
int32_t oracle_argmax_row(const float *row, size_t vocab);
/* infer/self_speculation.c:158-182: returns the new committed length. */
size_t oracle_verify_accept(uint8_t *x, const float *logits, size_t vocab, size_t l, size_t r, size_t target_len,
                            size_t *accepted);
/* infer/block_generation.c:65-81. */
void oracle_row_analyze(const float *row, size_t vocab, float *p_max, float *entropy);
/* infer/block_generation.c:20-31, :33-58, :139-152; infer/self_speculation.c:73-80. */
uint32_t oracle_unmask_select_confidence(const float *scores, const uint8_t *masked, size_t B, float alpha);
uint32_t oracle_unmask_select_eb(const float *scores, const uint8_t *masked, size_t B, float gamma);
size_t oracle_block_adapt_b(size_t cur_b, double rolling_acceptance, size_t b_min, size_t b_max, float target);
size_t oracle_aligned_commit_select(const fblt_patch_info *patches, size_t num_patches, size_t lo, size_t hi);

/* ops/reductions_cpu.c:179-197 and :199-233 (rotary tables and their application). */
void oracle_rope_precompute(size_t max_seq_len, float theta, size_t head_dim, float *cos_out, float *sin_out);
void oracle_rope_apply(const float *x, const float *cos_t, const float *sin_t, float *out, size_t rows, size_t heads,
                       size_t head_dim);

/* ops/linalg_cpu.c:8-18: out[m, n] = a[m, k] * b[k, n], one fp32 accumulator per output,
 * depth index ascending. */
void oracle_matmul(const float *a, const float *b, float *out, size_t m, size_t k, size_t n);

#endif
