/*
 * Reference-side binding: the file a maintainer of the reference adds to its
 * CUDA build in place of ops/mask_builder.cu, next to dropping
 * ops/attn_core.cu's forward operator, when linking against libfblt_attn.so.
 * It is compiled against the reference's own headers (-I<reference>/csrc),
 * so blt_tensor / blt_arena / blt_mask_config are the reference's types, not
 * re-declarations.
 *
 *   blt_attention_head_core_cuda          exported by the library itself
 *   blt_build_attention_mask_cuda         below  (declared at core/backend.c:190)
 *   blt_build_block_diffusion_mask_cuda   below  (declared at core/backend.c:191-192)
 *
 * Both builders keep handing back a real [nq, nk] tensor allocated from the
 * caller's arena, with their temporaries from the same arena, as
 * ops/mask_builder.cu:100-216 does, and keep the reference's failure mode: a
 * query row without an allowed key, or a violated precondition, is fatal.
 */
#include <stdint.h>

#include "core/allocator.h"
#include "core/backend.h"
#include "ops/mask_builder.h"

#include "../../include/fblt_attn.h"

/* The library's structs mirror the reference's field for field; a mismatch must not compile. */
#define GLUE_SAME(a, b, f) _Static_assert(offsetof(a, f) == offsetof(b, f), "layout of " #a "." #f)
_Static_assert(sizeof(blt_mask_config) == sizeof(fblt_mask_config), "blt_mask_config size");
GLUE_SAME(blt_mask_config, fblt_mask_config, seq_len_q);
GLUE_SAME(blt_mask_config, fblt_mask_config, seq_len_kv);
GLUE_SAME(blt_mask_config, fblt_mask_config, sliding_window);
GLUE_SAME(blt_mask_config, fblt_mask_config, doc_boundaries);
GLUE_SAME(blt_mask_config, fblt_mask_config, num_docs);
GLUE_SAME(blt_mask_config, fblt_mask_config, query_group_ids);
GLUE_SAME(blt_mask_config, fblt_mask_config, kv_group_ids);
GLUE_SAME(blt_mask_config, fblt_mask_config, bidirectional_within_group);
GLUE_SAME(blt_mask_config, fblt_mask_config, is_causal);
GLUE_SAME(blt_mask_config, fblt_mask_config, causal_offset);
_Static_assert(sizeof(blt_block_diffusion_config) == sizeof(fblt_block_diffusion_config), "blt_block_diffusion_config size");
GLUE_SAME(blt_block_diffusion_config, fblt_block_diffusion_config, mode);
GLUE_SAME(blt_block_diffusion_config, fblt_block_diffusion_config, seq_len);
GLUE_SAME(blt_block_diffusion_config, fblt_block_diffusion_config, num_clean);
GLUE_SAME(blt_block_diffusion_config, fblt_block_diffusion_config, block_size);
GLUE_SAME(blt_block_diffusion_config, fblt_block_diffusion_config, block_starts);
GLUE_SAME(blt_block_diffusion_config, fblt_block_diffusion_config, num_blocks);
_Static_assert((int)BLT_BDM_TRAIN == (int)FBLT_BDM_TRAIN && (int)BLT_BDM_INFER == (int)FBLT_BDM_INFER, "mode values");
_Static_assert((int)BLT_BACKEND_CUDA == (int)FBLT_BACKEND_CUDA, "backend values");

void blt_build_attention_mask_cuda(const blt_mask_config *config, blt_tensor *out_mask, blt_arena *arena) {
    BLT_REQUIRE(config != NULL && out_mask != NULL && arena != NULL,
                "blt_build_attention_mask: config, out_mask and arena cannot be NULL");
    BLT_REQUIRE(arena->backend == BLT_BACKEND_CUDA, "blt_build_attention_mask: CUDA implementation called with non-CUDA arena");
    size_t shape[2] = {config->seq_len_q, config->seq_len_kv};
    *out_mask = blt_tensor_create_uninit(arena, shape, 2, BLT_DTYPE_FP32);
    const fblt_mask_config *c = (const fblt_mask_config *)config;
    const size_t need = fblt_mask_dense_scratch_bytes(c);
    void *scratch = blt_arena_alloc(arena, need, 16);
    int32_t empty = 0;
    const int st = fblt_build_attention_mask_dense(c, (float *)out_mask->data, scratch, need, &empty, NULL);
    if (st != FBLT_OK) BLT_FATAL("blt_build_attention_mask: %s", fblt_last_error());
    if (empty != 0) BLT_FATAL("blt_build_attention_mask: query position has no valid key");
}

void blt_build_block_diffusion_mask_cuda(const blt_block_diffusion_config *config, blt_tensor *out_mask,
                                         blt_arena *arena) {
    BLT_REQUIRE(config != NULL && out_mask != NULL && arena != NULL,
                "blt_build_block_diffusion_mask: config, out_mask and arena cannot be NULL");
    BLT_REQUIRE(arena->backend == BLT_BACKEND_CUDA,
                "blt_build_block_diffusion_mask: CUDA implementation called with non-CUDA arena");
    size_t shape[2] = {config->seq_len, config->seq_len};
    *out_mask = blt_tensor_create_uninit(arena, shape, 2, BLT_DTYPE_FP32);
    const fblt_block_diffusion_config *c = (const fblt_block_diffusion_config *)config;
    const size_t need = fblt_block_diffusion_mask_scratch_bytes(c);
    void *scratch = blt_arena_alloc(arena, need, 16);
    int32_t empty = 0;
    const int st = fblt_build_block_diffusion_mask_dense(c, (float *)out_mask->data, scratch, need, &empty, NULL);
    if (st != FBLT_OK) BLT_FATAL("blt_build_block_diffusion_mask: %s", fblt_last_error());
    if (empty != 0) BLT_FATAL("blt_build_block_diffusion_mask: query position has no valid key");
}
