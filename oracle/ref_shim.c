/*
 * TEST INFRASTRUCTURE -- not part of the product.
 *
 * Flat-argument entry points over the reference's own CPU object code, so
 * that ctypes can call it without re-declaring blt_tensor / blt_arena. This
 * file is compiled together with the reference's C sources (from where they
 * are mounted) into oracle/_ref/libblt_ref.so; it contains no arithmetic of
 * its own -- every result comes from a reference function.
 *
 * The reference aborts the process on a violated requirement (for example a
 * mask row with no allowed key); callers check such inputs with the
 * restatement first.
 */
#include <math.h>
#include <pthread.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include "core/allocator.h"
#include "core/backend.h"
#include "infer/block_generation.h"
#include "infer/kv_cache.h"
#include "infer/self_speculation.h"
#include "models/attention.h"
#include "models/cross_attention.h"
#include "models/patcher.h"
#include "ops/attn_core.h"
#include "ops/mask_builder.h"
#include "ops/matmul.h"
#include "ops/patch_pool.h"
#include "ops/rope.h"
#include "ops/row_stats.h"

void ref_attention_head(const blt_attention_head_args *a) { blt_attention_head_core(BLT_BACKEND_CPU, a); }

typedef struct {
    const blt_attention_head_args *jobs;
    size_t n;
    size_t *next;
    pthread_mutex_t *lock;
} ref_pool;

static void *ref_worker(void *p) {
    ref_pool *c = (ref_pool *)p;
    float *scratch = NULL;
    size_t cap = 0;
    for (;;) {
        pthread_mutex_lock(c->lock);
        size_t idx = (*c->next)++;
        pthread_mutex_unlock(c->lock);
        if (idx >= c->n) break;
        blt_attention_head_args a = c->jobs[idx];
        if (!a.weights_out && !a.scores_scratch) {
            size_t need = a.nq * a.nk;
            if (need > cap || !scratch) { /* a job without keys (need == 0) still wants a non-NULL pointer */
                free(scratch);
                scratch = (float *)malloc(need * sizeof(float) + 16);
                cap = need;
            }
            a.scores_scratch = scratch;
        }
        blt_attention_head_core(BLT_BACKEND_CPU, &a);
    }
    free(scratch);
    return NULL;
}

/* Independent head jobs over a thread pool; the reference operator itself is
 * untouched and single-threaded per job. Returns wall seconds. */
double ref_run_heads(const blt_attention_head_args *jobs, size_t n, int nthreads) {
    if (nthreads < 1) nthreads = 1;
    size_t next = 0;
    pthread_mutex_t lock = PTHREAD_MUTEX_INITIALIZER;
    ref_pool ctx = {jobs, n, &next, &lock};
    struct timespec t0, t1;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    if (nthreads == 1) {
        ref_worker(&ctx);
    } else {
        pthread_t *th = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)nthreads);
        for (int t = 0; t < nthreads; ++t) pthread_create(&th[t], NULL, ref_worker, &ctx);
        for (int t = 0; t < nthreads; ++t) pthread_join(th[t], NULL);
        free(th);
    }
    clock_gettime(CLOCK_MONOTONIC, &t1);
    return (double)(t1.tv_sec - t0.tv_sec) + 1e-9 * (double)(t1.tv_nsec - t0.tv_nsec);
}

void ref_build_mask(size_t nq, size_t nk, size_t window, const size_t *doc_boundaries, size_t num_docs,
                    const size_t *q_groups, const size_t *k_groups, int bidirectional, int is_causal,
                    size_t causal_offset, float *out) {
    blt_arena *arena = blt_arena_create(nq * nk * sizeof(float) + (nq + nk) * 2 * sizeof(size_t) + 4096,
                                        BLT_BACKEND_CPU);
    blt_mask_config cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.seq_len_q = nq;
    cfg.seq_len_kv = nk;
    cfg.sliding_window = window;
    cfg.doc_boundaries = doc_boundaries;
    cfg.num_docs = num_docs;
    cfg.query_group_ids = q_groups;
    cfg.kv_group_ids = k_groups;
    cfg.bidirectional_within_group = bidirectional != 0;
    cfg.is_causal = is_causal != 0;
    cfg.causal_offset = causal_offset;
    blt_tensor m;
    memset(&m, 0, sizeof(m));
    blt_build_attention_mask(&cfg, &m, arena);
    memcpy(out, m.data, nq * nk * sizeof(float));
    blt_arena_destroy(arena);
}

void ref_block_diffusion_mask(int mode, size_t S, size_t N, size_t B, const size_t *block_starts,
                              size_t num_blocks, float *out) {
    blt_arena *arena = blt_arena_create(S * S * sizeof(float) + 4096, BLT_BACKEND_CPU);
    blt_block_diffusion_config cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.mode = mode == 1 ? BLT_BDM_INFER : BLT_BDM_TRAIN;
    cfg.seq_len = S;
    cfg.num_clean = N;
    cfg.block_size = B;
    cfg.block_starts = block_starts;
    cfg.num_blocks = num_blocks;
    blt_tensor m;
    memset(&m, 0, sizeof(m));
    blt_build_block_diffusion_mask(&cfg, &m, arena);
    memcpy(out, m.data, S * S * sizeof(float));
    blt_arena_destroy(arena);
}

void ref_patch_group_ids(const blt_patch_info *patches, size_t num_patches, size_t seq_len, size_t *q_groups,
                         size_t *k_groups) {
    blt_patch_build_group_ids(patches, num_patches, seq_len, q_groups, k_groups);
}

size_t ref_decoder_latent_at(const blt_patch_info *patches, size_t num_patches, size_t pos) {
    return blt_patch_decoder_latent_at(patches, num_patches, pos);
}

void ref_expand_group_ids(const size_t *in, size_t n, size_t k, size_t *out) {
    blt_patch_expand_group_ids(in, n, k, out);
}

uint32_t ref_unmask_select_confidence(const float *s, const uint8_t *m, size_t B, float alpha) {
    return blt_unmask_select_confidence(s, m, B, alpha);
}
uint32_t ref_unmask_select_eb(const float *s, const uint8_t *m, size_t B, float gamma) {
    return blt_unmask_select_eb(s, m, B, gamma);
}
size_t ref_block_adapt_b(size_t cur, double acc, size_t lo, size_t hi, float target) {
    return blt_block_adapt_b(cur, acc, lo, hi, target);
}
size_t ref_aligned_commit_select(const blt_patch_info *p, size_t n, size_t lo, size_t hi) {
    return blt_aligned_commit_select(p, n, lo, hi);
}

/* blt_kv_cache_common_patches reads only the boundary snapshot and its count. */
size_t ref_kv_common_patches(const blt_patch_info *cached, size_t num_cached, const blt_patch_info *patches,
                             size_t num_patches) {
    blt_kv_cache cache;
    memset(&cache, 0, sizeof(cache));
    cache.cached_patches = (blt_patch_info *)cached;
    cache.cross_num_patches = num_cached;
    return blt_kv_cache_common_patches(&cache, patches, num_patches);
}

/* out[m, n] = a[m, k] * b[k, n], the reference's CPU matmul. */
void ref_matmul(const float *a, const float *b, float *out, size_t m, size_t k, size_t n) {
    blt_tensor at, bt, ot;
    blt_tensor_view_2d(&at, (void *)a, m, k, BLT_BACKEND_CPU);
    blt_tensor_view_2d(&bt, (void *)b, k, n, BLT_BACKEND_CPU);
    blt_tensor_view_2d(&ot, out, m, n, BLT_BACKEND_CPU);
    blt_matmul(&at, &bt, &ot);
}

/* The reference's multi-head attention block on the CPU for one sequence. window > 0 or
 * num_docs > 0 go through a blt_mask_config (which then carries is_causal), as the callers in
 * models/local_common.c do. */
void ref_multihead_attention(const float *input, const float *w_qkv, const float *w_proj, float *output, size_t seq_len,
                             size_t embed_dim, size_t num_heads, int is_causal, int use_rope, float rope_theta,
                             size_t window, const size_t *doc_boundaries, size_t num_docs) {
    const size_t work = seq_len * (4 * embed_dim + 2 * seq_len + 8 * (embed_dim / num_heads) + 64) * sizeof(float) +
                        seq_len * seq_len * sizeof(float) + (1u << 20);
    blt_arena *arena = blt_arena_create(work, BLT_BACKEND_CPU);
    blt_tensor in, wq, wp, out;
    blt_tensor_view_2d(&in, (void *)input, seq_len, embed_dim, BLT_BACKEND_CPU);
    blt_tensor_view_2d(&wq, (void *)w_qkv, embed_dim, 3 * embed_dim, BLT_BACKEND_CPU);
    blt_tensor_view_2d(&wp, (void *)w_proj, embed_dim, embed_dim, BLT_BACKEND_CPU);
    blt_tensor_view_2d(&out, output, seq_len, embed_dim, BLT_BACKEND_CPU);
    blt_mask_config mc;
    memset(&mc, 0, sizeof(mc));
    mc.seq_len_q = mc.seq_len_kv = seq_len;
    mc.sliding_window = window;
    mc.doc_boundaries = doc_boundaries;
    mc.num_docs = num_docs;
    mc.is_causal = is_causal != 0;
    blt_attention_config cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.embed_dim = embed_dim;
    cfg.num_heads = num_heads;
    cfg.head_dim = embed_dim / num_heads;
    cfg.is_causal = is_causal != 0;
    cfg.use_rope = use_rope != 0;
    cfg.rope_theta = rope_theta;
    cfg.mask_config = (window > 0 || num_docs > 0) ? &mc : NULL;
    blt_multihead_attention(&in, &wq, &wp, &out, &cfg, arena);
    blt_arena_destroy(arena);
}

/* The reference's cross-attention block on the CPU for one sequence, no split (views already
 * in split form), group-id mask as its callers build it. */
void ref_cross_attention(const float *query_in, const float *kv_in, const float *wq, const float *wk, const float *wv,
                         const float *wp, float *output, size_t nq, size_t nk, size_t embed_dim, size_t num_heads,
                         const size_t *q_groups, const size_t *k_groups) {
    const size_t work = (2 * nq + 2 * nk) * embed_dim * sizeof(float) + 3 * nq * nk * sizeof(float) + (1u << 20);
    blt_arena *arena = blt_arena_create(work, BLT_BACKEND_CPU);
    blt_tensor q, kv, tq, tk, tv, tp, out;
    blt_tensor_view_2d(&q, (void *)query_in, nq, embed_dim, BLT_BACKEND_CPU);
    blt_tensor_view_2d(&kv, (void *)kv_in, nk, embed_dim, BLT_BACKEND_CPU);
    blt_tensor_view_2d(&tq, (void *)wq, embed_dim, embed_dim, BLT_BACKEND_CPU);
    blt_tensor_view_2d(&tk, (void *)wk, embed_dim, embed_dim, BLT_BACKEND_CPU);
    blt_tensor_view_2d(&tv, (void *)wv, embed_dim, embed_dim, BLT_BACKEND_CPU);
    blt_tensor_view_2d(&tp, (void *)wp, embed_dim, embed_dim, BLT_BACKEND_CPU);
    blt_tensor_view_2d(&out, output, nq, embed_dim, BLT_BACKEND_CPU);
    blt_cross_attention_weights w = {&tq, &tk, &tv, &tp};
    blt_mask_config mc;
    memset(&mc, 0, sizeof(mc));
    mc.seq_len_q = nq;
    mc.seq_len_kv = nk;
    mc.query_group_ids = q_groups;
    mc.kv_group_ids = k_groups;
    mc.bidirectional_within_group = true;
    blt_cross_attention_config cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.embed_dim = embed_dim;
    cfg.num_heads = num_heads;
    cfg.mask_config = &mc;
    blt_cross_attention_forward(&q, &kv, &w, &out, &cfg, arena);
    blt_arena_destroy(arena);
}

void ref_rope_precompute(size_t max_seq_len, float theta, size_t head_dim, float *cos_out, float *sin_out) {
    blt_rope_config cfg = {.theta = theta, .head_dim = head_dim};
    blt_tensor c, s;
    blt_tensor_view_2d(&c, cos_out, max_seq_len, head_dim / 2, BLT_BACKEND_CPU);
    blt_tensor_view_2d(&s, sin_out, max_seq_len, head_dim / 2, BLT_BACKEND_CPU);
    blt_rope_precompute(max_seq_len, &cfg, &c, &s);
}

void ref_rope_apply(const float *x, const float *cos_t, const float *sin_t, float *out, size_t rows, size_t heads,
                    size_t head_dim) {
    blt_tensor xt, ct, st, ot;
    blt_tensor_view_3d(&xt, (void *)x, rows, heads, head_dim, BLT_BACKEND_CPU);
    blt_tensor_view_3d(&ot, out, rows, heads, head_dim, BLT_BACKEND_CPU);
    blt_tensor_view_2d(&ct, (void *)cos_t, rows, head_dim / 2, BLT_BACKEND_CPU);
    blt_tensor_view_2d(&st, (void *)sin_t, rows, head_dim / 2, BLT_BACKEND_CPU);
    blt_rope_apply(&xt, &ct, &st, &ot);
}

/* sizeof / offsetof of the ABI structs, for the layout check of include/fblt_attn.h. */
/* Row argmax by the reference's public operator (ops/row_stats_cpu.c:30-47, the rule its
 * generation loops decide with: infer/self_speculation.c:301,332). */
void ref_argmax_rows(const float *logits, size_t rows, size_t vocab, uint32_t *ids_out) {
    blt_tensor t;
    memset(&t, 0, sizeof(t));
    t.data = (void *)logits;
    t.shape[0] = rows;
    t.shape[1] = vocab;
    t.strides[0] = vocab;
    t.strides[1] = 1;
    t.ndim = 2;
    t.numel = rows * vocab;
    t.dtype = BLT_DTYPE_FP32;
    t.backend = BLT_BACKEND_CPU;
    blt_argmax_rows(&t, ids_out);
}

size_t ref_struct_layout(size_t *out, size_t cap) {
    const size_t v[] = {
        sizeof(blt_attention_head_args),
        offsetof(blt_attention_head_args, q),
        offsetof(blt_attention_head_args, q_stride),
        offsetof(blt_attention_head_args, k),
        offsetof(blt_attention_head_args, k_stride),
        offsetof(blt_attention_head_args, v),
        offsetof(blt_attention_head_args, v_stride),
        offsetof(blt_attention_head_args, combined),
        offsetof(blt_attention_head_args, combined_stride),
        offsetof(blt_attention_head_args, combined_col_offset),
        offsetof(blt_attention_head_args, weights_out),
        offsetof(blt_attention_head_args, lse_out),
        offsetof(blt_attention_head_args, scores_scratch),
        offsetof(blt_attention_head_args, mask),
        offsetof(blt_attention_head_args, nq),
        offsetof(blt_attention_head_args, nk),
        offsetof(blt_attention_head_args, head_dim),
        offsetof(blt_attention_head_args, is_causal),
        offsetof(blt_attention_head_args, scale),
        sizeof(blt_patch_info),
        offsetof(blt_patch_info, start_idx),
        offsetof(blt_patch_info, length),
        offsetof(blt_patch_info, peak_entropy),
        (size_t)BLT_BACKEND_CPU,
        (size_t)BLT_BACKEND_CUDA,
    };
    const size_t n = sizeof(v) / sizeof(v[0]);
    for (size_t i = 0; i < n && i < cap; ++i) out[i] = v[i];
    return n;
}
