/*
 * TEST INFRASTRUCTURE -- not part of the product. See attn_oracle.h.
 *
 * The arithmetic below keeps the reference's operation order (ascending d in
 * every dot product, ascending j in every accumulation, division by the row
 * sum as a separate pass), so that results agree with the reference's object
 * code bit for bit when both are built with the same compiler flags.
 */
#include "attn_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

/* ---- the single-head operator ------------------------------------------ */

/* ops/vecmath_cpu.c:6-14 */
static float dot_ascending(const float *x, const float *y, size_t n) {
    float acc = 0.0f;
    for (size_t d = 0; d < n; ++d) acc += x[d] * y[d];
    return acc;
}

/* ops/vecmath_cpu.c:16-53 */
static void masked_softmax_row(float *row, size_t len, size_t row_index, int causal, const float *mask_row,
                               float scale) {
    float top = -INFINITY;
    for (size_t c = 0; c < len; ++c) {
        float s;
        if (mask_row) {
            s = row[c] * scale + mask_row[c];
        } else if (causal && c > row_index) {
            s = -INFINITY;
        } else {
            s = row[c] * scale;
        }
        row[c] = s;
        if (isfinite(s) && s > top) top = s;
    }
    float total = 0.0f;
    for (size_t c = 0; c < len; ++c) {
        if (isfinite(row[c])) {
            row[c] = expf(row[c] - top);
            total += row[c];
        } else {
            row[c] = 0.0f;
        }
    }
    if (total > 0.0f) {
        for (size_t c = 0; c < len; ++c) row[c] /= total;
    }
}

static void attention_head_with_scratch(const fblt_head_args *a, float *w) {
    /* ops/attn_core_cpu.c:26-37: scores then row softmax */
    for (size_t i = 0; i < a->nq; ++i) {
        const float *qi = a->q + i * a->q_stride;
        float *wi = w + i * a->nk;
        for (size_t j = 0; j < a->nk; ++j) wi[j] = dot_ascending(qi, a->k + j * a->k_stride, a->head_dim);
        masked_softmax_row(wi, a->nk, i, a->is_causal, a->mask ? a->mask + i * a->nk : NULL, a->scale);
    }
    /* ops/attn_core_cpu.c:39-56: weighted sum of value rows, zero weights skipped */
    for (size_t i = 0; i < a->nq; ++i) {
        float *oi = a->combined + i * a->combined_stride + a->combined_col_offset;
        const float *wi = w + i * a->nk;
        for (size_t d = 0; d < a->head_dim; ++d) oi[d] = 0.0f;
        for (size_t j = 0; j < a->nk; ++j) {
            const float p = wi[j];
            if (p == 0.0f) continue;
            const float *vj = a->v + j * a->v_stride;
            for (size_t d = 0; d < a->head_dim; ++d) oi[d] += p * vj[d];
        }
    }
}

void oracle_attention_head(const fblt_head_args *a) {
    float *w = a->weights_out ? a->weights_out : a->scores_scratch;
    float *own = NULL;
    if (!w) {
        own = (float *)malloc(a->nq * a->nk * sizeof(float) + 16);
        w = own;
    }
    attention_head_with_scratch(a, w);
    free(own);
}

typedef struct {
    const fblt_head_args *jobs;
    size_t n;
    size_t *next;
    pthread_mutex_t *lock;
} pool_ctx;

static void *pool_worker(void *p) {
    pool_ctx *c = (pool_ctx *)p;
    float *scratch = NULL;
    size_t cap = 0;
    for (;;) {
        pthread_mutex_lock(c->lock);
        size_t idx = (*c->next)++;
        pthread_mutex_unlock(c->lock);
        if (idx >= c->n) break;
        const fblt_head_args *a = &c->jobs[idx];
        float *w = a->weights_out ? a->weights_out : a->scores_scratch;
        if (!w) {
            size_t need = a->nq * a->nk;
            if (need > cap) {
                free(scratch);
                scratch = (float *)malloc(need * sizeof(float) + 16);
                cap = need;
            }
            w = scratch;
        }
        attention_head_with_scratch(a, w);
    }
    free(scratch);
    return NULL;
}

double oracle_run_heads(const fblt_head_args *jobs, size_t n, int nthreads) {
    if (nthreads < 1) nthreads = 1;
    struct timespec t0, t1;
    size_t next = 0;
    pthread_mutex_t lock = PTHREAD_MUTEX_INITIALIZER;
    pool_ctx ctx = {jobs, n, &next, &lock};
    clock_gettime(CLOCK_MONOTONIC, &t0);
    if (nthreads == 1) {
        pool_worker(&ctx);
    } else {
        pthread_t *th = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)nthreads);
        for (int t = 0; t < nthreads; ++t) pthread_create(&th[t], NULL, pool_worker, &ctx);
        for (int t = 0; t < nthreads; ++t) pthread_join(th[t], NULL);
        free(th);
    }
    clock_gettime(CLOCK_MONOTONIC, &t1);
    return (double)(t1.tv_sec - t0.tv_sec) + 1e-9 * (double)(t1.tv_nsec - t0.tv_nsec);
}

/* ---- dense masks --------------------------------------------------------- */

/* ops/mask_builder_cpu.c:10-19: position -> document index */
static void doc_index_table(const size_t *bounds, size_t num_docs, size_t len, size_t *out) {
    size_t d = 0;
    for (size_t p = 0; p < len; ++p) {
        while (d + 1 < num_docs && p >= bounds[d]) ++d;
        out[p] = d;
    }
}

size_t oracle_build_mask(size_t nq, size_t nk, size_t window, const size_t *doc_boundaries, size_t num_docs,
                         const size_t *q_groups, const size_t *k_groups, int bidirectional, int is_causal,
                         size_t causal_offset, float *out) {
    const int docs = doc_boundaries != NULL && num_docs > 0;
    const int groups = q_groups != NULL && k_groups != NULL;
    size_t *dq = NULL, *dk = NULL;
    if (docs) {
        dq = (size_t *)malloc(nq * sizeof(size_t));
        dk = (size_t *)malloc(nk * sizeof(size_t));
        doc_index_table(doc_boundaries, num_docs, nq, dq);
        doc_index_table(doc_boundaries, num_docs, nk, dk);
    }
    size_t empty_rows = 0;
    for (size_t i = 0; i < nq; ++i) {
        int any = 0;
        for (size_t j = 0; j < nk; ++j) {
            int ok = 1;
            if (is_causal && j > i + causal_offset) ok = 0; /* :52-55 */
            if (window > 0) {                               /* :57-76 */
                size_t dist;
                if (is_causal) {
                    const size_t diag = i + causal_offset;
                    dist = diag >= j ? diag - j : j - diag;
                } else {
                    dist = i >= j ? i - j : j - i;
                }
                if (dist >= window) ok = 0;
            }
            if (docs && dq[i] != dk[j]) ok = 0; /* :78-80 */
            if (groups) {                       /* :82-88 */
                if (q_groups[i] != k_groups[j]) ok = 0;
                else if (!bidirectional && j > i) ok = 0;
            }
            out[i * nk + j] = ok ? 0.0f : -INFINITY;
            any |= ok;
        }
        if (!any) ++empty_rows;
    }
    free(dq);
    free(dk);
    return empty_rows;
}

size_t oracle_block_diffusion_mask(int mode, size_t S, size_t N, size_t B, const size_t *block_starts,
                                   size_t num_blocks, float *out) {
    (void)num_blocks;
    size_t empty_rows = 0;
    for (size_t i = 0; i < S; ++i) {
        int any = 0;
        for (size_t j = 0; j < S; ++j) {
            int ok;
            if (i < N) {
                ok = (j < N) && (j <= i); /* :126-129 */
            } else if (mode == 1) {
                ok = 1; /* :130-132 */
            } else {
                const size_t blk = (i - N) / B; /* :133-146 */
                const size_t s = block_starts[blk];
                const int own = (j >= N) && ((j - N) / B == blk);
                ok = (j < s) || own;
            }
            out[i * S + j] = ok ? 0.0f : -INFINITY;
            any |= ok;
        }
        if (!any) ++empty_rows;
    }
    return empty_rows;
}

void oracle_decode_self_mask(size_t n, size_t base, size_t window, float *out) {
    const size_t total = base + n;
    for (size_t r = 0; r < n; ++r) {
        const size_t p = base + r;
        for (size_t j = 0; j < total; ++j) {
            int ok = (j <= p);
            if (ok && window > 0 && p - j >= window) ok = 0;
            out[r * total + j] = ok ? 0.0f : -INFINITY;
        }
    }
}

void oracle_decode_cross_mask(const fblt_patch_info *patches, size_t num_patches, size_t k, size_t n, size_t base,
                              int trailing_closed, float *out) {
    const size_t total_sub = num_patches * k;
    for (size_t r = 0; r < n; ++r) {
        size_t g = oracle_decoder_latent_at(patches, num_patches, base + r);
        if (trailing_closed && num_patches >= 1 && r == n - 1) g = num_patches - 1;
        for (size_t j = 0; j < total_sub; ++j) out[r * total_sub + j] = (j / k == g) ? 0.0f : -INFINITY;
    }
}

/* ---- patch helpers ------------------------------------------------------- */

int oracle_patch_group_ids(const fblt_patch_info *patches, size_t num_patches, size_t seq_len, size_t *q_groups,
                           size_t *k_groups) {
    for (size_t p = 0; p < num_patches; ++p) q_groups[p] = p;
    size_t pos = 0;
    for (size_t p = 0; p < num_patches; ++p) {
        if (patches[p].start_idx != pos || patches[p].length < 1) return 1;
        if (pos + patches[p].length > seq_len) return 1;
        for (size_t t = 0; t < patches[p].length; ++t) k_groups[pos++] = p;
    }
    return pos == seq_len ? 0 : 1;
}

size_t oracle_decoder_latent_at(const fblt_patch_info *patches, size_t num_patches, size_t pos) {
    if (pos < patches[0].start_idx) return 0;
    for (size_t p = 0; p < num_patches; ++p) {
        const size_t first = patches[p].start_idx;
        if (first > pos) break;
        const size_t end = first + patches[p].length;
        if (pos < end) {
            const int closes_patch = (pos + 1 == end) && (p + 1 < num_patches);
            if (closes_patch) return p;
            return p == 0 ? 0 : p - 1;
        }
    }
    return num_patches - 1;
}

void oracle_expand_group_ids(const size_t *in, size_t n, size_t k, size_t *out) {
    for (size_t i = 0; i < n; ++i)
        for (size_t s = 0; s < k; ++s) out[i * k + s] = in[i];
}

/* ---- decisions ----------------------------------------------------------- */

int32_t oracle_argmax_row(const float *row, size_t vocab) {
    size_t arg = 0;
    float top = row[0];
    for (size_t v = 1; v < vocab; ++v) {
        if (row[v] > top) {
            top = row[v];
            arg = v;
        }
    }
    return (int32_t)arg;
}

size_t oracle_verify_accept(uint8_t *x, const float *logits, size_t vocab, size_t l, size_t r, size_t target_len,
                            size_t *accepted) {
    const size_t cand = l + r;
    for (size_t p = l; p < cand; ++p) {
        const uint8_t want = (uint8_t)oracle_argmax_row(logits + (p - 1) * vocab, vocab);
        if (x[p] != want) {
            x[p] = want;
            if (accepted) *accepted = p - l;
            return p + 1;
        }
    }
    if (accepted) *accepted = r;
    if (cand < target_len) {
        x[cand] = (uint8_t)oracle_argmax_row(logits + (cand - 1) * vocab, vocab);
        return cand + 1;
    }
    return cand;
}

void oracle_row_analyze(const float *row, size_t vocab, float *p_max, float *entropy) {
    float top = row[0];
    for (size_t v = 1; v < vocab; ++v)
        if (row[v] > top) top = row[v];
    double z = 0.0;
    for (size_t v = 0; v < vocab; ++v) z += exp((double)row[v] - (double)top);
    double best = 0.0, h = 0.0;
    for (size_t v = 0; v < vocab; ++v) {
        const double p = exp((double)row[v] - (double)top) / z;
        if (p > best) best = p;
        if (p > 1e-12) h -= p * log(p);
    }
    *p_max = (float)best;
    *entropy = (float)h;
}

uint32_t oracle_unmask_select_confidence(const float *scores, const uint8_t *masked, size_t B, float alpha) {
    uint32_t chosen = 0;
    size_t top = SIZE_MAX;
    for (size_t b = 0; b < B; ++b) {
        if (!masked[b]) continue;
        if (top == SIZE_MAX || scores[b] > scores[top]) top = b;
        if (scores[b] >= alpha) chosen |= (uint32_t)1u << b;
    }
    if (chosen == 0 && top != SIZE_MAX) chosen = (uint32_t)1u << top;
    return chosen;
}

uint32_t oracle_unmask_select_eb(const float *scores, const uint8_t *masked, size_t B, float gamma) {
    size_t order[32];
    size_t n = 0;
    for (size_t b = 0; b < B; ++b) { /* stable insertion sort, ascending entropy */
        if (!masked[b]) continue;
        size_t at = n++;
        while (at > 0 && scores[order[at - 1]] > scores[b]) {
            order[at] = order[at - 1];
            --at;
        }
        order[at] = b;
    }
    if (n == 0) return 0;
    uint32_t chosen = 0;
    float spent = 0.0f;
    size_t t = 0;
    while (t < n && (t == 0 || spent + scores[order[t]] <= gamma)) {
        spent += scores[order[t]];
        chosen |= (uint32_t)1u << order[t];
        ++t;
    }
    if (chosen == 0) chosen = (uint32_t)1u << order[0];
    return chosen;
}

size_t oracle_block_adapt_b(size_t cur_b, double rolling_acceptance, size_t b_min, size_t b_max, float target) {
    const float margin = 0.10f; /* BLT_ADAPT_B_MARGIN, infer/block_generation.h:76 */
    if (b_max == 0 || b_max < b_min) return cur_b;
    size_t floor_b = b_min ? b_min : 1;
    if (floor_b > b_max) floor_b = b_max;
    size_t b = cur_b < floor_b ? floor_b : cur_b;
    if (b > b_max) b = b_max;
    if (!(rolling_acceptance >= 0.0)) return b;
    if (rolling_acceptance > (double)(target + margin)) {
        if (b < b_max) ++b;
    } else if (rolling_acceptance < (double)(target - margin)) {
        if (b > floor_b) --b;
    }
    return b;
}

size_t oracle_aligned_commit_select(const fblt_patch_info *patches, size_t num_patches, size_t lo, size_t hi) {
    size_t pick = 0;
    for (size_t p = 0; p < num_patches; ++p) {
        const size_t end = patches[p].start_idx + patches[p].length;
        if (end > lo && end <= hi && end > pick) pick = end;
    }
    return pick;
}

/* ---- rotary embedding (for the fused decode prologue) ---------------------- */

/* ops/reductions_cpu.c:179-197 */
void oracle_rope_precompute(size_t max_seq_len, float theta, size_t head_dim, float *cos_out, float *sin_out) {
    const size_t half = head_dim / 2;
    for (size_t pos = 0; pos < max_seq_len; ++pos) {
        for (size_t i = 0; i < half; ++i) {
            const float freq = 1.0f / powf(theta, (float)(2 * i) / (float)head_dim);
            const float angle = (float)pos * freq;
            cos_out[pos * half + i] = cosf(angle);
            sin_out[pos * half + i] = sinf(angle);
        }
    }
}

/* ops/reductions_cpu.c:199-233: x, out are [rows, heads, head_dim]; cos/sin [rows, head_dim/2] */
void oracle_rope_apply(const float *x, const float *cos_t, const float *sin_t, float *out, size_t rows,
                       size_t heads, size_t head_dim) {
    const size_t half = head_dim / 2;
    for (size_t t = 0; t < rows; ++t) {
        for (size_t h = 0; h < heads; ++h) {
            const float *xv = x + (t * heads + h) * head_dim;
            float *ov = out + (t * heads + h) * head_dim;
            for (size_t i = 0; i < half; ++i) {
                const float a = xv[2 * i], b = xv[2 * i + 1];
                ov[2 * i] = a * cos_t[t * half + i] - b * sin_t[t * half + i];
                ov[2 * i + 1] = b * cos_t[t * half + i] + a * sin_t[t * half + i];
            }
        }
    }
}

/* ---- projection matmul -------------------------------------------------------- */

/* ops/linalg_cpu.c:8-18 */
void oracle_matmul(const float *a, const float *b, float *out, size_t m, size_t k, size_t n) {
    for (size_t i = 0; i < m; ++i) {
        for (size_t j = 0; j < n; ++j) {
            float acc = 0.0f;
            for (size_t t = 0; t < k; ++t) acc += a[i * k + t] * b[t * n + j];
            out[i * n + j] = acc;
        }
    }
}
