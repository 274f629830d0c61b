// Multi-head self-attention block over a batch of packed sequences: the work of
// blt_multihead_attention (models/attention.c:130-207) -- QKV projection, rotary embedding of
// Q and K, per-head masked attention, output projection -- as three launches: the tcgen05
// matmul with the rotation in its epilogue (or, for odd shapes, fused into the attention
// kernel's loads), the batched attention kernel with the mask evaluated from the descriptor,
// and the matmul again. The reference runs, per sequence and
// layer, two GEMMs, 2 x heads rotary launches, a mask build and one attention launch per head.
#include "common.cuh"

#include <math.h>

namespace fblt {
int matmul_qkv_rotated(const float *a, int64_t lda, const void *packed_qkv, int64_t rows, int64_t E, int32_t head_dim,
                       const int32_t *cu_rows, int32_t batch, float *out, int64_t ldo, const float *rope_cos,
                       const float *rope_sin, int32_t precision, void *stream); // gemm5_kernel.cu
}

extern "C" int fblt_mha_forward(const fblt_mha_desc *d, void *stream) {
    fblt::NvtxRange nvtx_range("fblt_mha_forward");
    using namespace fblt;
    if (!d) return fail(FBLT_ERR_ARG, "mha: NULL descriptor");
    if (d->batch < 0 || d->num_heads <= 0 || d->head_dim <= 0 || d->total_rows < 0 || d->max_len < 0)
        return fail(FBLT_ERR_ARG, "mha: bad sizes");
    if (d->total_rows == 0 || d->batch == 0) return FBLT_OK;
    const int64_t E = (int64_t)d->num_heads * d->head_dim;
    if (!d->input || !d->output || !d->packed_qkv || !d->packed_proj || !d->qkv_work || !d->combined_work || !d->cu_rows)
        return fail(FBLT_ERR_ARG, "mha: buffers must not be NULL");
    if (d->input_stride < E || d->output_stride < E) return fail(FBLT_ERR_ARG, "mha: row strides below embed_dim");

    // With embed_dim and head_dim multiples of 32 the projection's epilogue rotates Q and K itself (query and
    // key positions coincide in a self-attention block unless the mask shifts the queries), and the attention
    // kernels, the TMA-fed one included, read rotated rows.
    const bool rotate_in_epilogue = d->rope_cos && d->rope_sin && !(E & 31) && !(d->head_dim & 31) && !d->mask.causal_offset &&
                                    !(((uintptr_t)d->qkv_work) & 15);
    int st;
    if (rotate_in_epilogue)
        st = matmul_qkv_rotated(d->input, d->input_stride, d->packed_qkv, d->total_rows, E, d->head_dim, d->cu_rows, d->batch,
                                d->qkv_work, 3 * E, d->rope_cos, d->rope_sin, d->precision, stream);
    else
        st = fblt_matmul(d->input, d->input_stride, d->packed_qkv, nullptr, d->qkv_work, 3 * E, d->total_rows, E, 3 * E,
                         d->precision, stream);
    if (st != FBLT_OK) return st;

    fblt_attn_desc a;
    memset(&a, 0, sizeof(a));
    a.batch = d->batch;
    a.num_heads = d->num_heads;
    a.head_dim = d->head_dim;
    a.max_q = a.max_k = d->max_len;
    if (d->total_rows <= 0x7fffffff) a.total_q_rows = a.total_k_rows = (int32_t)d->total_rows;
    a.impl = FBLT_IMPL_AUTO;
    a.precision = d->precision;
    a.cu_q = a.cu_k = d->cu_rows;
    a.q = d->qkv_work;
    a.k = d->qkv_work + E;
    a.v = d->qkv_work + 2 * E;
    a.q_stride = a.k_stride = a.v_stride = 3 * E;
    a.out = d->combined_work;
    a.out_stride = E;
    a.scale = 1.0f / sqrtf((float)d->head_dim); // models/attention.c:137
    a.mask = d->mask;
    if (!rotate_in_epilogue) {
        a.rope_cos = d->rope_cos;
        a.rope_sin = d->rope_sin;
    }
    st = fblt_attn_forward(&a, stream);
    if (st != FBLT_OK) return st;

    return fblt_matmul(d->combined_work, E, d->packed_proj, nullptr, d->output, d->output_stride, d->total_rows, E, E,
                       d->precision, stream);
}

// The cross-attention block of blt_cross_attention_forward (models/cross_attention.c:98-157):
// Q from query_in, K and V from kv_in (one matmul against [weight_k | weight_v]), masked
// attention under the patch rule of the descriptor, output projection. Four launches.
extern "C" int fblt_cross_attention_forward(const fblt_cross_desc *d, void *stream) {
    fblt::NvtxRange nvtx_range("fblt_cross_attention_forward");
    using namespace fblt;
    if (!d) return fail(FBLT_ERR_ARG, "cross: NULL descriptor");
    if (d->batch < 0 || d->num_heads <= 0 || d->head_dim <= 0 || d->total_q_rows < 0 || d->total_k_rows < 0)
        return fail(FBLT_ERR_ARG, "cross: bad sizes");
    if (d->total_q_rows == 0 || d->batch == 0) return FBLT_OK;
    const int64_t E = (int64_t)d->num_heads * d->head_dim;
    if (!d->query_in || !d->kv_in || !d->output || !d->packed_q || !d->packed_kv || !d->packed_proj || !d->q_work ||
        !d->kv_work || !d->combined_work || !d->cu_q || !d->cu_k)
        return fail(FBLT_ERR_ARG, "cross: buffers must not be NULL");
    if (d->query_stride < E || d->kv_stride < E || d->output_stride < E)
        return fail(FBLT_ERR_ARG, "cross: row strides below embed_dim");

    int st = fblt_matmul(d->query_in, d->query_stride, d->packed_q, nullptr, d->q_work, E, d->total_q_rows, E, E, d->precision,
                         stream);
    if (st != FBLT_OK) return st;
    st = fblt_matmul(d->kv_in, d->kv_stride, d->packed_kv, nullptr, d->kv_work, 2 * E, d->total_k_rows, E, 2 * E,
                     d->precision, stream);
    if (st != FBLT_OK) return st;

    fblt_attn_desc a;
    memset(&a, 0, sizeof(a));
    a.batch = d->batch;
    a.num_heads = d->num_heads;
    a.head_dim = d->head_dim;
    a.max_q = d->max_q;
    a.max_k = d->max_k;
    if (d->total_q_rows <= 0x7fffffff && d->total_k_rows <= 0x7fffffff) {
        a.total_q_rows = (int32_t)d->total_q_rows;
        a.total_k_rows = (int32_t)d->total_k_rows;
    }
    a.impl = FBLT_IMPL_AUTO;
    a.precision = d->precision;
    a.cu_q = d->cu_q;
    a.cu_k = d->cu_k;
    a.q = d->q_work;
    a.q_stride = E;
    a.k = d->kv_work;
    a.v = d->kv_work + E;
    a.k_stride = a.v_stride = 2 * E;
    a.out = d->combined_work;
    a.out_stride = E;
    a.scale = 1.0f / sqrtf((float)d->head_dim); // models/cross_attention.c:112
    a.mask = d->mask;
    st = fblt_attn_forward(&a, stream);
    if (st != FBLT_OK) return st;

    return fblt_matmul(d->combined_work, E, d->packed_proj, nullptr, d->output, d->output_stride, d->total_q_rows, E, E,
                       d->precision, stream);
}

// The self-attention part of one cache-aware decode step (infer/kv_cache.c:338-396) for a batch:
// qkv = rows * weight_qkv; Q and K rotated with position base + r; K / V written through to the
// cache at rows base .. base + n; attention of the n new rows over the cache; output projection.
// The reference does this per layer with 5 strided copies and 2 rotary launches per head and one
// operator launch per head; here it is the matmul, the decode kernel (rotation and write-through
// fused) and the matmul again; with embed_dim and head_dim multiples of 32 the first matmul's epilogue
// does the rotation and the write-through itself (attention.c:156 + kv_cache.c:347-366 in one launch).
namespace fblt {
int matmul_qkv_to_cache(const float *a, int64_t lda, const void *packed_qkv, int64_t rows, int64_t E, int32_t head_dim,
                        int32_t n_new, const int32_t *base_len, int32_t base_add, float *q_out, int64_t q_stride,
                        float *kc, float *vc, int64_t seq_stride, int64_t row_stride, const float *rope_cos,
                        const float *rope_sin, int32_t precision, void *stream); // gemm5_kernel.cu
}

extern "C" int fblt_kv_self_attention_step(const fblt_kv_step_desc *d, void *stream) {
    fblt::NvtxRange nvtx_range("fblt_kv_self_attention_step");
    using namespace fblt;
    if (!d) return fail(FBLT_ERR_ARG, "kv step: NULL descriptor");
    if (d->batch < 0 || d->num_heads <= 0 || d->head_dim <= 0 || d->n_new < 1)
        return fail(FBLT_ERR_ARG, "kv step: bad sizes");
    if (d->batch == 0) return FBLT_OK;
    const int64_t E = (int64_t)d->num_heads * d->head_dim, rows = (int64_t)d->batch * d->n_new;
    if (!d->input || !d->output || !d->packed_qkv || !d->packed_proj || !d->qkv_work || !d->combined_work)
        return fail(FBLT_ERR_ARG, "kv step: buffers must not be NULL");
    if (d->input_stride < E || d->output_stride < E) return fail(FBLT_ERR_ARG, "kv step: row strides below embed_dim");

    // Projection with the scatter epilogue where the shape allows (embed and head_dim multiples of 32):
    // the rotated K rows and the V rows go straight from the matmul's accumulators into the cache, the
    // rotated Q rows into the first E columns' worth of qkv_work; [rows, 3E] never exists in memory.
    const bool scatter = !(E & 31) && !(d->head_dim & 31);
    int st;
    if (scatter)
        st = matmul_qkv_to_cache(d->input, d->input_stride, d->packed_qkv, rows, E, d->head_dim, d->n_new, d->base_len, 0,
                                 d->qkv_work, E, d->k_cache, d->v_cache, d->cache_seq_stride, d->cache_row_stride,
                                 d->rope_cos, d->rope_sin, d->precision, stream);
    else
        st = fblt_matmul(d->input, d->input_stride, d->packed_qkv, nullptr, d->qkv_work, 3 * E, rows, E, 3 * E, d->precision,
                         stream);
    if (st != FBLT_OK) return st;

    fblt_decode_desc a;
    memset(&a, 0, sizeof(a));
    a.batch = d->batch;
    a.num_heads = d->num_heads;
    a.head_dim = d->head_dim;
    a.n_new = d->n_new;
    a.block_mode = d->block_mode;
    a.window = d->window;
    a.max_len = d->max_len;
    a.base_len = d->base_len;
    a.k_cache = d->k_cache;
    a.v_cache = d->v_cache;
    a.cache_seq_stride = d->cache_seq_stride;
    a.cache_row_stride = d->cache_row_stride;
    a.q = d->qkv_work;
    a.out = d->combined_work;
    a.out_stride = E;
    a.scale = 1.0f / sqrtf((float)d->head_dim); // infer/kv_cache.c:258
    if (scatter) { // rows already rotated and in place: the kernel reads the appended rows from the cache
        a.q_stride = E;
    } else {
        a.q_stride = 3 * E;
        a.k_new = d->qkv_work + E;
        a.v_new = d->qkv_work + 2 * E;
        a.kv_new_stride = 3 * E;
        a.rope_cos = d->rope_cos;
        a.rope_sin = d->rope_sin;
    }
    const size_t need = fblt_attn_decode_workspace(&a);
    if (need > d->workspace_bytes) a.splits = 1; // no room for split-K partials: one pass per (sequence, head)
    st = fblt_attn_decode(&a, d->workspace, d->workspace_bytes, stream);
    if (st != FBLT_OK) return st;

    return fblt_matmul(d->combined_work, E, d->packed_proj, nullptr, d->output, d->output_stride, rows, E, E, d->precision,
                       stream);
}
