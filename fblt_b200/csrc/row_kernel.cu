// L1 per-row kernel: one warp per (sequence, query row, head), plain fp32 FMA,
// online softmax, key loop restricted to the row's allowed range. Handles every
// mask rule (explicit group ids included) and any head_dim up to 256; it is the
// path for short key ranges (encoder cross-attention: a patch's own bytes;
// decoder cross-attention reference rule: one latent) and the fallback for
// shapes the tile kernel does not take.
#include "common.cuh"

namespace fblt {

constexpr int kRowWarps = 4;

// Rotary embedding when a lane holds columns lane + 32 t: the partner of an (even, odd) pair
// sits in the neighbouring lane.
template <int NT>
__device__ __forceinline__ void rope_lanes(float (&x)[NT], const float *cs, const float *sn, int pos, int hd, int lane) {
    const int half = hd >> 1;
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        const int dd = lane + 32 * t;
        const float other = __shfl_xor_sync(0xffffffffu, x[t], 1);
        if (dd < hd) {
            const float c = cs[(int64_t)pos * half + (dd >> 1)], s = sn[(int64_t)pos * half + (dd >> 1)];
            x[t] = (lane & 1) ? __fadd_rn(__fmul_rn(x[t], c), __fmul_rn(other, s))
                              : __fsub_rn(__fmul_rn(x[t], c), __fmul_rn(other, s));
        }
    }
}

template <int NT, bool ROPE>
__global__ void __launch_bounds__(kRowWarps * 32) row_attn_kernel(fblt_attn_desc d) {
    const int b = blockIdx.z, h = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q0 = d.cu_q[b], nq = d.cu_q[b + 1] - q0;
    const int k0 = d.cu_k[b], nk = d.cu_k[b + 1] - k0;
    const int i = blockIdx.x * kRowWarps + warp;
    if (i >= nq) return;
    const int hd = d.head_dim;

    const SeqMask s = resolve_mask(d.mask, b, q0, k0, nq, nk);
    int lo, hi;
    row_range(s, i, lo, hi, WarpSearch{lane}); // the whole warp works on row i
    const bool by_ids = s.group_rule == FBLT_GROUP_IDS;
    const int my_group = by_ids ? s.qg[i] : 0;

    const float qscale = d.scale * kLog2e; // scores live in the log2 domain
    const float *qrow = d.q + (int64_t)(q0 + i) * d.q_stride + (int64_t)h * hd;
    float qv[NT], acc[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        const int dd = lane + 32 * t;
        qv[t] = dd < hd ? qrow[dd] : 0.0f;
        acc[t] = 0.0f;
    }
    constexpr bool rope = ROPE; // a separate instantiation: the plain kernel keeps its register count
    const int32_t *kpos = rope ? d.rope_k_pos : nullptr; // optional gathered key positions of this sequence
    if (kpos) kpos += k0;
    if constexpr (rope)
        rope_lanes<NT>(qv, d.rope_cos, d.rope_sin, d.rope_q_pos ? d.rope_q_pos[q0 + i] : i + s.causal_off, hd, lane);
#pragma unroll
    for (int t = 0; t < NT; ++t) qv[t] *= qscale;
    float m = -INFINITY, l = 0.0f;
    const float *kb = d.k + (int64_t)k0 * d.k_stride + (int64_t)h * hd;
    const float *vb = d.v + (int64_t)k0 * d.v_stride + (int64_t)h * hd;

    // Four keys per step: their K and V pieces are requested together, so a row with a short
    // key range (a patch's bytes) pays one memory round trip, not one per key.
    constexpr int G = 4;
    const int grouped_end = (hi - lo >= G) ? hi : lo; // ranges shorter than a group use the tail loop only
    for (int j0 = lo; j0 < grouped_end; j0 += G) {
        float kk[G][NT], vv[G][NT];
        bool take[G];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const int j = j0 + g;
            const bool in_range = j < hi; // uniform over the warp
            take[g] = in_range && !(by_ids && s.kg[in_range ? j : lo] != my_group);
            const float *kj = kb + (int64_t)j * d.k_stride;
            const float *vj = vb + (int64_t)j * d.v_stride;
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                const int dd = lane + 32 * t;
                kk[g][t] = (in_range && dd < hd) ? kj[dd] : 0.0f;
                vv[g][t] = (in_range && dd < hd) ? vj[dd] : 0.0f;
            }
            if constexpr (rope) rope_lanes<NT>(kk[g], d.rope_cos, d.rope_sin, in_range ? (kpos ? kpos[j] : j) : 0, hd, lane);
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
            if (j0 + g >= hi) break; // past the end of the range (uniform over the warp)
            float part = 0.0f;
#pragma unroll
            for (int t = 0; t < NT; ++t) part += qv[t] * kk[g][t];
            part = warp_sum(part);
            if (!take[g] || !finite_f(part)) continue; // masked key, or non-finite score: weight 0
            const float mn = fmaxf(m, part);
            const float corr = exp2f(m - mn);
            const float p = exp2f(part - mn);
            l = l * corr + p;
#pragma unroll
            for (int t = 0; t < NT; ++t) acc[t] = acc[t] * corr + p * vv[g][t];
            m = mn;
        }
    }
    for (int j = grouped_end; j < hi; ++j) { // one or a few keys (decoder cross-attention: a single latent)
        if (by_ids && s.kg[j] != my_group) continue;
        const float *kj = kb + (int64_t)j * d.k_stride;
        const float *vj = vb + (int64_t)j * d.v_stride;
        float part = 0.0f, vloc[NT], kloc[NT];
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            const int dd = lane + 32 * t;
            kloc[t] = dd < hd ? kj[dd] : 0.0f;
            vloc[t] = dd < hd ? vj[dd] : 0.0f;
        }
        if constexpr (rope) rope_lanes<NT>(kloc, d.rope_cos, d.rope_sin, kpos ? kpos[j] : j, hd, lane);
#pragma unroll
        for (int t = 0; t < NT; ++t) part += qv[t] * kloc[t];
        part = warp_sum(part);
        if (!finite_f(part)) continue;
        const float mn = fmaxf(m, part);
        const float corr = exp2f(m - mn);
        const float p = exp2f(part - mn);
        l = l * corr + p;
#pragma unroll
        for (int t = 0; t < NT; ++t) acc[t] = acc[t] * corr + p * vloc[t];
        m = mn;
    }

    float *orow = d.out + (int64_t)(q0 + i) * d.out_stride + (int64_t)h * hd;
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        const int dd = lane + 32 * t;
        if (dd < hd) orow[dd] = l > 0.0f ? acc[t] / l : 0.0f;
    }
}

int launch_row_kernel(const fblt_attn_desc &d, cudaStream_t stream) {
    if (d.head_dim > 256) return fail(FBLT_ERR_UNSUPPORTED, "row kernel: head_dim %d > 256", d.head_dim);
    if (d.max_q <= 0 || d.batch <= 0) return FBLT_OK;
    if (d.num_heads > 65535 || d.batch > 65535) return fail(FBLT_ERR_LIMIT, "row kernel: batch/heads exceed 65535");
    dim3 grid((d.max_q + kRowWarps - 1) / kRowWarps, d.num_heads, d.batch);
    const int nt = (d.head_dim + 31) / 32;
#define FBLT_ROW_LAUNCH(NT_)                                                                  \
    do {                                                                                      \
        if (d.rope_cos) row_attn_kernel<NT_, true><<<grid, kRowWarps * 32, 0, stream>>>(d);   \
        else row_attn_kernel<NT_, false><<<grid, kRowWarps * 32, 0, stream>>>(d);             \
    } while (0)
    if (nt <= 1) FBLT_ROW_LAUNCH(1);
    else if (nt <= 2) FBLT_ROW_LAUNCH(2);
    else if (nt <= 4) FBLT_ROW_LAUNCH(4);
    else FBLT_ROW_LAUNCH(8);
#undef FBLT_ROW_LAUNCH
    count_launch();
    return check_launch("row_attn_kernel");
}

} // namespace fblt
