// L1 per-row kernel: one warp per (sequence, query row, head), plain fp32 FMA,
// online softmax, key loop restricted to the row's allowed range. Handles every
// mask rule (explicit group ids included) and any head_dim up to 256; it is the
// path for short key ranges (encoder cross-attention: a patch's own bytes;
// decoder cross-attention reference rule: one latent) and the fallback for
// shapes the tile kernel does not take.
#include "common.cuh"

#include <atomic>

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

// ---- four lanes per row ---------------------------------------------------------------------
// The same per-row attention for the shapes where a row has a handful of keys (encoder
// cross-attention: a patch's own bytes; decoder cross-attention: one latent): a warp per row is
// then one long chain of dependent round trips (row tables -> range -> q -> keys) with 32 lanes
// waiting on it. Here a row belongs to 4 lanes (head_dim / 4 columns each, 16-byte loads), so a
// warp keeps 8 independent rows in flight and a CTA 32. Range rules only (explicit group ids and
// the rotary embedding stay on the warp-per-row kernel).
constexpr int kQuadRows = 32;     // rows per CTA of 128 threads
constexpr int kQuadLongRow = 16;  // rows with more keys than this are walked by the whole warp

// 16 bytes global -> shared in the calling thread's cp.async group; `valid` false copies nothing and
// fills the destination with zeros.
__device__ __forceinline__ void cp_async_16_zfill(void *smem_dst, const float *gmem_src, bool valid) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)),
                 "l"(gmem_src), "r"(valid ? 16 : 0)
                 : "memory");
}

// Running softmax state of one row (or of one quad's share of a long row).
template <int NV>
struct QuadState {
    float m, l;
    float4 acc[NV];
    __device__ __forceinline__ void reset() {
        m = -INFINITY;
        l = 0.0f;
#pragma unroll
        for (int t = 0; t < NV; ++t) acc[t] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    __device__ __forceinline__ void take(float sc, const float4 (&vv)[NV]) {
        if (!finite_f(sc)) return; // non-finite score: weight 0
        const float mn = fmaxf(m, sc);
        const float corr = exp2f(m - mn), pe = exp2f(sc - mn);
        l = l * corr + pe;
#pragma unroll
        for (int t = 0; t < NV; ++t) {
            acc[t].x = acc[t].x * corr + pe * vv[t].x;
            acc[t].y = acc[t].y * corr + pe * vv[t].y;
            acc[t].z = acc[t].z * corr + pe * vv[t].z;
            acc[t].w = acc[t].w * corr + pe * vv[t].w;
        }
        m = mn;
    }
};

// Keys j and j + 1 (each if below hi) of one row: one round trip for their K and V pieces, the two
// scores summed over the row's four lanes, both folded into st. Every lane of the warp calls this
// together (full-mask shuffles); lanes without a key load nothing.
template <int NV>
__device__ __forceinline__ void quad_key_pair(QuadState<NV> &st, const float4 (&qv)[NV], const float *kb, const float *vb,
                                              int64_t k_stride, int64_t v_stride, int j, int hi) {
    const bool one = j < hi, two = j + 1 < hi;
    const float *k0p = kb + (int64_t)(one ? j : 0) * k_stride, *v0p = vb + (int64_t)(one ? j : 0) * v_stride;
    const float *k1p = k0p + (two ? k_stride : 0), *v1p = v0p + (two ? v_stride : 0);
    float4 ka[NV], va[NV], kc[NV], vc[NV];
#pragma unroll
    for (int t = 0; t < NV; ++t) {
        const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
        ka[t] = one ? __ldg(reinterpret_cast<const float4 *>(k0p + t * 16)) : z;
        va[t] = one ? __ldg(reinterpret_cast<const float4 *>(v0p + t * 16)) : z;
        kc[t] = two ? __ldg(reinterpret_cast<const float4 *>(k1p + t * 16)) : z;
        vc[t] = two ? __ldg(reinterpret_cast<const float4 *>(v1p + t * 16)) : z;
    }
    float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
    for (int t = 0; t < NV; ++t) {
        s0 += qv[t].x * ka[t].x + qv[t].y * ka[t].y + qv[t].z * ka[t].z + qv[t].w * ka[t].w;
        s1 += qv[t].x * kc[t].x + qv[t].y * kc[t].y + qv[t].z * kc[t].z + qv[t].w * kc[t].w;
    }
    s0 += __shfl_xor_sync(0xffffffffu, s0, 1);
    s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
    s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
    s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
    if (one) st.take(s0, va);
    if (two) st.take(s1, vc);
}

// The same walk over `trips` key pairs (keys j0 + it * jstep and the one after it), with the pieces of the
// next pair already on their way: every lane copies its own 16-byte pieces with cp.async into its slots of a
// two-stage ring in shared memory (slots [stage][piece][thread]: conflict-free, private to the lane, so
// the lane's own wait_group is all the synchronisation there is) and reads them back a trip later. A walk
// of n trips then waits for memory about once instead of n times. Keys at or past hi are zero-filled by
// the copy itself (source size 0) and fold nothing into the state.
template <int NV>
__device__ __forceinline__ void quad_walk_ring(QuadState<NV> &st, const float4 (&qv)[NV], const float *kb, const float *vb,
                                               int64_t k_stride, int64_t v_stride, int j0, int jstep, int trips, int hi,
                                               float4 *ring) {
    constexpr int PIECES = 4 * NV; // K and V pieces of two keys
    const int nthreads = blockDim.x, tid = threadIdx.x;
    auto stage_in = [&](int it) {
        const int j = j0 + it * jstep;
        const bool one = j < hi, two = j + 1 < hi;
        const float *k0p = kb + (int64_t)(one ? j : 0) * k_stride, *v0p = vb + (int64_t)(one ? j : 0) * v_stride;
        const float *k1p = k0p + (two ? k_stride : 0), *v1p = v0p + (two ? v_stride : 0);
        float4 *slot = ring + (size_t)(it & 1) * PIECES * nthreads + tid;
#pragma unroll
        for (int t = 0; t < NV; ++t) {
            cp_async_16_zfill(slot + (0 * NV + t) * nthreads, k0p + t * 16, one);
            cp_async_16_zfill(slot + (1 * NV + t) * nthreads, v0p + t * 16, one);
            cp_async_16_zfill(slot + (2 * NV + t) * nthreads, k1p + t * 16, two);
            cp_async_16_zfill(slot + (3 * NV + t) * nthreads, v1p + t * 16, two);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (trips > 0) stage_in(0);
    for (int it = 0; it < trips; ++it) {
        if (it + 1 < trips) {
            stage_in(it + 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        const int j = j0 + it * jstep;
        const bool one = j < hi, two = j + 1 < hi;
        const float4 *slot = ring + (size_t)(it & 1) * PIECES * nthreads + tid;
        float4 ka[NV], va[NV], kc[NV], vc[NV];
#pragma unroll
        for (int t = 0; t < NV; ++t) {
            ka[t] = slot[(0 * NV + t) * nthreads];
            va[t] = slot[(1 * NV + t) * nthreads];
            kc[t] = slot[(2 * NV + t) * nthreads];
            vc[t] = slot[(3 * NV + t) * nthreads];
        }
        float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
        for (int t = 0; t < NV; ++t) {
            s0 += qv[t].x * ka[t].x + qv[t].y * ka[t].y + qv[t].z * ka[t].z + qv[t].w * ka[t].w;
            s1 += qv[t].x * kc[t].x + qv[t].y * kc[t].y + qv[t].z * kc[t].z + qv[t].w * kc[t].w;
        }
        s0 += __shfl_xor_sync(0xffffffffu, s0, 1);
        s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
        s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
        s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
        if (one) st.take(s0, va);
        if (two) st.take(s1, vc);
    }
}

// LONG = false drops the long-row pass (and its registers) for rules whose ranges cannot be long.
template <int HD, bool LONG>
__global__ void __launch_bounds__(kQuadRows * 4) rowq_attn_kernel(fblt_attn_desc d) {
    constexpr int NV = HD / 16; // 16-byte pieces per lane; piece t of lane dl covers columns (t * 4 + dl) * 4 ..+3
    const int b = blockIdx.z, h = blockIdx.y;
    const int q0 = d.cu_q[b], nq = d.cu_q[b + 1] - q0;
    if ((int)blockIdx.x * kQuadRows >= nq) return;
    const int k0 = d.cu_k[b], nk = d.cu_k[b + 1] - k0;
    const int lane = threadIdx.x & 31, dl = lane & 3, qd = lane >> 2;
    const int i = blockIdx.x * kQuadRows + (threadIdx.x >> 2);
    const bool valid = i < nq;

    int lo = 0, hi = 0;
    if (valid) {
        const SeqMask s = resolve_mask(d.mask, b, q0, k0, nq, nk);
        row_range(s, i, lo, hi);
    }
    const float qscale = d.scale * kLog2e;
    const float *qrow = d.q + (int64_t)(q0 + (valid ? i : 0)) * d.q_stride + (int64_t)h * HD + dl * 4;
    float4 qv[NV];
#pragma unroll
    for (int t = 0; t < NV; ++t) {
        qv[t] = valid ? __ldg(reinterpret_cast<const float4 *>(qrow + t * 16)) : make_float4(0.f, 0.f, 0.f, 0.f);
        qv[t].x *= qscale;
        qv[t].y *= qscale;
        qv[t].z *= qscale;
        qv[t].w *= qscale;
    }
    QuadState<NV> st;
    st.reset();
    const float *kb = d.k + (int64_t)k0 * d.k_stride + (int64_t)h * HD + dl * 4;
    const float *vb = d.v + (int64_t)k0 * d.v_stride + (int64_t)h * HD + dl * 4;

    // Short rows: two keys per round trip, the eight rows of a warp in lockstep (trip count = the
    // longest short row of the warp). Shuffles under per-row masks would instead split the warp
    // into eight serial strands.
    const bool long_row = LONG && hi - lo > kQuadLongRow;
    const int trips = warp_max(long_row ? 0 : (hi - lo + 1) >> 1);
    extern __shared__ float4 quad_ring[]; // LONG only: 2 stages x 4 NV pieces x 128 threads
    if constexpr (LONG) {
        quad_walk_ring<NV>(st, qv, kb, vb, d.k_stride, d.v_stride, lo, 2, trips, long_row ? lo : hi, quad_ring);
    } else {
        for (int it = 0; it < trips; ++it) quad_key_pair<NV>(st, qv, kb, vb, d.k_stride, d.v_stride, lo + 2 * it, hi);
    }

    // Long rows (a patch that absorbed the rest of its sequence): one at a time, the eight quads
    // of the warp take every eighth key pair, then their partial softmax states are merged.
    unsigned pending = LONG ? __ballot_sync(0xffffffffu, long_row && dl == 0) : 0u;
    while (LONG && pending) {
        const int src = __ffs(pending) - 1; // lane 0 of the owning quad
        pending &= pending - 1;
        const int rlo = __shfl_sync(0xffffffffu, lo, src), rhi = __shfl_sync(0xffffffffu, hi, src);
        float4 rq[NV];
#pragma unroll
        for (int t = 0; t < NV; ++t) {
            rq[t].x = __shfl_sync(0xffffffffu, qv[t].x, src + dl);
            rq[t].y = __shfl_sync(0xffffffffu, qv[t].y, src + dl);
            rq[t].z = __shfl_sync(0xffffffffu, qv[t].z, src + dl);
            rq[t].w = __shfl_sync(0xffffffffu, qv[t].w, src + dl);
        }
        QuadState<NV> part;
        part.reset();
        const int trips8 = (rhi - rlo + 15) >> 4; // the same for every lane: 16 keys per warp trip
        quad_walk_ring<NV>(part, rq, kb, vb, d.k_stride, d.v_stride, rlo + 2 * qd, 16, trips8, rhi, quad_ring);
        // merge the eight partial states (each step pairs quads 1, 2 and 4 apart); afterwards every
        // quad holds the row's state
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
            const float om = __shfl_xor_sync(0xffffffffu, part.m, off), ol = __shfl_xor_sync(0xffffffffu, part.l, off);
            const float mn = fmaxf(part.m, om);
            const float ca = part.m == -INFINITY ? 0.0f : exp2f(part.m - mn), cb = om == -INFINITY ? 0.0f : exp2f(om - mn);
            part.l = part.l * ca + ol * cb;
#pragma unroll
            for (int t = 0; t < NV; ++t) {
                part.acc[t].x = part.acc[t].x * ca + __shfl_xor_sync(0xffffffffu, part.acc[t].x, off) * cb;
                part.acc[t].y = part.acc[t].y * ca + __shfl_xor_sync(0xffffffffu, part.acc[t].y, off) * cb;
                part.acc[t].z = part.acc[t].z * ca + __shfl_xor_sync(0xffffffffu, part.acc[t].z, off) * cb;
                part.acc[t].w = part.acc[t].w * ca + __shfl_xor_sync(0xffffffffu, part.acc[t].w, off) * cb;
            }
            part.m = mn;
        }
        if (qd == (src >> 2)) st = part;
    }

    if (valid) {
        const float inv = st.l > 0.0f ? 1.0f / st.l : 0.0f; // rows without keys give zeros
        float *orow = d.out + (int64_t)(q0 + i) * d.out_stride + (int64_t)h * HD + dl * 4;
#pragma unroll
        for (int t = 0; t < NV; ++t)
            *reinterpret_cast<float4 *>(orow + t * 16) =
                make_float4(st.acc[t].x * inv, st.acc[t].y * inv, st.acc[t].z * inv, st.acc[t].w * inv);
    }
}

bool rowq_kernel_supports(const fblt_attn_desc &d, const char **why) {
    if (d.head_dim != 32 && d.head_dim != 64) {
        *why = "quad-lane row kernel: head_dim must be 32 or 64";
        return false;
    }
    if (d.mask.group_rule == FBLT_GROUP_IDS) {
        *why = "explicit group ids are not a key range";
        return false;
    }
    if (d.rope_cos) {
        *why = "quad-lane row kernel: no rotary embedding";
        return false;
    }
    if ((d.q_stride | d.k_stride | d.v_stride | d.out_stride) & 3) {
        *why = "row strides must be multiples of 4 elements";
        return false;
    }
    if (((uintptr_t)d.q | (uintptr_t)d.k | (uintptr_t)d.v | (uintptr_t)d.out) & 15) {
        *why = "q/k/v/out must be 16-byte aligned";
        return false;
    }
    if (d.num_heads > 65535 || d.batch > 65535) {
        *why = "batch/heads exceed 65535";
        return false;
    }
    return true;
}

int launch_rowq_kernel(const fblt_attn_desc &d, cudaStream_t stream) {
    if (d.max_q <= 0 || d.batch <= 0) return FBLT_OK;
    dim3 grid((d.max_q + kQuadRows - 1) / kQuadRows, d.num_heads, d.batch);
    // the decoder's one-latent rule gives every row at most `subtokens` keys
    const bool may_be_long = !(d.mask.group_rule == FBLT_GROUP_PATCH_DEC && d.mask.subtokens <= kQuadLongRow);
    // the LONG variants stage their key walk through a two-stage ring: 2 x (4 * head_dim / 16) pieces per thread
    const size_t ring32 = (size_t)2 * 4 * 2 * kQuadRows * 4 * sizeof(float4), ring64 = 2 * ring32;
    if (may_be_long) {
        static std::atomic<uint64_t> configured{0}; // one bit per device ordinal: 64 KB of dynamic shared memory needs the opt-in
        int dev = 0;
        FBLT_CUDA_TRY(cudaGetDevice(&dev));
        const uint64_t bit = 1ull << (dev & 63);
        if (!(configured.load(std::memory_order_acquire) & bit)) {
            FBLT_CUDA_TRY(cudaFuncSetAttribute(rowq_attn_kernel<64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ring64));
            FBLT_CUDA_TRY(cudaFuncSetAttribute(rowq_attn_kernel<32, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ring32));
            configured.fetch_or(bit, std::memory_order_release);
        }
    }
    if (d.head_dim == 32) {
        if (may_be_long) rowq_attn_kernel<32, true><<<grid, kQuadRows * 4, ring32, stream>>>(d);
        else rowq_attn_kernel<32, false><<<grid, kQuadRows * 4, 0, stream>>>(d);
    } else {
        if (may_be_long) rowq_attn_kernel<64, true><<<grid, kQuadRows * 4, ring64, stream>>>(d);
        else rowq_attn_kernel<64, false><<<grid, kQuadRows * 4, 0, stream>>>(d);
    }
    count_launch();
    return check_launch("rowq_attn_kernel");
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
