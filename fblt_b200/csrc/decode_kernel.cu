// L1 KV-cache decode / block-verify attention: n_new fresh query rows per
// sequence over that sequence's cache rows, every sequence and head in one
// launch. Bandwidth-bound by construction (each K/V row is used for at most
// n_new dot products), so the kernel is a coalesced HBM streamer:
//
//   * CTA = (head, key-range split, sequence x query-group), 4 warps;
//   * a key row of one head (head_dim floats) is covered by head_dim/4 lanes
//     with one 16-byte load each, so a warp instruction fetches 32/(head_dim/4)
//     complete rows, and U such loads for K and V are in flight per lane;
//   * the partial scores of a chunk are reduced inside the lane group with a
//     transposing butterfly that leaves one complete score per lane; that lane
//     runs the online softmax (log2 domain) for it and the probabilities are
//     broadcast for the PV accumulation; groups / warps merge at the end;
//   * optionally the rotary embedding of the new q / k rows is applied on load;
//   * keys every row of the CTA can see take the unmasked path; the few keys at
//     the window edge and the freshly appended rows take a per-row checked path;
//   * split-K writes (m, l, acc) partials to caller scratch; a second small
//     kernel merges them (no inter-CTA waiting anywhere).
#include "common.cuh"

#include <atomic>

#include <limits.h>
#include <stdlib.h>
#include <string.h>

namespace fblt {

constexpr int kDecWarps = 4;
constexpr int kDecThreads = kDecWarps * 32;

struct DecodeParams {
    int batch, H, n_new, block_mode, window, splits, qgroups, base_add;
    const int32_t *base_len;
    float *kc, *vc;
    int64_t seq_stride, row_stride;
    const float *q;
    int64_t q_stride;
    const float *kn, *vn;
    int64_t new_stride;
    float *out;
    int64_t out_stride;
    float *ws;
    float qscale;
    const float *rope_cos, *rope_sin; // [positions, HD/2] tables, or NULL: q / k_new arrive rotated
};

__device__ __forceinline__ float4 ld4(const float *p) { return __ldg(reinterpret_cast<const float4 *>(p)); }
// 16 bytes global -> shared, bypassing L1, in the calling thread's current cp.async group
__device__ __forceinline__ void cp_async_16(void *smem_dst, const float *gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src)
                 : "memory");
}
// Packed fp32 pairs (one instruction for two multiply-adds): the stream is issue-bound once the power cap
// has pulled the SM clock down, and these two helpers are most of its arithmetic.
__device__ __forceinline__ float dot4(const float4 &a, const float4 &b) {
    float2 t = __fmul2_rn(make_float2(a.x, a.y), make_float2(b.x, b.y));
    t = __ffma2_rn(make_float2(a.z, a.w), make_float2(b.z, b.w), t);
    return t.x + t.y;
}
__device__ __forceinline__ void fma4(float4 &acc, float p, const float4 &v) {
    const float2 pp = make_float2(p, p);
    const float2 lo = __ffma2_rn(pp, make_float2(v.x, v.y), make_float2(acc.x, acc.y));
    const float2 hi = __ffma2_rn(pp, make_float2(v.z, v.w), make_float2(acc.z, acc.w));
    acc = make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ void scale4(float4 &a, float c) {
    a.x *= c;
    a.y *= c;
    a.z *= c;
    a.w *= c;
}

__device__ __forceinline__ float fast_exp2(float x) { // 2^x; -inf -> 0, tiny results flush to 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Sums CNT values per lane across the lanes of a group (xor offsets O, O/2, .. 1).
// While more than one value is left, a step keeps one half of the values and
// trades the other half with the partner lane (lanes with bit O set keep the
// upper half), so the value count halves each step; once a single value is
// left the remaining steps are plain butterfly adds. The result is in v[0].
template <int CNT, int O>
__device__ __forceinline__ void lane_group_transpose_reduce(float *v, int lane) {
    if constexpr (O >= 1) {
        if constexpr (CNT > 1) {
            constexpr int HALF = CNT / 2;
            const bool upper = (lane & O) != 0;
#pragma unroll
            for (int i = 0; i < HALF; ++i) {
                const float give = upper ? v[i] : v[i + HALF];
                const float keep = upper ? v[i + HALF] : v[i];
                v[i] = keep + __shfl_xor_sync(0xffffffffu, give, O);
            }
            lane_group_transpose_reduce<HALF, O / 2>(v, lane);
        } else {
            v[0] += __shfl_xor_sync(0xffffffffu, v[0], O);
            lane_group_transpose_reduce<1, O / 2>(v, lane);
        }
    }
}

// Rotary embedding of the two (even, odd) pairs a lane holds, for absolute position `pos`:
// out[2i] = x[2i] c_i - x[2i+1] s_i, out[2i+1] = x[2i+1] c_i + x[2i] s_i (ops/reductions_cpu.c:217-228).
// Products and sums are rounded separately, as the CPU code does, so rotated rows match it exactly.
__device__ __forceinline__ float4 rope_pairs(float4 x, const float *cs, const float *sn, int pos, int half, int pair0) {
    const float2 c = __ldg(reinterpret_cast<const float2 *>(cs + (int64_t)pos * half + pair0));
    const float2 s = __ldg(reinterpret_cast<const float2 *>(sn + (int64_t)pos * half + pair0));
    float4 o;
    o.x = __fsub_rn(__fmul_rn(x.x, c.x), __fmul_rn(x.y, s.x));
    o.y = __fadd_rn(__fmul_rn(x.y, c.x), __fmul_rn(x.x, s.x));
    o.z = __fsub_rn(__fmul_rn(x.z, c.y), __fmul_rn(x.w, s.y));
    o.w = __fadd_rn(__fmul_rn(x.w, c.y), __fmul_rn(x.z, s.y));
    return o;
}

template <int HD>
__host__ __device__ constexpr int dec_partial_floats() {
    return HD + 4; // acc[HD], m, l, 2 pad (keeps 16-byte alignment)
}

// Shared memory of one CTA: the warps' partial states meet here.
constexpr int kDecMaxU = 8; // (4, which would give the single-row decode a ring too, loses 2 % on long caches)
// Keys per lane group and chunk of the unmasked stream: as many as fit "one score per lane", at most kDecMaxU.
template <int HD, int NQ>
__host__ __device__ constexpr int dec_chunk_u() {
    return ((HD / 4) / NQ) > kDecMaxU ? kDecMaxU : (((HD / 4) / NQ) < 1 ? 1 : ((HD / 4) / NQ));
}
// Whether the grid form stages the stream through shared memory (see DecShared::ring): the shapes whose
// two-stage ring stays small enough for five CTAs per SM.
template <int HD, int NQ>
__host__ __device__ constexpr bool dec_ring_ok() {
    return dec_chunk_u<HD, NQ>() <= 4 && HD <= 64;
}

template <int HD, int NQ, bool RING>
struct DecShared {
    float4 acc[kDecWarps][NQ][HD / 4];
    float m[kDecWarps][NQ], l[kDecWarps][NQ];
    // RING: per warp two stages of one chunk (U key pieces + U value pieces per lane). Every lane copies its
    // own 16-byte pieces with cp.async and reads the same slots back, so a stage is in flight while the
    // previous one is consumed, at no cost in registers and with no synchronisation beyond the lane's own
    // wait_group.
    float4 ring[RING ? kDecWarps : 1][2][RING ? 2 * dec_chunk_u<HD, NQ>() : 1][RING ? 32 : 1];
};

// Key range a query group may attend to, over all of its rows: [lo_min, hi_max).
__device__ __forceinline__ void dec_group_range(const DecodeParams &p, int base, int r0, int nv, int &lo_min, int &hi_max) {
    const int total = base + p.n_new;
    hi_max = p.block_mode ? total : base + r0 + nv;
    lo_min = (p.window > 0 && !p.block_mode) ? max(0, base + r0 + 1 - p.window) : 0;
}

// One piece of work: query group qg of (sequence b, head h) over the keys [k0, k1) (already inside
// the group's range). The result goes to the output rows (direct) or, as (acc, m, l) partials, to
// wdst + q * wrow floats for row q of the group.
template <int HD, int NQ, bool RING>
__device__ __forceinline__ void decode_piece(const DecodeParams &p, DecShared<HD, NQ, RING> &sh, int b, int h, int qg, int base,
                                             int k0, int k1, bool direct, float *wdst, int64_t wrow,
                                             bool write_through) {
    constexpr int LPK = HD / 4;   // lanes per key row
    constexpr int KPW = 32 / LPK; // key rows per warp load
    // keys per lane group and chunk: as many as fit "one score per lane", at most 8
    constexpr int U = dec_chunk_u<HD, NQ>();
    constexpr int CH = KPW * U; // keys per warp per chunk

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int grp = lane / LPK, dl = lane % LPK;
    const int n = p.n_new;
    const int total = base + n;
    const int r0 = qg * NQ;
    const int nv = min(NQ, n - r0); // valid rows in this query group (>= 1)

    int lo_r[NQ], hi_r[NQ];
#pragma unroll
    for (int q = 0; q < NQ; ++q) {
        const int r = r0 + q;
        if (q < nv) {
            hi_r[q] = p.block_mode ? total : base + r + 1;
            lo_r[q] = (p.window > 0 && !p.block_mode) ? max(0, base + r + 1 - p.window) : 0;
        } else {
            hi_r[q] = 0;
            lo_r[q] = 0;
        }
    }
    // rows ascend, so do both bounds
    const int hi_min = hi_r[0];
    int lo_max = lo_r[0];
#pragma unroll
    for (int q = 1; q < NQ; ++q) {
        if (q < nv) lo_max = lo_r[q];
    }

    // keys all valid rows see, served from the cache
    int F0 = max(k0, lo_max);
    int F1 = min(k1, hi_min);
    if (p.kn) F1 = min(F1, base);
    if (F1 < F0) F1 = F0;
    const int nchunks = (F1 - F0) / CH;
    const int Fe = F0 + nchunks * CH;
    const int head_slow = F0 - k0;
    const int nslow = head_slow + (k1 - Fe);

    const int64_t hoff = (int64_t)h * HD + dl * 4;
    const float *kc = p.kc + (int64_t)b * p.seq_stride + hoff;
    const float *vc = p.vc + (int64_t)b * p.seq_stride + hoff;

    float4 qv[NQ], acc[NQ];
    float m[NQ], l[NQ];
#pragma unroll
    for (int q = 0; q < NQ; ++q) {
        if (q < nv) {
            qv[q] = ld4(p.q + (int64_t)(b * n + r0 + q) * p.q_stride + hoff);
            if (p.rope_cos) qv[q] = rope_pairs(qv[q], p.rope_cos, p.rope_sin, base + r0 + q, HD / 2, dl * 2);
            scale4(qv[q], p.qscale);
        } else {
            qv[q] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        acc[q] = make_float4(0.f, 0.f, 0.f, 0.f);
        m[q] = -INFINITY;
        l[q] = 0.0f;
    }

    // ---- unmasked stream -------------------------------------------------
    // The U*NQ partial scores of a chunk are reduced over the LPK lanes of a
    // key group with a transposing butterfly: each step halves the number of
    // values a lane carries, so the reduction costs V-1 shuffles instead of
    // V*log2(LPK), and leaves score (u, q) = (idx / NQ, idx % NQ) on the lanes
    // with dl / REP == idx. Those lanes run the softmax for their own score
    // only; probabilities and rescale factors are then broadcast for the PV
    // accumulation, which every lane does for its four value columns.
    {
        constexpr int V = U * NQ;
        static_assert(V <= LPK, "chunk shape must leave at most one score per lane");
        constexpr int REP = LPK / V;     // lanes holding the same score after the reduction
        const int idx = dl / REP;        // the score this lane owns
        const int q_own = idx % NQ;
        float m_own = -INFINITY, l_own = 0.0f;
        // running row pointers: the chunk loop adds one precomputed stride instead of redoing the
        // 64-bit row arithmetic for every load
        const int64_t ustep = (int64_t)KPW * p.row_stride, cstep = (int64_t)kDecWarps * CH * p.row_stride;
        const float *kp = kc + (int64_t)(F0 + warp * CH + grp) * p.row_stride;
        const float *vp = vc + (int64_t)(F0 + warp * CH + grp) * p.row_stride;
        // RING: the chunk after this one is already on its way into the warp's other stage
        auto stage_in = [&](const float *kq, const float *vq, int slot) {
            if constexpr (RING) {
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    cp_async_16(&sh.ring[warp][slot][u][lane], kq + u * ustep);
                    cp_async_16(&sh.ring[warp][slot][U + u][lane], vq + u * ustep);
                }
                asm volatile("cp.async.commit_group;" ::: "memory");
            }
        };
        if (RING && warp < nchunks) stage_in(kp, vp, 0);
        int ri = 0;
        for (int c = warp; c < nchunks; c += kDecWarps, kp += cstep, vp += cstep) {
            float4 kk[U], vv[U];
            if constexpr (RING) {
                if (c + kDecWarps < nchunks) {
                    stage_in(kp + cstep, vp + cstep, (ri + 1) & 1);
                    asm volatile("cp.async.wait_group 1;" ::: "memory");
                } else {
                    asm volatile("cp.async.wait_group 0;" ::: "memory");
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    kk[u] = sh.ring[warp][ri & 1][u][lane];
                    vv[u] = sh.ring[warp][ri & 1][U + u][lane];
                }
                ++ri;
            } else {
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    kk[u] = ld4(kp + u * ustep);
                    vv[u] = ld4(vp + u * ustep);
                }
            }
            float s[V];
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int q = 0; q < NQ; ++q) s[u * NQ + q] = dot4(qv[q], kk[u]);
            lane_group_transpose_reduce<V, LPK / 2>(s, lane);
            float sv = s[0];
            if (!finite_f(sv)) sv = -INFINITY;
            // m_own is the reference the exponentials are taken against. It follows the running
            // maximum only when a score is more than 2^8 above it (or at the first finite score), so
            // the common chunk needs neither the row-maximum butterfly nor the rescale of the
            // accumulators -- one warp vote instead -- and the probabilities stay below 2^8.
            // l_own sums this lane's own probabilities only (the lanes of a query row share its
            // reference, so their sums are added once, after the loop).
            float mn = m_own;
            if (__any_sync(0xffffffffu, sv > m_own + 8.0f || (m_own == -INFINITY && sv > -INFINITY))) {
                float cmax = sv;
#pragma unroll
                for (int o = NQ * REP; o < LPK; o <<= 1) cmax = fmaxf(cmax, __shfl_xor_sync(0xffffffffu, cmax, o));
                const bool move = cmax > m_own + 8.0f || m_own == -INFINITY;
                mn = move ? cmax : m_own;
                const float corr_own = move ? fast_exp2(m_own - (mn == -INFINITY ? 0.0f : mn)) : 1.0f;
                l_own *= corr_own;
#pragma unroll
                for (int q = 0; q < NQ; ++q) scale4(acc[q], __shfl_sync(0xffffffffu, corr_own, q * REP, LPK));
            }
            const float pe_own = fast_exp2(sv - (mn == -INFINITY ? 0.0f : mn));
            l_own += pe_own;
            m_own = mn;
#pragma unroll
            for (int q = 0; q < NQ; ++q) {
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const float pe = __shfl_sync(0xffffffffu, pe_own, (u * NQ + q) * REP, LPK);
                    fma4(acc[q], pe, vv[u]);
                }
            }
        }
#pragma unroll
        for (int o = NQ * REP; o < LPK; o <<= 1) l_own += __shfl_xor_sync(0xffffffffu, l_own, o);
        // hand the per-row state to every lane of the group for the code below
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
            m[q] = __shfl_sync(0xffffffffu, m_own, q * REP, LPK);
            l[q] = __shfl_sync(0xffffffffu, l_own, q * REP, LPK);
        }
        (void)q_own;
    }

    // ---- checked keys: window edge, chunk remainder, appended rows --------
    {
        const int iters = (nslow + kDecWarps * KPW - 1) / (kDecWarps * KPW);
        for (int it = 0; it < iters; ++it) {
            const int t = it * (kDecWarps * KPW) + warp * KPW + grp;
            const bool live = t < nslow;
            const int j = t < head_slow ? k0 + t : Fe + (t - head_slow);
            float4 kk = make_float4(0.f, 0.f, 0.f, 0.f), vv = kk;
            if (live) {
                if (p.kn && j >= base) {
                    const int64_t off = (int64_t)(b * n + (j - base)) * p.new_stride + hoff;
                    kk = ld4(p.kn + off);
                    vv = ld4(p.vn + off);
                    if (p.rope_cos) kk = rope_pairs(kk, p.rope_cos, p.rope_sin, j, HD / 2, dl * 2);
                } else {
                    const int64_t off = (int64_t)j * p.row_stride;
                    kk = ld4(kc + off);
                    vv = ld4(vc + off);
                }
            }
            float s[NQ];
#pragma unroll
            for (int q = 0; q < NQ; ++q) s[q] = dot4(qv[q], kk);
#pragma unroll
            for (int o = LPK / 2; o > 0; o >>= 1)
#pragma unroll
                for (int q = 0; q < NQ; ++q) s[q] += __shfl_xor_sync(0xffffffffu, s[q], o);
#pragma unroll
            for (int q = 0; q < NQ; ++q) {
                const bool vis = live && j >= lo_r[q] && j < hi_r[q] && finite_f(s[q]);
                const float sv = vis ? s[q] : -INFINITY;
                const float mn = fmaxf(m[q], sv);
                const float mref = mn == -INFINITY ? 0.0f : mn;
                const float corr = exp2f(m[q] - mref);
                const float pe = exp2f(sv - mref);
                l[q] = l[q] * corr + pe;
                scale4(acc[q], corr);
                // a key the row does not see contributes nothing, whatever its value row holds
                // (the reference skips zero weights, ops/attn_core_cpu.c:48)
                fma4(acc[q], pe, vis ? vv : make_float4(0.f, 0.f, 0.f, 0.f));
                m[q] = mn;
            }
        }
    }

    // ---- merge lane groups of the warp -------------------------------------
#pragma unroll
    for (int o = LPK; o < 32; o <<= 1) {
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
            const float mo = __shfl_xor_sync(0xffffffffu, m[q], o);
            const float lo2 = __shfl_xor_sync(0xffffffffu, l[q], o);
            float4 ao;
            ao.x = __shfl_xor_sync(0xffffffffu, acc[q].x, o);
            ao.y = __shfl_xor_sync(0xffffffffu, acc[q].y, o);
            ao.z = __shfl_xor_sync(0xffffffffu, acc[q].z, o);
            ao.w = __shfl_xor_sync(0xffffffffu, acc[q].w, o);
            const float mn = fmaxf(m[q], mo);
            const float mref = mn == -INFINITY ? 0.0f : mn;
            const float ca = exp2f(m[q] - mref), cb = exp2f(mo - mref);
            l[q] = l[q] * ca + lo2 * cb;
            acc[q].x = acc[q].x * ca + ao.x * cb;
            acc[q].y = acc[q].y * ca + ao.y * cb;
            acc[q].z = acc[q].z * ca + ao.z * cb;
            acc[q].w = acc[q].w * ca + ao.w * cb;
            m[q] = mn;
        }
    }

    // ---- merge warps through shared memory ---------------------------------
    auto &sm_acc = sh.acc;
    auto &sm_m = sh.m;
    auto &sm_l = sh.l;
    if (grp == 0) {
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
            sm_acc[warp][q][dl] = acc[q];
            if (dl == 0) {
                sm_m[warp][q] = m[q];
                sm_l[warp][q] = l[q];
            }
        }
    }
    __syncthreads();
    for (int t = tid; t < NQ * LPK; t += kDecThreads) {
        const int q = t / LPK, c = t - q * LPK;
        if (q >= nv) continue;
        float M = sm_m[0][q];
#pragma unroll
        for (int w = 1; w < kDecWarps; ++w) M = fmaxf(M, sm_m[w][q]);
        const float mref = M == -INFINITY ? 0.0f : M;
        float L = 0.0f;
        float4 A = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < kDecWarps; ++w) {
            const float cw = exp2f(sm_m[w][q] - mref);
            L += sm_l[w][q] * cw;
            fma4(A, cw, sm_acc[w][q][c]);
        }
        const int r = r0 + q;
        if (direct) {
            float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
            if (L > 0.0f) o = make_float4(A.x / L, A.y / L, A.z / L, A.w / L);
            *reinterpret_cast<float4 *>(p.out + (int64_t)(b * n + r) * p.out_stride + (int64_t)h * HD + c * 4) = o;
        } else {
            float *w = wdst + (int64_t)q * wrow;
            *reinterpret_cast<float4 *>(w + c * 4) = A;
            if (c == 0) {
                w[HD] = M;
                w[HD + 1] = L;
            }
        }
    }

    // ---- write-through of the appended rows --------------------------------
    if (write_through) {
        for (int t = tid; t < n * LPK; t += kDecThreads) {
            const int row = t / LPK, c = t - row * LPK;
            const int64_t src = (int64_t)(b * n + row) * p.new_stride + (int64_t)h * HD + c * 4;
            const int64_t dst = (int64_t)b * p.seq_stride + (int64_t)(base + row) * p.row_stride + (int64_t)h * HD + c * 4;
            float4 knew = ld4(p.kn + src);
            if (p.rope_cos) knew = rope_pairs(knew, p.rope_cos, p.rope_sin, base + row, HD / 2, c * 2);
            *reinterpret_cast<float4 *>(p.kc + dst) = knew;
            *reinterpret_cast<float4 *>(p.vc + dst) = ld4(p.vn + src);
        }
    }
}

template <int HD, int NQ>
__host__ __device__ constexpr int dec_chunk_keys() { // keys per warp per chunk of the unmasked stream (CH above)
    constexpr int LPK = HD / 4, KPW = 32 / LPK;
    return KPW * dec_chunk_u<HD, NQ>();
}

// Grid form: CTA = (head, key-range split, sequence x query group).
template <int HD, int NQ>
__global__ void __launch_bounds__(kDecThreads) decode_attn_kernel(DecodeParams p) {
    constexpr int CH = dec_chunk_keys<HD, NQ>();
    constexpr bool RING = dec_ring_ok<HD, NQ>();
    __shared__ DecShared<HD, NQ, RING> sh;
    const int h = blockIdx.x, sp = blockIdx.y;
    const int b = blockIdx.z / p.qgroups, qg = blockIdx.z - b * p.qgroups;
    const int base = p.base_len[b] + p.base_add;
    const int r0 = qg * NQ, nv = min(NQ, p.n_new - r0);
    int lo_min, hi_max;
    dec_group_range(p, base, r0, nv, lo_min, hi_max);
    // this CTA's share of [lo_min, hi_max)
    const int span = hi_max - lo_min;
    const int per = ((span + p.splits - 1) / p.splits + CH - 1) / CH * CH;
    const int k0 = min(hi_max, lo_min + sp * per);
    const int k1 = min(hi_max, k0 + per);
    float *w = p.ws + ((((int64_t)b * p.H + h) * p.n_new + r0) * p.splits + sp) * dec_partial_floats<HD>();
    decode_piece<HD, NQ, RING>(p, sh, b, h, qg, base, k0, k1, p.splits == 1, w, (int64_t)p.splits * dec_partial_floats<HD>(),
                         p.kn != nullptr && sp == p.splits - 1 && qg == 0);
}

// ---------------------------------------------------------------------------
// Stream form: a persistent grid, one CTA per resident slot of the GPU, over the
// linearised (sequence, query group, head, key block) space. Every CTA takes an
// equal, contiguous share of that space, so all of them stream about the same
// number of cache rows and finish together whatever the per-sequence lengths and
// however the unit count divides by the number of slots; a share may begin and
// end inside a unit, and such pieces leave (acc, m, l) partials that a second
// small launch merges. The lengths live in device memory, so every CTA derives
// the partition itself from a prefix sum over the sequences (shared memory).
// No CTA waits for another one anywhere.
// ---------------------------------------------------------------------------
constexpr int kPieceValid = 4, kPieceHead = 1, kPieceTail = 2;
struct DecStreamLayout { // workspace: [2 * G piece descriptors (unit, flags)] [2 * G * NQ partials]
    int2 *desc;
    float *part;
};
__host__ __device__ inline size_t dec_stream_desc_bytes(int G) { return ((size_t)G * 2 * sizeof(int2) + 255) & ~(size_t)255; }

// Key blocks of sequence b: the union of its query groups' ranges cut into pieces of `A` keys.
__device__ __forceinline__ void dec_seq_span(const DecodeParams &p, int base, int &lo_u, int &hi_u) {
    hi_u = base + p.n_new;
    lo_u = (p.window > 0 && !p.block_mode) ? max(0, base + 1 - p.window) : 0;
}

template <int HD, int NQ>
__global__ void __launch_bounds__(kDecThreads, NQ <= 4 ? 5 : 3) decode_stream_kernel(DecodeParams p, int2 *desc, float *part) {
    constexpr int A = dec_chunk_keys<HD, NQ>() * kDecWarps; // keys per block: one chunk for every warp
    constexpr int PF = dec_partial_floats<HD>();
    extern __shared__ int s_pref[]; // [batch + 1]: blocks before sequence b
    __shared__ DecShared<HD, NQ, false> sh; // no ring here: the prefix sum already takes the dynamic shared memory
    __shared__ int s_warp_sum[kDecWarps];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int units_per_seq = p.H * p.qgroups;

    // ---- prefix sum of the sequences' block counts ------------------------------
    {
        const int per_thread = (p.batch + kDecThreads - 1) / kDecThreads;
        const int b0 = tid * per_thread, b1 = min(p.batch, b0 + per_thread);
        int local = 0;
        for (int b = b0; b < b1; ++b) {
            int lo_u, hi_u;
            dec_seq_span(p, p.base_len[b] + p.base_add, lo_u, hi_u);
            const int nb = (hi_u - lo_u + A - 1) / A;
            s_pref[b] = local; // exclusive, within this thread's run
            local += nb * units_per_seq;
        }
        int incl = local;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += t;
        }
        if (lane == 31) s_warp_sum[warp] = incl;
        __syncthreads();
        int before = incl - local;
        for (int w = 0; w < warp; ++w) before += s_warp_sum[w];
        for (int b = b0; b < b1; ++b) s_pref[b] += before;
        if (tid == kDecThreads - 1) s_pref[p.batch] = before + local;
        __syncthreads();
    }
    const int64_t T = s_pref[p.batch];
    const int G = gridDim.x, g = blockIdx.x;
    int x = (int)(T * g / G);
    const int x_end = (int)(T * (g + 1) / G);
    if (tid == 0) {
        desc[g * 2] = make_int2(0, 0);
        desc[g * 2 + 1] = make_int2(0, 0);
    }
    bool first = true;
    int b = 0;
    while (x < x_end) {
        // sequence holding block x: s_pref[b] <= x < s_pref[b + 1] (pieces ascend, so does b)
        {
            int lo = b, hi = p.batch;
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (s_pref[mid] <= x) lo = mid;
                else hi = mid;
            }
            b = lo;
        }
        const int base = p.base_len[b] + p.base_add;
        int lo_u, hi_u;
        dec_seq_span(p, base, lo_u, hi_u);
        const int nb = (hi_u - lo_u + A - 1) / A;
        const int local = x - s_pref[b];
        const int ul = local / nb, blk0 = local - ul * nb;
        const int blk1 = min(nb, blk0 + (x_end - x));
        const int qg = ul / p.H, h = ul - qg * p.H;
        const int r0 = qg * NQ, nv = min(NQ, p.n_new - r0);
        int lo_min, hi_max;
        dec_group_range(p, base, r0, nv, lo_min, hi_max);
        int k0 = max(lo_min, lo_u + blk0 * A);
        int k1 = min(hi_max, lo_u + blk1 * A);
        if (k1 < k0) k1 = k0; // a block outside this group's own range: an empty piece
        const bool head = blk0 == 0, tail = blk1 == nb, whole = head && tail;
        const int slot = g * 2 + (first ? 0 : 1);
        if (!whole && tid == 0)
            desc[slot] = make_int2(b * units_per_seq + ul, kPieceValid | (head ? kPieceHead : 0) | (tail ? kPieceTail : 0));
        decode_piece<HD, NQ, false>(p, sh, b, h, qg, base, k0, k1, whole, part + (int64_t)slot * NQ * PF, PF,
                             p.kn != nullptr && tail && qg == 0);
        __syncthreads(); // the warps' shared state is reused by the next piece
        x += blk1 - blk0;
        first = false;
    }
}

// The CTA after gg that holds the next piece of `unit` (its first slot): CTAs whose share was empty
// (more CTAs than blocks) wrote no descriptor and are stepped over.
__device__ __forceinline__ bool next_piece(const int2 *desc, int G, int unit, int &gg) {
    for (++gg; gg < G; ++gg) {
        const int2 d = desc[gg * 2];
        if (!(d.y & kPieceValid)) continue;
        return d.x == unit && !(d.y & kPieceHead);
    }
    return false;
}

// Merge pass of the stream form: CTA g owns the unit whose first piece is g's last piece (or its
// only one) when that unit continues into the following CTAs; the continuation pieces are the
// first pieces of g + 1, g + 2, ... up to the one flagged as the unit's end.
template <int HD, int NQ>
__global__ void __launch_bounds__(128) decode_stream_merge_kernel(DecodeParams p, const int2 *desc, const float *part) {
    constexpr int LPK = HD / 4, PF = dec_partial_floats<HD>();
    const int g = blockIdx.x, G = gridDim.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int own = -1;
#pragma unroll
    for (int s = 0; s < 2; ++s) {
        const int2 d = desc[g * 2 + s];
        if ((d.y & kPieceValid) && (d.y & kPieceHead) && !(d.y & kPieceTail)) own = s;
    }
    if (own < 0) return;
    const int unit = desc[g * 2 + own].x;
    const int units_per_seq = p.H * p.qgroups;
    const int b = unit / units_per_seq, ul = unit - b * units_per_seq;
    const int qg = ul / p.H, h = ul - qg * p.H;
    const int nv = min(NQ, p.n_new - qg * NQ);
    for (int q = warp; q < nv; q += 4) {
        // pass 1: the row maximum over the pieces; pass 2: the weighted sums
        float M = -INFINITY;
        {
            int gg = g, s = own;
            while (true) {
                M = fmaxf(M, part[((int64_t)(gg * 2 + s) * NQ + q) * PF + HD]);
                if (desc[gg * 2 + s].y & kPieceTail) break;
                if (!next_piece(desc, G, unit, gg)) break;
                s = 0;
            }
        }
        const float mref = M == -INFINITY ? 0.0f : M;
        if (lane < LPK) {
            float L = 0.0f;
            float4 Acc = make_float4(0.f, 0.f, 0.f, 0.f);
            int gg = g, s = own;
            while (true) {
                const float *w = part + ((int64_t)(gg * 2 + s) * NQ + q) * PF;
                const float cw = exp2f(w[HD] - mref);
                L += w[HD + 1] * cw;
                fma4(Acc, cw, *reinterpret_cast<const float4 *>(w + lane * 4));
                if (desc[gg * 2 + s].y & kPieceTail) break;
                if (!next_piece(desc, G, unit, gg)) break;
                s = 0;
            }
            float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
            if (L > 0.0f) o = make_float4(Acc.x / L, Acc.y / L, Acc.z / L, Acc.w / L);
            *reinterpret_cast<float4 *>(p.out + (int64_t)(b * p.n_new + qg * NQ + q) * p.out_stride + (int64_t)h * HD + lane * 4) = o;
        }
    }
}

// One warp per (sequence, head, query row): merges the split partials.
template <int HD>
__global__ void __launch_bounds__(128) decode_combine_kernel(DecodeParams p) {
    constexpr int LPK = HD / 4;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t unit = (int64_t)blockIdx.x * 4 + warp;
    const int64_t units = (int64_t)p.batch * p.H * p.n_new;
    if (unit >= units) return;
    const int r = (int)(unit % p.n_new);
    const int h = (int)((unit / p.n_new) % p.H);
    const int b = (int)(unit / ((int64_t)p.n_new * p.H));
    const float *w0 = p.ws + unit * p.splits * dec_partial_floats<HD>();
    float M = -INFINITY;
    for (int s = 0; s < p.splits; ++s) M = fmaxf(M, w0[(int64_t)s * dec_partial_floats<HD>() + HD]);
    const float mref = M == -INFINITY ? 0.0f : M;
    if (lane < LPK) {
        float L = 0.0f;
        float4 A = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s = 0; s < p.splits; ++s) {
            const float *w = w0 + (int64_t)s * dec_partial_floats<HD>();
            const float cw = exp2f(w[HD] - mref);
            L += w[HD + 1] * cw;
            fma4(A, cw, *reinterpret_cast<const float4 *>(w + lane * 4));
        }
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
        if (L > 0.0f) o = make_float4(A.x / L, A.y / L, A.z / L, A.w / L);
        *reinterpret_cast<float4 *>(p.out + (int64_t)(b * p.n_new + r) * p.out_stride + (int64_t)h * HD + lane * 4) = o;
    }
}

static int pick_nq(int n_new) { return n_new <= 1 ? 1 : (n_new <= 2 ? 2 : (n_new <= 4 ? 4 : 8)); }

static int resolve_splits(const fblt_decode_desc *d) {
    if (d->splits > 0) return d->splits > 64 ? 64 : d->splits;
    const int nq = pick_nq(d->n_new);
    const int qgroups = (d->n_new + nq - 1) / nq;
    const int64_t ctas = (int64_t)d->batch * d->num_heads * qgroups;
    const int64_t target = 148 * 6;
    if (ctas >= target) return 1;
    int64_t s = (target + ctas - 1) / ctas;
    const int64_t cap = d->max_len / 128 > 1 ? d->max_len / 128 : 1;
    if (s > cap) s = cap;
    if (s > 64) s = 64;
    return (int)s;
}

static size_t partial_floats(int hd) { return (size_t)hd + 4; }

static int validate_decode(const fblt_decode_desc *d) {
    if (!d) return fail(FBLT_ERR_ARG, "decode: NULL descriptor");
    if (d->batch < 0 || d->num_heads <= 0) return fail(FBLT_ERR_ARG, "decode: bad batch/heads");
    if (d->head_dim != 32 && d->head_dim != 64 && d->head_dim != 128)
        return fail(FBLT_ERR_UNSUPPORTED, "decode: head_dim %d (32, 64 or 128)", d->head_dim);
    if (d->n_new < 1 || d->n_new > 32) return fail(FBLT_ERR_UNSUPPORTED, "decode: n_new %d outside 1..32", d->n_new);
    if (!d->base_len || !d->k_cache || !d->v_cache || !d->q || !d->out)
        return fail(FBLT_ERR_ARG, "decode: NULL buffer");
    if ((d->k_new == nullptr) != (d->v_new == nullptr)) return fail(FBLT_ERR_ARG, "decode: k_new and v_new go together");
    if ((d->rope_cos == nullptr) != (d->rope_sin == nullptr)) return fail(FBLT_ERR_ARG, "decode: rope_cos and rope_sin go together");
    if (d->rope_cos && !d->k_new) return fail(FBLT_ERR_ARG, "decode: rotary tables need k_new / v_new (rows still unrotated)");
    if (((uintptr_t)d->rope_cos | (uintptr_t)d->rope_sin) & 7) return fail(FBLT_ERR_ARG, "decode: rotary tables must be 8-byte aligned");
    const int64_t E = (int64_t)d->num_heads * d->head_dim;
    if (d->cache_row_stride < E || d->q_stride < E || d->out_stride < E || (d->k_new && d->kv_new_stride < E))
        return fail(FBLT_ERR_ARG, "decode: row stride smaller than num_heads*head_dim");
    if ((d->cache_row_stride | d->cache_seq_stride | d->q_stride | d->out_stride | (d->k_new ? d->kv_new_stride : 0)) & 3)
        return fail(FBLT_ERR_ARG, "decode: strides must be multiples of 4 elements");
    const uintptr_t ptrs = (uintptr_t)d->k_cache | (uintptr_t)d->v_cache | (uintptr_t)d->q | (uintptr_t)d->out |
                           (uintptr_t)d->k_new | (uintptr_t)d->v_new;
    if (ptrs & 15) return fail(FBLT_ERR_ARG, "decode: buffers must be 16-byte aligned");
    const int nq = pick_nq(d->n_new);
    if ((int64_t)d->batch * ((d->n_new + nq - 1) / nq) > 65535 || d->num_heads > 65535)
        return fail(FBLT_ERR_LIMIT, "decode: batch * query groups (or heads) exceed 65535 per launch");
    return FBLT_OK;
}

// ---- launch plan: grid form or stream form ---------------------------------------
struct DecodePlan {
    bool stream;  // persistent grid over equal shares of the key-block space
    int grid;     // stream form: number of CTAs
    int splits;   // grid form: key-range pieces per unit
    size_t need;  // bytes of scratch for partials (and, stream form, piece descriptors)
};

constexpr int kStreamMaxBatch = 8192; // the per-sequence prefix sum sits in shared memory

template <int HD, int NQ>
static int stream_slots_t(int *slots) {
    static std::atomic<int> cache[64]; // resident CTAs of this instantiation per device ordinal, 0 = not asked yet
    int dev = 0;
    FBLT_CUDA_TRY(cudaGetDevice(&dev));
    int v = dev < 64 ? cache[dev].load(std::memory_order_relaxed) : 0;
    if (!v) {
        int per_sm = 0, sms = 0;
        FBLT_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_stream_kernel<HD, NQ>, kDecThreads,
                                                                    (kStreamMaxBatch + 1) * sizeof(int)));
        FBLT_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        v = per_sm * sms;
        if (v < 1) return fail(FBLT_ERR_CUDA, "decode: the stream kernel does not fit an SM");
        if (dev < 64) cache[dev].store(v, std::memory_order_relaxed);
    }
    *slots = v;
    return FBLT_OK;
}

static int stream_slots(int hd, int nq, int *slots) {
#define FBLT_SLOTS(HD)                                                  \
    switch (nq) {                                                       \
    case 1: return stream_slots_t<HD, 1>(slots);                        \
    case 2: return stream_slots_t<HD, 2>(slots);                        \
    case 4: return stream_slots_t<HD, 4>(slots);                        \
    default: return stream_slots_t<HD, 8>(slots);                       \
    }
    switch (hd) {
    case 32: FBLT_SLOTS(32)
    case 64: FBLT_SLOTS(64)
    default: FBLT_SLOTS(128)
    }
#undef FBLT_SLOTS
}

static int chunk_keys(int hd, int nq) { // dec_chunk_keys<HD, NQ>() for run-time values
    const int lpk = hd / 4, kpw = 32 / lpk;
    int u = lpk / nq;
    u = u > kDecMaxU ? kDecMaxU : (u < 1 ? 1 : u);
    return kpw * u;
}

// splits > 0: the grid form with that many pieces. splits == 0: the library chooses -- the grid form with
// a split count from the launch width, which is the faster of the two on every measured shape (it keeps
// the CTAs that run together on neighbouring heads of the same cache rows); FBLT_DECODE_MODE=stream in
// the environment selects the stream form instead. splits < 0: the stream form or an error.
static int make_plan(const fblt_decode_desc *d, bool allow_stream, DecodePlan *plan) {
    const int nq = pick_nq(d->n_new);
    const int qgroups = (d->n_new + nq - 1) / nq;
    plan->stream = false;
    plan->grid = 0;
    bool want = allow_stream && d->splits < 0;
    if (allow_stream && d->splits == 0) {
        const char *e = getenv("FBLT_DECODE_MODE");
        if (e && !strcmp(e, "stream")) want = true;
    }
    const int A = chunk_keys(d->head_dim, nq) * kDecWarps;
    const int64_t max_blocks = (int64_t)d->batch * d->num_heads * qgroups * ((d->max_len > 0 ? d->max_len : 0) / A + 1);
    const bool fits = d->batch <= kStreamMaxBatch && d->max_len > 0 && max_blocks < (int64_t)1 << 30;
    if (want && fits) {
        int slots = 0;
        const int st = stream_slots(d->head_dim, nq, &slots);
        if (st != FBLT_OK) return st;
        // no more CTAs than there are shares of a few blocks each
        int64_t g = max_blocks / 4;
        if (g < 1) g = 1;
        if (g > slots) g = slots;
        plan->stream = true;
        plan->grid = (int)g;
        plan->splits = 1;
        plan->need = dec_stream_desc_bytes(plan->grid) + (size_t)plan->grid * 2 * nq * partial_floats(d->head_dim) * sizeof(float);
        return FBLT_OK;
    }
    if (d->splits < 0) return fail(FBLT_ERR_UNSUPPORTED, "decode: the stream form needs batch <= %d and max_len set", kStreamMaxBatch);
    plan->splits = resolve_splits(d);
    plan->need = plan->splits <= 1 ? 0
                                   : (size_t)d->batch * d->num_heads * d->n_new * plan->splits * partial_floats(d->head_dim) * sizeof(float);
    return FBLT_OK;
}

template <int HD, int NQ>
static int launch_decode_t(const DecodeParams &p, const DecodePlan &plan, cudaStream_t stream) {
    if (plan.stream) {
        int2 *desc = reinterpret_cast<int2 *>(p.ws);
        float *part = reinterpret_cast<float *>(reinterpret_cast<char *>(p.ws) + dec_stream_desc_bytes(plan.grid));
        decode_stream_kernel<HD, NQ><<<plan.grid, kDecThreads, (p.batch + 1) * sizeof(int), stream>>>(p, desc, part);
        count_launch();
        int st = check_launch("decode_stream_kernel");
        if (st != FBLT_OK) return st;
        decode_stream_merge_kernel<HD, NQ><<<plan.grid, 128, 0, stream>>>(p, desc, part);
        count_launch();
        return check_launch("decode_stream_merge_kernel");
    }
    dim3 grid(p.H, p.splits, p.batch * p.qgroups);
    decode_attn_kernel<HD, NQ><<<grid, kDecThreads, 0, stream>>>(p);
    count_launch();
    int st = check_launch("decode_attn_kernel");
    if (st != FBLT_OK) return st;
    if (p.splits > 1) {
        const int64_t units = (int64_t)p.batch * p.H * p.n_new;
        decode_combine_kernel<HD><<<(unsigned)((units + 3) / 4), 128, 0, stream>>>(p);
        count_launch();
        st = check_launch("decode_combine_kernel");
    }
    return st;
}

template <int HD>
static int launch_decode_hd(const DecodeParams &p, const DecodePlan &plan, int nq, cudaStream_t stream) {
    switch (nq) {
    case 1: return launch_decode_t<HD, 1>(p, plan, stream);
    case 2: return launch_decode_t<HD, 2>(p, plan, stream);
    case 4: return launch_decode_t<HD, 4>(p, plan, stream);
    default: return launch_decode_t<HD, 8>(p, plan, stream);
    }
}

// The one place a descriptor becomes kernel parameters; both entry points go through it.
static DecodeParams fill_decode_params(const fblt_decode_desc *d, const DecodePlan &plan, float *scratch) {
    DecodeParams p;
    p.batch = d->batch;
    p.H = d->num_heads;
    p.n_new = d->n_new;
    p.block_mode = d->block_mode ? 1 : 0;
    p.window = d->window > 0 ? d->window : 0;
    p.splits = plan.splits;
    const int nq = pick_nq(d->n_new);
    p.qgroups = (d->n_new + nq - 1) / nq;
    p.base_len = d->base_len;
    p.base_add = d->base_add;
    p.kc = d->k_cache;
    p.vc = d->v_cache;
    p.seq_stride = d->cache_seq_stride;
    p.row_stride = d->cache_row_stride;
    p.q = d->q;
    p.q_stride = d->q_stride;
    p.kn = d->k_new;
    p.vn = d->v_new;
    p.new_stride = d->kv_new_stride;
    p.out = d->out;
    p.out_stride = d->out_stride;
    p.ws = scratch;
    p.qscale = d->scale * kLog2e;
    p.rope_cos = d->rope_cos;
    p.rope_sin = d->rope_sin;
    return p;
}

static int launch_decode(const fblt_decode_desc *d, const DecodeParams &p, const DecodePlan &plan, cudaStream_t s) {
    const int nq = pick_nq(d->n_new);
    switch (d->head_dim) {
    case 32: return launch_decode_hd<32>(p, plan, nq, s);
    case 64: return launch_decode_hd<64>(p, plan, nq, s);
    default: return launch_decode_hd<128>(p, plan, nq, s);
    }
}

} // namespace fblt

extern "C" size_t fblt_attn_decode_workspace(const fblt_decode_desc *d) {
    if (!d || d->batch <= 0 || fblt::validate_decode(d) != FBLT_OK) return 0;
    fblt::DecodePlan plan;
    if (fblt::make_plan(d, true, &plan) != FBLT_OK) return 0;
    return plan.need;
}

extern "C" int fblt_attn_decode(const fblt_decode_desc *d, void *workspace, size_t workspace_bytes, void *stream) {
    fblt::NvtxRange nvtx_range("fblt_attn_decode");
    using namespace fblt;
    int st = validate_decode(d);
    if (st != FBLT_OK) return st;
    if (d->batch == 0) return FBLT_OK;
    DecodePlan plan;
    st = make_plan(d, true, &plan);
    if (st != FBLT_OK) return st;
    if (plan.need > 0) {
        if (!workspace || workspace_bytes < plan.need)
            return fail(FBLT_ERR_WORKSPACE, "decode: %zu bytes of workspace needed (fblt_attn_decode_workspace), got %zu",
                        plan.need, workspace_bytes);
        if ((uintptr_t)workspace & 15) return fail(FBLT_ERR_ARG, "decode: workspace must be 16-byte aligned");
    }
    const DecodeParams p = fill_decode_params(d, plan, (float *)workspace);
    return launch_decode(d, p, plan, (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------
// Allocation-free variant: split-K partials in a fixed device array.
// ---------------------------------------------------------------------------
namespace fblt {

// 4 MiB of partials, resident on every device that loads this library until
// the process exits.
constexpr size_t kStaticScratchBytes = (size_t)4 << 20;
static __device__ __align__(256) float g_decode_static_scratch[kStaticScratchBytes / sizeof(float)];

constexpr int kMaxDevices = 64;
// device address per device ordinal, null = not looked up yet; any host thread may read or fill a slot
static std::atomic<float *> g_static_scratch_addr[kMaxDevices];

// In host code `g_decode_static_scratch` is only a handle for the symbol; the
// address a kernel can dereference has to be asked for, once per device, with
// that device current.
static int static_scratch_address(float **out) {
    int dev = -1;
    FBLT_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(FBLT_ERR_LIMIT, "decode_static: device ordinal %d not supported", dev);
    float *p = g_static_scratch_addr[dev].load(std::memory_order_relaxed);
    if (!p) {
        void *addr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&addr, g_decode_static_scratch);
        if (e != cudaSuccess || !addr)
            return fail(FBLT_ERR_CUDA, "decode_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        p = static_cast<float *>(addr);
        g_static_scratch_addr[dev].store(p, std::memory_order_relaxed); // same value whichever thread gets here first
    }
    *out = p;
    return FBLT_OK;
}

} // namespace fblt

extern "C" size_t fblt_attn_decode_static_capacity(void) { return fblt::kStaticScratchBytes; }

extern "C" int fblt_attn_decode_static(const fblt_decode_desc *d, void *stream) {
    fblt::NvtxRange nvtx_range("fblt_attn_decode_static");
    using namespace fblt;
    int st = validate_decode(d);
    if (st != FBLT_OK) return st;
    if (d->batch == 0) return FBLT_OK;
    DecodePlan plan;
    st = make_plan(d, true, &plan);
    if (st != FBLT_OK) return st;
    if (plan.stream && plan.need > kStaticScratchBytes && d->splits == 0) { // stream form chosen by the environment
        st = make_plan(d, false, &plan); // the grid form may need less
        if (st != FBLT_OK) return st;
    }
    if (plan.need > kStaticScratchBytes)
        return fail(FBLT_ERR_LIMIT,
                    "decode_static: this call needs %zu bytes of partials; the built-in scratch holds %zu "
                    "(use fblt_attn_decode with a caller workspace, or set splits = 1)",
                    plan.need, kStaticScratchBytes);
    float *scratch = nullptr;
    st = static_scratch_address(&scratch);
    if (st != FBLT_OK) return st;
    // every slot the merge kernels read is written by the launch before them: nothing to clear
    const DecodeParams p = fill_decode_params(d, plan, scratch);
    return launch_decode(d, p, plan, (cudaStream_t)stream);
}
