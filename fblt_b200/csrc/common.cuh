// Shared pieces of the sm_100a attention library: status/error plumbing,
// launch accounting, and the on-the-fly mask rule evaluated from the patcher's
// boundary array (no dense mask is ever read by the batched kernels).
#pragma once

#include <cuda_runtime.h>
#include <math.h>
#include <nvtx3/nvToolsExt.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/fblt_attn.h"

namespace fblt {

// ---- host-side status -----------------------------------------------------
int fail(int status, const char *fmt, ...);
void count_launch(int n = 1);

// NVTX range over a host entry point, so that a timeline or an ncu --nvtx filter shows which
// library call a launch belongs to (the reference ships no ranges, docs/PROFILING.md:60-61).
// Header-only NVTX: without a tool attached a push / pop is a load and a branch.
struct NvtxRange {
    explicit NvtxRange(const char *name) { nvtxRangePushA(name); }
    ~NvtxRange() { nvtxRangePop(); }
    NvtxRange(const NvtxRange &) = delete;
    NvtxRange &operator=(const NvtxRange &) = delete;
};
int check_launch(const char *what);

#define FBLT_CUDA_TRY(expr)                                                                \
    do {                                                                                   \
        cudaError_t e__ = (expr);                                                          \
        if (e__ != cudaSuccess)                                                            \
            return ::fblt::fail(FBLT_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e__));  \
    } while (0)

// ---- device-side mask rule -------------------------------------------------

// Mask descriptor resolved for one sequence. Built once per CTA / warp.
struct SeqMask {
    int nq, nk;
    int is_causal, window, group_rule, subtokens, bidir;
    int causal_off;
    int num_clean;         // < 0: absent
    const int32_t *doc;    // boundaries of this sequence
    int ndoc;              // number of boundaries (= num_docs - 1)
    const int32_t *pb;     // patch bounds of this sequence, P + 1 entries
    int P;
    int q_pos_off;
    int trailing_closed;
    const int32_t *qg, *kg; // explicit ids, offset to this sequence's first row
};

__device__ __forceinline__ SeqMask resolve_mask(const fblt_mask_desc &m, int b, int q0, int k0, int nq, int nk) {
    SeqMask s;
    s.nq = nq;
    s.nk = nk;
    s.is_causal = m.is_causal;
    s.window = m.sliding_window;
    s.group_rule = m.group_rule;
    s.subtokens = m.subtokens > 0 ? m.subtokens : 1;
    s.bidir = m.bidirectional_within_group;
    s.causal_off = m.causal_offset ? m.causal_offset[b] : 0;
    s.num_clean = m.num_clean ? m.num_clean[b] : -1;
    if (m.cu_doc && m.doc_bounds) {
        const int d0 = m.cu_doc[b];
        s.doc = m.doc_bounds + d0;
        s.ndoc = m.cu_doc[b + 1] - d0;
    } else {
        s.doc = nullptr;
        s.ndoc = 0;
    }
    if (m.cu_patch && m.patch_bounds) {
        const int p0 = m.cu_patch[b];
        s.pb = m.patch_bounds + p0;
        s.P = m.cu_patch[b + 1] - p0 - 1;
    } else {
        s.pb = nullptr;
        s.P = 0;
    }
    s.q_pos_off = m.q_pos_offset ? m.q_pos_offset[b] : 0;
    s.trailing_closed = m.trailing_closed ? (int)m.trailing_closed[b] : 0;
    s.qg = m.q_group_ids ? m.q_group_ids + q0 : nullptr;
    s.kg = m.k_group_ids ? m.k_group_ids + k0 : nullptr;
    return s;
}

// Number of entries of a[0..n) that are <= x (a ascending): two ways to search.
// ThreadSearch: one thread, binary search (each step waits for the previous load).
struct ThreadSearch {
    __device__ __forceinline__ int count_le(const int32_t *a, int n, int x) const {
        int lo = 0, hi = n;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (a[mid] <= x) lo = mid + 1;
            else hi = mid;
        }
        return lo;
    }
};
// WarpSearch: all 32 lanes of a converged warp ask the same question; every lane tests
// its own entries (coalesced, independent loads) and the votes are counted.
struct WarpSearch {
    int lane;
    __device__ __forceinline__ int count_le(const int32_t *a, int n, int x) const {
        int c = 0;
        for (int base = 0; base < n; base += 32) {
            const int idx = base + lane;
            const bool le = idx < n && a[idx] <= x;
            c += __popc(__ballot_sync(0xffffffffu, le));
        }
        return c;
    }
};
__device__ __forceinline__ int count_le(const int32_t *a, int n, int x) { return ThreadSearch().count_le(a, n, x); }

// Patch that contains byte `pos`, clamped to [0, P-1].
template <class Search = ThreadSearch>
__device__ __forceinline__ int patch_of(const SeqMask &s, int pos, const Search &srch = Search()) {
    int p = srch.count_le(s.pb, s.P + 1, pos) - 1;
    if (p < 0) p = 0;
    if (p > s.P - 1) p = s.P - 1;
    return p;
}

// Decoder latent of byte `pos`: the rule of blt_patch_decoder_latent_at
// (ops/patch_pool_cpu.c:114-131) over a boundary array.
template <class Search = ThreadSearch>
__device__ __forceinline__ int latent_at(const SeqMask &s, int pos, const Search &srch = Search()) {
    if (pos < s.pb[0]) return 0;
    if (pos >= s.pb[s.P]) return s.P - 1;
    const int p = srch.count_le(s.pb, s.P + 1, pos) - 1;
    const bool closes = (pos + 1 == s.pb[p + 1]) && (p + 1 < s.P);
    if (closes) return p;
    return p == 0 ? 0 : p - 1;
}

// Group (patch / latent) a query row belongs to under the PATCH_* rules.
template <class Search = ThreadSearch>
__device__ __forceinline__ int query_group(const SeqMask &s, int i, const Search &srch = Search()) {
    if (s.group_rule == FBLT_GROUP_PATCH_ENC) return i / s.subtokens;
    if (s.group_rule == FBLT_GROUP_PATCH_DEC) {
        // with num_clean (block-diffusion cross-attention, models/block_diffusion.c:164-186): rows past
        // the clean prefix are the drafted block and read the last latent; the prefix ends at num_clean
        if (s.num_clean >= 0 && i >= s.num_clean) return s.P - 1;
        const int last = s.num_clean >= 0 ? s.num_clean - 1 : s.nq - 1;
        if (s.trailing_closed && i == last) return s.P - 1;
        return latent_at(s, s.q_pos_off + i, srch);
    }
    return patch_of(s, s.q_pos_off + i, srch); // PATCH_LEQ
}

// Contiguous key range [lo, hi) a query row may attend to. Valid for every
// rule except explicit group ids, whose equality test stays per key.
template <class Search = ThreadSearch>
__device__ __forceinline__ void row_range(const SeqMask &s, int i, int &lo_out, int &hi_out,
                                          const Search &srch = Search()) {
    int lo = 0, hi = s.nk;
    if (s.num_clean >= 0 && s.group_rule == FBLT_GROUP_NONE) { // block-diffusion INFER self-attention
        if (i < s.num_clean) hi = min(hi, min(s.num_clean, i + 1));
    } else {
        if (s.is_causal) hi = min(hi, i + s.causal_off + 1);
        if (s.window > 0) {
            const int c = s.is_causal ? i + s.causal_off : i;
            lo = max(lo, c - s.window + 1);
            hi = min(hi, c + s.window);
        }
    }
    if (s.ndoc > 0) {
        const int d = srch.count_le(s.doc, s.ndoc, i);
        if (d > 0) lo = max(lo, s.doc[d - 1]);
        if (d < s.ndoc) hi = min(hi, s.doc[d]);
    }
    if (s.group_rule != FBLT_GROUP_NONE && s.group_rule != FBLT_GROUP_IDS) {
        if (s.P <= 0) {
            hi = lo;
        } else {
            const int g = query_group(s, i, srch);
            if (s.group_rule == FBLT_GROUP_PATCH_ENC) {
                if (g < s.P) {
                    lo = max(lo, s.pb[g]);
                    hi = min(hi, s.pb[g + 1]);
                } else {
                    hi = lo;
                }
            } else if (s.group_rule == FBLT_GROUP_PATCH_DEC) {
                lo = max(lo, g * s.subtokens);
                hi = min(hi, (g + 1) * s.subtokens);
            } else {
                hi = min(hi, (g + 1) * s.subtokens);
            }
        }
        if (!s.bidir) hi = min(hi, i + 1);
    }
    if (s.group_rule == FBLT_GROUP_IDS && !s.bidir) hi = min(hi, i + 1);
    if (hi < lo) hi = lo;
    lo_out = lo;
    hi_out = hi;
}

// Pair predicate written independently of row_range(): each clause compares
// the pair directly, the way the reference's dense builder does
// (ops/mask_builder_cpu.c:49-94, :125-135).
__device__ __forceinline__ bool pair_allowed(const SeqMask &s, int i, int j) {
    bool ok = true;
    if (s.num_clean >= 0 && s.group_rule == FBLT_GROUP_NONE) {
        if (i < s.num_clean) ok = (j < s.num_clean) && (j <= i);
    } else {
        if (s.is_causal && j > i + s.causal_off) ok = false;
        if (s.window > 0) {
            const int c = s.is_causal ? i + s.causal_off : i;
            const int dist = c >= j ? c - j : j - c;
            if (dist >= s.window) ok = false;
        }
    }
    if (s.ndoc > 0 && count_le(s.doc, s.ndoc, i) != count_le(s.doc, s.ndoc, j)) ok = false;
    if (s.group_rule != FBLT_GROUP_NONE) {
        bool same;
        if (s.group_rule == FBLT_GROUP_IDS) {
            same = s.qg[i] == s.kg[j];
        } else if (s.P <= 0) {
            same = false;
        } else {
            const int g = query_group(s, i);
            if (s.group_rule == FBLT_GROUP_PATCH_ENC) {
                // key j is a byte; its patch is the one whose bounds contain it
                same = g < s.P && j >= s.pb[g] && j < s.pb[g + 1];
            } else if (s.group_rule == FBLT_GROUP_PATCH_DEC) {
                same = (j / s.subtokens) == g;
            } else {
                same = (j / s.subtokens) <= g;
            }
        }
        if (!same) ok = false;
        else if (!s.bidir && j > i) ok = false;
    }
    return ok;
}

// ---- rotary embedding ------------------------------------------------------------
// One (even, odd) pair: out0 = x0 c - x1 s, out1 = x1 c + x0 s (ops/reductions_cpu.c:217-228).
// Products and sums are rounded separately, as the CPU code does, so rotated values match it.
__device__ __forceinline__ void rope_rotate(float &x0, float &x1, float c, float s) {
    const float a = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
    const float b = __fadd_rn(__fmul_rn(x1, c), __fmul_rn(x0, s));
    x0 = a;
    x1 = b;
}
// The two pairs of a 16-byte piece starting at even column 2 * pair0, for position `pos`.
__device__ __forceinline__ float4 rope_rotate4(float4 x, const float *cs, const float *sn, int pos, int half, int pair0) {
    const float2 c = __ldg(reinterpret_cast<const float2 *>(cs + (int64_t)pos * half + pair0));
    const float2 s = __ldg(reinterpret_cast<const float2 *>(sn + (int64_t)pos * half + pair0));
    rope_rotate(x.x, x.y, c.x, s.x);
    rope_rotate(x.z, x.w, c.y, s.y);
    return x;
}

// ---- small device helpers ---------------------------------------------------

__device__ __forceinline__ bool finite_f(float x) { return fabsf(x) < INFINITY; }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

constexpr float kLog2e = 1.4426950408889634f;

} // namespace fblt
