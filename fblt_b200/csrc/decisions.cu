// Decision step of the speculative / block-diffusion loops: integer and
// comparison logic whose results must equal the reference's host code exactly.
#include "common.cuh"

namespace fblt {

// Strict-'>' scan from index 0 (infer/self_speculation.c:21-31): the lowest
// index among equal maxima wins; a NaN never wins a comparison, and a NaN in
// slot 0 makes every later comparison false, so slot 0 is returned.
__device__ __forceinline__ int warp_argmax_row(const float *x, int vocab, int lane) {
    const float first = x[0];
    float best = -INFINITY;
    int arg = 0x7fffffff;
    for (int v = lane; v < vocab; v += 32) {
        float val = x[v];
        if (val != val) val = -INFINITY;
        if (val > best || arg == 0x7fffffff) { // first element of the lane's slice, or strictly greater
            best = val;
            arg = v;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
        if (ob > best || (ob == best && oa < arg)) {
            best = ob;
            arg = oa;
        }
    }
    return (first != first) ? 0 : arg; // same value in every lane
}

__global__ void __launch_bounds__(128) argmax_rows_kernel(const float *logits, int64_t stride, int rows, int vocab,
                                                          int32_t *ids) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * 4 + warp;
    if (row >= rows) return;
    const int arg = warp_argmax_row(logits + (int64_t)row * stride, vocab, lane);
    if (lane == 0) ids[row] = arg;
}

// Algorithm 2 accept loop (infer/self_speculation.c:158-182), one thread per
// candidate.
__global__ void verify_accept_kernel(uint8_t *x, int64_t x_stride, const int32_t *pred, int64_t pred_stride,
                                     const int32_t *l, const int32_t *r, const int32_t *target_len, int batch,
                                     int32_t *new_len, int32_t *accepted) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= batch) return;
    uint8_t *xc = x + (int64_t)c * x_stride;
    const int32_t *pc = pred + (int64_t)c * pred_stride;
    const int lc = l[c], cand = lc + r[c];
    for (int p = lc; p < cand; ++p) {
        const uint8_t want = (uint8_t)pc[p - 1];
        if (xc[p] != want) {
            xc[p] = want;
            new_len[c] = p + 1;
            if (accepted) accepted[c] = p - lc;
            return;
        }
    }
    if (accepted) accepted[c] = r[c];
    if (cand < target_len[c]) {
        xc[cand] = (uint8_t)pc[cand - 1];
        new_len[c] = cand + 1;
    } else {
        new_len[c] = cand;
    }
}

// One verify-and-commit round for a batch of sequences that decode over a KV cache: the accept loop
// above with the predictions indexed from the first row the verifier computed in this round
// (position row0 = the cache length before the pass), followed by the roll-back of that sequence's
// cache (blt_kv_cache_truncate, infer/kv_cache.c:94-99) to the rows that were computed from bytes
// that stayed: committed length before the round + accepted drafts. One thread per sequence.
__global__ void dv_commit_kernel(uint8_t *x, int64_t x_stride, const int32_t *pred, int width, int32_t *l,
                                 const int32_t *r, const int32_t *target_len, int32_t *cache_len, int32_t *accepted,
                                 int batch) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= batch) return;
    uint8_t *xc = x + (int64_t)c * x_stride;
    const int32_t *pc = pred + (int64_t)c * width; // pc[i]: argmax of the row at position row0 + i, i.e. byte row0 + i + 1
    const int lc = l[c], cand = lc + r[c], row0 = cache_len[c];
    // every byte in [lc, cand] needs the row before it among the computed ones
    if (lc < 1 || r[c] < 0 || lc - 1 < row0 || cand - 1 - row0 >= width) {
        if (accepted) accepted[c] = -1; // malformed round: nothing is changed
        return;
    }
    int acc = r[c], nl = cand;
    bool replaced = false;
    for (int p = lc; p < cand; ++p) {
        const uint8_t want = (uint8_t)pc[p - 1 - row0];
        if (xc[p] != want) {
            xc[p] = want;
            nl = p + 1;
            acc = p - lc;
            replaced = true;
            break;
        }
    }
    if (!replaced && cand < target_len[c]) {
        xc[cand] = (uint8_t)pc[cand - 1 - row0];
        nl = cand + 1;
    }
    l[c] = nl;
    cache_len[c] = lc + acc;
    if (accepted) accepted[c] = acc;
}

// Cell selection of one unmask round (infer/block_generation.c:20-58); the same code runs
// on the host (the fblt_unmask_select_* entry points) and in unmask_step_kernel.
__host__ __device__ inline uint32_t select_confidence(const float *scores, const uint8_t *masked, size_t B, float alpha) {
    uint32_t picked = 0;
    long lead = -1;
    for (size_t b = 0; b < B; ++b) {
        if (!masked[b]) continue;
        if (lead < 0 || scores[b] > scores[lead]) lead = (long)b;
        if (scores[b] >= alpha) picked |= 1u << b;
    }
    if (!picked && lead >= 0) picked = 1u << lead; // always make progress
    return picked;
}

__host__ __device__ inline uint32_t select_eb(const float *scores, const uint8_t *masked, size_t B, float gamma) {
    size_t rank[32];
    size_t n = 0;
    for (size_t b = 0; b < B && b < 32; ++b) { // ascending entropy, stable
        if (!masked[b]) continue;
        size_t slot = n++;
        for (; slot > 0 && scores[rank[slot - 1]] > scores[b]; --slot) rank[slot] = rank[slot - 1];
        rank[slot] = b;
    }
    if (!n) return 0;
    uint32_t picked = 0;
    float budget_used = 0.0f;
    for (size_t t = 0; t < n; ++t) {
        if (t > 0 && !(budget_used + scores[rank[t]] <= gamma)) break;
        budget_used += scores[rank[t]];
        picked |= 1u << rank[t];
    }
    return picked;
}

__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// One unmask round of blt_draft_block for a batch of candidates (infer/block_generation.c:
// 225-252): a CTA per candidate; a warp per cell computes the softmax statistics of its
// logits row the way row_analyze does (:65-80 -- maximum probability and entropy in nats,
// accumulated in double) and the greedy byte (:82-92); one thread then runs the selection
// and writes the chosen cells' bytes.
constexpr int kUnmaskWarps = 8;
__global__ void __launch_bounds__(kUnmaskWarps * 32)
    unmask_step_kernel(const float *logits, int64_t stride, int B, int vocab, int strategy, float threshold,
                       uint8_t *masked, uint8_t *tokens, uint32_t *sel_out, float *conf_out, float *ent_out,
                       int32_t *remaining_out) {
    __shared__ float conf[32], ent[32];
    __shared__ int pred[32];
    const int c = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint8_t *mk = masked + (int64_t)c * B;
    for (int b = warp; b < B; b += kUnmaskWarps) {
        const float *row = logits + ((int64_t)c * B + b) * stride;
        float mx = -INFINITY; // row[0] then strict '>' == maximum over the row
        for (int v = lane; v < vocab; v += 32) mx = fmaxf(mx, row[v]);
        mx = warp_max(mx);
        double sum = 0.0;
        for (int v = lane; v < vocab; v += 32) sum += exp((double)row[v] - (double)mx);
        sum = warp_sum_d(sum);
        double pmax = 0.0, H = 0.0;
        for (int v = lane; v < vocab; v += 32) {
            const double p = exp((double)row[v] - (double)mx) / sum;
            if (p > pmax) pmax = p;
            if (p > 1e-12) H -= p * log(p);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) pmax = fmax(pmax, __shfl_xor_sync(0xffffffffu, pmax, o));
        H = warp_sum_d(H);
        const int arg = warp_argmax_row(row, vocab, lane);
        if (lane == 0) {
            conf[b] = (float)pmax;
            ent[b] = (float)H;
            pred[b] = arg;
            if (conf_out) conf_out[(int64_t)c * B + b] = (float)pmax;
            if (ent_out) ent_out[(int64_t)c * B + b] = (float)H;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t sel = strategy == FBLT_UNMASK_CONFIDENCE ? select_confidence(conf, mk, (size_t)B, threshold)
                                                                : select_eb(ent, mk, (size_t)B, threshold);
        int left = 0;
        for (int b = 0; b < B; ++b) {
            if (sel & (1u << b)) {
                tokens[(int64_t)c * B + b] = (uint8_t)pred[b];
                mk[b] = 0;
            }
            left += mk[b] ? 1 : 0;
        }
        if (sel_out) sel_out[c] = sel;
        if (remaining_out) remaining_out[c] = left;
    }
}

} // namespace fblt

extern "C" int fblt_argmax_rows(const float *logits, int64_t stride, int32_t rows, int32_t vocab, int32_t *ids_out,
                                void *stream) {
    fblt::NvtxRange nvtx_range("fblt_argmax_rows");
    using namespace fblt;
    if (!logits || !ids_out || vocab < 1 || rows < 0 || stride < vocab) return fail(FBLT_ERR_ARG, "argmax_rows: bad arguments");
    if (rows == 0) return FBLT_OK;
    argmax_rows_kernel<<<(rows + 3) / 4, 128, 0, (cudaStream_t)stream>>>(logits, stride, rows, vocab, ids_out);
    count_launch();
    return check_launch("argmax_rows_kernel");
}

extern "C" int fblt_verify_accept(uint8_t *x, int64_t x_stride, const int32_t *pred, int64_t pred_stride,
                                  const int32_t *l, const int32_t *r, const int32_t *target_len, int32_t batch,
                                  int32_t *new_len, int32_t *accepted, void *stream) {
    fblt::NvtxRange nvtx_range("fblt_verify_accept");
    using namespace fblt;
    if (!x || !pred || !l || !r || !target_len || !new_len || batch < 0) return fail(FBLT_ERR_ARG, "verify_accept: bad arguments");
    if (batch == 0) return FBLT_OK;
    verify_accept_kernel<<<(batch + 127) / 128, 128, 0, (cudaStream_t)stream>>>(x, x_stride, pred, pred_stride, l, r,
                                                                               target_len, batch, new_len, accepted);
    count_launch();
    return check_launch("verify_accept_kernel");
}

extern "C" int fblt_dv_commit(const float *logits, int64_t stride, int32_t width, int32_t vocab, int32_t batch, uint8_t *x,
                              int64_t x_stride, int32_t *l, const int32_t *r, const int32_t *target_len,
                              int32_t *cache_len, int32_t *accepted, int32_t *pred_scratch, void *stream) {
    fblt::NvtxRange nvtx_range("fblt_dv_commit");
    using namespace fblt;
    if (!logits || !x || !l || !r || !target_len || !cache_len || !pred_scratch || batch < 0 || width < 1 || vocab < 1 ||
        stride < vocab)
        return fail(FBLT_ERR_ARG, "dv_commit: bad arguments");
    if (vocab > 256) return fail(FBLT_ERR_LIMIT, "dv_commit: predictions are bytes (vocab %d > 256)", vocab);
    if (batch == 0) return FBLT_OK;
    const int64_t rows = (int64_t)batch * width;
    if (rows > 0x7fffffff) return fail(FBLT_ERR_LIMIT, "dv_commit: batch * width beyond int32");
    argmax_rows_kernel<<<(unsigned)((rows + 3) / 4), 128, 0, (cudaStream_t)stream>>>(logits, stride, (int)rows, vocab, pred_scratch);
    count_launch();
    int st = check_launch("argmax_rows_kernel");
    if (st != FBLT_OK) return st;
    dv_commit_kernel<<<(batch + 127) / 128, 128, 0, (cudaStream_t)stream>>>(x, x_stride, pred_scratch, width, l, r, target_len,
                                                                          cache_len, accepted, batch);
    count_launch();
    return check_launch("dv_commit_kernel");
}

extern "C" int fblt_unmask_step(const float *logits, int64_t stride, int32_t batch, int32_t B, int32_t vocab,
                                int32_t strategy, float threshold, uint8_t *masked, uint8_t *tokens,
                                uint32_t *sel_out, float *conf_out, float *ent_out, int32_t *remaining_out,
                                void *stream) {
    fblt::NvtxRange nvtx_range("fblt_unmask_step");
    using namespace fblt;
    if (!logits || !masked || !tokens || batch < 0 || vocab < 1 || stride < vocab)
        return fail(FBLT_ERR_ARG, "unmask_step: bad arguments");
    if (B < 1 || B > 32) return fail(FBLT_ERR_LIMIT, "unmask_step: block size %d outside 1..32", B);
    if (strategy != FBLT_UNMASK_CONFIDENCE && strategy != FBLT_UNMASK_ENTROPY_BOUNDED)
        return fail(FBLT_ERR_ARG, "unmask_step: unknown strategy %d", strategy);
    if (batch == 0) return FBLT_OK;
    unmask_step_kernel<<<batch, kUnmaskWarps * 32, 0, (cudaStream_t)stream>>>(
        logits, stride, B, vocab, strategy, threshold, masked, tokens, sel_out, conf_out, ent_out, remaining_out);
    count_launch();
    return check_launch("unmask_step_kernel");
}

extern "C" size_t fblt_kv_common_patches(const fblt_patch_info *cached, size_t num_cached,
                                         const fblt_patch_info *patches, size_t num_patches) {
    size_t same = 0;
    while (same < num_cached && same < num_patches && cached[same].start_idx == patches[same].start_idx &&
           cached[same].length == patches[same].length)
        ++same;
    return same;
}

// ---- host mirrors of the selection helpers --------------------------------------

extern "C" uint32_t fblt_unmask_select_confidence(const float *scores, const uint8_t *masked, size_t B, float alpha) {
    return fblt::select_confidence(scores, masked, B, alpha);
}

extern "C" uint32_t fblt_unmask_select_eb(const float *scores, const uint8_t *masked, size_t B, float gamma) {
    return fblt::select_eb(scores, masked, B, gamma);
}

extern "C" size_t fblt_aligned_commit_select(const fblt_patch_info *patches, size_t num_patches, size_t lo, size_t hi) {
    size_t chosen = 0;
    for (size_t p = 0; p < num_patches; ++p) {
        const size_t end = patches[p].start_idx + patches[p].length;
        if (end > lo && end <= hi && end > chosen) chosen = end;
    }
    return chosen;
}

extern "C" size_t fblt_block_adapt_b(size_t cur_b, double rolling_acceptance, size_t b_min, size_t b_max, float target) {
    const float band = 0.10f; // BLT_ADAPT_B_MARGIN (infer/block_generation.h:76)
    if (b_max == 0 || b_max < b_min) return cur_b;
    size_t low = b_min ? b_min : 1;
    if (low > b_max) low = b_max;
    size_t b = cur_b;
    if (b < low) b = low;
    if (b > b_max) b = b_max;
    if (!(rolling_acceptance >= 0.0)) return b; // no history yet (NaN)
    if (rolling_acceptance > (double)(target + band)) {
        if (b < b_max) ++b;
    } else if (rolling_acceptance < (double)(target - band)) {
        if (b > low) --b;
    }
    return b;
}
