// Host-buffer sessions: the call path of a host program that owns no device
// memory. A session allocates once (stream, staging for one batch, a batched
// KV cache [batch, cache_rows, E] and its length table); every per-step call
// copies its inputs host->device, runs the batched kernels, copies the result
// back and returns with the stream idle.
#include "common.cuh"

#include <stdlib.h>
#include <string.h>
#include <vector>

struct fblt_session {
    cudaStream_t stream = nullptr;
    int max_batch = 0, H = 0, hd = 0, cache_rows = 0, max_new = 0;
    int64_t E = 0, max_q_rows = 0, max_k_rows = 0;
    float *d_in = nullptr, *d_out = nullptr; // d_in: one block holding q rows, then k rows, then v rows
    int32_t *d_tab = nullptr;
    size_t tab_cap = 0; // int32 entries
    float *kc = nullptr, *vc = nullptr;
    int32_t *d_lens = nullptr, *h_lens = nullptr;
    float *d_qn = nullptr, *d_kn = nullptr, *d_vn = nullptr, *d_on = nullptr;
    // second staging slot, copy streams and events of the pipelined multi-step decode
    float *d_qn2 = nullptr, *d_kn2 = nullptr, *d_vn2 = nullptr, *d_on2 = nullptr;
    cudaStream_t copy_in = nullptr, copy_out = nullptr;
    cudaEvent_t ev_in[2] = {nullptr, nullptr}, ev_kernel[2] = {nullptr, nullptr}, ev_out[2] = {nullptr, nullptr};
    void *ws = nullptr;
    size_t ws_bytes = 0;
    // download stream and events of the non-blocking forward call
    cudaStream_t fwd_out = nullptr;
    cudaEvent_t ev_fwd_kernel = nullptr, ev_fwd_out = nullptr;
    bool fwd_pending = false;
};

namespace fblt {

static void session_free(fblt_session *s) {
    if (!s) return;
    cudaFree(s->d_in);
    cudaFree(s->d_out);
    cudaFree(s->d_tab);
    cudaFree(s->kc);
    cudaFree(s->vc);
    cudaFree(s->d_lens);
    cudaFree(s->d_qn);
    cudaFree(s->d_kn);
    cudaFree(s->d_vn);
    cudaFree(s->d_on);
    cudaFree(s->d_qn2);
    cudaFree(s->d_kn2);
    cudaFree(s->d_vn2);
    cudaFree(s->d_on2);
    for (int i = 0; i < 2; ++i) {
        if (s->ev_in[i]) cudaEventDestroy(s->ev_in[i]);
        if (s->ev_kernel[i]) cudaEventDestroy(s->ev_kernel[i]);
        if (s->ev_out[i]) cudaEventDestroy(s->ev_out[i]);
    }
    if (s->ev_fwd_kernel) cudaEventDestroy(s->ev_fwd_kernel);
    if (s->ev_fwd_out) cudaEventDestroy(s->ev_fwd_out);
    if (s->fwd_out) cudaStreamDestroy(s->fwd_out);
    if (s->copy_in) cudaStreamDestroy(s->copy_in);
    if (s->copy_out) cudaStreamDestroy(s->copy_out);
    cudaFree(s->ws);
    if (s->h_lens) cudaFreeHost(s->h_lens);
    if (s->stream) cudaStreamDestroy(s->stream);
    delete s;
}

// Bump placement of int32 tables in the session's device table arena.
struct TableArena {
    fblt_session *s;
    size_t used = 0;
    int status = FBLT_OK;
    const int32_t *put(const int32_t *host, size_t n) {
        if (!host || status != FBLT_OK) return nullptr;
        const size_t padded = (n + 3) & ~(size_t)3;
        if (used + padded > s->tab_cap) {
            status = fail(FBLT_ERR_CAPACITY, "session: mask tables exceed session capacity");
            return nullptr;
        }
        int32_t *dst = s->d_tab + used;
        cudaError_t e = cudaMemcpyAsync(dst, host, n * sizeof(int32_t), cudaMemcpyHostToDevice, s->stream);
        if (e != cudaSuccess) {
            status = fail(FBLT_ERR_CUDA, "session: table upload: %s", cudaGetErrorString(e));
            return nullptr;
        }
        used += padded;
        return dst;
    }
};

} // namespace fblt

extern "C" int fblt_session_create(fblt_session **out, int32_t max_batch, int32_t num_heads, int32_t head_dim,
                                   int64_t max_q_rows, int64_t max_k_rows, int32_t cache_rows, int32_t max_new) {
    using namespace fblt;
    if (!out || max_batch < 1 || num_heads < 1 || head_dim < 1 || max_q_rows < 0 || max_k_rows < 0 || cache_rows < 0 ||
        max_new < 0)
        return fail(FBLT_ERR_ARG, "session_create: bad arguments");
    fblt_session *s = new fblt_session();
    s->max_batch = max_batch;
    s->H = num_heads;
    s->hd = head_dim;
    s->E = (int64_t)num_heads * head_dim;
    s->max_q_rows = max_q_rows;
    s->max_k_rows = max_k_rows;
    s->cache_rows = cache_rows;
    s->max_new = max_new;
#define S_TRY(expr)                                                                          \
    do {                                                                                     \
        cudaError_t e__ = (expr);                                                            \
        if (e__ != cudaSuccess) {                                                            \
            session_free(s);                                                                 \
            return fail(FBLT_ERR_CUDA, "session_create: %s: %s", #expr, cudaGetErrorString(e__)); \
        }                                                                                    \
    } while (0)
    S_TRY(cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking));
    S_TRY(cudaStreamCreateWithFlags(&s->fwd_out, cudaStreamNonBlocking));
    S_TRY(cudaEventCreateWithFlags(&s->ev_fwd_kernel, cudaEventDisableTiming));
    S_TRY(cudaEventCreateWithFlags(&s->ev_fwd_out, cudaEventDisableTiming));
    const size_t fE = (size_t)s->E * sizeof(float);
    if (max_q_rows > 0) S_TRY(cudaMalloc(&s->d_out, (size_t)max_q_rows * fE));
    if (max_q_rows + max_k_rows > 0) S_TRY(cudaMalloc(&s->d_in, (size_t)(max_q_rows + 2 * max_k_rows) * fE));
    // tables: 8 per-sequence arrays plus doc / patch boundary lists
    s->tab_cap = (size_t)(max_batch + 4) * 10 + (size_t)max_k_rows + (size_t)max_q_rows + 2 * (size_t)max_batch + 64;
    S_TRY(cudaMalloc(&s->d_tab, s->tab_cap * sizeof(int32_t)));
    S_TRY(cudaMalloc(&s->d_lens, (size_t)max_batch * sizeof(int32_t)));
    S_TRY(cudaMallocHost(&s->h_lens, (size_t)max_batch * sizeof(int32_t)));
    memset(s->h_lens, 0, (size_t)max_batch * sizeof(int32_t));
    if (cache_rows > 0) {
        const size_t cache_bytes = (size_t)max_batch * cache_rows * fE;
        S_TRY(cudaMalloc(&s->kc, cache_bytes));
        S_TRY(cudaMalloc(&s->vc, cache_bytes));
    }
    if (max_new > 0) {
        const size_t nb = (size_t)max_batch * max_new * fE;
        S_TRY(cudaMalloc(&s->d_qn, nb));
        S_TRY(cudaMalloc(&s->d_kn, nb));
        S_TRY(cudaMalloc(&s->d_vn, nb));
        S_TRY(cudaMalloc(&s->d_on, nb));
        S_TRY(cudaMalloc(&s->d_qn2, nb));
        S_TRY(cudaMalloc(&s->d_kn2, nb));
        S_TRY(cudaMalloc(&s->d_vn2, nb));
        S_TRY(cudaMalloc(&s->d_on2, nb));
        S_TRY(cudaStreamCreateWithFlags(&s->copy_in, cudaStreamNonBlocking));
        S_TRY(cudaStreamCreateWithFlags(&s->copy_out, cudaStreamNonBlocking));
        for (int i = 0; i < 2; ++i) {
            S_TRY(cudaEventCreateWithFlags(&s->ev_in[i], cudaEventDisableTiming));
            S_TRY(cudaEventCreateWithFlags(&s->ev_kernel[i], cudaEventDisableTiming));
            S_TRY(cudaEventCreateWithFlags(&s->ev_out[i], cudaEventDisableTiming));
        }
        // split-K partials exist only while (sequences x heads) is below the
        // launch-width target, which bounds units x splits
        s->ws_bytes = (size_t)2048 * max_new * ((size_t)head_dim + 4) * sizeof(float);
        if (s->ws_bytes < ((size_t)8 << 20)) s->ws_bytes = (size_t)8 << 20; // the stream form: two partials per resident CTA
        S_TRY(cudaMalloc(&s->ws, s->ws_bytes));
    }
#undef S_TRY
    *out = s;
    return FBLT_OK;
}

extern "C" void fblt_session_destroy(fblt_session *s) { fblt::session_free(s); }

namespace fblt {
static int session_forward_impl(fblt_session *s, const fblt_attn_desc *hd, bool blocking);
int tcgen05_error_on_stream(cudaStream_t s); // tile5_kernel.cu
}

extern "C" int fblt_session_forward(fblt_session *s, const fblt_attn_desc *hd) {
    fblt::NvtxRange nvtx_range("fblt_session_forward");
    return fblt::session_forward_impl(s, hd, true);
}

extern "C" int fblt_session_forward_async(fblt_session *s, const fblt_attn_desc *hd) {
    fblt::NvtxRange nvtx_range("fblt_session_forward_async");
    return fblt::session_forward_impl(s, hd, false);
}

extern "C" int fblt_session_wait(fblt_session *s) {
    using namespace fblt;
    if (!s) return fail(FBLT_ERR_ARG, "session_wait: NULL session");
    FBLT_CUDA_TRY(cudaStreamSynchronize(s->stream));
    FBLT_CUDA_TRY(cudaStreamSynchronize(s->fwd_out));
    if (s->copy_in) FBLT_CUDA_TRY(cudaStreamSynchronize(s->copy_in));
    if (s->copy_out) FBLT_CUDA_TRY(cudaStreamSynchronize(s->copy_out));
    const bool had_forward = s->fwd_pending;
    s->fwd_pending = false;
    if (had_forward) {
        // the session's streams are idle, so its kernels have finished: read the error words on the
        // session's own stream instead of stalling every other stream of the device
        if (const int code = tcgen05_error_on_stream(s->stream))
            return fail(FBLT_ERR_CUDA, "session_wait: a tcgen05 CTA gave up on a bounded wait (code 0x%x)", code);
    }
    return FBLT_OK;
}

static int fblt::session_forward_impl(fblt_session *s, const fblt_attn_desc *hd, bool blocking) {
    if (!s || !hd) return fail(FBLT_ERR_ARG, "session_forward: NULL argument");
    if (hd->batch < 0 || hd->batch > s->max_batch) return fail(FBLT_ERR_CAPACITY, "session_forward: batch %d > %d", hd->batch, s->max_batch);
    if (hd->num_heads != s->H || hd->head_dim != s->hd) return fail(FBLT_ERR_ARG, "session_forward: heads/head_dim differ from the session");
    if (hd->batch == 0) return FBLT_OK;
    if (!hd->cu_q || !hd->cu_k || !hd->q || !hd->k || !hd->v || !hd->out) return fail(FBLT_ERR_ARG, "session_forward: NULL buffer");
    if (hd->mask.q_group_ids || hd->mask.k_group_ids) return fail(FBLT_ERR_UNSUPPORTED, "session_forward: explicit group ids are device-only");
    const int B = hd->batch;
    const int64_t tq = hd->cu_q[B], tk = hd->cu_k[B];
    if (tq > s->max_q_rows || tk > s->max_k_rows) return fail(FBLT_ERR_CAPACITY, "session_forward: %lld/%lld rows exceed session staging", (long long)tq, (long long)tk);
    const int64_t E = s->E;
    if (hd->q_stride < E || hd->k_stride < E || hd->v_stride < E || hd->out_stride < E) return fail(FBLT_ERR_ARG, "session_forward: row stride smaller than num_heads*head_dim");

    const size_t wb = (size_t)E * sizeof(float);
    float *dq = s->d_in, *dk = s->d_in + (size_t)s->max_q_rows * E, *dv = dk + (size_t)s->max_k_rows * E;
    int64_t dstride = E;
    // packed [T, 3E] rows (models/attention.c:95-98) travel as one contiguous copy and stay packed
    const bool packed = tq == tk && hd->k == hd->q + E && hd->v == hd->q + 2 * E && hd->q_stride == 3 * E &&
                        hd->k_stride == 3 * E && hd->v_stride == 3 * E;
    if (packed) {
        FBLT_CUDA_TRY(cudaMemcpyAsync(s->d_in, hd->q, (size_t)tq * 3 * wb, cudaMemcpyHostToDevice, s->stream));
        dk = dq + E;
        dv = dq + 2 * E;
        dstride = 3 * E;
    } else {
        FBLT_CUDA_TRY(cudaMemcpy2DAsync(dq, wb, hd->q, (size_t)hd->q_stride * 4, wb, (size_t)tq, cudaMemcpyHostToDevice, s->stream));
        FBLT_CUDA_TRY(cudaMemcpy2DAsync(dk, wb, hd->k, (size_t)hd->k_stride * 4, wb, (size_t)tk, cudaMemcpyHostToDevice, s->stream));
        FBLT_CUDA_TRY(cudaMemcpy2DAsync(dv, wb, hd->v, (size_t)hd->v_stride * 4, wb, (size_t)tk, cudaMemcpyHostToDevice, s->stream));
    }

    fblt_attn_desc d = *hd;
    TableArena ta{s};
    d.cu_q = ta.put(hd->cu_q, (size_t)B + 1);
    d.cu_k = ta.put(hd->cu_k, (size_t)B + 1);
    const fblt_mask_desc &hm = hd->mask;
    d.mask.causal_offset = ta.put(hm.causal_offset, (size_t)B);
    if (hm.cu_doc && hm.doc_bounds) {
        d.mask.cu_doc = ta.put(hm.cu_doc, (size_t)B + 1);
        d.mask.doc_bounds = ta.put(hm.doc_bounds, (size_t)hm.cu_doc[B] > 0 ? (size_t)hm.cu_doc[B] : 1);
    }
    if (hm.cu_patch && hm.patch_bounds) {
        d.mask.cu_patch = ta.put(hm.cu_patch, (size_t)B + 1);
        d.mask.patch_bounds = ta.put(hm.patch_bounds, (size_t)hm.cu_patch[B]);
    }
    d.mask.q_pos_offset = ta.put(hm.q_pos_offset, (size_t)B);
    d.mask.num_clean = ta.put(hm.num_clean, (size_t)B);
    if (hm.trailing_closed) {
        std::vector<int32_t> packed(((size_t)B + 3) / 4, 0);
        memcpy(packed.data(), hm.trailing_closed, (size_t)B);
        // bytes keep their order inside the int32 words on a little-endian host
        d.mask.trailing_closed = reinterpret_cast<const uint8_t *>(ta.put(packed.data(), packed.size()));
        // `packed` is pageable: the copy above has completed staging on return
    }
    if (ta.status != FBLT_OK) return ta.status;
    d.q = dq;
    d.k = dk;
    d.v = dv;
    d.out = s->d_out;
    d.q_stride = d.k_stride = d.v_stride = dstride;
    d.out_stride = E;
    d.total_q_rows = tq <= 0x7fffffff ? (int32_t)tq : 0; // the staged tensors end here
    d.total_k_rows = tk <= 0x7fffffff ? (int32_t)tk : 0;
    // the previous non-blocking call's rows must have left d_out before this kernel overwrites them
    if (s->fwd_pending) FBLT_CUDA_TRY(cudaStreamWaitEvent(s->stream, s->ev_fwd_out, 0));
    int st = fblt_attn_forward(&d, s->stream);
    if (st != FBLT_OK) return st;
    // the rows go home on a stream of their own, so that whatever the caller enqueues next on the
    // session (a cache load, decode steps) overlaps with the download
    FBLT_CUDA_TRY(cudaEventRecord(s->ev_fwd_kernel, s->stream));
    FBLT_CUDA_TRY(cudaStreamWaitEvent(s->fwd_out, s->ev_fwd_kernel, 0));
    FBLT_CUDA_TRY(cudaMemcpy2DAsync(hd->out, (size_t)hd->out_stride * 4, s->d_out, wb, wb, (size_t)tq, cudaMemcpyDeviceToHost, s->fwd_out));
    FBLT_CUDA_TRY(cudaEventRecord(s->ev_fwd_out, s->fwd_out));
    s->fwd_pending = true;
    return blocking ? fblt_session_wait(s) : FBLT_OK;
}

extern "C" int fblt_session_cache_load(fblt_session *s, int32_t batch, const int32_t *lens, const float *k_host,
                                       const float *v_host, int64_t host_seq_stride_rows) {
    using namespace fblt;
    if (!s || !lens || batch < 0) return fail(FBLT_ERR_ARG, "cache_load: bad arguments");
    if (batch > s->max_batch || !s->kc) return fail(FBLT_ERR_CAPACITY, "cache_load: batch %d exceeds the session cache", batch);
    const size_t rowb = (size_t)s->E * sizeof(float);
    int32_t max_len = 0;
    bool uniform = batch > 0;
    for (int b = 0; b < batch; ++b) {
        if (lens[b] < 0 || lens[b] > s->cache_rows) return fail(FBLT_ERR_CAPACITY, "cache_load: length %d exceeds cache_rows %d", lens[b], s->cache_rows);
        if (lens[b] > host_seq_stride_rows) return fail(FBLT_ERR_ARG, "cache_load: length exceeds the host stride");
        max_len = lens[b] > max_len ? lens[b] : max_len;
        uniform = uniform && lens[b] == lens[0];
        s->h_lens[b] = lens[b];
    }
    if (batch > 0 && max_len > 0) {
        if (!k_host || !v_host) return fail(FBLT_ERR_ARG, "cache_load: NULL host rows");
        if (uniform) {
            // one strided copy per array: `max_len` rows of every sequence
            const size_t width = (size_t)max_len * rowb;
            FBLT_CUDA_TRY(cudaMemcpy2DAsync(s->kc, (size_t)s->cache_rows * rowb, k_host, (size_t)host_seq_stride_rows * rowb, width, (size_t)batch, cudaMemcpyHostToDevice, s->stream));
            FBLT_CUDA_TRY(cudaMemcpy2DAsync(s->vc, (size_t)s->cache_rows * rowb, v_host, (size_t)host_seq_stride_rows * rowb, width, (size_t)batch, cudaMemcpyHostToDevice, s->stream));
        } else {
            for (int b = 0; b < batch; ++b) {
                if (!lens[b]) continue;
                const size_t bytes = (size_t)lens[b] * rowb;
                FBLT_CUDA_TRY(cudaMemcpyAsync(s->kc + (size_t)b * s->cache_rows * s->E, k_host + (size_t)b * host_seq_stride_rows * s->E, bytes, cudaMemcpyHostToDevice, s->stream));
                FBLT_CUDA_TRY(cudaMemcpyAsync(s->vc + (size_t)b * s->cache_rows * s->E, v_host + (size_t)b * host_seq_stride_rows * s->E, bytes, cudaMemcpyHostToDevice, s->stream));
            }
        }
    }
    FBLT_CUDA_TRY(cudaStreamSynchronize(s->stream));
    return FBLT_OK;
}

extern "C" int fblt_session_decode(fblt_session *s, int32_t batch, int32_t n_new, int32_t block_mode, int32_t window,
                                   float scale, const float *q_new, const float *k_new, const float *v_new, float *out,
                                   int32_t advance) {
    fblt::NvtxRange nvtx_range("fblt_session_decode");
    using namespace fblt;
    if (!s || !q_new || !k_new || !v_new || !out) return fail(FBLT_ERR_ARG, "session_decode: NULL argument");
    if (batch < 0 || batch > s->max_batch || !s->kc) return fail(FBLT_ERR_CAPACITY, "session_decode: batch %d exceeds the session", batch);
    if (n_new < 1 || n_new > s->max_new) return fail(FBLT_ERR_CAPACITY, "session_decode: n_new %d outside 1..%d", n_new, s->max_new);
    if (advance < 0 || advance > n_new) return fail(FBLT_ERR_ARG, "session_decode: advance must be in 0..n_new");
    if (batch == 0) return FBLT_OK;
    int32_t max_len = 0;
    for (int b = 0; b < batch; ++b) {
        if (s->h_lens[b] + n_new > s->cache_rows) return fail(FBLT_ERR_CAPACITY, "session_decode: sequence %d would exceed cache_rows %d", b, s->cache_rows);
        max_len = s->h_lens[b] + n_new > max_len ? s->h_lens[b] + n_new : max_len;
    }
    const size_t nb = (size_t)batch * n_new * s->E * sizeof(float);
    FBLT_CUDA_TRY(cudaMemcpyAsync(s->d_lens, s->h_lens, (size_t)batch * sizeof(int32_t), cudaMemcpyHostToDevice, s->stream));
    FBLT_CUDA_TRY(cudaMemcpyAsync(s->d_qn, q_new, nb, cudaMemcpyHostToDevice, s->stream));
    FBLT_CUDA_TRY(cudaMemcpyAsync(s->d_kn, k_new, nb, cudaMemcpyHostToDevice, s->stream));
    FBLT_CUDA_TRY(cudaMemcpyAsync(s->d_vn, v_new, nb, cudaMemcpyHostToDevice, s->stream));
    fblt_decode_desc d;
    memset(&d, 0, sizeof(d));
    d.batch = batch;
    d.num_heads = s->H;
    d.head_dim = s->hd;
    d.n_new = n_new;
    d.block_mode = block_mode;
    d.window = window;
    d.max_len = max_len;
    d.base_len = s->d_lens;
    d.k_cache = s->kc;
    d.v_cache = s->vc;
    d.cache_seq_stride = (int64_t)s->cache_rows * s->E;
    d.cache_row_stride = s->E;
    d.q = s->d_qn;
    d.q_stride = s->E;
    d.k_new = s->d_kn;
    d.v_new = s->d_vn;
    d.kv_new_stride = s->E;
    d.out = s->d_on;
    d.out_stride = s->E;
    d.scale = scale;
    if (fblt_attn_decode_workspace(&d) > s->ws_bytes) d.splits = 1;
    int st = fblt_attn_decode(&d, s->ws, s->ws_bytes, s->stream);
    if (st != FBLT_OK) return st;
    FBLT_CUDA_TRY(cudaMemcpyAsync(out, s->d_on, nb, cudaMemcpyDeviceToHost, s->stream));
    FBLT_CUDA_TRY(cudaStreamSynchronize(s->stream));
    for (int b = 0; b < batch; ++b) s->h_lens[b] += advance;
    return FBLT_OK;
}

extern "C" int fblt_session_decode_steps(fblt_session *s, int32_t batch, int32_t n_new, int32_t steps, int32_t block_mode,
                                         int32_t window, float scale, const float *q_new, const float *k_new,
                                         const float *v_new, int64_t in_step_stride, float *out,
                                         int64_t out_step_stride, int32_t advance) {
    fblt::NvtxRange nvtx_range("fblt_session_decode_steps");
    using namespace fblt;
    if (!s || !q_new || !k_new || !v_new || !out) return fail(FBLT_ERR_ARG, "session_decode_steps: NULL argument");
    if (batch < 0 || batch > s->max_batch || !s->kc) return fail(FBLT_ERR_CAPACITY, "session_decode_steps: batch %d exceeds the session", batch);
    if (n_new < 1 || n_new > s->max_new) return fail(FBLT_ERR_CAPACITY, "session_decode_steps: n_new %d outside 1..%d", n_new, s->max_new);
    if (advance < 0 || advance > n_new || steps < 0) return fail(FBLT_ERR_ARG, "session_decode_steps: bad advance / steps");
    if (batch == 0 || steps == 0) return FBLT_OK;
    int32_t max_len = 0;
    for (int b = 0; b < batch; ++b) {
        const int64_t last = (int64_t)s->h_lens[b] + (int64_t)(steps - 1) * advance + n_new;
        if (last > s->cache_rows) return fail(FBLT_ERR_CAPACITY, "session_decode_steps: sequence %d would exceed cache_rows %d", b, s->cache_rows);
        max_len = (int32_t)last > max_len ? (int32_t)last : max_len;
    }
    const size_t nb = (size_t)batch * n_new * s->E * sizeof(float);
    FBLT_CUDA_TRY(cudaMemcpyAsync(s->d_lens, s->h_lens, (size_t)batch * sizeof(int32_t), cudaMemcpyHostToDevice, s->stream));
    FBLT_CUDA_TRY(cudaStreamSynchronize(s->stream));
    float *dq[2] = {s->d_qn, s->d_qn2}, *dk[2] = {s->d_kn, s->d_kn2}, *dv[2] = {s->d_vn, s->d_vn2}, *dout[2] = {s->d_on, s->d_on2};
    for (int t = 0; t < steps; ++t) {
        const int slot = t & 1;
        // inputs of step t: once the kernel of step t-2 has finished reading this slot
        if (t >= 2) FBLT_CUDA_TRY(cudaStreamWaitEvent(s->copy_in, s->ev_kernel[slot], 0));
        FBLT_CUDA_TRY(cudaMemcpyAsync(dq[slot], q_new + (size_t)t * in_step_stride, nb, cudaMemcpyHostToDevice, s->copy_in));
        FBLT_CUDA_TRY(cudaMemcpyAsync(dk[slot], k_new + (size_t)t * in_step_stride, nb, cudaMemcpyHostToDevice, s->copy_in));
        FBLT_CUDA_TRY(cudaMemcpyAsync(dv[slot], v_new + (size_t)t * in_step_stride, nb, cudaMemcpyHostToDevice, s->copy_in));
        FBLT_CUDA_TRY(cudaEventRecord(s->ev_in[slot], s->copy_in));
        // kernel of step t: inputs present, and the output slot drained by step t-2's copy
        FBLT_CUDA_TRY(cudaStreamWaitEvent(s->stream, s->ev_in[slot], 0));
        if (t >= 2) FBLT_CUDA_TRY(cudaStreamWaitEvent(s->stream, s->ev_out[slot], 0));
        fblt_decode_desc d;
        memset(&d, 0, sizeof(d));
        d.batch = batch;
        d.num_heads = s->H;
        d.head_dim = s->hd;
        d.n_new = n_new;
        d.block_mode = block_mode;
        d.window = window;
        d.max_len = max_len;
        d.base_len = s->d_lens;
        d.base_add = t * advance;
        d.k_cache = s->kc;
        d.v_cache = s->vc;
        d.cache_seq_stride = (int64_t)s->cache_rows * s->E;
        d.cache_row_stride = s->E;
        d.q = dq[slot];
        d.q_stride = s->E;
        d.k_new = dk[slot];
        d.v_new = dv[slot];
        d.kv_new_stride = s->E;
        d.out = dout[slot];
        d.out_stride = s->E;
        d.scale = scale;
        if (fblt_attn_decode_workspace(&d) > s->ws_bytes) d.splits = 1;
        const int st = fblt_attn_decode(&d, s->ws, s->ws_bytes, s->stream);
        if (st != FBLT_OK) return st;
        FBLT_CUDA_TRY(cudaEventRecord(s->ev_kernel[slot], s->stream));
        // outputs of step t
        FBLT_CUDA_TRY(cudaStreamWaitEvent(s->copy_out, s->ev_kernel[slot], 0));
        FBLT_CUDA_TRY(cudaMemcpyAsync(out + (size_t)t * out_step_stride, dout[slot], nb, cudaMemcpyDeviceToHost, s->copy_out));
        FBLT_CUDA_TRY(cudaEventRecord(s->ev_out[slot], s->copy_out));
    }
    FBLT_CUDA_TRY(cudaStreamSynchronize(s->copy_out));
    FBLT_CUDA_TRY(cudaStreamSynchronize(s->stream));
    FBLT_CUDA_TRY(cudaStreamSynchronize(s->copy_in));
    for (int b = 0; b < batch; ++b) s->h_lens[b] += steps * advance;
    return FBLT_OK;
}

extern "C" int fblt_session_cache_truncate(fblt_session *s, int32_t batch, const int32_t *lens) {
    using namespace fblt;
    if (!s || !lens || batch < 0 || batch > s->max_batch) return fail(FBLT_ERR_ARG, "cache_truncate: bad arguments");
    if (!s->kc) return fail(FBLT_ERR_ARG, "cache_truncate: session has no cache");
    for (int b = 0; b < batch; ++b)
        if (lens[b] < 0 || lens[b] > s->cache_rows)
            return fail(FBLT_ERR_CAPACITY, "cache_truncate: length %d of sequence %d outside [0, %d]", lens[b], b, s->cache_rows);
    // earlier steps have completed (every session call returns with its stream idle)
    for (int b = 0; b < batch; ++b) s->h_lens[b] = lens[b];
    return FBLT_OK;
}

extern "C" int fblt_session_cache_reset(fblt_session *s) {
    using namespace fblt;
    if (!s) return fail(FBLT_ERR_ARG, "cache_reset: NULL session");
    memset(s->h_lens, 0, (size_t)s->max_batch * sizeof(int32_t));
    return FBLT_OK;
}

extern "C" int fblt_session_cache_lens(fblt_session *s, int32_t *lens_out, int32_t batch) {
    using namespace fblt;
    if (!s || !lens_out || batch < 0 || batch > s->max_batch) return fail(FBLT_ERR_ARG, "cache_lens: bad arguments");
    memcpy(lens_out, s->h_lens, (size_t)batch * sizeof(int32_t));
    return FBLT_OK;
}
