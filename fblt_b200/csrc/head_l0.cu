// L0: the reference's single-head attention operator (one sequence, one head,
// optional dense additive mask, optional weight / (m,l) outputs) as one launch.
// Semantics follow ops/attn_core_cpu.c:16-57 and ops/vecmath_cpu.c:16-53:
// mask wins over is_causal, the row maximum is taken over finite entries only,
// non-finite entries get weight 0, an all-masked row yields zeros, weights are
// normalised before the value sum and zero weights are skipped.
//
// One CTA per query row keeps the row's scores in shared memory (or, for rows
// longer than shared memory, in the caller's weights_out / scores_scratch), so
// no [nq, nk] score matrix is written unless the caller asks for the weights.
#include "common.cuh"

#include <stdlib.h>

namespace fblt {

constexpr int kL0Threads = 128;
constexpr int kL0Warps = kL0Threads / 32;
constexpr size_t kL0MaxSmem = 220 * 1024; // bytes of dynamic shared memory the kernel may ask for

__device__ __forceinline__ float block_reduce(float v, float *red, bool is_max) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = is_max ? warp_max(v) : warp_sum(v);
    __syncthreads(); // protect `red` from the previous use
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = red[0];
#pragma unroll
    for (int w = 1; w < kL0Warps; ++w) r = is_max ? fmaxf(r, red[w]) : r + red[w];
    return r;
}

__global__ void __launch_bounds__(kL0Threads) l0_head_kernel(fblt_head_args a, float *gscores, int scores_in_smem) {
    extern __shared__ float sm[];
    const int hd = (int)a.head_dim;
    const int hd_pad = (hd + 31) & ~31;
    float *qs = sm;
    float *red = qs + hd_pad;               // kL0Warps floats (32 reserved)
    float *part = red + 32;                 // kL0Warps * 32 floats
    float *sc_s = part + kL0Warps * 32;     // nk floats when scores_in_smem
    const size_t i = blockIdx.x;
    const size_t nk = a.nk;
    float *sc = scores_in_smem ? sc_s : gscores + i * nk;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    for (int d = tid; d < hd; d += kL0Threads) qs[d] = a.q[i * a.q_stride + d];
    __syncthreads();

    const float *mrow = a.mask ? a.mask + i * nk : nullptr;
    for (size_t j = warp; j < nk; j += kL0Warps) {
        const float *kj = a.k + j * a.k_stride;
        float p = 0.0f;
        for (int d = lane; d < hd; d += 32) p += qs[d] * kj[d];
        p = warp_sum(p);
        if (lane == 0) {
            float s;
            if (mrow) s = p * a.scale + mrow[j];
            else if (a.is_causal && j > i) s = -INFINITY;
            else s = p * a.scale;
            sc[j] = s;
        }
    }
    __syncthreads();

    float mx = -INFINITY;
    for (size_t j = tid; j < nk; j += kL0Threads) {
        const float s = sc[j];
        if (finite_f(s)) mx = fmaxf(mx, s);
    }
    mx = block_reduce(mx, red, true);

    float sum = 0.0f;
    for (size_t j = tid; j < nk; j += kL0Threads) {
        const float s = sc[j];
        const float e = finite_f(s) ? expf(s - mx) : 0.0f;
        sc[j] = e;
        sum += e;
    }
    sum = block_reduce(sum, red, false);

    if (sum > 0.0f) {
        for (size_t j = tid; j < nk; j += kL0Threads) sc[j] = sc[j] / sum;
    }
    __syncthreads();

    if (a.weights_out && sc != a.weights_out + i * nk) {
        for (size_t j = tid; j < nk; j += kL0Threads) a.weights_out[i * nk + j] = sc[j];
    }
    if (a.lse_out && tid == 0) {
        a.lse_out[i * 2] = mx;
        a.lse_out[i * 2 + 1] = sum;
    }

    float *out = a.combined + i * a.combined_stride + a.combined_col_offset;
    for (int d0 = 0; d0 < hd; d0 += 32) {
        const int d = d0 + lane;
        float acc = 0.0f;
        if (d < hd) {
            for (size_t j = warp; j < nk; j += kL0Warps) {
                const float w = sc[j];
                if (w != 0.0f) acc += w * a.v[j * a.v_stride + d];
            }
        }
        part[warp * 32 + lane] = acc;
        __syncthreads();
        if (warp == 0 && d < hd) {
            float t = part[lane];
#pragma unroll
            for (int w = 1; w < kL0Warps; ++w) t += part[w * 32 + lane];
            out[d] = t;
        }
        __syncthreads();
    }
}

static int launch_l0(const fblt_head_args *a, cudaStream_t stream) {
    if (!a || !a->q || !a->k || !a->v || !a->combined) return fail(FBLT_ERR_ARG, "head: buffers must not be NULL");
    if (a->head_dim == 0) return fail(FBLT_ERR_ARG, "head: head_dim must be > 0");
    if (a->nq == 0) return FBLT_OK;
    if (a->nq > 0x7fffffffu) return fail(FBLT_ERR_LIMIT, "head: nq too large");
    if (a->head_dim > 8192) return fail(FBLT_ERR_LIMIT, "head: head_dim %zu > 8192", a->head_dim);
    const size_t hd_pad = (a->head_dim + 31) & ~(size_t)31;
    const size_t fixed = (hd_pad + 32 + kL0Warps * 32) * sizeof(float);
    int in_smem = fixed + a->nk * sizeof(float) <= kL0MaxSmem;
    float *gscores = nullptr;
    if (!in_smem) {
        gscores = a->weights_out ? a->weights_out : a->scores_scratch;
        if (!gscores)
            return fail(FBLT_ERR_WORKSPACE, "head: nk=%zu exceeds shared memory; weights_out or scores_scratch needed",
                        a->nk);
    }
    const size_t smem = fixed + (in_smem ? a->nk * sizeof(float) : 0);
    if (smem > 48 * 1024) {
        // raised to the largest size this kernel ever uses; cheap and safe to repeat (per device, any thread)
        FBLT_CUDA_TRY(cudaFuncSetAttribute(l0_head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kL0MaxSmem));
    }
    l0_head_kernel<<<(unsigned)a->nq, kL0Threads, smem, stream>>>(*a, gscores, in_smem);
    count_launch();
    return check_launch("l0_head_kernel");
}

} // namespace fblt

extern "C" int fblt_attention_head(const fblt_head_args *args, void *stream) {
    fblt::NvtxRange nvtx_range("fblt_attention_head");
    return fblt::launch_l0(args, (cudaStream_t)stream);
}

// Reference error convention (core/backend.h:13-31): message to stderr, exit(1).
#define L0_REQUIRE(cond, msg)                                                                              \
    do {                                                                                                   \
        if (!(cond)) {                                                                                     \
            fprintf(stderr, "BLT Fatal Error [%s:%d]: Requirement '%s' failed: %s\n", __FILE__, __LINE__, \
                    #cond, msg);                                                                           \
            exit(EXIT_FAILURE);                                                                            \
        }                                                                                                  \
    } while (0)

extern "C" void blt_attention_head_core_cuda(int backend, const fblt_head_args *a) {
    L0_REQUIRE(backend == FBLT_BACKEND_CUDA, "blt_attention_head_core: CUDA implementation called with non-CUDA backend");
    L0_REQUIRE(a != NULL && a->q != NULL && a->k != NULL && a->v != NULL && a->combined != NULL,
               "blt_attention_head_core: buffers must not be NULL");
    L0_REQUIRE(a->weights_out != NULL || a->scores_scratch != NULL || a->lse_out != NULL,
               "blt_attention_head_core: need weights_out, scores_scratch, or lse_out");
    const int st = fblt::launch_l0(a, (cudaStream_t)0);
    if (st != FBLT_OK) {
        fprintf(stderr, "BLT Fatal Error [%s:%d]: blt_attention_head_core failed: %s\n", __FILE__, __LINE__,
                fblt_last_error());
        exit(EXIT_FAILURE);
    }
}

extern "C" void blt_attention_head_core_backward_cuda(int backend, const void *bwd_args) {
    (void)backend;
    (void)bwd_args;
    fprintf(stderr,
            "BLT Fatal Error [%s:%d]: blt_attention_head_core_backward: not available in this backend "
            "(inference-only attention library)\n",
            __FILE__, __LINE__);
    exit(EXIT_FAILURE);
}
