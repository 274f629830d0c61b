// Dense matmul out[M,N] = a[M,K] * b[K,N] (+ bias) in fp32, the projection GEMMs on both
// sides of the attention operator (blt_matmul: ops/linalg_cpu.c:8-18 on the CPU,
// cublasSgemm in ops/linalg.cu:134-136), on the 5th-generation tensor cores.
//
//   b      = packed once (weights are constant between calls): split into TF32 (hi, lo)
//            parts and laid out tile by tile in the exact shared-memory image the MMA reads
//            (no-swizzle K-major core matrices, [n][k] order), so one thread brings a
//            128 x 32 weight tile in with one bulk copy that completes on an mbarrier.
//   a      = 128 or 256 rows x 32 per step; eight producer warps load 16-byte pieces two
//            steps ahead into registers, split them into (hi, lo) and store them in the same
//            core-matrix layout, then arrive on the stage's mbarrier.
//   MMA    = one thread; per step and 128-row sub-tile 4 x (lo*hi, hi*lo -> small-term
//            accumulator; hi*hi -> main accumulator) tcgen05.mma of shape 128x128x8, fp32
//            accumulate in TMEM; tcgen05.commit hands the stage back to the producers. The
//            small terms are kept apart because the tensor core truncates when it adds into
//            the accumulator: one addition per 8-deep slice into the main sum, not three.
//   out    = the producer warps read main + small accumulators (warp w: TMEM lanes
//            32 (w & 3).., columns 64 (w >> 2)..), add the bias and store.
//   No __syncthreads in the main loop: the three roles meet only on mbarriers
//   (a ready, b ready, stage free, all done).
//
// Every mbarrier wait is bounded and watches a CTA-wide abort word; a role that gives up
// raises it, the CTA records an error code, waits (bounded) for its copies and MMAs in
// flight, frees its TMEM and returns.
#include "common.cuh"
#include "tc5.cuh"

#include <atomic>

namespace fblt {

constexpr int kGM = 128, kGN = 128, kGK = 32;
constexpr int kGProducers = 256;               // warps 0-7: stage a, then run the epilogue
constexpr int kGThreads = kGProducers + 64;    // warp 8: MMA issue (and TMEM owner); warp 9: weight copies
constexpr int kGPlane = kGM * kGK * 4;         // 16 KB: one (hi or lo) plane of a 128 x 32 operand tile
constexpr int kGPrefetch = 4;                  // steps of a held in registers ahead of the stores (covers the load latency)

// MT = 128-row sub-tiles of a per CTA; they share the weight tile.
template <int MT> struct GemmCfg {
    static constexpr int kStageBytes = (2 * MT + 2) * kGPlane; // MT x (A hi | A lo), B hi | B lo
    static constexpr int kStages = MT == 1 ? 3 : 2;
    static constexpr int kSmem = kStages * kStageBytes;
    static constexpr int kOffB = 2 * MT * kGPlane;
    static constexpr uint32_t kCols = 2 * MT * 128;            // MT main + MT small-term accumulators
};

__device__ unsigned int g_gemm_error; // 0 = ok; otherwise (code << 24) | low bits of blockIdx.x

// byte offset of element (row r, depth k) inside a 128 x 32 plane
__host__ __device__ constexpr uint32_t plane_offset(int r, int k) {
    return (uint32_t)((k >> 2) * 2048 + (r >> 3) * 128 + (r & 7) * 16 + (k & 3) * 4);
}

// b [K, N] row-major -> packed [n tile][k step][hi | lo][16 KB plane], zero padded.
__global__ void __launch_bounds__(256) gemm5_pack_kernel(const float *b, int64_t ldb, int K, int N, int ksteps,
                                                         int ntn, uint8_t *packed) {
    const int64_t np = (int64_t)ntn * kGN;
    const int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (idx >= np * ksteps * kGK) return;
    const int n = (int)(idx % np), k = (int)(idx / np);
    const float x = (k < K && n < N) ? b[(int64_t)k * ldb + n] : 0.0f;
    const uint32_t hi = t5_tf32(x);
    const float lo = x - __uint_as_float(hi);
    const int64_t tile = ((int64_t)(n / kGN) * ksteps + k / kGK) * 2 * kGPlane;
    const uint32_t off = plane_offset(n % kGN, k % kGK);
    *reinterpret_cast<uint32_t *>(packed + tile + off) = hi;
    *reinterpret_cast<float *>(packed + tile + kGPlane + off) = lo;
}

template <bool X3, int MT>
__global__ void __launch_bounds__(kGThreads, 1)
    gemm5_kernel(const float *__restrict__ a, int64_t lda, const uint8_t *__restrict__ packed, const float *bias,
                 float *__restrict__ out, int64_t ldo, int M, int K, int N, int ksteps, int ntn, int vec_out) {
    using Cfg = GemmCfg<MT>;
    constexpr int S = Cfg::kStages;
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ __align__(8) uint64_t bar_a[S], bar_b[S], bar_empty[S], bar_done;
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int s_abort;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nt = blockIdx.x % ntn, mt = blockIdx.x / ntn; // column tiles fastest: neighbours share rows of a
    const int row0 = mt * (kGM * MT);
    const uint32_t sbase = smem_u32(smem);

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < S; ++s) {
            mbar_init(&bar_a[s], kGProducers / 32); // one arrival per producer warp
            mbar_init(&bar_b[s], 1);
            mbar_init(&bar_empty[s], 1);
        }
        mbar_init(&bar_done, 1);
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) {
        tmem_alloc(&tmem_slot, Cfg::kCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    bool failed = false;

    if (warp < 8) {
        // ---- producers: a tiles -> (hi, lo) planes ---------------------------------------------
        constexpr int NP = 4 * MT; // 16-byte pieces per thread and step
        float4 ar[kGPrefetch][NP];
        auto load_a = [&](int s, float4 (&dst)[NP]) {
#pragma unroll
            for (int it = 0; it < NP; ++it) {
                const int bid = it * 8 + warp; // 0 .. 32 MT - 1
                const int r = (bid & (16 * MT - 1)) * 8 + (lane & 7), c = (bid / (16 * MT)) * 4 + (lane >> 3);
                const int row = row0 + r, k = s * kGK + c * 4;
                dst[it] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (row < M && k < K) dst[it] = __ldg(reinterpret_cast<const float4 *>(a + (int64_t)row * lda + k));
            }
        };
        auto store_a = [&](int stage, const float4 (&src)[NP]) {
            uint8_t *base = smem + stage * Cfg::kStageBytes;
#pragma unroll
            for (int it = 0; it < NP; ++it) {
                const int bid = it * 8 + warp;
                const int r = (bid & (16 * MT - 1)) * 8 + (lane & 7), c = (bid / (16 * MT)) * 4 + (lane >> 3);
                const uint32_t off = (uint32_t)(r >> 7) * 2 * kGPlane + plane_offset(r & 127, c * 4);
                const float e[4] = {src[it].x, src[it].y, src[it].z, src[it].w};
                uint4 hi, lo;
                uint32_t *h4 = &hi.x, *l4 = &lo.x;
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    h4[x] = t5_tf32(e[x]);
                    l4[x] = __float_as_uint(e[x] - __uint_as_float(h4[x]));
                }
                *reinterpret_cast<uint4 *>(base + off) = hi;
                if (X3) *reinterpret_cast<uint4 *>(base + kGPlane + off) = lo;
            }
        };
#pragma unroll
        for (int u = 0; u < kGPrefetch; ++u)
            if (u < ksteps) load_a(u, ar[u]);
        for (int s0 = 0; s0 < ksteps && !failed; s0 += kGPrefetch) {
#pragma unroll
            for (int u = 0; u < kGPrefetch; ++u) {
                const int s = s0 + u;
                if (s >= ksteps) break;
                const int stage = s % S;
                if (s >= S) { // one lane polls for the warp
                    int ok = 1;
                    if (lane == 0) ok = mbar_wait_abort(&bar_empty[stage], ((s / S) - 1) & 1, &s_abort);
                    if (!__shfl_sync(0xffffffffu, ok, 0)) {
                        failed = true; // the MMAs of step s - S never released the stage
                        break;
                    }
                }
                store_a(stage, ar[u]);
                if (s + kGPrefetch < ksteps) load_a(s + kGPrefetch, ar[u]);
                fence_async_smem(); // every writer makes its stores visible to the tensor core ...
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_a[stage]); // ... then the warp arrives once
            }
        }
    } else if (warp == 8) {
        // ---- MMA issue ------------------------------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t kIdesc = t5_idesc(kGM, kGN, 0);
            for (int s = 0; s < ksteps; ++s) {
                const int stage = s % S;
                const uint32_t par = (s / S) & 1;
                if (!mbar_wait_abort(&bar_a[stage], par, &s_abort) || !mbar_wait_abort(&bar_b[stage], par, &s_abort)) {
                    failed = true;
                    break;
                }
                tc_fence_after();
                const uint32_t sb = sbase + stage * Cfg::kStageBytes;
#pragma unroll
                for (int ks = 0; ks < kGK / 8; ++ks) {
                    const uint64_t bh = t5_desc(sb + Cfg::kOffB + ks * 4096, 2048, 128);
                    const uint64_t bl = t5_desc(sb + Cfg::kOffB + kGPlane + ks * 4096, 2048, 128);
                    const uint32_t acc = (s > 0 || ks > 0) ? 1u : 0u;
#pragma unroll
                    for (int mi = 0; mi < MT; ++mi) {
                        const uint64_t ah = t5_desc(sb + mi * 2 * kGPlane + ks * 4096, 2048, 128);
                        const uint64_t al = t5_desc(sb + mi * 2 * kGPlane + kGPlane + ks * 4096, 2048, 128);
                        if (X3) { // the two small products have an accumulator of their own
                            mma_ss(tmem + (MT + mi) * 128, al, bh, kIdesc, acc);
                            mma_ss(tmem + (MT + mi) * 128, ah, bl, kIdesc, 1);
                        }
                        mma_ss(tmem + mi * 128, ah, bh, kIdesc, acc);
                    }
                }
                tc_commit(&bar_empty[stage]);
            }
            tc_commit(&bar_done); // arrives when everything issued above has completed
        }
    } else {
        // ---- weight tiles: one bulk copy per step ---------------------------------------------
        if (lane == 0) {
            const uint8_t *bsrc = packed + (int64_t)nt * ksteps * 2 * kGPlane;
            constexpr uint32_t kBBytes = X3 ? 2 * kGPlane : kGPlane; // hi and lo planes are adjacent
            int issued = 0;
            for (int s = 0; s < ksteps; ++s) {
                const int stage = s % S;
                if (s >= S && !mbar_wait_abort(&bar_empty[stage], ((s / S) - 1) & 1, &s_abort)) {
                    failed = true;
                    break;
                }
                mbar_expect_tx(&bar_b[stage], kBBytes);
                bulk_load(smem + stage * Cfg::kStageBytes + Cfg::kOffB, bsrc + (int64_t)s * 2 * kGPlane, kBBytes,
                          &bar_b[stage]);
                ++issued;
            }
            if (failed) { // copies still on their way into this CTA's shared memory
                for (int x = issued > S ? issued - S : 0; x < issued; ++x) mbar_wait(&bar_b[x % S], (x / S) & 1);
            }
        }
    }
    if (failed) s_abort = 1;

    // ---- epilogue: warps 0-7 read the accumulators (warp w: lanes 32 (w & 3).., columns 64 (w >> 2)..) ----
    if (warp < 8) {
        bool ok = !failed && ksteps > 0 ? mbar_wait_abort(&bar_done, 0, &s_abort) : !failed;
        ok = __all_sync(0xffffffffu, ok); // the TMEM loads below are warp-wide
        failed = !ok;
        if (failed) s_abort = 1;
        tc_fence_after();
        const uint32_t trow = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        const int chalf = (warp >> 2) * 64;
#pragma unroll
        for (int mi = 0; mi < MT; ++mi) {
            const int row = row0 + mi * kGM + (warp & 3) * 32 + lane;
            float *orow = out + (int64_t)(row < M ? row : 0) * ldo;
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                float v[32];
                if (!failed && ksteps > 0) { // uniform over the warp
                    tmem_ld32(trow + mi * 128 + chalf + q * 32, v);
                    if (X3) {
                        float w[32];
                        tmem_ld32(trow + (MT + mi) * 128 + chalf + q * 32, w);
                        tc_wait_ld();
#pragma unroll
                        for (int c = 0; c < 32; ++c) v[c] += w[c];
                    } else {
                        tc_wait_ld();
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < 32; ++c) v[c] = 0.0f;
                }
                if (row < M && !failed) {
                    const int col0 = nt * kGN + chalf + q * 32;
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        const int col = col0 + c * 4;
                        float4 o = make_float4(v[c * 4], v[c * 4 + 1], v[c * 4 + 2], v[c * 4 + 3]);
                        if (vec_out && col + 3 < N) {
                            if (bias) {
                                const float4 bb = __ldg(reinterpret_cast<const float4 *>(bias + col));
                                o.x += bb.x; o.y += bb.y; o.z += bb.z; o.w += bb.w;
                            }
                            *reinterpret_cast<float4 *>(orow + col) = o;
                        } else {
                            const float e[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                            for (int x = 0; x < 4; ++x)
                                if (col + x < N) orow[col + x] = e[x] + (bias ? bias[col + x] : 0.0f);
                        }
                    }
                }
            }
        }
    } else if (warp == 8 && lane == 0 && failed) {
        mbar_wait(&bar_done, 0); // bounded: let the MMAs in flight finish before the TMEM goes back
    }
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && s_abort) atomicCAS(&g_gemm_error, 0u, (2u << 24) | (blockIdx.x & 0xffffffu));
    if (warp == 8) tmem_dealloc(tmem, Cfg::kCols);
}

static int gemm5_configure() {
    static std::atomic<uint64_t> configured{0}; // one bit per device ordinal
    int dev = 0;
    FBLT_CUDA_TRY(cudaGetDevice(&dev));
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        FBLT_CUDA_TRY(cudaFuncSetAttribute(gemm5_kernel<true, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmCfg<1>::kSmem));
        FBLT_CUDA_TRY(cudaFuncSetAttribute(gemm5_kernel<false, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmCfg<1>::kSmem));
        FBLT_CUDA_TRY(cudaFuncSetAttribute(gemm5_kernel<true, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmCfg<2>::kSmem));
        FBLT_CUDA_TRY(cudaFuncSetAttribute(gemm5_kernel<false, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmCfg<2>::kSmem));
        configured.fetch_or(bit, std::memory_order_release);
    }
    return FBLT_OK;
}

// Error word of the matmul kernel: returns and clears it (device already synchronised).
int gemm5_take_error() {
    unsigned int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof(v)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(zero));
    return (int)v;
}

// 0 = choose by shape; 128 / 256 = rows of a per CTA (tuning knob, see fblt_matmul_set_rows_per_cta)
static std::atomic<int> g_gemm_rows_per_cta{0};

static inline int64_t ceil_div(int64_t x, int64_t y) { return (x + y - 1) / y; }

} // namespace fblt

extern "C" size_t fblt_matmul_packed_bytes(int64_t K, int64_t N) {
    using namespace fblt;
    if (K <= 0 || N <= 0) return 0;
    return (size_t)(ceil_div(N, kGN) * ceil_div(K, kGK)) * 2 * kGPlane;
}

extern "C" int fblt_matmul_pack_weights(const float *b, int64_t ldb, int64_t K, int64_t N, void *packed,
                                        size_t packed_bytes, void *stream) {
    using namespace fblt;
    if (!b || !packed || K <= 0 || N <= 0 || ldb < N) return fail(FBLT_ERR_ARG, "matmul_pack_weights: bad arguments");
    if (K > (1 << 24) || N > (1 << 24)) return fail(FBLT_ERR_LIMIT, "matmul_pack_weights: K or N above 2^24");
    if (packed_bytes < fblt_matmul_packed_bytes(K, N))
        return fail(FBLT_ERR_WORKSPACE, "matmul_pack_weights: packed buffer holds %zu bytes, %zu needed", packed_bytes,
                    fblt_matmul_packed_bytes(K, N));
    if ((uintptr_t)packed & 15) return fail(FBLT_ERR_ARG, "matmul_pack_weights: packed buffer must be 16-byte aligned");
    const int ksteps = (int)ceil_div(K, kGK), ntn = (int)ceil_div(N, kGN);
    const int64_t total = (int64_t)ntn * kGN * ksteps * kGK;
    gemm5_pack_kernel<<<(unsigned)ceil_div(total, 256), 256, 0, (cudaStream_t)stream>>>(b, ldb, (int)K, (int)N, ksteps,
                                                                                         ntn, (uint8_t *)packed);
    count_launch();
    return check_launch("gemm5_pack_kernel");
}

extern "C" int fblt_matmul(const float *a, int64_t lda, const void *packed_b, const float *bias, float *out,
                           int64_t ldo, int64_t M, int64_t K, int64_t N, int32_t precision, void *stream) {
    using namespace fblt;
    if (M < 0 || K <= 0 || N <= 0 || lda < K || ldo < N) return fail(FBLT_ERR_ARG, "matmul: bad shape or stride");
    if (M == 0) return FBLT_OK;
    if (!a || !packed_b || !out) return fail(FBLT_ERR_ARG, "matmul: buffers must not be NULL");
    if ((K & 3) || (lda & 3) || ((uintptr_t)a & 15))
        return fail(FBLT_ERR_UNSUPPORTED, "matmul: K and lda must be multiples of 4 and a 16-byte aligned");
    if ((uintptr_t)packed_b & 15) return fail(FBLT_ERR_ARG, "matmul: packed weights must be 16-byte aligned");
    if (K > (1 << 24) || N > (1 << 24) || M > (int64_t)INT32_MAX) return fail(FBLT_ERR_LIMIT, "matmul: shape too large");
    const int ksteps = (int)ceil_div(K, kGK), ntn = (int)ceil_div(N, kGN);
    const int mtile = (g_gemm_rows_per_cta == 128 || (g_gemm_rows_per_cta == 0 && M <= 128 * 148)) ? 1 : 2;
    const int64_t tiles = ceil_div(M, kGM * mtile) * ntn;
    if (tiles > (int64_t)INT32_MAX) return fail(FBLT_ERR_LIMIT, "matmul: too many tiles");
    const int st = gemm5_configure();
    if (st != FBLT_OK) return st;
    const int vec_out = !((ldo & 3) || ((uintptr_t)out & 15) || (bias && ((uintptr_t)bias & 15)));
    const bool x3 = precision != FBLT_PREC_TF32;
#define FBLT_GEMM_LAUNCH(X3_, MT_)                                                                              \
    gemm5_kernel<X3_, MT_><<<(unsigned)tiles, kGThreads, GemmCfg<MT_>::kSmem, (cudaStream_t)stream>>>(          \
        a, lda, (const uint8_t *)packed_b, bias, out, ldo, (int)M, (int)K, (int)N, ksteps, ntn, vec_out)
    if (mtile == 1) {
        if (x3) FBLT_GEMM_LAUNCH(true, 1);
        else FBLT_GEMM_LAUNCH(false, 1);
    } else {
        if (x3) FBLT_GEMM_LAUNCH(true, 2);
        else FBLT_GEMM_LAUNCH(false, 2);
    }
#undef FBLT_GEMM_LAUNCH
    count_launch();
    return check_launch("gemm5_kernel");
}

extern "C" int fblt_matmul_set_rows_per_cta(int32_t rows) {
    if (rows != 0 && rows != 128 && rows != 256) return fblt::fail(FBLT_ERR_ARG, "matmul_set_rows_per_cta: 0, 128 or 256");
    fblt::g_gemm_rows_per_cta.store(rows);
    return FBLT_OK;
}
