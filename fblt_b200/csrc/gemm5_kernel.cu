// Dense matmul out[M,N] = a[M,K] * b[K,N] (+ bias) in fp32, the projection GEMMs on both
// sides of the attention operator (blt_matmul: ops/linalg_cpu.c:8-18 on the CPU,
// cublasSgemm in ops/linalg.cu:134-136), on the 5th-generation tensor cores.
//
//   b      = packed once (weights are constant between calls): split into TF32 (hi, lo)
//            parts and laid out tile by tile in the exact shared-memory image the MMA reads
//            (no-swizzle K-major core matrices, [n][k] order), so one thread brings a
//            128 x 32 weight tile in with one bulk copy that completes on an mbarrier.
//   a      = one thread brings each raw 128 x 32 fp32 tile in with a tiled TMA load (128-byte
//            swizzle, rows past M and depth past K filled with zeros by the copy engine).
//            The A operand of the MMA lives in TMEM, not in shared memory: a group of four
//            producer warps (thread = one row of the tile = one TMEM lane) reads its rows
//            from the swizzled tile without bank conflicts, splits them into (hi, lo) and
//            writes both with tcgen05.st. Two such groups take the steps in turn: one
//            conversion is a chain of waits, and the chains of consecutive steps overlap.
//   MMA    = one thread; per 8-deep slice one tcgen05.mma of shape 128x256x8 (A hi from TMEM
//            against the weight tile's high | low halves: hi*hi into the main accumulator,
//            hi*lo into the small-term accumulator beside it) and one of shape 128x128x8
//            (A lo * weight hi onto the small terms), fp32 accumulate in TMEM;
//            tcgen05.commit hands the stage back. Issuing an MMA costs the thread about as
//            long as the MMA runs, so fewer, wider instructions and one barrier per stage keep
//            the tensor pipe fed. The small terms are kept apart because the tensor core
//            truncates when it adds into the accumulator: one addition per 8-deep slice into
//            the main sum, not three.
//   out    = four epilogue warps (warp q: TMEM lanes 32 q ..) read main + small accumulators,
//            hand the TMEM back to the MMA thread, add the bias and store. The CTA is
//            persistent (one per SM), so the next tile's loads and conversions run meanwhile.
//   No __syncthreads in the main loop: the five roles meet only on mbarriers (raw a landed,
//   raw a read, a in TMEM + b landed, stage free, tile done, accumulators read).
//
// TMEM columns: [0,128) main accumulator, [128,256) small terms, 256 + 64 stage: A hi | A lo.
//
// Every mbarrier wait is bounded and watches a CTA-wide abort word; a role that gives up
// raises it, the CTA records an error code, waits (bounded) for its copies and MMAs in
// flight, frees its TMEM and returns.
#include "common.cuh"
#include "tc5.cuh"

#include <atomic>
#include <string.h>
#include <cuda.h> // CUtensorMap and its enums only; the encoder is looked up at run time

namespace fblt {

constexpr int kGM = 128, kGN = 128, kGK = 32;
constexpr int kGGroups = 2;                    // producer groups of four warps; group g converts steps g, g + 2, ...
constexpr int kGWarpEpi = kGGroups * 4;        // four epilogue warps follow the producer warps
constexpr int kGWarpMma = kGWarpEpi + 4, kGWarpB = kGWarpMma + 1; // MMA issue (and TMEM owner); weight copies; a tiles
constexpr int kGThreads = (kGWarpB + 2) * 32;
constexpr int kGPlane = kGN * kGK * 4;         // 16 KB: one (hi or lo) plane of a 128 x 32 weight tile
constexpr int kGStages = 4;
constexpr int kGStageBytes = 2 * kGPlane;      // B hi | B lo
constexpr int kGRawBytes = kGM * kGK * 4;      // 16 KB: one raw fp32 tile of a (row = 128 bytes, 128-byte swizzle)
constexpr int kGOffRaw = kGStages * kGStageBytes;
constexpr int kGSmem = kGOffRaw + kGStages * kGRawBytes;
constexpr uint32_t kGColSmall = 128, kGColA = 256, kGCols = 512;

// Epilogue of the QKV projection of a cache-aware decode step (infer/kv_cache.c:338-366): instead of
// storing the [rows, 3E] product, column section 0 (Q) is rotated and stored to q_out, sections 1 and 2
// (K, V) go straight to the cache rows of their positions, K rotated. Row = sequence b * n_new + r,
// position = base_len[b] + base_add + r. A 32-column chunk never straddles a section or a head
// (E and head_dim are multiples of 32). enabled == 0: the plain store.
struct QkvScatter {
    int enabled; // 0 plain store, 1 decode step (scatter into the cache), 2 prefill (rotate Q / K, store in place)
    int E, HD, n_new, base_add;
    const int32_t *base_len; // mode 2: cu_rows [batch + 1] of the packed sequences, batch in n_new
    float *q_out;
    int64_t q_stride;
    float *kc, *vc;
    int64_t seq_stride, row_stride;
    const float *rope_cos, *rope_sin; // [positions, HD / 2] or NULL
};

__device__ unsigned int g_gemm_error; // 0 = ok; otherwise (code << 24) | low bits of blockIdx.x

// Byte offset of the high part of weight element (column r of the tile, depth k) inside a
// 32 KB tile; the low part sits 2 KB further. Per 16-byte depth piece the tile holds 128 rows of
// the high plane and then 128 rows of the low plane, so that the pair reads as one 256-row
// K-major operand (high | low) and its first half as the 128-row high operand.
__host__ __device__ constexpr uint32_t plane_offset(int r, int k) {
    return (uint32_t)((k >> 2) * 4096 + (r >> 3) * 128 + (r & 7) * 16 + (k & 3) * 4);
}

// b [K, N] row-major -> packed [n tile][k step][32 KB tile, see plane_offset], zero padded.
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
    *reinterpret_cast<float *>(packed + tile + 2048 + off) = lo;
}

template <bool X3>
__global__ void __launch_bounds__(kGThreads, 1)
    gemm5_kernel(const __grid_constant__ CUtensorMap a_map, const uint8_t *__restrict__ packed, const float *bias,
                 float *__restrict__ out, int64_t ldo, int M, int N, int ksteps, int ntn, int tiles, int vec_out,
                 const QkvScatter sc) {
    constexpr int S = kGStages;
    extern __shared__ __align__(1024) uint8_t smem[];
    // bar_full: A operand in TMEM (4 warp arrivals) and weight tile landed (1 arrival + bytes);
    // bar_done: a tile's MMAs are complete; bar_acc_free: the epilogue has read the accumulators
    __shared__ __align__(8) uint64_t bar_full[S], bar_empty[S], bar_raw[S], bar_raw_free[S], bar_done, bar_acc_free;
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int s_abort;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t sbase = smem_u32(smem);

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < S; ++s) {
            mbar_init(&bar_full[s], 4 + 1);
            mbar_init(&bar_empty[s], 1);
            mbar_init(&bar_raw[s], 1);
            mbar_init(&bar_raw_free[s], 4);
        }
        mbar_init(&bar_done, 1);
        mbar_init(&bar_acc_free, 4);
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kGWarpMma) {
        tmem_alloc(&tmem_slot, kGCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    bool failed = false;

    // The CTA is persistent: it takes tiles blockIdx.x, blockIdx.x + gridDim.x, ... (column tiles
    // fastest, so CTAs running together share rows of a). Every role walks the same tile list
    // with a running step count g, which also gives ring stage and barrier parity.
    if (warp < kGWarpEpi) {
        // ---- producers: a rows -> (hi, lo) TF32 parts in TMEM -------------------------------------
        // The conversion of one step is a chain of waits (tile landed, stage free, TMEM store
        // done); the groups take the steps in turn so that the chains overlap.
        const int quarter = warp & 3, group = warp >> 2;
        const int r = quarter * 32 + lane; // row of the tile = TMEM lane
        const uint32_t tlane = tmem + ((uint32_t)(quarter * 32) << 16) + kGColA;
        int g0 = 0;
        for (int tile = blockIdx.x; tile < tiles && !failed; tile += gridDim.x, g0 += ksteps) {
            for (int s = 0; s < ksteps; ++s) {
                const int g = g0 + s;
                if (g % kGGroups != group) continue;
                const int stage = g % S;
                int ok = 1;
                if (lane == 0) ok = mbar_wait_abort(&bar_raw[stage], (g / S) & 1, &s_abort); // one lane polls for the warp
                if (!__shfl_sync(0xffffffffu, ok, 0)) {
                    failed = true;
                    break;
                }
                __syncwarp(); // lane 0's acquire of the barrier orders every lane's reads below
                // this row's 32 depth values: 16-byte piece c of row r sits at piece c ^ (r & 7)
                const uint8_t *raw = smem + kGOffRaw + stage * kGRawBytes + r * 128;
                float4 v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = *reinterpret_cast<const float4 *>(raw + ((j ^ (r & 7)) << 4));
                uint32_t hi[32], lo[32];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float e[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
                    for (int x = 0; x < 4; ++x) {
                        hi[j * 4 + x] = t5_tf32(e[x]);
                        lo[j * 4 + x] = __float_as_uint(e[x] - __uint_as_float(hi[j * 4 + x]));
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_raw_free[stage]); // the raw tile may be overwritten
                if (g >= S) {
                    if (lane == 0) ok = mbar_wait_abort(&bar_empty[stage], ((g / S) - 1) & 1, &s_abort);
                    if (!__shfl_sync(0xffffffffu, ok, 0)) {
                        failed = true; // the MMAs of step g - S never released the stage
                        break;
                    }
                    tc_fence_after();
                }
                tmem_st32(tlane + stage * 64, hi);
                if (X3) tmem_st32(tlane + stage * 64 + 32, lo);
                tc_wait_st();
                tc_fence_before(); // the TMEM stores are complete and ordered before ...
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_full[stage]); // ... the warp's arrival
            }
        }
    } else if (warp < kGWarpMma) {
        // ---- epilogue: warp q reads TMEM lanes 32 q .. (one output row per thread) ------------------
        const int quarter = warp - kGWarpEpi;
        const uint32_t trow = tmem + ((uint32_t)(quarter * 32) << 16);
        int it = 0;
        for (int tile = blockIdx.x; tile < tiles && !failed; tile += gridDim.x, ++it) {
            const int nt = tile % ntn, mt = tile / ntn;
            int ok = 1;
            if (lane == 0) ok = mbar_wait_abort(&bar_done, it & 1, &s_abort);
            if (!__shfl_sync(0xffffffffu, ok, 0)) {
                failed = true;
                break;
            }
            tc_fence_after();
            const int row = mt * kGM + quarter * 32 + lane;
            float *orow = out + (int64_t)(row < M ? row : 0) * ldo;
            int pos_row = -1;
#pragma unroll
            for (int q = 0; q < kGN / 32; ++q) {
                float v[32];
                tmem_ld32(trow + q * 32, v);
                if (X3) {
                    float w[32];
                    tmem_ld32(trow + kGColSmall + q * 32, w);
                    tc_wait_ld();
#pragma unroll
                    for (int c = 0; c < 32; ++c) v[c] += w[c];
                } else {
                    tc_wait_ld();
                }
                if (q == kGN / 32 - 1) { // everything is in registers: the next tile may overwrite the accumulators
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bar_acc_free);
                }
                if (row < M && sc.enabled == 2) {
                    // prefill: position = row index inside the packed sequence that holds the row
                    const int col0 = nt * kGN + q * 32;
                    if (col0 < N) {
                        const int section = col0 / sc.E, dcol = (col0 - section * sc.E) % sc.HD;
                        if (section < 2) {
                            if (q == 0 || pos_row < 0) { // upper bound of row in cu_rows, once per tile
                                int lo = 0, hi = sc.n_new;
                                while (hi - lo > 1) {
                                    const int mid = (lo + hi) >> 1;
                                    if (__ldg(sc.base_len + mid) <= row) lo = mid;
                                    else hi = mid;
                                }
                                pos_row = row - __ldg(sc.base_len + lo);
                            }
                            const int half = sc.HD / 2;
                            const float *cs = sc.rope_cos + (int64_t)pos_row * half + dcol / 2;
                            const float *sn = sc.rope_sin + (int64_t)pos_row * half + dcol / 2;
#pragma unroll
                            for (int pr = 0; pr < 16; pr += 2) {
                                const float2 c2 = __ldg(reinterpret_cast<const float2 *>(cs + pr));
                                const float2 s2 = __ldg(reinterpret_cast<const float2 *>(sn + pr));
                                rope_rotate(v[2 * pr], v[2 * pr + 1], c2.x, s2.x);
                                rope_rotate(v[2 * pr + 2], v[2 * pr + 3], c2.y, s2.y);
                            }
                        }
#pragma unroll
                        for (int c = 0; c < 8; ++c)
                            *reinterpret_cast<float4 *>(orow + col0 + c * 4) = make_float4(v[c * 4], v[c * 4 + 1], v[c * 4 + 2], v[c * 4 + 3]);
                    }
                } else if (row < M && sc.enabled) {
                    const int col0 = nt * kGN + q * 32;
                    if (col0 < N) {
                        const int section = col0 / sc.E, ce = col0 - section * sc.E, dcol = ce % sc.HD;
                        const int b = row / sc.n_new, r = row - b * sc.n_new;
                        const int pos = sc.base_len[b] + sc.base_add + r;
                        if (section < 2 && sc.rope_cos) { // interleaved pairs, products and sums rounded separately
                            const int half = sc.HD / 2;
                            const float *cs = sc.rope_cos + (int64_t)pos * half + dcol / 2;
                            const float *sn = sc.rope_sin + (int64_t)pos * half + dcol / 2;
#pragma unroll
                            for (int pr = 0; pr < 16; pr += 2) {
                                const float2 c2 = __ldg(reinterpret_cast<const float2 *>(cs + pr));
                                const float2 s2 = __ldg(reinterpret_cast<const float2 *>(sn + pr));
                                rope_rotate(v[2 * pr], v[2 * pr + 1], c2.x, s2.x);
                                rope_rotate(v[2 * pr + 2], v[2 * pr + 3], c2.y, s2.y);
                            }
                        }
                        float *dst = section == 0 ? sc.q_out + (int64_t)row * sc.q_stride + ce
                                                  : (section == 1 ? sc.kc : sc.vc) + (int64_t)b * sc.seq_stride +
                                                        (int64_t)pos * sc.row_stride + ce;
#pragma unroll
                        for (int c = 0; c < 8; ++c)
                            *reinterpret_cast<float4 *>(dst + c * 4) = make_float4(v[c * 4], v[c * 4 + 1], v[c * 4 + 2], v[c * 4 + 3]);
                    }
                } else if (row < M) {
                    const int col0 = nt * kGN + q * 32;
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
    } else if (warp == kGWarpMma) {
        // ---- MMA issue ------------------------------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t kIdesc128 = t5_idesc(kGM, kGN, 0), kIdesc256 = t5_idesc(kGM, 2 * kGN, 0);
            const uint64_t desc0 = t5_desc(sbase, 4096, 128); // + (byte offset >> 4) selects stage and depth slice
            int g = 0, it = 0;
            for (int tile = blockIdx.x; tile < tiles && !failed; tile += gridDim.x, ++it) {
                if (it > 0) { // the previous tile's accumulators must have been read out
                    if (!mbar_wait_abort(&bar_acc_free, (it - 1) & 1, &s_abort)) {
                        failed = true;
                        break;
                    }
                    tc_fence_after();
                }
                for (int s = 0; s < ksteps; ++s, ++g) {
                    const int stage = g % S;
                    if (!mbar_wait_abort(&bar_full[stage], (g / S) & 1, &s_abort)) {
                        failed = true;
                        break;
                    }
                    tc_fence_after();
                    const uint64_t db = desc0 + (uint64_t)(stage * (kGStageBytes >> 4));
                    const uint32_t ta = tmem + kGColA + stage * 64;
#pragma unroll
                    for (int ks = 0; ks < kGK / 8; ++ks) {
                        const uint64_t bd = db + (uint64_t)(ks * (8192 >> 4));
                        const uint32_t ah = ta + ks * 8, al = ta + 32 + ks * 8;
                        const uint32_t acc = (s > 0 || ks > 0) ? 1u : 0u;
                        if (X3) {
                            // one 256-wide MMA: columns [0,128) += hi*hi, columns [128,256) += hi*lo (the
                            // small terms keep an accumulator of their own); then lo*hi onto the small terms
                            mma_ts(tmem, ah, bd, kIdesc256, acc);
                            mma_ts(tmem + kGColSmall, al, bd, kIdesc128, 1);
                        } else {
                            mma_ts(tmem, ah, bd, kIdesc128, acc);
                        }
                    }
                    tc_commit(&bar_empty[stage]);
                }
                if (!failed) tc_commit(&bar_done); // arrives when this tile's MMAs have completed
            }
        }
    } else if (warp == kGWarpB) {
        // ---- weight tiles: one bulk copy per step ---------------------------------------------
        if (lane == 0) {
            constexpr uint32_t kBBytes = X3 ? 2 * kGPlane : kGPlane;
            int g = 0, issued = 0;
            for (int tile = blockIdx.x; tile < tiles && !failed; tile += gridDim.x) {
                const uint8_t *bsrc = packed + (int64_t)(tile % ntn) * ksteps * 2 * kGPlane;
                for (int s = 0; s < ksteps; ++s, ++g) {
                    const int stage = g % S;
                    if (g >= S && !mbar_wait_abort(&bar_empty[stage], ((g / S) - 1) & 1, &s_abort)) {
                        failed = true;
                        break;
                    }
                    mbar_expect_tx(&bar_full[stage], kBBytes);
                    if (X3) {
                        bulk_load(smem + stage * kGStageBytes, bsrc + (int64_t)s * 2 * kGPlane, kBBytes, &bar_full[stage]);
                    } else { // single pass: only the high halves of the eight depth pieces
#pragma unroll
                        for (int pc = 0; pc < 8; ++pc)
                            bulk_load(smem + stage * kGStageBytes + pc * 4096, bsrc + (int64_t)s * 2 * kGPlane + pc * 4096,
                                      2048, &bar_full[stage]);
                    }
                    ++issued;
                }
            }
            if (failed) { // copies still on their way into this CTA's shared memory
                for (int x = issued > S ? issued - S : 0; x < issued; ++x) mbar_wait(&bar_full[x % S], (x / S) & 1);
            }
        }
    } else {
        // ---- raw a tiles: one tiled TMA load per step -----------------------------------------
        if (lane == 0) {
            int g = 0, issued = 0;
            for (int tile = blockIdx.x; tile < tiles && !failed; tile += gridDim.x) {
                const int row0 = (tile / ntn) * kGM;
                for (int s = 0; s < ksteps; ++s, ++g) {
                    const int stage = g % S;
                    if (g >= S && !mbar_wait_abort(&bar_raw_free[stage], ((g / S) - 1) & 1, &s_abort)) {
                        failed = true;
                        break;
                    }
                    mbar_expect_tx(&bar_raw[stage], kGRawBytes);
                    tma_load_2d(smem + kGOffRaw + stage * kGRawBytes, &a_map, s * kGK, row0, &bar_raw[stage]);
                    ++issued;
                }
            }
            if (failed) {
                for (int x = issued > S ? issued - S : 0; x < issued; ++x) mbar_wait(&bar_raw[x % S], (x / S) & 1);
            }
        }
    }
    if (failed) s_abort = 1;
    if (warp == kGWarpMma && lane == 0 && failed) {
        tc_commit(&bar_done);
        mbar_wait(&bar_done, 0); // bounded: let the MMAs in flight finish before the TMEM goes back
        mbar_wait(&bar_done, 1);
    }
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && s_abort) atomicCAS(&g_gemm_error, 0u, (2u << 24) | (blockIdx.x & 0xffffffu));
    if (warp == kGWarpMma) tmem_dealloc(tmem, kGCols);
}

// cuTensorMapEncodeTiled, looked up through the runtime so that the library does not link libcuda.
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn tensor_map_encoder() {
    static std::atomic<EncodeTiledFn> cached{nullptr};
    EncodeTiledFn fn = cached.load(std::memory_order_acquire);
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        fn = (EncodeTiledFn)p;
        cached.store(fn, std::memory_order_release);
    }
    return fn;
}

// Map of a [M, K] (row stride lda) for 128-row x 32-column boxes, 128-byte swizzle, zero fill.
static int make_a_map(CUtensorMap *map, const float *a, int64_t lda, int64_t M, int64_t K) {
    EncodeTiledFn enc = tensor_map_encoder();
    if (!enc) return fail(FBLT_ERR_CUDA, "matmul: cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)lda * sizeof(float)};
    const cuuint32_t box[2] = {(cuuint32_t)kGK, (cuuint32_t)kGM};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void *)a, dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(FBLT_ERR_CUDA, "matmul: cuTensorMapEncodeTiled failed with code %d", (int)r);
    return FBLT_OK;
}

static int gemm5_configure() {
    static std::atomic<uint64_t> configured{0}; // one bit per device ordinal
    int dev = 0;
    FBLT_CUDA_TRY(cudaGetDevice(&dev));
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        FBLT_CUDA_TRY(cudaFuncSetAttribute(gemm5_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kGSmem));
        FBLT_CUDA_TRY(cudaFuncSetAttribute(gemm5_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kGSmem));
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

int gemm5_take_error_on(cudaStream_t s) { // the same, ordered with one stream only
    unsigned int v = 0, zero = 0;
    if (cudaMemcpyFromSymbolAsync(&v, g_gemm_error, sizeof(v), 0, cudaMemcpyDeviceToHost, s) != cudaSuccess) return -1;
    if (cudaStreamSynchronize(s) != cudaSuccess) return -1;
    if (v) {
        cudaMemcpyToSymbolAsync(g_gemm_error, &zero, sizeof(zero), 0, cudaMemcpyHostToDevice, s);
        cudaStreamSynchronize(s);
    }
    return (int)v;
}

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

namespace fblt {
static int matmul_impl(const float *a, int64_t lda, const void *packed_b, const float *bias, float *out, int64_t ldo,
                       int64_t M, int64_t K, int64_t N, int32_t precision, void *stream, const QkvScatter &sc) {
    if (M < 0 || K <= 0 || N <= 0 || lda < K || (sc.enabled != 1 && ldo < N)) return fail(FBLT_ERR_ARG, "matmul: bad shape or stride");
    if (M == 0) return FBLT_OK;
    if (!a || !packed_b || !out) return fail(FBLT_ERR_ARG, "matmul: buffers must not be NULL");
    if ((K & 3) || (lda & 3) || ((uintptr_t)a & 15))
        return fail(FBLT_ERR_UNSUPPORTED, "matmul: K and lda must be multiples of 4 and a 16-byte aligned");
    if ((uintptr_t)packed_b & 15) return fail(FBLT_ERR_ARG, "matmul: packed weights must be 16-byte aligned");
    if (K > (1 << 24) || N > (1 << 24) || M > (int64_t)INT32_MAX) return fail(FBLT_ERR_LIMIT, "matmul: shape too large");
    const int ksteps = (int)ceil_div(K, kGK), ntn = (int)ceil_div(N, kGN);
    const int64_t tiles = ceil_div(M, kGM) * ntn;
    if (tiles > (int64_t)INT32_MAX) return fail(FBLT_ERR_LIMIT, "matmul: too many tiles");
    const int st = gemm5_configure();
    if (st != FBLT_OK) return st;
    const int vec_out = !((ldo & 3) || ((uintptr_t)out & 15) || (bias && ((uintptr_t)bias & 15)));
    CUtensorMap a_map;
    const int mst = make_a_map(&a_map, a, lda, M, K);
    if (mst != FBLT_OK) return mst;
    int dev = 0, sms = 0;
    FBLT_CUDA_TRY(cudaGetDevice(&dev));
    FBLT_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const unsigned grid = (unsigned)(tiles < sms ? tiles : sms); // one persistent CTA per SM
    if (precision != FBLT_PREC_TF32)
        gemm5_kernel<true><<<grid, kGThreads, kGSmem, (cudaStream_t)stream>>>(
            a_map, (const uint8_t *)packed_b, bias, out, ldo, (int)M, (int)N, ksteps, ntn, (int)tiles, vec_out, sc);
    else
        gemm5_kernel<false><<<grid, kGThreads, kGSmem, (cudaStream_t)stream>>>(
            a_map, (const uint8_t *)packed_b, bias, out, ldo, (int)M, (int)N, ksteps, ntn, (int)tiles, vec_out, sc);
    count_launch();
    return check_launch("gemm5_kernel");
}

// The QKV projection of a decode step with the scatter epilogue: rotated Q rows to q_out, rotated K and
// V rows straight into the cache (see QkvScatter). E and head_dim must be multiples of 32.
int matmul_qkv_to_cache(const float *a, int64_t lda, const void *packed_qkv, int64_t rows, int64_t E, int32_t head_dim,
                        int32_t n_new, const int32_t *base_len, int32_t base_add, float *q_out, int64_t q_stride,
                        float *kc, float *vc, int64_t seq_stride, int64_t row_stride, const float *rope_cos,
                        const float *rope_sin, int32_t precision, void *stream) {
    if ((E & 31) || (head_dim & 31) || head_dim <= 0 || E % head_dim)
        return fail(FBLT_ERR_UNSUPPORTED, "qkv scatter: embed_dim and head_dim must be multiples of 32");
    if (((uintptr_t)q_out | (uintptr_t)kc | (uintptr_t)vc) & 15 || ((q_stride | seq_stride | row_stride) & 3))
        return fail(FBLT_ERR_ARG, "qkv scatter: destinations must be 16-byte aligned with strides in multiples of 4");
    if (((uintptr_t)rope_cos | (uintptr_t)rope_sin) & 7) return fail(FBLT_ERR_ARG, "qkv scatter: rotary tables must be 8-byte aligned");
    QkvScatter sc;
    sc.enabled = 1;
    sc.E = (int)E;
    sc.HD = head_dim;
    sc.n_new = n_new;
    sc.base_add = base_add;
    sc.base_len = base_len;
    sc.q_out = q_out;
    sc.q_stride = q_stride;
    sc.kc = kc;
    sc.vc = vc;
    sc.seq_stride = seq_stride;
    sc.row_stride = row_stride;
    sc.rope_cos = rope_cos;
    sc.rope_sin = rope_sin;
    return matmul_impl(a, lda, packed_qkv, nullptr, q_out, q_stride, rows, E, 3 * E, precision, stream, sc);
}

// The QKV projection of a self-attention prefill with the rotation in the epilogue: out [rows, 3E] holds
// Q and K rotated with each row's position inside its packed sequence (cu_rows [batch + 1]) and V as it is
// (models/attention.c:156-160 in one launch). E and head_dim multiples of 32, out 16-byte aligned, ldo % 4 == 0.
int matmul_qkv_rotated(const float *a, int64_t lda, const void *packed_qkv, int64_t rows, int64_t E, int32_t head_dim,
                       const int32_t *cu_rows, int32_t batch, float *out, int64_t ldo, const float *rope_cos,
                       const float *rope_sin, int32_t precision, void *stream) {
    if ((E & 31) || (head_dim & 31) || head_dim <= 0 || E % head_dim)
        return fail(FBLT_ERR_UNSUPPORTED, "qkv rotation: embed_dim and head_dim must be multiples of 32");
    if (((uintptr_t)out & 15) || (ldo & 3) || ldo < 3 * E)
        return fail(FBLT_ERR_ARG, "qkv rotation: out must be 16-byte aligned with a row stride >= 3E in multiples of 4");
    if (!cu_rows || batch < 1 || !rope_cos || !rope_sin) return fail(FBLT_ERR_ARG, "qkv rotation: tables must not be NULL");
    if (((uintptr_t)rope_cos | (uintptr_t)rope_sin) & 7) return fail(FBLT_ERR_ARG, "qkv rotation: rotary tables must be 8-byte aligned");
    QkvScatter sc;
    memset(&sc, 0, sizeof(sc));
    sc.enabled = 2;
    sc.E = (int)E;
    sc.HD = head_dim;
    sc.n_new = batch;
    sc.base_len = cu_rows;
    sc.rope_cos = rope_cos;
    sc.rope_sin = rope_sin;
    return matmul_impl(a, lda, packed_qkv, nullptr, out, ldo, rows, E, 3 * E, precision, stream, sc);
}
} // namespace fblt

extern "C" int fblt_matmul(const float *a, int64_t lda, const void *packed_b, const float *bias, float *out,
                           int64_t ldo, int64_t M, int64_t K, int64_t N, int32_t precision, void *stream) {
    fblt::NvtxRange nvtx_range("fblt_matmul");
    fblt::QkvScatter none;
    memset(&none, 0, sizeof(none));
    return fblt::matmul_impl(a, lda, packed_b, bias, out, ldo, M, K, N, precision, stream, none);
}
