// L1 tcgen05 tile kernel (head_dim 64): the same range-masked attention as
// tile_kernel.cu, with both GEMMs on the 5th-generation tensor cores.
//
//   CTA   = (128 query rows, head, sequence), 128 threads: thread t owns row t,
//           which is also TMEM lane t, so the softmax needs no shuffles.
//   Q     = loaded once, split into TF32 (hi, lo) parts, kept in TMEM as the A
//           operand of S = Q K^T (128 columns).
//   K, V  = 64-key tiles; every thread loads 16-byte pieces from HBM, splits
//           them into (hi, lo) and stores them in the no-swizzle K-major UMMA
//           core-matrix layout (K as [key][dim], V transposed to [dim][key]).
//   S     = 3 x 8 tcgen05.mma (lo*hi + hi*lo + hi*hi) of shape 128x64x8 into
//           64 TMEM columns; one elected thread issues, tcgen05.commit arrives on
//           an mbarrier, every thread reads its row back with tcgen05.ld.
//   P     = softmax in registers (log2 domain, finite-only maximum, key range per
//           row), split into (hi, lo), stored K-major in shared memory; the hi
//           plane reuses the K tile's space, which is free once S is complete.
//   O     = 3 x 8 tcgen05.mma of shape 128x64x8 accumulating in 64 TMEM columns;
//           rescaled in TMEM only when a row's maximum moved.
//
// 96 KB of shared memory and 256 TMEM columns per CTA: two CTAs share an SM and
// overlap each other's load / MMA / softmax phases.
//
// Every mbarrier wait is bounded: after kSpinLimit polls the CTA records an
// error code, stops issuing work, frees its TMEM and returns.
#include "common.cuh"
#include "tc5.cuh"

#include <atomic>
#include <limits.h>

namespace fblt {

constexpr int kT5Rows = 128, kT5Keys = 64, kT5HD = 64, kT5Threads = 128;
constexpr int kPlaneKV = kT5Keys * kT5HD * 4;   // 16 KB: one (hi or lo) plane of a K or V tile
constexpr int kPlaneP = kT5Rows * kT5Keys * 4;  // 32 KB: one plane of P
// shared memory map (bytes): [0,32K) K hi|lo, reused by P hi; [32K,64K) V hi|lo; [64K,96K) P lo
constexpr int kOffK = 0, kOffV = 2 * kPlaneKV, kOffPlo = 4 * kPlaneKV, kT5Smem = 4 * kPlaneKV + kPlaneP;
// TMEM columns
constexpr uint32_t kColQhi = 0, kColQlo = 64, kColS = 128, kColO = 192, kT5Cols = 256;

__device__ unsigned int g_t5_error; // 0 = ok; otherwise (code << 24) | blockIdx.x of the first CTA that gave up

// ---- the kernel -----------------------------------------------------------------

// Rounding of an input element. With the low part present (three-pass mode) a NaN or an infinity in
// the element reaches the score through hi or through lo = x - hi whatever the rounding does to
// the bit pattern, so the pass-through test of t5_tf32 is only needed in single-pass mode.
template <bool X3>
__device__ __forceinline__ uint32_t t5_round_in(float x) {
    return X3 ? t5_tf32_finite(x) : t5_tf32(x);
}

template <bool X3>
__global__ void __launch_bounds__(kT5Threads, 2) tile5_attn_kernel(fblt_attn_desc d) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ __align__(8) uint64_t bar_s, bar_o, bar_fin; // bar_fin: used once, on the failure path
    __shared__ uint32_t tmem_slot;
    __shared__ int s_lo[4], s_hi[4]; // per-warp minimum / maximum of the rows' key ranges

    const int b = blockIdx.z, h = blockIdx.y, qt = blockIdx.x;
    const int q0 = d.cu_q[b], nq = d.cu_q[b + 1] - q0;
    const int k0 = d.cu_k[b], nk = d.cu_k[b + 1] - k0;
    if (qt * kT5Rows >= nq) return; // before any allocation or barrier
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int i = qt * kT5Rows + tid; // this thread's query row
    const uint32_t sbase = smem_u32(smem);

    if (tid == 0) {
        mbar_init(&bar_s, 1);
        mbar_init(&bar_o, 1);
        mbar_init(&bar_fin, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        tmem_alloc(&tmem_slot, kT5Cols);
        tmem_relinquish();
    }
    int lo = INT_MAX, hi = 0;
    if (i < nq) {
        const SeqMask s = resolve_mask(d.mask, b, q0, k0, nq, nk);
        row_range(s, i, lo, hi);
        if (hi <= lo) {
            lo = INT_MAX;
            hi = 0;
        }
    }
    {
        int wl = lo, wh = hi;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            wl = min(wl, __shfl_xor_sync(0xffffffffu, wl, o));
            wh = max(wh, __shfl_xor_sync(0xffffffffu, wh, o));
        }
        if (lane == 0) {
            s_lo[warp] = wl;
            s_hi[warp] = wh;
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    const uint32_t trow = tmem + ((uint32_t)(warp * 32) << 16); // this warp's lanes

    const int cmin = min(min(s_lo[0], s_lo[1]), min(s_lo[2], s_lo[3]));
    const int cmax = max(max(s_hi[0], s_hi[1]), max(s_hi[2], s_hi[3]));
    const int kt_begin = cmax > 0 ? cmin / kT5Keys : 0;
    const int kt_end = cmax > 0 ? (cmax + kT5Keys - 1) / kT5Keys : 0;

    constexpr uint32_t kIdescS = t5_idesc(kT5Rows, kT5Keys, 0);
    constexpr uint32_t kIdescO = t5_idesc(kT5Rows, kT5HD, 0);
    const float *kbase = d.k + (int64_t)k0 * d.k_stride + (int64_t)h * kT5HD;
    const float *vbase = d.v + (int64_t)k0 * d.v_stride + (int64_t)h * kT5HD;

    float m = -INFINITY, l = 0.0f;
    bool failed = false;
    uint32_t phase = 0;

    // K/V tile staging. Loads: 16-byte pieces into registers (issued one tile ahead so that HBM
    // latency hides behind the previous tile's MMAs and softmax). Stores: K as [key][dim] core
    // matrices with 16-byte stores; V transposed to [dim][key] with 4-byte stores whose lane
    // mapping (4 keys x 2 pieces x 4 rotations of the element order) touches 32 distinct banks.
    float4 kr[8], vr[8];
    const int v_rl = (lane & 3) + 4 * (lane >> 3), v_cl = (lane >> 2) & 1, v_xo = lane >> 3;
    auto load_tile = [&](int kt) {
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int bid = it * 4 + warp;
            {   // K: 8 keys x 4 pieces per warp step
                const int r = (bid & 7) * 8 + (lane & 7), c = (bid >> 3) * 4 + (lane >> 3);
                const int j = kt * kT5Keys + r;
                kr[it] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (j < nk) {
                    kr[it] = __ldg(reinterpret_cast<const float4 *>(kbase + (int64_t)j * d.k_stride + c * 4));
                    if (d.rope_cos)
                        kr[it] = rope_rotate4(kr[it], d.rope_cos, d.rope_sin, d.rope_k_pos ? d.rope_k_pos[k0 + j] : j,
                                              kT5HD / 2, c * 2);
                }
            }
            {   // V: 16 keys x 2 pieces per warp step
                const int r = (bid & 3) * 16 + v_rl, c = (bid >> 2) * 2 + v_cl;
                const int j = kt * kT5Keys + r;
                vr[it] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (j < nk) vr[it] = __ldg(reinterpret_cast<const float4 *>(vbase + (int64_t)j * d.v_stride + c * 4));
            }
        }
    };
    auto store_tile = [&]() {
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int bid = it * 4 + warp;
            {
                const int r = (bid & 7) * 8 + (lane & 7), c = (bid >> 3) * 4 + (lane >> 3);
                const uint32_t koff = c * 1024 + (r >> 3) * 128 + (r & 7) * 16;
                const float ke[4] = {kr[it].x, kr[it].y, kr[it].z, kr[it].w};
                uint4 khi, klo;
                uint32_t *kh = &khi.x, *kl = &klo.x;
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    kh[x] = t5_round_in<X3>(ke[x]);
                    kl[x] = __float_as_uint(ke[x] - __uint_as_float(kh[x]));
                }
                *reinterpret_cast<uint4 *>(smem + kOffK + koff) = khi;
                if (X3) *reinterpret_cast<uint4 *>(smem + kOffK + kPlaneKV + koff) = klo;
            }
            {
                const int r = (bid & 3) * 16 + v_rl, c = (bid >> 2) * 2 + v_cl;
                // rotate the four elements by v_xo so that store step s writes element (s + v_xo) & 3
                float e0 = vr[it].x, e1 = vr[it].y, e2 = vr[it].z, e3 = vr[it].w;
                if (v_xo & 1) {
                    const float t = e0;
                    e0 = e1; e1 = e2; e2 = e3; e3 = t;
                }
                if (v_xo & 2) {
                    float t = e0;
                    e0 = e2; e2 = t;
                    t = e1;
                    e1 = e3; e3 = t;
                }
                const float ve[4] = {e0, e1, e2, e3};
                const uint32_t vbase_off = (r >> 2) * 1024 + (r & 3) * 4;
#pragma unroll
                for (int st = 0; st < 4; ++st) {
                    const int n = c * 4 + ((st + v_xo) & 3);
                    const uint32_t o = vbase_off + (n >> 3) * 128 + (n & 7) * 16;
                    const uint32_t vh = t5_round_in<X3>(ve[st]);
                    *reinterpret_cast<uint32_t *>(smem + kOffV + o) = vh;
                    if (X3) *reinterpret_cast<uint32_t *>(smem + kOffV + kPlaneKV + o) = __float_as_uint(ve[st] - __uint_as_float(vh));
                }
            }
        }
    };

    if (kt_begin < kt_end) load_tile(kt_begin);

    // ---- Q row -> (hi, lo) TF32 parts in TMEM --------------------------------------
    {
        const float qscale = d.scale * kLog2e;
        const float *qrow = d.q + (int64_t)(q0 + (i < nq ? i : 0)) * d.q_stride + (int64_t)h * kT5HD;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            uint32_t qh[32], ql[32];
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (i < nq) {
                    v = __ldg(reinterpret_cast<const float4 *>(qrow + half * 32 + c * 4));
                    if (d.rope_cos)
                        v = rope_rotate4(v, d.rope_cos, d.rope_sin,
                                         d.rope_q_pos ? d.rope_q_pos[q0 + i]
                                                      : i + (d.mask.causal_offset ? d.mask.causal_offset[b] : 0),
                                         kT5HD / 2, half * 16 + c * 2);
                }
                const float e[4] = {v.x * qscale, v.y * qscale, v.z * qscale, v.w * qscale};
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    qh[c * 4 + x] = t5_round_in<X3>(e[x]);
                    ql[c * 4 + x] = __float_as_uint(e[x] - __uint_as_float(qh[c * 4 + x]));
                }
            }
            tmem_st32(trow + kColQhi + half * 32, qh);
            if (X3) tmem_st32(trow + kColQlo + half * 32, ql);
        }
        tc_wait_st();
    }


    for (int kt = kt_begin; kt < kt_end; ++kt) {
        // ---- previous tile's O MMAs must be done before V / P are overwritten -------
        if (kt > kt_begin) {
            const bool ok = mbar_wait(&bar_o, phase ^ 1);
            if (__syncthreads_or(!ok)) {
                failed = true;
                break;
            }
            tc_fence_after();
        }
        store_tile();
        fence_async_smem();
        tc_fence_before();
        __syncthreads();

        // ---- S = Q K^T ----------------------------------------------------------------
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const uint64_t bh = t5_desc(sbase + kOffK + ks * 2048, 1024, 128);
                const uint64_t bl = t5_desc(sbase + kOffK + kPlaneKV + ks * 2048, 1024, 128);
                const uint32_t ah = tmem + kColQhi + ks * 8, al = tmem + kColQlo + ks * 8;
                if (X3) {
                    mma_ts(tmem + kColS, al, bh, kIdescS, ks > 0);
                    mma_ts(tmem + kColS, ah, bl, kIdescS, 1);
                    mma_ts(tmem + kColS, ah, bh, kIdescS, 1);
                } else {
                    mma_ts(tmem + kColS, ah, bh, kIdescS, ks > 0);
                }
            }
            tc_commit(&bar_s);
        }
        if (kt + 1 < kt_end) load_tile(kt + 1); // in flight while S completes and the softmax runs
        {
            const bool ok = mbar_wait(&bar_s, phase);
            if (__syncthreads_or(!ok)) {
                failed = true;
                break;
            }
            tc_fence_after();
        }

        // ---- softmax of this thread's row; P -> shared memory as the next A operand -----
        const int j0 = kt * kT5Keys;
        float corr = 1.0f;
        {
            float s[64];
            {
                float t0[32], t1[32];
                tmem_ld32(trow + kColS, t0);
                tmem_ld32(trow + kColS + 32, t1);
                tc_wait_ld();
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    s[c] = t0[c];
                    s[32 + c] = t1[c];
                }
            }
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < 64; ++c) {
                const int j = j0 + c;
                const bool ok = finite_f(s[c]) && j >= lo && j < hi;
                s[c] = ok ? s[c] : -INFINITY;
                mx = fmaxf(mx, s[c]);
            }
            const float mn = fmaxf(m, mx);
            const float ref = mn == -INFINITY ? 0.0f : mn;
            corr = t5_ex2(m - ref);
            m = mn;
            float rs = 0.0f;
            const uint32_t prow = (tid >> 3) * 128 + (tid & 7) * 16;
#pragma unroll
            for (int kc = 0; kc < 16; ++kc) {
                uint4 ph, pl;
                uint32_t *h4 = &ph.x, *l4 = &pl.x;
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    const float p = t5_ex2(s[kc * 4 + x] - ref);
                    rs += p;
                    h4[x] = t5_tf32_finite(p); // p is in [0, 1]
                    l4[x] = __float_as_uint(p - __uint_as_float(h4[x]));
                }
                *reinterpret_cast<uint4 *>(smem + kOffK + kc * 2048 + prow) = ph; // K tile space, S is complete
                if (X3) *reinterpret_cast<uint4 *>(smem + kOffPlo + kc * 2048 + prow) = pl;
            }
            l = l * corr + rs;
        }
        // ---- rescale the running output where a row maximum moved -------------------------
        if (kt > kt_begin && __any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                float o[32];
                uint32_t w[32];
                tmem_ld32(trow + kColO + half * 32, o);
                tc_wait_ld();
#pragma unroll
                for (int c = 0; c < 32; ++c) w[c] = __float_as_uint(o[c] * corr);
                tmem_st32(trow + kColO + half * 32, w);
            }
            tc_wait_st();
        }
        fence_async_smem();
        tc_fence_before();
        __syncthreads();

        // ---- O += P V ----------------------------------------------------------------------
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const uint64_t ah = t5_desc(sbase + kOffK + ks * 4096, 2048, 128);
                const uint64_t al = t5_desc(sbase + kOffPlo + ks * 4096, 2048, 128);
                const uint64_t bh = t5_desc(sbase + kOffV + ks * 2048, 1024, 128);
                const uint64_t bl = t5_desc(sbase + kOffV + kPlaneKV + ks * 2048, 1024, 128);
                const uint32_t first = (kt > kt_begin || ks > 0) ? 1u : 0u;
                if (X3) {
                    mma_ss(tmem + kColO, al, bh, kIdescO, first);
                    mma_ss(tmem + kColO, ah, bl, kIdescO, 1);
                    mma_ss(tmem + kColO, ah, bh, kIdescO, 1);
                } else {
                    mma_ss(tmem + kColO, ah, bh, kIdescO, first);
                }
            }
            tc_commit(&bar_o);
        }
        phase ^= 1;
    }

    // ---- epilogue ----------------------------------------------------------------------------
    if (!failed && kt_begin < kt_end) {
        const bool ok = mbar_wait(&bar_o, phase ^ 1);
        if (__syncthreads_or(!ok)) failed = true;
        tc_fence_after();
    }
    if (failed) {
        if (tid == 0) {
            atomicCAS(&g_t5_error, 0u, (1u << 24) | (blockIdx.x & 0xffffffu));
            // MMAs this thread issued may still be running: one more bounded wait for all of them
            // before the TMEM they write is given back
            tc_commit(&bar_fin);
            mbar_wait(&bar_fin, 0);
        }
    } else {
        float *orow = d.out + (int64_t)(q0 + (i < nq ? i : 0)) * d.out_stride + (int64_t)h * kT5HD;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            float o[32];
            if (kt_begin < kt_end) {
                tmem_ld32(trow + kColO + half * 32, o);
                tc_wait_ld();
            } else {
#pragma unroll
                for (int c = 0; c < 32; ++c) o[c] = 0.0f;
            }
            if (i < nq) {
                const float inv = l > 0.0f ? 1.0f / l : 0.0f; // rows without keys give zeros
#pragma unroll
                for (int c = 0; c < 8; ++c)
                    *reinterpret_cast<float4 *>(orow + half * 32 + c * 4) =
                        make_float4(o[c * 4] * inv, o[c * 4 + 1] * inv, o[c * 4 + 2] * inv, o[c * 4 + 3] * inv);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, kT5Cols);
}

int gemm5_take_error(); // gemm5_kernel.cu
int gemm5_take_error_on(cudaStream_t s);
int unit5_take_error(); // unit5_kernel.cu
int unit5_take_error_on(cudaStream_t s);

// The same report for a caller that has just synchronised its own streams: reads (and, when set,
// clears) the two error words in order with `s` and waits for `s` only -- other streams of the
// device keep running.
int tcgen05_error_on_stream(cudaStream_t s) {
    unsigned int v = 0, zero = 0;
    if (cudaMemcpyFromSymbolAsync(&v, g_t5_error, sizeof(v), 0, cudaMemcpyDeviceToHost, s) != cudaSuccess) return -1;
    if (cudaStreamSynchronize(s) != cudaSuccess) return -1;
    if (v) {
        cudaMemcpyToSymbolAsync(g_t5_error, &zero, sizeof(zero), 0, cudaMemcpyHostToDevice, s);
        cudaStreamSynchronize(s);
    }
    const int g = gemm5_take_error_on(s);
    const int u5 = unit5_take_error_on(s);
    return v ? (int)v : (u5 ? u5 : g);
}

bool tile5_kernel_supports(const fblt_attn_desc &d, const char **why) {
    if (d.head_dim != 64) {
        *why = "tcgen05 kernel: head_dim must be 64";
        return false;
    }
    if (d.mask.group_rule == FBLT_GROUP_IDS) {
        *why = "explicit group ids are not a key range";
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
    if (d.batch > 65535 || d.num_heads > 65535) {
        *why = "batch/heads exceed 65535";
        return false;
    }
    return true;
}

template <bool X3>
static int launch_tile5_t(const fblt_attn_desc &d, cudaStream_t stream) {
    static std::atomic<uint64_t> configured{0}; // one bit per device ordinal; the attribute is per device
    int dev = 0;
    FBLT_CUDA_TRY(cudaGetDevice(&dev));
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        FBLT_CUDA_TRY(cudaFuncSetAttribute(tile5_attn_kernel<X3>, cudaFuncAttributeMaxDynamicSharedMemorySize, kT5Smem));
        configured.fetch_or(bit, std::memory_order_release);
    }
    dim3 grid((d.max_q + kT5Rows - 1) / kT5Rows, d.num_heads, d.batch);
    tile5_attn_kernel<X3><<<grid, kT5Threads, kT5Smem, stream>>>(d);
    count_launch();
    return check_launch("tile5_attn_kernel");
}

int launch_tile5_kernel(const fblt_attn_desc &d, cudaStream_t stream) {
    return d.precision != FBLT_PREC_TF32 ? launch_tile5_t<true>(d, stream) : launch_tile5_t<false>(d, stream);
}

} // namespace fblt

// 0 when no tcgen05 CTA has given up on a bounded wait since the last call; otherwise the
// recorded code. Synchronises the device and clears the word.
extern "C" int fblt_tcgen05_error(void) {
    unsigned int v = 0, zero = 0;
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(&v, fblt::g_t5_error, sizeof(v)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(fblt::g_t5_error, &zero, sizeof(zero));
    const int g = fblt::gemm5_take_error();
    const int u5 = fblt::unit5_take_error();
    return v ? (int)v : (u5 ? u5 : g);
}
