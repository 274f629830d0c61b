// L1 tensor-core tile kernel: varlen batched attention whose mask is a key
// range per query row (causal / sliding window / document / block-diffusion
// INFER / patch rules), for prefill self-attention and the "patches <= its
// patch" decoder cross-attention.
//
//   CTA  = (64 query rows, head, sequence), 4 warps x 16 rows
//   K/V  = 64-key tiles staged raw (fp32) in shared memory by 16-byte async
//          copies, two stages, so the next tile streams in while this one is
//          multiplied; rows padded by 4 floats -> conflict-free fragment reads
//   QK^T = mma.sync m16n8k8 TF32; in the fp32-equivalent mode every operand is
//          split on the fly into (hi, lo) TF32 parts and three MMAs recover
//          ~fp32 products (lo*hi + hi*lo + hi*hi)
//   softmax = online, in registers, log2 domain, finite-only maximum
//   PV   = same MMA; the score fragment is reused as the A operand by pairing
//          key 2t with k-slot t and key 2t+1 with slot t+4 on both operands
//
// Key tiles outside the union of the CTA's row ranges are never loaded; tiles
// inside every row's range skip the per-element range test.
#include "common.cuh"

#include <atomic>
#include <limits.h>

namespace fblt {

constexpr int kBM = 64, kBN = 64, kTileThreads = 128;

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gmem_src, int src_bytes) {
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem_src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ uint32_t to_tf32(float x) {
    // Round to nearest, ties away from zero, to 10 mantissa bits -- the result of
    // cvt.rna.tf32.f32 -- with integer instructions: the conversion instruction runs on the
    // low-rate special-function pipe, which these kernels need for exp2. Inf / NaN pass through.
    const uint32_t b = __float_as_uint(x);
    const uint32_t r = (b + 0x1000u) & 0xFFFFE000u;
    return (b & 0x7F800000u) == 0x7F800000u ? b : r;
}
// x = hi + lo with hi the TF32 rounding of x; lo is consumed by the tensor core
// with its low mantissa bits ignored, which is below fp32 resolution of x.
// With the low part in use (three-pass mode) the rounding needs no Inf / NaN pass-through:
// whatever it does to such a bit pattern, the low part x - hi is then not finite, so the score
// still is not. In single-pass mode only hi reaches the tensor core, so Q and K keep the test.
// Probabilities and V rows (finite by contract) never need it.
template <bool CHECKED>
__device__ __forceinline__ void split_tf32(float x, uint32_t &hi, uint32_t &lo) {
    hi = CHECKED ? to_tf32(x) : ((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u);
    lo = __float_as_uint(x - __uint_as_float(hi));
}
__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__device__ __forceinline__ float ex2_fast(float x) { // 2^x; -inf -> 0, results below 2^-126 flush to 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// STAGES = 2 double-buffers the K/V tiles (long key ranges); STAGES = 1 keeps
// one tile and lets four CTAs share an SM instead (key ranges of one or two tiles).
template <int HD, bool X3, int STAGES>
__global__ void __launch_bounds__(kTileThreads, STAGES == 1 ? 4 : 2) tile_attn_kernel(fblt_attn_desc d) {
    constexpr int LDS = HD + 4;    // padded row, floats
    constexpr int CPR = HD / 4;    // 16-byte chunks per row
    constexpr int NT_O = HD / 8;   // output n-tiles
    constexpr int KS_S = HD / 8;   // k-steps of QK^T
    extern __shared__ __align__(16) float smem[];
    float *sQ = smem;
    float *sK = sQ + kBM * LDS;
    float *sV = sK + STAGES * kBN * LDS;
    __shared__ int s_lo[kBM], s_hi[kBM];

    const int b = blockIdx.z, h = blockIdx.y;
    const int qt = gridDim.x - 1 - blockIdx.x; // long rows first
    const int q0 = d.cu_q[b], nq = d.cu_q[b + 1] - q0;
    const int k0 = d.cu_k[b], nk = d.cu_k[b + 1] - k0;
    if (qt * kBM >= nq) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;

    if (tid < kBM) {
        const int i = qt * kBM + tid;
        int lo = INT_MAX, hi = 0;
        if (i < nq) {
            const SeqMask s = resolve_mask(d.mask, b, q0, k0, nq, nk);
            row_range(s, i, lo, hi);
            if (hi <= lo) {
                lo = INT_MAX;
                hi = 0;
            }
        }
        s_lo[tid] = lo;
        s_hi[tid] = hi;
    }
    __syncthreads();
    int cmin = INT_MAX, cmax = 0;
    for (int r = 0; r < kBM; ++r) {
        cmin = min(cmin, s_lo[r]);
        cmax = max(cmax, s_hi[r]);
    }
    const int kt_begin = cmax > 0 ? cmin / kBN : 0;
    const int kt_end = cmax > 0 ? (cmax + kBN - 1) / kBN : 0;

    const int wr = warp * 16;
    const int lo0 = s_lo[wr + g], hi0 = s_hi[wr + g];
    const int lo1 = s_lo[wr + g + 8], hi1 = s_hi[wr + g + 8];
    int wlo = min(lo0, lo1), whi = max(hi0, hi1);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        wlo = min(wlo, __shfl_xor_sync(0xffffffffu, wlo, o));
        whi = max(whi, __shfl_xor_sync(0xffffffffu, whi, o));
    }

    const float *qbase = d.q + (int64_t)q0 * d.q_stride + (int64_t)h * HD;
    const float *kbase = d.k + (int64_t)k0 * d.k_stride + (int64_t)h * HD;
    const float *vbase = d.v + (int64_t)k0 * d.v_stride + (int64_t)h * HD;

    // ---- stage Q and the first K/V tile ---------------------------------
    for (int c = tid; c < kBM * CPR; c += kTileThreads) {
        const int r = c / CPR, cc = c - r * CPR;
        const int i = qt * kBM + r;
        const bool ok = i < nq;
        cp_async16(sQ + r * LDS + cc * 4, qbase + (int64_t)(ok ? i : 0) * d.q_stride + cc * 4, ok ? 16 : 0);
    }
    auto load_kv = [&](int kt, int stage) {
        float *dk = sK + stage * kBN * LDS;
        float *dv = sV + stage * kBN * LDS;
        for (int c = tid; c < kBN * CPR; c += kTileThreads) {
            const int r = c / CPR, cc = c - r * CPR;
            const int j = kt * kBN + r;
            const bool ok = j < nk;
            const int64_t row = ok ? j : 0;
            cp_async16(dk + r * LDS + cc * 4, kbase + row * d.k_stride + cc * 4, ok ? 16 : 0);
            cp_async16(dv + r * LDS + cc * 4, vbase + row * d.v_stride + cc * 4, ok ? 16 : 0);
        }
    };
    if (kt_begin < kt_end) load_kv(kt_begin, 0);
    cp_async_commit();

    float oacc[NT_O][4];
#pragma unroll
    for (int n = 0; n < NT_O; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) oacc[n][e] = 0.0f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;
    const float qscale = d.scale * kLog2e;

    for (int kt = kt_begin; kt < kt_end; ++kt) {
        int stage = 0;
        if (STAGES == 2) {
            stage = (kt - kt_begin) & 1;
            if (kt + 1 < kt_end) load_kv(kt + 1, stage ^ 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            if (kt > kt_begin) {
                load_kv(kt, 0);
                cp_async_commit();
            }
            cp_async_wait<0>();
        }
        __syncthreads();

        const int j0 = kt * kBN;
        if (d.rope_cos) { // rotate the freshly landed K tile (and, once, the Q tile) in shared memory
            float *rK = sK + stage * kBN * LDS;
            for (int c = tid; c < kBN * CPR; c += kTileThreads) {
                const int r = c / CPR, cc = c - r * CPR;
                if (j0 + r < nk) {
                    float4 *p4 = reinterpret_cast<float4 *>(rK + r * LDS + cc * 4);
                    *p4 = rope_rotate4(*p4, d.rope_cos, d.rope_sin, d.rope_k_pos ? d.rope_k_pos[k0 + j0 + r] : j0 + r,
                                       HD / 2, cc * 2);
                }
            }
            if (kt == kt_begin) {
                const int off = d.mask.causal_offset ? d.mask.causal_offset[b] : 0;
                for (int c = tid; c < kBM * CPR; c += kTileThreads) {
                    const int r = c / CPR, cc = c - r * CPR;
                    if (qt * kBM + r < nq) {
                        float4 *p4 = reinterpret_cast<float4 *>(sQ + r * LDS + cc * 4);
                        const int iq = qt * kBM + r;
                        *p4 = rope_rotate4(*p4, d.rope_cos, d.rope_sin, d.rope_q_pos ? d.rope_q_pos[q0 + iq] : iq + off,
                                           HD / 2, cc * 2);
                    }
                }
            }
            __syncthreads();
        }
        if (whi > j0 && wlo < j0 + kBN) {
            const float *tK = sK + stage * kBN * LDS;
            const float *tV = sV + stage * kBN * LDS;
            // 8-key column blocks of this tile that some row of the warp can see
            const int nlo = wlo > j0 ? (wlo - j0) >> 3 : 0;
            const int nhi = whi < j0 + kBN ? (whi - j0 + 7) >> 3 : 8;

            float sacc[8][4];
#pragma unroll
            for (int n = 0; n < 8; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) sacc[n][e] = 0.0f;

#pragma unroll
            for (int ks = 0; ks < KS_S; ++ks) {
                uint32_t ahi[4], alo[4];
                split_tf32<!X3>(sQ[(wr + g) * LDS + ks * 8 + t] * qscale, ahi[0], alo[0]);
                split_tf32<!X3>(sQ[(wr + g + 8) * LDS + ks * 8 + t] * qscale, ahi[1], alo[1]);
                split_tf32<!X3>(sQ[(wr + g) * LDS + ks * 8 + t + 4] * qscale, ahi[2], alo[2]);
                split_tf32<!X3>(sQ[(wr + g + 8) * LDS + ks * 8 + t + 4] * qscale, ahi[3], alo[3]);
#pragma unroll
                for (int n = 0; n < 8; ++n) {
                    if (n < nlo || n >= nhi) continue; // scores stay 0 and are masked below
                    uint32_t bhi[2], blo[2];
                    split_tf32<!X3>(tK[(n * 8 + g) * LDS + ks * 8 + t], bhi[0], blo[0]);
                    split_tf32<!X3>(tK[(n * 8 + g) * LDS + ks * 8 + t + 4], bhi[1], blo[1]);
                    if (X3) {
                        mma_tf32(sacc[n], alo, bhi);
                        mma_tf32(sacc[n], ahi, blo);
                    }
                    mma_tf32(sacc[n], ahi, bhi);
                }
            }

            // ---- range test + online softmax -------------------------------
            const bool inside = lo0 <= j0 && hi0 >= j0 + kBN && lo1 <= j0 && hi1 >= j0 + kBN;
            const bool need_mask = !__all_sync(0xffffffffu, inside);
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int n = 0; n < 8; ++n) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = j0 + n * 8 + 2 * t + (e & 1);
                    float s = sacc[n][e];
                    bool ok = finite_f(s);
                    if (need_mask) ok = ok && (e < 2 ? (j >= lo0 && j < hi0) : (j >= lo1 && j < hi1));
                    s = ok ? s : -INFINITY;
                    sacc[n][e] = s;
                    if (e < 2) mx0 = fmaxf(mx0, s);
                    else mx1 = fmaxf(mx1, s);
                }
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
            const float ref0 = mn0 == -INFINITY ? 0.0f : mn0, ref1 = mn1 == -INFINITY ? 0.0f : mn1;
            const float c0 = ex2_fast(m0 - ref0), c1 = ex2_fast(m1 - ref1);
            m0 = mn0;
            m1 = mn1;
            float rs0 = 0.0f, rs1 = 0.0f;
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                sacc[n][0] = ex2_fast(sacc[n][0] - ref0);
                sacc[n][1] = ex2_fast(sacc[n][1] - ref0);
                sacc[n][2] = ex2_fast(sacc[n][2] - ref1);
                sacc[n][3] = ex2_fast(sacc[n][3] - ref1);
                rs0 += sacc[n][0] + sacc[n][1];
                rs1 += sacc[n][2] + sacc[n][3];
            }
            l0 = l0 * c0 + rs0;
            l1 = l1 * c1 + rs1;
#pragma unroll
            for (int n = 0; n < NT_O; ++n) {
                oacc[n][0] *= c0;
                oacc[n][1] *= c0;
                oacc[n][2] *= c1;
                oacc[n][3] *= c1;
            }

            // ---- O += P V ----------------------------------------------------
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                if (ks < nlo || ks >= nhi) continue; // every probability in this block is 0
                uint32_t ahi[4], alo[4];
                split_tf32<false>(sacc[ks][0], ahi[0], alo[0]); // row g,   key 2t
                split_tf32<false>(sacc[ks][2], ahi[1], alo[1]); // row g+8, key 2t
                split_tf32<false>(sacc[ks][1], ahi[2], alo[2]); // row g,   key 2t+1
                split_tf32<false>(sacc[ks][3], ahi[3], alo[3]); // row g+8, key 2t+1
#pragma unroll
                for (int n = 0; n < NT_O; ++n) {
                    uint32_t bhi[2], blo[2];
                    split_tf32<false>(tV[(ks * 8 + 2 * t) * LDS + n * 8 + g], bhi[0], blo[0]);
                    split_tf32<false>(tV[(ks * 8 + 2 * t + 1) * LDS + n * 8 + g], bhi[1], blo[1]);
                    if (X3) {
                        mma_tf32(oacc[n], alo, bhi);
                        mma_tf32(oacc[n], ahi, blo);
                    }
                    mma_tf32(oacc[n], ahi, bhi);
                }
            }
        }
        __syncthreads(); // the tile is overwritten by the next load
    }
    cp_async_wait<0>();

    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

    const int i0 = qt * kBM + wr + g, i1 = i0 + 8;
    float *obase = d.out + (int64_t)q0 * d.out_stride + (int64_t)h * HD;
#pragma unroll
    for (int n = 0; n < NT_O; ++n) {
        if (i0 < nq) {
            float2 o = make_float2(0.f, 0.f);
            if (l0 > 0.0f) o = make_float2(oacc[n][0] / l0, oacc[n][1] / l0);
            *reinterpret_cast<float2 *>(obase + (int64_t)i0 * d.out_stride + n * 8 + 2 * t) = o;
        }
        if (i1 < nq) {
            float2 o = make_float2(0.f, 0.f);
            if (l1 > 0.0f) o = make_float2(oacc[n][2] / l1, oacc[n][3] / l1);
            *reinterpret_cast<float2 *>(obase + (int64_t)i1 * d.out_stride + n * 8 + 2 * t) = o;
        }
    }
}

bool tile_kernel_supports(const fblt_attn_desc &d, const char **why) {
    if (d.head_dim != 32 && d.head_dim != 64 && d.head_dim != 128) {
        *why = "head_dim must be 32, 64 or 128";
        return false;
    }
    if (d.mask.group_rule == FBLT_GROUP_IDS) {
        *why = "explicit group ids are not a key range";
        return false;
    }
    if ((d.q_stride | d.k_stride | d.v_stride) & 3) {
        *why = "q/k/v row strides must be multiples of 4 elements";
        return false;
    }
    if (d.out_stride & 1) {
        *why = "out row stride must be even";
        return false;
    }
    if (((uintptr_t)d.q | (uintptr_t)d.k | (uintptr_t)d.v) & 15) {
        *why = "q/k/v must be 16-byte aligned";
        return false;
    }
    if ((uintptr_t)d.out & 7) {
        *why = "out must be 8-byte aligned";
        return false;
    }
    if (d.batch > 65535 || d.num_heads > 65535) {
        *why = "batch/heads exceed 65535";
        return false;
    }
    return true;
}

template <int HD, bool X3, int STAGES>
static int launch_tile_s(const fblt_attn_desc &d, cudaStream_t stream) {
    constexpr size_t smem = (size_t)(kBM + 2 * STAGES * kBN) * (HD + 4) * sizeof(float);
    static std::atomic<uint64_t> configured{0}; // one bit per device ordinal; the attribute is per device
    int dev = 0;
    FBLT_CUDA_TRY(cudaGetDevice(&dev));
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        FBLT_CUDA_TRY(cudaFuncSetAttribute(tile_attn_kernel<HD, X3, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured.fetch_or(bit, std::memory_order_release);
    }
    dim3 grid((d.max_q + kBM - 1) / kBM, d.num_heads, d.batch);
    tile_attn_kernel<HD, X3, STAGES><<<grid, kTileThreads, smem, stream>>>(d);
    count_launch();
    return check_launch("tile_attn_kernel");
}

template <int HD, bool X3>
static int launch_tile_t(const fblt_attn_desc &d, cudaStream_t stream) {
    // at most two key tiles per sequence: occupancy beats intra-CTA prefetch.
    const bool single = d.max_k <= 2 * kBN;
    if (single && HD <= 64) return launch_tile_s<HD, X3, 1>(d, stream);
    return launch_tile_s<HD, X3, 2>(d, stream);
}

int launch_tile_kernel(const fblt_attn_desc &d, cudaStream_t stream) {
    const bool x3 = d.precision != FBLT_PREC_TF32;
    switch (d.head_dim) {
    case 32: return x3 ? launch_tile_t<32, true>(d, stream) : launch_tile_t<32, false>(d, stream);
    case 64: return x3 ? launch_tile_t<64, true>(d, stream) : launch_tile_t<64, false>(d, stream);
    default: return x3 ? launch_tile_t<128, true>(d, stream) : launch_tile_t<128, false>(d, stream);
    }
}

} // namespace fblt
