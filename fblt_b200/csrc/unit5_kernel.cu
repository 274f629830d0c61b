// L1 tcgen05 kernel for short sequences (head_dim 64, at most 128 query rows and 128 keys per
// sequence: the patch-transformer shapes): one (sequence, head) unit = one 128 x 128 score tile,
// so the softmax is a single pass with no running maximum and no rescale of the output.
//
// Persistent, one CTA per SM, roles that meet only on mbarriers:
//   loader (1 thread)   raw fp32 Q, K, V tiles of the NEXT unit by tiled TMA (128-byte swizzle, no
//                       multicast, this GPU's memory only): Q / K as soon as the score MMAs that read
//                       the current ones have completed, V as soon as the current raw V tile has been
//                       transposed away;
//   issuer (1 thread)   S = Q K^T as 16 tcgen05.mma (Q_hi x [K_hi | K_lo] is ONE 128 x 256 x 8
//                       instruction into a main and a small-term accumulator, Q_lo x K_hi a second
//                       one), O = P V as 32 (P_hi x [V_hi | V_lo], P_lo x V_hi) with P read from TMEM,
//                       completion by tcgen05.commit;
//   workers (8 warps)   two threads per query row (warps w and w + 4 both reach TMEM lanes 32 w ..): in
//                       turn they transpose this unit's V into its (hi, lo) planes, read main + small
//                       scores for their half of the key chunks, trade the row maximum, write P (hi, lo)
//                       over the scores in TMEM, split the next unit's Q / K in place into TF32 (hi, lo)
//                       planes -- an elementwise pass over the swizzled bytes -- while this unit's P V
//                       runs, then read O, scale by 1 / row sum and store whole 128-byte row segments
//                       (rows are traded through shared memory first).
// TMEM: 256 columns of scores / probabilities + two output accumulators of 128 columns.
// Shared memory: 64 KB each for Q and K (raw / hi plane and lo plane), 32 KB for the raw V tile and
// 64 KB for V^T, single-buffered.
//
// Measured on the scaled prefill (2048 sequences x 16 heads, 4.2 GB): 1.43 ms against 2.06 ms for the
// two-CTA-per-SM tile kernel. What bounds it now is shared-memory traffic and the length of one
// unit's chain (the MMAs alone read ~290 KB of operands per unit, the conversions move ~350 KB more),
// not the tensor pipe (25 % active) or HBM (32 %). Computing the scores one unit ahead into a second
// TMEM buffer was measured and changed nothing (1.53 ms): the workers are the critical resource.
//
// Every mbarrier wait is bounded; a role that gives up raises the CTA's abort word, records a code
// (fblt_tcgen05_error), and all roles leave their loops, wait (bounded) for what is in flight, free
// the TMEM and return.
#include "common.cuh"
#include "tc5.cuh"

#include <atomic>
#include <cuda.h> // CUtensorMap and its enums only; the encoder is looked up at run time
#include <limits.h>

namespace fblt {

constexpr int kU5Rows = 128, kU5HD = 64;
constexpr int kU5Threads = 32 * 10; // warps 0-7 workers (conversion, softmax, output), 8 issuer, 9 loader
constexpr int kU5Atom = 16384;      // one 128-row x 32-column fp32 box (128-byte swizzle)
// shared memory map (bytes). Q and K: per 32-column atom the raw / hi plane followed by the lo plane,
// so that [K_hi | K_lo] of an atom is one 256-row operand. V: both raw atoms, then both lo atoms, so
// that [V_hi | V_lo] is four 32-column blocks at one stride.
constexpr int kU5OffQ = 0, kU5OffK = 4 * kU5Atom, kU5OffV = 8 * kU5Atom, kU5OffVT = 10 * kU5Atom;
constexpr int kU5Smem = 14 * kU5Atom; // + < 3 KB of static shared memory: the 227 KB of an SM, to the byte
constexpr int kU5VtLbo = 2048; // V^T: 16 row groups (64 hi + 64 lo value columns) of 128 bytes per 4-key column
// TMEM columns
constexpr uint32_t kU5ColS = 0, kU5ColSmall = 128, kU5ColO = 256, kU5Cols = 512;

__device__ unsigned int g_u5_error; // 0 = ok; otherwise (code << 24) | blockIdx.x of the first CTA that gave up

struct U5Bars {
    uint64_t qk_full, v_full, qk_conv, v_conv, s_done, p_ready, o_done, o_free[2], fin;
};

// Shared-memory matrix descriptor for the 128-byte-swizzled layouts a tiled TMA load produces
// (rows of 128 bytes, 8-row groups of 1024 bytes): descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t u5_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) | (2ull << 61);
}

#ifdef U5_DEBUG
// cycle counters of CTA 0, one row per role: [role][slot]
__device__ unsigned long long g_u5_dbg[8][16];
#define U5_T0() long long t__ = clock64()
#define U5_ACC(role, slot)                                                         \
    do {                                                                           \
        const long long n__ = clock64();                                           \
        if (blockIdx.x == 0) g_u5_dbg[role][slot] += (unsigned long long)(n__ - t__); \
        t__ = n__;                                                                 \
    } while (0)
#else
#define U5_T0() do { } while (0)
#define U5_ACC(role, slot) do { } while (0)
#endif

struct U5Unit {
    int b, h, q0, nq, k0, nk;
};

// Unit `u` of the launch, or nq == 0 for units with nothing to do (skipped by every role alike).
__device__ __forceinline__ U5Unit u5_unit(const fblt_attn_desc &d, int u) {
    U5Unit t;
    t.b = u / d.num_heads;
    t.h = u - t.b * d.num_heads;
    t.q0 = d.cu_q[t.b];
    t.nq = d.cu_q[t.b + 1] - t.q0;
    t.k0 = d.cu_k[t.b];
    t.nk = d.cu_k[t.b + 1] - t.k0;
    return t;
}

__global__ void __launch_bounds__(kU5Threads, 1)
    unit5_attn_kernel(fblt_attn_desc d, const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                      const __grid_constant__ CUtensorMap v_map, int units) {
    extern __shared__ __align__(1024) uint8_t smem[]; // swizzle atoms: 1 KB alignment
    __shared__ __align__(8) U5Bars bars;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_word;
    __shared__ float xmax[2][kU5Rows], xsum[2][kU5Rows]; // the two halves of a row trade maximum and sum
    const uint32_t sbase = smem_u32(smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        mbar_init(&bars.qk_full, 1);
        mbar_init(&bars.v_full, 1);
        mbar_init(&bars.qk_conv, 8);
        mbar_init(&bars.v_conv, 8);
        mbar_init(&bars.s_done, 1);
        mbar_init(&bars.p_ready, 8);
        mbar_init(&bars.o_done, 1);
        mbar_init(&bars.o_free[0], 8);
        mbar_init(&bars.o_free[1], 8);
        mbar_init(&bars.fin, 1);
        abort_word = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        tmem_alloc(&tmem_slot, kU5Cols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    volatile int *abortp = &abort_word;
    auto give_up = [&](unsigned code) {
        *abortp = 1;
        atomicCAS(&g_u5_error, 0u, (code << 24) | (blockIdx.x & 0xffffffu));
    };

    if (warp == 9) {
        // ================= loader =================
        if (lane == 0) {
            int k = 0; // processed units of this CTA
            for (int u = blockIdx.x; u < units && !*abortp; u += gridDim.x) {
                const U5Unit t = u5_unit(d, u);
                if (t.nq <= 0 || t.nk <= 0) continue;
                // Q / K of the previous unit have been read once its score MMAs completed
                if (k > 0 && !mbar_wait_abort(&bars.s_done, (k - 1) & 1, abortp)) {
                    give_up(0x11);
                    break;
                }
                mbar_expect_tx(&bars.qk_full, 4 * kU5Atom);
#pragma unroll
                for (int a = 0; a < 2; ++a) {
                    tma_load_2d(smem + kU5OffQ + a * 2 * kU5Atom, &q_map, t.h * kU5HD + a * 32, t.q0, &bars.qk_full);
                    tma_load_2d(smem + kU5OffK + a * 2 * kU5Atom, &k_map, t.h * kU5HD + a * 32, t.k0, &bars.qk_full);
                }
                // V once the previous unit's raw tile has been transposed away
                if (k > 0 && !mbar_wait_abort(&bars.v_conv, (k - 1) & 1, abortp)) {
                    give_up(0x12);
                    break;
                }
                mbar_expect_tx(&bars.v_full, 2 * kU5Atom);
#pragma unroll
                for (int a = 0; a < 2; ++a)
                    tma_load_2d(smem + kU5OffV + a * kU5Atom, &v_map, t.h * kU5HD + a * 32, t.k0, &bars.v_full);
                ++k;
            }
            // copies still in flight must have landed before the CTA's shared memory is given up
            // (only an aborted run can get here with any outstanding)
            if (k > 0) {
                mbar_wait(&bars.qk_full, (k - 1) & 1);
                if (!*abortp) mbar_wait(&bars.v_full, (k - 1) & 1);
            }
        }
    } else if (warp == 8) {
        // ================= MMA issuer =================
        if (lane == 0) {
            constexpr uint32_t kIdS256 = t5_idesc(kU5Rows, 256, 0), kIdS128 = t5_idesc(kU5Rows, 128, 0);
            constexpr uint32_t kIdO128 = t5_idesc(kU5Rows, 128, 0), kIdO64 = t5_idesc(kU5Rows, 64, 0);
            int k = 0;
            for (int u = blockIdx.x; u < units && !*abortp; u += gridDim.x) {
                const U5Unit t = u5_unit(d, u);
                if (t.nq <= 0 || t.nk <= 0) continue;
                U5_T0();
                // ---- S = Q K^T: main terms in columns [0, 128), small terms in [128, 256) ----
                if (!mbar_wait_abort(&bars.qk_conv, k & 1, abortp)) {
                    give_up(0x21);
                    break;
                }
                U5_ACC(0, 0);
                // the score columns still hold the previous unit's probabilities until its P V is done
                if (k > 0 && !mbar_wait_abort(&bars.o_done, (k - 1) & 1, abortp)) {
                    give_up(0x22);
                    break;
                }
                U5_ACC(0, 1);
                tc_fence_after();
#pragma unroll
                for (int a = 0; a < 2; ++a) {
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        const uint32_t qa = sbase + kU5OffQ + a * 2 * kU5Atom + kk * 32;
                        const uint32_t ka = sbase + kU5OffK + a * 2 * kU5Atom + kk * 32;
                        const uint64_t q_hi = u5_desc_sw128(qa, 16, 1024), q_lo = u5_desc_sw128(qa + kU5Atom, 16, 1024);
                        const uint64_t k_wide = u5_desc_sw128(ka, 16, 1024); // 256 rows: hi plane then lo plane
                        mma_ss(tmem + kU5ColS, q_hi, k_wide, kIdS256, (a | kk) ? 1u : 0u);
                        mma_ss(tmem + kU5ColSmall, q_lo, k_wide, kIdS128, 1u);
                    }
                }
                tc_commit(&bars.s_done);
                U5_ACC(0, 2);
                // ---- O = P V: main terms in 64 columns, small terms in the next 64 ----
                if (!mbar_wait_abort(&bars.v_conv, k & 1, abortp)) {
                    give_up(0x23);
                    break;
                }
                U5_ACC(0, 3);
                if (!mbar_wait_abort(&bars.p_ready, k & 1, abortp)) {
                    give_up(0x24);
                    break;
                }
                U5_ACC(0, 4);
                if (k >= 2 && !mbar_wait_abort(&bars.o_free[k & 1], ((k - 2) >> 1) & 1, abortp)) {
                    give_up(0x25);
                    break;
                }
                tc_fence_after();
                const uint32_t ocol = tmem + kU5ColO + (uint32_t)(k & 1) * 128;
#pragma unroll
                for (int ks = 0; ks < 16; ++ks) {
                    // 8 keys per step: two 4-key columns of V^T; rows 0-63 hi, 64-127 lo
                    const uint64_t v_wide = t5_desc(sbase + kU5OffVT + ks * 2 * kU5VtLbo, kU5VtLbo, 128);
                    mma_ts(ocol, tmem + kU5ColS + ks * 8, v_wide, kIdO128, ks ? 1u : 0u);
                    mma_ts(ocol + 64, tmem + kU5ColSmall + ks * 8, v_wide, kIdO64, 1u);
                }
                tc_commit(&bars.o_done);
                U5_ACC(0, 5);
                ++k;
            }
            // whatever was issued has completed before the TMEM is given back
            tc_commit(&bars.fin);
            mbar_wait(&bars.fin, 0);
        }
    } else {
        // ================= workers (warps 0-7) =================
        // Row i of the unit is TMEM lane i; warps w and w + 4 may both touch lanes 32 (w & 3) .. + 31, so
        // two threads share a row: `half` 0 takes key chunks 0 and 2 and output columns 0-31, half 1
        // chunks 1 and 3 and columns 32-63. Between the pieces of the softmax the same threads split the
        // next unit's Q / K and transpose this unit's V, so that those passes run beside the MMAs.
        const int rg = warp & 3, half = warp >> 2, row = rg * 32 + lane;
        const uint32_t trow = tmem + ((uint32_t)(rg * 32) << 16);
        const float qscale = d.scale * kLog2e;
        auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + rg) : "memory"); };
        // next unit at or after u that every role processes; rows of sequences without keys get their zeros here
        auto next_unit = [&](int u) {
            for (; u < units; u += gridDim.x) {
                const U5Unit t = u5_unit(d, u);
                if (t.nq > 0 && t.nk > 0) break;
                if (t.nq > 0 && row < t.nq) {
                    float *o = d.out + (int64_t)(t.q0 + row) * d.out_stride + (int64_t)t.h * kU5HD + half * 32;
#pragma unroll
                    for (int c = 0; c < 8; ++c) *reinterpret_cast<float4 *>(o + c * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
            return u;
        };
        // Q and K: four atoms of 1024 16-byte pieces; hi = value rounded to TF32 (written back in place),
        // lo = value - hi. The swizzle permutes pieces inside a 128-byte row only, so an elementwise pass
        // needs no address arithmetic beyond the plane offset.
        auto convert_qk = [&](int kk) -> bool {
            if (!mbar_wait_abort(&bars.qk_full, kk & 1, abortp)) {
                give_up(0x31);
                return false;
            }
#pragma unroll
            for (int op = 0; op < 2; ++op) {
#pragma unroll
                for (int a = 0; a < 2; ++a) {
                    uint8_t *plane = smem + (op ? kU5OffK : kU5OffQ) + a * 2 * kU5Atom;
#pragma unroll
                    for (int it = 0; it < 4; ++it) {
                        const int f = it * 256 + tid;
                        float4 x = *reinterpret_cast<const float4 *>(plane + f * 16);
                        const float e[4] = {x.x, x.y, x.z, x.w};
                        uint4 hi4, lo4;
                        uint32_t *hp = &hi4.x, *lp = &lo4.x;
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            hp[c] = t5_tf32_finite(e[c]);
                            lp[c] = __float_as_uint(e[c] - __uint_as_float(hp[c]));
                        }
                        *reinterpret_cast<uint4 *>(plane + f * 16) = hi4;
                        *reinterpret_cast<uint4 *>(plane + kU5Atom + f * 16) = lo4;
                    }
                }
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars.qk_conv);
            return true;
        };

        int k = 0;
        int u = next_unit(blockIdx.x);
        bool ok = true;
        if (u < units) ok = convert_qk(0);
        while (ok && u < units && !*abortp) {
            const U5Unit t = u5_unit(d, u);
            U5_T0();
            // ---- (1) V^T of this unit; the previous unit's P V must have finished reading the old one ----
            if (!mbar_wait_abort(&bars.v_full, k & 1, abortp)) {
                give_up(0x32);
                break;
            }
            if (k > 0 && !mbar_wait_abort(&bars.o_done, (k - 1) & 1, abortp)) {
                give_up(0x33);
                break;
            }
            if (tid == 96) U5_ACC(1, 0);
            {
                // Rows at and past the sequence's last key belong to the next sequence (or are the load's
                // zero fill) and are cleared: their probabilities are zero, but 0 x inf would not be. A
                // warp step covers 16 keys x 8 value columns: every lane reads one 16-byte piece and writes
                // its four elements in a rotated order, so that the 32 lanes of a store hit 32 banks.
                const int rl = (lane & 3) + 4 * (lane >> 3), cl = (lane >> 2) & 1, xo = lane >> 3;
#pragma unroll 4
                for (int it = 0; it < 8; ++it) {
                    const int blk = it * 8 + warp;            // 64 blocks: 8 key groups x 8 column pairs
                    const int r = (blk & 7) * 16 + rl;        // key
                    const int c = (blk >> 3) * 2 + cl;        // 16-byte piece of the row: value columns 4c .. 4c + 3
                    const uint8_t *src = smem + kU5OffV + (c >> 3) * kU5Atom + r * 128 + (((c & 7) ^ (r & 7)) << 4);
                    float4 x = *reinterpret_cast<const float4 *>(src);
                    if (r >= t.nk) x = make_float4(0.f, 0.f, 0.f, 0.f);
                    float e0 = x.x, e1 = x.y, e2 = x.z, e3 = x.w;
                    if (xo & 1) {
                        const float tt = e0;
                        e0 = e1; e1 = e2; e2 = e3; e3 = tt;
                    }
                    if (xo & 2) {
                        float tt = e0;
                        e0 = e2; e2 = tt;
                        tt = e1;
                        e1 = e3; e3 = tt;
                    }
                    const float ve[4] = {e0, e1, e2, e3};
                    uint8_t *dst = smem + kU5OffVT + (r >> 2) * kU5VtLbo + (r & 3) * 4;
#pragma unroll
                    for (int st = 0; st < 4; ++st) {
                        const int n = c * 4 + ((st + xo) & 3);
                        const uint32_t o = (n >> 3) * 128 + (n & 7) * 16;
                        const uint32_t vh = t5_tf32_finite(ve[st]);
                        *reinterpret_cast<uint32_t *>(dst + o) = vh;
                        *reinterpret_cast<uint32_t *>(dst + 1024 + o) = __float_as_uint(ve[st] - __uint_as_float(vh));
                    }
                }
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars.v_conv);
            if (tid == 96) U5_ACC(1, 1);
            // ---- (2) scores -> probabilities, this thread's two key chunks of its row ----
            int lo = 0, hi = 0;
            if (row < t.nq) {
                const SeqMask sm = resolve_mask(d.mask, t.b, t.q0, t.k0, t.nq, t.nk);
                row_range(sm, row, lo, hi);
                if (hi <= lo) lo = hi = 0;
            }
            int whi = hi; // 32-key chunks the row group has to look at: up to the largest key any row may see
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) whi = max(whi, __shfl_xor_sync(0xffffffffu, whi, o));
            const int nch = (whi + 31) >> 5;
            if (!mbar_wait_abort(&bars.s_done, k & 1, abortp)) {
                give_up(0x41);
                break;
            }
            if (tid == 96) U5_ACC(1, 2);
            tc_fence_after();
            float sc[2][32];
            float mx = -INFINITY;
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
                const int ch = half + 2 * cc;
                if (ch < nch) {
                    float a[32], b[32];
                    tmem_ld32(trow + kU5ColS + ch * 32, a);
                    tmem_ld32(trow + kU5ColSmall + ch * 32, b);
                    tc_wait_ld();
                    // a chunk that every row of the warp sees whole needs no per-key range test
                    const bool whole = __all_sync(0xffffffffu, lo <= ch * 32 && hi >= ch * 32 + 32);
                    if (whole) {
#pragma unroll
                        for (int c = 0; c < 32; ++c) {
                            const float sv = (a[c] + b[c]) * qscale;
                            sc[cc][c] = finite_f(sv) ? sv : -INFINITY;
                            mx = fmaxf(mx, sc[cc][c]);
                        }
                    } else {
#pragma unroll
                        for (int c = 0; c < 32; ++c) {
                            const int j = ch * 32 + c;
                            const float sv = (a[c] + b[c]) * qscale;
                            sc[cc][c] = (j >= lo && j < hi && finite_f(sv)) ? sv : -INFINITY;
                            mx = fmaxf(mx, sc[cc][c]);
                        }
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < 32; ++c) sc[cc][c] = -INFINITY;
                }
            }
            if (tid == 96) U5_ACC(1, 9);
            xmax[half][row] = mx;
            pair_sync();
            if (tid == 96) U5_ACC(1, 10);
            mx = fmaxf(mx, xmax[half ^ 1][row]);
            const float ref = mx == -INFINITY ? 0.0f : mx;
            float l = 0.0f;
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
                const int ch = half + 2 * cc;
                uint32_t ph[32], pl[32];
                if (ch < nch) {
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        const float p = t5_ex2(sc[cc][c] - ref); // masked entries are -inf: 0
                        l += p;
                        ph[c] = t5_tf32_finite(p);
                        pl[c] = __float_as_uint(p - __uint_as_float(ph[c]));
                    }
                } else { // columns past the row group's range: the MMA still reads them
#pragma unroll
                    for (int c = 0; c < 32; ++c) ph[c] = pl[c] = 0u;
                }
                tmem_st32(trow + kU5ColS + ch * 32, ph);
                tmem_st32(trow + kU5ColSmall + ch * 32, pl);
            }
            xsum[half][row] = l;
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars.p_ready);
            if (tid == 96) U5_ACC(1, 3);
            // ---- (3) the next unit's Q / K planes, while this unit's P V runs ----
            const int un = next_unit(u + gridDim.x);
            if (un < units && !convert_qk(k + 1)) break;
            if (tid == 96) U5_ACC(1, 4);
            // ---- (4) output: (main + small) / row sum, this thread's 32 columns ----
            if (!mbar_wait_abort(&bars.o_done, k & 1, abortp)) {
                give_up(0x42);
                break;
            }
            if (tid == 96) U5_ACC(1, 5);
            tc_fence_after();
            pair_sync(); // the partner's sum is there; and its reads of this round's maximum are over
            if (tid == 96) U5_ACC(1, 7);
            l = xsum[0][row] + xsum[1][row];
            const float inv = l > 0.0f ? 1.0f / l : 0.0f; // rows without keys give zeros
            {
                const uint32_t ocol = trow + kU5ColO + (uint32_t)(k & 1) * 128 + half * 32;
                float a[32], b[32];
                tmem_ld32(ocol, a);
                tmem_ld32(ocol + 64, b);
                tc_wait_ld();
                if (tid == 96) U5_ACC(1, 8);
                // A thread holds 128 contiguous bytes of one row; stored as they are, a warp's store would
                // touch 32 rows with 16 bytes each. The warp trades them through shared memory (4 KB of
                // the V^T region, which nobody uses between this unit's P V and the next transposition;
                // pieces XOR-swizzled by row so that both passes are conflict-free) and then writes four
                // whole 128-byte row segments per instruction.
                uint8_t *stage = smem + kU5OffVT + warp * 4096;
#pragma unroll
                for (int c = 0; c < 8; ++c)
                    *reinterpret_cast<float4 *>(stage + lane * 128 + ((c ^ (lane & 7)) << 4)) =
                        make_float4((a[c * 4] + b[c * 4]) * inv, (a[c * 4 + 1] + b[c * 4 + 1]) * inv,
                                    (a[c * 4 + 2] + b[c * 4 + 2]) * inv, (a[c * 4 + 3] + b[c * 4 + 3]) * inv);
                __syncwarp();
                const int pr = lane >> 3, pc = lane & 7;
                float *obase = d.out + (int64_t)t.q0 * d.out_stride + (int64_t)t.h * kU5HD + half * 32 + pc * 4;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int rr = j * 4 + pr; // row inside this warp's 32
                    const float4 v4 = *reinterpret_cast<const float4 *>(stage + rr * 128 + ((pc ^ (rr & 7)) << 4));
                    if (rg * 32 + rr < t.nq) *reinterpret_cast<float4 *>(obase + (int64_t)(rg * 32 + rr) * d.out_stride) = v4;
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars.o_free[k & 1]);
            if (tid == 96) U5_ACC(1, 6);
            // every warp has read its staged rows back before anyone's next transposition writes there
            asm volatile("bar.sync 5, 256;" ::: "memory");
            u = un;
            ++k;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, kU5Cols);
}

// Error word of this kernel: returns and clears it (device already synchronised).
int unit5_take_error() {
    unsigned int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_u5_error, sizeof(v)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_u5_error, &zero, sizeof(zero));
    return (int)v;
}
int unit5_take_error_on(cudaStream_t s) {
    unsigned int v = 0, zero = 0;
    if (cudaMemcpyFromSymbolAsync(&v, g_u5_error, sizeof(v), 0, cudaMemcpyDeviceToHost, s) != cudaSuccess) return -1;
    if (cudaStreamSynchronize(s) != cudaSuccess) return -1;
    if (v) {
        cudaMemcpyToSymbolAsync(g_u5_error, &zero, sizeof(zero), 0, cudaMemcpyHostToDevice, s);
        cudaStreamSynchronize(s);
    }
    return (int)v;
}

// ---- host side -----------------------------------------------------------------------------

bool unit5_kernel_supports(const fblt_attn_desc &d, const char **why) {
    if (d.head_dim != kU5HD) {
        *why = "unit kernel: head_dim must be 64";
        return false;
    }
    if (d.max_q > kU5Rows || d.max_k > kU5Rows) {
        *why = "unit kernel: at most 128 query rows and 128 keys per sequence";
        return false;
    }
    if (d.total_q_rows <= 0 || d.total_k_rows <= 0) {
        *why = "unit kernel: total_q_rows / total_k_rows must be given (the tiled loads need the tensors' extents)";
        return false;
    }
    if (d.mask.group_rule == FBLT_GROUP_IDS) {
        *why = "explicit group ids are not a key range";
        return false;
    }
    if (d.rope_cos || d.precision != FBLT_PREC_FP32) {
        *why = "unit kernel: no fused rotary embedding, fp32-equivalent precision only";
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
    if ((int64_t)d.batch * d.num_heads > 0x7fffffff) {
        *why = "batch * heads beyond int32";
        return false;
    }
    return true;
}

typedef CUresult (*U5EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                    const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static U5EncodeTiledFn u5_encoder() {
    static std::atomic<U5EncodeTiledFn> cached{nullptr};
    U5EncodeTiledFn fn = cached.load(std::memory_order_acquire);
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        fn = (U5EncodeTiledFn)p;
        cached.store(fn, std::memory_order_release);
    }
    return fn;
}

// Map of the head columns of a [rows, row stride] fp32 tensor for 128-row x 32-column boxes with the
// 128-byte swizzle; rows past `rows` read as zeros and are never touched in memory.
static int u5_make_map(CUtensorMap *map, const float *base, int64_t stride, int64_t rows, int64_t cols) {
    U5EncodeTiledFn enc = u5_encoder();
    if (!enc) return fail(FBLT_ERR_CUDA, "attn: cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)stride * sizeof(float)};
    const cuuint32_t box[2] = {32, (cuuint32_t)kU5Rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void *)base, dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(FBLT_ERR_CUDA, "attn: cuTensorMapEncodeTiled failed with code %d", (int)r);
    return FBLT_OK;
}

int launch_unit5_kernel(const fblt_attn_desc &d, cudaStream_t stream) {
    static std::atomic<uint64_t> configured{0}; // one bit per device ordinal; the attribute is per device
    static std::atomic<int> sm_count[64];
    int dev = 0;
    FBLT_CUDA_TRY(cudaGetDevice(&dev));
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        FBLT_CUDA_TRY(cudaFuncSetAttribute(unit5_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kU5Smem));
        int sms = 0;
        FBLT_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        sm_count[dev & 63].store(sms, std::memory_order_relaxed);
        configured.fetch_or(bit, std::memory_order_release);
    }
    const int64_t cols = (int64_t)d.num_heads * kU5HD;
    CUtensorMap qm, km, vm;
    int st = u5_make_map(&qm, d.q, d.q_stride, d.total_q_rows, cols);
    if (st == FBLT_OK) st = u5_make_map(&km, d.k, d.k_stride, d.total_k_rows, cols);
    if (st == FBLT_OK) st = u5_make_map(&vm, d.v, d.v_stride, d.total_k_rows, cols);
    if (st != FBLT_OK) return st;
    const int units = d.batch * d.num_heads;
    const int sms = sm_count[dev & 63].load(std::memory_order_relaxed);
    const int grid = units < sms ? units : sms;
    unit5_attn_kernel<<<grid, kU5Threads, kU5Smem, stream>>>(d, qm, km, vm, units);
    count_launch();
    return check_launch("unit5_attn_kernel");
}

#ifdef U5_DEBUG
} // namespace fblt
extern "C" int fblt_u5_debug_read(unsigned long long *out, int clear) {
    unsigned long long z[8][16] = {};
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out, fblt::g_u5_dbg, sizeof(z));
    if (clear) cudaMemcpyToSymbol(fblt::g_u5_dbg, z, sizeof(z));
    return 0;
}
namespace fblt {
#endif
} // namespace fblt
