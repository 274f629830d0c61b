// L1 tcgen05 kernel for sequences of at most 128 keys (head_dim 64: the patch-transformer shapes, and byte
// queries over a sequence's patches): one (sequence, head, 128 query rows) unit = one 128 x 128 score
// tile, so the softmax is a single pass with no running maximum and no rescale of the output.
//
// Persistent, one CTA per SM, roles that meet only on mbarriers:
//   loader (1 thread)   raw fp32 Q, K, V tiles of the NEXT unit by tiled TMA (no multicast, this
//                       GPU's memory only): Q / K (128-byte swizzle, K-major operands) as soon as the
//                       score MMAs that read the current ones have completed, V (128-byte swizzle of
//                       32-byte chunks: the only layout an MN-major TF32 operand may have, so the tile
//                       is used as it lands, keys along K, without a transposition) as soon as the
//                       current unit's P V has completed;
//   issuer (1 thread)   S = Q K^T as 24 tcgen05.mma into one accumulator (Q_hi K_lo + Q_lo K_hi first,
//                       then Q_hi K_hi), O = P V as 32 (P_hi x [V_hi | V_lo] is ONE 128 x 128 x 8
//                       instruction into a main and a small-term accumulator, P_lo x V_hi a second
//                       one) with P read from TMEM, completion by tcgen05.commit;
//   workers (16 warps)  four threads per query row (warps w, w + 4, w + 8, w + 12 all reach TMEM lanes
//                       32 (w & 3) ..): in turn they split this unit's V in place into TF32 (hi, lo)
//                       planes -- an elementwise pass over the swizzled bytes, like the one for Q / K --
//                       read the scores of their quarter of the keys, trade the row maximum, write P
//                       (hi, lo) to TMEM, split the next unit's Q / K while this unit's P V runs, then
//                       read their 16 columns of O, scale by 1 / row sum and store whole 64-byte row
//                       pieces (rows are traded through shared memory first).
// TMEM: 128 columns of scores / P_hi, 128 of P_lo, two output accumulators of 128 columns.
// Shared memory: 64 KB each for Q, K and V (raw / hi plane and lo plane), 32 KB of output staging.
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
constexpr int kU5Workers = 16;                       // worker warps: conversion, softmax, output
constexpr int kU5Threads = 32 * (kU5Workers + 3);    // + warp 16 issuer, warp 17 loader, warp 18 output storer
constexpr int kU5Atom = 16384;                       // one 128-row x 32-column fp32 box (rows of 128 bytes)
// shared memory map (bytes). Q and K: per 32-column atom the raw / hi plane followed by the lo plane.
// V: both raw / hi atoms, then both lo atoms, so that [V_hi | V_lo] is four 32-column blocks at one stride.
constexpr int kU5OffQ = 0, kU5OffK = 4 * kU5Atom, kU5OffV = 8 * kU5Atom, kU5OffStage = 12 * kU5Atom;
constexpr int kU5Smem = 14 * kU5Atom; // + < 3 KB of static shared memory: the 227 KB of an SM
// TMEM columns
constexpr uint32_t kU5ColS = 0, kU5ColPhi = 128, kU5ColPlo = 256, kU5ColO = 384, kU5Cols = 512;

__device__ unsigned int g_u5_error; // 0 = ok; otherwise (code << 24) | blockIdx.x of the first CTA that gave up

struct U5Bars {
    uint64_t qk_full, v_full, qk_conv, v_conv, s_done, p_ready, o_done, out_full, out_free, fin;
};

// Shared-memory matrix descriptor for the 128-byte-swizzled layouts a tiled TMA load produces
// (rows of 128 bytes, 8-row groups of 1024 bytes): descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t u5_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) | (2ull << 61);
}
// The same for an MN-major 32-bit operand: rows of 128 bytes whose 32-byte chunks are swizzled over
// groups of 4 rows (layout type 1). Leading offset = stride between 32-element blocks along N, stride
// offset = stride between 4-row groups along K.
__device__ __forceinline__ uint64_t u5_desc_mn32(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) | (1ull << 61);
}

#ifdef U5_DEBUG
// cycle counters of CTA 0, one row per role: [role][slot]
__device__ unsigned long long g_u5_dbg[8][16];
__device__ int g_u5_knob[4];
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

// One unit: 128 query rows (tile number qrow0 / 128 of sequence b) of head h over all keys of the sequence.
// q0 / nq are the tile's first packed row and row count, sq0 / snq the sequence's.
struct U5Unit {
    int b, h, q0, nq, k0, nk, qrow0, sq0, snq;
};
// What the loader publishes for each unit it loads (u < 0: no more units for this CTA).
struct U5Geo {
    int u, b, h, q0, nq, k0, nk, qrow0, sq0, snq, pad0, pad1;
};
// Output maps: boxes of 128, 64, ... 1 rows x 32 columns, so that a unit's nq rows go out as one store
// per set bit of nq and column half, without touching the next sequence's rows.
struct U5OutMaps {
    CUtensorMap m[8];
};

// Unit `u` of the launch (heads fastest, then query tiles, then sequences), or nq <= 0 for units with
// nothing to do (skipped by every role alike).
__device__ __forceinline__ U5Unit u5_unit(const fblt_attn_desc &d, int u, int qtiles) {
    U5Unit t;
    const int per_seq = d.num_heads * qtiles;
    t.b = u / per_seq;
    const int rem = u - t.b * per_seq, qt = rem / d.num_heads;
    t.h = rem - qt * d.num_heads;
    t.sq0 = d.cu_q[t.b];
    t.snq = d.cu_q[t.b + 1] - t.sq0;
    t.qrow0 = qt * kU5Rows;
    t.q0 = t.sq0 + t.qrow0;
    t.nq = min(kU5Rows, t.snq - t.qrow0);
    t.k0 = d.cu_k[t.b];
    t.nk = d.cu_k[t.b + 1] - t.k0;
    return t;
}

__global__ void __launch_bounds__(kU5Threads, 1)
    unit5_attn_kernel(fblt_attn_desc d, const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                      const __grid_constant__ CUtensorMap v_map, const __grid_constant__ U5OutMaps out_maps, int units, int qtiles) {
    extern __shared__ __align__(1024) uint8_t smem[]; // swizzle atoms: 1 KB alignment
    __shared__ __align__(8) U5Bars bars;
    __shared__ __align__(16) U5Geo geo[4];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_word;
    __shared__ float xsum[4][kU5Rows]; // the four quarters of a row trade their sums here, their maxima through the staging area
    const uint32_t sbase = smem_u32(smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        mbar_init(&bars.qk_full, 1);
        mbar_init(&bars.v_full, 1);
        mbar_init(&bars.qk_conv, kU5Workers);
        mbar_init(&bars.v_conv, kU5Workers);
        mbar_init(&bars.s_done, 1);
        mbar_init(&bars.p_ready, kU5Workers);
        mbar_init(&bars.o_done, 1);
        mbar_init(&bars.out_full, kU5Workers);
        mbar_init(&bars.out_free, 1);
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

    if (warp == kU5Workers + 1) {
        // ================= loader =================
        if (lane == 0) {
            int k = 0; // processed units of this CTA
            for (int u = blockIdx.x; u < units && !*abortp; u += gridDim.x) {
                const U5Unit t = u5_unit(d, u, qtiles);
                if (t.nq <= 0) continue;
                if (t.nk <= 0) { // a sequence without keys: its rows are zeros, and no other role sees the unit
                    for (int i = 0; i < t.nq * (kU5HD / 4); ++i)
                        *reinterpret_cast<float4 *>(d.out + (int64_t)(t.q0 + i / (kU5HD / 4)) * d.out_stride +
                                                    (int64_t)t.h * kU5HD + (i % (kU5HD / 4)) * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
                    continue;
                }
                // Q / K of the previous unit have been read once its score MMAs completed
                if (k > 0 && !mbar_wait_abort(&bars.s_done, (k - 1) & 1, abortp)) {
                    give_up(0x11);
                    break;
                }
                // the unit's geometry travels with the barrier: whoever has waited for qk_full may read it.
                // Slot k & 3 was last read for unit k - 4, two score rounds ago.
                geo[k & 3] = U5Geo{u, t.b, t.h, t.q0, t.nq, t.k0, t.nk, t.qrow0, t.sq0, t.snq, 0, 0};
                mbar_expect_tx(&bars.qk_full, 4 * kU5Atom);
#pragma unroll
                for (int a = 0; a < 2; ++a) {
                    tma_load_2d(smem + kU5OffQ + a * 2 * kU5Atom, &q_map, t.h * kU5HD + a * 32, t.q0, &bars.qk_full);
                    tma_load_2d(smem + kU5OffK + a * 2 * kU5Atom, &k_map, t.h * kU5HD + a * 32, t.k0, &bars.qk_full);
                }
                // V (read in place by the P V MMAs) once the previous unit's P V has completed
                if (k > 0 && !mbar_wait_abort(&bars.o_done, (k - 1) & 1, abortp)) {
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
            bool landed = true;
            if (k > 0) {
                landed = mbar_wait(&bars.qk_full, (k - 1) & 1);
                if (!*abortp) landed = mbar_wait(&bars.v_full, (k - 1) & 1) && landed;
            }
            // The end marker is one more phase of qk_full. It must not complete before the workers have
            // seen the last load's phase (a parity wait cannot tell two phases on from none): the last
            // unit's score MMAs, issued after the workers split its Q / K, have completed by then.
            if (landed && !*abortp && (k == 0 || mbar_wait_abort(&bars.s_done, (k - 1) & 1, abortp))) {
                geo[k & 3].u = -1;
                mbar_arrive(&bars.qk_full);
            }
        }
    } else if (warp == kU5Workers + 2) {
        // ================= output storer =================
        // Lane 2 b + a sends the 2^(7-b) rows that bit (7 - b) of nq stands for (they start at nq with that
        // bit and the lower ones cleared), column half a: the staged tile leaves as at most 14 tiled TMA stores.
        // After the last unit the workers arrive once more, with the loader's end marker in the slot. (This
        // warp runs a unit behind the others, so it must not wait on qk_full itself: that barrier may by
        // then be two phases on, which a parity wait cannot tell from none.)
        for (int k = 0; !*abortp; ++k) {
            if (!mbar_wait_abort(&bars.out_full, k & 1, abortp)) {
                if (lane == 0) give_up(0x52);
                break;
            }
            const U5Geo g = geo[k & 3];
            if (g.u < 0) break;
            if (lane < 16) {
                const int bit = 7 - (lane >> 1), a = lane & 1, r = 1 << bit;
                if (g.nq & r) {
                    const int r0 = g.nq & ~(2 * r - 1);
                    tma_store_2d(&out_maps.m[lane >> 1], g.h * kU5HD + a * 32, g.q0 + r0,
                                 smem + kU5OffStage + a * kU5Atom + r0 * 128);
                }
                bulk_commit();
                bulk_wait_read(); // the staging tile may be written again
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars.out_free);
        }
        bulk_wait_all(); // the stores have completed before the CTA's shared memory goes away
    } else if (warp == kU5Workers) {
        // ================= MMA issuer =================
        if (lane == 0) {
            constexpr uint32_t kIdS = t5_idesc(kU5Rows, 128, 0);
            constexpr uint32_t kIdO128 = t5_idesc(kU5Rows, 128, 1), kIdO64 = t5_idesc(kU5Rows, 64, 1);
            // S = Q K^T of unit number kk of this CTA into columns [0, 128): the two small products first,
            // then the main one. The columns are free: the workers copied the previous scores out before
            // they signalled p_ready, which the caller has seen.
            auto issue_scores = [&](int kk) -> bool {
                if (!mbar_wait_abort(&bars.qk_conv, kk & 1, abortp)) {
                    give_up(0x21);
                    return false;
                }
                tc_fence_after();
#pragma unroll
                for (int pass = 0; pass < 2; ++pass) {
#pragma unroll
                    for (int a = 0; a < 2; ++a) {
#pragma unroll
                        for (int kq = 0; kq < 4; ++kq) {
                            const uint32_t qa = sbase + kU5OffQ + a * 2 * kU5Atom + kq * 32;
                            const uint32_t ka = sbase + kU5OffK + a * 2 * kU5Atom + kq * 32;
                            const uint64_t q_hi = u5_desc_sw128(qa, 16, 1024), q_lo = u5_desc_sw128(qa + kU5Atom, 16, 1024);
                            const uint64_t k_hi = u5_desc_sw128(ka, 16, 1024), k_lo = u5_desc_sw128(ka + kU5Atom, 16, 1024);
                            if (pass == 0) {
                                mma_ss(tmem + kU5ColS, q_hi, k_lo, kIdS, (a | kq) ? 1u : 0u);
                                mma_ss(tmem + kU5ColS, q_lo, k_hi, kIdS, 1u);
                            } else {
                                mma_ss(tmem + kU5ColS, q_hi, k_hi, kIdS, 1u);
                            }
                        }
                    }
                }
                tc_commit(&bars.s_done);
                return true;
            };
            auto next_unit = [&](int u) {
                for (; u < units; u += gridDim.x) {
                    const U5Unit t = u5_unit(d, u, qtiles);
                    if (t.nq > 0 && t.nk > 0) break;
                }
                return u;
            };
            int k = 0;
            int u = next_unit(blockIdx.x);
            bool ok = u < units ? issue_scores(0) : true;
            while (ok && u < units && !*abortp) {
                U5_T0();
                // ---- O = P V: main terms in 64 columns, small terms in the next 64. The accumulator is
                // free: every worker read the previous output before it signalled this unit's p_ready. ----
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
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < 16; ++ks) {
                    // 8 keys per step = 8 rows of 128 bytes; N runs over the four 32-column blocks
                    // V_hi[0:32] V_hi[32:64] V_lo[0:32] V_lo[32:64], one atom apart
                    const uint64_t v_wide = u5_desc_mn32(sbase + kU5OffV + ks * 1024, kU5Atom, 512);
                    mma_ts(tmem + kU5ColO, tmem + kU5ColPhi + ks * 8, v_wide, kIdO128, ks ? 1u : 0u);
                    mma_ts(tmem + kU5ColO + 64, tmem + kU5ColPlo + ks * 8, v_wide, kIdO64, 1u);
                }
                tc_commit(&bars.o_done);
                U5_ACC(0, 5);
                // ---- the next unit's scores queue up right behind: they run while the workers store this output ----
                u = next_unit(u + gridDim.x);
                ++k;
                if (u < units) ok = issue_scores(k);
                U5_ACC(0, 2);
            }
            // whatever was issued has completed before the TMEM is given back
            tc_commit(&bars.fin);
            mbar_wait(&bars.fin, 0);
        }
    } else {
        // ================= workers (warps 0-15) =================
        // Row i of the unit is TMEM lane i; warp w may touch lanes 32 (w & 3) .. + 31 only, so the four
        // warps with the same w & 3 share 32 rows: `qt` = w >> 2 takes key chunk qt of the scores and
        // output columns 16 qt .. + 15. Between the pieces of the softmax the same threads split this
        // unit's V and the next unit's Q / K, so that those passes run beside the MMAs.
        const int rg = warp & 3, qt = warp >> 2, row = rg * 32 + lane;
        const uint32_t trow = tmem + ((uint32_t)(rg * 32) << 16);
        const float qscale = d.scale * kLog2e;
        auto group_sync = [&]() { asm volatile("bar.sync %0, 128;" ::"r"(1 + rg) : "memory"); };
        // One 16-byte piece: the raw fp32 bits stay where they are as the hi operand (a TF32 MMA reads the
        // upper 19 bits of each word), lo = value - (value with the low 13 mantissa bits cleared). Both
        // swizzles permute pieces inside a 128-byte row only, so an elementwise pass needs no address
        // arithmetic beyond the plane offset.
        auto split_piece = [&](uint8_t *hi_at, uint8_t *lo_at, bool keep) {
            float4 x = *reinterpret_cast<const float4 *>(hi_at);
            if (!keep) {
                x = make_float4(0.f, 0.f, 0.f, 0.f);
                *reinterpret_cast<float4 *>(hi_at) = x;
            }
            const float e[4] = {x.x, x.y, x.z, x.w};
            uint4 lo4;
            uint32_t *lp = &lo4.x;
#pragma unroll
            for (int c = 0; c < 4; c += 2) { // x - trunc(x) for two words per instruction (packed fp32 multiply-add)
                const float2 t = make_float2(__uint_as_float(__float_as_uint(e[c]) & 0xFFFFE000u),
                                             __uint_as_float(__float_as_uint(e[c + 1]) & 0xFFFFE000u));
                const float2 r = __ffma2_rn(t, make_float2(-1.0f, -1.0f), make_float2(e[c], e[c + 1]));
                lp[c] = __float_as_uint(r.x);
                lp[c + 1] = __float_as_uint(r.y);
            }
            *reinterpret_cast<uint4 *>(lo_at) = lo4;
        };
        // Geometry of this CTA's unit number kk and this thread's key range in it, then the split of its
        // Q and K (four atoms of 1024 pieces). g.u < 0: no such unit (or the wait gave up).
        struct Work {
            U5Geo g;
            int lo, hi;
        };
        auto fetch_and_convert = [&](int kk) -> Work {
            Work w;
            w.lo = w.hi = 0;
            if (!mbar_wait_abort(&bars.qk_full, kk & 1, abortp)) {
                give_up(0x31);
                w.g.u = -1;
                return w;
            }
            w.g = geo[kk & 3];
            if (w.g.u < 0) return w;
            if (row < w.g.nq) {
                const SeqMask sm = resolve_mask(d.mask, w.g.b, w.g.sq0, w.g.k0, w.g.snq, w.g.nk);
                row_range(sm, w.g.qrow0 + row, w.lo, w.hi);
                if (w.hi <= w.lo) w.lo = w.hi = 0;
            }
#pragma unroll
            for (int op = 0; op < 2; ++op) {
#pragma unroll
                for (int a = 0; a < 2; ++a) {
                    uint8_t *plane = smem + (op ? kU5OffK : kU5OffQ) + a * 2 * kU5Atom;
#pragma unroll
                    for (int it = 0; it < 1024 / (32 * kU5Workers); ++it) {
                        const int f = it * 32 * kU5Workers + tid;
                        split_piece(plane + f * 16, plane + kU5Atom + f * 16, true);
                    }
                }
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars.qk_conv);
            return w;
        };
        // This thread's 16 output columns in the staging tile: two 128-row x 128-byte atoms with the
        // 128-byte swizzle of the output maps; the first word of the first piece carries the thread's
        // maximum during the softmax.
        uint8_t *const srow = smem + kU5OffStage + row * 128;
        auto piece_at = [&](int q, int c) { return srow + (q >> 1) * kU5Atom + ((((q & 1) * 4 + c) ^ (row & 7)) << 4); };

        int k = 0;
        Work w = fetch_and_convert(0);
        while (w.g.u >= 0 && !*abortp) {
            const U5Geo t = w.g;
            const int lo = w.lo, hi = w.hi;
            U5_T0();
            // ---- (1) V of this unit, in place. Rows at and past the sequence's last key belong to the
            // next sequence (or are the load's zero fill) and are cleared: their probabilities are
            // zero, but 0 x inf would not be. ----
            if (!mbar_wait_abort(&bars.v_full, k & 1, abortp)) {
                give_up(0x32);
                break;
            }
            if (tid == 96) U5_ACC(1, 0);
#pragma unroll
            for (int a = 0; a < 2; ++a) {
#pragma unroll
                for (int it = 0; it < 1024 / (32 * kU5Workers); ++it) {
                    const int f = it * 32 * kU5Workers + tid; // piece f of the atom: key f >> 3
                    uint8_t *at = smem + kU5OffV + a * kU5Atom + f * 16;
                    split_piece(at, at + 2 * kU5Atom, (f >> 3) < t.nk);
                }
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars.v_conv);
            if (tid == 96) U5_ACC(1, 1);
            // ---- (2) scores -> probabilities, this thread's key chunk of its row ----
            int whi = hi; // 32-key chunks the row group has to look at: up to the largest key any row may see
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) whi = max(whi, __shfl_xor_sync(0xffffffffu, whi, o));
            const bool live = qt * 32 < whi;
            if (!mbar_wait_abort(&bars.s_done, k & 1, abortp)) {
                give_up(0x41);
                break;
            }
            if (tid == 96) U5_ACC(1, 2);
            tc_fence_after();
            // The scores stay unscaled in registers: scale > 0 keeps the order, and the scale folds into the
            // exponent's multiply-add. Non-finite scores count as masked; whether there is one is found by
            // one multiply-add per score (x * 0 is NaN for them), the per-score test runs only then.
            float sc[32];
            float mx = -INFINITY, qs = qscale;
            if (live) {
                tmem_ld32(trow + kU5ColS + qt * 32, sc);
                tc_wait_ld();
                float2 odd2 = make_float2(0.0f, 0.0f);
#pragma unroll
                for (int c = 0; c < 32; c += 2) odd2 = __ffma2_rn(make_float2(sc[c], sc[c + 1]), make_float2(0.0f, 0.0f), odd2);
                const float odd = odd2.x + odd2.y;
                if (odd != odd || !(qscale > 0.0f)) {
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        const float sv = sc[c] * qscale;
                        sc[c] = finite_f(sv) ? sv : -INFINITY;
                    }
                    qs = 1.0f;
                }
                // a chunk that every row of the warp sees whole needs no per-key range test
                const bool whole = __all_sync(0xffffffffu, lo <= qt * 32 && hi >= qt * 32 + 32);
                if (whole) {
#pragma unroll
                    for (int c = 0; c < 32; ++c) mx = fmaxf(mx, sc[c]);
                } else {
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        const int j = qt * 32 + c;
                        sc[c] = (j >= lo && j < hi) ? sc[c] : -INFINITY;
                        mx = fmaxf(mx, sc[c]);
                    }
                }
                mx *= qs; // the four quarters of a row trade their maxima in the scaled domain
            }
            if (tid == 96) U5_ACC(1, 9);
            // the staging tile is free again once the previous unit's stores have read it
            if (k > 0 && !mbar_wait_abort(&bars.out_free, (k - 1) & 1, abortp)) {
                give_up(0x43);
                break;
            }
            *reinterpret_cast<float *>(piece_at(qt, 0)) = mx;
            group_sync();
            if (tid == 96) U5_ACC(1, 10);
            mx = fmaxf(fmaxf(*reinterpret_cast<const float *>(piece_at(0, 0)), *reinterpret_cast<const float *>(piece_at(1, 0))),
                       fmaxf(*reinterpret_cast<const float *>(piece_at(2, 0)), *reinterpret_cast<const float *>(piece_at(3, 0))));
            const float ref = mx == -INFINITY ? 0.0f : mx;
            float2 l2 = make_float2(0.0f, 0.0f);
#pragma unroll
            for (int pc = 0; pc < 2; ++pc) {
                uint32_t ph[16], pl[16];
                if (live) {
#pragma unroll
                    for (int c = 0; c < 16; c += 2) { // two scores per packed instruction; masked entries are -inf: 0
                        const float2 x = __ffma2_rn(make_float2(sc[pc * 16 + c], sc[pc * 16 + c + 1]), make_float2(qs, qs),
                                                    make_float2(-ref, -ref));
                        const float2 pp = make_float2(t5_ex2(x.x), t5_ex2(x.y));
                        l2 = __fadd2_rn(l2, pp);
                        ph[c] = __float_as_uint(pp.x);
                        ph[c + 1] = __float_as_uint(pp.y);
                        const float2 lo2 = __ffma2_rn(make_float2(__uint_as_float(ph[c] & 0xFFFFE000u), __uint_as_float(ph[c + 1] & 0xFFFFE000u)),
                                                      make_float2(-1.0f, -1.0f), pp);
                        pl[c] = __float_as_uint(lo2.x);
                        pl[c + 1] = __float_as_uint(lo2.y);
                    }
                } else { // columns past the row group's range: the MMA still reads them
#pragma unroll
                    for (int c = 0; c < 16; ++c) ph[c] = pl[c] = 0u;
                }
                tmem_st16(trow + kU5ColPhi + qt * 32 + pc * 16, ph);
                tmem_st16(trow + kU5ColPlo + qt * 32 + pc * 16, pl);
            }
            float l = l2.x + l2.y;
            xsum[qt][row] = l;
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars.p_ready);
            if (tid == 96) U5_ACC(1, 3);
            // ---- (3) the next unit's geometry and Q / K planes, while this unit's P V runs ----
            w = fetch_and_convert(k + 1);
            if (tid == 96) U5_ACC(1, 4);
            // ---- (4) output: (main + small) / row sum, this thread's 16 columns ----
            if (!mbar_wait_abort(&bars.o_done, k & 1, abortp)) {
                give_up(0x42);
                break;
            }
            if (tid == 96) U5_ACC(1, 5);
            tc_fence_after();
            {
                float a[16], b[16];
                tmem_ld16(trow + kU5ColO + qt * 16, a);
                tmem_ld16(trow + kU5ColO + 64 + qt * 16, b);
                group_sync(); // the partners' sums are there; and their reads of this round's maxima are over
                if (tid == 96) U5_ACC(1, 7);
                l = (xsum[0][row] + xsum[1][row]) + (xsum[2][row] + xsum[3][row]);
                const float inv = l > 0.0f ? 1.0f / l : 0.0f; // rows without keys give zeros
                tc_wait_ld();
                if (tid == 96) U5_ACC(1, 8);
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    *reinterpret_cast<float4 *>(piece_at(qt, c)) =
                        make_float4((a[c * 4] + b[c * 4]) * inv, (a[c * 4 + 1] + b[c * 4 + 1]) * inv,
                                    (a[c * 4 + 2] + b[c * 4 + 2]) * inv, (a[c * 4 + 3] + b[c * 4 + 3]) * inv);
            }
            // the storer warp sends the tile out by TMA: the stores leave the workers' instruction streams
            fence_async_smem();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars.out_full);
            if (tid == 96) U5_ACC(1, 6);
            ++k;
        }
        // end of this CTA's units: wake the storer with the end marker in its slot
        // (once it has taken the last tile: two phases of out_full must not complete unseen)
        if (w.g.u < 0 && !*abortp && (k == 0 || mbar_wait_abort(&bars.out_free, (k - 1) & 1, abortp))) {
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars.out_full);
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
    if (d.max_k > kU5Rows || d.max_q < 1 || d.max_q > 64 * kU5Rows) {
        *why = "unit kernel: at most 128 keys per sequence (and 8192 query rows)";
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
    if ((int64_t)d.batch * d.num_heads * ((d.max_q + kU5Rows - 1) / kU5Rows) > 0x7fffffff) {
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

// Map of the head columns of a [rows, row stride] fp32 tensor for 128-row x 32-column boxes with one of
// the 128-byte swizzles (16-byte chunks for K-major operands, 32-byte chunks for the MN-major one);
// rows past `rows` read as zeros and are never touched in memory.
static int u5_make_map(CUtensorMap *map, const float *base, int64_t stride, int64_t rows, int64_t cols, CUtensorMapSwizzle swz,
                       int box_rows = kU5Rows) {
    U5EncodeTiledFn enc = u5_encoder();
    if (!enc) return fail(FBLT_ERR_CUDA, "attn: cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)stride * sizeof(float)};
    const cuuint32_t box[2] = {32, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void *)base, dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
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
    // The eleven tensor maps depend on the tensors only; a host loop that launches over the same buffers
    // again (a decode loop, a benchmark) reuses the last set of its thread.
    struct MapSet {
        const float *q, *k, *v;
        float *out;
        int64_t qs, ks, vs, os, cols;
        int32_t tq, tk;
        CUtensorMap qm, km, vm;
        U5OutMaps om;
        bool valid;
    };
    static thread_local MapSet ms = {};
    if (!(ms.valid && ms.q == d.q && ms.k == d.k && ms.v == d.v && ms.out == d.out && ms.qs == d.q_stride &&
          ms.ks == d.k_stride && ms.vs == d.v_stride && ms.os == d.out_stride && ms.cols == cols &&
          ms.tq == d.total_q_rows && ms.tk == d.total_k_rows)) {
        ms.valid = false;
        int st = u5_make_map(&ms.qm, d.q, d.q_stride, d.total_q_rows, cols, CU_TENSOR_MAP_SWIZZLE_128B);
        if (st == FBLT_OK) st = u5_make_map(&ms.km, d.k, d.k_stride, d.total_k_rows, cols, CU_TENSOR_MAP_SWIZZLE_128B);
        if (st == FBLT_OK) st = u5_make_map(&ms.vm, d.v, d.v_stride, d.total_k_rows, cols, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
        for (int b = 0; b < 8 && st == FBLT_OK; ++b)
            st = u5_make_map(&ms.om.m[b], d.out, d.out_stride, d.total_q_rows, cols, CU_TENSOR_MAP_SWIZZLE_128B, kU5Rows >> b);
        if (st != FBLT_OK) return st;
        ms.q = d.q, ms.k = d.k, ms.v = d.v, ms.out = d.out;
        ms.qs = d.q_stride, ms.ks = d.k_stride, ms.vs = d.v_stride, ms.os = d.out_stride, ms.cols = cols;
        ms.tq = d.total_q_rows, ms.tk = d.total_k_rows;
        ms.valid = true;
    }
    const int qtiles = (d.max_q + kU5Rows - 1) / kU5Rows; // query tiles per sequence; all of them read the sequence's keys
    const int units = d.batch * d.num_heads * qtiles;
    const int sms = sm_count[dev & 63].load(std::memory_order_relaxed);
    const int grid = units < sms ? units : sms;
    unit5_attn_kernel<<<grid, kU5Threads, kU5Smem, stream>>>(d, ms.qm, ms.km, ms.vm, ms.om, units, qtiles);
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
extern "C" int fblt_u5_debug_knob(int i, int v) {
    cudaMemcpyToSymbol(fblt::g_u5_knob, &v, sizeof(int), sizeof(int) * i);
    return 0;
}
namespace fblt {
#endif
} // namespace fblt
