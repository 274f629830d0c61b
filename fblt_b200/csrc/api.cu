// L1 dispatch (fblt_attn_forward), the mask inspection entry points and the
// host-side patch boundary helpers.
#include "common.cuh"

#include <atomic>
#include <stdlib.h>
#include <string.h>

namespace fblt {

int launch_row_kernel(const fblt_attn_desc &d, cudaStream_t stream);
int launch_rowq_kernel(const fblt_attn_desc &d, cudaStream_t stream);
bool rowq_kernel_supports(const fblt_attn_desc &d, const char **why);
int launch_tile_kernel(const fblt_attn_desc &d, cudaStream_t stream);
bool tile_kernel_supports(const fblt_attn_desc &d, const char **why);
int launch_tile5_kernel(const fblt_attn_desc &d, cudaStream_t stream);
bool tile5_kernel_supports(const fblt_attn_desc &d, const char **why);
int launch_unit5_kernel(const fblt_attn_desc &d, cudaStream_t stream);
bool unit5_kernel_supports(const fblt_attn_desc &d, const char **why);

static int validate_desc(const fblt_attn_desc *d) {
    if (!d) return fail(FBLT_ERR_ARG, "attn: NULL descriptor");
    if (d->batch < 0 || d->num_heads <= 0 || d->head_dim <= 0) return fail(FBLT_ERR_ARG, "attn: bad batch/heads/head_dim");
    if (d->batch == 0) return FBLT_OK;
    if (!d->cu_q || !d->cu_k) return fail(FBLT_ERR_ARG, "attn: cu_q / cu_k required");
    if (!d->q || !d->k || !d->v || !d->out) return fail(FBLT_ERR_ARG, "attn: NULL tensor");
    const int64_t E = (int64_t)d->num_heads * d->head_dim;
    if (d->q_stride < E || d->k_stride < E || d->v_stride < E || d->out_stride < E)
        return fail(FBLT_ERR_ARG, "attn: row stride smaller than num_heads*head_dim");
    const fblt_mask_desc &m = d->mask;
    if (m.sliding_window < 0) return fail(FBLT_ERR_ARG, "attn: negative window");
    switch (m.group_rule) {
    case FBLT_GROUP_NONE: break;
    case FBLT_GROUP_PATCH_ENC:
    case FBLT_GROUP_PATCH_DEC:
    case FBLT_GROUP_PATCH_LEQ:
        if (!m.cu_patch || !m.patch_bounds) return fail(FBLT_ERR_ARG, "attn: patch rule needs cu_patch / patch_bounds");
        if (m.subtokens < 1) return fail(FBLT_ERR_ARG, "attn: subtokens must be >= 1");
        break;
    case FBLT_GROUP_IDS:
        if (!m.q_group_ids || !m.k_group_ids) return fail(FBLT_ERR_ARG, "attn: GROUP_IDS needs q_group_ids / k_group_ids");
        break;
    default: return fail(FBLT_ERR_ARG, "attn: unknown group rule %d", m.group_rule);
    }
    if ((m.cu_doc == nullptr) != (m.doc_bounds == nullptr)) return fail(FBLT_ERR_ARG, "attn: cu_doc and doc_bounds go together");
    if ((d->rope_cos == nullptr) != (d->rope_sin == nullptr)) return fail(FBLT_ERR_ARG, "attn: rope_cos and rope_sin go together");
    if (!d->rope_cos && (d->rope_q_pos || d->rope_k_pos)) return fail(FBLT_ERR_ARG, "attn: rotary positions without rotary tables");
    if (d->rope_cos && (d->head_dim & 1)) return fail(FBLT_ERR_ARG, "attn: rotary embedding needs an even head_dim");
    if (((uintptr_t)d->rope_cos | (uintptr_t)d->rope_sin) & 7) return fail(FBLT_ERR_ARG, "attn: rotary tables must be 8-byte aligned");
    return FBLT_OK;
}

// ---- mask inspection ---------------------------------------------------------

__global__ void mask_bitmap_kernel(fblt_attn_desc d, uint8_t *bitmap, int use_range) {
    const int b = blockIdx.y;
    const int q0 = d.cu_q[b], nq = d.cu_q[b + 1] - q0;
    const int k0 = d.cu_k[b], nk = d.cu_k[b + 1] - k0;
    const int64_t cell = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t cells = (int64_t)d.max_q * d.max_k;
    if (cell >= cells) return;
    const int i = (int)(cell / d.max_k), j = (int)(cell % d.max_k);
    uint8_t bit = 0;
    if (i < nq && j < nk) {
        const SeqMask s = resolve_mask(d.mask, b, q0, k0, nq, nk);
        if (use_range) {
            int lo, hi;
            row_range(s, i, lo, hi);
            bit = (j >= lo && j < hi) ? 1 : 0;
        } else {
            bit = pair_allowed(s, i, j) ? 1 : 0;
        }
    }
    bitmap[(int64_t)b * cells + cell] = bit;
}

// Counters for rows without an allowed key: one word per call in flight, handed out round-robin, so
// that concurrent fblt_mask_materialize calls (other streams, other host threads) do not share one.
constexpr int kEmptyRowSlots = 64;
__device__ int g_empty_rows[kEmptyRowSlots];

__global__ void mask_materialize_kernel(fblt_attn_desc d, int b, float *out, int slot) {
    const int q0 = d.cu_q[b], nq = d.cu_q[b + 1] - q0;
    const int k0 = d.cu_k[b], nk = d.cu_k[b + 1] - k0;
    const int i = blockIdx.x;
    if (i >= nq) return;
    const SeqMask s = resolve_mask(d.mask, b, q0, k0, nq, nk);
    int any = 0;
    for (int j = threadIdx.x; j < nk; j += blockDim.x) {
        const bool ok = pair_allowed(s, i, j);
        out[(int64_t)i * nk + j] = ok ? 0.0f : -INFINITY;
        any |= ok ? 1 : 0;
    }
    any = __syncthreads_or(any);
    if (threadIdx.x == 0 && !any) atomicAdd(&g_empty_rows[slot], 1);
}

} // namespace fblt

// Environment toggles for callers that pass FBLT_IMPL_AUTO / FBLT_PREC_FP32 (the defaults), in the
// manner of the reference's BLT_FLASH_ATTN switch (models/attention.c:111-119):
//   FBLT_ATTN_IMPL      = auto | row | quad | tile | tcgen05
//   FBLT_ATTN_PRECISION = fp32 | tf32
// Read at every call, so a host program may change them between calls. Unknown values are an error.
static int env_overrides(fblt_attn_desc &d) {
    if (d.impl == FBLT_IMPL_AUTO) {
        if (const char *e = getenv("FBLT_ATTN_IMPL")) {
            if (!strcmp(e, "row")) d.impl = FBLT_IMPL_ROW;
            else if (!strcmp(e, "quad")) d.impl = FBLT_IMPL_ROW_QUAD;
            else if (!strcmp(e, "tile")) d.impl = FBLT_IMPL_TILE;
            else if (!strcmp(e, "tcgen05")) d.impl = FBLT_IMPL_TCGEN05;
            else if (!strcmp(e, "unit")) d.impl = FBLT_IMPL_UNIT;
            else if (strcmp(e, "auto") && *e) return fblt::fail(FBLT_ERR_ARG, "FBLT_ATTN_IMPL=%s (auto, row, quad, tile, tcgen05, unit)", e);
        }
    }
    if (d.precision == FBLT_PREC_FP32) {
        if (const char *e = getenv("FBLT_ATTN_PRECISION")) {
            if (!strcmp(e, "tf32")) d.precision = FBLT_PREC_TF32;
            else if (strcmp(e, "fp32") && *e) return fblt::fail(FBLT_ERR_ARG, "FBLT_ATTN_PRECISION=%s (fp32, tf32)", e);
        }
    }
    return FBLT_OK;
}

extern "C" int fblt_attn_forward(const fblt_attn_desc *desc, void *stream) {
    fblt::NvtxRange nvtx_range("fblt_attn_forward");
    using namespace fblt;
    int st = validate_desc(desc);
    if (st != FBLT_OK) return st;
    if (desc->batch == 0 || desc->max_q <= 0) return FBLT_OK;
    fblt_attn_desc local = *desc;
    st = env_overrides(local);
    if (st != FBLT_OK) return st;
    const fblt_attn_desc *d = &local;
    cudaStream_t s = (cudaStream_t)stream;
    const char *why = "";
    switch (d->impl) {
    case FBLT_IMPL_ROW: return launch_row_kernel(*d, s);
    case FBLT_IMPL_TILE:
        if (!tile_kernel_supports(*d, &why)) return fail(FBLT_ERR_UNSUPPORTED, "tile kernel: %s", why);
        return launch_tile_kernel(*d, s);
    case FBLT_IMPL_TCGEN05:
        if (!tile5_kernel_supports(*d, &why)) return fail(FBLT_ERR_UNSUPPORTED, "%s", why);
        return launch_tile5_kernel(*d, s);
    case FBLT_IMPL_ROW_QUAD:
        if (!rowq_kernel_supports(*d, &why)) return fail(FBLT_ERR_UNSUPPORTED, "%s", why);
        return launch_rowq_kernel(*d, s);
    case FBLT_IMPL_UNIT:
        if (!unit5_kernel_supports(*d, &why)) return fail(FBLT_ERR_UNSUPPORTED, "%s", why);
        return launch_unit5_kernel(*d, s);
    case FBLT_IMPL_AUTO:
        // short per-row key ranges (a patch's own bytes, one latent) stay on the row kernel
        if ((d->mask.group_rule == FBLT_GROUP_NONE || d->mask.group_rule == FBLT_GROUP_PATCH_LEQ) && d->max_k >= 32) {
            // sequences of up to 128 keys: one tcgen05 tile per (sequence, head, 128 query rows), persistent
            if (d->max_q >= 32 && unit5_kernel_supports(*d, &why)) return launch_unit5_kernel(*d, s);
            // 128-row tcgen05 tiles once sequences fill most of a tile; 64-row mma.sync tiles otherwise
            if (d->max_q >= 96 && tile5_kernel_supports(*d, &why)) return launch_tile5_kernel(*d, s);
            if (tile_kernel_supports(*d, &why)) return launch_tile_kernel(*d, s);
        }
        // what is left has short key ranges per row (or needs the general kernel): four lanes per row
        // where the shape allows, a warp per row otherwise
        if (d->max_k <= 4096 && rowq_kernel_supports(*d, &why)) return launch_rowq_kernel(*d, s);
        return launch_row_kernel(*d, s);
    default: return fail(FBLT_ERR_ARG, "attn: unknown impl %d", d->impl);
    }
}

extern "C" int fblt_mask_bitmap(const fblt_attn_desc *d, uint8_t *bitmap, int use_range, void *stream) {
    using namespace fblt;
    int st = validate_desc(d);
    if (st != FBLT_OK) return st;
    if (!bitmap) return fail(FBLT_ERR_ARG, "mask_bitmap: NULL bitmap");
    if (use_range && d->mask.group_rule == FBLT_GROUP_IDS)
        return fail(FBLT_ERR_UNSUPPORTED, "mask_bitmap: explicit group ids have no key range");
    if (d->batch == 0 || d->max_q <= 0 || d->max_k <= 0) return FBLT_OK;
    const int64_t cells = (int64_t)d->max_q * d->max_k;
    dim3 grid((unsigned)((cells + 255) / 256), d->batch);
    mask_bitmap_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(*d, bitmap, use_range);
    count_launch();
    return check_launch("mask_bitmap_kernel");
}

extern "C" int fblt_mask_materialize(const fblt_attn_desc *d, int32_t seq, float *mask_out, int32_t *empty_rows_out,
                                     void *stream) {
    using namespace fblt;
    int st = validate_desc(d);
    if (st != FBLT_OK) return st;
    if (!mask_out || seq < 0 || seq >= d->batch) return fail(FBLT_ERR_ARG, "mask_materialize: bad arguments");
    if (d->max_q <= 0) return FBLT_OK;
    cudaStream_t s = (cudaStream_t)stream;
    static std::atomic<unsigned> next_slot{0};
    const int slot = (int)(next_slot.fetch_add(1, std::memory_order_relaxed) % kEmptyRowSlots);
    const int zero = 0;
    FBLT_CUDA_TRY(cudaMemcpyToSymbolAsync(g_empty_rows, &zero, sizeof(int), slot * sizeof(int), cudaMemcpyHostToDevice, s));
    mask_materialize_kernel<<<d->max_q, 128, 0, s>>>(*d, seq, mask_out, slot);
    count_launch();
    st = check_launch("mask_materialize_kernel");
    if (st != FBLT_OK) return st;
    if (empty_rows_out) {
        int v = 0;
        FBLT_CUDA_TRY(cudaMemcpyFromSymbolAsync(&v, g_empty_rows, sizeof(int), slot * sizeof(int), cudaMemcpyDeviceToHost, s));
        FBLT_CUDA_TRY(cudaStreamSynchronize(s));
        *empty_rows_out = v;
    }
    return FBLT_OK;
}

// ---- host helpers --------------------------------------------------------------

extern "C" int fblt_patch_bounds(const fblt_patch_info *patches, size_t num_patches, size_t seq_len, int32_t *bounds_out) {
    using namespace fblt;
    if ((!patches && num_patches) || !bounds_out) return fail(FBLT_ERR_ARG, "patch_bounds: NULL argument");
    size_t pos = 0;
    for (size_t p = 0; p < num_patches; ++p) {
        if (patches[p].start_idx != pos) return fail(FBLT_ERR_ARG, "patch_bounds: patches must tile [0, seq_len) contiguously");
        if (patches[p].length < 1) return fail(FBLT_ERR_ARG, "patch_bounds: empty patch");
        bounds_out[p] = (int32_t)pos;
        pos += patches[p].length;
    }
    if (pos != seq_len) return fail(FBLT_ERR_ARG, "patch_bounds: patches do not cover [0, seq_len) exactly");
    bounds_out[num_patches] = (int32_t)pos;
    return FBLT_OK;
}

extern "C" int32_t fblt_patch_latent_at(const int32_t *bounds, int32_t num_patches, int32_t pos) {
    if (pos < bounds[0]) return 0;
    if (pos >= bounds[num_patches]) return num_patches - 1;
    int32_t lo = 0, hi = num_patches; // patch p with bounds[p] <= pos < bounds[p+1]
    while (hi - lo > 1) {
        const int32_t mid = (lo + hi) / 2;
        if (bounds[mid] <= pos) lo = mid;
        else hi = mid;
    }
    const bool closes = (pos + 1 == bounds[lo + 1]) && (lo + 1 < num_patches);
    if (closes) return lo;
    return lo == 0 ? 0 : lo - 1;
}

// sizeof of every ABI struct, for bindings that re-declare them (ctypes, cgo).
extern "C" size_t fblt_abi_sizes(size_t *out, size_t cap) {
    const size_t v[] = {sizeof(fblt_head_args), sizeof(fblt_patch_info), sizeof(fblt_mask_desc), sizeof(fblt_attn_desc),
                        sizeof(fblt_decode_desc), sizeof(fblt_mha_desc), sizeof(fblt_cross_desc),
                        sizeof(fblt_kv_step_desc)};
    const size_t n = sizeof(v) / sizeof(v[0]);
    for (size_t i = 0; i < n && i < cap; ++i) out[i] = v[i];
    return n;
}
