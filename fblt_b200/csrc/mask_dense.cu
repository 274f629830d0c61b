// Dense-mask hand-back for callers that still want the tensor: the two mask builders of the
// reference's CUDA backend (blt_build_attention_mask_cuda, blt_build_block_diffusion_mask_cuda;
// ops/mask_builder.cu:100-216, declared for the dispatcher at core/backend.c:190-192) behind
// config structs with the reference's layout. The batched attention kernels never read such a
// tensor; these entry points exist so that an unmodified host keeps linking and its callers that
// download the mask (tests/parity/parity_cuda_composites.c:97-105) keep working.
//
// The attention rule is evaluated by the same pair predicate the batched kernels are checked
// against (common.cuh: pair_allowed); the block-diffusion rule has its own kernel because its
// TRAIN form (ops/mask_builder_cpu.c:136-147) is used by training only.
#include "common.cuh"

#include <stdlib.h>
#include <vector>

namespace fblt {

__global__ void dense_mask_kernel(SeqMask s, float *out, int *empty_rows) {
    const int i = blockIdx.x;
    if (i >= s.nq) return;
    int any = 0;
    for (int j = threadIdx.x; j < s.nk; j += blockDim.x) {
        const bool ok = pair_allowed(s, i, j);
        out[(int64_t)i * s.nk + j] = ok ? 0.0f : -INFINITY;
        any |= ok ? 1 : 0;
    }
    any = __syncthreads_or(any);
    if (threadIdx.x == 0 && !any) atomicAdd(empty_rows, 1);
}

// Rows i < N: causal over the clean prefix. Rows past it: everything (INFER), or the clean
// columns before the block's start plus the row's own block (TRAIN).
__global__ void block_diffusion_mask_kernel(float *out, int S, int N, int B, int infer, const int32_t *starts,
                                            int *empty_rows) {
    const int i = blockIdx.x;
    if (i >= S) return;
    int any = 0;
    const int blk = (i >= N && !infer) ? (i - N) / B : 0;
    const int s_blk = (i >= N && !infer) ? starts[blk] : 0;
    for (int j = threadIdx.x; j < S; j += blockDim.x) {
        bool ok;
        if (i < N) ok = j < N && j <= i;
        else if (infer) ok = true;
        else ok = j < s_blk || (j >= N && (j - N) / B == blk);
        out[(int64_t)i * S + j] = ok ? 0.0f : -INFINITY;
        any |= ok ? 1 : 0;
    }
    any = __syncthreads_or(any);
    if (threadIdx.x == 0 && !any) atomicAdd(empty_rows, 1);
}

static size_t align16(size_t n) { return (n + 15) & ~(size_t)15; }

// Scratch layout: [counter, 16 bytes][doc bounds][query ids][key ids] / [counter][block starts], int32.
static int finish(int *counter, int32_t *empty_rows_out, cudaStream_t s) {
    if (empty_rows_out) {
        int v = 0;
        FBLT_CUDA_TRY(cudaMemcpyAsync(&v, counter, sizeof(int), cudaMemcpyDeviceToHost, s));
        FBLT_CUDA_TRY(cudaStreamSynchronize(s));
        *empty_rows_out = v;
    }
    return FBLT_OK;
}

static bool narrow(const size_t *src, size_t n, std::vector<int32_t> &dst) {
    for (size_t i = 0; i < n; ++i) {
        if (src[i] > 0x7fffffffu) return false;
        dst.push_back((int32_t)src[i]);
    }
    return true;
}

} // namespace fblt

extern "C" size_t fblt_mask_dense_scratch_bytes(const fblt_mask_config *c) {
    using namespace fblt;
    if (!c) return 0;
    size_t n = 16;
    if (c->doc_boundaries && c->num_docs > 1) n += align16((c->num_docs - 1) * sizeof(int32_t));
    if (c->query_group_ids && c->kv_group_ids) n += align16(c->seq_len_q * sizeof(int32_t)) + align16(c->seq_len_kv * sizeof(int32_t));
    return n;
}

extern "C" int fblt_build_attention_mask_dense(const fblt_mask_config *c, float *mask_out, void *scratch,
                                               size_t scratch_bytes, int32_t *empty_rows_out, void *stream) {
    using namespace fblt;
    NvtxRange nvtx_range("fblt_build_attention_mask_dense");
    if (!c || !mask_out) return fail(FBLT_ERR_ARG, "mask_dense: NULL argument");
    if (c->seq_len_q > 0x7fffffffu || c->seq_len_kv > 0x7fffffffu || c->sliding_window > 0x7fffffffu ||
        c->causal_offset > 0x3fffffffu)
        return fail(FBLT_ERR_LIMIT, "mask_dense: sizes beyond int32");
    if (!scratch || scratch_bytes < fblt_mask_dense_scratch_bytes(c))
        return fail(FBLT_ERR_WORKSPACE, "mask_dense: scratch of %zu bytes needed", fblt_mask_dense_scratch_bytes(c));
    if ((uintptr_t)scratch & 15) return fail(FBLT_ERR_ARG, "mask_dense: scratch must be 16-byte aligned");
    if (empty_rows_out) *empty_rows_out = 0;
    if (c->seq_len_q == 0 || c->seq_len_kv == 0) return FBLT_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const bool has_docs = c->doc_boundaries && c->num_docs > 1;
    const bool has_groups = c->query_group_ids && c->kv_group_ids;

    // host ids are size_t (ops/mask_builder.h:19-24); the device rule reads int32
    std::vector<int32_t> host;
    const size_t nd = has_docs ? c->num_docs - 1 : 0;
    bool ok = true;
    if (has_docs) ok = ok && narrow(c->doc_boundaries, nd, host);
    while (host.size() % 4) host.push_back(0);
    const size_t q_at = host.size();
    if (has_groups) ok = ok && narrow(c->query_group_ids, c->seq_len_q, host);
    while (host.size() % 4) host.push_back(0);
    const size_t k_at = host.size();
    if (has_groups) ok = ok && narrow(c->kv_group_ids, c->seq_len_kv, host);
    if (!ok) return fail(FBLT_ERR_LIMIT, "mask_dense: an id or boundary exceeds int32");
    for (size_t d = 1; d < nd; ++d)
        if (c->doc_boundaries[d] < c->doc_boundaries[d - 1]) return fail(FBLT_ERR_ARG, "mask_dense: doc_boundaries must ascend");

    int *counter = (int *)scratch;
    int32_t *ids = (int32_t *)((char *)scratch + 16);
    FBLT_CUDA_TRY(cudaMemsetAsync(counter, 0, 16, s));
    // pageable source: the runtime has staged the bytes by the time the call returns
    if (!host.empty()) FBLT_CUDA_TRY(cudaMemcpyAsync(ids, host.data(), host.size() * sizeof(int32_t), cudaMemcpyHostToDevice, s));

    SeqMask m;
    m.nq = (int)c->seq_len_q;
    m.nk = (int)c->seq_len_kv;
    m.is_causal = c->is_causal ? 1 : 0;
    m.window = (int)c->sliding_window;
    m.group_rule = has_groups ? FBLT_GROUP_IDS : FBLT_GROUP_NONE;
    m.subtokens = 1;
    m.bidir = c->bidirectional_within_group ? 1 : 0;
    m.causal_off = c->is_causal ? (int)c->causal_offset : 0;
    m.num_clean = -1;
    m.doc = has_docs ? ids : nullptr;
    m.ndoc = (int)nd;
    m.pb = nullptr;
    m.P = 0;
    m.q_pos_off = 0;
    m.trailing_closed = 0;
    m.qg = has_groups ? ids + q_at : nullptr;
    m.kg = has_groups ? ids + k_at : nullptr;
    dense_mask_kernel<<<(unsigned)m.nq, 128, 0, s>>>(m, mask_out, counter);
    count_launch();
    const int st = check_launch("dense_mask_kernel");
    if (st != FBLT_OK) return st;
    return finish(counter, empty_rows_out, s);
}

extern "C" size_t fblt_block_diffusion_mask_scratch_bytes(const fblt_block_diffusion_config *c) {
    if (!c) return 0;
    return 16 + (c->mode == FBLT_BDM_TRAIN ? fblt::align16(c->num_blocks * sizeof(int32_t)) : 0);
}

extern "C" int fblt_build_block_diffusion_mask_dense(const fblt_block_diffusion_config *c, float *mask_out,
                                                     void *scratch, size_t scratch_bytes, int32_t *empty_rows_out,
                                                     void *stream) {
    using namespace fblt;
    NvtxRange nvtx_range("fblt_build_block_diffusion_mask_dense");
    if (!c || !mask_out) return fail(FBLT_ERR_ARG, "block_mask_dense: NULL argument");
    const size_t S = c->seq_len, N = c->num_clean;
    // the preconditions of ops/mask_builder_cpu.c:103-117
    if (S < 1 || N < 1 || N > S) return fail(FBLT_ERR_ARG, "block_mask_dense: need 1 <= num_clean <= seq_len");
    if (S > 0x7fffffffu) return fail(FBLT_ERR_LIMIT, "block_mask_dense: seq_len beyond int32");
    const bool train = c->mode == FBLT_BDM_TRAIN;
    if (!train && c->mode != FBLT_BDM_INFER) return fail(FBLT_ERR_ARG, "block_mask_dense: unknown mode %d", (int)c->mode);
    std::vector<int32_t> host;
    if (train) {
        if (c->block_size < 1) return fail(FBLT_ERR_ARG, "block_mask_dense: TRAIN needs block_size >= 1");
        if ((S - N) % c->block_size) return fail(FBLT_ERR_ARG, "block_mask_dense: block section must tile exactly");
        if (!c->block_starts && S > N) return fail(FBLT_ERR_ARG, "block_mask_dense: TRAIN needs block_starts");
        if (c->num_blocks != (S - N) / c->block_size) return fail(FBLT_ERR_ARG, "block_mask_dense: num_blocks must equal (S - N) / block_size");
        for (size_t b = 0; b < c->num_blocks; ++b) {
            if (c->block_starts[b] >= N) return fail(FBLT_ERR_ARG, "block_mask_dense: block start outside the clean prefix");
            host.push_back((int32_t)c->block_starts[b]);
        }
    }
    if (!scratch || scratch_bytes < fblt_block_diffusion_mask_scratch_bytes(c))
        return fail(FBLT_ERR_WORKSPACE, "block_mask_dense: scratch of %zu bytes needed", fblt_block_diffusion_mask_scratch_bytes(c));
    if ((uintptr_t)scratch & 15) return fail(FBLT_ERR_ARG, "block_mask_dense: scratch must be 16-byte aligned");
    cudaStream_t s = (cudaStream_t)stream;
    int *counter = (int *)scratch;
    int32_t *starts = (int32_t *)((char *)scratch + 16);
    FBLT_CUDA_TRY(cudaMemsetAsync(counter, 0, 16, s));
    if (!host.empty()) FBLT_CUDA_TRY(cudaMemcpyAsync(starts, host.data(), host.size() * sizeof(int32_t), cudaMemcpyHostToDevice, s));
    block_diffusion_mask_kernel<<<(unsigned)S, 128, 0, s>>>(mask_out, (int)S, (int)N, train ? (int)c->block_size : 1,
                                                             train ? 0 : 1, starts, counter);
    count_launch();
    const int st = check_launch("block_diffusion_mask_kernel");
    if (st != FBLT_OK) return st;
    if (empty_rows_out) *empty_rows_out = 0;
    return finish(counter, empty_rows_out, s);
}
