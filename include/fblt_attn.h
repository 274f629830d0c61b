/*
 * fblt_attn.h -- C ABI of the B200 (sm_100a) attention path for fBLT.
 *
 * Two levels:
 *
 *   L0  strict drop-in for the reference backend symbols that core/backend.c
 *       links against (core/backend.c:66-67, 484-487): one sequence, one head,
 *       dense additive mask, reference struct layout, reference error
 *       convention (print + exit(1)).
 *
 *   L1  batched entry points (all sequences and all heads per launch, varlen,
 *       mask given as a descriptor derived from the patcher's boundary array,
 *       never a dense matrix). These return an int status and never exit.
 *
 * All tensors are fp32. Pointers named "device" must be CUDA device pointers
 * of the current device; everything else is host memory. No entry point
 * requires the caller to synchronise; work is ordered on the stream passed in
 * (NULL = the legacy default stream, which is what the reference uses,
 * ops/memory.cu:54-77).
 *
 * There is no CPU fallback anywhere in this library.
 */
#ifndef FBLT_ATTN_H
#define FBLT_ATTN_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------ */
/* status                                                                    */
/* ------------------------------------------------------------------------ */

typedef enum {
    FBLT_OK = 0,
    FBLT_ERR_ARG = 1,         /* NULL pointer, bad stride, bad size          */
    FBLT_ERR_UNSUPPORTED = 2, /* shape the requested kernel cannot run       */
    FBLT_ERR_WORKSPACE = 3,   /* workspace missing or too small              */
    FBLT_ERR_CUDA = 4,        /* a CUDA runtime call failed                  */
    FBLT_ERR_CAPACITY = 5,    /* KV cache / session capacity exceeded        */
    FBLT_ERR_LIMIT = 6,       /* size beyond a documented fixed maximum      */
    FBLT_ERR_PEER = 7,        /* another rank announced a failure            */
    FBLT_ERR_TIMEOUT = 8      /* a host-side deadline passed                 */
} fblt_status;

/* Text of the last error raised on the calling thread ("" if none). */
const char *fblt_last_error(void);
const char *fblt_status_string(int status);
/* Library build identification: "fblt_attn sm_100a <n>". */
const char *fblt_version(void);

/* ------------------------------------------------------------------------ */
/* L0: single-head operator, reference layout                                */
/* ------------------------------------------------------------------------ */

/* Values of the reference's blt_backend enum (core/tensor.h:15). */
enum { FBLT_BACKEND_CPU = 0, FBLT_BACKEND_CUDA = 1 };

/*
 * Field-for-field layout of blt_attention_head_args (ops/attn_core.h:25-44);
 * a pointer to either type may be passed to the L0 symbols.
 *
 *   scores_ij = dot(q_i, k_j); w = softmax(scale*scores + mask); out = w @ v
 *   `mask` (additive, [nq*nk]) wins over is_causal; with mask == NULL and
 *   is_causal, keys j > i are masked. The row maximum is taken over finite
 *   entries only; non-finite entries get weight 0; a row with no finite entry
 *   produces zeros (ops/vecmath_cpu.c:16-53). Only head_dim columns at
 *   combined_col_offset are written (ops/attn_core_cpu.c:39-55).
 */
typedef struct {
    const float *q;
    size_t q_stride;
    const float *k;
    size_t k_stride;
    const float *v;
    size_t v_stride;
    float *combined;
    size_t combined_stride;
    size_t combined_col_offset;
    float *weights_out;    /* optional [nq*nk]: post-softmax weights          */
    float *lse_out;        /* optional [nq*2]: (row max m, row sum l)          */
    float *scores_scratch; /* optional; unused here (no global score buffer)   */
    const float *mask;     /* optional [nq*nk] additive mask                   */
    size_t nq;
    size_t nk;
    size_t head_dim;
    bool is_causal;
    float scale;
} fblt_head_args;

/*
 * Replaces blt_attention_head_core_cuda (ops/attn_core.cu:288-312; declared
 * for the dispatcher at core/backend.c:66). Same preconditions and the same
 * failure mode: a violated requirement prints "BLT Fatal Error ..." to stderr
 * and exits (core/backend.h:13-31). Launches on the default stream.
 */
void blt_attention_head_core_cuda(int backend, const fblt_head_args *args);

/*
 * Link stub for blt_attention_head_core_backward_cuda (ops/attn_core.cu:505,
 * core/backend.c:67). Training is outside this library: calling it is fatal,
 * which is the reference's own convention for an unavailable backend op
 * (core/backend.c:102).
 */
void blt_attention_head_core_backward_cuda(int backend, const void *bwd_args);

/* Status-returning form of the same operator on an explicit stream. */
int fblt_attention_head(const fblt_head_args *args, void *stream);

/* ------------------------------------------------------------------------ */
/* patch boundary helpers (host, integer logic)                              */
/* ------------------------------------------------------------------------ */

/* Layout of blt_patch_info (models/patcher.h:16-20). */
typedef struct {
    size_t start_idx;
    size_t length;
    float peak_entropy;
} fblt_patch_info;

/*
 * Boundary array of one sequence: bounds[p] = first byte of patch p,
 * bounds[num_patches] = one past the last byte. Requires the patches to tile
 * [0, seq_len) contiguously with no empty patch, like
 * blt_patch_build_group_ids (ops/patch_pool_cpu.c:98-112). Returns FBLT_OK or
 * FBLT_ERR_ARG.
 */
int fblt_patch_bounds(const fblt_patch_info *patches, size_t num_patches, size_t seq_len, int32_t *bounds_out);

/*
 * Decoder latent index of byte `pos` (Fast-BLT 3.1.1), as
 * blt_patch_decoder_latent_at (ops/patch_pool_cpu.c:114-131) computes it, from
 * a boundary array: final byte of a non-last patch j -> j; any other byte of
 * patch j -> max(j-1, 0); pos before bounds[0] -> 0; pos at or past the end ->
 * num_patches-1.
 */
int32_t fblt_patch_latent_at(const int32_t *bounds, int32_t num_patches, int32_t pos);

/* ------------------------------------------------------------------------ */
/* L1: mask descriptor                                                       */
/* ------------------------------------------------------------------------ */

typedef enum {
    FBLT_GROUP_NONE = 0,
    /* Encoder cross-attention (models/local_encoder.c:70-74): query row i is
     * sub-token i of patch i / subtokens; key row j is byte j; allowed iff
     * byte j lies in that patch. */
    FBLT_GROUP_PATCH_ENC = 1,
    /* Decoder cross-attention, reference rule (models/local_decoder.c:82-94,
     * infer/kv_cache.c:206-218): query row i is byte q_pos_offset + i; key row
     * j is sub-token j; allowed iff j / subtokens == latent_at(byte); with
     * trailing_closed the last query row of the sequence reads latent P-1. */
    FBLT_GROUP_PATCH_DEC = 2,
    /* Decoder cross-attention, "patches <= its patch" rule: allowed iff
     * j / subtokens <= patch containing the byte (bytes past the end -> P-1). */
    FBLT_GROUP_PATCH_LEQ = 3,
    /* Explicit ids per packed row: q_group_ids[i] == k_group_ids[j]
     * (ops/mask_builder_cpu.c:82-88). Runs on the per-row kernel only. */
    FBLT_GROUP_IDS = 4
} fblt_group_rule;

/*
 * Batched counterpart of blt_mask_config (ops/mask_builder.h:12-32) plus the
 * INFER rule of blt_block_diffusion_config (ops/mask_builder.h:55-68).
 * Within one sequence, with i/j the row indices local to that sequence:
 *
 *   allowed(i,j) =  (!is_causal  || j <= i + causal_offset)
 *                && (window == 0 || dist < window)     dist = |i + causal_offset - j| if causal else |i - j|
 *                && (no docs     || doc(i) == doc(j))
 *                && group rule
 *                && (group rule == NONE || bidirectional_within_group || j <= i)
 *
 * and, when num_clean is given without a group rule (block-diffusion INFER
 * self-attention), the first two lines are replaced by:
 * i < N ? (j < N && j <= i) : true   (ops/mask_builder_cpu.c:127-135).
 * With FBLT_GROUP_PATCH_DEC, num_clean describes the cross-attention of the
 * same pass (models/block_diffusion.c:164-186): rows i < N use the decoder
 * latent rule (trailing_closed applies to row N - 1), rows i >= N are the
 * drafted block and read the last latent.
 *
 * All array members are device pointers to int32 (uint8 for trailing_closed);
 * NULL means "absent".
 */
typedef struct {
    int32_t is_causal;
    int32_t sliding_window;
    int32_t group_rule; /* fblt_group_rule */
    int32_t subtokens;  /* k >= 1 sub-tokens per patch (PATCH_* rules) */
    int32_t bidirectional_within_group;
    int32_t reserved;
    const int32_t *causal_offset;   /* [batch] */
    const int32_t *cu_doc;          /* [batch+1] offsets into doc_bounds */
    const int32_t *doc_bounds;      /* per sequence: first position of document d+1, ascending */
    const int32_t *cu_patch;        /* [batch+1] offsets into patch_bounds; sequence b owns P_b + 1 entries */
    const int32_t *patch_bounds;    /* per sequence: fblt_patch_bounds() output */
    const int32_t *q_pos_offset;    /* [batch] byte position of the first query row (PATCH_DEC / PATCH_LEQ) */
    const uint8_t *trailing_closed; /* [batch] (PATCH_DEC) */
    const int32_t *q_group_ids;     /* [total q rows] (GROUP_IDS) */
    const int32_t *k_group_ids;     /* [total k rows] (GROUP_IDS) */
    const int32_t *num_clean;       /* [batch] N: switches on the block-diffusion INFER rule */
} fblt_mask_desc;

/* ------------------------------------------------------------------------ */
/* L1: batched prefill / cross attention                                     */
/* ------------------------------------------------------------------------ */

typedef enum {
    FBLT_IMPL_AUTO = 0,   /* pick per shape */
    FBLT_IMPL_ROW = 1,    /* one warp per (query row, head), fp32 FMA; any head_dim up to 256, any mask */
    FBLT_IMPL_TILE = 2,   /* tensor-core tiles, mma.sync TF32 (head_dim 32/64/128, range masks) */
    FBLT_IMPL_TCGEN05 = 3, /* tensor-core tiles, tcgen05 + TMEM (head_dim 64, range masks) */
    FBLT_IMPL_ROW_QUAD = 4, /* four lanes per (query row, head), fp32 FMA; head_dim 32/64, range masks, no rotary tables */
    FBLT_IMPL_UNIT = 5     /* tcgen05 + TMA, one 128 x 128 tile per (sequence, head, 128 query rows): head_dim 64, at
                            * most 128 keys per sequence, range masks, total_q_rows / total_k_rows given */
} fblt_impl;

typedef enum {
    FBLT_PREC_FP32 = 0, /* fp32-equivalent: error-compensated 3xTF32 on tensor cores, plain fp32 on the row kernel */
    FBLT_PREC_TF32 = 1  /* single-pass TF32 tensor cores (tile kernel only) */
} fblt_precision;

/*
 * One call = every (sequence, head) of a batch. Sequence b owns query rows
 * [cu_q[b], cu_q[b+1]) of q/out and key rows [cu_k[b], cu_k[b+1]) of k/v (for
 * self-attention pass the same table twice). Head h lives at columns
 * [h*head_dim, (h+1)*head_dim) of every row, which covers the packed
 * [T, 3E] layout of models/attention.c:95-107 (q = base, k = base + E,
 * v = base + 2E, strides 3E) as well as the [rows, E] layout of
 * models/cross_attention.c:78-86.
 *
 * Replaces the per-head loops at models/attention.c:199-202,
 * models/cross_attention.c:147-150, models/block_diffusion.c:293-319.
 * A query row with no allowed key yields zeros.
 */
typedef struct {
    int32_t batch;
    int32_t num_heads;
    int32_t head_dim;
    int32_t max_q; /* host-known upper bound of rows per sequence (grid sizing) */
    int32_t max_k;
    int32_t impl;      /* fblt_impl */
    int32_t precision; /* fblt_precision */
    int32_t total_q_rows; /* host-known cu_q[batch] (rows of q / out), 0 = not given: needed by the kernels that
                           * load tiles by TMA (the unit kernel), which must know where the tensors end */
    const int32_t *cu_q; /* device [batch+1] */
    const int32_t *cu_k; /* device [batch+1] */
    const float *q;      /* device */
    int64_t q_stride;    /* elements per row */
    const float *k;
    int64_t k_stride;
    const float *v;
    int64_t v_stride;
    float *out;
    int64_t out_stride;
    float scale;
    int32_t total_k_rows; /* host-known cu_k[batch] (rows of k / v), 0 = not given */
    fblt_mask_desc mask;
    /* Optional fused rotary embedding for self-attention prefill (replaces the 2 x heads
     * blt_rope_apply_packed launches of models/attention.c:73-89): device tables
     * [positions, head_dim/2] as blt_rope_precompute fills them. When given, q and k hold the
     * un-rotated QKV projection; query row i is rotated with position i + causal_offset[b]
     * and key row j with position j (interleaved pairs, ops/reductions_cpu.c:217-228)
     * as they are loaded. NULL: q / k arrive rotated. head_dim must be even.
     * rope_q_pos / rope_k_pos (optional, device int32, one entry per packed q / k row)
     * replace those default positions: the gathered positions of the block-diffusion
     * pass (models/block_diffusion.c:153-162 -- identity for clean rows, the recorded
     * original position for block rows). Packed self-attention passes one array twice. */
    const float *rope_cos;
    const float *rope_sin;
    const int32_t *rope_q_pos;
    const int32_t *rope_k_pos;
} fblt_attn_desc;

/*
 * Environment toggles, read at every call, for descriptors that leave impl at FBLT_IMPL_AUTO /
 * precision at FBLT_PREC_FP32 (the reference switches kernels the same way, BLT_FLASH_ATTN in
 * models/attention.c:111-119): FBLT_ATTN_IMPL = auto | row | quad | tile | tcgen05,
 * FBLT_ATTN_PRECISION = fp32 | tf32. An unknown value is FBLT_ERR_ARG; a kernel that does not
 * take the shape is FBLT_ERR_UNSUPPORTED, as when it is named in the descriptor.
 */
int fblt_attn_forward(const fblt_attn_desc *desc, void *stream);

/*
 * Debug / parity: writes allowed(i,j) as bytes (1/0) for sequence-local
 * (i,j) into bitmap[b * max_q * max_k + i * max_k + j] (device). `use_range`
 * != 0 evaluates the [lo,hi) key range the tile and streaming kernels use
 * instead of the per-pair predicate; both must equal the reference's dense
 * mask (ops/mask_builder_cpu.c:49-94) wherever the rule is a range.
 * FBLT_ERR_UNSUPPORTED if use_range is asked for GROUP_IDS.
 */
int fblt_mask_bitmap(const fblt_attn_desc *desc, uint8_t *bitmap, int use_range, void *stream);

/*
 * Dense additive fp32 mask (0 / -inf) for one sequence of the descriptor,
 * [nq, nk] row-major into device memory: what a kept
 * blt_build_attention_mask_cuda / blt_build_block_diffusion_mask_cuda
 * (core/backend.c:190-192) would hand back to callers that still want a
 * tensor. *empty_rows_out (host, optional) receives the number of query rows
 * with no allowed key, the condition the reference treats as fatal
 * (ops/mask_builder_cpu.c:93).
 */
int fblt_mask_materialize(const fblt_attn_desc *desc, int32_t seq, float *mask_out, int32_t *empty_rows_out,
                          void *stream);

/*
 * The reference's two dense mask builders behind its own config structs, for a
 * host that keeps calling blt_build_attention_mask / blt_build_block_diffusion_mask
 * on the CUDA backend (dispatcher: core/backend.c:190-192; replaced:
 * ops/mask_builder.cu:100-216). Field-for-field layouts of blt_mask_config
 * (ops/mask_builder.h:12-32) and blt_block_diffusion_config
 * (ops/mask_builder.h:43-68); a pointer to either type may be passed. The id
 * arrays are HOST pointers, as in the reference (ops/mask_builder.cu:10-13).
 */
typedef struct {
    size_t seq_len_q;
    size_t seq_len_kv;
    size_t sliding_window;
    const size_t *doc_boundaries; /* num_docs - 1 entries, ascending */
    size_t num_docs;
    const size_t *query_group_ids;
    const size_t *kv_group_ids;
    bool bidirectional_within_group;
    bool is_causal;
    size_t causal_offset;
} fblt_mask_config;

typedef enum { FBLT_BDM_TRAIN = 0, FBLT_BDM_INFER = 1 } fblt_block_diffusion_mode;

typedef struct {
    fblt_block_diffusion_mode mode;
    size_t seq_len;
    size_t num_clean;
    size_t block_size;
    const size_t *block_starts; /* TRAIN only, num_blocks entries */
    size_t num_blocks;
} fblt_block_diffusion_config;

/*
 * mask_out: device [seq_len_q, seq_len_kv] (square [seq_len, seq_len] for the
 * block-diffusion form), 0 where attention is allowed and -inf elsewhere,
 * bit-equal to the reference's CPU builders (ops/mask_builder_cpu.c:21-154).
 * scratch: device memory of at least *_scratch_bytes(config), 16-byte aligned,
 * supplied by the caller (the reference takes its temporaries from the arena
 * it is handed, ops/mask_builder.cu:23-28); it may be reused once the stream
 * has passed the call. *empty_rows_out (host, optional; asking for it
 * synchronises the stream) = query rows with no allowed key, which the
 * reference treats as fatal (ops/mask_builder_cpu.c:93,152). Preconditions of
 * the reference that fail here return FBLT_ERR_ARG instead of exiting.
 * fblt_b200/csrc/blt_backend_glue.c wraps both into the reference's symbols.
 */
size_t fblt_mask_dense_scratch_bytes(const fblt_mask_config *config);
int fblt_build_attention_mask_dense(const fblt_mask_config *config, float *mask_out, void *scratch,
                                    size_t scratch_bytes, int32_t *empty_rows_out, void *stream);
size_t fblt_block_diffusion_mask_scratch_bytes(const fblt_block_diffusion_config *config);
int fblt_build_block_diffusion_mask_dense(const fblt_block_diffusion_config *config, float *mask_out, void *scratch,
                                          size_t scratch_bytes, int32_t *empty_rows_out, void *stream);

/* ------------------------------------------------------------------------ */
/* L1: KV-cache decode / block verify                                        */
/* ------------------------------------------------------------------------ */

/*
 * Attention of n_new fresh query rows per sequence over that sequence's KV
 * cache: the two per-head loops of blt_kv_decode_step
 * (infer/kv_cache.c:369-390) for every sequence and head at once, with the
 * visibility rule of infer/kv_cache.c:229-236 evaluated in the kernel:
 *
 *   block_mode == 0: row r (position p = base + r) sees key j iff
 *                    j <= p && (window == 0 || p - j < window)
 *   block_mode == 1: every row sees all base + n_new keys (the block rows of
 *                    the INFER mask, ops/mask_builder_cpu.c:130-135).
 *
 * Cache row = absolute byte position (infer/kv_cache.h:45-65); sequence b's
 * rows start at cache + b * cache_seq_stride. When k_new/v_new are given, the
 * kernel attends to them as rows [base, base + n_new) and also writes them
 * into the cache (the write-through of infer/kv_cache.c:352-365); otherwise
 * the cache must already hold those rows. base_len is not modified.
 */
typedef struct {
    int32_t batch;
    int32_t num_heads;
    int32_t head_dim; /* 32, 64 or 128 */
    int32_t n_new;    /* 1..32 (block_generation.c:154 caps the block size at 32) */
    int32_t block_mode;
    int32_t window;
    int32_t max_len;  /* host-known upper bound of base_len[b] + n_new */
    int32_t splits;   /* > 0: key-range pieces per (sequence, head), one CTA each; 0 = choose;
                       * < 0: persistent grid over equal shares of all key blocks (batch <= 8192,
                       * max_len required), for few sequences of very unequal length */
    const int32_t *base_len; /* device [batch] */
    float *k_cache;          /* device */
    float *v_cache;
    int64_t cache_seq_stride; /* elements */
    int64_t cache_row_stride; /* elements, >= num_heads*head_dim */
    const float *q;           /* device [batch*n_new rows] */
    int64_t q_stride;
    const float *k_new; /* optional device [batch*n_new rows] */
    const float *v_new;
    int64_t kv_new_stride;
    float *out; /* device [batch*n_new rows] */
    int64_t out_stride;
    float scale;
    int32_t base_add; /* added to every base_len[b]: lets a run of steps share one length table */
    /* Optional fused rotary embedding (the per-head rope_apply + strided copies of
     * infer/kv_cache.c:347-366): device tables [positions, head_dim/2] as
     * blt_rope_precompute fills them (ops/reductions_cpu.c:179-197). When given, q and
     * k_new hold the un-rotated rows of the QKV projection; the kernel rotates row r with
     * position base + r (interleaved pairs, ops/reductions_cpu.c:217-228), attends, and
     * writes the rotated K rows to the cache. NULL: rows arrive already rotated. */
    const float *rope_cos;
    const float *rope_sin;
} fblt_decode_desc;

/* Bytes of device scratch fblt_attn_decode needs for this descriptor (0 when
 * the key range is not split). */
size_t fblt_attn_decode_workspace(const fblt_decode_desc *desc);
int fblt_attn_decode(const fblt_decode_desc *desc, void *workspace, size_t workspace_bytes, void *stream);

/*
 * fblt_attn_decode without any allocation by anyone. (No counterpart in the
 * reference: its operators take every temporary from the caller's arena.)
 *
 * Who needs it: a host loop that gave all device memory to a bump arena at
 * start-up (the way the reference's runtime does) has nothing left to size a
 * split-K workspace from in the middle of a generation, and a latency-bound
 * decode loop cannot afford cudaMalloc, which may synchronise the whole device
 * and can fail. Here the split-K partials live in a fixed array inside the
 * library instead: fblt_attn_decode_static_capacity() bytes (4 MiB) of device
 * memory on every GPU that loads the library, held until the process exits.
 *
 * Same descriptor, same results as fblt_attn_decode. Differences:
 *   - a descriptor whose partials (fblt_attn_decode_workspace(desc) bytes)
 *     exceed the capacity is rejected with FBLT_ERR_LIMIT; pass splits = 1
 *     (no partials at all) or use fblt_attn_decode for those;
 *   - the first call on each device looks the array's device address up
 *     (cudaGetSymbolAddress, with that device current) and keeps it for the
 *     life of the process. Make that first call during set-up, before any
 *     stream capture begins. The kept address does not survive a
 *     cudaDeviceReset(): a process that resets a device must not call this
 *     entry point on it afterwards;
 *   - all calls share the one array and it keeps whatever the last call left
 *     there. Nothing has to start at zero: each call overwrites every slot it
 *     later reads. Two calls whose kernels can overlap on the GPU (different
 *     streams, or different host threads on one device) would overwrite each
 *     other's partials: serialise them.
 * The call itself uses no cudaMalloc, cudaFree or allocating library routine.
 */
size_t fblt_attn_decode_static_capacity(void);
int fblt_attn_decode_static(const fblt_decode_desc *desc, void *stream);

/* ------------------------------------------------------------------------ */
/* L1: decision step (bit-exact integer / compare logic)                     */
/* ------------------------------------------------------------------------ */

/*
 * Row argmax with the reference tie rule: strict '>' scan from index 0, so
 * the lowest index wins (infer/self_speculation.c:21-31,
 * ops/row_stats.cu:46-83). logits: device [rows, vocab] with row stride
 * `stride`; ids_out: device [rows].
 */
int fblt_argmax_rows(const float *logits, int64_t stride, int32_t rows, int32_t vocab, int32_t *ids_out,
                     void *stream);

/*
 * Accept-until-first-mismatch of Algorithm 2 as blt_verify_draft runs it on
 * the host (infer/self_speculation.c:160-182), for a batch of candidates.
 * Candidate c has committed length l[c] and draft length r[c]; x is
 * [batch, x_stride] bytes; pred is the argmax byte of every candidate
 * position ([batch, pred_stride], pred[p] = argmax of logits row p). For each
 * candidate writes new_len[c] and fixes x in place exactly as the reference:
 * first p in [l, l+r) with x[p] != pred[p-1] -> x[p] = pred[p-1], new_len =
 * p+1; none -> if l+r < target_len: x[l+r] = pred[l+r-1], new_len = l+r+1,
 * else new_len = l+r. accepted[c] receives the number of accepted draft
 * bytes. All pointers device.
 */
int fblt_verify_accept(uint8_t *x, int64_t x_stride, const int32_t *pred, int64_t pred_stride, const int32_t *l,
                       const int32_t *r, const int32_t *target_len, int32_t batch, int32_t *new_len,
                       int32_t *accepted, void *stream);

/*
 * One verify-and-commit round of block drafting with verification (BLT-DV) for a batch of
 * independent sequences that decode over a KV cache, entirely on the device: the verifier's
 * argmax, the accept loop of blt_verify_draft (infer/self_speculation.c:154-182) as the
 * generation loop calls it (infer/block_generation.c:436-453) and the per-sequence cache
 * roll-back (blt_kv_cache_truncate, infer/kv_cache.c:94-99) -- no logits, bytes or lengths
 * travel to the host between the verifier's last layer and the next round's launch.
 *
 * Sequence c has committed bytes x[c][0 .. l[c]) followed by r[c] drafted bytes, and its cache
 * held cache_len[c] valid rows before the verifier ran (cache_len[c] <= l[c] - 1: the rows of
 * bytes cache_len[c] .. l[c] + r[c] - 1 were computed in this round). logits is
 * [batch * width, stride]: row c * width + i is the verifier's output at position
 * cache_len[c] + i, i.e. its prediction for byte cache_len[c] + i + 1; width >= l[c] + r[c] -
 * cache_len[c] for every c. Effects, per sequence, exactly as the reference's host loop: drafts
 * are accepted up to the first mismatch, which is replaced by the prediction; on a full match one
 * free byte is appended unless target_len[c] is reached. l[c] receives the new committed length,
 * accepted[c] (optional) the number of accepted drafts, and cache_len[c] becomes the old l[c] +
 * accepted[c]: the rows computed from bytes that stayed (what follows was computed from a
 * rejected draft and is overwritten by the next round). A sequence whose lengths do not fit the
 * description is left untouched and reports accepted = -1.
 * pred_scratch: device [batch * width] int32. All pointers device. Bytes: vocab <= 256.
 */
int fblt_dv_commit(const float *logits, int64_t stride, int32_t width, int32_t vocab, int32_t batch, uint8_t *x,
                   int64_t x_stride, int32_t *l, const int32_t *r, const int32_t *target_len, int32_t *cache_len,
                   int32_t *accepted, int32_t *pred_scratch, void *stream);

/* Host mirrors of the selection helpers (same names minus the prefix, same
 * results): blt_unmask_select_confidence / _eb (infer/block_generation.c:20-58),
 * blt_aligned_commit_select (infer/self_speculation.c:73-80),
 * blt_block_adapt_b (infer/block_generation.c:139-152). */
uint32_t fblt_unmask_select_confidence(const float *scores, const uint8_t *masked, size_t B, float alpha);
uint32_t fblt_unmask_select_eb(const float *scores, const uint8_t *masked, size_t B, float gamma);
size_t fblt_aligned_commit_select(const fblt_patch_info *patches, size_t num_patches, size_t lo, size_t hi);
size_t fblt_block_adapt_b(size_t cur_b, double rolling_acceptance, size_t b_min, size_t b_max, float target);

/*
 * One unmask round of the block-diffusion drafter for a batch of candidates,
 * on the device: replaces the full-logit download, row_analyze / row_argmax
 * host loops and the selection call of infer/block_generation.c:225-252.
 * logits is [batch * B, stride] (row c * B + b = cell b of candidate c, the
 * block rows only); masked and tokens are [batch, B] bytes, updated in
 * place: every selected cell gets tokens = argmax byte, masked = 0.
 * Per cell p_max and entropy (nats) of softmax(row) are accumulated in double
 * like the reference; strategy FBLT_UNMASK_CONFIDENCE selects masked cells
 * with p_max >= threshold (else the most confident one), ENTROPY_BOUNDED the
 * largest ascending-entropy prefix whose sum stays <= threshold. Optional
 * outputs: sel_out [batch] bit b = cell b chosen, conf_out / ent_out
 * [batch, B], remaining_out [batch] = cells still masked. 1 <= B <= 32.
 * All pointers device.
 */
enum { FBLT_UNMASK_CONFIDENCE = 0, FBLT_UNMASK_ENTROPY_BOUNDED = 1 }; /* blt_unmask_strategy, block_generation.h:37-41 */
int fblt_unmask_step(const float *logits, int64_t stride, int32_t batch, int32_t B, int32_t vocab, int32_t strategy,
                     float threshold, uint8_t *masked, uint8_t *tokens, uint32_t *sel_out, float *conf_out,
                     float *ent_out, int32_t *remaining_out, void *stream);

/* Leading patches identical (start and length) in a cached boundary snapshot and a new
 * segmentation: blt_kv_cache_common_patches (infer/kv_cache.c:101-109) over plain arrays.
 * Host arrays. */
size_t fblt_kv_common_patches(const fblt_patch_info *cached, size_t num_cached, const fblt_patch_info *patches,
                              size_t num_patches);

/* ------------------------------------------------------------------------ */
/* projection GEMMs on both sides of the attention operator                 */
/* ------------------------------------------------------------------------ */

/*
 * out[M, N] = a[M, K] * b[K, N] (+ bias[N]), fp32 row-major: blt_matmul
 * (ops/matmul.h:8; CPU loop ops/linalg_cpu.c:8-18, cublasSgemm call
 * ops/linalg.cu:134-136) as used for the QKV and output projections
 * (models/attention.c:156,206; models/cross_attention.c:139-141,154).
 * The weight matrix is packed once -- split into TF32 (hi, lo) parts and
 * laid out in the tile order the tensor-core kernel consumes -- and reused
 * by every call; activations are split on the fly. FBLT_PREC_FP32 runs three
 * TF32 products per term (lo*hi + hi*lo + hi*hi, fp32 accumulate: fp32-class
 * accuracy), FBLT_PREC_TF32 one. K and lda must be multiples of 4 and `a`
 * 16-byte aligned; M, N are arbitrary. All pointers device.
 */
size_t fblt_matmul_packed_bytes(int64_t K, int64_t N);
int fblt_matmul_pack_weights(const float *b, int64_t ldb, int64_t K, int64_t N, void *packed, size_t packed_bytes,
                             void *stream);
int fblt_matmul(const float *a, int64_t lda, const void *packed_b, const float *bias, float *out, int64_t ldo,
                int64_t M, int64_t K, int64_t N, int32_t precision, void *stream);

/*
 * The multi-head self-attention block of blt_multihead_attention
 * (models/attention.h:12-26, models/attention.c:130-207) for a batch of packed
 * sequences: qkv = input * weight_qkv; Q, K rotated when rope tables are given
 * (position = row index within the sequence); per-head attention under `mask`
 * with scale 1/sqrt(head_dim); output = combined * weight_proj. Weights are the
 * fblt_matmul_pack_weights images of weight_qkv [E, 3E] and weight_proj [E, E].
 * qkv_work [total_rows, 3E] and combined_work [total_rows, E] are caller-provided
 * scratch. Three launches: with embed_dim and head_dim multiples of 32 (and no
 * causal_offset in the mask) the first matmul's epilogue rotates Q and K, so qkv_work
 * holds the rotated projection afterwards and every attention kernel, the TMA-fed one
 * for sequences of at most 128 keys included, takes the rows as they are; otherwise
 * qkv_work holds the un-rotated projection and the attention kernel rotates as it loads.
 * total_rows is the host copy of cu_rows[batch]; max_len bounds the sequence
 * lengths. All pointers device.
 */
typedef struct {
    int32_t batch, num_heads, head_dim, max_len;
    int64_t total_rows;
    const int32_t *cu_rows; /* [batch + 1] */
    const float *input;
    int64_t input_stride;
    const void *packed_qkv;
    const void *packed_proj;
    float *output;
    int64_t output_stride;
    float *qkv_work;
    float *combined_work;
    fblt_mask_desc mask; /* is_causal / sliding_window / documents of blt_attention_config.mask_config */
    const float *rope_cos; /* NULL: no rotary embedding (use_rope = false) */
    const float *rope_sin;
    int32_t precision; /* FBLT_PREC_FP32 or FBLT_PREC_TF32, for the matmuls and the attention */
    int32_t reserved;
} fblt_mha_desc;

int fblt_mha_forward(const fblt_mha_desc *desc, void *stream);

/*
 * The cross-attention block of blt_cross_attention_forward
 * (models/cross_attention.h:54-56, models/cross_attention.c:98-157) for a batch:
 * Q = query_in * weight_q; K, V = kv_in * [weight_k | weight_v]; attention under
 * `mask` (the patch rules FBLT_GROUP_PATCH_ENC / _DEC replace the group-id
 * arrays), no rotary embedding; output = combined * weight_proj. query_in and
 * kv_in are the split-form views [rows, E] the reference builds for its split
 * modes. packed_kv is one buffer of fblt_matmul_packed_bytes(E, 2E) bytes: the
 * packed weight_k followed by the packed weight_v (packing [E, E] twice into
 * the two halves equals packing the concatenation). Scratch: q_work
 * [total_q_rows, E], kv_work [total_k_rows, 2E], combined_work [total_q_rows, E].
 * All pointers device.
 */
typedef struct {
    int32_t batch, num_heads, head_dim, max_q, max_k;
    int32_t precision;
    int64_t total_q_rows, total_k_rows;
    const int32_t *cu_q; /* [batch + 1] */
    const int32_t *cu_k;
    const float *query_in;
    int64_t query_stride;
    const float *kv_in;
    int64_t kv_stride;
    const void *packed_q;
    const void *packed_kv;
    const void *packed_proj;
    float *output;
    int64_t output_stride;
    float *q_work;
    float *kv_work;
    float *combined_work;
    fblt_mask_desc mask;
} fblt_cross_desc;

int fblt_cross_attention_forward(const fblt_cross_desc *desc, void *stream);

/*
 * The self-attention part of one cache-aware decode step, blt_kv_decode_step
 * (infer/kv_cache.c:338-396), for a batch of sequences with their own cache
 * lengths: qkv = input * weight_qkv for the batch * n_new new rows (row
 * b * n_new + r = sequence b, absolute position base_len[b] + r); Q and K
 * rotated with that position when rope tables are given; K and V written
 * through to cache rows base .. base + n_new; attention of the new rows over
 * the cache (causal inside the new rows, or all-visible with block_mode; optional
 * window); output = combined * weight_proj. Cache layout and the other fields as
 * in fblt_decode_desc. workspace may be NULL (then the key range is not split).
 * Does not advance base_len. All pointers device.
 * The call only enqueues launches on `stream` (no allocation, no wait) and the
 * lengths are read from base_len on the device when the kernels run, so a loop
 * of steps can be captured once in a CUDA graph and replayed while the caches
 * grow; max_len must then bound base_len[b] + n_new over every replay.
 */
typedef struct {
    int32_t batch, num_heads, head_dim, n_new;
    int32_t block_mode, window, max_len, precision;
    const int32_t *base_len;
    float *k_cache;
    float *v_cache;
    int64_t cache_seq_stride, cache_row_stride;
    const float *input;
    int64_t input_stride;
    const void *packed_qkv;
    const void *packed_proj;
    float *output;
    int64_t output_stride;
    float *qkv_work;      /* [batch * n_new, 3E] */
    float *combined_work; /* [batch * n_new, E] */
    void *workspace;
    size_t workspace_bytes;
    const float *rope_cos;
    const float *rope_sin;
} fblt_kv_step_desc;

int fblt_kv_self_attention_step(const fblt_kv_step_desc *desc, void *stream);

/* ------------------------------------------------------------------------ */
/* host-buffer sessions (what a host-side caller with no device memory uses) */
/* ------------------------------------------------------------------------ */

typedef struct fblt_session fblt_session;

/*
 * A session owns a stream, device staging for one batch and, optionally, a
 * batched two-array KV cache [batch, cache_rows, E] (the layout
 * blt_kv_cache_create_batched reserves, infer/kv_cache.h:71-75). All
 * allocation happens here; the per-step calls below allocate nothing.
 * max_q_rows / max_k_rows bound the packed row counts of one forward call.
 */
int fblt_session_create(fblt_session **out, int32_t max_batch, int32_t num_heads, int32_t head_dim,
                        int64_t max_q_rows, int64_t max_k_rows, int32_t cache_rows, int32_t max_new);
void fblt_session_destroy(fblt_session *s);

/*
 * Host-memory form of fblt_attn_forward: every pointer in `desc` (tensors and
 * the int32 tables of desc->mask) is HOST memory; rows are copied to the
 * device, the batch runs, `out` rows are copied back and the call returns
 * after the stream is idle. q/k/v may alias one packed buffer.
 * mask.q_group_ids / k_group_ids are not supported here.
 */
int fblt_session_forward(fblt_session *s, const fblt_attn_desc *host_desc);
/*
 * The same call without the final wait: the output rows travel home on a stream of their own
 * while the caller goes on (fblt_session_cache_load, fblt_session_decode_steps, ... on the same
 * session run beside the download). Every host buffer and table of `host_desc` must stay valid
 * and `out` must not be read until fblt_session_wait() has returned.
 */
int fblt_session_forward_async(fblt_session *s, const fblt_attn_desc *host_desc);
/* Returns when everything enqueued on the session has completed (and reports a tcgen05 bounded-
 * wait failure of a forward call, if any). */
int fblt_session_wait(fblt_session *s);

/* Loads `lens[b]` rows of host K/V ([batch, rows_stride_rows, E] with the
 * given per-sequence stride in rows) into the session cache and sets the
 * cache lengths. */
int fblt_session_cache_load(fblt_session *s, int32_t batch, const int32_t *lens, const float *k_host,
                            const float *v_host, int64_t host_seq_stride_rows);
/*
 * One decode / block-verify step from host rows: q_new, k_new, v_new are
 * [batch*n_new, E] host arrays; rows are written through to the cache, the
 * attention runs, out ([batch*n_new, E] host) is filled, and every cache
 * length grows by `advance` (<= n_new; the rows past base + advance are
 * overwritten by the next step, the rollback of infer/kv_cache.c:252-336).
 */
int fblt_session_decode(fblt_session *s, int32_t batch, int32_t n_new, int32_t block_mode, int32_t window,
                        float scale, const float *q_new, const float *k_new, const float *v_new, float *out,
                        int32_t advance);
/*
 * A run of `steps` decode / block-verify steps whose input rows are all known up front
 * (step t reads q_new + t * in_step_stride etc., writes out + t * out_step_stride; a stride
 * of 0 re-reads the same rows). Same result as calling fblt_session_decode `steps` times,
 * but the host->device copy of step t+1, the kernel of step t and the device->host copy of
 * step t-1 overlap on three streams over double-buffered staging. Returns when all outputs
 * are in host memory.
 */
int fblt_session_decode_steps(fblt_session *s, int32_t batch, int32_t n_new, int32_t steps, int32_t block_mode,
                              int32_t window, float scale, const float *q_new, const float *k_new,
                              const float *v_new, int64_t in_step_stride, float *out, int64_t out_step_stride,
                              int32_t advance);
/* Per-sequence blt_kv_cache_truncate (infer/kv_cache.c:94-99): sets the valid length of
 * every sequence's cache tier to lens[b] (<= cache_rows; shrinking rolls back, growing
 * covers rows the caller has just written). No data is cleared. */
int fblt_session_cache_truncate(fblt_session *s, int32_t batch, const int32_t *lens);
/* blt_kv_cache_reset (infer/kv_cache.c:89-92): all lengths to 0. */
int fblt_session_cache_reset(fblt_session *s);
/* Current cache lengths (host copy), for checks. */
int fblt_session_cache_lens(fblt_session *s, int32_t *lens_out, int32_t batch);

/*
 * The tcgen05 kernels (attention tile and unit kernels, matmul) bound every mbarrier wait; a CTA whose wait runs
 * out records a code, waits (bounded) for what it has in flight, frees its TMEM and returns without writing its
 * rows -- the launching call has long returned FBLT_OK by then. A caller that launches fblt_attn_forward,
 * fblt_mha_forward, fblt_cross_attention_forward, fblt_kv_self_attention_step or fblt_matmul on its own stream
 * therefore polls this word where it synchronises anyway (the session entry points do it in
 * fblt_session_wait). This call synchronises the device, returns that code (0 = none, -1 = CUDA error) and
 * clears it.
 */
int fblt_tcgen05_error(void);

/* ------------------------------------------------------------------------ */
/* One process per GPU: batch sharding and the output gather                 */
/* ------------------------------------------------------------------------ */

/*
 * The reference runs one sequence at a time in one process (infer.c); its plan for batches
 * is a [batch, ...] cache (infer/kv_cache.h:71-75). Independent sequences shard by batch with
 * no exchange inside attention: rank `rank` of `world` owns units [*begin, *end), contiguous,
 * the first units % world ranks one unit longer.
 */
int fblt_shard_partition(int64_t units, int32_t world, int32_t rank, int64_t *begin, int64_t *end);

/*
 * Host-side all-gather of one small blob per rank through a directory every rank can reach
 * (a tmpfs on one box), with a deadline: the check-in that comes before the first device copy
 * towards a peer. all[r * bytes ..] receives rank r's blob. FBLT_ERR_TIMEOUT names the first
 * absent rank in fblt_last_error(); a rank that timed out, or that called
 * fblt_rendezvous_report_failure, makes every later arrival fail with FBLT_ERR_PEER instead of
 * going on alone. `tag` must be unique per rendezvous within the directory.
 */
int fblt_rendezvous_files(const char *dir, const char *tag, int32_t rank, int32_t world, const void *mine,
                          size_t bytes, void *all, int32_t deadline_ms);
int fblt_rendezvous_report_failure(const char *dir, const char *tag, int32_t rank);

/*
 * Gather of output rows onto every GPU of one box. Each rank owns a receive buffer
 * [world, max_rows, row_elems] (fblt_gather_buffer, device memory of the current device,
 * allocated by fblt_gather_create); fblt_gather_rows copies `nrows` of this rank's rows
 * (device) to rows [row_offset, row_offset + nrows) of slot [rank] of EVERY rank's buffer with
 * asynchronous device-to-device copies on `stream` (copy engines over NVLink; no kernel, no
 * load from a peer, no waiting on the device). Set-up: every rank creates, exports its
 * fblt_gather_handle_bytes()-byte handle, the job all-gathers the handles on the host
 * (fblt_rendezvous_files, or its own store) and every rank connects with the world * bytes
 * array. A rank's buffer holds everybody's rows once every rank's copies have completed: the
 * caller orders that (a barrier of the job after synchronising `stream`). Destroy only after
 * such a barrier: peers write into the buffer until then.
 */
typedef struct fblt_gather fblt_gather;
size_t fblt_gather_handle_bytes(void);
int fblt_gather_create(fblt_gather **out, int32_t rank, int32_t world, size_t max_rows, size_t row_elems);
int fblt_gather_export(fblt_gather *g, void *handle_out);
int fblt_gather_connect(fblt_gather *g, const void *all_handles);
int fblt_gather_rows(fblt_gather *g, const float *rows, size_t nrows, size_t row_offset, void *stream);
float *fblt_gather_buffer(fblt_gather *g);
void fblt_gather_destroy(fblt_gather *g);

/* Number of kernels this library has launched in this process (all threads). With
 * FBLT_REPORT_LAUNCHES=1 in the environment the same count is printed to stderr when the
 * process ends ("[fblt] N kernel launches"). */
uint64_t fblt_launch_count(void);
/* sizeof of {fblt_head_args, fblt_patch_info, fblt_mask_desc, fblt_attn_desc,
 * fblt_decode_desc, fblt_mha_desc, fblt_cross_desc, fblt_kv_step_desc}, for bindings that re-declare the structs. Returns the count. */
size_t fblt_abi_sizes(size_t *out, size_t cap);

#ifdef __cplusplus
}
#endif
#endif /* FBLT_ATTN_H */
