"""ctypes binding of libfblt_attn.so (the C ABI declared in include/fblt_attn.h).

Loading fails loudly when the library has not been built: there is no other
implementation behind these calls.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libfblt_attn.so"

c_float_p = C.POINTER(C.c_float)
c_i32_p = C.POINTER(C.c_int32)
c_u8_p = C.POINTER(C.c_uint8)

OK, ERR_ARG, ERR_UNSUPPORTED, ERR_WORKSPACE, ERR_CUDA, ERR_CAPACITY, ERR_LIMIT, ERR_PEER, ERR_TIMEOUT = range(9)
BACKEND_CPU, BACKEND_CUDA = 0, 1
GROUP_NONE, GROUP_PATCH_ENC, GROUP_PATCH_DEC, GROUP_PATCH_LEQ, GROUP_IDS = range(5)
IMPL_AUTO, IMPL_ROW, IMPL_TILE, IMPL_TCGEN05, IMPL_ROW_QUAD, IMPL_UNIT = range(6)
PREC_FP32, PREC_TF32 = 0, 1


class HeadArgs(C.Structure):
    """fblt_head_args == blt_attention_head_args (ops/attn_core.h:25-44)."""
    _fields_ = [
        ("q", C.c_void_p), ("q_stride", C.c_size_t),
        ("k", C.c_void_p), ("k_stride", C.c_size_t),
        ("v", C.c_void_p), ("v_stride", C.c_size_t),
        ("combined", C.c_void_p), ("combined_stride", C.c_size_t), ("combined_col_offset", C.c_size_t),
        ("weights_out", C.c_void_p), ("lse_out", C.c_void_p), ("scores_scratch", C.c_void_p),
        ("mask", C.c_void_p),
        ("nq", C.c_size_t), ("nk", C.c_size_t), ("head_dim", C.c_size_t),
        ("is_causal", C.c_bool), ("scale", C.c_float),
    ]


class PatchInfo(C.Structure):
    """fblt_patch_info == blt_patch_info (models/patcher.h:16-20)."""
    _fields_ = [("start_idx", C.c_size_t), ("length", C.c_size_t), ("peak_entropy", C.c_float)]


class MaskDesc(C.Structure):
    _fields_ = [
        ("is_causal", C.c_int32), ("sliding_window", C.c_int32), ("group_rule", C.c_int32),
        ("subtokens", C.c_int32), ("bidirectional_within_group", C.c_int32), ("reserved", C.c_int32),
        ("causal_offset", C.c_void_p), ("cu_doc", C.c_void_p), ("doc_bounds", C.c_void_p),
        ("cu_patch", C.c_void_p), ("patch_bounds", C.c_void_p), ("q_pos_offset", C.c_void_p),
        ("trailing_closed", C.c_void_p), ("q_group_ids", C.c_void_p), ("k_group_ids", C.c_void_p),
        ("num_clean", C.c_void_p),
    ]


class MaskConfig(C.Structure):
    """fblt_mask_config == blt_mask_config (ops/mask_builder.h:12-32); id arrays are host size_t."""
    _fields_ = [
        ("seq_len_q", C.c_size_t), ("seq_len_kv", C.c_size_t), ("sliding_window", C.c_size_t),
        ("doc_boundaries", C.c_void_p), ("num_docs", C.c_size_t),
        ("query_group_ids", C.c_void_p), ("kv_group_ids", C.c_void_p),
        ("bidirectional_within_group", C.c_bool), ("is_causal", C.c_bool), ("causal_offset", C.c_size_t),
    ]


class BlockDiffusionConfig(C.Structure):
    """fblt_block_diffusion_config == blt_block_diffusion_config (ops/mask_builder.h:43-68)."""
    _fields_ = [
        ("mode", C.c_int), ("seq_len", C.c_size_t), ("num_clean", C.c_size_t), ("block_size", C.c_size_t),
        ("block_starts", C.c_void_p), ("num_blocks", C.c_size_t),
    ]


class MhaDesc(C.Structure):
    _fields_ = [
        ("batch", C.c_int32), ("num_heads", C.c_int32), ("head_dim", C.c_int32), ("max_len", C.c_int32),
        ("total_rows", C.c_int64), ("cu_rows", C.c_void_p),
        ("input", C.c_void_p), ("input_stride", C.c_int64),
        ("packed_qkv", C.c_void_p), ("packed_proj", C.c_void_p),
        ("output", C.c_void_p), ("output_stride", C.c_int64),
        ("qkv_work", C.c_void_p), ("combined_work", C.c_void_p),
        ("mask", MaskDesc),
        ("rope_cos", C.c_void_p), ("rope_sin", C.c_void_p),
        ("precision", C.c_int32), ("reserved", C.c_int32),
    ]


class CrossDesc(C.Structure):
    _fields_ = [
        ("batch", C.c_int32), ("num_heads", C.c_int32), ("head_dim", C.c_int32), ("max_q", C.c_int32),
        ("max_k", C.c_int32), ("precision", C.c_int32),
        ("total_q_rows", C.c_int64), ("total_k_rows", C.c_int64),
        ("cu_q", C.c_void_p), ("cu_k", C.c_void_p),
        ("query_in", C.c_void_p), ("query_stride", C.c_int64),
        ("kv_in", C.c_void_p), ("kv_stride", C.c_int64),
        ("packed_q", C.c_void_p), ("packed_kv", C.c_void_p), ("packed_proj", C.c_void_p),
        ("output", C.c_void_p), ("output_stride", C.c_int64),
        ("q_work", C.c_void_p), ("kv_work", C.c_void_p), ("combined_work", C.c_void_p),
        ("mask", MaskDesc),
    ]


class KvStepDesc(C.Structure):
    _fields_ = [
        ("batch", C.c_int32), ("num_heads", C.c_int32), ("head_dim", C.c_int32), ("n_new", C.c_int32),
        ("block_mode", C.c_int32), ("window", C.c_int32), ("max_len", C.c_int32), ("precision", C.c_int32),
        ("base_len", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p),
        ("cache_seq_stride", C.c_int64), ("cache_row_stride", C.c_int64),
        ("input", C.c_void_p), ("input_stride", C.c_int64),
        ("packed_qkv", C.c_void_p), ("packed_proj", C.c_void_p),
        ("output", C.c_void_p), ("output_stride", C.c_int64),
        ("qkv_work", C.c_void_p), ("combined_work", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("rope_cos", C.c_void_p), ("rope_sin", C.c_void_p),
    ]


class AttnDesc(C.Structure):
    _fields_ = [
        ("batch", C.c_int32), ("num_heads", C.c_int32), ("head_dim", C.c_int32),
        ("max_q", C.c_int32), ("max_k", C.c_int32), ("impl", C.c_int32), ("precision", C.c_int32),
        ("total_q_rows", C.c_int32),
        ("cu_q", C.c_void_p), ("cu_k", C.c_void_p),
        ("q", C.c_void_p), ("q_stride", C.c_int64),
        ("k", C.c_void_p), ("k_stride", C.c_int64),
        ("v", C.c_void_p), ("v_stride", C.c_int64),
        ("out", C.c_void_p), ("out_stride", C.c_int64),
        ("scale", C.c_float), ("total_k_rows", C.c_int32),
        ("mask", MaskDesc),
        ("rope_cos", C.c_void_p), ("rope_sin", C.c_void_p), ("rope_q_pos", C.c_void_p), ("rope_k_pos", C.c_void_p),
    ]


class DecodeDesc(C.Structure):
    _fields_ = [
        ("batch", C.c_int32), ("num_heads", C.c_int32), ("head_dim", C.c_int32), ("n_new", C.c_int32),
        ("block_mode", C.c_int32), ("window", C.c_int32), ("max_len", C.c_int32), ("splits", C.c_int32),
        ("base_len", C.c_void_p),
        ("k_cache", C.c_void_p), ("v_cache", C.c_void_p),
        ("cache_seq_stride", C.c_int64), ("cache_row_stride", C.c_int64),
        ("q", C.c_void_p), ("q_stride", C.c_int64),
        ("k_new", C.c_void_p), ("v_new", C.c_void_p), ("kv_new_stride", C.c_int64),
        ("out", C.c_void_p), ("out_stride", C.c_int64),
        ("scale", C.c_float), ("base_add", C.c_int32),
        ("rope_cos", C.c_void_p), ("rope_sin", C.c_void_p),
    ]


# name -> (restype, argtypes): every symbol include/fblt_attn.h declares
SYMBOLS = {
    "fblt_last_error": (C.c_char_p, []),
    "fblt_status_string": (C.c_char_p, [C.c_int]),
    "fblt_version": (C.c_char_p, []),
    "blt_attention_head_core_cuda": (None, [C.c_int, C.POINTER(HeadArgs)]),
    "blt_attention_head_core_backward_cuda": (None, [C.c_int, C.c_void_p]),
    "fblt_attention_head": (C.c_int, [C.POINTER(HeadArgs), C.c_void_p]),
    "fblt_patch_bounds": (C.c_int, [C.POINTER(PatchInfo), C.c_size_t, C.c_size_t, c_i32_p]),
    "fblt_patch_latent_at": (C.c_int32, [c_i32_p, C.c_int32, C.c_int32]),
    "fblt_attn_forward": (C.c_int, [C.POINTER(AttnDesc), C.c_void_p]),
    "fblt_mask_bitmap": (C.c_int, [C.POINTER(AttnDesc), C.c_void_p, C.c_int, C.c_void_p]),
    "fblt_mask_materialize": (C.c_int, [C.POINTER(AttnDesc), C.c_int32, C.c_void_p, c_i32_p, C.c_void_p]),
    "fblt_shard_partition": (C.c_int, [C.c_int64, C.c_int32, C.c_int32, C.POINTER(C.c_int64), C.POINTER(C.c_int64)]),
    "fblt_rendezvous_files": (C.c_int, [C.c_char_p, C.c_char_p, C.c_int32, C.c_int32, C.c_void_p, C.c_size_t, C.c_void_p,
                                        C.c_int32]),
    "fblt_rendezvous_report_failure": (C.c_int, [C.c_char_p, C.c_char_p, C.c_int32]),
    "fblt_gather_handle_bytes": (C.c_size_t, []),
    "fblt_gather_create": (C.c_int, [C.POINTER(C.c_void_p), C.c_int32, C.c_int32, C.c_size_t, C.c_size_t]),
    "fblt_gather_export": (C.c_int, [C.c_void_p, C.c_void_p]),
    "fblt_gather_connect": (C.c_int, [C.c_void_p, C.c_void_p]),
    "fblt_gather_rows": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p]),
    "fblt_gather_buffer": (C.c_void_p, [C.c_void_p]),
    "fblt_gather_destroy": (None, [C.c_void_p]),
    "fblt_mask_dense_scratch_bytes": (C.c_size_t, [C.POINTER(MaskConfig)]),
    "fblt_build_attention_mask_dense": (C.c_int, [C.POINTER(MaskConfig), C.c_void_p, C.c_void_p, C.c_size_t, c_i32_p,
                                                  C.c_void_p]),
    "fblt_block_diffusion_mask_scratch_bytes": (C.c_size_t, [C.POINTER(BlockDiffusionConfig)]),
    "fblt_build_block_diffusion_mask_dense": (C.c_int, [C.POINTER(BlockDiffusionConfig), C.c_void_p, C.c_void_p,
                                                        C.c_size_t, c_i32_p, C.c_void_p]),
    "fblt_attn_decode_workspace": (C.c_size_t, [C.POINTER(DecodeDesc)]),
    "fblt_attn_decode": (C.c_int, [C.POINTER(DecodeDesc), C.c_void_p, C.c_size_t, C.c_void_p]),
    "fblt_attn_decode_static_capacity": (C.c_size_t, []),
    "fblt_attn_decode_static": (C.c_int, [C.POINTER(DecodeDesc), C.c_void_p]),
    "fblt_argmax_rows": (C.c_int, [C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "fblt_verify_accept": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p,
                                     C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]),
    "fblt_dv_commit": (C.c_int, [C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_int64, C.c_void_p,
                                 C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "fblt_unmask_select_confidence": (C.c_uint32, [c_float_p, c_u8_p, C.c_size_t, C.c_float]),
    "fblt_unmask_select_eb": (C.c_uint32, [c_float_p, c_u8_p, C.c_size_t, C.c_float]),
    "fblt_aligned_commit_select": (C.c_size_t, [C.POINTER(PatchInfo), C.c_size_t, C.c_size_t, C.c_size_t]),
    "fblt_block_adapt_b": (C.c_size_t, [C.c_size_t, C.c_double, C.c_size_t, C.c_size_t, C.c_float]),
    "fblt_unmask_step": (C.c_int, [C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_float,
                                   C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "fblt_kv_common_patches": (C.c_size_t, [C.POINTER(PatchInfo), C.c_size_t, C.POINTER(PatchInfo), C.c_size_t]),
    "fblt_matmul_packed_bytes": (C.c_size_t, [C.c_int64, C.c_int64]),
    "fblt_matmul_pack_weights": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_size_t,
                                           C.c_void_p]),
    "fblt_matmul": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64,
                              C.c_int64, C.c_int64, C.c_int32, C.c_void_p]),
    "fblt_mha_forward": (C.c_int, [C.POINTER(MhaDesc), C.c_void_p]),
    "fblt_cross_attention_forward": (C.c_int, [C.POINTER(CrossDesc), C.c_void_p]),
    "fblt_kv_self_attention_step": (C.c_int, [C.POINTER(KvStepDesc), C.c_void_p]),
    "fblt_session_create": (C.c_int, [C.POINTER(C.c_void_p), C.c_int32, C.c_int32, C.c_int32, C.c_int64, C.c_int64,
                                      C.c_int32, C.c_int32]),
    "fblt_session_destroy": (None, [C.c_void_p]),
    "fblt_session_forward": (C.c_int, [C.c_void_p, C.POINTER(AttnDesc)]),
    "fblt_session_forward_async": (C.c_int, [C.c_void_p, C.POINTER(AttnDesc)]),
    "fblt_session_wait": (C.c_int, [C.c_void_p]),
    "fblt_session_cache_load": (C.c_int, [C.c_void_p, C.c_int32, c_i32_p, C.c_void_p, C.c_void_p, C.c_int64]),
    "fblt_session_decode": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_float, C.c_void_p,
                                      C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32]),
    "fblt_session_decode_steps": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_float,
                                            C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64,
                                            C.c_int32]),
    "fblt_session_cache_truncate": (C.c_int, [C.c_void_p, C.c_int32, c_i32_p]),
    "fblt_session_cache_reset": (C.c_int, [C.c_void_p]),
    "fblt_session_cache_lens": (C.c_int, [C.c_void_p, c_i32_p, C.c_int32]),
    "fblt_tcgen05_error": (C.c_int, []),
    "fblt_launch_count": (C.c_uint64, []),
    "fblt_abi_sizes": (C.c_size_t, [C.POINTER(C.c_size_t), C.c_size_t]),
}

UNMASK_CONFIDENCE, UNMASK_ENTROPY_BOUNDED = 0, 1

_lib = None


class FbltError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"fblt status {status}: {message}")
        self.status = status


def load() -> C.CDLL:
    """Load libfblt_attn.so (built by `python -m fblt_b200.build`). Raises if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(f"{LIB_PATH} is missing: build it with `python -m fblt_b200.build` "
                          "(there is no fallback implementation)")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    sizes = (C.c_size_t * 16)()
    n = lib.fblt_abi_sizes(sizes, 16)
    want = [C.sizeof(HeadArgs), C.sizeof(PatchInfo), C.sizeof(MaskDesc), C.sizeof(AttnDesc), C.sizeof(DecodeDesc), C.sizeof(MhaDesc), C.sizeof(CrossDesc), C.sizeof(KvStepDesc)]
    if list(sizes[:n]) != want:
        raise ImportError(f"ABI mismatch between lib.py and libfblt_attn.so: {list(sizes[:n])} vs {want}")
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != OK:
        raise FbltError(status, load().fblt_last_error().decode())
