"""TEST INFRASTRUCTURE -- ctypes access to the CPU oracle.

`liboracle.so` is the C restatement kept in this folder; `_ref/libblt_ref.so`
is the reference's own object code (built by oracle/Makefile where the
reference tree is mounted). `prefer_ref=True` picks the latter when present.
Only tests, the smoke check and the benchmark's CPU-baseline leg import this.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path
from typing import List, Optional, Sequence

import numpy as np

from fblt_b200.lib import HeadArgs, PatchInfo

HERE = Path(__file__).resolve().parent
ORACLE_SO = HERE / "liboracle.so"
REF_SO = HERE / "_ref" / "libblt_ref.so"

c_sz_p = C.POINTER(C.c_size_t)
c_f_p = C.POINTER(C.c_float)
_oracle = None
_ref = None


def reference_tree() -> Optional[Path]:
    """Where the upstream source tree is mounted: FBLT_REFERENCE_TREE, else a folder named
    `reference` beside the repository. None when absent (as on the GPU box, which uses the
    prebuilt files under oracle/_ref)."""
    cands = [os.environ.get("FBLT_REFERENCE_TREE"), HERE.parent.parent / "reference"]
    for c in cands:
        if c and (Path(c) / "csrc" / "ops" / "attn_core_cpu.c").exists():
            return Path(c)
    return None


def build(accept: bool = True) -> None:
    """make -C oracle: the restatement always; where the reference's sources are mounted also its
    CPU object code and (accept=True, library already built) the two acceptance executables."""
    cmd = ["make", "-C", str(HERE), "-j8"]
    tree = reference_tree()
    if tree is not None:
        cmd.append(f"REF={tree}")
    subprocess.run(cmd + ["all"], check=True, stdout=subprocess.DEVNULL)
    if accept and tree is not None and (HERE.parent / "fblt_b200" / "libfblt_attn.so").exists():
        subprocess.run(cmd + ["accept"], check=True, stdout=subprocess.DEVNULL)


def oracle() -> C.CDLL:
    global _oracle
    if _oracle is None:
        if not ORACLE_SO.exists():
            build()
        lib = C.CDLL(str(ORACLE_SO))
        lib.oracle_run_heads.restype = C.c_double
        lib.oracle_run_heads.argtypes = [C.POINTER(HeadArgs), C.c_size_t, C.c_int]
        lib.oracle_attention_head.argtypes = [C.POINTER(HeadArgs)]
        lib.oracle_build_mask.restype = C.c_size_t
        lib.oracle_build_mask.argtypes = [C.c_size_t, C.c_size_t, C.c_size_t, c_sz_p, C.c_size_t, c_sz_p, c_sz_p,
                                          C.c_int, C.c_int, C.c_size_t, c_f_p]
        lib.oracle_block_diffusion_mask.restype = C.c_size_t
        lib.oracle_block_diffusion_mask.argtypes = [C.c_int, C.c_size_t, C.c_size_t, C.c_size_t, c_sz_p, C.c_size_t,
                                                    c_f_p]
        lib.oracle_decode_self_mask.argtypes = [C.c_size_t, C.c_size_t, C.c_size_t, c_f_p]
        lib.oracle_decode_cross_mask.argtypes = [C.POINTER(PatchInfo), C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t,
                                                 C.c_int, c_f_p]
        lib.oracle_patch_group_ids.restype = C.c_int
        lib.oracle_patch_group_ids.argtypes = [C.POINTER(PatchInfo), C.c_size_t, C.c_size_t, c_sz_p, c_sz_p]
        lib.oracle_decoder_latent_at.restype = C.c_size_t
        lib.oracle_decoder_latent_at.argtypes = [C.POINTER(PatchInfo), C.c_size_t, C.c_size_t]
        lib.oracle_expand_group_ids.argtypes = [c_sz_p, C.c_size_t, C.c_size_t, c_sz_p]
        lib.oracle_argmax_row.restype = C.c_int32
        lib.oracle_argmax_row.argtypes = [c_f_p, C.c_size_t]
        lib.oracle_verify_accept.restype = C.c_size_t
        lib.oracle_verify_accept.argtypes = [C.POINTER(C.c_uint8), c_f_p, C.c_size_t, C.c_size_t, C.c_size_t,
                                             C.c_size_t, c_sz_p]
        lib.oracle_row_analyze.argtypes = [c_f_p, C.c_size_t, c_f_p, c_f_p]
        for nm in ("oracle_unmask_select_confidence", "oracle_unmask_select_eb"):
            getattr(lib, nm).restype = C.c_uint32
            getattr(lib, nm).argtypes = [c_f_p, C.POINTER(C.c_uint8), C.c_size_t, C.c_float]
        lib.oracle_block_adapt_b.restype = C.c_size_t
        lib.oracle_block_adapt_b.argtypes = [C.c_size_t, C.c_double, C.c_size_t, C.c_size_t, C.c_float]
        lib.oracle_aligned_commit_select.restype = C.c_size_t
        lib.oracle_aligned_commit_select.argtypes = [C.POINTER(PatchInfo), C.c_size_t, C.c_size_t, C.c_size_t]
        _oracle = lib
    return _oracle


def have_ref() -> bool:
    return REF_SO.exists()


def ref() -> C.CDLL:
    global _ref
    if _ref is None:
        lib = C.CDLL(str(REF_SO))
        lib.ref_run_heads.restype = C.c_double
        lib.ref_run_heads.argtypes = [C.POINTER(HeadArgs), C.c_size_t, C.c_int]
        lib.ref_attention_head.argtypes = [C.POINTER(HeadArgs)]
        lib.ref_build_mask.argtypes = [C.c_size_t, C.c_size_t, C.c_size_t, c_sz_p, C.c_size_t, c_sz_p, c_sz_p, C.c_int,
                                       C.c_int, C.c_size_t, c_f_p]
        lib.ref_block_diffusion_mask.argtypes = [C.c_int, C.c_size_t, C.c_size_t, C.c_size_t, c_sz_p, C.c_size_t, c_f_p]
        lib.ref_patch_group_ids.argtypes = [C.POINTER(PatchInfo), C.c_size_t, C.c_size_t, c_sz_p, c_sz_p]
        lib.ref_decoder_latent_at.restype = C.c_size_t
        lib.ref_decoder_latent_at.argtypes = [C.POINTER(PatchInfo), C.c_size_t, C.c_size_t]
        lib.ref_expand_group_ids.argtypes = [c_sz_p, C.c_size_t, C.c_size_t, c_sz_p]
        for nm in ("ref_unmask_select_confidence", "ref_unmask_select_eb"):
            getattr(lib, nm).restype = C.c_uint32
            getattr(lib, nm).argtypes = [c_f_p, C.POINTER(C.c_uint8), C.c_size_t, C.c_float]
        lib.ref_block_adapt_b.restype = C.c_size_t
        lib.ref_block_adapt_b.argtypes = [C.c_size_t, C.c_double, C.c_size_t, C.c_size_t, C.c_float]
        lib.ref_aligned_commit_select.restype = C.c_size_t
        lib.ref_aligned_commit_select.argtypes = [C.POINTER(PatchInfo), C.c_size_t, C.c_size_t, C.c_size_t]
        lib.ref_kv_common_patches.restype = C.c_size_t
        lib.ref_kv_common_patches.argtypes = [C.POINTER(PatchInfo), C.c_size_t, C.POINTER(PatchInfo), C.c_size_t]
        lib.ref_argmax_rows.argtypes = [c_f_p, C.c_size_t, C.c_size_t, C.POINTER(C.c_uint32)]
        lib.ref_struct_layout.restype = C.c_size_t
        lib.ref_struct_layout.argtypes = [c_sz_p, C.c_size_t]
        _ref = lib
    return _ref


def rope_tables(max_len: int, head_dim: int, theta: float = 500000.0, use_ref: bool = False):
    """cos/sin tables [max_len, head_dim/2] as blt_rope_precompute fills them."""
    cs = np.empty((max_len, head_dim // 2), dtype=np.float32)
    sn = np.empty_like(cs)
    fn = ref().ref_rope_precompute if use_ref else oracle().oracle_rope_precompute
    fn.argtypes = [C.c_size_t, C.c_float, C.c_size_t, c_f_p, c_f_p]
    fn.restype = None
    fn(max_len, theta, head_dim, _fp(cs), _fp(sn))
    return cs, sn


def rope_apply(x: np.ndarray, cos_rows: np.ndarray, sin_rows: np.ndarray, heads: int, head_dim: int,
               use_ref: bool = False) -> np.ndarray:
    """x: [rows, heads*head_dim]; cos_rows/sin_rows: [rows, head_dim/2] (already gathered per row)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    cos_rows = np.ascontiguousarray(cos_rows, dtype=np.float32)
    sin_rows = np.ascontiguousarray(sin_rows, dtype=np.float32)
    out = np.empty_like(x)
    fn = ref().ref_rope_apply if use_ref else oracle().oracle_rope_apply
    fn.argtypes = [c_f_p, c_f_p, c_f_p, c_f_p, C.c_size_t, C.c_size_t, C.c_size_t]
    fn.restype = None
    fn(_fp(x), _fp(cos_rows), _fp(sin_rows), _fp(out), x.shape[0], heads, head_dim)
    return out


def matmul(a: np.ndarray, b: np.ndarray, use_ref: bool = False) -> np.ndarray:
    """out = a @ b the way blt_matmul's CPU branch computes it (sequential fp32 accumulation)."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    out = np.empty((a.shape[0], b.shape[1]), dtype=np.float32)
    fn = ref().ref_matmul if use_ref else oracle().oracle_matmul
    fn.argtypes = [c_f_p, c_f_p, c_f_p, C.c_size_t, C.c_size_t, C.c_size_t]
    fn.restype = None
    fn(_fp(a), _fp(b), _fp(out), a.shape[0], a.shape[1], b.shape[1])
    return out


def ref_multihead_attention(x: np.ndarray, w_qkv: np.ndarray, w_proj: np.ndarray, num_heads: int, *, is_causal: bool,
                            use_rope: bool, theta: float = 500000.0, window: int = 0, doc_boundaries=None) -> np.ndarray:
    """blt_multihead_attention of the reference on the CPU, one sequence x [T, E]."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    w_qkv = np.ascontiguousarray(w_qkv, dtype=np.float32)
    w_proj = np.ascontiguousarray(w_proj, dtype=np.float32)
    out = np.empty_like(x)
    docs = np.ascontiguousarray(doc_boundaries, dtype=np.uint64) if doc_boundaries is not None and len(doc_boundaries) else None
    fn = ref().ref_multihead_attention
    fn.argtypes = [c_f_p, c_f_p, c_f_p, c_f_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_int, C.c_int, C.c_float,
                   C.c_size_t, c_sz_p, C.c_size_t]
    fn.restype = None
    fn(_fp(x), _fp(w_qkv), _fp(w_proj), _fp(out), x.shape[0], x.shape[1], num_heads, int(is_causal), int(use_rope),
       theta, window, docs.ctypes.data_as(c_sz_p) if docs is not None else None, 0 if docs is None else len(docs) + 1)
    return out


def ref_cross_attention(query_in, kv_in, wq, wk, wv, wp, num_heads: int, q_groups, k_groups) -> np.ndarray:
    """blt_cross_attention_forward of the reference on the CPU, one sequence, group-id mask."""
    arrs = [np.ascontiguousarray(a, dtype=np.float32) for a in (query_in, kv_in, wq, wk, wv, wp)]
    out = np.empty_like(arrs[0])
    qg, kg = _sz(q_groups), _sz(k_groups)
    fn = ref().ref_cross_attention
    fn.argtypes = [c_f_p] * 7 + [C.c_size_t] * 4 + [c_sz_p, c_sz_p]
    fn.restype = None
    fn(*[_fp(a) for a in arrs], _fp(out), arrs[0].shape[0], arrs[1].shape[0], arrs[0].shape[1], num_heads, _szp(qg), _szp(kg))
    return out


def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


# ------------------------------------------------------------------ helpers

def _sz(a) -> Optional[np.ndarray]:
    return None if a is None else np.ascontiguousarray(np.asarray(a, dtype=np.uint64))


def _szp(a):
    return None if a is None else a.ctypes.data_as(c_sz_p)


def _fp(a: np.ndarray):
    return a.ctypes.data_as(c_f_p)


def patch_array(bounds: Sequence[int]):
    n = len(bounds) - 1
    arr = (PatchInfo * max(n, 1))()
    for p in range(n):
        arr[p].start_idx, arr[p].length, arr[p].peak_entropy = int(bounds[p]), int(bounds[p + 1] - bounds[p]), 0.0
    return arr, n


def build_mask(nq: int, nk: int, *, window: int = 0, doc_boundaries=None, q_groups=None, k_groups=None,
               bidirectional: bool = True, is_causal: bool = False, causal_offset: int = 0, use_ref: bool = False):
    """Dense additive mask [nq, nk] and the count of rows with no allowed key. With use_ref the
    reference's builder runs (only when no row is empty: the reference aborts on those)."""
    out = np.empty((nq, nk), dtype=np.float32)
    db, qg, kg = _sz(doc_boundaries), _sz(q_groups), _sz(k_groups)
    ndocs = 0 if db is None else len(db) + 1
    empty = oracle().oracle_build_mask(nq, nk, window, _szp(db), ndocs, _szp(qg), _szp(kg), int(bidirectional),
                                       int(is_causal), causal_offset, _fp(out))
    if use_ref and empty == 0:
        out_r = np.empty((nq, nk), dtype=np.float32)
        ref().ref_build_mask(nq, nk, window, _szp(db), ndocs, _szp(qg), _szp(kg), int(bidirectional), int(is_causal),
                             causal_offset, _fp(out_r))
        return out_r, 0
    return out, int(empty)


def block_diffusion_mask(mode: int, S: int, N: int, B: int = 0, block_starts=None, use_ref: bool = False):
    out = np.empty((S, S), dtype=np.float32)
    bs = _sz(block_starts)
    nb = 0 if bs is None else len(bs)
    if use_ref:
        ref().ref_block_diffusion_mask(mode, S, N, B, _szp(bs), nb, _fp(out))
        return out, 0
    empty = oracle().oracle_block_diffusion_mask(mode, S, N, B, _szp(bs), nb, _fp(out))
    return out, int(empty)


def decode_self_mask(n: int, base: int, window: int = 0) -> np.ndarray:
    out = np.empty((n, base + n), dtype=np.float32)
    oracle().oracle_decode_self_mask(n, base, window, _fp(out))
    return out


def decode_cross_mask(bounds, k: int, n: int, base: int, trailing_closed: bool) -> np.ndarray:
    arr, P = patch_array(bounds)
    out = np.empty((n, P * k), dtype=np.float32)
    oracle().oracle_decode_cross_mask(arr, P, k, n, base, int(trailing_closed), _fp(out))
    return out


def latent_at(bounds, pos: int, use_ref: bool = False) -> int:
    arr, P = patch_array(bounds)
    if use_ref:
        return int(ref().ref_decoder_latent_at(arr, P, pos))
    return int(oracle().oracle_decoder_latent_at(arr, P, pos))


def patch_group_ids(bounds, use_ref: bool = False):
    arr, P = patch_array(bounds)
    T = int(bounds[-1])
    qg = np.zeros(max(P, 1), dtype=np.uint64)
    kg = np.zeros(max(T, 1), dtype=np.uint64)
    if use_ref:
        ref().ref_patch_group_ids(arr, P, T, _szp(qg), _szp(kg))
    else:
        rc = oracle().oracle_patch_group_ids(arr, P, T, _szp(qg), _szp(kg))
        assert rc == 0
    return qg[:P].astype(np.int64), kg[:T].astype(np.int64)


class HeadJobs:
    """A list of single-head jobs over numpy buffers (keeps the buffers alive)."""

    def __init__(self):
        self.jobs: List[HeadArgs] = []
        self.keep = []

    def add(self, q: np.ndarray, k: np.ndarray, v: np.ndarray, out: np.ndarray, *, col: int, head_dim: int,
            q_col: int, k_col: int, v_col: int, scale: float, mask: Optional[np.ndarray] = None,
            is_causal: bool = False, weights_out: Optional[np.ndarray] = None, nq: Optional[int] = None,
            nk: Optional[int] = None, q_row: int = 0, k_row: int = 0) -> None:
        """q/k/v/out are 2-D float32 arrays; *_col is the head's first column; *_row the first row."""
        a = HeadArgs()
        isz = 4
        a.q = q.ctypes.data + (q_row * q.strides[0]) + q_col * isz
        a.q_stride = q.strides[0] // isz
        a.k = k.ctypes.data + (k_row * k.strides[0]) + k_col * isz
        a.k_stride = k.strides[0] // isz
        a.v = v.ctypes.data + (k_row * v.strides[0]) + v_col * isz
        a.v_stride = v.strides[0] // isz
        a.combined = out.ctypes.data + q_row * out.strides[0]
        a.combined_stride = out.strides[0] // isz
        a.combined_col_offset = col
        a.weights_out = weights_out.ctypes.data if weights_out is not None else None
        a.mask = mask.ctypes.data if mask is not None else None
        a.nq = q.shape[0] - q_row if nq is None else nq
        a.nk = k.shape[0] - k_row if nk is None else nk
        a.head_dim = head_dim
        a.is_causal = bool(is_causal)
        a.scale = float(scale)
        self.jobs.append(a)
        self.keep += [q, k, v, out, mask, weights_out]

    def run(self, nthreads: int = 0, use_ref: bool = False) -> float:
        """Runs every job; returns wall seconds inside the thread pool."""
        n = len(self.jobs)
        arr = (HeadArgs * max(n, 1))(*self.jobs)
        nt = nthreads if nthreads > 0 else host_cores()
        if use_ref:
            return float(ref().ref_run_heads(arr, n, nt))
        return float(oracle().oracle_run_heads(arr, n, nt))


def batched_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, cu_q, cu_k, num_heads: int, head_dim: int,
                      scale: float, masks: Sequence[Optional[np.ndarray]], *, is_causal: bool = False,
                      q_col0: int = 0, k_col0: int = 0, v_col0: int = 0, use_ref: bool = False,
                      nthreads: int = 0):
    """CPU attention of a packed varlen batch: one reference-operator call per (sequence, head),
    masks[b] being that sequence's dense additive mask (or None). Returns (out [rows_q, E], seconds)."""
    E = num_heads * head_dim
    out = np.zeros((q.shape[0], E), dtype=np.float32)
    jobs = HeadJobs()
    for b in range(len(cu_q) - 1):
        nq, nk = int(cu_q[b + 1] - cu_q[b]), int(cu_k[b + 1] - cu_k[b])
        if nq == 0:
            continue
        for h in range(num_heads):
            jobs.add(q, k, v, out, col=h * head_dim, head_dim=head_dim, q_col=q_col0 + h * head_dim,
                     k_col=k_col0 + h * head_dim, v_col=v_col0 + h * head_dim, scale=scale, mask=masks[b],
                     is_causal=is_causal, nq=nq, nk=nk, q_row=int(cu_q[b]), k_row=int(cu_k[b]))
    secs = jobs.run(nthreads, use_ref)
    return out, secs
