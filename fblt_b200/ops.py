"""Host-side mirror of the reference's attention operator interface over the C ABI.

Names follow the reference: `attention_head_core` is blt_attention_head_core
(ops/attn_core.h:46) on the CUDA backend; `MaskConfig` is the batched
blt_mask_config (ops/mask_builder.h:12-32); `attn_forward` / `attn_decode`
replace the per-head loops of models/attention.c:199-202,
models/cross_attention.c:147-150 and infer/kv_cache.c:303-324,369-390.

torch is used only to own device memory and streams; every computation goes
through libfblt_attn.so.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch

from . import lib as L


def _ptr(t) -> Optional[int]:
    if t is None:
        return None
    if isinstance(t, torch.Tensor):
        return t.data_ptr()
    if isinstance(t, np.ndarray):
        return t.ctypes.data
    raise TypeError(type(t))


def _stream_ptr(stream) -> Optional[int]:
    if stream is None:
        return torch.cuda.current_stream().cuda_stream or None
    if isinstance(stream, torch.cuda.Stream):
        return stream.cuda_stream or None
    return stream


# --------------------------------------------------------------------------- L0

def attention_head_core(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, combined: torch.Tensor, *,
                        col_offset: int, head_dim: int, scale: float, is_causal: bool = False,
                        mask: Optional[torch.Tensor] = None, weights_out: Optional[torch.Tensor] = None,
                        lse_out: Optional[torch.Tensor] = None, scores_scratch: Optional[torch.Tensor] = None,
                        fatal: bool = False) -> None:
    """One head of one sequence. q/k/v are 2-D fp32 CUDA views whose first column is the
    head's first column (row stride = .stride(0)); `combined` is the full [nq, E] output
    buffer and only `head_dim` columns at `col_offset` are written.

    fatal=True goes through the reference-named symbol (errors exit the process, as in
    the reference); otherwise the status-returning twin is used.
    """
    lib = L.load()
    a = L.HeadArgs()
    a.q, a.q_stride = q.data_ptr(), q.stride(0)
    a.k, a.k_stride = k.data_ptr(), k.stride(0)
    a.v, a.v_stride = v.data_ptr(), v.stride(0)
    a.combined, a.combined_stride, a.combined_col_offset = combined.data_ptr(), combined.stride(0), col_offset
    a.weights_out = _ptr(weights_out)
    a.lse_out = _ptr(lse_out)
    a.scores_scratch = _ptr(scores_scratch)
    a.mask = _ptr(mask)
    a.nq, a.nk, a.head_dim = q.shape[0], k.shape[0], head_dim
    a.is_causal, a.scale = bool(is_causal), float(scale)
    if fatal:
        lib.blt_attention_head_core_cuda(L.BACKEND_CUDA, C.byref(a))
    else:
        L.check(lib.fblt_attention_head(C.byref(a), _stream_ptr(None)))


# --------------------------------------------------------------------------- patches

def patch_bounds(starts: Sequence[int], lengths: Sequence[int], seq_len: int) -> np.ndarray:
    """Boundary array [P+1] from (start_idx, length) pairs, validated like the reference
    validates tiling (ops/patch_pool_cpu.c:98-112)."""
    lib = L.load()
    n = len(starts)
    arr = (L.PatchInfo * max(n, 1))()
    for i, (s, ln) in enumerate(zip(starts, lengths)):
        arr[i].start_idx, arr[i].length, arr[i].peak_entropy = int(s), int(ln), 0.0
    out = np.zeros(n + 1, dtype=np.int32)
    L.check(lib.fblt_patch_bounds(arr, n, seq_len, out.ctypes.data_as(L.c_i32_p)))
    return out


def patch_latent_at(bounds: np.ndarray, pos: int) -> int:
    b = np.ascontiguousarray(bounds, dtype=np.int32)
    return int(L.load().fblt_patch_latent_at(b.ctypes.data_as(L.c_i32_p), len(b) - 1, int(pos)))


# --------------------------------------------------------------------------- masks

@dataclass
class MaskConfig:
    """Batched blt_mask_config. Per-sequence lists hold one numpy array per sequence."""
    is_causal: bool = False
    sliding_window: int = 0
    group_rule: int = L.GROUP_NONE
    subtokens: int = 1
    bidirectional_within_group: bool = True
    causal_offset: Optional[Sequence[int]] = None          # [batch]
    doc_bounds: Optional[List[np.ndarray]] = None           # per sequence: first position of doc d+1
    patch_bounds: Optional[List[np.ndarray]] = None         # per sequence: [P+1]
    q_pos_offset: Optional[Sequence[int]] = None            # [batch]
    trailing_closed: Optional[Sequence[int]] = None         # [batch]
    num_clean: Optional[Sequence[int]] = None               # [batch] -> block-diffusion INFER rule
    q_group_ids: Optional[np.ndarray] = None                # [total q rows]
    k_group_ids: Optional[np.ndarray] = None                # [total k rows]

    def host_tables(self, batch: int):
        """int32 numpy tables in the layout the C descriptor wants."""
        t = {}

        def i32(x):
            return np.ascontiguousarray(np.asarray(x, dtype=np.int32))

        if self.causal_offset is not None:
            t["causal_offset"] = i32(self.causal_offset)
        if self.doc_bounds is not None:
            cu = np.zeros(batch + 1, dtype=np.int32)
            cu[1:] = np.cumsum([len(d) for d in self.doc_bounds])
            flat = np.concatenate([i32(d) for d in self.doc_bounds]) if cu[-1] else np.zeros(1, np.int32)
            t["cu_doc"], t["doc_bounds"] = cu, i32(flat)
        if self.patch_bounds is not None:
            cu = np.zeros(batch + 1, dtype=np.int32)
            cu[1:] = np.cumsum([len(p) for p in self.patch_bounds])
            t["cu_patch"], t["patch_bounds"] = cu, i32(np.concatenate([i32(p) for p in self.patch_bounds]))
        if self.q_pos_offset is not None:
            t["q_pos_offset"] = i32(self.q_pos_offset)
        if self.trailing_closed is not None:
            t["trailing_closed"] = np.ascontiguousarray(np.asarray(self.trailing_closed, dtype=np.uint8))
        if self.num_clean is not None:
            t["num_clean"] = i32(self.num_clean)
        if self.q_group_ids is not None:
            t["q_group_ids"] = i32(self.q_group_ids)
        if self.k_group_ids is not None:
            t["k_group_ids"] = i32(self.k_group_ids)
        return t

    def fill(self, m: L.MaskDesc, tables: dict) -> None:
        m.is_causal = int(self.is_causal)
        m.sliding_window = int(self.sliding_window)
        m.group_rule = int(self.group_rule)
        m.subtokens = int(self.subtokens)
        m.bidirectional_within_group = int(self.bidirectional_within_group)
        for name in ("causal_offset", "cu_doc", "doc_bounds", "cu_patch", "patch_bounds", "q_pos_offset",
                     "trailing_closed", "q_group_ids", "k_group_ids", "num_clean"):
            setattr(m, name, _ptr(tables.get(name)))


@dataclass
class AttnBatch:
    """Device-resident descriptor of one batched forward call; keeps its tables alive."""
    desc: L.AttnDesc
    keep: list = field(default_factory=list)


def make_batch(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor, cu_q: Sequence[int],
               cu_k: Sequence[int], num_heads: int, head_dim: int, scale: float,
               mask: Optional[MaskConfig] = None, impl: int = L.IMPL_AUTO, precision: int = L.PREC_FP32,
               rope_cos: Optional[torch.Tensor] = None, rope_sin: Optional[torch.Tensor] = None,
               rope_q_pos: Optional[torch.Tensor] = None, rope_k_pos: Optional[torch.Tensor] = None) -> AttnBatch:
    """q/k/v/out: 2-D fp32 CUDA views (rows packed over sequences, row stride = .stride(0),
    first column = head 0). cu_q / cu_k: row offsets [batch+1] (host)."""
    dev = q.device
    cu_q_h = np.asarray(cu_q, dtype=np.int32)
    cu_k_h = np.asarray(cu_k, dtype=np.int32)
    batch = len(cu_q_h) - 1
    mask = mask or MaskConfig()
    d = L.AttnDesc()
    d.batch, d.num_heads, d.head_dim = batch, num_heads, head_dim
    d.max_q = int(np.max(np.diff(cu_q_h))) if batch else 0
    d.max_k = int(np.max(np.diff(cu_k_h))) if batch else 0
    d.impl, d.precision = impl, precision
    d.total_q_rows = int(cu_q_h[-1]) if batch else 0       # where the tensors end: the TMA-loading kernel needs it
    d.total_k_rows = int(cu_k_h[-1]) if batch else 0
    keep = []

    def dev_i32(a):
        t = torch.from_numpy(np.ascontiguousarray(a)).to(dev)
        keep.append(t)
        return t

    d.cu_q = dev_i32(cu_q_h).data_ptr()
    d.cu_k = dev_i32(cu_k_h).data_ptr()
    d.q, d.q_stride = q.data_ptr(), q.stride(0)
    d.k, d.k_stride = k.data_ptr(), k.stride(0)
    d.v, d.v_stride = v.data_ptr(), v.stride(0)
    d.out, d.out_stride = out.data_ptr(), out.stride(0)
    d.scale = float(scale)
    tables = {name: dev_i32(arr) for name, arr in mask.host_tables(batch).items()}
    mask.fill(d.mask, tables)
    if rope_cos is not None:
        d.rope_cos, d.rope_sin = rope_cos.data_ptr(), rope_sin.data_ptr()
        keep += [rope_cos, rope_sin]
        if rope_q_pos is not None:
            d.rope_q_pos = rope_q_pos.data_ptr()
            keep.append(rope_q_pos)
        if rope_k_pos is not None:
            d.rope_k_pos = rope_k_pos.data_ptr()
            keep.append(rope_k_pos)
    keep += [q, k, v, out]
    return AttnBatch(d, keep)


def attn_forward(batch: AttnBatch, stream=None) -> None:
    L.check(L.load().fblt_attn_forward(C.byref(batch.desc), _stream_ptr(stream)))


def mask_bitmap(batch: AttnBatch, use_range: bool = False) -> torch.Tensor:
    """uint8 [batch, max_q, max_k] of allowed(i, j), evaluated by the library on the device."""
    d = batch.desc
    bm = torch.zeros((d.batch, d.max_q, d.max_k), dtype=torch.uint8, device="cuda")
    L.check(L.load().fblt_mask_bitmap(C.byref(d), bm.data_ptr(), int(use_range), _stream_ptr(None)))
    return bm


def mask_materialize(batch: AttnBatch, seq: int):
    d = batch.desc
    cu_q = batch.keep[0].cpu().numpy()
    cu_k = batch.keep[1].cpu().numpy()
    nq, nk = int(cu_q[seq + 1] - cu_q[seq]), int(cu_k[seq + 1] - cu_k[seq])
    m = torch.empty((nq, nk), dtype=torch.float32, device="cuda")
    empty = C.c_int32(0)
    L.check(L.load().fblt_mask_materialize(C.byref(d), seq, m.data_ptr(), C.byref(empty), _stream_ptr(None)))
    return m, empty.value


def _host_sizes(a):
    """Host size_t array (the reference passes its id arrays as host pointers) or None."""
    if a is None:
        return None
    return np.ascontiguousarray(np.asarray(a, dtype=np.uint64))


def build_attention_mask(nq: int, nk: int, *, window: int = 0, doc_boundaries=None, q_groups=None, k_groups=None,
                         bidirectional: bool = True, is_causal: bool = False, causal_offset: int = 0, stream=None):
    """blt_build_attention_mask on the CUDA backend: dense [nq, nk] 0 / -inf tensor and the number of
    query rows without an allowed key (fatal in the reference, ops/mask_builder_cpu.c:93)."""
    lib = L.load()
    c = L.MaskConfig()
    c.seq_len_q, c.seq_len_kv, c.sliding_window = nq, nk, window
    db, qg, kg = _host_sizes(doc_boundaries), _host_sizes(q_groups), _host_sizes(k_groups)
    if db is not None:
        c.doc_boundaries, c.num_docs = db.ctypes.data, len(db) + 1
    if qg is not None:
        c.query_group_ids, c.kv_group_ids = qg.ctypes.data, kg.ctypes.data
    c.bidirectional_within_group, c.is_causal, c.causal_offset = bool(bidirectional), bool(is_causal), causal_offset
    need = lib.fblt_mask_dense_scratch_bytes(C.byref(c))
    scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
    m = torch.full((nq, nk), float("nan"), dtype=torch.float32, device="cuda")
    empty = C.c_int32(-1)
    L.check(lib.fblt_build_attention_mask_dense(C.byref(c), m.data_ptr(), scratch.data_ptr(), need, C.byref(empty),
                                                _stream_ptr(stream)))
    return m, empty.value


def build_block_diffusion_mask(mode: int, S: int, N: int, B: int = 0, block_starts=None, stream=None):
    """blt_build_block_diffusion_mask on the CUDA backend (mode 0 = TRAIN, 1 = INFER): [S, S] and the
    number of empty rows."""
    lib = L.load()
    c = L.BlockDiffusionConfig()
    c.mode, c.seq_len, c.num_clean, c.block_size = mode, S, N, B
    bs = _host_sizes(block_starts)
    if bs is not None:
        c.block_starts, c.num_blocks = bs.ctypes.data, len(bs)
    need = lib.fblt_block_diffusion_mask_scratch_bytes(C.byref(c))
    scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
    m = torch.full((S, S), float("nan"), dtype=torch.float32, device="cuda")
    empty = C.c_int32(-1)
    L.check(lib.fblt_build_block_diffusion_mask_dense(C.byref(c), m.data_ptr(), scratch.data_ptr(), need,
                                                      C.byref(empty), _stream_ptr(stream)))
    return m, empty.value


# --------------------------------------------------------------------------- decode

def make_decode(k_cache: torch.Tensor, v_cache: torch.Tensor, base_len: torch.Tensor, q: torch.Tensor,
                out: torch.Tensor, num_heads: int, head_dim: int, n_new: int, scale: float, *,
                block_mode: bool = False, window: int = 0, k_new: Optional[torch.Tensor] = None,
                v_new: Optional[torch.Tensor] = None, max_len: Optional[int] = None, splits: int = 0,
                rope_cos: Optional[torch.Tensor] = None, rope_sin: Optional[torch.Tensor] = None) -> L.DecodeDesc:
    """k_cache / v_cache: [batch, cache_rows, E] fp32 CUDA; base_len: int32 CUDA [batch];
    q/out (and k_new/v_new): [batch * n_new, E]."""
    d = L.DecodeDesc()
    d.batch, d.num_heads, d.head_dim, d.n_new = k_cache.shape[0], num_heads, head_dim, n_new
    d.block_mode, d.window = int(block_mode), int(window)
    d.max_len = int(max_len) if max_len is not None else int(k_cache.shape[1])
    d.splits = splits
    d.base_len = base_len.data_ptr()
    d.k_cache, d.v_cache = k_cache.data_ptr(), v_cache.data_ptr()
    d.cache_seq_stride, d.cache_row_stride = k_cache.stride(0), k_cache.stride(1)
    d.q, d.q_stride = q.data_ptr(), q.stride(0)
    if k_new is not None:
        d.k_new, d.v_new, d.kv_new_stride = k_new.data_ptr(), v_new.data_ptr(), k_new.stride(0)
    d.out, d.out_stride = out.data_ptr(), out.stride(0)
    d.scale = float(scale)
    if rope_cos is not None:
        d.rope_cos, d.rope_sin = rope_cos.data_ptr(), rope_sin.data_ptr()
    return d


def decode_workspace(d: L.DecodeDesc) -> Optional[torch.Tensor]:
    n = L.load().fblt_attn_decode_workspace(C.byref(d))
    return torch.empty(n, dtype=torch.uint8, device="cuda") if n else None


def attn_decode(d: L.DecodeDesc, workspace: Optional[torch.Tensor] = None, stream=None) -> None:
    wp = workspace.data_ptr() if workspace is not None else None
    wn = workspace.numel() if workspace is not None else 0
    L.check(L.load().fblt_attn_decode(C.byref(d), wp, wn, _stream_ptr(stream)))


# --------------------------------------------------------------------------- decisions

def argmax_rows(logits: torch.Tensor) -> torch.Tensor:
    ids = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    L.check(L.load().fblt_argmax_rows(logits.data_ptr(), logits.stride(0), logits.shape[0], logits.shape[1],
                                      ids.data_ptr(), _stream_ptr(None)))
    return ids


class PackedWeights:
    """b [K, N] packed for fblt_matmul (device buffer + shape)."""

    def __init__(self, b: torch.Tensor):
        assert b.dim() == 2 and b.dtype == torch.float32 and b.is_cuda and b.stride(1) == 1
        self.K, self.N = int(b.shape[0]), int(b.shape[1])
        lib = L.load()
        nbytes = lib.fblt_matmul_packed_bytes(self.K, self.N)
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=b.device)
        L.check(lib.fblt_matmul_pack_weights(b.data_ptr(), b.stride(0), self.K, self.N, self.buf.data_ptr(), nbytes,
                                             _stream_ptr(None)))


def matmul(a: torch.Tensor, w: PackedWeights, out: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
           precision: int = L.PREC_FP32) -> torch.Tensor:
    """out = a @ b (+ bias) with b given as PackedWeights; a [M, K] float32 with unit column stride."""
    assert a.dim() == 2 and a.dtype == torch.float32 and a.stride(1) == 1 and a.shape[1] == w.K
    if out is None:
        out = torch.empty(a.shape[0], w.N, dtype=torch.float32, device=a.device)
    L.check(L.load().fblt_matmul(a.data_ptr(), a.stride(0), w.buf.data_ptr(), bias.data_ptr() if bias is not None else None,
                                 out.data_ptr(), out.stride(0), a.shape[0], w.K, w.N, precision, _stream_ptr(None)))
    return out


def mha_forward(x: torch.Tensor, w_qkv: PackedWeights, w_proj: PackedWeights, cu_rows: Sequence[int], num_heads: int,
                mask: Optional[MaskConfig] = None, rope_cos: Optional[torch.Tensor] = None,
                rope_sin: Optional[torch.Tensor] = None, precision: int = L.PREC_FP32) -> torch.Tensor:
    """The multi-head self-attention block over packed sequences (x [rows, E]); returns [rows, E]."""
    rows, E = int(x.shape[0]), int(x.shape[1])
    dev = x.device
    cu_h = np.asarray(cu_rows, dtype=np.int32)
    batch = len(cu_h) - 1
    mask = mask or MaskConfig()
    d = L.MhaDesc()
    d.batch, d.num_heads, d.head_dim = batch, num_heads, E // num_heads
    d.max_len = int(np.max(np.diff(cu_h))) if batch else 0
    d.total_rows = rows
    keep = []

    def dev_i32(a):
        t = torch.from_numpy(np.ascontiguousarray(a)).to(dev)
        keep.append(t)
        return t

    d.cu_rows = dev_i32(cu_h).data_ptr()
    out = torch.empty(rows, E, dtype=torch.float32, device=dev)
    qkv = torch.empty(rows, 3 * E, dtype=torch.float32, device=dev)
    comb = torch.empty(rows, E, dtype=torch.float32, device=dev)
    d.input, d.input_stride = x.data_ptr(), x.stride(0)
    d.packed_qkv, d.packed_proj = w_qkv.buf.data_ptr(), w_proj.buf.data_ptr()
    d.output, d.output_stride = out.data_ptr(), out.stride(0)
    d.qkv_work, d.combined_work = qkv.data_ptr(), comb.data_ptr()
    tables = {name: dev_i32(arr) for name, arr in mask.host_tables(batch).items()}
    mask.fill(d.mask, tables)
    if rope_cos is not None:
        d.rope_cos, d.rope_sin = rope_cos.data_ptr(), rope_sin.data_ptr()
    d.precision = precision
    L.check(L.load().fblt_mha_forward(C.byref(d), _stream_ptr(None)))
    torch.cuda.current_stream().synchronize()   # the scratch tensors above die with this call
    return out


def cross_attention_forward(query_in: torch.Tensor, kv_in: torch.Tensor, w_q: PackedWeights, w_kv: PackedWeights,
                            w_proj: PackedWeights, cu_q: Sequence[int], cu_k: Sequence[int], num_heads: int,
                            mask: MaskConfig, precision: int = L.PREC_FP32) -> torch.Tensor:
    """The cross-attention block over packed sequences; w_kv packs [weight_k | weight_v] ([E, 2E])."""
    E = int(query_in.shape[1])
    dev = query_in.device
    cu_q_h, cu_k_h = np.asarray(cu_q, dtype=np.int32), np.asarray(cu_k, dtype=np.int32)
    batch = len(cu_q_h) - 1
    d = L.CrossDesc()
    d.batch, d.num_heads, d.head_dim = batch, num_heads, E // num_heads
    d.max_q = int(np.max(np.diff(cu_q_h))) if batch else 0
    d.max_k = int(np.max(np.diff(cu_k_h))) if batch else 0
    d.precision = precision
    d.total_q_rows, d.total_k_rows = int(query_in.shape[0]), int(kv_in.shape[0])
    keep = []

    def dev_i32(a):
        t = torch.from_numpy(np.ascontiguousarray(a)).to(dev)
        keep.append(t)
        return t

    d.cu_q, d.cu_k = dev_i32(cu_q_h).data_ptr(), dev_i32(cu_k_h).data_ptr()
    out = torch.empty(d.total_q_rows, E, dtype=torch.float32, device=dev)
    qw = torch.empty(d.total_q_rows, E, dtype=torch.float32, device=dev)
    kvw = torch.empty(d.total_k_rows, 2 * E, dtype=torch.float32, device=dev)
    comb = torch.empty(d.total_q_rows, E, dtype=torch.float32, device=dev)
    d.query_in, d.query_stride = query_in.data_ptr(), query_in.stride(0)
    d.kv_in, d.kv_stride = kv_in.data_ptr(), kv_in.stride(0)
    d.packed_q, d.packed_kv, d.packed_proj = w_q.buf.data_ptr(), w_kv.buf.data_ptr(), w_proj.buf.data_ptr()
    d.output, d.output_stride = out.data_ptr(), out.stride(0)
    d.q_work, d.kv_work, d.combined_work = qw.data_ptr(), kvw.data_ptr(), comb.data_ptr()
    tables = {name: dev_i32(arr) for name, arr in mask.host_tables(batch).items()}
    mask.fill(d.mask, tables)
    L.check(L.load().fblt_cross_attention_forward(C.byref(d), _stream_ptr(None)))
    torch.cuda.current_stream().synchronize()   # the scratch tensors above die with this call
    return out


def kv_self_attention_step(x: torch.Tensor, w_qkv: PackedWeights, w_proj: PackedWeights, k_cache: torch.Tensor,
                           v_cache: torch.Tensor, base_len: torch.Tensor, num_heads: int, n_new: int, *,
                           rope_cos: Optional[torch.Tensor] = None, rope_sin: Optional[torch.Tensor] = None,
                           block_mode: bool = False, window: int = 0, max_len: int = 0,
                           precision: int = L.PREC_FP32) -> torch.Tensor:
    """Self-attention part of a decode step: x [batch*n_new, E] rows -> [batch*n_new, E]; K/V rows are
    written into the caches ([batch, rows, E]) at base_len .. base_len + n_new."""
    rows, E = int(x.shape[0]), int(x.shape[1])
    dev = x.device
    d = L.KvStepDesc()
    d.batch, d.num_heads, d.head_dim, d.n_new = rows // n_new, num_heads, E // num_heads, n_new
    d.block_mode, d.window, d.precision = int(block_mode), window, precision
    d.max_len = max_len or int(k_cache.shape[1])
    d.base_len = base_len.data_ptr()
    d.k_cache, d.v_cache = k_cache.data_ptr(), v_cache.data_ptr()
    d.cache_seq_stride, d.cache_row_stride = k_cache.stride(0), k_cache.stride(1)
    out = torch.empty(rows, E, dtype=torch.float32, device=dev)
    qkv = torch.empty(rows, 3 * E, dtype=torch.float32, device=dev)
    comb = torch.empty(rows, E, dtype=torch.float32, device=dev)
    ws = torch.empty(8 << 20, dtype=torch.uint8, device=dev)
    d.input, d.input_stride = x.data_ptr(), x.stride(0)
    d.packed_qkv, d.packed_proj = w_qkv.buf.data_ptr(), w_proj.buf.data_ptr()
    d.output, d.output_stride = out.data_ptr(), out.stride(0)
    d.qkv_work, d.combined_work = qkv.data_ptr(), comb.data_ptr()
    d.workspace, d.workspace_bytes = ws.data_ptr(), ws.numel()
    if rope_cos is not None:
        d.rope_cos, d.rope_sin = rope_cos.data_ptr(), rope_sin.data_ptr()
    L.check(L.load().fblt_kv_self_attention_step(C.byref(d), _stream_ptr(None)))
    torch.cuda.current_stream().synchronize()   # the scratch tensors above die with this call
    return out


class KvStepPlan:
    """The decode-step block with every buffer allocated up front: run() only enqueues the three
    launches (no allocation, no synchronisation), so a loop of steps can be captured once in a CUDA
    graph and replayed while the caches grow -- the cache lengths are read from device memory
    (base_len), not baked into the launches. x is the static input [batch*n_new, E]; out the static
    output. max_len must bound base_len + n_new over every replay (default: the cache capacity)."""

    def __init__(self, w_qkv: PackedWeights, w_proj: PackedWeights, k_cache: torch.Tensor, v_cache: torch.Tensor,
                 base_len: torch.Tensor, num_heads: int, n_new: int, *, rope_cos: Optional[torch.Tensor] = None,
                 rope_sin: Optional[torch.Tensor] = None, block_mode: bool = False, window: int = 0,
                 max_len: int = 0, precision: int = L.PREC_FP32):
        batch, E, dev = int(k_cache.shape[0]), int(k_cache.shape[2]), k_cache.device
        rows = batch * n_new
        self.x = torch.zeros(rows, E, dtype=torch.float32, device=dev)
        self.out = torch.empty(rows, E, dtype=torch.float32, device=dev)
        self._qkv = torch.empty(rows, 3 * E, dtype=torch.float32, device=dev)
        self._comb = torch.empty(rows, E, dtype=torch.float32, device=dev)
        self._ws = torch.empty(8 << 20, dtype=torch.uint8, device=dev)
        self._keep = [w_qkv, w_proj, k_cache, v_cache, base_len, rope_cos, rope_sin]
        d = self.desc = L.KvStepDesc()
        d.batch, d.num_heads, d.head_dim, d.n_new = batch, num_heads, E // num_heads, n_new
        d.block_mode, d.window, d.precision = int(block_mode), window, precision
        d.max_len = max_len or int(k_cache.shape[1])
        d.base_len = base_len.data_ptr()
        d.k_cache, d.v_cache = k_cache.data_ptr(), v_cache.data_ptr()
        d.cache_seq_stride, d.cache_row_stride = k_cache.stride(0), k_cache.stride(1)
        d.input, d.input_stride = self.x.data_ptr(), self.x.stride(0)
        d.packed_qkv, d.packed_proj = w_qkv.buf.data_ptr(), w_proj.buf.data_ptr()
        d.output, d.output_stride = self.out.data_ptr(), self.out.stride(0)
        d.qkv_work, d.combined_work = self._qkv.data_ptr(), self._comb.data_ptr()
        d.workspace, d.workspace_bytes = self._ws.data_ptr(), self._ws.numel()
        if rope_cos is not None:
            d.rope_cos, d.rope_sin = rope_cos.data_ptr(), rope_sin.data_ptr()

    def run(self, stream=None) -> None:
        L.check(L.load().fblt_kv_self_attention_step(C.byref(self.desc), _stream_ptr(stream)))


def unmask_step(logits: torch.Tensor, masked: torch.Tensor, tokens: torch.Tensor, strategy: int, threshold: float):
    """One unmask round over a batch of candidates. logits [batch*B, V] float32, masked/tokens
    [batch, B] uint8 (updated in place). Returns (sel [batch] int64 bit masks, conf [batch,B],
    ent [batch,B], remaining [batch])."""
    batch, B = masked.shape
    dev = logits.device
    sel = torch.empty(batch, dtype=torch.int32, device=dev)          # same bits as the uint32 the kernel writes
    conf = torch.empty(batch, B, dtype=torch.float32, device=dev)
    ent = torch.empty(batch, B, dtype=torch.float32, device=dev)
    left = torch.empty(batch, dtype=torch.int32, device=dev)
    L.check(L.load().fblt_unmask_step(logits.data_ptr(), logits.stride(0), batch, B, logits.shape[1], strategy,
                                      float(threshold), masked.data_ptr(), tokens.data_ptr(), sel.data_ptr(),
                                      conf.data_ptr(), ent.data_ptr(), left.data_ptr(), _stream_ptr(None)))
    return sel.to(torch.int64) & 0xFFFFFFFF, conf, ent, left


def verify_accept(x: torch.Tensor, pred: torch.Tensor, l: torch.Tensor, r: torch.Tensor, target_len: torch.Tensor):
    """In-place accept-until-mismatch over a batch of candidates; returns (new_len, accepted)."""
    batch = x.shape[0]
    new_len = torch.empty(batch, dtype=torch.int32, device=x.device)
    accepted = torch.empty(batch, dtype=torch.int32, device=x.device)
    L.check(L.load().fblt_verify_accept(x.data_ptr(), x.stride(0), pred.data_ptr(), pred.stride(0), l.data_ptr(),
                                        r.data_ptr(), target_len.data_ptr(), batch, new_len.data_ptr(),
                                        accepted.data_ptr(), _stream_ptr(None)))
    return new_len, accepted


def dv_commit(logits: torch.Tensor, width: int, x: torch.Tensor, l: torch.Tensor, r: torch.Tensor,
              target_len: torch.Tensor, cache_len: torch.Tensor, stream=None) -> torch.Tensor:
    """One batched verify-and-commit round on the device (fblt_dv_commit): x, l and cache_len are
    updated in place; returns the accepted counts. logits: [batch * width, vocab]."""
    batch = x.shape[0]
    accepted = torch.empty(batch, dtype=torch.int32, device=x.device)
    pred = torch.empty(batch * width, dtype=torch.int32, device=x.device)
    L.check(L.load().fblt_dv_commit(logits.data_ptr(), logits.stride(0), width, logits.shape[1], batch, x.data_ptr(),
                                    x.stride(0), l.data_ptr(), r.data_ptr(), target_len.data_ptr(), cache_len.data_ptr(),
                                    accepted.data_ptr(), pred.data_ptr(), _stream_ptr(stream)))
    return accepted


# --------------------------------------------------------------------------- host-buffer sessions

class Session:
    """Host-buffer path: inputs and outputs are host arrays (numpy, or pinned torch CPU
    tensors); every call copies host->device, computes, copies back and returns idle."""

    def __init__(self, max_batch: int, num_heads: int, head_dim: int, max_q_rows: int = 0, max_k_rows: int = 0,
                 cache_rows: int = 0, max_new: int = 0):
        self._lib = L.load()
        self._h = C.c_void_p()
        L.check(self._lib.fblt_session_create(C.byref(self._h), max_batch, num_heads, head_dim, max_q_rows,
                                              max_k_rows, cache_rows, max_new))
        self.num_heads, self.head_dim = num_heads, head_dim

    def close(self) -> None:
        if self._h:
            self._lib.fblt_session_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def forward(self, q, k, v, out, cu_q, cu_k, scale: float, mask: Optional[MaskConfig] = None, *,
                q_stride=None, k_stride=None, v_stride=None, out_stride=None, impl: int = L.IMPL_AUTO,
                precision: int = L.PREC_FP32, wait: bool = True) -> None:
        """q/k/v/out: host arrays; strides in elements (default: the arrays' own row stride).
        wait=False returns once the work is enqueued (the rows come home beside whatever is called
        next on the session); `out` may be read after wait()."""
        def rs(a, s):
            if s is not None:
                return s
            return a.stride(0) if isinstance(a, torch.Tensor) else a.strides[0] // a.itemsize
        cu_q_h = np.ascontiguousarray(np.asarray(cu_q, dtype=np.int32))
        cu_k_h = np.ascontiguousarray(np.asarray(cu_k, dtype=np.int32))
        batch = len(cu_q_h) - 1
        mask = mask or MaskConfig()
        d = L.AttnDesc()
        d.batch, d.num_heads, d.head_dim = batch, self.num_heads, self.head_dim
        d.max_q = int(np.max(np.diff(cu_q_h))) if batch else 0
        d.max_k = int(np.max(np.diff(cu_k_h))) if batch else 0
        d.impl, d.precision = impl, precision
        d.cu_q, d.cu_k = cu_q_h.ctypes.data, cu_k_h.ctypes.data
        d.q, d.q_stride = _ptr(q), rs(q, q_stride)
        d.k, d.k_stride = _ptr(k), rs(k, k_stride)
        d.v, d.v_stride = _ptr(v), rs(v, v_stride)
        d.out, d.out_stride = _ptr(out), rs(out, out_stride)
        d.scale = float(scale)
        tables = mask.host_tables(batch)
        mask.fill(d.mask, tables)
        fn = self._lib.fblt_session_forward if wait else self._lib.fblt_session_forward_async
        L.check(fn(self._h, C.byref(d)))

    def wait(self) -> None:
        L.check(self._lib.fblt_session_wait(self._h))

    def cache_load(self, lens, k_host, v_host, host_seq_stride_rows: int) -> None:
        lens_h = np.ascontiguousarray(np.asarray(lens, dtype=np.int32))
        L.check(self._lib.fblt_session_cache_load(self._h, len(lens_h), lens_h.ctypes.data_as(L.c_i32_p),
                                                  _ptr(k_host), _ptr(v_host), host_seq_stride_rows))

    def decode(self, batch: int, n_new: int, q_new, k_new, v_new, out, scale: float, *, block_mode: bool = False,
               window: int = 0, advance: Optional[int] = None) -> None:
        L.check(self._lib.fblt_session_decode(self._h, batch, n_new, int(block_mode), window, float(scale),
                                              _ptr(q_new), _ptr(k_new), _ptr(v_new), _ptr(out),
                                              n_new if advance is None else advance))

    def decode_steps(self, batch: int, n_new: int, steps: int, q_new, k_new, v_new, out, scale: float, *,
                     in_step_stride: int = 0, out_step_stride: int = 0, block_mode: bool = False, window: int = 0,
                     advance: Optional[int] = None) -> None:
        """`steps` decode steps with known inputs, copies and kernels overlapped (strides in elements)."""
        L.check(self._lib.fblt_session_decode_steps(self._h, batch, n_new, steps, int(block_mode), window, float(scale),
                                                    _ptr(q_new), _ptr(k_new), _ptr(v_new), in_step_stride, _ptr(out),
                                                    out_step_stride, n_new if advance is None else advance))

    def cache_truncate(self, lens) -> None:
        lens_h = np.ascontiguousarray(np.asarray(lens, dtype=np.int32))
        L.check(self._lib.fblt_session_cache_truncate(self._h, len(lens_h), lens_h.ctypes.data_as(L.c_i32_p)))

    def cache_reset(self) -> None:
        L.check(self._lib.fblt_session_cache_reset(self._h))

    def cache_lens(self, batch: int) -> np.ndarray:
        out = np.zeros(batch, dtype=np.int32)
        L.check(self._lib.fblt_session_cache_lens(self._h, out.ctypes.data_as(L.c_i32_p), batch))
        return out
