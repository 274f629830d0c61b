"""The five benchmark configurations as concrete seeded host inputs.

Each builder returns plain numpy arrays plus the MaskConfig that describes the
visibility rule, so the same object feeds the GPU path (after upload) and the
CPU oracle (which turns the rule into dense masks with the reference's own
builder). `batch` can be reduced for oracle-sized checks; element i of every
tensor depends only on (seed, tensor tag, i), so a reduced batch is a prefix of
the full one.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np

from . import lib as L
from . import synth
from .ops import MaskConfig


@dataclass
class ForwardCase:
    name: str
    num_heads: int
    head_dim: int
    scale: float
    q: np.ndarray            # [rows_q, q_stride] view, head 0 at column 0
    k: np.ndarray
    v: np.ndarray
    cu_q: np.ndarray
    cu_k: np.ndarray
    mask: MaskConfig
    packed: Optional[np.ndarray] = None   # backing [T, 3E] buffer when q/k/v are views of one
    meta: dict = field(default_factory=dict)

    @property
    def embed(self) -> int:
        return self.num_heads * self.head_dim

    def algorithmic_bytes(self) -> int:
        """Q + K + V read once, O written once (fp32)."""
        E = self.embed
        return 4 * E * (2 * int(self.cu_q[-1]) + 2 * int(self.cu_k[-1]))


def _packed_qkv(seed: int, rows: int, E: int, std: float):
    buf = np.empty((rows, 3 * E), dtype=np.float32)
    buf[:, 0:E] = synth.normal(seed, synth.TAG_Q, rows * E, std).reshape(rows, E)
    buf[:, E:2 * E] = synth.normal(seed, synth.TAG_K, rows * E, std).reshape(rows, E)
    buf[:, 2 * E:] = synth.normal(seed, synth.TAG_V, rows * E, std).reshape(rows, E)
    return buf


def c1_byte_self_attention(seq_len: int = 512, window: int = 512) -> ForwardCase:
    """Causal sliding-window byte self-attention: batch 1, 4 heads x 32, packed [T, 3E], seed 0."""
    H, hd = 4, 32
    E = H * hd
    buf = _packed_qkv(0, seq_len, E, 1.0 / np.sqrt(32.0))
    cu = np.array([0, seq_len], dtype=np.int32)
    return ForwardCase("c1_byte_self", H, hd, 1.0 / np.sqrt(32.0), buf[:, 0:E], buf[:, E:2 * E], buf[:, 2 * E:], cu, cu,
                       MaskConfig(is_causal=True, sliding_window=window), packed=buf)


def patch_self_attention(seed: int, batch: int, num_heads: int, name: str, with_tensors: bool = True) -> ForwardCase:
    """Block-causal patch-transformer attention: patch i attends to patches <= i; head_dim 64.
    with_tensors=False returns only the patch structure (row tables and mask); q/k/v are then
    empty [0, 3E] views for callers that fill device tensors themselves."""
    hd = 64
    E = num_heads * hd
    pb = synth.patch_batch(seed, batch)
    cu = np.zeros(batch + 1, dtype=np.int32)
    cu[1:] = np.cumsum(pb.num_patches)
    buf = _packed_qkv(seed, int(cu[-1]), E, 1.0 / 8.0) if with_tensors else np.zeros((0, 3 * E), np.float32)
    return ForwardCase(name, num_heads, hd, 1.0 / 8.0, buf[:, 0:E], buf[:, E:2 * E], buf[:, 2 * E:], cu, cu,
                       MaskConfig(is_causal=True), packed=buf,
                       meta={"patches": pb, "capped": pb.capped})


def c2_patch_attention(batch: int = 16) -> ForwardCase:
    return patch_self_attention(1, batch, 8, "c2_patch_self")


def c5_prefill(batch: int = 2048, with_tensors: bool = True) -> ForwardCase:
    return patch_self_attention(4, batch, 16, "c5_prefill", with_tensors)


def c3_cross_attention(direction: str, batch: int = 32, seq_len: int = 512) -> ForwardCase:
    """Local encoder / decoder cross-attention, 4 heads x 64, seed 2.

    direction "enc": patch queries over byte keys, each patch sees its own bytes.
    direction "dec_leq": byte queries over patch keys, patches <= the byte's patch.
    direction "dec_paper": byte queries over patch keys, the reference's one-latent rule.
    """
    H, hd = 4, 64
    E = H * hd
    pb = synth.patch_batch(2, batch, seq_len)
    cu_p = np.zeros(batch + 1, dtype=np.int32)
    cu_p[1:] = np.cumsum(pb.num_patches)
    cu_b = np.arange(batch + 1, dtype=np.int32) * seq_len
    nb, npatch = batch * seq_len, int(cu_p[-1])
    byte_a = synth.normal(2, synth.TAG_K, nb * E, 0.125).reshape(nb, E)
    byte_b = synth.normal(2, synth.TAG_V, nb * E, 0.125).reshape(nb, E)
    patch_a = synth.normal(2, synth.TAG_Q, npatch * E, 0.125).reshape(npatch, E)
    patch_b = synth.normal(2, synth.TAG_AUX, npatch * E, 0.125).reshape(npatch, E)
    meta = {"patches": pb}
    if direction == "enc":
        mask = MaskConfig(group_rule=L.GROUP_PATCH_ENC, subtokens=1, patch_bounds=pb.bounds)
        return ForwardCase("c3_enc", H, hd, 0.125, patch_a, byte_a, byte_b, cu_p, cu_b, mask, meta=meta)
    rule = L.GROUP_PATCH_LEQ if direction == "dec_leq" else L.GROUP_PATCH_DEC
    mask = MaskConfig(group_rule=rule, subtokens=1, patch_bounds=pb.bounds)
    return ForwardCase("c3_" + direction, H, hd, 0.125, byte_a, patch_a, patch_b, cu_b, cu_p, mask, meta=meta)


@dataclass
class DecodeCase:
    name: str
    num_heads: int
    head_dim: int
    scale: float
    n_new: int
    block_mode: bool
    window: int
    base_len: np.ndarray      # [batch]
    cache_rows: int
    k_cache: np.ndarray       # [batch, cache_rows, E]; rows >= base_len are zero
    v_cache: np.ndarray
    q: np.ndarray             # [batch * n_new, E]
    k_new: np.ndarray
    v_new: np.ndarray

    @property
    def embed(self) -> int:
        return self.num_heads * self.head_dim

    def algorithmic_bytes(self) -> int:
        """K and V rows of every visible position read once, q read and out written once."""
        E = self.embed
        rows = int(self.base_len.sum()) + len(self.base_len) * self.n_new
        return 4 * E * (2 * rows + 2 * len(self.base_len) * self.n_new)


def decode_case(seed: int, batch: int, num_heads: int, n_new: int, block_mode: bool, *, lens=None,
                cache_rows: Optional[int] = None, window: int = 0, name: str = "decode") -> DecodeCase:
    hd = 64
    E = num_heads * hd
    base = synth.cache_lengths(seed, batch) if lens is None else np.asarray(lens, dtype=np.int32)
    rows = int(cache_rows if cache_rows is not None else (int(base.max()) + n_new + 3) // 4 * 4)
    kc = synth.normal(seed, synth.TAG_K, batch * rows * E).reshape(batch, rows, E)
    vc = synth.normal(seed, synth.TAG_V, batch * rows * E).reshape(batch, rows, E)
    live = np.arange(rows)[None, :] < base[:, None]
    kc *= live[:, :, None]
    vc *= live[:, :, None]
    q = synth.normal(seed, synth.TAG_Q, batch * n_new * E).reshape(batch * n_new, E)
    kn = synth.normal(seed, synth.TAG_AUX, batch * n_new * E).reshape(batch * n_new, E)
    vn = synth.normal(seed, synth.TAG_AUX + 1, batch * n_new * E).reshape(batch * n_new, E)
    return DecodeCase(name, num_heads, hd, 0.125, n_new, block_mode, window, base, rows, kc, vc, q, kn, vn)


def c4_decode(batch: int = 256) -> DecodeCase:
    """KV-cache decode: cache lengths U{64..512}, one query byte per step, 4 heads x 64, seed 3."""
    return decode_case(3, batch, 4, 1, False, name="c4_decode")


def c4_block_verify(batch: int = 256) -> DecodeCase:
    """BLT-DV verify / diffusion variant: a block of 4 query rows, bidirectional inside the
    block and attending the whole cache."""
    return decode_case(3, batch, 4, 4, True, name="c4_block")


def c5_decode(batch: int, base_len: int = 512, steps: int = 64) -> DecodeCase:
    """One block-verify step of the scaled workload: 16 heads x 64, B = 4, caches start at
    `base_len` rows and grow by 4 per step for `steps` steps (every draft accepted)."""
    lens = np.full(batch, base_len, dtype=np.int32)
    return decode_case(4, batch, 16, 4, True, lens=lens, cache_rows=base_len + 4 * steps, name="c5_decode")
