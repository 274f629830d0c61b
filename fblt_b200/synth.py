"""Seeded synthetic inputs for the attention workloads (host side, numpy).

Deterministic and counter-based so any slice of a stream can be produced on its
own: value i of stream (seed, tag) is splitmix64 applied to
`seed * 0x1000003 + tag + (i + 1) * GAMMA` -- the splitmix64 finaliser the
reference itself uses for sampling (infer/block_generation.c:11-18).
Uniforms take the top 24 bits; normals are Box-Muller pairs computed in double
and cast to float32.

These stand in for the TinyStories prompts and trained checkpoints the
reference benchmarks on (docs/BENCHMARKS.md:23-26): only their shapes are kept
(512-byte windows, patches of at most 16 bytes, ~4-byte mean patch).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

import numpy as np

_GAMMA = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)

TAG_Q, TAG_K, TAG_V, TAG_LEN, TAG_AUX = 1, 2, 3, 4, 5


def splitmix64(seed: int, tag: int, start: int, n: int) -> np.ndarray:
    with np.errstate(over="ignore"):
        base = np.uint64((seed * 0x1000003 + tag) & 0xFFFFFFFFFFFFFFFF)
        z = base + np.arange(start + 1, start + n + 1, dtype=np.uint64) * _GAMMA
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
        return z ^ (z >> np.uint64(31))


def uniform(seed: int, tag: int, start: int, n: int) -> np.ndarray:
    """float64 in [0, 1) with 24 random bits."""
    return (splitmix64(seed, tag, start, n) >> np.uint64(40)).astype(np.float64) / 16777216.0


def normal(seed: int, tag: int, n: int, scale: float = 1.0, start: int = 0) -> np.ndarray:
    """n float32 N(0, scale^2) values; element i depends only on (seed, tag, i)."""
    first = start - (start & 1)
    m = (start + n + 1 - first) // 2
    u = uniform(seed, tag, first, 2 * m)
    r = np.sqrt(-2.0 * np.log(1.0 - u[0::2]))
    ang = 2.0 * np.pi * u[1::2]
    z = np.empty(2 * m, dtype=np.float64)
    z[0::2] = r * np.cos(ang)
    z[1::2] = r * np.sin(ang)
    off = start - first
    return (z[off:off + n] * scale).astype(np.float32)


def geometric_patches(seed: int, seq_index: int, total_bytes: int = 512, p: float = 0.25, max_len: int = 16,
                      max_patches: int = 128) -> np.ndarray:
    """Patch lengths drawn i.i.d. geometric(p) clipped to [1, max_len] until `total_bytes`
    are covered; the last patch is truncated to fit. If `max_patches - 1` patches are
    placed and bytes remain, the last patch absorbs the remainder (the reference only
    requires that patches tile the window, ops/patch_pool_cpu.c:105-111)."""
    u = uniform(seed, TAG_LEN, seq_index * 4096, total_bytes)
    lens = np.minimum(max_len, 1 + np.floor(np.log(1.0 - u) / np.log(1.0 - p))).astype(np.int64)
    ends = np.cumsum(lens)
    n = int(np.searchsorted(ends, total_bytes, side="left")) + 1
    out = lens[:n].copy()
    out[-1] = total_bytes - (ends[n - 2] if n > 1 else 0)
    if n > max_patches:
        out = out[:max_patches].copy()
        out[-1] = total_bytes - int(out[:-1].sum())
    return out


def bounds_from_lengths(lens: np.ndarray) -> np.ndarray:
    b = np.zeros(len(lens) + 1, dtype=np.int32)
    b[1:] = np.cumsum(lens)
    return b


@dataclass
class PatchBatch:
    lengths: List[np.ndarray]      # per sequence
    bounds: List[np.ndarray]       # per sequence [P+1]
    num_patches: np.ndarray        # [batch]
    capped: int                    # sequences that hit the max_patches cap


def patch_batch(seed: int, batch: int, total_bytes: int = 512, max_patches: int = 128, first_seq: int = 0) -> PatchBatch:
    lens = [geometric_patches(seed, first_seq + s, total_bytes, max_patches=max_patches) for s in range(batch)]
    capped = sum(1 for l in lens if len(l) == max_patches and l[-1] > 16)
    return PatchBatch(lens, [bounds_from_lengths(l) for l in lens], np.array([len(l) for l in lens], dtype=np.int32),
                      capped)


def cache_lengths(seed: int, batch: int, lo: int = 64, hi: int = 512) -> np.ndarray:
    x = splitmix64(seed, TAG_LEN, 0, batch)
    return (lo + (x % np.uint64(hi - lo + 1))).astype(np.int32)
