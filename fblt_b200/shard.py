"""Batch sharding of independent sequences over the GPUs of one box.

Attention has no exchange step: every (sequence, head) is independent, so each
rank owns a contiguous range of sequences together with their Q/K/V rows and KV
caches, and the only collective is the gather of finished output rows. The
helpers are backend-agnostic (NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

from typing import List, Tuple

import torch
import torch.distributed as dist


def partition(num_sequences: int, world_size: int) -> List[Tuple[int, int]]:
    """Contiguous [begin, end) sequence ranges, sizes differing by at most one."""
    base, extra = divmod(num_sequences, world_size)
    out, start = [], 0
    for r in range(world_size):
        n = base + (1 if r < extra else 0)
        out.append((start, start + n))
        start += n
    return out


def gather_rows(local: torch.Tensor, rows_per_rank: List[int], group=None, padded: torch.Tensor = None,
                gathered: torch.Tensor = None):
    """All-gather of row blocks with unequal row counts.

    `local` is this rank's [rows_per_rank[rank], E] block. Every rank contributes a block
    padded to max(rows_per_rank) rows (all_gather needs equal sizes); the result is the
    [world, max_rows, E] buffer plus the list of valid row counts. `padded` / `gathered` may be
    passed in to avoid allocation inside a timed region.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    max_rows = max(rows_per_rank)
    E = local.shape[1]
    assert local.shape[0] == rows_per_rank[rank]
    if local.shape[0] == max_rows and local.is_contiguous():
        send = local
    else:
        send = padded if padded is not None else local.new_zeros((max_rows, E))
        send[: local.shape[0]].copy_(local)
    if gathered is None:
        gathered = local.new_empty((world, max_rows, E))
    dist.all_gather_into_tensor(gathered.view(world * max_rows, E), send, group=group)
    return gathered, rows_per_rank


def unpad(gathered: torch.Tensor, rows_per_rank: List[int]) -> torch.Tensor:
    """Concatenate the valid rows of a gather_rows() result in rank order."""
    return torch.cat([gathered[r, :n] for r, n in enumerate(rows_per_rank)], dim=0)
