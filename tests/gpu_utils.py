"""Helpers for the gpu-marked tests: run a workload case through the C ABI on cuda:0."""
from __future__ import annotations

import numpy as np
import torch

from fblt_b200 import lib as L
from fblt_b200 import ops
from fblt_b200.workloads import DecodeCase, ForwardCase


def upload_case(case: ForwardCase):
    """Device copies that keep the host layout (packed [T, 3E] stays packed)."""
    if case.packed is not None:
        E = case.embed
        buf = torch.from_numpy(case.packed).cuda()
        return buf[:, 0:E], buf[:, E:2 * E], buf[:, 2 * E:]
    return (torch.from_numpy(np.ascontiguousarray(case.q)).cuda(),
            torch.from_numpy(np.ascontiguousarray(case.k)).cuda(),
            torch.from_numpy(np.ascontiguousarray(case.v)).cuda())


def forward_gpu(case: ForwardCase, impl: int = L.IMPL_AUTO, precision: int = L.PREC_FP32, fill: float = float("nan"),
                rope=None, rope_pos=None):
    """rope: optional (cos, sin) numpy tables [positions, head_dim/2]; the kernels then rotate Q and K.
    rope_pos: optional (q_pos, k_pos) int32 arrays, one position per packed row."""
    q, k, v = upload_case(case)
    rope_kw = {}
    if rope is not None:
        rope_kw = dict(rope_cos=torch.from_numpy(rope[0]).cuda(), rope_sin=torch.from_numpy(rope[1]).cuda())
        if rope_pos is not None:
            rope_kw.update(rope_q_pos=torch.from_numpy(np.ascontiguousarray(rope_pos[0], np.int32)).cuda(),
                           rope_k_pos=torch.from_numpy(np.ascontiguousarray(rope_pos[1], np.int32)).cuda())
    out = torch.full((int(case.cu_q[-1]), case.embed), fill, dtype=torch.float32, device="cuda")
    batch = ops.make_batch(q, k, v, out, case.cu_q, case.cu_k, case.num_heads, case.head_dim, case.scale, case.mask,
                           impl=impl, precision=precision, **rope_kw)
    ops.attn_forward(batch)
    torch.cuda.synchronize()
    return out.cpu().numpy(), batch


def decode_gpu(case: DecodeCase, *, fused_append: bool = True, splits: int = 0, seqs=None):
    """One decode / block-verify step. With fused_append the new rows are passed separately
    and written through by the kernel; otherwise they are placed in the cache beforehand."""
    n, E = case.n_new, case.embed
    kc = torch.from_numpy(case.k_cache).cuda()
    vc = torch.from_numpy(case.v_cache).cuda()
    base = torch.from_numpy(case.base_len).cuda()
    q = torch.from_numpy(case.q).cuda()
    kn = torch.from_numpy(case.k_new).cuda()
    vn = torch.from_numpy(case.v_new).cuda()
    batch = kc.shape[0]
    if not fused_append:
        rows = (base.long()[:, None] + torch.arange(n, device="cuda")[None, :])
        idx = rows[:, :, None].expand(batch, n, E)
        kc.scatter_(1, idx, kn.view(batch, n, E))
        vc.scatter_(1, idx, vn.view(batch, n, E))
    out = torch.full((batch * n, E), float("nan"), dtype=torch.float32, device="cuda")
    d = ops.make_decode(kc, vc, base, q, out, case.num_heads, case.head_dim, n, case.scale, block_mode=case.block_mode,
                        window=case.window, k_new=kn if fused_append else None, v_new=vn if fused_append else None,
                        max_len=int(case.base_len.max()) + n, splits=splits)
    ws = ops.decode_workspace(d)
    ops.attn_decode(d, ws)
    torch.cuda.synchronize()
    return out.cpu().numpy(), kc, vc
