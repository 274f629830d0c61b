"""Helpers for the gpu-marked tests: run a workload case through the C ABI on cuda:0."""
from __future__ import annotations

import numpy as np
import torch

from fblt_b200 import lib as L
from fblt_b200 import ops
from fblt_b200.workloads import DecodeCase, ForwardCase


# Output buffers sit between guard rows holding a sentinel; a kernel that writes outside the rows it
# owns is caught here even when the result rows themselves are right.
GUARD_ROWS, SENTINEL = 8, 12345.678


def guarded_rows(rows: int, cols: int, fill: float):
    buf = torch.full((rows + 2 * GUARD_ROWS, cols), SENTINEL, dtype=torch.float32, device="cuda")
    view = buf[GUARD_ROWS:GUARD_ROWS + rows]
    view.fill_(fill)
    return buf, view


def check_guards(buf: torch.Tensor, what: str) -> None:
    sent = torch.tensor(SENTINEL, dtype=torch.float32, device=buf.device)
    ok = bool((buf[:GUARD_ROWS] == sent).all()) and bool((buf[-GUARD_ROWS:] == sent).all())
    assert ok, f"{what}: rows outside the output were written"


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
    guard, out = guarded_rows(int(case.cu_q[-1]), case.embed, fill)
    batch = ops.make_batch(q, k, v, out, case.cu_q, case.cu_k, case.num_heads, case.head_dim, case.scale, case.mask,
                           impl=impl, precision=precision, **rope_kw)
    ops.attn_forward(batch)
    torch.cuda.synchronize()
    check_guards(guard, f"forward impl={impl}")
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
    guard, out = guarded_rows(batch * n, E, float("nan"))
    kc_before, vc_before = (kc.clone(), vc.clone()) if fused_append else (None, None)
    d = ops.make_decode(kc, vc, base, q, out, case.num_heads, case.head_dim, n, case.scale, block_mode=case.block_mode,
                        window=case.window, k_new=kn if fused_append else None, v_new=vn if fused_append else None,
                        max_len=int(case.base_len.max()) + n, splits=splits)
    ws = ops.decode_workspace(d)
    ops.attn_decode(d, ws)
    torch.cuda.synchronize()
    check_guards(guard, "decode")
    if fused_append:
        # the write-through touches cache rows base .. base + n of every sequence and nothing else
        rows = torch.arange(kc.shape[1], device="cuda")[None, :]
        lo = base.long()[:, None]
        untouched = ((rows < lo) | (rows >= lo + n))[:, :, None].expand_as(kc)
        same = lambda a, b: bool((a.view(torch.int32)[untouched] == b.view(torch.int32)[untouched]).all())  # bit patterns
        assert same(kc, kc_before), "K cache rows outside the appended block changed"
        assert same(vc, vc_before), "V cache rows outside the appended block changed"
    return out.cpu().numpy(), kc, vc
