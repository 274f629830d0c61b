"""The allocation-free decode entry point (fblt_attn_decode_static): for callers that cannot
allocate device memory in the middle of a generation -- everything they own sits in an arena
sized at start-up, or they run a latency-bound loop where cudaMalloc's device-wide
synchronisation is not acceptable. Its split-K partials live in a fixed array inside the
library, so it must give the same result as the workspace-taking entry point, also when
called twice in a row (the array is shared and keeps the previous call's contents).

Collected last on purpose: a run that stops at the first failure has then already run
everything else."""
import ctypes as C

import numpy as np
import pytest
import torch

from fblt_b200 import lib as L
from fblt_b200 import ops, workloads

pytestmark = pytest.mark.gpu


def _run_both(case, splits):
    lib = L.load()
    kc, vc = torch.from_numpy(case.k_cache).cuda(), torch.from_numpy(case.v_cache).cuda()
    base, q = torch.from_numpy(case.base_len).cuda(), torch.from_numpy(case.q).cuda()
    kn, vn = torch.from_numpy(case.k_new).cuda(), torch.from_numpy(case.v_new).cuda()
    out_a = torch.full_like(q, float("nan"))
    out_b = torch.full_like(q, float("nan"))
    common = dict(block_mode=case.block_mode, window=case.window, k_new=kn, v_new=vn,
                  max_len=int(case.base_len.max()) + case.n_new, splits=splits)
    d_a = ops.make_decode(kc, vc, base, q, out_a, case.num_heads, case.head_dim, case.n_new, case.scale, **common)
    ws = ops.decode_workspace(d_a)
    assert ws is not None, "the case must exercise the scratch (splits > 1)"
    ops.attn_decode(d_a, ws)
    d_b = ops.make_decode(kc, vc, base, q, out_b, case.num_heads, case.head_dim, case.n_new, case.scale, **common)
    L.check(lib.fblt_attn_decode_static(C.byref(d_b), None))
    torch.cuda.synchronize()
    return out_a.cpu().numpy(), out_b.cpu().numpy()


def test_static_scratch_matches_workspace_entry_twice_in_a_row(cuda_lib):
    # two different calls back to back: the second one finds the first one's partials in the array
    first = workloads.decode_case(201, 6, 4, 4, True, lens=[300, 64, 511, 129, 400, 256])
    second = workloads.decode_case(202, 3, 2, 1, False, lens=[500, 77, 260], window=200)
    for case, splits in ((first, 4), (second, 3), (first, 2)):
        want, got = _run_both(case, splits)
        assert np.isfinite(got).all()
        err = np.abs(got - want)
        assert (err <= 1e-4 + 1e-3 * np.abs(want)).all(), f"max abs err {err.max():.3e}"


def test_static_scratch_rejects_oversized_requests(cuda_lib):
    lib = L.load()
    cap = lib.fblt_attn_decode_static_capacity()
    assert cap == 4 << 20
    B, H, n, rows = 256, 16, 4, 520
    kc = torch.zeros((B, rows, H * 64), device="cuda")
    base = torch.full((B,), 512, dtype=torch.int32, device="cuda")
    q = torch.zeros((B * n, H * 64), device="cuda")
    d = ops.make_decode(kc, kc, base, q, torch.empty_like(q), H, 64, n, 0.125, block_mode=True, max_len=516, splits=4)
    assert lib.fblt_attn_decode_workspace(C.byref(d)) > cap
    assert lib.fblt_attn_decode_static(C.byref(d), None) == L.ERR_LIMIT
    assert b"built-in scratch" in lib.fblt_last_error()
    d.splits = 1                                   # no partials: always fits
    L.check(lib.fblt_attn_decode_static(C.byref(d), None))
    torch.cuda.synchronize()
