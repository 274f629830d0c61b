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
from helpers import assert_close, oracle_decode

pytestmark = pytest.mark.gpu


def _run_both(case, splits, stream=None):
    """Outputs of the workspace entry point and of the static-scratch entry point for one step.
    splits = 0 leaves the number of key-range pieces to the library. `stream`: a torch stream the
    static call is issued on (the inputs are ready before it starts)."""
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
    assert ws is not None, "the case must exercise the scratch (more than one piece per key range)"
    ops.attn_decode(d_a, ws)
    torch.cuda.synchronize()
    d_b = ops.make_decode(kc, vc, base, q, out_b, case.num_heads, case.head_dim, case.n_new, case.scale, **common)
    L.check(lib.fblt_attn_decode_static(C.byref(d_b), None if stream is None else C.c_void_p(stream.cuda_stream)))
    torch.cuda.synchronize()
    return out_a.cpu().numpy(), out_b.cpu().numpy()


def _check(case, splits, stream=None):
    want_ws, got = _run_both(case, splits, stream)
    assert_close(got, want_ws, "static scratch vs caller workspace")
    want_cpu, _ = oracle_decode(case)                    # and against the CPU operator itself
    assert_close(got, want_cpu, "static scratch vs oracle")


def test_static_scratch_matches_workspace_entry_twice_in_a_row(cuda_lib):
    # two different calls back to back: the second one finds the first one's partials in the array
    first = workloads.decode_case(201, 6, 4, 4, True, lens=[300, 64, 511, 129, 400, 256])
    second = workloads.decode_case(202, 3, 2, 1, False, lens=[500, 77, 260], window=200)
    for case, splits in ((first, 4), (second, 3), (first, 2)):
        _check(case, splits)


def test_static_scratch_with_the_library_choosing_the_split(cuda_lib):
    # few sequences over long caches: left to itself (splits = 0) the library cuts every key range
    # into several pieces, so this is the path a caller gets without tuning anything
    case = workloads.decode_case(203, 2, 4, 4, True, lens=[3000, 1777])
    _check(case, 0)
    _check(case, 0)


def test_static_scratch_on_a_side_stream(cuda_lib):
    side = torch.cuda.Stream()
    case = workloads.decode_case(204, 5, 2, 2, False, lens=[700, 64, 333, 512, 90], window=0)
    _check(case, 4, stream=side)
    _check(case, 2, stream=side)


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
