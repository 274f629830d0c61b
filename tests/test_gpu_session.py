"""Host-buffer sessions: the call a host program without device memory makes."""
import numpy as np
import pytest
import torch

from fblt_b200 import lib as L
from fblt_b200 import ops, workloads
from helpers import assert_close, oracle_decode, oracle_forward

pytestmark = pytest.mark.gpu


def test_session_forward_packed_and_cross(cuda_lib):
    case = workloads.c2_patch_attention(batch=5)
    want, _, _ = oracle_forward(case)
    rows, E = int(case.cu_q[-1]), case.embed
    s = ops.Session(8, case.num_heads, case.head_dim, max_q_rows=rows, max_k_rows=rows)
    out = np.full((rows, E), np.nan, dtype=np.float32)
    s.forward(case.q, case.k, case.v, out, case.cu_q, case.cu_k, case.scale, case.mask)   # views of one [T, 3E] buffer
    assert_close(out, want, "session packed")
    s.close()
    for direction in ("enc", "dec_paper", "dec_leq"):
        c = workloads.c3_cross_attention(direction, batch=3)
        want, _, _ = oracle_forward(c)
        s = ops.Session(4, c.num_heads, c.head_dim, max_q_rows=int(c.cu_q[-1]), max_k_rows=int(c.cu_k[-1]))
        out = np.full((int(c.cu_q[-1]), c.embed), np.nan, dtype=np.float32)
        s.forward(c.q, c.k, c.v, out, c.cu_q, c.cu_k, c.scale, c.mask)
        assert_close(out, want, "session " + direction)
        with pytest.raises(L.FbltError) as e:
            big = workloads.c3_cross_attention(direction, batch=5)
            s.forward(big.q, big.k, big.v, np.zeros((int(big.cu_q[-1]), big.embed), np.float32), big.cu_q, big.cu_k,
                      big.scale, big.mask)
        assert e.value.status == L.ERR_CAPACITY
        s.close()


def test_session_decode_steps_and_rollback(cuda_lib):
    base = np.array([10, 64, 200, 33], dtype=np.int32)
    n, steps = 4, 3
    case = workloads.decode_case(120, 4, 4, n, True, lens=base, cache_rows=256)
    E = case.embed
    s = ops.Session(4, 4, 64, cache_rows=256, max_new=8)
    s.cache_load(base, case.k_cache, case.v_cache, 256)
    rng = np.random.default_rng(3)
    lens = base.copy()
    for step in range(steps):
        advance = n if step != 1 else 2        # step 1 keeps only two of the four drafted rows
        case.base_len = lens.copy()
        case.q, case.k_new, case.v_new = (rng.standard_normal((4 * n, E)).astype(np.float32) for _ in range(3))
        want, _ = oracle_decode(case)
        out = np.full((4 * n, E), np.nan, dtype=np.float32)
        s.decode(4, n, case.q, case.k_new, case.v_new, out, case.scale, block_mode=True, advance=advance)
        assert_close(out, want, f"session decode step {step}")
        for b in range(4):                      # host mirror of the cache, with the same rollback
            case.k_cache[b, lens[b]:lens[b] + n] = case.k_new[b * n:(b + 1) * n]
            case.v_cache[b, lens[b]:lens[b] + n] = case.v_new[b * n:(b + 1) * n]
        lens += advance
        assert (s.cache_lens(4) == lens).all()
    # plain one-byte causal decode with a window on the same cache
    case.n_new, case.block_mode, case.window, case.base_len = 1, False, 24, lens.copy()
    case.q, case.k_new, case.v_new = (rng.standard_normal((4, E)).astype(np.float32) for _ in range(3))
    want, _ = oracle_decode(case)
    out = np.full((4, E), np.nan, dtype=np.float32)
    s.decode(4, 1, case.q, case.k_new, case.v_new, out, case.scale, window=24)
    assert_close(out, want, "session decode n=1 window")
    with pytest.raises(L.FbltError) as e:
        s.decode(4, 9, case.q, case.k_new, case.v_new, out, case.scale)
    assert e.value.status == L.ERR_CAPACITY
    # per-sequence truncate: roll every sequence back by a different amount and decode again
    for b in range(4):
        case.k_cache[b, lens[b]] = case.k_new[b]
        case.v_cache[b, lens[b]] = case.v_new[b]
    lens = lens + 1 - np.array([0, 3, 50, 7], dtype=np.int32)
    s.cache_truncate(lens)
    assert (s.cache_lens(4) == lens).all()
    case.base_len = lens.copy()
    case.q, case.k_new, case.v_new = (rng.standard_normal((4, E)).astype(np.float32) for _ in range(3))
    want, _ = oracle_decode(case)
    s.decode(4, 1, case.q, case.k_new, case.v_new, out, case.scale, window=24)
    assert_close(out, want, "session decode after truncate")
    with pytest.raises(L.FbltError) as e:
        s.cache_truncate([0, 0, 257, 0])
    assert e.value.status == L.ERR_CAPACITY
    s.cache_reset()
    assert (s.cache_lens(4) == 0).all()
    s.close()


def test_session_decode_steps_pipeline_equals_single_steps(cuda_lib):
    """The overlapped multi-step call must return what the same steps give one at a time."""
    base = np.array([7, 64, 130], dtype=np.int32)
    n, steps, B = 4, 5, 3
    case = workloads.decode_case(121, B, 4, n, True, lens=base, cache_rows=192)
    E = case.embed
    rng = np.random.default_rng(9)
    q_all, k_all, v_all = (rng.standard_normal((steps, B * n, E)).astype(np.float32) for _ in range(3))
    outs = []
    for pipelined in (False, True):
        s = ops.Session(B, 4, 64, cache_rows=192, max_new=n)
        s.cache_load(base, case.k_cache, case.v_cache, 192)
        out = np.full((steps, B * n, E), np.nan, dtype=np.float32)
        if pipelined:
            s.decode_steps(B, n, steps, q_all, k_all, v_all, out, case.scale, in_step_stride=B * n * E,
                           out_step_stride=B * n * E, block_mode=True, advance=3)
        else:
            for t in range(steps):
                s.decode(B, n, q_all[t], k_all[t], v_all[t], out[t], case.scale, block_mode=True, advance=3)
        assert (s.cache_lens(B) == base + steps * 3).all()
        outs.append(out)
        s.close()
    assert np.isfinite(outs[1]).all()
    assert outs[0].tobytes() == outs[1].tobytes()
    # and step 0 against the oracle
    case.q, case.k_new, case.v_new = q_all[0], k_all[0], v_all[0]
    want, _ = oracle_decode(case)
    assert_close(outs[1][0], want, "pipelined step 0")


def test_session_forward_async_equals_blocking(cuda_lib):
    """The non-blocking forward call followed by other session work and wait() returns the same rows."""
    case = workloads.c5_prefill(batch=6)
    E = case.embed
    lens = np.array([5, 9, 0, 33, 64, 7], dtype=np.int32)
    dcase = workloads.decode_case(140, 6, case.num_heads, 4, True, lens=lens, cache_rows=128)
    outs = []
    for wait in (True, False):
        s = ops.Session(6, case.num_heads, 64, max_q_rows=case.q.shape[0], max_k_rows=case.k.shape[0], cache_rows=128,
                        max_new=4)
        out = np.full((case.q.shape[0], E), np.nan, dtype=np.float32)
        s.forward(case.q, case.k, case.v, out, case.cu_q, case.cu_k, case.scale, case.mask, wait=wait)
        s.cache_load(lens, dcase.k_cache, dcase.v_cache, 128)        # runs beside the download when wait=False
        s.wait()
        assert np.isfinite(out).all()
        outs.append(out)
        s.close()
    assert outs[0].tobytes() == outs[1].tobytes()
    want, _, _ = oracle_forward(case)
    assert_close(outs[1], want, "async session forward")
