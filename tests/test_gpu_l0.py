"""L0 drop-in operator (blt_attention_head_core on the CUDA backend) against the oracle."""
from pathlib import Path

import numpy as np
import pytest
import torch

from fblt_b200 import ops
from helpers import assert_close, use_ref
from oracle import binding as ob

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


def run_l0(q, k, v, H, hd, scale, mask=None, is_causal=False, want_weights=False, want_lse=False, fatal=False,
           q_col0=0, k_col0=0, v_col0=0, scratch=False):
    nq, nk = q.shape[0], k.shape[0]
    qd, kd, vd = (torch.from_numpy(np.ascontiguousarray(x)).cuda() for x in (q, k, v))
    md = torch.from_numpy(mask).cuda() if mask is not None else None
    out = torch.zeros((nq, H * hd), dtype=torch.float32, device="cuda")
    weights = torch.full((H, nq, nk), float("nan"), device="cuda") if want_weights else None
    lse = torch.full((H, nq, 2), float("nan"), device="cuda") if want_lse else None
    sc = torch.empty((nq, nk), device="cuda") if scratch else None
    for h in range(H):
        ops.attention_head_core(qd[:, q_col0 + h * hd:], kd[:, k_col0 + h * hd:], vd[:, v_col0 + h * hd:], out,
                                col_offset=h * hd, head_dim=hd, scale=scale, is_causal=is_causal, mask=md,
                                weights_out=weights[h] if want_weights else None,
                                lse_out=lse[h] if want_lse else None, scores_scratch=sc, fatal=fatal)
    torch.cuda.synchronize()
    return (out.cpu().numpy(), weights.cpu().numpy() if want_weights else None,
            lse.cpu().numpy() if want_lse else None)


def oracle_weights(q, k, v, H, hd, scale, mask, is_causal):
    nq, nk = q.shape[0], k.shape[0]
    out = np.zeros((nq, H * hd), np.float32)
    w = np.zeros((H, nq, nk), np.float32)
    jobs = ob.HeadJobs()
    for h in range(H):
        jobs.add(q, k, v, out, col=h * hd, head_dim=hd, q_col=h * hd, k_col=h * hd, v_col=h * hd, scale=scale,
                 mask=mask, is_causal=is_causal, weights_out=w[h])
    jobs.run(1, use_ref())
    return out, w


def test_known_answer(cuda_lib):
    x = np.array([[1, 0, 1, 0], [0, 1, 0, 1]], dtype=np.float32)
    qkv = np.concatenate([x, x, x], axis=1).copy()
    out, _, _ = run_l0(qkv, qkv, qkv, 2, 2, 1 / np.sqrt(2.0), k_col0=4, v_col0=8, scratch=True, fatal=True)
    want = np.array([[0.6697615, 0.3302385, 0.6697615, 0.3302385], [0.3302385, 0.6697615, 0.3302385, 0.6697615]])
    assert np.abs(out - want).max() < 1e-6


def test_golden_head_fixtures(cuda_lib):
    for f in sorted(GOLDEN.glob("head_*.npz")):
        g = np.load(f)
        mask = g["mask"] if "mask" in g.files else None
        out, _, _ = run_l0(g["q"], g["k"], g["v"], int(g["num_heads"]), int(g["head_dim"]), float(g["scale"]),
                           mask=mask, is_causal=bool(g["is_causal"]), scratch=True)
        assert_close(out, g["out"], f.name)


@pytest.mark.parametrize("T", [1, 2, 31, 32, 33, 127, 128, 129])
@pytest.mark.parametrize("hd", [2, 16, 32, 64, 100, 128])
def test_shapes_weights_and_lse(cuda_lib, T, hd):
    rng = np.random.default_rng(T * 1000 + hd)
    H, S = 2, max(1, T + 3 - (T % 5))
    q = rng.standard_normal((T, H * hd)).astype(np.float32)
    k = rng.standard_normal((S, H * hd)).astype(np.float32)
    v = rng.standard_normal((S, H * hd)).astype(np.float32)
    mask = np.where(rng.random((T, S)) < 0.7, 0.0, -np.inf).astype(np.float32)
    mask[0, :] = -np.inf  # all-masked row -> zeros, weights zero
    scale = 1.0 / np.sqrt(hd)
    want, ww = oracle_weights(q, k, v, H, hd, scale, mask, False)
    got, gw, lse = run_l0(q, k, v, H, hd, scale, mask=mask, want_weights=True, want_lse=True)
    assert_close(got, want, "combined")
    assert_close(gw, ww, "weights", atol=1e-6, rtol=1e-4)
    assert (got[0] == 0).all() and (gw[:, 0] == 0).all()
    assert np.isneginf(lse[:, 0, 0]).all() and (lse[:, 0, 1] == 0).all()
    # (m, l): weights = exp(s - m) / l, so every live row has l >= 1
    live = (mask == 0).any(axis=1)
    assert (lse[:, live, 1] >= 1.0 - 1e-5).all()


def test_causal_flag_and_column_isolation(cuda_lib):
    rng = np.random.default_rng(0)
    T, H, hd = 50, 3, 8
    q, k, v = (rng.standard_normal((T, H * hd)).astype(np.float32) for _ in range(3))
    want, _ = oracle_weights(q, k, v, H, hd, 0.3, None, True)
    got, _, _ = run_l0(q, k, v, H, hd, 0.3, is_causal=True, scratch=True)
    assert_close(got, want, "is_causal")
    # only head_dim columns at col_offset may be written (ops/attn_core.h:32)
    qd, kd, vd = (torch.from_numpy(x).cuda() for x in (q, k, v))
    out = torch.full((T, H * hd), 7.0, device="cuda")
    ops.attention_head_core(qd[:, hd:], kd[:, hd:], vd[:, hd:], out, col_offset=hd, head_dim=hd, scale=0.3,
                            is_causal=True, lse_out=torch.empty((T, 2), device="cuda"))
    o = out.cpu().numpy()
    assert (o[:, :hd] == 7.0).all() and (o[:, 2 * hd:] == 7.0).all()
    assert_close(o[:, hd:2 * hd], want[:, hd:2 * hd], "head 1")


def test_additive_bias_and_nonfinite_inputs(cuda_lib):
    rng = np.random.default_rng(1)
    T, S, hd = 20, 30, 16
    q, k, v = rng.standard_normal((T, hd)).astype(np.float32), rng.standard_normal((S, hd)).astype(np.float32), \
        rng.standard_normal((S, hd)).astype(np.float32)
    mask = rng.standard_normal((T, S)).astype(np.float32)
    mask[3, 4] = np.inf      # non-finite entries carry weight 0 (ops/vecmath_cpu.c:33-52)
    mask[5, 6] = np.nan
    want, ww = oracle_weights(q, k, v, 1, hd, 0.25, mask, False)
    got, gw, _ = run_l0(q, k, v, 1, hd, 0.25, mask=mask, want_weights=True)
    assert_close(got, want, "bias")
    assert gw[0, 3, 4] == 0 and gw[0, 5, 6] == 0
    assert_close(gw, ww, "weights", atol=1e-6, rtol=1e-4)


def test_long_row_uses_caller_scratch(cuda_lib):
    rng = np.random.default_rng(2)
    T, S, hd = 3, 60000, 8
    q = rng.standard_normal((T, hd)).astype(np.float32)
    k = rng.standard_normal((S, hd)).astype(np.float32)
    v = rng.standard_normal((S, hd)).astype(np.float32)
    want, _ = oracle_weights(q, k, v, 1, hd, 0.35, None, False)
    got, _, _ = run_l0(q, k, v, 1, hd, 0.35, scratch=True)
    assert_close(got, want, "nk=60000")
