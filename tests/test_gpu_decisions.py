"""Decision step: argmax tie rule and accept-until-mismatch must equal the host reference
logic exactly (integer / compare results, no tolerance)."""
import ctypes as C

import numpy as np
import pytest
import torch

from fblt_b200 import ops, workloads
from gpu_utils import decode_gpu
from helpers import oracle_decode
from oracle import binding as ob

pytestmark = pytest.mark.gpu


def oracle_argmax(logits: np.ndarray) -> np.ndarray:
    o = ob.oracle()
    return np.array([o.oracle_argmax_row(np.ascontiguousarray(r).ctypes.data_as(ob.c_f_p), len(r)) for r in logits],
                    dtype=np.int32)


def test_argmax_tie_rule_bit_exact(cuda_lib):
    rng = np.random.default_rng(0)
    for vocab in (1, 2, 31, 32, 33, 256, 260):
        x = rng.standard_normal((200, vocab)).astype(np.float32)
        x[::3] = np.round(x[::3] * 2) / 2            # many exact ties
        x[5, :] = 1.0                                # all equal -> index 0
        x[6, :] = -np.inf
        if vocab > 2:
            x[7, 1] = np.nan                         # NaN never wins
            x[8, 0] = np.nan                         # NaN in slot 0 -> 0 (strict '>' scan)
            x[9, vocab - 1] = np.inf
        got = ops.argmax_rows(torch.from_numpy(x).cuda()).cpu().numpy()
        assert (got == oracle_argmax(x)).all(), vocab
    big = rng.standard_normal((64, 300)).astype(np.float32)
    view = torch.from_numpy(big).cuda()[:, :256]      # row stride != vocab
    assert (ops.argmax_rows(view).cpu().numpy() == oracle_argmax(big[:, :256])).all()


def test_verify_accept_matches_host_loop(cuda_lib):
    rng = np.random.default_rng(1)
    batch, V, width = 300, 256, 48
    o = ob.oracle()
    x = rng.integers(0, 256, (batch, width), dtype=np.uint8)
    logits = rng.standard_normal((batch, width, V)).astype(np.float32)
    l = rng.integers(1, 20, batch).astype(np.int32)
    r = rng.integers(0, 17, batch).astype(np.int32)
    target = (l + r + rng.integers(0, 2, batch)).astype(np.int32)
    pred = np.stack([oracle_argmax(logits[c]) for c in range(batch)])
    # make most drafts agree with the prediction for a random prefix
    for c in range(batch):
        keep = rng.integers(0, r[c] + 2)
        for p in range(l[c], min(l[c] + keep, l[c] + r[c])):
            x[c, p] = pred[c, p - 1]
    want_x, want_len, want_acc = x.copy(), np.zeros(batch, np.int32), np.zeros(batch, np.int32)
    for c in range(batch):
        acc = C.c_size_t(0)
        row = np.ascontiguousarray(want_x[c])
        want_len[c] = o.oracle_verify_accept(row.ctypes.data_as(C.POINTER(C.c_uint8)),
                                             np.ascontiguousarray(logits[c]).ctypes.data_as(ob.c_f_p), V, int(l[c]),
                                             int(r[c]), int(target[c]), C.byref(acc))
        want_x[c] = row
        want_acc[c] = acc.value
    xd = torch.from_numpy(x.copy()).cuda()
    # device path: argmax on the device, then the accept kernel
    pred_d = ops.argmax_rows(torch.from_numpy(logits).cuda().view(batch * width, V)).view(batch, width)
    assert (pred_d.cpu().numpy() == pred).all()
    new_len, accepted = ops.verify_accept(xd, pred_d, torch.from_numpy(l).cuda(), torch.from_numpy(r).cuda(),
                                          torch.from_numpy(target).cuda())
    assert (new_len.cpu().numpy() == want_len).all()
    assert (accepted.cpu().numpy() == want_acc).all()
    assert (xd.cpu().numpy() == want_x).all()


def test_argmax_over_attention_outputs_agrees_with_cpu(cuda_lib):
    """CPU-vs-GPU decisions on identical seeded inputs: project the block-verify attention
    output to 256 logits on the host for both paths and compare the argmax bytes. fp32
    reassociation can flip near-ties only; any disagreement must sit on a top-2 margin below
    the attention tolerance."""
    case = workloads.decode_case(7, 64, 4, 4, True, lens=np.full(64, 200))
    want, _ = oracle_decode(case)
    got, _, _ = decode_gpu(case)
    w = np.random.default_rng(2).standard_normal((case.embed, 256)).astype(np.float32) / 16
    lw, lg = want @ w, got @ w
    aw = oracle_argmax(lw)
    ag = ops.argmax_rows(torch.from_numpy(lg).cuda()).cpu().numpy()
    diff = np.nonzero(aw != ag)[0]
    for i in diff:
        top2 = np.sort(lw[i])[-2:]
        assert top2[1] - top2[0] < 1e-3, f"row {i}: argmax differs with margin {top2[1] - top2[0]}"
    assert len(diff) <= 2


def oracle_unmask_round(logits, masked, tokens, B, strategy, thr):
    """Host loop of infer/block_generation.c:229-252 over the oracle's functions."""
    o = ob.oracle()
    batch = masked.shape[0]
    conf = np.zeros((batch, B), np.float32)
    ent = np.zeros((batch, B), np.float32)
    sel = np.zeros(batch, np.int64)
    for c in range(batch):
        pred = np.zeros(B, np.int32)
        for b in range(B):
            row = np.ascontiguousarray(logits[c * B + b])
            pm, en = C.c_float(), C.c_float()
            o.oracle_row_analyze(row.ctypes.data_as(ob.c_f_p), len(row), C.byref(pm), C.byref(en))
            conf[c, b], ent[c, b] = pm.value, en.value
            pred[b] = o.oracle_argmax_row(row.ctypes.data_as(ob.c_f_p), len(row))
        m = np.ascontiguousarray(masked[c])
        mp = m.ctypes.data_as(C.POINTER(C.c_uint8))
        if strategy == 0:
            s = o.oracle_unmask_select_confidence(conf[c].ctypes.data_as(ob.c_f_p), mp, B, thr)
        else:
            s = o.oracle_unmask_select_eb(ent[c].ctypes.data_as(ob.c_f_p), mp, B, thr)
        sel[c] = s
        for b in range(B):
            if s & (1 << b):
                tokens[c, b] = pred[b]
                masked[c, b] = 0
    return sel, conf, ent


@pytest.mark.parametrize("strategy,thr", [(0, 0.3), (0, 2.0), (1, 2.5), (1, 0.0)])
def test_unmask_step_matches_host_loop(cuda_lib, strategy, thr):
    """Rounds of the drafter's unmask loop on the device against the host loop: statistics to
    float rounding of a double accumulation, selections / bytes / masks exactly."""
    rng = np.random.default_rng(17 + strategy)
    for B, V in ((1, 256), (4, 260), (16, 256), (32, 300)):
        batch = 37
        masked = (rng.random((batch, B)) < 0.8).astype(np.uint8)
        masked[0] = 0                                   # nothing left to choose
        masked[1] = 1
        tokens = rng.integers(0, 256, (batch, B)).astype(np.uint8)
        m_d, t_d = torch.from_numpy(masked.copy()).cuda(), torch.from_numpy(tokens.copy()).cuda()
        for rnd in range(3):
            sharp = rng.random((batch * B, 1)).astype(np.float32) * 6
            logits = (rng.standard_normal((batch * B, V)).astype(np.float32) * sharp).astype(np.float32)
            logits[3] = 0.25                            # uniform row: p_max = 1/V, entropy = ln V, argmax 0
            want_sel, want_conf, want_ent = oracle_unmask_round(logits, masked, tokens, B, strategy, thr)
            sel, conf, ent, left = ops.unmask_step(torch.from_numpy(logits).cuda(), m_d, t_d, strategy, thr)
            np.testing.assert_allclose(conf.cpu().numpy(), want_conf, rtol=2e-6, atol=1e-9)
            np.testing.assert_allclose(ent.cpu().numpy(), want_ent, rtol=2e-6, atol=1e-7)
            assert (sel.cpu().numpy() == want_sel).all(), (B, V, rnd)
            assert (m_d.cpu().numpy() == masked).all() and (t_d.cpu().numpy() == tokens).all()
            assert (left.cpu().numpy() == masked.sum(axis=1)).all()
