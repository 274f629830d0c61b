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


def test_dv_commit_matches_host_loop(cuda_lib):
    """fblt_dv_commit against the reference's host loop run one sequence at a time: the verifier's rows
    start at each sequence's own cache length, bytes / lengths / accepted counts / cache roll-back
    must match exactly."""
    rng = np.random.default_rng(21)
    batch, V, xw = 257, 256, 64
    o = ob.oracle()
    l = rng.integers(1, 24, batch).astype(np.int32)
    r = rng.integers(0, 9, batch).astype(np.int32)
    cache = (l - 1 - rng.integers(0, 2, batch)).clip(0).astype(np.int32)   # last byte's row pending, or one more
    target = (l + r + rng.integers(0, 2, batch)).astype(np.int32)
    width = int((l + r - cache).max())
    x = rng.integers(0, 256, (batch, xw), dtype=np.uint8)
    absolute = rng.standard_normal((batch, xw, V)).astype(np.float32)       # logits by absolute position
    absolute[::7] = np.round(absolute[::7] * 2) / 2                          # ties: lowest index wins
    pred = np.stack([oracle_argmax(absolute[c]) for c in range(batch)])
    for c in range(batch):
        keep = rng.integers(0, r[c] + 2)
        for p in range(l[c], min(l[c] + keep, l[c] + r[c])):
            x[c, p] = pred[c, p - 1]
    want_x, want_len, want_acc = x.copy(), np.zeros(batch, np.int32), np.zeros(batch, np.int32)
    for c in range(batch):
        acc = C.c_size_t(0)
        row = np.ascontiguousarray(want_x[c])
        want_len[c] = o.oracle_verify_accept(row.ctypes.data_as(C.POINTER(C.c_uint8)),
                                             np.ascontiguousarray(absolute[c]).ctypes.data_as(ob.c_f_p), V, int(l[c]),
                                             int(r[c]), int(target[c]), C.byref(acc))
        want_x[c], want_acc[c] = row, acc.value
    # what the verifier hands over: `width` rows per sequence starting at its cache length
    rel = np.zeros((batch, width, V), np.float32)
    for c in range(batch):
        n = min(width, xw - cache[c])
        rel[c, :n] = absolute[c, cache[c]:cache[c] + n]
    xd, ld, cd = torch.from_numpy(x.copy()).cuda(), torch.from_numpy(l.copy()).cuda(), torch.from_numpy(cache.copy()).cuda()
    acc_d = ops.dv_commit(torch.from_numpy(rel).cuda().view(batch * width, V), width, xd, ld, torch.from_numpy(r).cuda(),
                          torch.from_numpy(target).cuda(), cd)
    assert (acc_d.cpu().numpy() == want_acc).all()
    assert (ld.cpu().numpy() == want_len).all()
    assert (xd.cpu().numpy() == want_x).all()
    assert (cd.cpu().numpy() == l + want_acc).all()             # roll-back point: rows computed from bytes that stayed
    # a sequence whose rows do not cover its drafts is left alone and flagged
    bad_cache = torch.from_numpy((l + 1).astype(np.int32)).cuda()
    x2, l2 = torch.from_numpy(x.copy()).cuda(), torch.from_numpy(l.copy()).cuda()
    flagged = ops.dv_commit(torch.from_numpy(rel).cuda().view(batch * width, V), width, x2, l2, torch.from_numpy(r).cuda(),
                            torch.from_numpy(target).cuda(), bad_cache)
    assert (flagged.cpu().numpy() == -1).all() and (x2.cpu().numpy() == x).all() and (l2.cpu().numpy() == l).all()


def _dv_generate(seqs, prompts, steps, B, tables, cache_rows=160):
    """A toy generation loop of draft -> verify -> commit rounds for the sequences `seqs` as ONE batch,
    everything on the device between rounds: K / V / Q rows of a byte are table rows of that byte plus
    a position term, the verifier is cache attention (causal, fblt_attn_decode with write-through)
    followed by a projection to 256 logits (fblt_matmul), the commit is fblt_dv_commit, which also rolls
    the cache lengths back. Drafts are wrong on purpose every few positions, so roll-backs happen."""
    H, hd, V = 2, 64, 256
    E = H * hd
    ek, ev, eq, pos, w_head = tables
    n = len(seqs)
    xw = 8 + steps * (B + 1) + B + 8
    x = torch.zeros((n, xw), dtype=torch.uint8, device="cuda")
    for i, s in enumerate(seqs):
        x[i, :len(prompts[s])] = torch.tensor(list(prompts[s]), dtype=torch.uint8)
    l = torch.tensor([len(prompts[s]) for s in seqs], dtype=torch.int32, device="cuda")
    cache_len = torch.zeros(n, dtype=torch.int32, device="cuda")
    target = torch.full((n,), xw - 1, dtype=torch.int32, device="cuda")
    kc = torch.zeros((n, cache_rows, E), device="cuda")
    vc = torch.zeros((n, cache_rows, E), device="cuda")
    head = ops.PackedWeights(w_head)
    seq_id = torch.tensor(seqs, device="cuda")
    width = B + 3   # rows per sequence and pass: the pending byte (or the prompt) plus the drafts; the same
    #                 count in every run, so that a sequence meets the same kernel alone and in a batch
    ar = torch.arange(n, device="cuda")

    def verifier_rows():
        """Logits of the rows at positions cache_len .. cache_len + width - 1 of every sequence."""
        p_rows = cache_len.long()[:, None] + torch.arange(width, device="cuda")[None, :]
        byte = x.gather(1, p_rows.clamp(max=xw - 1)).long()
        q = (eq[byte] + pos[p_rows]).view(n * width, E).contiguous()
        k = (ek[byte] + pos[p_rows]).view(n * width, E).contiguous()
        v = ev[byte].view(n * width, E).contiguous()
        out = torch.empty_like(q)
        d = ops.make_decode(kc, vc, cache_len, q, out, H, hd, width, 0.125, block_mode=False, k_new=k, v_new=v,
                            max_len=cache_rows, splits=1)
        ops.attn_decode(d, None)
        return ops.matmul(out, head)

    for step in range(steps):
        r = torch.full((n,), B, dtype=torch.int32, device="cuda")
        # drafter: greedy bytes from the same model, one at a time (the cache lengths do not move, so the
        # rows these passes write are overwritten later), then spoiled at a position that depends on
        # the sequence and the round -- some rounds keep every draft, most are cut short
        for i in range(B):
            pred = ops.argmax_rows(verifier_rows()).view(n, width)
            at = (l + i - 1 - cache_len).long()
            x[ar, (l + i).long()] = pred[ar, at].to(torch.uint8)
        spoil = (seq_id * 3 + step) % (B + 2)
        hit = spoil < B
        x[ar[hit], (l.long() + spoil)[hit]] ^= 0x55
        ops.dv_commit(verifier_rows(), width, x, l, r, target, cache_len)
    torch.cuda.synchronize()
    return x.cpu().numpy(), l.cpu().numpy(), cache_len.cpu().numpy()


def test_dv_rounds_batched_equal_one_at_a_time(cuda_lib):
    """Draft -> verify -> accept -> roll back per row (infer/block_generation.c:405-453) for a batch of
    independent sequences gives byte-identical output to running each sequence alone."""
    g = torch.Generator(device="cuda").manual_seed(9)
    E, V = 128, 256
    tables = (torch.randn((256, E), device="cuda", generator=g), torch.randn((256, E), device="cuda", generator=g),
              torch.randn((256, E), device="cuda", generator=g), 0.3 * torch.randn((512, E), device="cuda", generator=g),
              torch.randn((E, V), device="cuda", generator=g))
    prompts = [bytes([65 + s, 66, 67 + 2 * s][: 1 + s % 3]) for s in range(9)]
    seqs = list(range(9))
    xb, lb, cb = _dv_generate(seqs, prompts, steps=7, B=4, tables=tables)
    gained = lb - np.array([len(p) for p in prompts])
    assert (gained >= 7).all() and gained.max() >= 7 * 2                  # every round commits; some keep several drafts
    assert len(set(gained.tolist())) > 1                                  # and the rows advance by different amounts
    for s in seqs:
        x1, l1, c1 = _dv_generate([s], prompts, steps=7, B=4, tables=tables)
        assert l1[0] == lb[s] and c1[0] == cb[s]
        assert x1[0, :l1[0]].tobytes() == xb[s, :lb[s]].tobytes(), f"sequence {s}"
