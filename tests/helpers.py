"""Shared test plumbing: dense masks and CPU results from the oracle for a workload case."""
from __future__ import annotations

import numpy as np

from fblt_b200 import lib as L
from fblt_b200.workloads import DecodeCase, ForwardCase
from oracle import binding as ob

# fp32 parity bar of the attention path: |gpu - ref| <= ATOL + RTOL * |ref|
ATOL, RTOL = 1e-4, 1e-3


def use_ref() -> bool:
    """Prefer the reference's own object code when it was built (oracle/_ref)."""
    return ob.have_ref()


def assert_close(got: np.ndarray, want: np.ndarray, what: str = "", atol: float = ATOL, rtol: float = RTOL):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    err = np.abs(got - want)
    bound = atol + rtol * np.abs(want)
    bad = err > bound
    assert not bad.any(), (f"{what}: {int(bad.sum())} of {bad.size} outside tolerance; max abs err {err.max():.3e} "
                           f"at {np.unravel_index(err.argmax(), err.shape)}")
    return float(err.max())


def dense_masks(case: ForwardCase, ref: bool = False):
    """One dense additive mask per sequence, built by the reference's mask builder (or the
    restatement) from the case's MaskConfig; rules the builder cannot express are written as
    host loops, the way infer/kv_cache.c:220-251 builds its own."""
    m = case.mask
    out = []
    for b in range(len(case.cu_q) - 1):
        nq = int(case.cu_q[b + 1] - case.cu_q[b])
        nk = int(case.cu_k[b + 1] - case.cu_k[b])
        if nq == 0 or nk == 0:
            out.append(np.full((nq, nk), -np.inf, dtype=np.float32))
            continue
        off = int(m.causal_offset[b]) if m.causal_offset is not None else 0
        docs = m.doc_bounds[b] if m.doc_bounds is not None and len(m.doc_bounds[b]) else None
        k = m.subtokens
        if m.num_clean is not None and m.group_rule == L.GROUP_NONE:
            mask, _ = ob.block_diffusion_mask(1, nq, int(m.num_clean[b]), use_ref=ref)
        elif m.group_rule == L.GROUP_NONE:
            mask, _ = ob.build_mask(nq, nk, window=m.sliding_window, doc_boundaries=docs, is_causal=m.is_causal,
                                    causal_offset=off, use_ref=ref)
        elif m.group_rule == L.GROUP_IDS:
            qg = m.q_group_ids[case.cu_q[b]:case.cu_q[b + 1]]
            kg = m.k_group_ids[case.cu_k[b]:case.cu_k[b + 1]]
            mask, _ = ob.build_mask(nq, nk, window=m.sliding_window, doc_boundaries=docs, q_groups=qg, k_groups=kg,
                                    bidirectional=m.bidirectional_within_group, is_causal=m.is_causal,
                                    causal_offset=off, use_ref=ref)
        else:
            bounds = m.patch_bounds[b]
            P = len(bounds) - 1
            qpos = int(m.q_pos_offset[b]) if m.q_pos_offset is not None else 0
            if m.group_rule == L.GROUP_PATCH_ENC:
                _, byte_patch = ob.patch_group_ids(bounds, use_ref=ref)
                qg = np.arange(nq) // k
                mask, _ = ob.build_mask(nq, nk, q_groups=qg, k_groups=byte_patch[:nk],
                                        bidirectional=m.bidirectional_within_group, use_ref=ref)
            elif m.group_rule == L.GROUP_PATCH_DEC:
                qg = np.array([ob.latent_at(bounds, qpos + i, use_ref=ref) for i in range(nq)])
                # block-diffusion cross-attention (models/block_diffusion.c:164-186): the clean prefix ends
                # at num_clean, the drafted rows behind it read the last latent
                n_clean = int(m.num_clean[b]) if m.num_clean is not None else nq
                qg[n_clean:] = P - 1
                if m.trailing_closed is not None and m.trailing_closed[b] and n_clean > 0:
                    qg[n_clean - 1] = P - 1
                kg = np.arange(nk) // k
                mask, _ = ob.build_mask(nq, nk, q_groups=qg, k_groups=kg,
                                        bidirectional=m.bidirectional_within_group, use_ref=ref)
            else:  # PATCH_LEQ: key patch <= the byte's patch (no reference builder for "<=")
                pos = qpos + np.arange(nq)
                patch = np.clip(np.searchsorted(bounds, pos, side="right") - 1, 0, P - 1)
                kg = np.arange(nk) // k
                allowed = kg[None, :] <= patch[:, None]
                mask = np.where(allowed, 0.0, -np.inf).astype(np.float32)
        out.append(np.ascontiguousarray(mask))
    return out


def oracle_forward(case: ForwardCase, nthreads: int = 0, ref: bool | None = None):
    ref = use_ref() if ref is None else ref
    masks = dense_masks(case, ref)
    # an all-masked row is legal for the operator (zeros) even though the builder would abort
    out, secs = ob.batched_attention(case.q, case.k, case.v, case.cu_q, case.cu_k, case.num_heads, case.head_dim,
                                     case.scale, masks, use_ref=ref, nthreads=nthreads)
    return out, masks, secs


def oracle_decode(case: DecodeCase, nthreads: int = 0, ref: bool | None = None, seqs=None):
    """CPU result of one decode / block-verify step: per sequence, K/V = cache rows [0, base)
    followed by the n_new appended rows, mask from the incremental decoder's host loop
    (infer/kv_cache.c:225-236) or all-visible for block rows."""
    ref = use_ref() if ref is None else ref
    E, n = case.embed, case.n_new
    batch = len(case.base_len)
    seqs = range(batch) if seqs is None else seqs
    out = np.zeros((batch * n, E), dtype=np.float32)
    jobs = ob.HeadJobs()
    for b in seqs:
        base = int(case.base_len[b])
        kk = np.ascontiguousarray(np.concatenate([case.k_cache[b, :base], case.k_new[b * n:(b + 1) * n]]))
        vv = np.ascontiguousarray(np.concatenate([case.v_cache[b, :base], case.v_new[b * n:(b + 1) * n]]))
        if case.block_mode:
            mask = np.zeros((n, base + n), dtype=np.float32)
        else:
            mask = ob.decode_self_mask(n, base, case.window)
        for h in range(case.num_heads):
            c = h * case.head_dim
            jobs.add(case.q, kk, vv, out, col=c, head_dim=case.head_dim, q_col=c, k_col=c, v_col=c,
                     scale=case.scale, mask=mask, nq=n, nk=base + n, q_row=b * n, k_row=0)
    secs = jobs.run(nthreads, ref)
    return out, secs


# ---- the attention blocks composed from the oracle's pieces --------------------------------------

def oracle_mha_block(x, w_qkv, w_proj, num_heads, *, use_rope, window=0, theta=500000.0, ref=False):
    """blt_multihead_attention (models/attention.c:130-207) as a chain of oracle functions: matmul,
    rotary embedding of Q and K at position = row, dense causal (+ window) mask, the head operator per
    head, matmul. Every piece is the restatement (ref=False) or the reference's own object code."""
    T, E = x.shape
    hd = E // num_heads
    qkv = ob.matmul(x, w_qkv, use_ref=ref)
    q, k, v = (np.ascontiguousarray(qkv[:, i * E:(i + 1) * E]) for i in range(3))
    if use_rope:
        cs, sn = ob.rope_tables(T, hd, theta, use_ref=ref)
        q, k = ob.rope_apply(q, cs, sn, num_heads, hd, use_ref=ref), ob.rope_apply(k, cs, sn, num_heads, hd, use_ref=ref)
    mask = None
    if window > 0:
        mask, _ = ob.build_mask(T, T, window=window, is_causal=True, use_ref=ref)
    comb, _ = ob.batched_attention(q, k, v, [0, T], [0, T], num_heads, hd, 1.0 / np.sqrt(np.float32(hd)), [mask],
                                   is_causal=True, use_ref=ref, nthreads=1)
    return ob.matmul(comb, w_proj, use_ref=ref)


def oracle_cross_block(xq, xk, wq, wk, wv, wp, num_heads, q_groups, k_groups, ref=False):
    """blt_cross_attention_forward (models/cross_attention.c:98-157) as a chain of oracle functions."""
    E = xq.shape[1]
    hd = E // num_heads
    q, k, v = ob.matmul(xq, wq, use_ref=ref), ob.matmul(xk, wk, use_ref=ref), ob.matmul(xk, wv, use_ref=ref)
    mask, _ = ob.build_mask(xq.shape[0], xk.shape[0], q_groups=q_groups, k_groups=k_groups, use_ref=ref)
    comb, _ = ob.batched_attention(q, k, v, [0, xq.shape[0]], [0, xk.shape[0]], num_heads, hd,
                                   1.0 / np.sqrt(np.float32(hd)), [mask], use_ref=ref, nthreads=1)
    return ob.matmul(comb, wp, use_ref=ref)
