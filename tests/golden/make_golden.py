"""Generates the golden fixtures in this folder from the reference's own CPU object code
(oracle/_ref/libblt_ref.so, built by `make -C oracle` where the reference tree is mounted).

    python tests/golden/make_golden.py

Each .npz holds the inputs and the reference's outputs of one small case; tests replay the
inputs through the oracle (tests/test_oracle.py) and through the CUDA path (tests/test_gpu_*.py).
Inputs come from the seeded generators of fblt_b200.synth, so the files are reproducible.
"""
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

from fblt_b200 import synth  # noqa: E402
from oracle import binding as ob  # noqa: E402


def head_case(name, seed, T, S, H, hd, scale, mask=None, is_causal=False):
    E = H * hd
    q = synth.normal(seed, synth.TAG_Q, T * E).reshape(T, E)
    k = synth.normal(seed, synth.TAG_K, S * E).reshape(S, E)
    v = synth.normal(seed, synth.TAG_V, S * E).reshape(S, E)
    out, _ = ob.batched_attention(q, k, v, [0, T], [0, S], H, hd, scale, [mask], is_causal=is_causal, use_ref=True,
                                  nthreads=1)
    d = dict(kind="head", q=q, k=k, v=v, cu_q=np.array([0, T]), cu_k=np.array([0, S]), num_heads=H, head_dim=hd,
             scale=np.float32(scale), is_causal=is_causal, out=out)
    if mask is not None:
        d["mask"] = mask
    np.savez_compressed(HERE / f"{name}.npz", **d)


def mask_case(name, nq, nk, **kw):
    args = dict(window=0, bidirectional=True, is_causal=False, causal_offset=0)
    args.update(kw)
    m, empty = ob.build_mask(nq, nk, use_ref=True, **args)
    assert empty == 0
    d = dict(kind="mask", nq=nq, nk=nk, mask=m)
    for k_, v_ in args.items():
        d[k_] = np.asarray(v_)
    np.savez_compressed(HERE / f"{name}.npz", **d)


def block_cases():
    """Projection matmul and the two attention blocks (models/attention.c:130-207,
    models/cross_attention.c:98-157) run by the reference on the CPU."""
    rng = np.random.default_rng(11)
    a = rng.standard_normal((37, 52)).astype(np.float32)
    b = rng.standard_normal((52, 45)).astype(np.float32)
    np.savez_compressed(HERE / "matmul_37x52x45.npz", kind="matmul", a=a, b=b, out=ob.matmul(a, b, use_ref=True))
    E, H, T = 64, 2, 21
    x = rng.standard_normal((T, E)).astype(np.float32)
    w_qkv = (rng.standard_normal((E, 3 * E)) / np.sqrt(E)).astype(np.float32)
    w_proj = (rng.standard_normal((E, E)) / np.sqrt(E)).astype(np.float32)
    for name, kw in (("mha_block_rope_causal", dict(use_rope=True, window=0)),
                     ("mha_block_window", dict(use_rope=False, window=6))):
        out = ob.ref_multihead_attention(x, w_qkv, w_proj, H, is_causal=True, **kw)
        np.savez_compressed(HERE / f"{name}.npz", kind="mha", x=x, w_qkv=w_qkv, w_proj=w_proj, num_heads=H,
                            use_rope=kw["use_rope"], window=kw["window"], out=out)
    bounds = synth.bounds_from_lengths(synth.geometric_patches(12, 0, 40))
    P = len(bounds) - 1
    _, byte_patch = ob.patch_group_ids(bounds, use_ref=True)
    xq = rng.standard_normal((P, E)).astype(np.float32)
    xk = rng.standard_normal((40, E)).astype(np.float32)
    ws = [(rng.standard_normal((E, E)) / np.sqrt(E)).astype(np.float32) for _ in range(4)]
    out = ob.ref_cross_attention(xq, xk, *ws, H, np.arange(P), byte_patch[:40])
    np.savez_compressed(HERE / "cross_block_encoder.npz", kind="cross", xq=xq, xk=xk, wq=ws[0], wk=ws[1], wv=ws[2],
                        wp=ws[3], num_heads=H, bounds=bounds, out=out)


def main():
    assert ob.have_ref(), "build oracle/_ref first (make -C oracle)"
    block_cases()
    # shape of tests/parity/parity_transformer.c:19-61 (T=6, E=16, H=4, causal)
    head_case("head_causal_t6_h4", 101, 6, 6, 4, 4, 0.5, is_causal=True)
    # ragged sizes around warp / tile edges, non-causal, arbitrary additive mask values
    rng = np.random.default_rng(7)
    m = np.where(rng.random((33, 47)) < 0.5, 0.0, -np.inf).astype(np.float32)
    m[5, :] = -np.inf                      # fully masked row -> zeros
    m[6, :] = 0.25 * rng.standard_normal(47).astype(np.float32)  # finite additive bias
    head_case("head_masked_33x47_h2_d16", 102, 33, 47, 2, 16, 0.25, mask=m)
    # config-1 shape, shortened: causal + window, packed-width heads of 32
    wm, _ = ob.build_mask(96, 96, window=40, is_causal=True, use_ref=True)
    head_case("head_window_96_h4_d32", 103, 96, 96, 4, 32, 1 / np.sqrt(32.0), mask=wm)
    # decode shape: 4 block rows over a 70-row cache, 64-wide heads
    head_case("head_block_4x74_h2_d64", 104, 4, 74, 2, 64, 0.125, mask=np.zeros((4, 74), np.float32))
    mask_case("mask_causal_window_docs", 40, 40, window=9, is_causal=True, doc_boundaries=[7, 19, 31])
    mask_case("mask_offset_window", 6, 30, window=11, is_causal=True, causal_offset=24)
    mask_case("mask_symmetric_window", 17, 17, window=4)
    lens = synth.geometric_patches(9, 0, 128)
    bounds = synth.bounds_from_lengths(lens)
    qg, kg = ob.patch_group_ids(bounds, use_ref=True)
    mask_case("mask_encoder_groups", len(lens), 128, q_groups=qg, k_groups=kg)
    pos = np.arange(0, 140)
    lat = np.array([ob.latent_at(bounds, int(p), use_ref=True) for p in pos])
    np.savez_compressed(HERE / "latent_geometric_128.npz", kind="latent", bounds=bounds, pos=pos, latent=lat)
    print("wrote", len(list(HERE.glob("*.npz"))), "fixtures")


if __name__ == "__main__":
    main()
