"""The multi-head self-attention block (fblt_mha_forward: QKV matmul, fused rotary embedding,
masked attention, output matmul) against the reference's own blt_multihead_attention on the
CPU, sequence by sequence."""
import numpy as np
import pytest
import torch

from fblt_b200 import lib as L
from fblt_b200 import ops
from fblt_b200.ops import MaskConfig
from helpers import assert_close
from oracle import binding as ob

pytestmark = pytest.mark.gpu


def run_case(E, H, lens, seed, *, use_rope, window=0, docs=None, precision=L.PREC_FP32):
    if not ob.have_ref():
        pytest.skip("reference object code not built")
    rng = np.random.default_rng(seed)
    hd = E // H
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    x = rng.standard_normal((int(cu[-1]), E)).astype(np.float32)
    w_qkv = (rng.standard_normal((E, 3 * E)) / np.sqrt(E)).astype(np.float32)
    w_proj = (rng.standard_normal((E, E)) / np.sqrt(E)).astype(np.float32)
    want = np.zeros_like(x)
    for b, n in enumerate(lens):
        if n == 0:
            continue
        db = None if docs is None else docs[b]
        want[cu[b]:cu[b + 1]] = ob.ref_multihead_attention(x[cu[b]:cu[b + 1]], w_qkv, w_proj, H, is_causal=True,
                                                           use_rope=use_rope, window=window, doc_boundaries=db)
    mask = MaskConfig(is_causal=True, sliding_window=window, doc_bounds=docs)
    rope = {}
    if use_rope:
        cs, sn = ob.rope_tables(max(max(lens), 1), hd, use_ref=True)
        rope = dict(rope_cos=torch.from_numpy(cs).cuda(), rope_sin=torch.from_numpy(sn).cuda())
    got = ops.mha_forward(torch.from_numpy(x).cuda(), ops.PackedWeights(torch.from_numpy(w_qkv).cuda()),
                          ops.PackedWeights(torch.from_numpy(w_proj).cuda()), cu, H, mask, precision=precision, **rope)
    assert L.load().fblt_tcgen05_error() == 0
    return got.cpu().numpy(), want


def test_mha_block_matches_reference(cuda_lib):
    got, want = run_case(256, 4, [200, 1, 37, 0, 130], 1, use_rope=True)
    assert_close(got, want, "mha rope causal")
    got, want = run_case(128, 4, [96, 300], 2, use_rope=True, window=48)       # head_dim 32: mma.sync / row kernels
    assert_close(got, want, "mha rope window")
    got, want = run_case(256, 4, [150, 64], 3, use_rope=False,
                         docs=[np.array([40, 90]), np.array([], dtype=np.int64)])
    assert_close(got, want, "mha documents")


def test_mha_block_tf32_mode(cuda_lib):
    got, want = run_case(256, 4, [128, 77], 4, use_rope=True, precision=L.PREC_TF32)
    assert_close(got, want, "mha tf32", atol=5e-3, rtol=2e-2)     # single-pass TF32 in all three stages
