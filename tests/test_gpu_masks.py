"""The on-the-fly mask rule against the reference's dense mask builder: bit-exact, both as
the per-pair predicate and as the per-row key range the tile / streaming kernels use."""
import numpy as np
import pytest
import torch

from fblt_b200 import lib as L
from fblt_b200 import ops, synth, workloads
from fblt_b200.ops import MaskConfig
from fblt_b200.workloads import ForwardCase
from helpers import dense_masks, use_ref

pytestmark = pytest.mark.gpu


def bitmap_matches(case: ForwardCase, expect_empty_rows: bool = False):
    E = case.embed
    dummy_q = torch.zeros((int(case.cu_q[-1]), E), device="cuda")
    dummy_k = torch.zeros((int(case.cu_k[-1]), E), device="cuda")
    batch = ops.make_batch(dummy_q, dummy_k, dummy_k, dummy_q.clone(), case.cu_q, case.cu_k, case.num_heads,
                           case.head_dim, 1.0, case.mask)
    want = dense_masks(case, use_ref() and not expect_empty_rows)
    forms = [False] if case.mask.group_rule == L.GROUP_IDS else [False, True]
    for use_range in forms:
        bm = ops.mask_bitmap(batch, use_range=use_range).cpu().numpy()
        for b, m in enumerate(want):
            nq, nk = m.shape
            got = bm[b, :nq, :nk].astype(bool)
            assert (got == (m == 0)).all(), f"{case.name} seq {b} use_range={use_range}"
            assert not bm[b, nq:, :].any() and not bm[b, :, nk:].any()
    for b in (0, len(want) - 1):
        if want[b].size == 0:
            continue
        dm, empty = ops.mask_materialize(batch, b)
        assert dm.cpu().numpy().tobytes() == want[b].tobytes()
        assert empty == int((~(want[b] == 0).any(axis=1)).sum())


def simple_case(name, cu_q, cu_k, mask, H=1, hd=32):
    z = np.zeros((1, H * hd), np.float32)
    return ForwardCase(name, H, hd, 1.0, z, z, z, np.asarray(cu_q, np.int32), np.asarray(cu_k, np.int32), mask)


def test_benchmark_config_masks(cuda_lib):
    bitmap_matches(workloads.c1_byte_self_attention())
    bitmap_matches(workloads.c2_patch_attention())
    for direction in ("enc", "dec_leq", "dec_paper"):
        bitmap_matches(workloads.c3_cross_attention(direction, batch=8))
    bitmap_matches(workloads.c5_prefill(batch=6))


def test_causal_window_docs_offsets(cuda_lib):
    cu = [0, 40, 40, 57, 121]
    docs = [np.array([7, 19, 31]), np.array([], np.int64), np.array([5]), np.array([1, 2, 60])]
    for causal in (True, False):
        for w in (0, 1, 4, 9, 200):
            bitmap_matches(simple_case("cwd", cu, cu, MaskConfig(is_causal=causal, sliding_window=w, doc_bounds=docs)),
                           expect_empty_rows=False)
    # chunked decode over a cached prefix: nq < nk with a per-sequence causal offset
    cu_q, cu_k = [0, 6, 9, 10], [0, 30, 42, 43]
    for w in (0, 11):
        bitmap_matches(simple_case("off", cu_q, cu_k, MaskConfig(is_causal=True, sliding_window=w,
                                                                  causal_offset=[24, 9, 0])))


def test_patch_rules_with_subtokens_and_offsets(cuda_lib):
    lens = [synth.geometric_patches(31, s, 96) for s in range(3)]
    bounds = [synth.bounds_from_lengths(l) for l in lens]
    P = np.array([len(l) for l in lens])
    for k in (1, 3):
        cu_p = np.concatenate([[0], np.cumsum(P * k)])
        cu_b = np.arange(4) * 96
        bitmap_matches(simple_case("enc", cu_p, cu_b, MaskConfig(group_rule=L.GROUP_PATCH_ENC, subtokens=k,
                                                                  patch_bounds=bounds)))
        for rule in (L.GROUP_PATCH_DEC, L.GROUP_PATCH_LEQ):
            bitmap_matches(simple_case("dec", cu_b, cu_p, MaskConfig(group_rule=rule, subtokens=k, patch_bounds=bounds)))
        # incremental decode: 5 fresh byte rows at positions base.., some past the last patch end
        cu_n = np.arange(4) * 5
        for tc in ([0, 0, 0], [1, 0, 1]):
            bitmap_matches(simple_case("dec_step", cu_n, cu_p,
                                       MaskConfig(group_rule=L.GROUP_PATCH_DEC, subtokens=k, patch_bounds=bounds,
                                                  q_pos_offset=[90, 17, 94], trailing_closed=tc)))


def test_block_diffusion_infer_rule(cuda_lib):
    cu = [0, 7, 7 + 40, 47 + 5]
    bitmap_matches(simple_case("bd", cu, cu, MaskConfig(num_clean=[3, 36, 1])))


def test_explicit_group_ids(cuda_lib):
    rng = np.random.default_rng(4)
    cu_q, cu_k = [0, 12, 30], [0, 20, 33]
    qg = rng.integers(0, 4, 30)
    kg = rng.integers(0, 4, 33)
    for bidir in (True, False):
        bitmap_matches(simple_case("ids", cu_q, cu_k, MaskConfig(group_rule=L.GROUP_IDS, q_group_ids=qg, k_group_ids=kg,
                                                                  bidirectional_within_group=bidir)),
                       expect_empty_rows=True)
