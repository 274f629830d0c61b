"""The two dense mask builders behind the reference's config structs (the symbols its dispatcher
binds at core/backend.c:190-192) against the reference's CPU builders: bit-equal tensors."""
import numpy as np
import pytest

from fblt_b200 import lib as L
from fblt_b200 import ops
from helpers import use_ref
from oracle import binding as ob

pytestmark = pytest.mark.gpu


def check(nq, nk, **kw):
    want, empty_want = ob.build_mask(nq, nk, use_ref=False, **kw)
    if use_ref() and empty_want == 0:
        ref_mask, _ = ob.build_mask(nq, nk, use_ref=True, **kw)
        assert ref_mask.tobytes() == want.tobytes()
    got, empty = ops.build_attention_mask(nq, nk, **kw)
    assert got.cpu().numpy().tobytes() == want.tobytes(), kw
    assert empty == empty_want


def test_attention_mask_variants(cuda_lib):
    # the variant matrix of the reference's CUDA parity test (tests/parity/parity_cuda_composites.c:53-79)
    sq, skv = 19, 23
    docs = [7, 15, 15]
    qg, kg = np.arange(sq) % 3, np.arange(skv) % 3
    check(sq, skv, is_causal=True)
    check(sq, skv, window=5)
    check(sq, skv, is_causal=True, window=4, doc_boundaries=docs)
    check(sq, skv, doc_boundaries=docs)
    check(sq, skv, is_causal=True, q_groups=qg, k_groups=kg, bidirectional=True)
    check(sq, skv, is_causal=True, q_groups=qg, k_groups=kg, bidirectional=False)
    check(sq, skv, is_causal=True, window=6, doc_boundaries=docs, q_groups=qg, k_groups=kg, bidirectional=True)


def test_attention_mask_offsets_and_sizes(cuda_lib):
    rng = np.random.default_rng(5)
    for nq, nk in ((1, 1), (1, 300), (300, 1), (129, 257), (512, 512)):
        check(nq, nk, is_causal=True, causal_offset=max(0, nk - nq))
        check(nq, nk, is_causal=True, causal_offset=max(0, nk - nq), window=7)
        check(nq, nk, window=3)
        g = int(rng.integers(1, 6))
        check(nq, nk, q_groups=rng.integers(0, g, nq), k_groups=rng.integers(0, g, nk))  # rows may come out empty
    # kv-cache decode step over a cached prefix (infer/kv_cache.c:229-236): offset = base
    check(4, 68, is_causal=True, causal_offset=64, window=16)


def test_block_diffusion_masks(cuda_lib):
    for mode, S, N, B, starts in ((1, 24, 12, 0, None), (0, 24, 12, 2, [0, 4, 1, 7, 3, 11]), (0, 9, 9, 3, []),
                                  (1, 1, 1, 0, None), (0, 40, 16, 8, [15, 0, 8]), (1, 516, 512, 0, None)):
        want, _ = ob.block_diffusion_mask(mode, S, N, B, starts)
        if use_ref():
            ref_mask, _ = ob.block_diffusion_mask(mode, S, N, B, starts, use_ref=True)
            assert ref_mask.tobytes() == want.tobytes()
        got, empty = ops.build_block_diffusion_mask(mode, S, N, B, starts)
        assert got.cpu().numpy().tobytes() == want.tobytes(), (mode, S, N, B)
        assert empty == 0


def test_preconditions_return_statuses(cuda_lib):
    import ctypes as C
    import torch
    lib = cuda_lib
    c = L.BlockDiffusionConfig()
    c.mode, c.seq_len, c.num_clean = 1, 8, 9          # num_clean > seq_len (ops/mask_builder_cpu.c:105)
    buf = torch.empty(64, dtype=torch.float32, device="cuda")
    scr = torch.empty(64, dtype=torch.uint8, device="cuda")
    assert lib.fblt_build_block_diffusion_mask_dense(C.byref(c), buf.data_ptr(), scr.data_ptr(), 64, None, None) == L.ERR_ARG
    c.mode, c.seq_len, c.num_clean, c.block_size, c.num_blocks = 0, 8, 4, 3, 1   # does not tile
    assert lib.fblt_build_block_diffusion_mask_dense(C.byref(c), buf.data_ptr(), scr.data_ptr(), 64, None, None) == L.ERR_ARG
    m = L.MaskConfig()
    m.seq_len_q, m.seq_len_kv = 4, 4
    assert lib.fblt_build_attention_mask_dense(C.byref(m), buf.data_ptr(), None, 0, None, None) == L.ERR_WORKSPACE
