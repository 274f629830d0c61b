"""CPU-side checks of the product library: it loads, exports every symbol the header
declares, its structs have the sizes the bindings assume, and its host-only functions
(patch boundary helpers, selection helpers) agree with the oracle. No kernel runs here."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

from fblt_b200 import lib as L
from fblt_b200 import ops, synth
from oracle import binding as ob

ROOT = Path(__file__).resolve().parent.parent


def declared_functions():
    text = (ROOT / "include" / "fblt_attn.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b((?:fblt|blt)_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    lib = L.load()
    names = declared_functions()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/fblt_attn.h but not exported"
        assert n in L.SYMBOLS, f"{n} has no ctypes signature in fblt_b200/lib.py"


def test_version_and_status_strings():
    lib = L.load()
    assert lib.fblt_version().decode().startswith("fblt_attn sm_100a")
    assert lib.fblt_status_string(0) == b"ok"
    assert b"workspace" in lib.fblt_status_string(L.ERR_WORKSPACE)


def test_argument_validation_without_gpu():
    lib = L.load()
    assert lib.fblt_attn_forward(None, None) == L.ERR_ARG
    d = L.AttnDesc()
    d.batch, d.num_heads, d.head_dim = 1, 2, 64
    assert lib.fblt_attn_forward(C.byref(d), None) == L.ERR_ARG and b"cu_q" in lib.fblt_last_error()
    dd = L.DecodeDesc()
    dd.batch, dd.num_heads, dd.head_dim, dd.n_new = 1, 2, 48, 1
    assert lib.fblt_attn_decode(C.byref(dd), None, 0, None) == L.ERR_UNSUPPORTED
    dd.head_dim, dd.n_new = 64, 40
    assert lib.fblt_attn_decode(C.byref(dd), None, 0, None) == L.ERR_UNSUPPORTED
    assert lib.fblt_attention_head(None, None) == L.ERR_ARG


def test_patch_bounds_and_validation():
    b = ops.patch_bounds([0, 3, 7, 8, 15], [3, 4, 1, 7, 1], 16)
    assert list(b) == [0, 3, 7, 8, 15, 16]
    with pytest.raises(L.FbltError):
        ops.patch_bounds([0, 4], [3, 2], 6)       # gap
    with pytest.raises(L.FbltError):
        ops.patch_bounds([0, 3], [3, 2], 6)       # does not cover
    with pytest.raises(L.FbltError):
        ops.patch_bounds([0, 3], [3, 0], 3)       # empty patch


def test_latent_rule_matches_oracle():
    want = [0, 0, 0, 0, 0, 0, 1, 2, 2, 2, 2, 2, 2, 2, 3, 3]
    b = np.array([0, 3, 7, 8, 15, 16], dtype=np.int32)
    assert [ops.patch_latent_at(b, p) for p in range(16)] == want
    assert ops.patch_latent_at(b, 16) == 4 and ops.patch_latent_at(b, 100) == 4
    for s in range(6):
        bounds = synth.bounds_from_lengths(synth.geometric_patches(21, s, 200))
        for pos in range(0, 210):
            assert ops.patch_latent_at(bounds, pos) == ob.latent_at(bounds, pos, use_ref=ob.have_ref())
    one = np.array([0, 5], dtype=np.int32)
    assert [ops.patch_latent_at(one, p) for p in range(7)] == [0] * 7


def test_selection_helpers_match_oracle():
    lib, o = L.load(), ob.oracle()
    rng = np.random.default_rng(3)
    for _ in range(300):
        B = int(rng.integers(1, 33))
        s = rng.random(B).astype(np.float32)
        s[rng.random(B) < 0.2] = 0.5  # ties
        m = (rng.random(B) < 0.7).astype(np.uint8)
        thr = float(rng.random() * 3 - 0.5)
        sp, mp = s.ctypes.data_as(L.c_float_p), m.ctypes.data_as(L.c_u8_p)
        assert lib.fblt_unmask_select_confidence(sp, mp, B, thr) == o.oracle_unmask_select_confidence(sp, mp, B, thr)
        assert lib.fblt_unmask_select_eb(sp, mp, B, thr) == o.oracle_unmask_select_eb(sp, mp, B, thr)
    arr, n = ob.patch_array([0, 4, 6, 7, 12, 15])
    for lo in range(0, 16):
        for hi in range(lo, 17):
            assert lib.fblt_aligned_commit_select(arr, n, lo, hi) == o.oracle_aligned_commit_select(arr, n, lo, hi)
    for cur in (1, 3, 8, 16, 20):
        for acc in (float("nan"), 0.0, 0.39, 0.41, 0.5, 0.59, 0.61, 1.0):
            for lo, hi in ((0, 16), (4, 16), (4, 0), (8, 4), (16, 16)):
                assert lib.fblt_block_adapt_b(cur, acc, lo, hi, 0.5) == o.oracle_block_adapt_b(cur, acc, lo, hi, 0.5)


def test_common_patches_matches_reference_or_definition():
    """Leading patches equal in start and length (infer/kv_cache.c:101-109)."""
    lib = L.load()
    rng = np.random.default_rng(11)
    for _ in range(200):
        cuts_a = np.unique(np.concatenate([[0], rng.integers(1, 64, size=int(rng.integers(0, 12))), [64]]))
        cuts_b = cuts_a.copy()
        if rng.random() < 0.8 and len(cuts_b) > 2:                      # perturb one interior boundary
            k = int(rng.integers(1, len(cuts_b) - 1))
            cuts_b = np.unique(np.concatenate([cuts_b[:k], [min(int(cuts_b[k]) + 1, 63)], cuts_b[k + 1:]]))
        a, na = ob.patch_array(cuts_a.tolist())
        b, nb = ob.patch_array(cuts_b.tolist())
        ncached = int(rng.integers(0, na + 1))
        want = 0
        while (want < ncached and want < nb and a[want].start_idx == b[want].start_idx
               and a[want].length == b[want].length):
            want += 1
        assert lib.fblt_kv_common_patches(a, ncached, b, nb) == want
        if ob.have_ref():
            assert ob.ref().ref_kv_common_patches(a, ncached, b, nb) == want


def test_matmul_packed_size():
    """One 32 KB (hi | lo) tile per 128 output columns and 32 of depth, both rounded up."""
    lib = L.load()
    for K, N in ((1024, 3072), (1024, 1024), (4, 1), (33, 129), (100, 130)):
        assert lib.fblt_matmul_packed_bytes(K, N) == -(-N // 128) * -(-K // 32) * 32768
    assert lib.fblt_matmul_packed_bytes(0, 8) == 0 and lib.fblt_matmul_packed_bytes(8, -1) == 0


def test_synth_is_deterministic_and_sliceable():
    a = synth.normal(5, synth.TAG_Q, 1000)
    b = synth.normal(5, synth.TAG_Q, 400, start=333)
    assert (a[333:733] == b).all()
    assert abs(float(a.mean())) < 0.15 and 0.85 < float(a.std()) < 1.15
    for s in range(50):
        lens = synth.geometric_patches(1, s)
        assert lens.sum() == 512 and lens.min() >= 1 and len(lens) <= 128
        assert (lens[:-1] <= 16).all()
    lens = synth.cache_lengths(3, 256)
    assert lens.min() >= 64 and lens.max() <= 512
