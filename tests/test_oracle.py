"""Pins the CPU oracle: the restatement (oracle/attn_oracle.c) and, where built, the
reference's own object code (oracle/_ref) against the known-answer vectors the
reference's tests hold for the attention path, against each other bit for bit, and
against the committed golden fixtures."""
from pathlib import Path

import numpy as np
import pytest

from fblt_b200 import synth
from helpers import oracle_cross_block, oracle_mha_block
from oracle import binding as ob

GOLDEN = Path(__file__).resolve().parent / "golden"
IMPLS = [False] + ([True] if ob.have_ref() else [])


@pytest.mark.parametrize("ref", IMPLS)
def test_known_answer_two_head_attention(ref):
    # tests/unit/models/unit_attention.c:10-93: identity projections, 2 heads x 2, non-causal
    x = np.array([[1, 0, 1, 0], [0, 1, 0, 1]], dtype=np.float32)
    qkv = np.concatenate([x, x, x], axis=1).copy()
    out, _ = ob.batched_attention(qkv, qkv, qkv, [0, 2], [0, 2], 2, 2, 1 / np.sqrt(2.0), [None], k_col0=4, v_col0=8,
                                  use_ref=ref, nthreads=1)
    want = np.array([[0.6697615, 0.3302385, 0.6697615, 0.3302385], [0.3302385, 0.6697615, 0.3302385, 0.6697615]])
    assert np.abs(out - want).max() < 1e-6


@pytest.mark.parametrize("ref", IMPLS)
def test_mask_config_causal_equals_is_causal(ref):
    # tests/unit/models/unit_attention.c:95-189: a causal mask_config equals the in-op causal flag
    T, H, hd = 9, 2, 4
    E = H * hd
    qkv = synth.normal(11, 1, T * 3 * E).reshape(T, 3 * E)
    m, _ = ob.build_mask(T, T, is_causal=True, use_ref=ref)
    a, _ = ob.batched_attention(qkv, qkv, qkv, [0, T], [0, T], H, hd, 0.5, [m], k_col0=E, v_col0=2 * E, use_ref=ref)
    b, _ = ob.batched_attention(qkv, qkv, qkv, [0, T], [0, T], H, hd, 0.5, [None], is_causal=True, k_col0=E,
                                v_col0=2 * E, use_ref=ref)
    assert np.abs(a - b).max() < 1e-6


@pytest.mark.parametrize("ref", IMPLS)
def test_mask_builder_vectors(ref):
    # tests/unit/backend/unit_mask.c:14-192
    m, _ = ob.build_mask(4, 4, is_causal=True, use_ref=ref)
    assert ((m == 0) == np.tril(np.ones((4, 4), bool))).all()
    m, _ = ob.build_mask(6, 6, is_causal=True, window=3, use_ref=ref)
    assert list(m[5] == 0) == [False, False, False, True, True, True]
    m, _ = ob.build_mask(6, 6, doc_boundaries=[3], use_ref=ref)
    assert m[1, 2] == 0 and m[4, 5] == 0 and np.isinf(m[2, 3]) and np.isinf(m[5, 0])
    m, _ = ob.build_mask(4, 4, q_groups=[0, 0, 1, 1], k_groups=[0, 0, 1, 1], bidirectional=False, use_ref=ref)
    assert np.isinf(m[0, 2]) and np.isinf(m[3, 1]) and m[1, 0] == 0 and np.isinf(m[0, 1])


@pytest.mark.parametrize("ref", IMPLS)
def test_paper_rule_vector(ref):
    # tests/unit/models/unit_local_decoder.c:87-116
    bounds = np.array([0, 3, 7, 8, 15, 16])
    want = [0, 0, 0, 0, 0, 0, 1, 2, 2, 2, 2, 2, 2, 2, 3, 3]
    assert [ob.latent_at(bounds, p, use_ref=ref) for p in range(16)] == want
    assert ob.latent_at(bounds, 16, use_ref=ref) == 4 and ob.latent_at(bounds, 100, use_ref=ref) == 4
    qg, kg = ob.patch_group_ids(bounds, use_ref=ref)
    assert list(qg) == [0, 1, 2, 3, 4]
    assert list(kg) == [0] * 3 + [1] * 4 + [2] + [3] * 7 + [4]


@pytest.mark.parametrize("ref", IMPLS)
def test_block_diffusion_bitmaps(ref):
    # tests/unit/models/unit_block_diffusion.c:115-176 (Figure-5 TRAIN fixture and the INFER rule)
    want = ["10000000000000", "11000000000000", "11100000000000", "11110000000000", "11111000000000",
            "11111100000000", "11000011110000", "11000011110000", "11000011110000", "11000011110000",
            "11110000001111", "11110000001111", "11110000001111", "11110000001111"]
    m, _ = ob.block_diffusion_mask(0, 14, 6, 4, [2, 4], use_ref=ref)
    got = ["".join("1" if v == 0 else "0" for v in row) for row in m]
    assert got == want
    m, _ = ob.block_diffusion_mask(1, 7, 3, use_ref=ref)
    for i in range(7):
        for j in range(7):
            assert (m[i, j] == 0) == ((j <= i) if i < 3 else True)


def _sel(fn_name, ref, scores, masked, thr):
    import ctypes as C
    lib = ob.ref() if ref else ob.oracle()
    fn = getattr(lib, ("ref_" if ref else "oracle_") + fn_name)
    s = np.asarray(scores, dtype=np.float32)
    m = np.asarray(masked, dtype=np.uint8)
    return fn(s.ctypes.data_as(ob.c_f_p), m.ctypes.data_as(C.POINTER(C.c_uint8)), len(s), thr)


@pytest.mark.parametrize("ref", IMPLS)
def test_selection_bitmasks(ref):
    # tests/unit/infer/unit_block_generation.c:367-418
    assert _sel("unmask_select_confidence", ref, [0.95, 0.80, 0.60, 0.30], [1, 1, 1, 1], 0.7) == 0x3
    assert _sel("unmask_select_confidence", ref, [0.10, 0.50, 0.20], [1, 1, 1], 0.9) == 0x2
    assert _sel("unmask_select_confidence", ref, [0.99] * 4, [0, 1, 0, 1], 0.5) == 0xA
    assert _sel("unmask_select_eb", ref, [2.0, 0.5, 1.5, 1.0], [1, 1, 0, 1], 1.4) == 0x2
    assert _sel("unmask_select_eb", ref, [3.0, 1.0, 2.0], [1, 1, 1], 100.0) == 0x7
    assert _sel("unmask_select_eb", ref, [2.0, 0.5, 1.0], [1, 1, 1], -1.0) == 0x2
    assert _sel("unmask_select_confidence", ref, [1.0, 1.0], [0, 0], 0.0) == 0
    assert _sel("unmask_select_eb", ref, [1.0, 1.0], [0, 0], 10.0) == 0


@pytest.mark.parametrize("ref", IMPLS)
def test_commit_select_and_adapt_b(ref):
    # tests/unit/infer/unit_block_generation.c:582-615
    lib = ob.ref() if ref else ob.oracle()
    pre = "ref_" if ref else "oracle_"
    arr, n = ob.patch_array([0, 4, 6, 7, 12, 15])
    sel = getattr(lib, pre + "aligned_commit_select")
    assert [sel(arr, n, lo, hi) for lo, hi in [(0, 4), (4, 6), (5, 10), (7, 11), (7, 12), (13, 15)]] == [4, 6, 7, 0, 12, 15]
    ab = getattr(lib, pre + "block_adapt_b")
    cases = [((8, 0.9, 4, 16), 9), ((8, 0.2, 4, 16), 7), ((8, 0.55, 4, 16), 8), ((16, 0.9, 4, 16), 16),
             ((4, 0.2, 4, 16), 4), ((8, 0.2, 0, 16), 7), ((1, 0.2, 0, 16), 1), ((8, 0.9, 0, 16), 9),
             ((8, 0.2, 4, 0), 8), ((3, 0.9, 4, 16), 5), ((20, 0.2, 4, 16), 15)]
    for (cur, acc, lo, hi), want in cases:
        assert ab(cur, acc, lo, hi, 0.5) == want


def _verify(x, l, r, target, logits):
    import ctypes as C
    buf = np.zeros(16, np.uint8)
    buf[:len(x)] = x
    acc = C.c_size_t(0)
    n = ob.oracle().oracle_verify_accept(buf.ctypes.data_as(C.POINTER(C.c_uint8)), logits.ctypes.data_as(ob.c_f_p),
                                         logits.shape[1], l, r, target, C.byref(acc))
    return n, buf, acc.value


def test_verify_accept_cases_of_the_reference():
    """The four hand-computable branches of the reference's verify step
    (tests/unit/infer/unit_self_speculation.c:178-255): its model there predicts byte 0 at every row
    (all logits equal, lowest index wins), which is an all-zero logit matrix here."""
    logits = np.zeros((16, 256), np.float32)
    n, x, acc = _verify([7, 7, 5, 5], 2, 2, 16, logits)          # A: first draft byte wrong
    assert (n, acc) == (3, 0) and x[:3].tolist() == [7, 7, 0]
    n, x, acc = _verify([7, 7, 0, 0, 0], 2, 2, 16, logits)       # B: all right, one free byte
    assert (n, acc) == (5, 2) and x[:5].tolist() == [7, 7, 0, 0, 0]
    n, x, acc = _verify([7, 7, 0, 0], 2, 2, 4, logits)           # C: all right, budget reached
    assert (n, acc) == (4, 2)
    n, x, acc = _verify([9, 9, 0, 5, 5], 2, 3, 16, logits)       # D: second draft byte wrong
    assert (n, acc) == (4, 1) and x[2:4].tolist() == [0, 0]


@pytest.mark.skipif(not ob.have_ref(), reason="reference object code not built here")
def test_argmax_rule_equals_reference_operator():
    """The restated row argmax against the reference's public operator (ops/row_stats_cpu.c:30-47)
    on rows full of exact ties, infinities and a single element: same index everywhere."""
    import ctypes as C
    rng = np.random.default_rng(11)
    o, r = ob.oracle(), ob.ref()
    for vocab in (1, 2, 7, 256, 300):
        x = rng.standard_normal((64, vocab)).astype(np.float32)
        x[::2] = np.round(x[::2])                        # many ties
        x[3, :] = 0.25
        x[5, :] = -np.inf
        if vocab > 2:
            x[7, 1], x[7, vocab - 1] = np.inf, np.inf
        x = np.ascontiguousarray(x)
        ids = np.zeros(64, np.uint32)
        r.ref_argmax_rows(x.ctypes.data_as(ob.c_f_p), 64, vocab, ids.ctypes.data_as(C.POINTER(C.c_uint32)))
        mine = [o.oracle_argmax_row(x[i].ctypes.data_as(ob.c_f_p), vocab) for i in range(64)]
        assert mine == ids.tolist()


def test_decode_masks_match_builder():
    # the incremental decoder's host loop (infer/kv_cache.c:229-236) is the builder's rule with a causal offset
    for base, n, w in [(0, 3, 0), (7, 4, 0), (9, 2, 4), (20, 5, 6)]:
        a = ob.decode_self_mask(n, base, w)
        b, _ = ob.build_mask(n, base + n, window=w, is_causal=True, causal_offset=base, use_ref=ob.have_ref())
        assert ((a == 0) == (b == 0)).all()


@pytest.mark.skipif(not ob.have_ref(), reason="reference object code not built here")
def test_restatement_equals_reference_bitwise():
    rng = np.random.default_rng(5)
    for (T, S, H, hd) in [(1, 1, 1, 2), (7, 5, 2, 6), (33, 65, 3, 16), (64, 64, 2, 32)]:
        E = H * hd
        q = rng.standard_normal((T, E)).astype(np.float32)
        k = rng.standard_normal((S, E)).astype(np.float32)
        v = rng.standard_normal((S, E)).astype(np.float32)
        mask = np.where(rng.random((T, S)) < 0.6, 0.0, -np.inf).astype(np.float32)
        mask[0, :] = -np.inf  # an all-masked row must give zeros in both
        if T > 1:
            mask[1, 0] = 0.0
        a, _ = ob.batched_attention(q, k, v, [0, T], [0, S], H, hd, 0.3, [mask], use_ref=False)
        b, _ = ob.batched_attention(q, k, v, [0, T], [0, S], H, hd, 0.3, [mask], use_ref=True)
        assert a.tobytes() == b.tobytes()
        assert (a[0] == 0).all()
    for args in [dict(nq=9, nk=9, is_causal=True, window=4), dict(nq=5, nk=12, is_causal=True, causal_offset=7),
                 dict(nq=10, nk=10, doc_boundaries=[2, 7], is_causal=True), dict(nq=8, nk=8, window=3)]:
        nq, nk = args.pop("nq"), args.pop("nk")
        a, _ = ob.build_mask(nq, nk, use_ref=False, **args)
        b, _ = ob.build_mask(nq, nk, use_ref=True, **args)
        assert a.tobytes() == b.tobytes()


@pytest.mark.skipif(not ob.have_ref(), reason="reference object code not built here")
def test_struct_layout_matches_reference_headers():
    import ctypes as C
    from fblt_b200.lib import HeadArgs, PatchInfo
    buf = (C.c_size_t * 32)()
    n = ob.ref().ref_struct_layout(buf, 32)
    got = list(buf[:n])
    h = HeadArgs
    want = [C.sizeof(h)] + [getattr(h, f).offset for f, _ in h._fields_] + \
           [C.sizeof(PatchInfo)] + [getattr(PatchInfo, f).offset for f, _ in PatchInfo._fields_] + [0, 1]
    assert got == want


def test_golden_fixtures():
    """Outputs of the reference's own object code, committed with the script that made them
    (tests/golden/make_golden.py); both oracle flavours must reproduce them exactly."""
    files = sorted(GOLDEN.glob("*.npz"))
    assert files, "golden fixtures missing"
    for f in files:
        g = np.load(f)
        kind = str(g["kind"])
        for ref in IMPLS:
            if kind == "head":
                H, hd = int(g["num_heads"]), int(g["head_dim"])
                mask = g["mask"] if "mask" in g.files else None
                out, _ = ob.batched_attention(g["q"], g["k"], g["v"], g["cu_q"], g["cu_k"], H, hd, float(g["scale"]),
                                              [mask], is_causal=bool(g["is_causal"]), use_ref=ref)
                assert out.tobytes() == g["out"].tobytes(), f.name
            elif kind == "mask":
                kw = {k: g[k] for k in ("doc_boundaries", "q_groups", "k_groups") if k in g.files}
                m, _ = ob.build_mask(int(g["nq"]), int(g["nk"]), window=int(g["window"]),
                                     bidirectional=bool(g["bidirectional"]), is_causal=bool(g["is_causal"]),
                                     causal_offset=int(g["causal_offset"]), use_ref=ref, **kw)
                assert m.tobytes() == g["mask"].tobytes(), f.name
            elif kind == "latent":
                got = [ob.latent_at(g["bounds"], int(p), use_ref=ref) for p in g["pos"]]
                assert got == list(g["latent"]), f.name
            elif kind == "matmul":
                assert ob.matmul(g["a"], g["b"], use_ref=ref).tobytes() == g["out"].tobytes(), f.name
            elif kind == "mha":
                # the block is exactly the chain of its pieces, in either oracle flavour
                out = oracle_mha_block(g["x"], g["w_qkv"], g["w_proj"], int(g["num_heads"]), use_rope=bool(g["use_rope"]),
                                       window=int(g["window"]), ref=ref)
                assert out.tobytes() == g["out"].tobytes(), f.name
            elif kind == "cross":
                bounds = g["bounds"]
                _, byte_patch = ob.patch_group_ids(bounds, use_ref=ref)
                out = oracle_cross_block(g["xq"], g["xk"], g["wq"], g["wk"], g["wv"], g["wp"], int(g["num_heads"]),
                                         np.arange(len(bounds) - 1), byte_patch[:g["xk"].shape[0]], ref=ref)
                assert out.tobytes() == g["out"].tobytes(), f.name
            else:
                raise AssertionError(f"unknown fixture kind {kind}")


def test_matmul_restatement_equals_reference():
    if not ob.have_ref():
        pytest.skip("reference object code not built")
    rng = np.random.default_rng(5)
    for m, k, n in ((1, 1, 1), (7, 33, 5), (64, 256, 96)):
        a = rng.standard_normal((m, k)).astype(np.float32)
        b = rng.standard_normal((k, n)).astype(np.float32)
        assert ob.matmul(a, b).tobytes() == ob.matmul(a, b, use_ref=True).tobytes()
