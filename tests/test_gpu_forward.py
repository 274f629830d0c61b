"""Batched prefill / cross attention (fblt_attn_forward) against the CPU oracle on the
benchmark configurations and on ragged edge cases, for both kernels and both precisions."""
import numpy as np
import pytest
import torch

from fblt_b200 import lib as L
from fblt_b200 import ops, synth, workloads
from fblt_b200.ops import MaskConfig
from fblt_b200.workloads import ForwardCase
from gpu_utils import forward_gpu
import dataclasses

import oracle.binding as ob
from helpers import assert_close, oracle_forward

pytestmark = pytest.mark.gpu

KERNELS = [(L.IMPL_ROW, L.PREC_FP32), (L.IMPL_TILE, L.PREC_FP32), (L.IMPL_TILE, L.PREC_TF32)]
# single-pass TF32 rounds every product to 11 bits: stated tolerance of that mode
TF32_ATOL, TF32_RTOL = 2e-3, 2e-2


T5_KERNELS = [(L.IMPL_TCGEN05, L.PREC_FP32), (L.IMPL_TCGEN05, L.PREC_TF32)]


def check(case: ForwardCase, kernels=KERNELS):
    want, masks, _ = oracle_forward(case)
    if kernels is KERNELS and case.head_dim == 64 and case.mask.group_rule != L.GROUP_IDS:
        kernels = KERNELS + T5_KERNELS          # the tcgen05 kernel takes head_dim 64
    if kernels[0][0] == L.IMPL_ROW and case.head_dim in (32, 64) and case.mask.group_rule != L.GROUP_IDS:
        kernels = kernels + [(L.IMPL_ROW_QUAD, L.PREC_FP32)]   # four lanes per row: same shapes, range rules
    fits_unit = (case.head_dim == 64 and case.mask.group_rule != L.GROUP_IDS and len(case.cu_q) > 1 and
                 int(np.diff(case.cu_q).max()) >= 1 and int(np.diff(case.cu_k).max()) <= 128)
    if fits_unit and (L.IMPL_UNIT, L.PREC_FP32) not in kernels:
        kernels = list(kernels) + [(L.IMPL_UNIT, L.PREC_FP32)]   # one 128 x 128 tcgen05 tile per (sequence, head)
    for impl, prec in kernels:
        got, _ = forward_gpu(case, impl, prec)
        what = f"{case.name} impl={impl} prec={prec}"
        if prec == L.PREC_TF32:
            assert_close(got, want, what, atol=TF32_ATOL, rtol=TF32_RTOL)
        else:
            assert_close(got, want, what)
        if impl in (L.IMPL_TCGEN05, L.IMPL_UNIT):
            assert L.load().fblt_tcgen05_error() == 0, "a tcgen05 CTA gave up on a bounded wait"
    return want


def test_c1_byte_self_attention(cuda_lib):
    check(workloads.c1_byte_self_attention())
    check(workloads.c1_byte_self_attention(seq_len=300, window=77))


def test_c2_patch_transformer_attention(cuda_lib):
    case = workloads.c2_patch_attention()
    assert case.q.shape[1] == 512 and len(case.cu_q) == 17
    check(case)


def test_c3_cross_attention(cuda_lib):
    check(workloads.c3_cross_attention("enc"))
    check(workloads.c3_cross_attention("dec_paper"))
    check(workloads.c3_cross_attention("dec_leq"))
    # default dispatch: short ranges -> row kernel, "<=" rule -> tile kernel; both must agree with the oracle
    for d in ("enc", "dec_paper", "dec_leq"):
        check(workloads.c3_cross_attention(d, batch=4), kernels=[(L.IMPL_AUTO, L.PREC_FP32)])


@pytest.mark.parametrize("hd", [32, 64])
@pytest.mark.parametrize("k", [1, 3])
def test_decode_step_cross_tier(cuda_lib, hd, k):
    """Cross-attention of an incremental decode step (infer/kv_cache.c:303-324): n fresh byte rows at
    absolute positions base.. read the tier-2 latents under the mask of infer/kv_cache.c:206-218,
    245-249 -- one latent group per row by the decoder rule, the last row redirected to the final
    latent when the trailing patch is closed. Numeric result of every kernel that takes the shape
    against the reference operator under exactly that host-built mask."""
    seq_bytes = 96
    lens = [synth.geometric_patches(77, s, seq_bytes) for s in range(4)]
    bounds = [synth.bounds_from_lengths(l) for l in lens]
    P = np.array([len(l) for l in lens])
    cu_k = np.concatenate([[0], np.cumsum(P * k)])
    # bases: start of the sequence, inside a patch, on a patch's final byte, rows running past the end
    bases = [0, int(bounds[1][3]) + 1, int(bounds[2][5]) - 1, seq_bytes - 2]
    for n in (1, 4):
        cu_q = np.arange(5) * n
        for tc in ([0, 0, 0, 0], [1, 0, 1, 1]):
            mask = MaskConfig(group_rule=L.GROUP_PATCH_DEC, subtokens=k, patch_bounds=bounds, q_pos_offset=bases,
                              trailing_closed=tc)
            case = random_case(500 + 10 * n + k, cu_q, cu_k, 4, hd, mask)
            want, masks, _ = oracle_forward(case)
            for b in range(4):   # the oracle's mask is the decode step's own
                step_mask = ob.decode_cross_mask(bounds[b], k, n, bases[b], bool(tc[b]))
                assert masks[b].tobytes() == step_mask.tobytes(), (n, k, tc, b)
                assert (step_mask == 0).sum(axis=1).tolist() == [k] * n      # one latent group per row
            check(case)


def test_c5_prefill_sample(cuda_lib):
    check(workloads.c5_prefill(batch=8))


def random_case(seed, cu_q, cu_k, H, hd, mask, std=1.0):
    E = H * hd
    nq, nk = int(cu_q[-1]), int(cu_k[-1])
    q = synth.normal(seed, 1, max(nq, 1) * E, std).reshape(-1, E)[:nq]
    k = synth.normal(seed, 2, max(nk, 1) * E, std).reshape(-1, E)[:nk]
    v = synth.normal(seed, 3, max(nk, 1) * E, std).reshape(-1, E)[:nk]
    return ForwardCase(f"rand{seed}", H, hd, 1.0 / np.sqrt(hd), q, k, v, np.asarray(cu_q, np.int32),
                       np.asarray(cu_k, np.int32), mask)


@pytest.mark.parametrize("hd", [32, 64, 128])
def test_ragged_lengths_all_head_dims(cuda_lib, hd):
    # empty sequence, length 1, lengths around the 64-row tile edge
    cu = np.concatenate([[0], np.cumsum([1, 0, 63, 64, 65, 130, 2, 200])])
    check(random_case(40 + hd, cu, cu, 2, hd, MaskConfig(is_causal=True)))
    check(random_case(41 + hd, cu, cu, 2, hd, MaskConfig(is_causal=True, sliding_window=48)))
    check(random_case(42 + hd, cu, cu, 2, hd, MaskConfig()))  # bidirectional, no mask


@pytest.mark.parametrize("hd", [2, 16, 32, 64, 128])
def test_small_lengths_at_every_edge(cuda_lib, hd):
    """Sequence lengths 1, 2 and one below / at / above the 32- and 128-row edges, for every head_dim
    class (2 and 16 only the per-row kernel takes), causal and windowed, every kernel that takes the
    shape; outputs sit between guard rows (gpu_utils), so a write past a short sequence is caught."""
    lens = [1, 2, 31, 32, 33, 127, 128, 129]
    cu = np.concatenate([[0], np.cumsum(lens)])
    kernels = KERNELS if hd in (32, 64, 128) else [(L.IMPL_ROW, L.PREC_FP32), (L.IMPL_AUTO, L.PREC_FP32)]
    check(random_case(300 + hd, cu, cu, 3, hd, MaskConfig(is_causal=True)), kernels=kernels)
    check(random_case(301 + hd, cu, cu, 3, hd, MaskConfig(is_causal=True, sliding_window=5)), kernels=kernels)
    # cross shape: one query row per sequence over the same key counts
    cu_q = np.arange(len(lens) + 1)
    check(random_case(302 + hd, cu_q, cu, 3, hd, MaskConfig()), kernels=kernels)


def test_unit_kernel_many_units_per_cta(cuda_lib):
    """The persistent unit kernel with more units than CTAs: 700 sequences x 4 heads on one CTA per SM, lengths
    0 .. 128 (empty sequences and full tiles included), so every CTA walks a queue of loads, conversions,
    MMAs and TMA stores of different row counts; then a cross shape with sequences that have queries but
    no keys (zeros, written by the loader) and keys but no queries. Repeated launches must agree bit
    for bit (the roles meet on barriers only)."""
    rng = np.random.default_rng(77)
    lens = rng.integers(0, 129, 700)
    lens[::50] = 128
    lens[7::90] = 0
    cu = np.concatenate([[0], np.cumsum(lens)])
    unit = [(L.IMPL_UNIT, L.PREC_FP32)]
    case = random_case(70, cu, cu, 4, 64, MaskConfig(is_causal=True))
    check(case, kernels=unit)
    first, _ = forward_gpu(case, L.IMPL_UNIT)
    for _ in range(3):
        again, _ = forward_gpu(case, L.IMPL_UNIT)
        assert np.array_equal(first, again)
    check(random_case(71, cu, cu, 4, 64, MaskConfig(is_causal=True, sliding_window=20)), kernels=unit)
    qlens = rng.integers(0, 129, 300)
    klens = rng.integers(0, 129, 300)
    klens[3::17] = 0
    qlens[5::19] = 0
    cu_q, cu_k = np.concatenate([[0], np.cumsum(qlens)]), np.concatenate([[0], np.cumsum(klens)])
    check(random_case(72, cu_q, cu_k, 2, 64, MaskConfig()), kernels=unit)
    # several 128-row query tiles over one sequence's keys (byte rows over a sequence's patches)
    qlens = np.array([700, 1, 128, 129, 0, 300, 513])
    klens = np.array([128, 5, 100, 128, 7, 0, 31])
    cu_q, cu_k = np.concatenate([[0], np.cumsum(qlens)]), np.concatenate([[0], np.cumsum(klens)])
    check(random_case(73, cu_q, cu_k, 4, 64, MaskConfig()), kernels=unit)
    check(random_case(74, cu_q, cu_k, 4, 64, MaskConfig(is_causal=True, causal_offset=[0, 2, 5, 0, 3, 0, 10])),
          kernels=unit)
    assert L.load().fblt_tcgen05_error() == 0


def test_docs_offsets_and_block_infer(cuda_lib):
    cu = np.array([0, 150, 150 + 97])
    docs = [np.array([40, 41, 120]), np.array([64])]
    check(random_case(50, cu, cu, 2, 64, MaskConfig(is_causal=True, doc_bounds=docs)))
    check(random_case(51, cu, cu, 2, 64, MaskConfig(is_causal=False, sliding_window=30, doc_bounds=docs)))
    cu_q, cu_k = np.array([0, 5, 70]), np.array([0, 135, 135 + 201])
    check(random_case(52, cu_q, cu_k, 2, 64, MaskConfig(is_causal=True, causal_offset=[130, 136], sliding_window=100)))
    check(random_case(53, cu, cu, 2, 64, MaskConfig(num_clean=[146, 90])))


def test_rows_without_keys_give_zeros(cuda_lib):
    # window smaller than the causal offset gap: every key masked for the first rows of sequence 1
    cu_q, cu_k = np.array([0, 4, 12]), np.array([0, 10, 30])
    case = random_case(60, cu_q, cu_k, 1, 32, MaskConfig(is_causal=True, causal_offset=[6, 30], sliding_window=3))
    want = check(case)
    assert (want[4:] == 0).all()


def test_explicit_group_ids_row_kernel(cuda_lib):
    rng = np.random.default_rng(8)
    cu_q, cu_k = np.array([0, 40, 75]), np.array([0, 50, 90])
    m = MaskConfig(group_rule=L.GROUP_IDS, q_group_ids=rng.integers(0, 3, 75), k_group_ids=rng.integers(0, 3, 90))
    check(random_case(61, cu_q, cu_k, 2, 48, m), kernels=[(L.IMPL_ROW, L.PREC_FP32), (L.IMPL_AUTO, L.PREC_FP32)])
    case = random_case(62, cu_q, cu_k, 2, 64, m)
    q, k, v = (torch.from_numpy(np.ascontiguousarray(x)).cuda() for x in (case.q, case.k, case.v))
    out = torch.empty((75, 128), device="cuda")
    b = ops.make_batch(q, k, v, out, cu_q, cu_k, 2, 64, 1.0, m, impl=L.IMPL_TILE)
    with pytest.raises(L.FbltError) as e:
        ops.attn_forward(b)
    assert e.value.status == L.ERR_UNSUPPORTED


def test_odd_head_dim_falls_back_to_row_kernel(cuda_lib):
    cu = np.array([0, 33, 70])
    check(random_case(63, cu, cu, 3, 20, MaskConfig(is_causal=True)), kernels=[(L.IMPL_AUTO, L.PREC_FP32)])


def test_full_size_prefill_properties(cuda_lib):
    """Config-5 prefill at full batch (2048 sequences, 16 heads x 64): properties that need no
    CPU pass. (1) softmax weights sum to one: V == 1 gives out == 1 on every row; (2) the two
    independent kernels agree; (3) linearity in V."""
    case = workloads.c5_prefill(batch=2048, with_tensors=False)  # patch structure from the seeded generator
    E = case.embed
    rows = int(case.cu_q[-1])
    gen = torch.Generator(device="cuda").manual_seed(4)
    buf = torch.randn((rows, 3 * E), generator=gen, device="cuda") * 0.125
    q, k, v = buf[:, 0:E], buf[:, E:2 * E], buf[:, 2 * E:]

    def run(vv, impl, prec=L.PREC_FP32):
        out = torch.full((rows, E), float("nan"), device="cuda")
        b = ops.make_batch(q, k, vv, out, case.cu_q, case.cu_k, case.num_heads, case.head_dim, case.scale, case.mask,
                           impl=impl, precision=prec)
        ops.attn_forward(b)
        torch.cuda.synchronize()
        return out

    ones = torch.ones((rows, E), device="cuda")
    o1 = run(ones, L.IMPL_TILE)
    assert float((o1 - 1).abs().max()) < 1e-5
    o_tile = run(v, L.IMPL_TILE)
    o_row = run(v, L.IMPL_ROW)
    err = (o_tile - o_row).abs()
    assert float((err - (1e-4 + 1e-3 * o_row.abs())).max()) <= 0
    o_t5 = run(v, L.IMPL_TCGEN05)
    assert L.load().fblt_tcgen05_error() == 0
    err = (o_t5 - o_row).abs()
    assert float((err - (1e-4 + 1e-3 * o_row.abs())).max()) <= 0
    del o_t5
    v2 = torch.roll(v, 1, 0).contiguous()
    o2 = run(v2, L.IMPL_TILE)
    o12 = run((v + v2).contiguous(), L.IMPL_TILE)
    assert float((o12 - (o_tile + o2)).abs().max()) < 1e-4
    # the first row of every sequence sees only itself: out == v exactly there
    first = torch.from_numpy(case.cu_q[:-1].astype(np.int64)).cuda()
    assert float((o_tile[first] - v[first]).abs().max()) < 1e-6


def test_long_sequences_many_key_tiles(cuda_lib):
    """Eleven 64-key tiles per row block: exercises the running-maximum rescale of the
    accumulator in TMEM (tcgen05 kernel) and the two-stage pipeline (mma.sync kernel)."""
    cu = np.array([0, 700, 700 + 130])
    check(random_case(70, cu, cu, 2, 64, MaskConfig(is_causal=True)))
    check(random_case(71, cu, cu, 2, 64, MaskConfig(is_causal=True, sliding_window=150)))
    check(random_case(72, cu, cu, 2, 64, MaskConfig()))
    # rectangular: 300 queries over 700 keys with a causal offset
    cu_q, cu_k = np.array([0, 300]), np.array([0, 700])
    check(random_case(73, cu_q, cu_k, 2, 64, MaskConfig(is_causal=True, causal_offset=[400])))


@pytest.mark.parametrize("hd", [32, 64, 128])
def test_fused_rotary_embedding(cuda_lib, hd):
    """Unrotated Q/K plus the cos/sin tables: the kernels rotate query row i with position
    i + causal_offset and key row j with position j (the order of models/attention.c:
    rope_apply on Q and K, then the head operator). The oracle rotates on the CPU first."""
    H = 2
    lens_k = [200, 65, 1, 0, 130]
    lens_q = [200, 65, 1, 0, 30]               # last sequence: queries are the tail of the keys
    off = [0, 0, 0, 0, 100]
    cu_q = np.concatenate([[0], np.cumsum(lens_q)])
    cu_k = np.concatenate([[0], np.cumsum(lens_k)])
    cs, sn = ob.rope_tables(256, hd)
    for mask in (MaskConfig(is_causal=True, causal_offset=off),
                 MaskConfig(is_causal=True, sliding_window=48, causal_offset=off)):
        raw = random_case(70 + hd, cu_q, cu_k, H, hd, mask)
        pos_q = np.concatenate([np.arange(n) + o for n, o in zip(lens_q, off)]).astype(np.int64)
        pos_k = np.concatenate([np.arange(n) for n in lens_k]).astype(np.int64)
        rotated = dataclasses.replace(raw, q=ob.rope_apply(raw.q, cs[pos_q], sn[pos_q], H, hd),
                                      k=ob.rope_apply(raw.k, cs[pos_k], sn[pos_k], H, hd))
        want, _, _ = oracle_forward(rotated)
        kernels = KERNELS + (T5_KERNELS if hd == 64 else [])
        for impl, prec in kernels:
            got, _ = forward_gpu(raw, impl, prec, rope=(cs, sn))
            tol = dict(atol=TF32_ATOL, rtol=TF32_RTOL) if prec == L.PREC_TF32 else {}
            assert_close(got, want, f"rope hd={hd} impl={impl} prec={prec}", **tol)


def test_block_diffusion_pass_gathered_positions_and_cross_rule(cuda_lib):
    """The drafter's dense pass (models/block_diffusion.c:139-225): S = N + B rows, block rows carry
    their recorded positions for the rotary embedding, self-attention under the INFER rule, and
    cross-attention where clean rows read latent_at(i) and block rows the last latent."""
    H, hd, B = 2, 64, 4
    Ns = [60, 9, 130]
    S = [n + B for n in Ns]
    cu = np.concatenate([[0], np.cumsum(S)]).astype(np.int32)
    cs, sn = ob.rope_tables(512, hd)
    rng = np.random.default_rng(7)
    pos = np.concatenate([np.concatenate([np.arange(n), n + rng.permutation(40)[:B]]) for n in Ns]).astype(np.int64)
    raw = random_case(95, cu, cu, H, hd, MaskConfig(num_clean=Ns))
    rotated = dataclasses.replace(raw, q=ob.rope_apply(raw.q, cs[pos], sn[pos], H, hd),
                                  k=ob.rope_apply(raw.k, cs[pos], sn[pos], H, hd))
    want, _, _ = oracle_forward(rotated)
    for impl, prec in KERNELS + T5_KERNELS:
        got, _ = forward_gpu(raw, impl, prec, rope=(cs, sn), rope_pos=(pos, pos))
        tol = dict(atol=TF32_ATOL, rtol=TF32_RTOL) if prec == L.PREC_TF32 else {}
        assert_close(got, want, f"diffusion self impl={impl} prec={prec}", **tol)
    # cross-attention of the same pass: queries = the S rows, keys = P latents
    bounds = [synth.bounds_from_lengths(synth.geometric_patches(31, b, n)) for b, n in enumerate(Ns)]
    P = [len(x) - 1 for x in bounds]
    cu_k = np.concatenate([[0], np.cumsum(P)]).astype(np.int32)
    for trailing in ([0, 0, 0], [1, 0, 1]):
        mask = MaskConfig(group_rule=L.GROUP_PATCH_DEC, patch_bounds=bounds, num_clean=Ns, trailing_closed=trailing)
        check(random_case(96, cu, cu_k, H, hd, mask), kernels=[(L.IMPL_ROW, L.PREC_FP32), (L.IMPL_AUTO, L.PREC_FP32)])


def test_rotary_tables_are_validated(cuda_lib):
    cs, sn = ob.rope_tables(64, 32)
    case = random_case(90, [0, 8], [0, 8], 1, 32, MaskConfig(is_causal=True))
    q, k, v = (torch.from_numpy(x).cuda() for x in (case.q, case.k, case.v))
    out = torch.empty_like(q)
    batch = ops.make_batch(q, k, v, out, case.cu_q, case.cu_k, 1, 32, case.scale, case.mask,
                           rope_cos=torch.from_numpy(cs).cuda(), rope_sin=torch.from_numpy(sn).cuda())
    batch.desc.rope_sin = None                  # one table without the other
    with pytest.raises(L.FbltError):
        ops.attn_forward(batch)


def test_environment_toggles(cuda_lib, monkeypatch):
    """FBLT_ATTN_IMPL / FBLT_ATTN_PRECISION steer descriptors that ask for the defaults, are read at
    every call, and reject unknown values."""
    case = random_case(91, [0, 40, 150], [0, 40, 150], 2, 32, MaskConfig(is_causal=True))
    want, _, _ = oracle_forward(case)
    for name in ("auto", "row", "quad", "tile"):
        monkeypatch.setenv("FBLT_ATTN_IMPL", name)
        got, _ = forward_gpu(case, L.IMPL_AUTO, L.PREC_FP32)
        assert_close(got, want, f"FBLT_ATTN_IMPL={name}")
    monkeypatch.setenv("FBLT_ATTN_IMPL", "tcgen05")          # honoured: that kernel does not take head_dim 32
    with pytest.raises(L.FbltError):
        forward_gpu(case, L.IMPL_AUTO, L.PREC_FP32)
    got, _ = forward_gpu(case, L.IMPL_TILE, L.PREC_FP32)     # an explicit choice in the descriptor wins
    assert_close(got, want, "explicit impl beside the toggle")
    monkeypatch.setenv("FBLT_ATTN_IMPL", "fastest")
    with pytest.raises(L.FbltError):
        forward_gpu(case, L.IMPL_AUTO, L.PREC_FP32)
    monkeypatch.setenv("FBLT_ATTN_IMPL", "tile")
    monkeypatch.setenv("FBLT_ATTN_PRECISION", "tf32")
    got_tf32, _ = forward_gpu(case, L.IMPL_AUTO, L.PREC_FP32)
    assert_close(got_tf32, want, "FBLT_ATTN_PRECISION=tf32", atol=TF32_ATOL, rtol=TF32_RTOL)
    assert np.abs(got_tf32 - want).max() > np.abs(got - want).max()   # single-pass rounding is visible
    monkeypatch.setenv("FBLT_ATTN_PRECISION", "bf16")
    with pytest.raises(L.FbltError):
        forward_gpu(case, L.IMPL_AUTO, L.PREC_FP32)


def test_non_finite_scores_weigh_zero(cuda_lib):
    """A key whose score is not finite (infinity or any NaN bit pattern in its K row) carries weight
    0 for every query, as in ops/vecmath_cpu.c:33-52; the other keys are unaffected."""
    cu = np.array([0, 150], dtype=np.int32)
    case = random_case(77, cu, cu, 2, 64, MaskConfig(is_causal=True))
    k = case.k.copy()
    k[5, 3] = np.inf
    k[17, 64 + 9] = -np.inf
    k[40, 20] = np.nan
    kv = k.view(np.uint32)
    kv[66, 1] = 0x7FFFFFFF            # NaN with every payload bit set
    kv[101, 70] = 0xFFFFF001          # negative NaN, large payload
    case = dataclasses.replace(case, k=k)
    want, _, _ = oracle_forward(case)
    assert np.isfinite(want).all()
    for impl, prec in KERNELS + T5_KERNELS + [(L.IMPL_ROW_QUAD, L.PREC_FP32)]:
        got, _ = forward_gpu(case, impl, prec)
        assert np.isfinite(got).all(), (impl, prec)
        tol = dict(atol=TF32_ATOL, rtol=TF32_RTOL) if prec == L.PREC_TF32 else {}
        assert_close(got, want, f"non-finite keys impl={impl} prec={prec}", **tol)
