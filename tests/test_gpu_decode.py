"""KV-cache decode / block-verify attention (fblt_attn_decode) against the CPU oracle."""
import numpy as np
import pytest
import torch

from fblt_b200 import lib as L
from fblt_b200 import ops, workloads
from gpu_utils import decode_gpu
from helpers import assert_close, oracle_decode

pytestmark = pytest.mark.gpu


def check(case, **kw):
    want, _ = oracle_decode(case)
    got, kc, vc = decode_gpu(case, **kw)
    assert_close(got, want, f"{case.name} {kw}")
    return got, kc, vc


def test_c4_decode_and_block_verify(cuda_lib):
    dec = workloads.c4_decode()
    assert dec.k_cache.shape[0] == 256 and dec.base_len.min() >= 64 and dec.base_len.max() <= 512
    check(dec)
    blk = workloads.c4_block_verify()
    got, kc, vc = check(blk)
    # write-through (infer/kv_cache.c:352-365): the appended rows are in the cache, bit for bit,
    # and no other row changed
    n, E = blk.n_new, blk.embed
    kc_h, vc_h = kc.cpu().numpy(), vc.cpu().numpy()
    for b in (0, 1, 17, 255):
        base = int(blk.base_len[b])
        assert kc_h[b, base:base + n].tobytes() == blk.k_new[b * n:(b + 1) * n].tobytes()
        assert vc_h[b, base:base + n].tobytes() == blk.v_new[b * n:(b + 1) * n].tobytes()
        assert kc_h[b, :base].tobytes() == blk.k_cache[b, :base].tobytes()
        assert (kc_h[b, base + n:] == 0).all()
    # same result when the rows are already in the cache and when the key range is split
    got2, _, _ = decode_gpu(blk, fused_append=False)
    assert_close(got2, got, "pre-appended vs fused", atol=1e-6, rtol=1e-5)
    for s in (2, 5):
        got3, _, _ = decode_gpu(blk, splits=s)
        assert_close(got3, got, f"splits={s}", atol=1e-6, rtol=1e-5)


@pytest.mark.parametrize("n_new", [1, 2, 3, 4, 5, 8, 13, 16, 32])
@pytest.mark.parametrize("block_mode", [False, True])
def test_query_counts_and_modes(cuda_lib, n_new, block_mode):
    lens = [0, 1, 5, 31, 32, 33, 64, 100, 257]
    case = workloads.decode_case(70 + n_new, len(lens), 2, n_new, block_mode, lens=lens)
    check(case)                     # the library's choice of pieces
    check(case, splits=-1)          # persistent grid over equal shares
    check(case, fused_append=False, splits=3)


@pytest.mark.parametrize("window", [1, 3, 16, 50])
def test_sliding_window(cuda_lib, window):
    lens = [0, 2, 40, 200]
    for n_new in (1, 4, 7):
        case = workloads.decode_case(80 + window, len(lens), 2, n_new, False, lens=lens, window=window)
        check(case)
        check(case, splits=4, fused_append=False)


@pytest.mark.parametrize("hd", [32, 128])
def test_other_head_dims(cuda_lib, hd):
    rng = np.random.default_rng(hd)
    case = workloads.decode_case(90, 5, 2, 4, True, lens=[3, 70, 129, 64, 300])
    # rebuild the tensors for this head_dim (decode_case is fixed at 64)
    E = 2 * hd
    shp = case.k_cache.shape[:2] + (E,)
    case.head_dim = hd
    case.scale = 1.0 / np.sqrt(hd)
    case.k_cache = rng.standard_normal(shp).astype(np.float32)
    case.v_cache = rng.standard_normal(shp).astype(np.float32)
    case.q, case.k_new, case.v_new = (rng.standard_normal((5 * 4, E)).astype(np.float32) for _ in range(3))
    check(case)
    case.block_mode = False
    check(case, splits=2)


@pytest.mark.parametrize("shape", ["few_long", "many_short", "ragged_window", "one"])
def test_stream_form_partitions(cuda_lib, shape):
    """The persistent form cuts the (sequence, head, key block) space into equal shares: units that span
    many CTAs, CTAs that cover many units, shares that begin and end inside a unit, empty sequences."""
    rng = np.random.default_rng(12)
    if shape == "few_long":
        case = workloads.decode_case(301, 3, 2, 4, True, lens=[4000, 1, 2500])
    elif shape == "many_short":
        case = workloads.decode_case(302, 700, 4, 1, False, lens=rng.integers(0, 90, 700))
    elif shape == "ragged_window":
        case = workloads.decode_case(303, 37, 2, 7, False, lens=rng.integers(0, 600, 37), window=130)
    else:
        case = workloads.decode_case(304, 1, 1, 2, True, lens=[777])
    got_s, _, _ = check(case, splits=-1)
    got_g, _, _ = check(case, splits=1)
    assert_close(got_s, got_g, "stream vs grid", atol=1e-6, rtol=1e-5)
    check(case, splits=-1, fused_append=False)


def test_zero_weight_keys_ignore_their_values(cuda_lib):
    """A key a row does not see contributes nothing even when its value row holds Inf or NaN (the
    reference skips zero weights, ops/attn_core_cpu.c:48): rows in front of the window and, for the
    earlier rows of a causal block, the appended rows behind them."""
    n, window = 4, 40
    case = workloads.decode_case(305, 3, 2, n, False, lens=[100, 64, 300], window=window)
    want, _ = oracle_decode(case)
    for b, base in enumerate(case.base_len):
        case.v_cache[b, :max(0, int(base) + 1 - window)] = np.inf        # before every row's window
        case.v_cache[b, max(0, int(base) + 1 - window)] = 1.0e30          # seen by row 0 only: finite, large
    case.v_new[n - 1::n] = np.nan                                         # last appended row: only row n-1 sees it
    want2, _ = oracle_decode(case)
    keep = np.ones(len(want), bool)
    keep[n - 1::n] = False
    for sp in (0, 1, 2):
        got, _, _ = decode_gpu(case, splits=sp)
        assert np.isfinite(got[keep]).all(), f"splits={sp}"
        assert_close(got[keep], want2[keep], f"zero-weight values, splits={sp}", atol=1e-4, rtol=1e-3)


def test_c5_decode_sample(cuda_lib):
    case = workloads.c5_decode(batch=6, base_len=512, steps=2)
    check(case)
    case2 = workloads.c5_decode(batch=3, base_len=764, steps=1)
    check(case2)


def test_workspace_and_argument_errors(cuda_lib):
    case = workloads.decode_case(95, 2, 2, 4, True, lens=[300, 400])
    kc, vc = torch.from_numpy(case.k_cache).cuda(), torch.from_numpy(case.v_cache).cuda()
    base, q = torch.from_numpy(case.base_len).cuda(), torch.from_numpy(case.q).cuda()
    out = torch.empty_like(q)
    d = ops.make_decode(kc, vc, base, q, out, 2, 64, 4, 0.125, block_mode=True, splits=4)
    with pytest.raises(L.FbltError) as e:
        ops.attn_decode(d, None)
    assert e.value.status == L.ERR_WORKSPACE
    d2 = ops.make_decode(kc, vc, base, q[:, 1:], out, 2, 64, 4, 0.125)
    with pytest.raises(L.FbltError) as e:
        ops.attn_decode(d2, None)
    assert e.value.status == L.ERR_ARG


def test_full_size_decode_properties(cuda_lib):
    """Config-5 decode at full batch (2048 sequences, 16 heads x 64, B = 4, 768-row caches):
    (1) V == 1 gives out == 1; (2) split-K agrees with the single pass; (3) a block-verify
    step equals the same rows computed by the prefill kernel with a causal offset."""
    B, H, hd, n, base_len, rows = 2048, 16, 64, 4, 764, 768
    E = H * hd
    gen = torch.Generator(device="cuda").manual_seed(44)
    kc = torch.randn((B, rows, E), generator=gen, device="cuda")
    vc = torch.randn((B, rows, E), generator=gen, device="cuda")
    q = torch.randn((B * n, E), generator=gen, device="cuda")
    base = torch.full((B,), base_len, dtype=torch.int32, device="cuda")
    out = torch.full((B * n, E), float("nan"), device="cuda")

    def run(vcache, splits=0, block=True):
        d = ops.make_decode(kc, vcache, base, q, out, H, hd, n, 0.125, block_mode=block, max_len=rows, splits=splits)
        ops.attn_decode(d, ops.decode_workspace(d))
        torch.cuda.synchronize()
        return out.clone()

    o1 = run(torch.ones_like(vc))
    assert float((o1 - 1).abs().max()) < 1e-5
    del o1
    o_a = run(vc)
    o_b = run(vc, splits=3)
    assert float((o_a - o_b).abs().max()) < 1e-5
    # causal rows through the streaming kernel vs the tile kernel with causal_offset = base_len
    o_c = run(vc, block=False)
    sub = 64  # sequences compared through the second implementation
    cu_q = np.arange(sub + 1, dtype=np.int32) * n
    cu_k = np.arange(sub + 1, dtype=np.int32) * rows
    out2 = torch.empty((sub * n, E), device="cuda")
    batch = ops.make_batch(q[:sub * n], kc[:sub].reshape(sub * rows, E), vc[:sub].reshape(sub * rows, E), out2,
                           cu_q, cu_k, H, hd, 0.125, ops.MaskConfig(is_causal=True, causal_offset=[base_len] * sub),
                           impl=L.IMPL_TILE)
    ops.attn_forward(batch)
    torch.cuda.synchronize()
    err = (out2 - o_c[:sub * n]).abs()
    assert float((err - (1e-4 + 1e-3 * out2.abs())).max()) <= 0


@pytest.mark.parametrize("n_new,block_mode", [(1, False), (4, True), (6, False)])
def test_fused_rotary_prologue(cuda_lib, n_new, block_mode):
    """q / k_new handed over un-rotated with the rotary tables: the kernel must give what the
    reference gives when it rotates per head first (infer/kv_cache.c:347-366) and then attends,
    and the K rows it writes through must equal the CPU-rotated rows bit for bit."""
    import copy
    from oracle import binding as ob
    from helpers import use_ref
    lens = np.array([0, 5, 130, 300], dtype=np.int32)
    case = workloads.decode_case(150 + n_new, len(lens), 4, n_new, block_mode, lens=lens)
    H, hd, E = case.num_heads, case.head_dim, case.embed
    cos_t, sin_t = ob.rope_tables(512, hd, use_ref=use_ref())
    pos = (lens[:, None] + np.arange(n_new)[None, :]).reshape(-1)
    rot = copy.copy(case)
    rot.q = ob.rope_apply(case.q, cos_t[pos], sin_t[pos], H, hd, use_ref=use_ref())
    rot.k_new = ob.rope_apply(case.k_new, cos_t[pos], sin_t[pos], H, hd, use_ref=use_ref())
    want, _ = oracle_decode(rot)

    kc, vc = torch.from_numpy(case.k_cache).cuda(), torch.from_numpy(case.v_cache).cuda()
    base, q = torch.from_numpy(case.base_len).cuda(), torch.from_numpy(case.q).cuda()
    kn, vn = torch.from_numpy(case.k_new).cuda(), torch.from_numpy(case.v_new).cuda()
    out = torch.full_like(q, float("nan"))
    cos_d, sin_d = torch.from_numpy(cos_t).cuda(), torch.from_numpy(sin_t).cuda()   # must outlive the descriptor
    for splits in (1, 3):
        d = ops.make_decode(kc, vc, base, q, out, H, hd, n_new, case.scale, block_mode=block_mode, k_new=kn, v_new=vn,
                            max_len=int(lens.max()) + n_new, splits=splits, rope_cos=cos_d, rope_sin=sin_d)
        ops.attn_decode(d, ops.decode_workspace(d))
        torch.cuda.synchronize()
        assert_close(out.cpu().numpy(), want, f"fused rotary splits={splits}")
    kc_h = kc.cpu().numpy()
    for b in range(len(lens)):
        got = kc_h[b, lens[b]:lens[b] + n_new]
        assert got.tobytes() == rot.k_new[b * n_new:(b + 1) * n_new].tobytes()
