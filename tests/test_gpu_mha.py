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
    # patch-transformer shape: sequences of at most 128 rows, head_dim 64 -- the projection's epilogue rotates
    # Q / K and the TMA-fed unit kernel does the attention
    got, want = run_case(512, 8, [128, 77, 1, 0, 100, 128], 5, use_rope=True)
    assert_close(got, want, "mha rope, unit kernel")
    got, want = run_case(256, 4, [64, 128], 6, use_rope=True, window=32)
    assert_close(got, want, "mha rope window, unit kernel")
    got, want = run_case(96, 3, [50, 20], 7, use_rope=True)                   # embed not a multiple of 32: rotation in the loads
    assert_close(got, want, "mha rope, head_dim 32, odd embed")


def test_mha_block_tf32_mode(cuda_lib):
    got, want = run_case(256, 4, [128, 77], 4, use_rope=True, precision=L.PREC_TF32)
    assert_close(got, want, "mha tf32", atol=5e-3, rtol=2e-2)     # single-pass TF32 in all three stages


def packed_kv(wk: np.ndarray, wv: np.ndarray) -> ops.PackedWeights:
    """[weight_k | weight_v] as one packed [E, 2E] weight."""
    return ops.PackedWeights(torch.from_numpy(np.ascontiguousarray(np.concatenate([wk, wv], axis=1))).cuda())


@pytest.mark.parametrize("direction", ["enc", "dec"])
def test_cross_attention_block_matches_reference(cuda_lib, direction):
    """Encoder (patch queries over their own bytes) and decoder (byte queries over their latent)
    cross-attention blocks against blt_cross_attention_forward run on the CPU with the
    group-id arrays its callers build (models/local_encoder.c:70-74, models/local_decoder.c:82-94)."""
    if not ob.have_ref():
        pytest.skip("reference object code not built")
    from fblt_b200 import synth
    E, H = 256, 4
    rng = np.random.default_rng(21)
    nbytes = [200, 64, 17]
    bounds = [synth.bounds_from_lengths(synth.geometric_patches(41, b, n)) for b, n in enumerate(nbytes)]
    P = [len(x) - 1 for x in bounds]
    wq, wk, wv, wp = ((rng.standard_normal((E, E)) / np.sqrt(E)).astype(np.float32) for _ in range(4))
    if direction == "enc":
        q_rows, k_rows = P, nbytes
        mask = MaskConfig(group_rule=L.GROUP_PATCH_ENC, patch_bounds=bounds)
    else:
        q_rows, k_rows = nbytes, P
        mask = MaskConfig(group_rule=L.GROUP_PATCH_DEC, patch_bounds=bounds, trailing_closed=[1, 0, 1])
    cu_q = np.concatenate([[0], np.cumsum(q_rows)]).astype(np.int32)
    cu_k = np.concatenate([[0], np.cumsum(k_rows)]).astype(np.int32)
    xq = rng.standard_normal((int(cu_q[-1]), E)).astype(np.float32)
    xk = rng.standard_normal((int(cu_k[-1]), E)).astype(np.float32)
    want = np.zeros_like(xq)
    for b in range(len(nbytes)):
        _, byte_patch = ob.patch_group_ids(bounds[b], use_ref=True)
        if direction == "enc":
            qg, kg = np.arange(P[b]), byte_patch[:nbytes[b]]
        else:
            qg = np.array([ob.latent_at(bounds[b], i, use_ref=True) for i in range(nbytes[b])])
            if mask.trailing_closed[b]:
                qg[-1] = P[b] - 1
            kg = np.arange(P[b])
        want[cu_q[b]:cu_q[b + 1]] = ob.ref_cross_attention(xq[cu_q[b]:cu_q[b + 1]], xk[cu_k[b]:cu_k[b + 1]], wq, wk, wv, wp,
                                                           H, qg, kg)
    got = ops.cross_attention_forward(torch.from_numpy(xq).cuda(), torch.from_numpy(xk).cuda(),
                                      ops.PackedWeights(torch.from_numpy(wq).cuda()), packed_kv(wk, wv),
                                      ops.PackedWeights(torch.from_numpy(wp).cuda()), cu_q, cu_k, H, mask)
    assert L.load().fblt_tcgen05_error() == 0
    assert_close(got.cpu().numpy(), want, f"cross block {direction}")


@pytest.mark.parametrize("block_mode,window", [(False, 0), (True, 0), (False, 24)])
def test_kv_decode_step_self_attention_block(cuda_lib, block_mode, window):
    """fblt_kv_self_attention_step against the same chain built from the reference's CPU pieces in
    the order of infer/kv_cache.c:338-396: matmul, rotary embedding at position base + r, rows
    written through to the cache, the head operator over the cache, matmul."""
    if not ob.have_ref():
        pytest.skip("reference object code not built")
    from fblt_b200 import workloads
    from helpers import oracle_decode
    H, hd, n, batch, cache_rows = 4, 64, 4, 5, 256
    E = H * hd
    rng = np.random.default_rng(33)
    base = np.array([10, 64, 200, 33, 0], dtype=np.int32)
    case = workloads.decode_case(130, batch, H, n, block_mode, lens=base, cache_rows=cache_rows)
    case.window = window
    x = rng.standard_normal((batch * n, E)).astype(np.float32)
    w_qkv = (rng.standard_normal((E, 3 * E)) / np.sqrt(E)).astype(np.float32)
    w_proj = (rng.standard_normal((E, E)) / np.sqrt(E)).astype(np.float32)
    cs, sn = ob.rope_tables(cache_rows, hd, use_ref=True)
    # reference chain
    qkv = ob.matmul(x, w_qkv, use_ref=True)
    pos = (base[:, None] + np.arange(n)[None, :]).reshape(-1)
    case.q = ob.rope_apply(qkv[:, :E], cs[pos], sn[pos], H, hd, use_ref=True)
    case.k_new = ob.rope_apply(qkv[:, E:2 * E], cs[pos], sn[pos], H, hd, use_ref=True)
    case.v_new = np.ascontiguousarray(qkv[:, 2 * E:])
    combined, _ = oracle_decode(case)
    want = ob.matmul(combined, w_proj, use_ref=True)
    # device
    kc, vc = torch.from_numpy(case.k_cache).cuda(), torch.from_numpy(case.v_cache).cuda()
    got = ops.kv_self_attention_step(torch.from_numpy(x).cuda(), ops.PackedWeights(torch.from_numpy(w_qkv).cuda()),
                                     ops.PackedWeights(torch.from_numpy(w_proj).cuda()), kc, vc,
                                     torch.from_numpy(base).cuda(), H, n, rope_cos=torch.from_numpy(cs).cuda(),
                                     rope_sin=torch.from_numpy(sn).cuda(), block_mode=block_mode, window=window,
                                     max_len=int(base.max()) + n)
    assert L.load().fblt_tcgen05_error() == 0
    assert_close(got.cpu().numpy(), want, f"kv step block_mode={block_mode} window={window}")
    # write-through: the cache rows base .. base + n now hold the rotated K and the V rows
    for b in range(batch):
        rows = slice(int(base[b]), int(base[b]) + n)
        assert_close(kc[b, rows].cpu().numpy(), case.k_new[b * n:(b + 1) * n], f"cache K rows of sequence {b}")
        assert_close(vc[b, rows].cpu().numpy(), case.v_new[b * n:(b + 1) * n], f"cache V rows of sequence {b}")


def test_kv_decode_steps_replayed_from_a_cuda_graph(cuda_lib):
    """Eight decode steps captured once (step + length update) and replayed while the caches grow:
    outputs and caches must equal the eager loop bit for bit, because the launches read the cache
    lengths from device memory and allocate nothing."""
    H, hd, n, batch, cache_rows, steps = 4, 64, 4, 6, 128, 8
    E = H * hd
    rng = np.random.default_rng(77)
    base0 = np.array([0, 3, 17, 40, 64, 90], dtype=np.int32)
    xs = torch.from_numpy(rng.standard_normal((steps, batch * n, E)).astype(np.float32)).cuda()
    wq_h = (rng.standard_normal((E, 3 * E)) / np.sqrt(E)).astype(np.float32)
    wp_h = (rng.standard_normal((E, E)) / np.sqrt(E)).astype(np.float32)
    w_qkv, w_proj = ops.PackedWeights(torch.from_numpy(wq_h).cuda()), ops.PackedWeights(torch.from_numpy(wp_h).cuda())
    csn, snn = ob.rope_tables(cache_rows, hd, use_ref=False)
    cs, sn = torch.from_numpy(csn).cuda(), torch.from_numpy(snn).cuda()
    cache0 = torch.from_numpy(rng.standard_normal((2, batch, cache_rows, E)).astype(np.float32)).cuda()

    def fresh():
        kc, vc = cache0[0].clone(), cache0[1].clone()
        base = torch.from_numpy(base0).cuda()
        return kc, vc, base, ops.KvStepPlan(w_qkv, w_proj, kc, vc, base, H, n, rope_cos=cs, rope_sin=sn)

    # eager loop
    kc_e, vc_e, base_e, plan_e = fresh()
    outs_e = []
    for t in range(steps):
        plan_e.x.copy_(xs[t])
        plan_e.run()
        base_e.add_(n)
        outs_e.append(plan_e.out.clone())
    torch.cuda.synchronize()

    # captured once, replayed
    kc_g, vc_g, base_g, plan_g = fresh()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        plan_g.x.copy_(xs[0])
        with torch.cuda.graph(graph, stream=side):
            plan_g.run(side)
            base_g.add_(n)
    torch.cuda.current_stream().wait_stream(side)
    # the capture itself ran nothing: caches and lengths are still the initial ones
    assert torch.equal(base_g.cpu(), torch.from_numpy(base0))
    outs_g = []
    for t in range(steps):
        plan_g.x.copy_(xs[t])
        graph.replay()
        outs_g.append(plan_g.out.clone())
    torch.cuda.synchronize()
    assert L.load().fblt_tcgen05_error() == 0
    assert torch.equal(base_g.cpu(), torch.from_numpy(base0 + steps * n))
    for t in range(steps):
        assert torch.equal(outs_g[t], outs_e[t]), f"step {t}: graph replay differs from the eager launch"
    assert torch.equal(kc_g, kc_e) and torch.equal(vc_g, vc_e)
    # and the last step agrees with the CPU chain over the cache the loop has built
    from helpers import oracle_decode
    from fblt_b200 import workloads
    base_last = base0 + (steps - 1) * n
    case = workloads.decode_case(1, batch, H, n, False, lens=base_last, cache_rows=cache_rows)
    case.k_cache, case.v_cache = kc_e.cpu().numpy(), vc_e.cpu().numpy()
    qkv = ob.matmul(xs[-1].cpu().numpy(), wq_h, use_ref=False)
    pos = (base_last[:, None] + np.arange(n)[None, :]).reshape(-1)
    case.q = ob.rope_apply(qkv[:, :E], csn[pos], snn[pos], H, hd, use_ref=False)
    case.k_new = ob.rope_apply(qkv[:, E:2 * E], csn[pos], snn[pos], H, hd, use_ref=False)
    case.v_new = np.ascontiguousarray(qkv[:, 2 * E:])
    combined, _ = oracle_decode(case, ref=False)
    want = ob.matmul(combined, wp_h, use_ref=False)
    assert_close(outs_e[-1].cpu().numpy(), want, "last replayed step against the CPU chain")


def test_blocks_against_committed_fixtures(cuda_lib):
    """The committed outputs of the reference's own CPU code (tests/golden/make_golden.py) for the
    projection matmul and the two attention blocks: no reference object code needed at run time."""
    from pathlib import Path
    golden = Path(__file__).resolve().parent / "golden"
    seen = set()
    for f in sorted(golden.glob("*.npz")):
        g = np.load(f)
        kind = str(g["kind"])
        if kind == "matmul":
            w = ops.PackedWeights(torch.from_numpy(g["b"]).cuda())
            a = np.zeros((g["a"].shape[0], 52), np.float32)
            a[:, :g["a"].shape[1]] = g["a"]
            got = ops.matmul(torch.from_numpy(a).cuda()[:, :g["a"].shape[1]], w).cpu().numpy()
        elif kind == "mha":
            H, T, E = int(g["num_heads"]), g["x"].shape[0], g["x"].shape[1]
            rope = {}
            if bool(g["use_rope"]):
                cs, sn = ob.rope_tables(T, E // H)
                rope = dict(rope_cos=torch.from_numpy(cs).cuda(), rope_sin=torch.from_numpy(sn).cuda())
            got = ops.mha_forward(torch.from_numpy(g["x"]).cuda(), ops.PackedWeights(torch.from_numpy(g["w_qkv"]).cuda()),
                                  ops.PackedWeights(torch.from_numpy(g["w_proj"]).cuda()), [0, T], H,
                                  MaskConfig(is_causal=True, sliding_window=int(g["window"])), **rope).cpu().numpy()
        elif kind == "cross":
            H, bounds = int(g["num_heads"]), g["bounds"]
            got = ops.cross_attention_forward(
                torch.from_numpy(g["xq"]).cuda(), torch.from_numpy(g["xk"]).cuda(),
                ops.PackedWeights(torch.from_numpy(g["wq"]).cuda()), packed_kv(g["wk"], g["wv"]),
                ops.PackedWeights(torch.from_numpy(g["wp"]).cuda()), [0, g["xq"].shape[0]], [0, g["xk"].shape[0]], H,
                MaskConfig(group_rule=L.GROUP_PATCH_ENC, patch_bounds=[bounds])).cpu().numpy()
        else:
            continue
        seen.add(kind)
        assert L.load().fblt_tcgen05_error() == 0
        assert_close(got, g["out"], f.name)
    assert seen == {"matmul", "mha", "cross"}
