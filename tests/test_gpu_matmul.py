"""Projection matmul (fblt_matmul, tcgen05) against the CPU matmul of the reference and an
exact float64 product: ragged shapes, depth not a multiple of the 32-deep step, row strides,
bias, both precisions."""
import numpy as np
import pytest
import torch

from fblt_b200 import lib as L
from fblt_b200 import ops
from oracle import binding as ob

pytestmark = pytest.mark.gpu

# Single-pass TF32 rounds both factors to 11 bits: stated tolerance of that mode, relative
# to sqrt(K) (the size of a sum of K unit-variance products).
TF32_REL = 2e-3


def run(a, b, bias=None, precision=L.PREC_FP32, lda=None, ldo=None):
    m, k = a.shape
    n = b.shape[1]
    a_d = torch.zeros(m, lda or k, dtype=torch.float32, device="cuda")
    a_d[:, :k] = torch.from_numpy(a)
    w = ops.PackedWeights(torch.from_numpy(b).cuda())
    out_full = torch.full((m, ldo or n), float("nan"), dtype=torch.float32, device="cuda")
    out = out_full[:, :n]
    ops.matmul(a_d[:, :k], w, out=out, bias=None if bias is None else torch.from_numpy(bias).cuda(), precision=precision)
    torch.cuda.synchronize()
    assert L.load().fblt_tcgen05_error() == 0, "a matmul CTA gave up on a bounded wait"
    if ldo and ldo > n:
        assert torch.isnan(out_full[:, n:]).all(), "columns past N were written"
    return out.cpu().numpy()


def check(m, k, n, seed, *, bias=False, lda=None, ldo=None):
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = (rng.standard_normal((k, n)) / np.sqrt(k)).astype(np.float32)
    bv = rng.standard_normal(n).astype(np.float32) if bias else None
    exact = a.astype(np.float64) @ b.astype(np.float64) + (0.0 if bv is None else bv.astype(np.float64))
    want = ob.matmul(a, b, use_ref=ob.have_ref()) + (0.0 if bv is None else bv)
    ref_err = float(np.abs(want - exact).max()) if want.size else 0.0
    got = run(a, b, bv, L.PREC_FP32, lda, ldo)
    err = float(np.abs(got - exact).max()) if got.size else 0.0
    # Three-pass TF32 with fp32 accumulation in the tensor core, which truncates on every
    # addition into the accumulator: a small multiple of the CPU loop's own rounding error,
    # and inside the operator's tolerance (max-abs 1e-4 / rel 1e-3) against the CPU result.
    assert err <= max(8.0 * ref_err, 2e-6), (m, k, n, err, ref_err)
    np.testing.assert_allclose(got, want, rtol=1e-3, atol=1e-4)
    got1 = run(a, b, bv, L.PREC_TF32, lda, ldo)
    if not exact.size:
        return
    assert float(np.abs(got1 - exact).max()) <= TF32_REL * max(1.0, float(np.abs(exact).max())), (m, k, n)


def test_matmul_projection_shapes(cuda_lib):
    check(256, 1024, 3072, 1)           # QKV projection of a 256-row batch, E = 1024
    check(300, 1024, 1024, 2)           # output projection, ragged rows


def test_matmul_ragged_and_strided(cuda_lib):
    check(1, 4, 1, 3)
    check(5, 36, 7, 4)                  # depth not a multiple of 32, N not a multiple of 4
    check(129, 100, 130, 5, bias=True)
    check(128, 32, 128, 6, lda=40, ldo=132)
    check(257, 520, 260, 7, bias=True, lda=524, ldo=261)   # odd output stride: scalar stores
    check(0, 64, 64, 8)


def test_matmul_argument_checks(cuda_lib):
    a = torch.zeros(8, 6, device="cuda")
    w = ops.PackedWeights(torch.zeros(6, 8, device="cuda"))
    with pytest.raises(L.FbltError) as e:
        ops.matmul(a, w)                # K = 6 is not a multiple of 4
    assert e.value.status == L.ERR_UNSUPPORTED
