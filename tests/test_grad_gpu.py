"""Both gradient products of a matrix multiplication in one launch, against the oracle's
two accumulating products (the operand table of the reference's backward pass)."""
import numpy as np
import pytest
import torch

from niutensor_b200 import capi, ops
from niutensor_b200.capi import X_TRANS, X_NOTRANS
from oracle.oracle import grad_matmul, rel_fro, round_to_half

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {torch.float32: 1e-5, torch.float16: 2e-3}


def dev(x, dtype):
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV).to(dtype)


def stored(rng, lead, rows, cols, trans):
    shp = tuple(lead) + ((cols, rows) if trans == X_TRANS else (rows, cols))
    return rng.uniform(-1.0, 1.0, shp).astype(np.float32)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("tA", [X_TRANS, X_NOTRANS])
@pytest.mark.parametrize("tB", [X_TRANS, X_NOTRANS])
def test_gradient_pair(dtype, tA, tB, oracle):
    rng = np.random.default_rng(500 + 2 * tA + tB)
    L = capi.lib()
    # aligned shapes take one grouped tensor-core launch; the ragged one two FFMA launches
    for (lead, M, N, K, alpha, launches) in [((), 256, 136, 192, 1.0, 1), ((3,), 72, 200, 64, 0.5, 1),
                                             ((), 512, 512, 512, 1.0, 1), ((2,), 37, 29, 53, 1.0, 2)]:
        a = stored(rng, lead, M, K, tA)
        b = stored(rng, lead, K, N, tB)
        dedc = rng.normal(size=lead + (M, N)).astype(np.float32)
        deda0 = rng.normal(size=a.shape).astype(np.float32)
        dedb0 = rng.normal(size=b.shape).astype(np.float32)
        if dtype == torch.float16:
            a, b, dedc, deda0, dedb0 = [round_to_half(t) for t in (a, b, dedc, deda0, dedb0)]
        if not lead:
            want_a, want_b = grad_matmul(oracle, a[None], tA, b[None], tB, dedc[None], deda0[None], dedb0[None], alpha)
            want_a, want_b = want_a[0], want_b[0]
        else:
            want_a, want_b = grad_matmul(oracle, a, tA, b, tB, dedc, deda0, dedb0, alpha)
        deda, dedb = dev(deda0, dtype), dev(dedb0, dtype)
        before = L.ntb_launch_count()
        ops.GradMatrixMul(dev(a, dtype), tA, dev(b, dtype), tB, dev(dedc, dtype), deda, dedb, alpha)
        assert L.ntb_launch_count() - before in (launches, 2), (M, N, K)     # 2: a product that takes a cluster kernel
        assert rel_fro(deda.float().cpu().numpy(), want_a) <= TOL[dtype], ("deda", M, N, K)
        assert rel_fro(dedb.float().cpu().numpy(), want_b) <= TOL[dtype], ("dedb", M, N, K)
        # one gradient only
        deda2 = dev(deda0, dtype)
        ops.GradMatrixMul(dev(a, dtype), tA, dev(b, dtype), tB, dev(dedc, dtype), deda2, None, alpha)
        assert torch.equal(deda2, deda)
    assert L.ntb_device_status(0) == capi.OK


def test_gradient_pair_matches_two_separate_products_bit_for_bit():
    g = torch.Generator(device=DEV)
    g.manual_seed(9)
    a = torch.randn(1024, 768, device=DEV, generator=g).half()
    b = torch.randn(768, 640, device=DEV, generator=g).half()
    dedc = torch.randn(1024, 640, device=DEV, generator=g).half()
    deda = torch.zeros_like(a)
    dedb = torch.zeros_like(b)
    ops.GradMatrixMul(a, X_NOTRANS, b, X_NOTRANS, dedc, deda, dedb)
    da2 = torch.zeros_like(a)
    db2 = torch.zeros_like(b)
    ops._MatrixMul(dedc, X_NOTRANS, b, X_TRANS, da2, 1.0, 1.0)
    ops._MatrixMul(a, X_TRANS, dedc, X_NOTRANS, db2, 1.0, 1.0)
    assert torch.equal(deda, da2) and torch.equal(dedb, db2)
