"""Large fp32 products on the fp16 tensor pipe (every value as two scaled half-precision
pieces, three products, chains of 512 of K added into c in fp32): parity with the CPU oracle
at the fp32 tolerance of 1e-5 relative Frobenius error for every transposition, ragged
extents, alpha / beta, rows and columns of wildly different magnitude, a long K, and the
fused bias + rectifier; products below the size threshold stay on the kind::tf32 kernel."""
import numpy as np
import pytest
import torch

from niutensor_b200 import capi, ops
from niutensor_b200.capi import X_TRANS, X_NOTRANS
from oracle.oracle import rel_fro      # checker only

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 1e-5


def _run(a, tA, b, tB, c0, alpha, beta):
    c = torch.from_numpy(c0).to(DEV)
    ops._MatrixMul2D(torch.from_numpy(a).to(DEV), tA, torch.from_numpy(b).to(DEV), tB, c, alpha, beta)
    torch.cuda.synchronize()
    return c.cpu().numpy(), capi.lib().ntb_last_route()


@pytest.mark.parametrize("tA", [X_NOTRANS, X_TRANS])
@pytest.mark.parametrize("tB", [X_NOTRANS, X_TRANS])
def test_all_transpositions_ragged(tA, tB, oracle):
    rng = np.random.default_rng(500 + 2 * tA + tB)
    M, N, K = 1000, 1160, 3704
    a = rng.uniform(-1, 1, (K, M) if tA == X_TRANS else (M, K)).astype(np.float32)
    b = rng.uniform(-1, 1, (N, K) if tB == X_TRANS else (K, N)).astype(np.float32)
    c0 = rng.normal(size=(M, N)).astype(np.float32)
    for alpha, beta in ((1.0, 0.0), (0.75, 0.5)):
        got, route = _run(a, tA, b, tB, c0, alpha, beta)
        assert route == capi.ROUTE_TC_F16X2
        want = oracle.matmul2d(a, tA, b, tB, alpha, beta, c0)
        assert rel_fro(got, want) <= TOL, (tA, tB, alpha, beta, rel_fro(got, want))
    assert capi.lib().ntb_device_status(0) == capi.OK


def test_rows_and_columns_of_very_different_magnitude(oracle):
    rng = np.random.default_rng(77)
    M, N, K = 1024, 1024, 4096
    a = rng.normal(size=(M, K)).astype(np.float32)
    b = rng.normal(size=(K, N)).astype(np.float32)
    a *= np.exp2(rng.integers(-40, 40, size=(M, 1))).astype(np.float32)     # per-row magnitudes over 24 orders
    b *= np.exp2(rng.integers(-30, 10, size=(1, N))).astype(np.float32)
    a[5, :] = 0.0                                                            # an all-zero row
    a[17, :] = rng.normal(size=K).astype(np.float32) * 1e-3
    a[17, 100] = 1.0e30                                                      # a lone huge element: its row scales down
    got, route = _run(a, X_NOTRANS, b, X_NOTRANS, np.zeros((M, N), np.float32), 1.0, 0.0)
    assert route == capi.ROUTE_TC_F16X2
    want = oracle.matmul2d(a, X_NOTRANS, b, X_NOTRANS, 1.0, 0.0)
    # every row against its own norm: scaling is per row, so small rows are as exact as large ones
    rows = [r for r in range(M) if r != 5]
    got, want = got.astype(np.float64), want.astype(np.float64)
    err = np.linalg.norm(got[rows] - want[rows], axis=1) / np.linalg.norm(want[rows], axis=1)
    assert err.max() <= TOL, err.max()
    assert np.all(got[5] == 0.0)
    # and every column against its own norm
    err = np.linalg.norm(got[rows] - want[rows], axis=0) / np.linalg.norm(want[rows], axis=0)
    assert err.max() <= TOL, err.max()


def test_long_k_does_not_accumulate_truncation_error(oracle):
    rng = np.random.default_rng(78)
    M, N, K = 512, 512, 16384
    a = rng.uniform(0, 1, (M, K)).astype(np.float32)        # all positive: partial sums grow, the worst case
    b = rng.uniform(0, 1, (N, K)).astype(np.float32)
    got, route = _run(a, X_NOTRANS, b, X_TRANS, np.zeros((M, N), np.float32), 1.0, 0.0)
    assert route == capi.ROUTE_TC_F16X2
    want = a.astype(np.float64) @ b.astype(np.float64).T
    assert rel_fro(got.astype(np.float64), want) <= TOL, rel_fro(got.astype(np.float64), want)


def test_bias_and_rectifier_on_the_last_chain(oracle):
    rng = np.random.default_rng(79)
    x = rng.normal(size=(2048, 1024)).astype(np.float32)
    w = (rng.normal(size=(1024, 2048)) / 32).astype(np.float32)
    bias = rng.normal(size=2048).astype(np.float32)
    out = ops.MulAndShift(torch.from_numpy(x).to(DEV), torch.from_numpy(w).to(DEV), torch.from_numpy(bias).to(DEV),
                          act=capi.ACT_RECTIFY)
    torch.cuda.synchronize()
    assert capi.lib().ntb_last_route() == capi.ROUTE_TC_F16X2
    want = oracle.mulandshift(x, w, bias, rectify=True)
    assert rel_fro(out.cpu().numpy(), want) <= TOL


def test_small_batched_and_pinned_products_keep_the_tf32_kernel(oracle):
    L = capi.lib()
    rng = np.random.default_rng(80)
    a = rng.uniform(-1, 1, (256, 320)).astype(np.float32)
    b = rng.uniform(-1, 1, (320, 256)).astype(np.float32)
    _, route = _run(a, X_NOTRANS, b, X_NOTRANS, np.zeros((256, 256), np.float32), 1.0, 0.0)
    assert route == capi.ROUTE_TC_3XTF32
    big_a = rng.uniform(-1, 1, (1024, 4096)).astype(np.float32)
    big_b = rng.uniform(-1, 1, (4096, 1024)).astype(np.float32)
    assert L.ntb_set_route(capi.ROUTE_TC_3XTF32) == capi.OK
    try:
        got, route = _run(big_a, X_NOTRANS, big_b, X_NOTRANS, np.zeros((1024, 1024), np.float32), 1.0, 0.0)
    finally:
        L.ntb_set_route(0)
    assert route == capi.ROUTE_TC_3XTF32
    assert rel_fro(got, oracle.matmul2d(big_a, X_NOTRANS, big_b, X_NOTRANS)) <= TOL
