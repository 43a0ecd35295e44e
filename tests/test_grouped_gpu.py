"""ntb_gemm_grouped: a list of products of unequal shapes in shared launches (eight problems
per launch), against the CPU oracle problem by problem; fewer launches than problems;
misaligned items and an item with an empty inner dimension ride along on their own."""
import ctypes

import numpy as np
import pytest
import torch

from niutensor_b200 import capi
from niutensor_b200.capi import X_TRANS, X_NOTRANS
from oracle.oracle import rel_fro, round_to_half      # checker only

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _call(tensors_a, tA, tensors_b, tB, tensors_c, code_ab, code_c, alpha, beta):
    n = len(tensors_a)
    vp = ctypes.c_void_p
    arr = lambda ts: (vp * n)(*[t.data_ptr() for t in ts])
    ia = lambda vals: (ctypes.c_int * n)(*vals)
    return capi.lib().ntb_gemm_grouped(
        0, None, n, arr(tensors_a), tA, arr(tensors_b), tB, arr(tensors_c), code_ab, code_c,
        ia([t.shape[0] for t in tensors_a]), ia([t.shape[1] for t in tensors_a]),
        ia([t.shape[0] for t in tensors_b]), ia([t.shape[1] for t in tensors_b]),
        ia([t.shape[0] for t in tensors_c]), ia([t.shape[1] for t in tensors_c]), alpha, beta)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("tA,tB", [(X_NOTRANS, X_NOTRANS), (X_TRANS, X_NOTRANS), (X_NOTRANS, X_TRANS)])
def test_unequal_shapes_share_launches(dtype, tA, tB, oracle):
    L = capi.lib()
    rng = np.random.default_rng(400 + tA * 2 + tB)
    shapes = [(128, 128, 64), (256, 384, 192), (8, 8, 8), (136, 200, 72), (64, 520, 264), (384, 72, 40),
              (512, 512, 256), (1, 8, 16), (37, 29, 53), (264, 8, 1032), (200, 136, 328)]
    alpha, beta = 0.5, 0.25
    a_np, b_np, c_np, ta, tb, tc = [], [], [], [], [], []
    for (M, N, K) in shapes:
        a = rng.uniform(-1, 1, (K, M) if tA == X_TRANS else (M, K)).astype(np.float32)
        b = rng.uniform(-1, 1, (N, K) if tB == X_TRANS else (K, N)).astype(np.float32)
        c0 = rng.normal(size=(M, N)).astype(np.float32)
        if dtype == torch.float16:
            a, b, c0 = round_to_half(a), round_to_half(b), round_to_half(c0)
        a_np.append(a); b_np.append(b); c_np.append(c0)
        ta.append(torch.from_numpy(a).to(DEV).to(dtype))
        tb.append(torch.from_numpy(b).to(DEV).to(dtype))
        tc.append(torch.from_numpy(c0).to(DEV).to(dtype))
    code = capi.X_FLOAT16 if dtype == torch.float16 else capi.X_FLOAT
    before = L.ntb_launch_count()
    assert _call(ta, tA, tb, tB, tc, code, code, alpha, beta) == capi.OK
    torch.cuda.synchronize()
    launches = L.ntb_launch_count() - before
    # ten TMA-addressable problems in two shared launches, the ragged one (37 x 29 x 53) on its own
    assert launches <= 4, launches
    tol = 2e-3 if dtype == torch.float16 else 1e-5
    for i, (M, N, K) in enumerate(shapes):
        want = oracle.matmul2d(a_np[i], tA, b_np[i], tB, alpha, beta, c_np[i])
        assert rel_fro(tc[i].float().cpu().numpy(), want) <= tol, (i, M, N, K)
    assert L.ntb_device_status(0) == capi.OK


def test_empty_items_and_shape_errors():
    L = capi.lib()
    a = [torch.zeros(8, 8, device=DEV), torch.zeros(0, 8, device=DEV), torch.ones(16, 0, device=DEV)]
    b = [torch.zeros(8, 8, device=DEV), torch.zeros(8, 8, device=DEV), torch.ones(0, 24, device=DEV)]
    c = [torch.ones(8, 8, device=DEV), torch.zeros(0, 8, device=DEV), torch.full((16, 24), 2.0, device=DEV)]
    assert _call(a, X_NOTRANS, b, X_NOTRANS, c, capi.X_FLOAT, capi.X_FLOAT, 1.0, 0.5) == capi.OK
    torch.cuda.synchronize()
    assert torch.all(c[0] == 0.5)                 # 0 * 0 + 0.5 * 1
    assert torch.all(c[2] == 1.0)                 # empty inner dimension: beta * c
    bad = [torch.zeros(8, 9, device=DEV)]
    assert _call(bad, X_NOTRANS, [torch.zeros(8, 8, device=DEV)], X_NOTRANS, [torch.zeros(8, 8, device=DEV)],
                 capi.X_FLOAT, capi.X_FLOAT, 1.0, 0.0) == capi.ERR_SHAPE
    assert L.ntb_device_status(0) == capi.OK
