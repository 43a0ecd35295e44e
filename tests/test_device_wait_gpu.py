"""The give-up path of the kernels' bounded waits, exercised without faulting anything: the
test hook makes the copy producers leave out one k-block and shortens the wait limit to a
couple of milliseconds, so the consumer's wait runs out. The kernel must come back by
itself, the device status must report NTB_ERR_DEVICE_WAIT exactly once, and the device
must be fully usable afterwards (tensor memory released, next product correct)."""
import os

import numpy as np
import pytest
import torch

from niutensor_b200 import capi, ops
from niutensor_b200.capi import X_TRANS, X_NOTRANS
from oracle.oracle import rel_fro, round_to_half      # checker only

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("route", [capi.ROUTE_TC_F16, capi.ROUTE_TC_F16_PAIR, capi.ROUTE_TC_3XTF32])
def test_a_wait_that_runs_out_is_reported_and_the_device_stays_usable(route, oracle):
    L = capi.lib()
    rng = np.random.default_rng(300 + route)
    dtype = torch.float32 if route == capi.ROUTE_TC_3XTF32 else torch.float16
    M, N, K = 512, 512, 1024
    a = round_to_half(rng.uniform(-1, 1, (M, K)).astype(np.float32))
    b = round_to_half(rng.uniform(-1, 1, (K, N)).astype(np.float32))
    ta, tb = torch.from_numpy(a).to(DEV).to(dtype), torch.from_numpy(b).to(DEV).to(dtype)
    c = torch.zeros(M, N, device=DEV, dtype=dtype)
    assert L.ntb_device_status(0) == capi.OK
    assert L.ntb_set_route(route if route != capi.ROUTE_TC_3XTF32 else 0) == capi.OK
    try:
        # k-block 3 of every CTA's first tile never arrives; waits give up after ~4M clocks (about 2 ms)
        assert L.ntb_debug_inject(0, 3, 4096) == capi.OK
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        ops._MatrixMul2D(ta, X_NOTRANS, tb, X_NOTRANS, c, 1.0, 0.0)
        assert L.ntb_last_route() == route
        t1.record()
        torch.cuda.synchronize()
        assert t0.elapsed_time(t1) < 500.0           # it came back by itself, quickly
        assert L.ntb_device_status(0) == capi.ERR_DEVICE_WAIT
        assert L.ntb_device_status(0) == capi.OK     # cleared on read
    finally:
        assert L.ntb_debug_inject(0, -1, 0) == capi.OK
    # the device is as good as new: same kernels, full result
    for _ in range(2):
        c.zero_()
        ops._MatrixMul2D(ta, X_NOTRANS, tb, X_NOTRANS, c, 1.0, 0.0)
        torch.cuda.synchronize()
        assert L.ntb_last_route() == route
        want = oracle.matmul2d(a, X_NOTRANS, b, X_NOTRANS, 1.0, 0.0)
        assert rel_fro(c.float().cpu().numpy(), want) <= (1e-5 if dtype == torch.float32 else 2e-3)
    assert L.ntb_set_route(0) == capi.OK
    assert L.ntb_device_status(0) == capi.OK
