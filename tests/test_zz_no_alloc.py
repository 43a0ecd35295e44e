"""ntb_gemm_host_noalloc -- the entry point for callers that must not allocate device
memory at call time (a process whose memory pools already own the GPU, or threads sharing
a device that cudaMalloc / cudaFree would stall). Its scratch is a fixed array inside the
library that every call reuses, so the checks here run it twice in a row, with different
shapes, data types and routes, and compare each result with the regular host-buffer entry
point on the same inputs; the stale contents the first call leaves behind must not leak
into the second. Every result is also checked against the CPU oracle, and from the second
call on the device's free memory must not move across a call (the first call on a device
is when the driver may load the module that holds the array). This file sorts last so that
a failure here cannot hide another test."""
import numpy as np
import pytest

from niutensor_b200 import capi
from niutensor_b200.capi import X_TRANS, X_NOTRANS
from oracle.oracle import rel_fro           # checker only

pytestmark = pytest.mark.gpu


def _free_bytes():
    import torch
    torch.cuda.synchronize(0)
    return torch.cuda.mem_get_info(0)[0]


def _both(L, a, tA, b, tB, c0, code_ab, code_c, alpha, beta, steady=False):
    na, ma = a.shape
    nb, mb = b.shape
    nc, mc = c0.shape
    want = c0.copy()
    rc = L.ntb_gemm_host(0, None, a.ctypes.data, tA, b.ctypes.data, tB, want.ctypes.data, code_ab, code_c,
                         na, ma, nb, mb, nc, mc, 0, 0, 0, 1, alpha, beta)
    assert rc == capi.OK
    got = c0.copy()
    free0 = _free_bytes() if steady else None
    rc = L.ntb_gemm_host_noalloc(0, None, a.ctypes.data, tA, b.ctypes.data, tB, got.ctypes.data, code_ab, code_c,
                                 na, ma, nb, mb, nc, mc, alpha, beta)
    assert rc == capi.OK
    if steady:
        # nothing was allocated or freed on the device by this call
        assert _free_bytes() == free0
    return got, want


def test_two_calls_in_a_row_match_the_allocating_entry_point(oracle):
    L = capi.lib()
    rng = np.random.default_rng(41)
    # call 1: fp16, tensor-core route, beta != 0 (c is staged and read)
    a = rng.uniform(-1, 1, (384, 256)).astype(np.float16)
    b = rng.uniform(-1, 1, (200, 256)).astype(np.float16)          # used transposed
    c0 = rng.normal(size=(384, 200)).astype(np.float16)
    got, want = _both(L, a, X_NOTRANS, b, X_TRANS, c0, capi.X_FLOAT16, capi.X_FLOAT16, 0.5, 0.5)
    # same kernels on the same values: identical bits, well inside the 2e-3 fp16 tolerance
    assert np.array_equal(got, want)
    assert np.isfinite(got.astype(np.float32)).all() and np.abs(got.astype(np.float32)).max() > 0
    ref = oracle.matmul2d(a.astype(np.float32), X_NOTRANS, b.astype(np.float32), X_TRANS, 0.5, 0.5, c0.astype(np.float32))
    assert rel_fro(got.astype(np.float32), ref) <= 2e-3
    # call 2, straight after: fp32, smaller, ragged (packed pitches TMA could not address: the staged
    # copies get padded rows), beta == 0 -- the scratch still holds call 1's operands and result
    a = rng.uniform(-1, 1, (53, 37)).astype(np.float32)             # stored K x M, used transposed
    b = rng.uniform(-1, 1, (53, 29)).astype(np.float32)
    c0 = np.full((37, 29), np.nan, np.float32)
    got, want = _both(L, a, X_TRANS, b, X_NOTRANS, c0, capi.X_FLOAT, capi.X_FLOAT, 1.0, 0.0, steady=True)
    assert np.array_equal(got, want)
    assert np.isfinite(got).all()
    assert rel_fro(got, oracle.matmul2d(a, X_TRANS, b, X_NOTRANS, 1.0, 0.0)) <= 1e-5
    # call 3: fp32 on the tensor-core route
    a = rng.uniform(-1, 1, (256, 320)).astype(np.float32)
    b = rng.uniform(-1, 1, (320, 128)).astype(np.float32)
    c0 = rng.normal(size=(256, 128)).astype(np.float32)
    got, want = _both(L, a, X_NOTRANS, b, X_NOTRANS, c0, capi.X_FLOAT, capi.X_FLOAT, 1.0, 1.0, steady=True)
    assert np.array_equal(got, want)
    assert rel_fro(got, oracle.matmul2d(a, X_NOTRANS, b, X_NOTRANS, 1.0, 1.0, c0)) <= 1e-5
    assert L.ntb_device_status(0) == capi.OK


def test_a_problem_that_fills_the_scratch_exactly_is_accepted():
    L = capi.lib()
    rng = np.random.default_rng(43)
    # fp16: a 4 MiB + b 4 MiB + c 8 MiB = NTB_NOALLOC_MAX_BYTES to the byte
    a = rng.uniform(-1, 1, (2048, 1024)).astype(np.float16)
    b = rng.uniform(-1, 1, (1024, 2048)).astype(np.float16)
    c0 = rng.normal(size=(2048, 2048)).astype(np.float16)
    assert a.nbytes + b.nbytes + c0.nbytes == capi.NOALLOC_MAX_BYTES
    got, want = _both(L, a, X_NOTRANS, b, X_NOTRANS, c0, capi.X_FLOAT16, capi.X_FLOAT16, 1.0, 0.5)
    assert np.array_equal(got, want)
    rows = slice(1000, 1032)
    ref = a[rows].astype(np.float64) @ b.astype(np.float64) + 0.5 * c0[rows].astype(np.float64)
    assert rel_fro(got[rows].astype(np.float64), ref) <= 2e-3
    # one more column no longer fits
    b1 = np.zeros((1024, 2056), np.float16)
    c1 = np.zeros((2048, 2056), np.float16)
    rc = L.ntb_gemm_host_noalloc(0, None, a.ctypes.data, X_NOTRANS, b1.ctypes.data, X_NOTRANS, c1.ctypes.data,
                                 capi.X_FLOAT16, capi.X_FLOAT16, 2048, 1024, 1024, 2056, 2048, 2056, 1.0, 0.0)
    assert rc == capi.ERR_LIMIT


def test_sizes_beyond_the_fixed_scratch_are_refused():
    L = capi.lib()
    n = 2048                                    # 3 x 2048^2 fp32 = 48 MiB > 16 MiB
    a = np.zeros((n, n), np.float32)
    c = np.zeros((n, n), np.float32)
    rc = L.ntb_gemm_host_noalloc(0, None, a.ctypes.data, X_NOTRANS, a.ctypes.data, X_NOTRANS, c.ctypes.data,
                                 capi.X_FLOAT, capi.X_FLOAT, n, n, n, n, n, n, 1.0, 0.0)
    assert rc == capi.ERR_LIMIT
    assert "limit" in capi.strerror(rc)
    # shape and type errors are reported as by the other entry points
    rc = L.ntb_gemm_host_noalloc(0, None, a.ctypes.data, X_NOTRANS, a.ctypes.data, X_NOTRANS, c.ctypes.data,
                                 capi.X_FLOAT, capi.X_FLOAT, 8, 9, 8, 8, 8, 8, 1.0, 0.0)
    assert rc == capi.ERR_SHAPE
