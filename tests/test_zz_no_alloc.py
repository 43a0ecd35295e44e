"""ntb_gemm_host_noalloc -- the entry point for callers that must not allocate device
memory at call time (a process whose memory pools already own the GPU, or threads sharing
a device that cudaMalloc / cudaFree would stall). Its scratch is a fixed array inside the
library that every call reuses, so the checks here run it twice in a row, with different
shapes, data types and routes, and compare each result with the regular host-buffer entry
point on the same inputs; the stale contents the first call leaves behind must not leak
into the second. This file sorts last so that a failure here cannot hide another test."""
import numpy as np
import pytest

from niutensor_b200 import capi
from niutensor_b200.capi import X_TRANS, X_NOTRANS

pytestmark = pytest.mark.gpu


def _both(L, a, tA, b, tB, c0, code_ab, code_c, alpha, beta):
    na, ma = a.shape
    nb, mb = b.shape
    nc, mc = c0.shape
    want = c0.copy()
    rc = L.ntb_gemm_host(0, None, a.ctypes.data, tA, b.ctypes.data, tB, want.ctypes.data, code_ab, code_c,
                         na, ma, nb, mb, nc, mc, 0, 0, 0, 1, alpha, beta)
    assert rc == capi.OK
    got = c0.copy()
    rc = L.ntb_gemm_host_noalloc(0, None, a.ctypes.data, tA, b.ctypes.data, tB, got.ctypes.data, code_ab, code_c,
                                 na, ma, nb, mb, nc, mc, alpha, beta)
    assert rc == capi.OK
    return got, want


def test_two_calls_in_a_row_match_the_allocating_entry_point():
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
    # call 2, straight after: fp32, smaller, ragged (FFMA route), beta == 0 -- the scratch
    # still holds call 1's operands and result
    a = rng.uniform(-1, 1, (53, 37)).astype(np.float32)             # stored K x M, used transposed
    b = rng.uniform(-1, 1, (53, 29)).astype(np.float32)
    c0 = np.full((37, 29), np.nan, np.float32)
    got, want = _both(L, a, X_TRANS, b, X_NOTRANS, c0, capi.X_FLOAT, capi.X_FLOAT, 1.0, 0.0)
    assert np.array_equal(got, want)
    assert np.isfinite(got).all()
    ref = a.T.astype(np.float64) @ b.astype(np.float64)
    assert np.linalg.norm(got - ref) / np.linalg.norm(ref) <= 1e-5
    # call 3: fp32 on the tensor-core route
    a = rng.uniform(-1, 1, (256, 320)).astype(np.float32)
    b = rng.uniform(-1, 1, (320, 128)).astype(np.float32)
    c0 = rng.normal(size=(256, 128)).astype(np.float32)
    got, want = _both(L, a, X_NOTRANS, b, X_NOTRANS, c0, capi.X_FLOAT, capi.X_FLOAT, 1.0, 1.0)
    assert np.array_equal(got, want)
    assert L.ntb_device_status(0) == capi.OK


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
