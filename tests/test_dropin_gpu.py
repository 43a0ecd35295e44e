"""Drop-in check at link level: the reference's GPU build with its matrix-multiplication
translation units replaced by niutensor_b200/host/nts_matmul_shim.cpp (built by
`make -C oracle dropin` into oracle/_ref/, which exists only where the reference sources
were available at build time). The reference's own unit tests for this path then run on
the new kernels, and user-level calls the reference has no test for are compared with the
CPU oracle.

Only the GPU halves of the reference's unit tests are evidence here: for tensors on the CPU
(devID < 0) the shim hands the product to the reference's untouched _MatrixMul2DParallel, so
the CPU halves, and TestMatrixMul2DParallel as a whole, are the reference checking itself.
The tensors of the reference's unit tests are allocated without a memory pool (mem == NULL);
tensors that live in XMem pools are covered by the pool test at the end of this file, by
tests/test_samples_gpu.py (the transformer sample allocates from its pools) and by the
misaligned-operand cases of tests/test_gemm_gpu.py."""
import ctypes
import os

import numpy as np
import pytest

from oracle.oracle import rel_fro, X_NOTRANS, X_TRANS

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "oracle", "_ref", "libnts_dropin.so")


@pytest.fixture(scope="module")
def dropin():
    if not os.path.exists(LIB):
        pytest.skip("drop-in check library not built (needs the reference sources)")
    from niutensor_b200 import capi
    capi.lib()                                  # libntb_gemm.so first, by its full path
    lib = ctypes.CDLL(LIB)
    lib.dropin_run_reference_tests.restype = ctypes.c_int
    return lib


def test_reference_unit_tests_pass_on_the_new_kernels(dropin):
    mask = dropin.dropin_run_reference_tests()
    assert mask == 0b1111, "TestMatrixMul / 2D / 2DParallel / Batched bitmask: %s" % bin(mask)


def test_user_level_bmmul_on_half_tensors(dropin, oracle):
    rng = np.random.default_rng(31)
    batch, length, dk = 6, 128, 64
    q = rng.normal(size=(batch, length, dk)).astype(np.float16)
    k = rng.normal(size=(batch, length, dk)).astype(np.float16)
    s = np.zeros((batch, length, length), np.float16)
    u16 = ctypes.POINTER(ctypes.c_ushort)
    rc = dropin.dropin_bmmul_half(0, batch, length, dk, q.ctypes.data_as(u16), k.ctypes.data_as(u16),
                                  s.ctypes.data_as(u16), ctypes.c_float(0.125))
    assert rc == 0
    want = oracle.matmul_batched(q.astype(np.float32), X_NOTRANS, k.astype(np.float32), X_TRANS, 0.125)
    assert rel_fro(s.astype(np.float32), want) <= 2e-3


def test_reference_mulandshift_runs_on_the_shim(dropin, oracle):
    rng = np.random.default_rng(32)
    rows, din, dout = 96, 128, 160
    x = rng.normal(size=(rows, din)).astype(np.float32)
    w = (rng.normal(size=(din, dout)) / np.sqrt(din)).astype(np.float32)
    b = rng.normal(size=(dout,)).astype(np.float32)
    y = np.zeros((rows, dout), np.float32)
    fp = ctypes.POINTER(ctypes.c_float)
    rc = dropin.dropin_mulandshift_f32(0, rows, din, dout, x.ctypes.data_as(fp), w.ctypes.data_as(fp),
                                       b.ctypes.data_as(fp), y.ctypes.data_as(fp))
    assert rc == 0
    want = oracle.matmul2d(x, X_NOTRANS, w, X_NOTRANS) + b[None, :]
    assert rel_fro(y, want) <= 1e-5


def test_wrapper_list_of_unequal_shapes(dropin, oracle):
    """_CudaBLASMatrixMULList with items of different shapes (the reference loops over single
    cuBLAS calls, XTensorBLAS.cu:373-385; the shim passes the list to one grouped launch),
    called through the reference's own signature with TensorLists of GPU tensors."""
    from niutensor_b200 import capi
    rng = np.random.default_rng(33)
    shapes = [(64, 72, 40), (128, 256, 96), (8, 8, 8), (200, 136, 64), (32, 520, 128)]
    a = [rng.normal(size=(m, k)).astype(np.float32) for m, n, k in shapes]
    b = [rng.normal(size=(k, n)).astype(np.float32) for m, n, k in shapes]
    c0 = [rng.normal(size=(m, n)).astype(np.float32) for m, n, k in shapes]
    pack = lambda xs: np.ascontiguousarray(np.concatenate([x.reshape(-1) for x in xs]))
    pa, pb, pc = pack(a), pack(b), pack(c0)
    ia = lambda col: (ctypes.c_int * len(shapes))(*[s[col] for s in shapes])
    fp = ctypes.POINTER(ctypes.c_float)
    before = capi.lib().ntb_launch_count()
    rc = dropin.dropin_list_unequal_f32(0, len(shapes), ia(0), ia(1), ia(2), pa.ctypes.data_as(fp), pb.ctypes.data_as(fp),
                                        pc.ctypes.data_as(fp), ctypes.c_float(0.5), ctypes.c_float(0.25))
    assert rc == 0
    assert capi.lib().ntb_launch_count() == before + 1          # one grouped launch, not five
    off = 0
    for (m, n, k), x, y, z in zip(shapes, a, b, c0):
        got = pc[off:off + m * n].reshape(m, n)
        off += m * n
        assert rel_fro(got, oracle.matmul2d(x, X_NOTRANS, y, X_NOTRANS, 0.5, 0.25, z)) <= 1e-5, (m, n, k)


def test_wrapper_device_pointer_tables(dropin, oracle):
    """_CudaBLASMatrixMULBatched as cublasGemmBatchedEx took it: device arrays of device pointers,
    here in an order no stride pattern describes."""
    rng = np.random.default_rng(34)
    count, m, n, k = 7, 72, 136, 48
    a = rng.normal(size=(count, m, k)).astype(np.float32)
    b = rng.normal(size=(count, k, n)).astype(np.float32)
    c0 = rng.normal(size=(count, m, n)).astype(np.float32)
    c = c0.copy()
    fp = ctypes.POINTER(ctypes.c_float)
    rc = dropin.dropin_batched_pointer_tables_f32(0, count, m, n, k, a.ctypes.data_as(fp), b.ctypes.data_as(fp),
                                                  c.ctypes.data_as(fp), ctypes.c_float(1.0), ctypes.c_float(0.5))
    assert rc == 0
    assert rel_fro(c, oracle.matmul_batched(a, X_NOTRANS, b, X_NOTRANS, 1.0, 0.5, c0)) <= 1e-5


@pytest.mark.parametrize("pad", [64, 3])
def test_matmul_with_beta_on_tensors_from_a_memory_pool(dropin, oracle, pad):
    """The C++ overload MatrixMul(a, tA, b, tB, c, alpha, beta) with beta != 0 on tensors
    allocated from an XMem pool; with an odd-sized tensor ahead of them in the pool the
    matrices need not start on a 16-byte boundary, and the product stays on the tensor cores."""
    from niutensor_b200 import capi
    rng = np.random.default_rng(35 + pad)
    m, n, k = 200, 136, 72
    a = rng.normal(size=(m, k)).astype(np.float32)
    b = rng.normal(size=(k, n)).astype(np.float32)
    c0 = rng.normal(size=(m, n)).astype(np.float32)
    c = c0.copy()
    fp = ctypes.POINTER(ctypes.c_float)
    aligned = ctypes.c_int(-1)
    simt_before = capi.lib().ntb_route_count(capi.ROUTE_SIMT)
    rc = dropin.dropin_matmul_beta_in_pool_f32(0, pad, m, n, k, a.ctypes.data_as(fp), b.ctypes.data_as(fp), c.ctypes.data_as(fp),
                                               ctypes.c_float(0.5), ctypes.c_float(0.25), ctypes.byref(aligned))
    assert rc == 0
    assert aligned.value in (0, 1)
    assert capi.lib().ntb_route_count(capi.ROUTE_SIMT) == simt_before       # no product fell back to FFMA
    assert rel_fro(c, oracle.matmul2d(a, X_NOTRANS, b, X_NOTRANS, 0.5, 0.25, c0)) <= 1e-5
