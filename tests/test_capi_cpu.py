"""CPU-side checks of the drop-in boundary: the shared library loads, exports every
symbol the header declares, validates arguments with the reference's shape rules before
touching CUDA, and refuses to compute without a device (there is no CPU fallback)."""
import ctypes
import os
import re

import pytest

from niutensor_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "ntb_gemm.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return set(re.findall(r"\b(ntb_\w+)\s*\(", text))


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(capi.LIB_PATH)
    names = header_symbols()
    assert names, "no declarations found"
    for n in names:
        assert hasattr(lib, n), n
    assert names == set(capi.PROTOTYPES), names ^ set(capi.PROTOTYPES)


def test_argument_checks_run_before_cuda():
    L = capi.lib()
    p = 4096  # any non-null address; never dereferenced on these paths
    f16 = capi.X_FLOAT16
    # inner dimensions differ: a 4x5, b 6x4
    assert L.ntb_gemm(0, None, p, 1, p, 1, p, f16, f16, 4, 5, 6, 4, 4, 4, 5, 4, 4, 1.0, 0.0) == capi.ERR_SHAPE
    # output shape wrong
    assert L.ntb_gemm(0, None, p, 1, p, 1, p, f16, f16, 4, 5, 5, 4, 4, 3, 5, 4, 3, 1.0, 0.0) == capi.ERR_SHAPE
    # transposition flag outside the enum
    assert L.ntb_gemm(0, None, p, 2, p, 1, p, f16, f16, 4, 4, 4, 4, 4, 4, 4, 4, 4, 1.0, 0.0) == capi.ERR_ARG
    # X_DOUBLE, X_INT are not supported
    assert L.ntb_gemm(0, None, p, 1, p, 1, p, capi.X_DOUBLE, capi.X_DOUBLE, 4, 4, 4, 4, 4, 4, 4, 4, 4, 1.0, 0.0) == capi.ERR_DTYPE
    assert L.ntb_gemm(0, None, p, 1, p, 1, p, capi.X_INT, capi.X_INT, 4, 4, 4, 4, 4, 4, 4, 4, 4, 1.0, 0.0) == capi.ERR_DTYPE
    # fp32 inputs cannot produce a half result
    assert L.ntb_gemm(0, None, p, 1, p, 1, p, capi.X_FLOAT, f16, 4, 4, 4, 4, 4, 4, 4, 4, 4, 1.0, 0.0) == capi.ERR_DTYPE
    # pitch smaller than the row
    assert L.ntb_gemm(0, None, p, 1, p, 1, p, f16, f16, 4, 4, 4, 4, 4, 4, 3, 4, 4, 1.0, 0.0) == capi.ERR_ARG
    # NULL operand
    assert L.ntb_gemm(0, None, None, 1, p, 1, p, f16, f16, 4, 4, 4, 4, 4, 4, 4, 4, 4, 1.0, 0.0) == capi.ERR_ARG
    # empty problems are a no-op, as in the reference's list path (XTensorBLAS.cu:261-262)
    assert L.ntb_gemm_strided_batched(0, None, p, 1, p, 1, p, f16, f16, 4, 4, 4, 4, 4, 4, 4, 4, 4,
                                      16, 16, 16, 0, 1.0, 0.0) == capi.OK
    assert L.ntb_gemm_list(0, None, None, 1, None, 1, None, f16, f16, 0, 4, 4, 4, 4, 4, 4, 1.0, 0.0) == capi.OK
    assert L.ntb_set_route(7) == capi.ERR_ARG
    assert capi.strerror(capi.ERR_SHAPE) == "unmatched tensors in multiplication"


def test_shard_range_matches_the_python_split():
    from niutensor_b200 import shard
    L = capi.lib()
    lo, hi = ctypes.c_int(), ctypes.c_int()
    for total in (0, 1, 7, 8, 1000, 8192, 65536):
        for shards in (1, 2, 3, 4, 8):
            for mult in (1, 8):
                for r in range(shards):
                    L.ntb_shard_range(total, shards, r, mult, ctypes.byref(lo), ctypes.byref(hi))
                    assert (lo.value, hi.value) == shard.split_range(total, shards, r, mult)


def test_sharded_entry_checks_arguments_before_cuda():
    L = capi.lib()
    f16 = capi.X_FLOAT16
    vp = ctypes.c_void_p

    def arr(n, v=4096):
        return (vp * n)(*([v] * n))

    def call(n_dev=2, devs=None, a=None, ta=1, tb=1, dims=(8, 8, 8, 8, 8, 8), dt=(f16, f16), count=1, axis=0, gather=0):
        devs = (ctypes.c_int * max(1, n_dev))(*(devs or [0] * max(1, n_dev)))
        return L.ntb_gemm_sharded(devs, n_dev, None, a if a is not None else arr(max(1, n_dev)), ta, arr(max(1, n_dev)), tb,
                                  arr(max(1, n_dev)), dt[0], dt[1], *dims, count, axis, gather, 1.0, 0.0)

    assert call(n_dev=0) == capi.ERR_ARG
    assert call(n_dev=capi.MAX_PEERS + 2) == capi.ERR_LIMIT
    assert call(axis=5) == capi.ERR_ARG
    assert call(ta=3) == capi.ERR_ARG
    assert call(dims=(8, 8, 9, 8, 8, 8)) == capi.ERR_SHAPE
    assert call(dt=(capi.X_DOUBLE, capi.X_DOUBLE)) == capi.ERR_DTYPE
    assert call(devs=[0, -1]) == capi.ERR_ARG
    assert call(count=2, axis=capi.SHARD_COLUMNS) == capi.ERR_ARG       # column shards are for the 2-D form
    assert call(count=0, axis=capi.SHARD_BATCH) == capi.OK               # nothing to do
    # un-interleave helper: misaligned shard width (3 halves = 6 bytes)
    assert L.ntb_unshard_columns(0, None, 4096, 8192, f16, 4, 2, 3, 6) == capi.ERR_ARG
    assert L.ntb_unshard_columns(0, None, 4096, 8192, f16, 4, 2, 8, 15) == capi.ERR_ARG   # pitch below the row
    assert L.ntb_unshard_columns(0, None, 4096, 8192, f16, 0, 2, 8, 16) == capi.OK


def test_grouped_and_multicast_entries_check_arguments_before_cuda():
    L = capi.lib()
    f16 = capi.X_FLOAT16
    vp = ctypes.c_void_p
    ptrs = (vp * 2)(4096, 4096)
    ia = lambda *v: (ctypes.c_int * 2)(*v)
    ok = (ia(8, 16), ia(8, 8), ia(8, 8), ia(8, 24), ia(8, 16), ia(8, 24))
    assert L.ntb_gemm_grouped(0, None, 0, None, 1, None, 1, None, f16, f16, None, None, None, None, None, None, 1.0, 0.0) == capi.OK
    assert L.ntb_gemm_grouped(0, None, -1, ptrs, 1, ptrs, 1, ptrs, f16, f16, *ok, 1.0, 0.0) == capi.ERR_ARG
    assert L.ntb_gemm_grouped(0, None, 2, ptrs, 5, ptrs, 1, ptrs, f16, f16, *ok, 1.0, 0.0) == capi.ERR_ARG
    assert L.ntb_gemm_grouped(0, None, 2, ptrs, 1, ptrs, 1, ptrs, capi.X_INT, capi.X_INT, *ok, 1.0, 0.0) == capi.ERR_DTYPE
    bad = (ia(8, 16), ia(8, 9), ia(8, 8), ia(8, 24), ia(8, 16), ia(8, 24))     # second item: inner extents 9 and 8
    assert L.ntb_gemm_grouped(0, None, 2, ptrs, 1, ptrs, 1, ptrs, f16, f16, *bad, 1.0, 0.0) == capi.ERR_SHAPE
    # multicast destination: NULL, misaligned, or a column count that is not a whole number of 16-byte units
    args = (0, None, 4096, 1, 4096, 1, 4096)
    tail = (f16, f16, 8, 8, 8, 16, 8, 16, 8, 16, 16, 1.0, 0.0)
    assert L.ntb_gemm_multicast(*args, None, *tail) == capi.ERR_ARG
    assert L.ntb_gemm_multicast(*args, 4098, *tail) == capi.ERR_ARG
    assert L.ntb_gemm_multicast(*args, 8192, f16, f16, 8, 8, 8, 12, 8, 12, 8, 12, 16, 1.0, 0.0) == capi.ERR_ARG


def test_no_cpu_fallback_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    L = capi.lib()
    p = 4096
    rc = L.ntb_gemm(0, None, p, 1, p, 1, p, capi.X_FLOAT16, capi.X_FLOAT16,
                    4, 4, 4, 4, 4, 4, 4, 4, 4, 1.0, 0.0)
    assert rc == capi.ERR_CUDA


def test_ops_refuse_cpu_tensors():
    import torch
    from niutensor_b200 import ops
    a = torch.zeros(2, 3)
    b = torch.zeros(3, 2)
    c = torch.zeros(2, 2)
    with pytest.raises(ops.NtError):
        ops._MatrixMul(a, capi.X_NOTRANS, b, capi.X_NOTRANS, c)


def test_product_package_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "niutensor_b200")
    for dirpath, _, files in os.walk(pkg):
        for fn in files:
            if fn.endswith((".py", ".cu", ".h", ".cpp", ".cuh")):
                text = open(os.path.join(dirpath, fn)).read()
                assert "oracle" not in text.lower(), fn


def test_tile_cost_model_choices_for_the_benchmark_configurations():
    """ntb_plan runs the host-side cost model without a device: 148 SMs, the shapes of the
    benchmark configurations and of a weight gradient."""
    L = capi.lib()
    f16, f32 = capi.X_FLOAT16, capi.X_FLOAT
    assert L.ntb_plan(f16, 8192, 8192, 8192, 1, 148) == capi.PLAN_PAIR_512X256     # config 5
    assert L.ntb_plan(f16, 4096, 2048, 512, 1, 148) == capi.PLAN_PAIR_256X256      # config 2a
    assert L.ntb_plan(f16, 4096, 512, 2048, 1, 148) == capi.PLAN_PAIR_256X128      # config 2b: 128 CTAs, less B traffic
    assert L.ntb_plan(f16, 256, 65536, 512, 1, 148) in (capi.PLAN_PAIR_256X256, capi.PLAN_PAIR_512X256)   # config 4
    assert L.ntb_plan(f16, 256, 64, 256, 64, 148) == 64                            # config 3b: one tile per m-block
    assert L.ntb_plan(f16, 256, 256, 64, 64, 148) in (128, 256)                    # config 3a
    assert L.ntb_plan(f16, 1024, 512, 4096, 1, 148) in (capi.PLAN_SPLIT_K2, capi.PLAN_SPLIT_K4)   # weight gradient
    assert L.ntb_plan(f16, 4096, 512, 8192, 1, 148) == capi.PLAN_PAIRSPLIT_K2      # 32 tiles of 256 x 256 with a long K: two pairs each
    assert L.ntb_plan(f16, 1024, 1024, 8192, 1, 148) == capi.PLAN_PAIRSPLIT_K4     # weight gradient over 8192 tokens: four pairs per tile
    assert L.ntb_plan(f32, 512, 512, 512, 1, 148) in (64, 128)                     # config 1: no cluster kernel for fp32
    assert L.ntb_plan(f32, 8192, 8192, 8192, 1, 148) == 128
    assert L.ntb_plan(f16, 8192, 8192, 8192, 1, 1) > 0                             # one SM: no pairs, no clusters
    assert L.ntb_plan(7, 8, 8, 8, 1, 148) < -50 and L.ntb_plan(f16, 0, 8, 8, 1, 148) < -50
