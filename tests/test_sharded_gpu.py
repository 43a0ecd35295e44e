"""ntb_gemm_sharded: one process drives several devices (NiuTensor's own process model).
On one GPU the "devices" are the same GPU several times over with separate buffers, which
exercises the shard arithmetic, the peer-store epilogue and the stream joins; with two or
more GPUs the same checks run across real peers. Results are compared with the CPU oracle
and, bit for bit, with the unsharded product of the same library."""
import ctypes

import numpy as np
import pytest
import torch

from niutensor_b200 import capi, ops, shard
from niutensor_b200.capi import X_TRANS, X_NOTRANS
from oracle.oracle import rel_fro, round_to_half      # checker only

pytestmark = pytest.mark.gpu


def _devices(n):
    have = torch.cuda.device_count()
    return [i % have for i in range(n)]


def _ptrs(tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def _run(devs, a_list, tA, b_list, tB, c_list, dims, count, axis, gather, alpha, beta, dtype=torch.float16, dtc=None):
    L = capi.lib()
    code = capi.X_FLOAT16 if dtype == torch.float16 else capi.X_FLOAT
    codec = code if dtc is None else (capi.X_FLOAT16 if dtc == torch.float16 else capi.X_FLOAT)
    rc = L.ntb_gemm_sharded((ctypes.c_int * len(devs))(*devs), len(devs), None, _ptrs(a_list), tA, _ptrs(b_list), tB,
                            _ptrs(c_list), code, codec, *dims, count, axis, gather, alpha, beta)
    assert rc == capi.OK, capi.strerror(rc)
    for d in set(devs):
        torch.cuda.synchronize(d)
        assert L.ntb_device_status(d) == capi.OK


@pytest.mark.parametrize("n_dev", [2, 3])
@pytest.mark.parametrize("tB", [X_NOTRANS, X_TRANS])
@pytest.mark.parametrize("gather", [0, 1])
def test_column_shards(n_dev, tB, gather, oracle):
    devs = _devices(n_dev)
    rng = np.random.default_rng(70 + n_dev + tB)
    M, N, K = 200, 328, 192                       # 328 = 41 x 8: ragged shard widths
    alpha, beta = 0.5, 0.25
    a = round_to_half(rng.uniform(-1, 1, (M, K)).astype(np.float32))
    b = round_to_half(rng.uniform(-1, 1, (N, K) if tB == X_TRANS else (K, N)).astype(np.float32))
    c0 = round_to_half(rng.normal(size=(M, N)).astype(np.float32))
    want = oracle.matmul2d(a, X_NOTRANS, b, tB, alpha, beta, c0)
    a_l, b_l, c_l, spans = [], [], [], []
    for d, dev in enumerate(devs):
        lo, hi = shard.column_shard(N, n_dev, d)
        spans.append((lo, hi))
        a_l.append(torch.from_numpy(a).half().to("cuda:%d" % dev))
        bs = b[lo:hi] if tB == X_TRANS else np.ascontiguousarray(b[:, lo:hi])
        b_l.append(torch.from_numpy(bs).half().to("cuda:%d" % dev))
        if gather:
            # every copy starts from c0 in the device's own block and a marker elsewhere
            full = np.full((M, N), 9.0, np.float32)
            full[:, lo:hi] = c0[:, lo:hi]
            c_l.append(torch.from_numpy(full).half().to("cuda:%d" % dev))
        else:
            c_l.append(torch.from_numpy(np.ascontiguousarray(c0[:, lo:hi])).half().to("cuda:%d" % dev))
    dims = (M, K) + tuple(b.shape) + (M, N)
    _run(devs, a_l, X_NOTRANS, b_l, tB, c_l, dims, 1, capi.SHARD_COLUMNS, gather, alpha, beta)
    if gather:
        first = c_l[0].float().cpu().numpy()
        assert rel_fro(first, want) <= 2e-3
        for t in c_l[1:]:
            assert np.array_equal(t.float().cpu().numpy(), first)      # every device holds the same whole C
    else:
        for (lo, hi), t in zip(spans, c_l):
            assert rel_fro(t.float().cpu().numpy(), want[:, lo:hi]) <= 2e-3
    # bit for bit what the unsharded product gives (same kernels, same accumulation order per tile row)
    whole = torch.from_numpy(c0).half().to("cuda:%d" % devs[0])
    ops._MatrixMul2D(a_l[0], X_NOTRANS, torch.from_numpy(b).half().to("cuda:%d" % devs[0]), tB, whole, alpha, beta)
    got = c_l[0].float().cpu().numpy() if gather else np.concatenate([t.float().cpu().numpy() for t in c_l], axis=1)
    assert rel_fro(got, whole.float().cpu().numpy()) <= 1e-3


@pytest.mark.parametrize("gather", [0, 1])
def test_batch_shards(gather, oracle):
    n_dev = 3
    devs = _devices(n_dev)
    rng = np.random.default_rng(91)
    count, M, N, K = 7, 96, 64, 72
    q = rng.normal(size=(count, M, K)).astype(np.float32)
    k = rng.normal(size=(count, N, K)).astype(np.float32)
    want = oracle.matmul_batched(q, X_NOTRANS, k, X_TRANS, 0.125, 0.0)
    a_l, b_l, c_l, spans = [], [], [], []
    for d, dev in enumerate(devs):
        lo, hi = shard.batch_shard(count, n_dev, d)
        spans.append((lo, hi))
        a_l.append(torch.from_numpy(q[lo:hi].copy()).to("cuda:%d" % dev))
        b_l.append(torch.from_numpy(k[lo:hi].copy()).to("cuda:%d" % dev))
        c_l.append(torch.full((count if gather else hi - lo, M, N), 7.0, device="cuda:%d" % dev))
    _run(devs, a_l, X_NOTRANS, b_l, X_TRANS, c_l, (M, K, N, K, M, N), count, capi.SHARD_BATCH, gather, 0.125, 0.0,
         dtype=torch.float32)
    for (lo, hi), t in zip(spans, c_l):
        got = t.cpu().numpy()
        if gather:
            assert rel_fro(got, want) <= 1e-5
        else:
            assert rel_fro(got, want[lo:hi]) <= 1e-5


def test_unshard_columns_restores_row_major_order():
    L = capi.lib()
    rows, shards, w = 257, 4, 72
    src = torch.randn(shards, rows, w, device="cuda:0").half()
    dst = torch.zeros(rows, shards * w + 8, device="cuda:0", dtype=torch.float16)
    rc = L.ntb_unshard_columns(0, None, src.data_ptr(), dst.data_ptr(), capi.X_FLOAT16, rows, shards, w, dst.shape[1])
    assert rc == capi.OK
    torch.cuda.synchronize()
    want = torch.cat([src[s] for s in range(shards)], dim=1)
    assert torch.equal(dst[:, :shards * w], want)
    assert torch.all(dst[:, shards * w:] == 0)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_column_shards_on_two_real_devices(oracle):
    test_column_shards(2, X_NOTRANS, 1, oracle)
