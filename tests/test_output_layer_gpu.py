"""The normalised output layer, LogSoftmax(h w^T): one GPU, shards combined by hand on one
GPU, and two NCCL ranks (skipped where fewer than two GPUs are visible). Tolerances: the
relative Frobenius budgets of the matrix product (1e-5 fp32, 2e-3 fp16)."""
import os
import socket

import numpy as np
import pytest
import torch

from niutensor_b200 import capi, ops, shard
from niutensor_b200.capi import X_TRANS, X_NOTRANS
from oracle.oracle import rel_fro, round_to_half
from tests.golden.cases import output_layer_cases

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def dev(x, dtype):
    return torch.from_numpy(np.ascontiguousarray(x)).to(DEV).to(dtype)


def test_fp32_against_stored_reference_outputs():
    z = np.load(os.path.join(GOLD, "ref_output_layer.npz"))
    for i, (h, w) in enumerate(output_layer_cases()):
        y = shard.vocab_parallel_output(dev(h, torch.float32), dev(w, torch.float32))
        want = z["y%d" % i]
        assert tuple(y.shape) == want.shape
        assert rel_fro(y.cpu().numpy(), want) <= 1e-5, i
        assert float(y.min()) >= -20.0
    assert capi.lib().ntb_device_status(0) == capi.OK


def test_logsoftmax_edge_rows():
    x = torch.tensor([[0.0, 0.0, 0.0, 0.0],
                      [-float("inf"), 1.0, 2.0, -float("inf")],
                      [100.0, -100.0, 0.0, 50.0]], device=DEV)
    y = ops.LogSoftmax(x).cpu().numpy()
    assert np.allclose(y[0], np.log(0.25))
    assert y[1, 0] == -20.0 and y[1, 3] == -20.0          # -inf becomes the floor
    assert np.allclose(y[1, 1:3], [np.log(1 / (1 + np.e)), np.log(np.e / (1 + np.e))], atol=1e-6)
    assert y[2, 1] == -20.0 and y[2, 2] == -20.0 and abs(y[2, 0]) < 1e-6
    # unaligned row pitch and odd width take the scalar path
    big = torch.randn(7, 1003, device=DEV)
    view = big[:, 1:1000]
    mx, sm = ops.RowStats(view)
    ref = torch.log_softmax(view, dim=-1).clamp_min(-20.0)
    out = ops.LogSoftmaxApply(view.clone(), mx, sm)
    assert float((out - ref).abs().max()) <= 1e-5


@pytest.mark.parametrize("dtype,tol", [(torch.float16, 2e-3), (torch.float32, 1e-5)])
def test_benchmark_output_layer_with_shards_combined_by_hand(dtype, tol, oracle):
    """Config 4 (H 256 x 512, W 65536 x 512, std 0.02): shards of the vocabulary computed
    one after the other on one GPU, their row statistics combined as the ranks would."""
    rng = np.random.default_rng(1004)
    h = rng.normal(size=(256, 512)).astype(np.float32)
    w = (rng.normal(size=(65536, 512)) * 0.02).astype(np.float32)
    if dtype == torch.float16:
        h, w = round_to_half(h), round_to_half(w)
    want = oracle.output_layer(h, w)
    th, tw = dev(h, dtype), dev(w, dtype)
    one = shard.vocab_parallel_output(th, tw)
    assert rel_fro(one.float().cpu().numpy(), want) <= tol
    for world in (2, 8):
        logits, stats = [], []
        for r in range(world):
            lo, hi = shard.column_shard(65536, world, r)
            l = ops.MatrixMul(th, X_NOTRANS, tw[lo:hi], X_TRANS)
            logits.append(l)
            stats.append(ops.RowStats(l))
        gmx = torch.stack([m for m, _ in stats]).max(dim=0).values
        gsm = sum(s * torch.exp(m - gmx) for m, s in stats)
        full = torch.cat([ops.LogSoftmaxApply(l, gmx, gsm) for l in logits], dim=1)
        assert rel_fro(full.float().cpu().numpy(), want) <= tol
    assert capi.lib().ntb_device_status(0) == capi.OK


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _rank_main(rank, world, port, out):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        rng = np.random.default_rng(77)
        h = round_to_half(rng.normal(size=(64, 512)).astype(np.float32))
        w = round_to_half((rng.normal(size=(4096, 512)) * 0.05).astype(np.float32))
        d = torch.device("cuda", rank)
        th = torch.from_numpy(h).to(d).half()
        tw = torch.from_numpy(w).to(d).half()
        w_local = shard.local_b(tw, X_TRANS, world, rank).contiguous()
        y_local = shard.vocab_parallel_output(th, w_local)
        full = shard.gather_columns(y_local, 4096)
        torch.cuda.synchronize()
        if rank == 0:
            out["y"] = full.float().cpu().numpy()
            out["h"], out["w"] = h, w
    finally:
        dist.destroy_process_group()


def test_two_nccl_ranks_share_the_vocabulary(oracle):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    port = _free_port()
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_rank_main, args=(2, port, out), nprocs=2, join=True)
        want = oracle.output_layer(out["h"], out["w"])
        assert rel_fro(out["y"], want) <= 2e-3
