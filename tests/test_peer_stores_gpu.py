"""The product whose epilogue also writes its column block of C into the other ranks' copies
(ntb_gemm_peers over symmetric memory): two NCCL ranks, one per GPU. Plain peer stores; no
multicast object is bound (NVLS off)."""
import os
import socket

import numpy as np
import pytest
import torch

from niutensor_b200 import shard
from niutensor_b200.capi import X_TRANS, X_NOTRANS
from oracle.oracle import rel_fro, round_to_half

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"     # peer mappings only, no multicast object
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        rng = np.random.default_rng(91)
        M, N, K = 384, 1000, 512
        a = round_to_half(rng.uniform(-1, 1, (M, K)).astype(np.float32))
        b = round_to_half(rng.uniform(-1, 1, (N, K)).astype(np.float32))
        d = torch.device("cuda", rank)
        ta = torch.from_numpy(a).to(d).half()
        tb = torch.from_numpy(b).to(d).half()
        c_sym, peers = shard.symmetric_matrix(M, N, torch.float16, d)
        c_sym.fill_(-3.0)
        torch.cuda.synchronize()
        dist.barrier()
        b_local = shard.local_b(tb, X_TRANS, world, rank).contiguous()
        shard.matmul_column_shard_to_all(ta, X_NOTRANS, b_local, X_TRANS, c_sym, peers, N, alpha=0.5)
        out["c%d" % rank] = c_sym.float().cpu().numpy()
        if rank == 0:
            out["a"], out["b"] = a, b
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_ranks_gather_c_through_the_epilogue(oracle):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    port = _free_port()
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_rank_main, args=(2, port, out), nprocs=2, join=True)
        want = oracle.matmul2d(out["a"], X_NOTRANS, out["b"], X_TRANS, 0.5, 0.0)
        assert rel_fro(out["c0"], want) <= 2e-3
        assert np.array_equal(out["c0"], out["c1"])


def _rank_main_multicast(rank, world, port, out):
    import torch.distributed as dist
    from niutensor_b200 import ops
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        rng = np.random.default_rng(92)
        M, N, K = 520, 1024, 320
        a = round_to_half(rng.uniform(-1, 1, (M, K)).astype(np.float32))
        b = round_to_half(rng.uniform(-1, 1, (K, N)).astype(np.float32))
        c0 = round_to_half(rng.normal(size=(M, N)).astype(np.float32))
        d = torch.device("cuda", rank)
        c_sym, peers, mc = shard.symmetric_matrix(M, N, torch.float16, d, multicast=True)
        out["mc%d" % rank] = int(mc != 0)
        if mc != 0:
            c_sym.copy_(torch.from_numpy(c0).to(d).half())
            torch.cuda.synchronize()
            dist.barrier()
            lo, hi = shard.column_shard(N, world, rank)
            b_local = torch.from_numpy(np.ascontiguousarray(b[:, lo:hi])).to(d).half()
            ops.MatrixMul2DToMulticast(torch.from_numpy(a).to(d).half(), X_NOTRANS, b_local, X_NOTRANS, c_sym, lo, mc, 0.5, 0.25)
            torch.cuda.synchronize()
            dist.barrier()
            out["c%d" % rank] = c_sym.float().cpu().numpy()
        if rank == 0:
            out["a"], out["b"], out["init"] = a, b, c0
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_ranks_gather_c_through_the_switch(oracle):
    """ntb_gemm_multicast: every rank writes its block once, with multimem.st, to the multicast
    address of the symmetric C; the NVLink switch delivers it to both ranks. Both ranks exit
    normally; skipped where the platform offers no multicast object."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    port = _free_port()
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_rank_main_multicast, args=(2, port, out), nprocs=2, join=True)
        if not (out["mc0"] and out["mc1"]):
            pytest.skip("no NVLink multicast object on this platform")
        want = oracle.matmul2d(out["a"], X_NOTRANS, out["b"], X_NOTRANS, 0.5, 0.25, out["init"])
        got0, got1 = out["c0"], out["c1"]
        assert rel_fro(got0, want) <= 2e-3
        assert np.array_equal(got0, got1)
