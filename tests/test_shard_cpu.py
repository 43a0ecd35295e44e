"""Host logic of the multi-rank path on CPU: two gloo ranks each hold a column (or batch)
shard; the gathered result must equal the unsharded product. The per-rank product itself
is computed by the CPU oracle here -- on GPUs it is the CUDA library (tests marked gpu)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from niutensor_b200 import shard
from niutensor_b200.capi import X_TRANS, X_NOTRANS


def test_split_range_covers_everything_once():
    for total in (0, 1, 7, 8, 65536, 8192, 1000):
        for world in (1, 2, 3, 4, 8):
            for mult in (1, 8):
                spans = [shard.split_range(total, world, r, mult) for r in range(world)]
                assert spans[0][0] == 0 and spans[-1][1] == total
                for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
                    assert a1 == b0 and a0 <= a1
                if mult == 8:
                    assert all(lo % 8 == 0 for lo, _ in spans)
    with pytest.raises(ValueError):
        shard.split_range(10, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle.oracle import Oracle
        o = Oracle()
        rng = np.random.default_rng(5)                      # same data on every rank
        # output layer shape in miniature: H [M, K] times W^T, W [V, K], shard rows of W
        M, K, V = 24, 40, 100
        h = rng.normal(size=(M, K)).astype(np.float32)
        w = rng.normal(size=(V, K)).astype(np.float32)
        w_local = shard.local_b(torch.from_numpy(w), X_TRANS, world, rank)
        c_local = torch.from_numpy(o.matmul2d(h, X_NOTRANS, w_local.numpy(), X_TRANS))
        full = shard.gather_columns(c_local, V)
        ok1 = np.array_equal(full.numpy(), o.matmul2d(h, X_NOTRANS, w, X_TRANS))
        # N/N: shard columns of the stored B
        b = rng.normal(size=(K, V)).astype(np.float32)
        b_local = shard.local_b(torch.from_numpy(b), X_NOTRANS, world, rank).contiguous()
        c_local = torch.from_numpy(o.matmul2d(h, X_NOTRANS, b_local.numpy(), X_NOTRANS))
        full = shard.gather_columns(c_local, V)
        ok2 = np.array_equal(full.numpy(), o.matmul2d(h, X_NOTRANS, b, X_NOTRANS))
        # batched: shard the batch
        count = 5
        q = rng.normal(size=(count, 6, 8)).astype(np.float32)
        k = rng.normal(size=(count, 6, 8)).astype(np.float32)
        lo, hi = shard.batch_shard(count, world, rank)
        s_local = torch.from_numpy(o.matmul_batched(q[lo:hi], X_NOTRANS, k[lo:hi], X_TRANS, 0.125)) \
            if hi > lo else torch.zeros((0, 6, 6))
        s_full = shard.gather_batch(s_local, count)
        ok3 = np.array_equal(s_full.numpy(), o.matmul_batched(q, X_NOTRANS, k, X_TRANS, 0.125))
        out[rank] = int(ok1) + 2 * int(ok2) + 4 * int(ok3)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_products_gather_to_the_full_result(world):
    port = _free_port()
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
        assert dict(out) == {r: 7 for r in range(world)}


def _leaver(rank, world, port, out):
    import datetime
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    piece = torch.full((4, 8), float(rank))
    full = shard.gather_columns(piece, 16)                  # a step in which every rank takes part
    out["first_%d" % rank] = full.tolist()
    if rank == 1:
        # this rank leaves between two steps, with nothing of its own in flight
        dist.destroy_process_group()
        return
    try:
        shard.guarded(shard.gather_columns, piece, 16)
        out["second"] = "completed"
    except shard.RankLost as exc:
        out["second"] = "lost: " + str(exc)[:60]


def test_a_rank_that_leaves_between_steps_is_reported_on_the_host():
    """Failure detection without any device fault: rank 1 leaves after a complete step; rank 0's
    next collective ends with shard.RankLost (closed connection or the group's 8 s timeout)
    instead of hanging."""
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_leaver, args=(2, _free_port(), out), nprocs=2, join=True)
    assert out["first_0"] == out["first_1"]
    assert out["first_0"][0] == [0.0] * 8 + [1.0] * 8
    assert out["second"].startswith("lost: "), out["second"]
