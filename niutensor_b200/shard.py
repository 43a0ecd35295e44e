"""Sharding one matrix product across the ranks of a process group (one process per GPU).

Output tiles of a product are independent, so the path shards with no exchange:

* 2-D products shard the columns of C: A is replicated, rank r owns the columns
  [n0, n1) of op(B) -- rows of the stored B when transposedB == X_TRANS (the output layer:
  rows of the vocabulary matrix), columns of the stored B otherwise -- and produces
  C[:, n0:n1].
* batched products (BMMul) shard the leading (batch) extent.

A collective is needed only when a caller wants the whole C on every rank:
`gather_columns` / `gather_batch` (all_gather over the group's backend -- NCCL over NVLink
on GPUs, gloo in CPU tests -- plus the local re-interleave, because column shards of a
row-major matrix are not contiguous).
"""
import torch
import torch.distributed as dist

from .capi import X_TRANS, X_NOTRANS


def split_range(total, world, rank, multiple=1):
    """[lo, hi) of `total` units for `rank`: contiguous, balanced in units of `multiple`
    (the last rank takes the ragged remainder)."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError("bad rank %d of %d" % (rank, world))
    blocks = (total + multiple - 1) // multiple
    lo = (blocks * rank // world) * multiple
    hi = (blocks * (rank + 1) // world) * multiple
    return min(lo, total), min(hi, total)


def column_shard(n_cols, world, rank):
    """Columns of C owned by `rank`; multiples of 8 keep fp16 row segments 16-byte aligned,
    which the TMA-fed kernels need when the shard is addressed inside a resident matrix."""
    return split_range(n_cols, world, rank, 8)


def local_b(b_full, transposedB, world, rank):
    """The part of a full stored B that `rank` multiplies by (a view, no copy)."""
    if transposedB == X_TRANS:
        lo, hi = column_shard(b_full.shape[-2], world, rank)
        return b_full[..., lo:hi, :]
    lo, hi = column_shard(b_full.shape[-1], world, rank)
    return b_full[..., :, lo:hi]


def matmul_column_shard(a, transposedA, b_local, transposedB, alpha=1.0, beta=0.0, c_local=None):
    """This rank's columns of C = alpha * op(a) * op(b) + beta * C from its packed shard of B."""
    from . import ops
    if not b_local.is_contiguous():
        b_local = b_local.contiguous()
    return ops.MatrixMul(a, transposedA, b_local, transposedB, alpha, beta, c=c_local)


def symmetric_matrix(rows, cols, dtype, device, group=None, multicast=False):
    """A [rows, cols] matrix allocated on every rank of the group in symmetric memory, and
    the device addresses under which this process can write the other ranks' copies (NVLink
    peer mappings). Returns (tensor, {rank: address}) -- plain stores, no multicast object:
    TORCH_SYMM_MEM_DISABLE_MULTICAST is set unless the caller chose otherwise -- or, with
    multicast=True, (tensor, {rank: address}, multicast address or 0): the address under which
    one multimem store reaches every rank's copy, 0 where the platform offers no NVLink
    multicast. The first symmetric allocation of a process decides which of the two it gets."""
    import os
    if multicast:
        os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "0"
    else:
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    import torch.distributed._symmetric_memory as symm
    group = group if group is not None else dist.group.WORLD
    t = symm.empty((rows, cols), dtype=dtype, device=device)
    hdl = symm.rendezvous(t, group)
    me = dist.get_rank(group)
    peers = {r: int(hdl.buffer_ptrs[r]) for r in range(dist.get_world_size(group)) if r != me}
    if not multicast:
        return t, peers
    mc = 0
    try:
        mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
    except Exception:
        mc = 0
    return t, peers, mc


def matmul_column_shard_to_all(a, transposedA, b_local, transposedB, c_sym, peer_addrs, n_cols, group=None,
                               alpha=1.0, beta=0.0):
    """Every rank computes its column block of C from its packed shard of B and its epilogue
    writes the block into its own c_sym and into every other rank's (ntb_gemm_peers): after
    the closing barrier all ranks hold the full C. Replaces product + all-gather + the
    re-interleaving pass of gather_columns."""
    from . import ops
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    lo, hi = column_shard(n_cols, world, rank)
    if not b_local.is_contiguous():
        b_local = b_local.contiguous()
    ops.MatrixMul2DToPeers(a, transposedA, b_local, transposedB, c_sym, lo, [peer_addrs[r] for r in sorted(peer_addrs)],
                           alpha, beta)
    torch.cuda.current_stream(c_sym.device).synchronize()
    dist.barrier(group)
    return c_sym


class RankLost(RuntimeError):
    """A collective of the sharded path did not complete: a rank left, never joined, or the
    group's timeout ran out. The caller's step is void; nothing was left half-launched on this
    rank (the error surfaces on the host, between launches)."""


def guarded(collective, *args, **kwargs):
    """Runs one collective-bearing call of this module (gather_columns, vocab_parallel_output,
    ...) and turns the backend's own errors -- a closed connection, the process group's
    timeout -- into RankLost, so that a trainer can tell "a peer is gone" from a bug. The
    reference has no counterpart: its workers share one process (source/train/XWorkerJob.cpp)
    and cannot lose one another. Give the process group a short timeout
    (init_process_group(..., timeout=...)) for this to answer quickly."""
    try:
        out = collective(*args, **kwargs)
        if torch.cuda.is_available() and any(isinstance(a, torch.Tensor) and a.is_cuda for a in args):
            torch.cuda.current_stream().synchronize()     # NCCL reports a lost peer when the work is waited for
        return out
    except (RuntimeError, dist.DistBackendError, dist.DistNetworkError) as exc:
        raise RankLost("collective failed: %s" % (str(exc).splitlines()[0] if str(exc) else type(exc).__name__)) from exc


def gather_columns(c_local, n_cols, group=None):
    """All ranks receive the full [..., M, n_cols] matrix from the per-rank column shards.

    Equal shards on CUDA devices take one collective and one pass: all_gather_into_tensor
    leaves the packed shards one after the other ([world][rows][w]) and one kernel
    (ntb_unshard_columns) writes them to their columns of the row-major result. Ragged
    shards, and CPU tensors in the gloo tests, are padded to a common width, gathered as a
    list and copied into place."""
    world = dist.get_world_size(group)
    widths = [column_shard(n_cols, world, r) for r in range(world)]
    wmax = max(hi - lo for lo, hi in widths)
    lead = tuple(c_local.shape[:-1])
    es = c_local.element_size()
    uniform = all(hi - lo == wmax for lo, hi in widths) and wmax * world == n_cols
    if uniform and c_local.is_cuda and c_local.dtype in (torch.float16, torch.float32) and (wmax * es) % 16 == 0:
        from . import capi
        piece = c_local if c_local.is_contiguous() else c_local.contiguous()
        rows = piece.numel() // wmax
        packed = torch.empty((world,) + lead + (wmax,), dtype=piece.dtype, device=piece.device)
        dist.all_gather_into_tensor(packed, piece, group=group)
        full = torch.empty(lead + (n_cols,), dtype=piece.dtype, device=piece.device)
        code = capi.X_FLOAT16 if piece.dtype == torch.float16 else capi.X_FLOAT
        rc = capi.lib().ntb_unshard_columns(piece.device.index, torch.cuda.current_stream(piece.device).cuda_stream,
                                            packed.data_ptr(), full.data_ptr(), code, rows, world, wmax, n_cols)
        capi.check(rc, "ntb_unshard_columns")
        return full
    # equal-sized pieces for all_gather: pad the narrower shards
    piece = torch.zeros(lead + (wmax,), dtype=c_local.dtype, device=c_local.device)
    piece[..., :c_local.shape[-1]] = c_local
    pieces = [torch.empty_like(piece) for _ in range(world)]
    dist.all_gather(pieces, piece, group=group)
    full = torch.empty(lead + (n_cols,), dtype=c_local.dtype, device=c_local.device)
    for r, (lo, hi) in enumerate(widths):
        full[..., lo:hi] = pieces[r][..., :hi - lo]
    return full


def batch_shard(count, world, rank):
    return split_range(count, world, rank, 1)


def gather_batch(c_local, count, group=None):
    """All ranks receive all `count` result matrices from per-rank batch shards."""
    world = dist.get_world_size(group)
    sizes = [batch_shard(count, world, r) for r in range(world)]
    bmax = max(hi - lo for lo, hi in sizes)
    tail = tuple(c_local.shape[1:])
    piece = torch.zeros((bmax,) + tail, dtype=c_local.dtype, device=c_local.device)
    piece[:c_local.shape[0]] = c_local
    pieces = [torch.empty_like(piece) for _ in range(world)]
    dist.all_gather(pieces, piece, group=group)
    return torch.cat([pieces[r][:hi - lo] for r, (lo, hi) in enumerate(sizes)], dim=0)


def vocab_parallel_output(h, w_local, group=None, normalized=True):
    """The output layer with the vocabulary matrix sharded by rows across the group
    (source/sample/transformer/submodel/Output.cpp:86-101: MMul(h, w^T), then LogSoftmax
    over the vocabulary for beam search). Every rank holds all of h [rows, hidden] and its
    rows of w [vocab / world, hidden]; it returns its columns of the log-probabilities.
    The logits are never gathered: the ranks exchange one maximum and one sum per row."""
    from . import ops
    logits = ops.MatrixMul(h.reshape(-1, h.shape[-1]), X_NOTRANS, w_local, X_TRANS)
    if not normalized:
        return logits
    mx, sm = ops.RowStats(logits)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        gmx = mx.clone()
        dist.all_reduce(gmx, op=dist.ReduceOp.MAX, group=group)
        # a shard whose row is entirely -inf contributes nothing
        sm = torch.where(torch.isinf(mx) & (mx < 0), torch.zeros_like(sm), sm * torch.exp(mx - gmx))
        dist.all_reduce(sm, op=dist.ReduceOp.SUM, group=group)
        mx = gmx
    return ops.LogSoftmaxApply(logits, mx, sm)
