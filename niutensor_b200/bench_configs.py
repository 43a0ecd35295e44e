"""Per-configuration timing of the MatrixMul path on one GPU.

    python -m niutensor_b200.bench_configs [--configs 1,2a,...] [--iters N] [--no-graph] [--cublas]

For each of the benchmark configurations (seeded synthetic operands of the stated shapes
and distributions) prints one JSON line: microseconds per call, TFLOP/s, algorithmic GB/s
and both roofline fractions against the measured peaks in MEASURED_PEAKS.json (fallback
figures if the file is absent). Operand sets rotate through a ring larger than twice the
126 MB L2, so every call reads its operands from HBM. Calls are replayed from a CUDA graph
by default so that host launch gaps do not count as kernel time (after 30 ms of the same
replay to bring the SM clock out of idle; median of five timed replays); `--no-graph` times plain
back-to-back calls instead. `--cublas` adds torch.matmul / torch.bmm (cuBLAS) on the same
operands as a black-box comparator.
"""
import argparse
import json
import math
import os
import sys

import torch

from . import capi, ops
from .capi import X_TRANS, X_NOTRANS

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
L2_BYTES = 126 * 1024 * 1024
OFFSET_ELEMS = 0        # --offset-elems: operands start this many elements past a 16-byte boundary

# name: (dtype, batch, M, N, K, transposedA, transposedB, alpha, beta, bound, note)
CONFIGS = {
    "1":    (torch.float32, 1, 512, 512, 512, X_NOTRANS, X_NOTRANS, 1.0, 0.0, "latency", "fp32 512^3"),
    "2a":   (torch.float16, 1, 4096, 2048, 512, X_NOTRANS, X_NOTRANS, 1.0, 0.0, "tensor", "FFN X*W1"),
    "2b":   (torch.float16, 1, 4096, 512, 2048, X_NOTRANS, X_NOTRANS, 1.0, 0.0, "tensor", "FFN H*W2"),
    "3a":   (torch.float16, 64, 256, 256, 64, X_NOTRANS, X_TRANS, 0.125, 0.0, "hbm", "attention Q*K^T"),
    "3b":   (torch.float16, 64, 256, 64, 256, X_NOTRANS, X_NOTRANS, 1.0, 0.0, "hbm", "attention P*V"),
    "4":    (torch.float16, 1, 256, 65536, 512, X_NOTRANS, X_TRANS, 1.0, 0.0, "hbm", "output layer H*W^T"),
    "5":    (torch.float16, 1, 8192, 8192, 8192, X_NOTRANS, X_NOTRANS, 1.0, 0.5, "tensor", "8192^3 fp16"),
    "5f32": (torch.float32, 1, 8192, 8192, 8192, X_NOTRANS, X_NOTRANS, 1.0, 0.5, "tensor", "8192^3 fp32"),
    # not in the benchmark list: a weight gradient as XBackwardMath forms it (a^T * dE/dc accumulated
    # into dE/db, 8192 tokens), the shape class the split on CTA pairs serves
    "wgrad": (torch.float16, 1, 1024, 1024, 8192, X_TRANS, X_NOTRANS, 1.0, 1.0, "tensor", "weight gradient a^T * dE/dc, 8192 tokens"),
}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["bf16_tflops"]), float(d["hbm_gbs"]), "measured"
    return 1590.0, 6650.0, "fallback"


def time_calls(fn, n_round, use_graph):
    """Microseconds per call of fn(i), i = 0 .. n_round-1. The sequence is replayed for at
    least 30 ms first, so that the SM clock has left its idle state, then timed five times;
    the median is returned."""
    for i in range(min(n_round, 8) + 3):
        fn(i)
    torch.cuda.synchronize()
    if use_graph:
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                for i in range(n_round):
                    fn(i)

        def once():
            graph.replay()
    else:
        def once():
            for i in range(n_round):
                fn(i)
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    once()
    e1.record()
    torch.cuda.synchronize()
    first_ms = max(e0.elapsed_time(e1), 1e-3)
    for _ in range(min(2000, int(30.0 / first_ms) + 1)):
        once()
    torch.cuda.synchronize()
    samples = []
    for _ in range(5):
        e0.record()
        once()
        e1.record()
        torch.cuda.synchronize()
        samples.append(e0.elapsed_time(e1) * 1e3 / n_round)
    samples.sort()
    return samples[2]


def make_set(cfg, dev, seed):
    dtype, batch, M, N, K, tA, tB, alpha, beta, _, _ = cfg
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    lead = (batch,) if batch > 1 else ()
    a_shape = lead + ((K, M) if tA == X_TRANS else (M, K))
    b_shape = lead + ((N, K) if tB == X_TRANS else (K, N))
    a = torch.randn(a_shape, device=dev, generator=g).to(dtype)
    b = (torch.randn(b_shape, device=dev, generator=g) / math.sqrt(K)).to(dtype)
    c = torch.randn(lead + (M, N), device=dev, generator=g).to(dtype)
    if OFFSET_ELEMS:
        # the operands as a memory pool would hand them out: the same values, starting
        # OFFSET_ELEMS elements past a 16-byte boundary (no tensor map can address them)
        def shifted(x):
            buf = torch.empty(x.numel() + 16, device=dev, dtype=dtype)
            view = buf[OFFSET_ELEMS:OFFSET_ELEMS + x.numel()].view(x.shape)
            view.copy_(x)
            return view
        a, b = shifted(a), shifted(b)
    return a, b, c


def run_config(name, iters, use_graph, with_cublas, dev):
    cfg = CONFIGS[name]
    dtype, batch, M, N, K, tA, tB, alpha, beta, bound, note = cfg
    es = 2 if dtype == torch.float16 else 4
    flops = 2.0 * M * N * K * batch
    nbytes = es * batch * (M * K + K * N + M * N * (2 if beta != 0 else 1))
    ring = max(1, min(64, int(math.ceil(2.0 * L2_BYTES / nbytes))))
    sets = [make_set(cfg, dev, 1000 + i) for i in range(ring)]
    call = ops._MatrixMulBatched if batch > 1 else ops._MatrixMul2D

    def ours(i):
        a, b, c = sets[i % ring]
        call(a, tA, b, tB, c, alpha, beta)

    def cublas(i):
        a, b, c = sets[i % ring]
        x = a.transpose(-1, -2) if tA == X_TRANS else a
        y = b.transpose(-1, -2) if tB == X_TRANS else b
        if beta != 0:
            torch.baddbmm(c, x, y, beta=beta, alpha=alpha, out=c) if batch > 1 else \
                torch.addmm(c, x, y, beta=beta, alpha=alpha, out=c)
        else:
            torch.matmul(x, y, out=c)

    def time_fn(fn):
        return time_calls(fn, ring * max(1, iters // ring), use_graph)

    us = time_fn(ours)
    route = capi.lib().ntb_last_route()
    peak_tf, peak_gb, src = peaks()
    line = {"config": name, "what": note, "dtype": "f16" if es == 2 else "f32", "batch": batch,
            "M": M, "N": N, "K": K, "us_per_call": us, "tflops": flops / us / 1e6,
            "algorithmic_mb": nbytes / 1e6, "algorithmic_gb_per_s": nbytes / us / 1e3,
            "frac_of_tensor_peak": flops / us / 1e6 / peak_tf, "frac_of_hbm_peak": nbytes / us / 1e3 / peak_gb,
            "bound": bound, "peaks": src, "route": route, "ring_sets": ring,
            "timing": "cuda graph replay" if use_graph else "back-to-back calls"}
    if with_cublas:
        cu = time_fn(cublas)
        line["cublas_us_per_call"] = cu
        line["speedup_vs_cublas"] = cu / us
    del sets
    torch.cuda.empty_cache()
    return line


def run_attention(iters, use_graph, with_cublas, dev):
    """Config 3 as one fused call: 64 blocks (8 heads x 8 sentences), length 256, head 64."""
    blocks, length, d = 64, 256, 64
    flops = 2.0 * 2 * blocks * length * length * d
    nbytes = 2.0 * 4 * blocks * length * d                   # q, k, v in, out out; scores never reach HBM
    ring = int(math.ceil(2.0 * L2_BYTES / nbytes))
    g = torch.Generator(device=dev)
    g.manual_seed(1003)
    sets = [tuple(torch.randn(blocks, length, d, device=dev, generator=g).half() for _ in range(3)) for _ in range(ring)]
    outs = [None] * ring

    def fused(i):
        q, k, v = sets[i % ring]
        outs[i % ring] = ops.ScaledDotProductAttention(q, k, v)

    def chain(i):
        q, k, v = sets[i % ring]
        s = ops.BMMul(q, X_NOTRANS, k, X_TRANS, 0.125)
        p = torch.softmax(s.float(), dim=-1).half()
        outs[i % ring] = ops.BMMul(p, X_NOTRANS, v, X_NOTRANS)

    def sdpa(i):
        q, k, v = sets[i % ring]
        outs[i % ring] = torch.nn.functional.scaled_dot_product_attention(q, k, v)

    def time_fn(fn):
        return time_calls(fn, ring * max(1, iters // ring), use_graph)

    us = time_fn(fused)
    peak_tf, peak_gb, src = peaks()
    line = {"config": "3fused", "what": "attention: softmax(q k^T / 8) v in one kernel", "dtype": "f16", "batch": blocks,
            "M": length, "N": length, "K": d, "us_per_call": us, "tflops": flops / us / 1e6,
            "algorithmic_mb": nbytes / 1e6, "algorithmic_gb_per_s": nbytes / us / 1e3,
            "frac_of_tensor_peak": flops / us / 1e6 / peak_tf, "frac_of_hbm_peak": nbytes / us / 1e3 / peak_gb,
            "bound": "hbm", "peaks": src, "ring_sets": ring,
            "timing": "cuda graph replay" if use_graph else "back-to-back calls",
            "unfused_chain_us": time_fn(chain)}
    if with_cublas:
        line["torch_sdpa_us"] = time_fn(sdpa)
    return line


def run_output_layer(iters, use_graph, with_cublas, dev):
    """Config 4 followed by the log-softmax over the vocabulary (one shard = the whole of it)."""
    from . import shard
    rows, hidden, vocab = 256, 512, 65536
    g = torch.Generator(device=dev)
    g.manual_seed(1004)
    ring = 3
    sets = [(torch.randn(rows, hidden, device=dev, generator=g).half(),
             (torch.randn(vocab, hidden, device=dev, generator=g) * 0.02).half()) for _ in range(ring)]

    def ours(i):
        h, w = sets[i % ring]
        shard.vocab_parallel_output(h, w)

    def cublas(i):
        h, w = sets[i % ring]
        torch.log_softmax(torch.matmul(h, w.t()).float(), dim=-1).half()

    us = time_calls(ours, ring * max(1, iters // ring), use_graph)
    flops = 2.0 * rows * hidden * vocab
    nbytes = 2.0 * (rows * hidden + vocab * hidden + 3 * rows * vocab)     # logits written, read twice, written once more... see note
    peak_tf, peak_gb, src = peaks()
    line = {"config": "4lsm", "what": "output layer + LogSoftmax over the vocabulary (3 kernels)", "dtype": "f16",
            "M": rows, "N": vocab, "K": hidden, "us_per_call": us, "tflops": flops / us / 1e6,
            "algorithmic_mb": 2.0 * (rows * hidden + vocab * hidden + rows * vocab) / 1e6,
            "moved_mb_by_three_kernels": nbytes / 1e6, "bound": "hbm", "peaks": src,
            "frac_of_hbm_peak": 2.0 * (rows * hidden + vocab * hidden + rows * vocab) / us / 1e3 / peak_gb,
            "timing": "cuda graph replay" if use_graph else "back-to-back calls"}
    if with_cublas:
        line["torch_matmul_log_softmax_us"] = time_calls(cublas, ring * max(1, iters // ring), use_graph)
    return line


def _compact(line):
    """The fields of a run_config line that the benchmark's one-line summary carries."""
    bound = line.get("bound", "tensor")
    frac = line.get("frac_of_hbm_peak") if bound == "hbm" else line.get("frac_of_tensor_peak")
    out = {"what": line["what"], "us": round(line["us_per_call"], 2), "tflops": round(line["tflops"], 1),
           "algorithmic_gb_per_s": round(line["algorithmic_gb_per_s"], 1) if "algorithmic_gb_per_s" in line else None,
           "bound": bound, "frac": round(frac, 4) if frac is not None else None,
           "frac_of": "measured HBM copy GB/s" if bound == "hbm" else "measured bf16 cuBLAS burst TFLOP/s",
           "route": line.get("route")}
    for k in ("cublas_us_per_call", "unfused_chain_us", "torch_sdpa_us", "torch_matmul_log_softmax_us"):
        if k in line:
            out[k.replace("_per_call", "")] = round(line[k], 2)
    return out


def driver_table(dev, iters=60):
    """Every benchmark configuration except the headline one, timed in this process on one
    GPU (CUDA-graph replay over an operand ring larger than twice the L2), each beside
    cuBLAS / torch on the same operands."""
    table = {}
    for name in ("1", "2a", "2b", "3a", "3b", "3fused", "4", "4lsm", "5f32", "wgrad"):
        try:
            if name == "3fused":
                line = run_attention(iters, True, True, dev)
            elif name == "4lsm":
                line = run_output_layer(iters, True, True, dev)
            else:
                line = run_config(name, iters if name != "5f32" else 8, True, True, dev)
            table[name] = _compact(line)
        except Exception as exc:
            table[name] = {"failed": repr(exc)}
    return table


def sharded_table(dev, world, rank, timed):
    """N > 1: the output layer with the vocabulary sharded over the ranks, logits left
    sharded (config 4), and the fp32 form of the large square product, column-sharded with C
    left distributed. `timed(fn, steps)` is the caller's barrier-bracketed timer (max over
    ranks)."""
    from . import shard
    table = {}
    g = torch.Generator(device=dev)
    g.manual_seed(1004)
    rows, hidden, vocab = 256, 512, 65536
    lo, hi = shard.split_range(vocab, world, rank, 8)
    nbytes = 2.0 * (rows * hidden + (hi - lo) * hidden + rows * (hi - lo))
    ring = max(1, min(64, int(math.ceil(2.0 * L2_BYTES / nbytes))))
    sets = [(torch.randn(rows, hidden, device=dev, generator=g).half(),
             (torch.randn(hi - lo, hidden, device=dev, generator=g) * 0.02).half(),
             torch.empty(rows, hi - lo, device=dev, dtype=torch.float16)) for _ in range(ring)]
    state = {"i": 0}

    def out_layer():
        h, w_local, c = sets[state["i"] % ring]
        state["i"] += 1
        ops._MatrixMul2D(h, X_NOTRANS, w_local, X_TRANS, c, 1.0, 0.0)

    for _ in range(ring):
        out_layer()
    ms, _, _ = timed(out_layer, 4 * ring)
    flops = 2.0 * rows * hidden * vocab
    table["4"] = {"what": "output layer H*W^T, vocabulary rows sharded over %d ranks, logits left sharded" % world,
                  "us": round(ms * 1e3, 2), "tflops": round(flops / ms / 1e9, 1),
                  "algorithmic_gb_per_s_per_gpu": round(nbytes / ms / 1e6, 1), "bound": "hbm",
                  "timing": "back-to-back calls from Python, max over ranks (host launch gaps included)"}
    del sets
    torch.cuda.empty_cache()
    n = 8192
    clo, chi = shard.column_shard(n, world, rank)
    a = (torch.rand(n, n, device=dev, generator=g) * 2 - 1)
    b = (torch.rand(n, chi - clo, device=dev, generator=g) * 2 - 1)
    c = torch.randn(n, chi - clo, device=dev, generator=g)

    def big_f32():
        ops._MatrixMul2D(a, X_NOTRANS, b, X_NOTRANS, c, 1.0, 0.5)

    for _ in range(2):
        big_f32()
    ms, _, _ = timed(big_f32, 5)
    table["5f32"] = {"what": "fp32 8192^3, beta 0.5, column-sharded over %d ranks, C left distributed" % world,
                     "us": round(ms * 1e3, 1), "tflops": round(2.0 * n * n * n / ms / 1e9, 1), "bound": "tensor"}
    return table


def run_accuracy(dev):
    """fp32 products against the float64 product of the same fp32 inputs, for K from 256 to
    16384, on both fp32 routes (three kind::tf32 passes with chains of 256 of K; two half pieces
    per value with chains of 512) and for torch.matmul (cuBLAS SGEMM): relative Frobenius error
    and mean signed relative error. Inputs U[-1, 1] ("sym") and U[0, 1] ("pos": partial sums
    only grow, the worst case for a truncating accumulator)."""
    g = torch.Generator(device=dev)
    g.manual_seed(77)
    L = capi.lib()
    for (M, N, K) in ((512, 512, 256), (512, 512, 1024), (512, 512, 4096), (512, 512, 16384), (2048, 2048, 2048)):
        for kind in ("sym", "pos"):
            a = torch.rand(M, K, device=dev, generator=g)
            b = torch.rand(K, N, device=dev, generator=g)
            if kind == "sym":
                a, b = a * 2 - 1, b * 2 - 1
            truth = a.double() @ b.double()
            row = {"M": M, "N": N, "K": K, "inputs": kind}
            for name, env in (("tf32x3", "0"), ("f16x2", "1")):
                os.environ["NTB_F32_SPLIT"] = env
                c = torch.zeros(M, N, device=dev)
                ops._MatrixMul2D(a, X_NOTRANS, b, X_NOTRANS, c, 1.0, 0.0)
                torch.cuda.synchronize()
                d = c.double() - truth
                row[name] = {"route": L.ntb_last_route(), "rel_fro": float(d.norm() / truth.norm()),
                             "signed": float((d / truth.abs().clamp_min(1e-30)).mean()) if kind == "pos" else None}
            os.environ.pop("NTB_F32_SPLIT", None)
            d = (a @ b).double() - truth
            row["cublas_sgemm_rel_fro"] = float(d.norm() / truth.norm())
            print(json.dumps(row), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--configs", default="1,2a,2b,3a,3b,3fused,4,4lsm,5,5f32")
    ap.add_argument("--iters", type=int, default=60)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--cublas", action="store_true")
    ap.add_argument("--shapes", default="",
                    help="extra fp16 products M x N x K (a row-major, b stored N x K, beta 0), e.g. 4096x512x2048,2048x1024x4096")
    ap.add_argument("--f32-shapes", default="",
                    help="extra fp32 products M x N x K (a and b row-major, beta 0.5), e.g. 4096x4096x4096")
    ap.add_argument("--offset-elems", type=int, default=0,
                    help="place a and b this many elements past a 16-byte boundary, as a memory pool may "
                         "(NTB_REPACK=0 then times the loader-warp kernel instead of the realigning pre-pass)")
    ap.add_argument("--accuracy", action="store_true", help="fp32 routes against float64 instead of timings")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("no CUDA device; this path has no CPU implementation")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    if args.accuracy:
        run_accuracy(dev)
        return 0
    global OFFSET_ELEMS
    OFFSET_ELEMS = max(0, min(15, args.offset_elems))
    names = [n for n in args.configs.split(",") if n]
    for shape in [x for x in args.shapes.split(",") if x]:
        M, N, K = (int(v) for v in shape.lower().split("x"))
        CONFIGS[shape] = (torch.float16, 1, M, N, K, X_NOTRANS, X_TRANS, 1.0, 0.0, "tensor", "fp16 " + shape)
        names.append(shape)
    for shape in [x for x in args.f32_shapes.split(",") if x]:
        M, N, K = (int(v) for v in shape.lower().split("x"))
        CONFIGS["f32 " + shape] = (torch.float32, 1, M, N, K, X_NOTRANS, X_NOTRANS, 1.0, 0.5, "tensor", "fp32 " + shape)
        names.append("f32 " + shape)
    for name in names:
        if name == "4lsm":
            print(json.dumps(run_output_layer(args.iters, not args.no_graph, args.cublas, dev)), flush=True)
            continue
        if name == "3fused":
            print(json.dumps(run_attention(args.iters, not args.no_graph, args.cublas, dev)), flush=True)
            continue
        iters = args.iters if not name.startswith("5") else max(5, args.iters // 6)
        print(json.dumps(run_config(name, iters, not args.no_graph, args.cublas, dev)), flush=True)
    status = capi.lib().ntb_device_status(0)
    if status != capi.OK:
        raise SystemExit("device status %d" % status)


if __name__ == "__main__":
    sys.exit(main())
