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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--configs", default="1,2a,2b,3a,3b,3fused,4,4lsm,5,5f32")
    ap.add_argument("--iters", type=int, default=60)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--cublas", action="store_true")
    ap.add_argument("--shapes", default="",
                    help="extra fp16 products M x N x K (a row-major, b stored N x K, beta 0), e.g. 4096x512x2048,2048x1024x4096")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("no CUDA device; this path has no CPU implementation")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    names = [n for n in args.configs.split(",") if n]
    for shape in [x for x in args.shapes.split(",") if x]:
        M, N, K = (int(v) for v in shape.lower().split("x"))
        CONFIGS[shape] = (torch.float16, 1, M, N, K, X_NOTRANS, X_TRANS, 1.0, 0.0, "tensor", "fp16 " + shape)
        names.append(shape)
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
