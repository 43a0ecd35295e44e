"""Per-configuration timing of the MatrixMul path on one GPU.

    python -m niutensor_b200.bench_configs [--configs 1,2a,...] [--iters N] [--no-graph] [--cublas]

For each of the benchmark configurations (seeded synthetic operands of the stated shapes
and distributions) prints one JSON line: microseconds per call, TFLOP/s, algorithmic GB/s
and both roofline fractions against the measured peaks in MEASURED_PEAKS.json (fallback
figures if the file is absent). Operand sets rotate through a ring larger than twice the
126 MB L2, so every call reads its operands from HBM. Calls are replayed from a CUDA graph
by default so that host launch gaps do not count as kernel time; `--no-graph` times plain
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
        n_round = ring * max(1, iters // ring)
        for i in range(min(ring, 8) + 3):
            fn(i)
        torch.cuda.synchronize()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        if use_graph:
            side = torch.cuda.Stream()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    for i in range(n_round):
                        fn(i)
            graph.replay()
            torch.cuda.synchronize()
            e0.record()
            graph.replay()
            e1.record()
        else:
            e0.record()
            for i in range(n_round):
                fn(i)
            e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / n_round

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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--configs", default="1,2a,2b,3a,3b,4,5,5f32")
    ap.add_argument("--iters", type=int, default=60)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--cublas", action="store_true")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("no CUDA device; this path has no CPU implementation")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    for name in args.configs.split(","):
        iters = args.iters if not name.startswith("5") else max(5, args.iters // 6)
        print(json.dumps(run_config(name, iters, not args.no_graph, args.cublas, dev)), flush=True)
    status = capi.lib().ntb_device_status(0)
    if status != capi.OK:
        raise SystemExit("device status %d" % status)


if __name__ == "__main__":
    sys.exit(main())
