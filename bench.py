#!/usr/bin/env python
"""Benchmark of the MatrixMul hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (`config.workload`): the large square product of the benchmark list,
C = 1.0 * A * B + 0.5 * C0 with A, B 8192 x 8192 ~ U[-1, 1] and C0 ~ N(0, 1), fp16 tensors,
no transposition. With N ranks the product is N-sharded: A is replicated, rank r owns
column block r of B, C0 and C (8192 columns each), so the global problem is
8192 x (8192 N) x 8192 and per-GPU work is fixed ("weak" scaling); there is no data-path
collective. One step = one MatrixMul over the resident operands. Inputs are seeded
synthetic data of the stated distributions.

One JSON line on stdout (rank 0). `value` is TFLOP/s with operands resident in HBM;
`e2e` is the same metric through the host-buffer entry point of the C ABI, host-to-device
and device-to-host copies inside the timed region.

`--impl reference` times the reference's own CPU MatrixMul (the NiuTensor library built
into oracle/_ref by `make -C oracle ref`: OpenBLAS build with every host thread if
present, else its built-in single-thread loops on a row sample; if neither exists, the
plain-C restatement) on the same operands, fp16 values carried in fp32 because the
reference has no CPU half arithmetic.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

N_DIM = 8192
ALPHA, BETA = 1.0, 0.5
WORKLOAD = "MatrixMul fp16 8192x8192x8192 N/N alpha=1 beta=0.5 (benchmark config 5), column-sharded x n_gpus"
FLOPS_PER_RANK = 2.0 * N_DIM * N_DIM * N_DIM
# algorithmic bytes of one launch: read A, B and C0 once, write C once (fp16)
BYTES_PER_RANK = 4.0 * N_DIM * N_DIM * 2
# DRAM traffic of one launch measured by ncu (dram__bytes_read.sum + dram__bytes_write.sum),
# profiles/gemm_f16_8192_ncu.md (CTA-pair kernel with 512 x 256 tiles, the one this shape runs on)
NCU_TRAFFIC_BYTES = 1.075e9


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"burst": float(d["bf16_tflops"]), "sustained": float(d["bf16_tflops_sustained"]),
                "hbm": float(d["hbm_gbs"]), "source": "measured"}
    return {"burst": 1590.0, "sustained": 1400.0, "hbm": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.12)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        inside = [l for (t, l) in self.lines if t0 <= t <= t1 + 0.05] or [l for (_, l) in self.lines]
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for l in inside:
            parts = [x.strip() for x in l.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": float(max(mx)) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------ CPU reference arm

def host_operands(rows=N_DIM):
    """Rank-0 operands as fp16-valued float32 host arrays (A is cut to `rows` rows)."""
    rng = np.random.default_rng(1005)
    a = rng.uniform(-1, 1, (rows, N_DIM)).astype(np.float16).astype(np.float32)
    b = rng.uniform(-1, 1, (N_DIM, N_DIM)).astype(np.float16).astype(np.float32)
    c0 = rng.normal(size=(rows, N_DIM)).astype(np.float16).astype(np.float32)
    return a, b, c0


def cpu_reference_runner():
    """Returns (kind, cores, sample description, rows, callable(a, b, c0) -> seconds)."""
    from oracle import oracle as orc          # checker / CPU baseline only
    cores = os.cpu_count() or 1
    if orc.ref_available("openblas"):
        try:
            ref = orc.Reference("openblas")
            ref.set_threads(cores)
            rows = N_DIM

            def run(a, b, c0):
                t = time.perf_counter()
                ref.run(ref.FORM_GENERAL, a, orc.X_NOTRANS, b, orc.X_NOTRANS, ALPHA, BETA, c0, inplace=True)
                return time.perf_counter() - t
            return ("reference", cores, "whole 8192^3 product, reference built with USE_BLAS on OpenBLAS, "
                    "%d threads, fp16 values in fp32" % cores, rows, run)
        except OSError:
            pass
    if orc.ref_available("builtin"):
        ref = orc.Reference("builtin")
        rows = 64

        def run(a, b, c0):
            t = time.perf_counter()
            ref.run(ref.FORM_GENERAL, a, orc.X_NOTRANS, b, orc.X_NOTRANS, ALPHA, BETA, c0, inplace=True)
            return time.perf_counter() - t
        return ("reference", 1, "first 64 of 8192 rows (64x8192x8192), reference built-in loops, 1 thread",
                rows, run)
    o = orc.Oracle()
    o.set_threads(cores)
    rows = 8 * cores

    def run(a, b, c0):
        t = time.perf_counter()
        o.matmul2d(a, orc.X_NOTRANS, b, orc.X_NOTRANS, ALPHA, BETA, c0)
        return time.perf_counter() - t
    return ("port", cores, "first %d of 8192 rows, C restatement of the built-in loops, %d threads" % (rows, cores),
            rows, run)


def time_cpu(steps, warmup):
    kind, cores, sample, rows, run = cpu_reference_runner()
    a, b, c0 = host_operands(rows)
    for _ in range(warmup):
        run(a, b, c0)
    times = [run(a, b, c0) for _ in range(steps)]
    flops = 2.0 * rows * N_DIM * N_DIM
    tflops = flops / (sum(times) / len(times)) / 1e12
    return {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": kind, "sample": sample,
            "ms_per_step": 1e3 * sum(times) / len(times)}


def main_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    steps = max(1, min(args.steps, 5))
    warm = max(1, min(args.warmup, 1))
    r = time_cpu(steps, warm)
    line = {"impl": "reference", "metric": "MatrixMul TFLOP/s", "value": r["value"], "unit": "TFLOP/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": warm, "ms_per_step": r["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic", "config": {"workload": WORKLOAD, "device": "host CPU"},
            "cpu_baseline": {"value": r["value"], "unit": "TFLOP/s", "cores": r["cores"], "kind": r["kind"],
                             "sample": r["sample"]},
            "e2e": {"value": r["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)
    return 0


# ------------------------------------------------------------------ GPU arm

def main_ours(args):
    import torch
    import torch.distributed as dist
    from niutensor_b200 import capi, ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the MatrixMul path has no CPU implementation")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    L = capi.lib()

    # rank r owns column block r of B, C0 and C; A is replicated
    g = torch.Generator(device=dev)
    g.manual_seed(1005)
    a = (torch.rand(N_DIM, N_DIM, device=dev, generator=g) * 2 - 1).half()
    g.manual_seed(2005 + rank)
    b = (torch.rand(N_DIM, N_DIM, device=dev, generator=g) * 2 - 1).half()
    c0 = torch.randn(N_DIM, N_DIM, device=dev, generator=g).half()
    c = c0.clone()

    def step():
        ops._MatrixMul(a, capi.X_NOTRANS, b, capi.X_NOTRANS, c, ALPHA, BETA)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    c.copy_(c0)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.15)
    barrier()
    launches0 = L.ntb_launch_count()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    w0 = time.time()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    w1 = time.time()
    launches = L.ntb_launch_count() - launches0
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    total_ms = float(ms.item())
    clocks = sampler.stop(w0, w1) if rank == 0 else None
    status = L.ntb_device_status(local)
    if status != capi.OK:
        raise SystemExit("bench.py: device status %d after the timed region" % status)

    ms_per_step = total_ms / args.steps
    tflops = FLOPS_PER_RANK * world / (ms_per_step * 1e-3) / 1e12
    per_gpu_tflops = tflops / world

    # optional: what a caller who wants the whole C on every rank pays on top (not in `value`)
    gather_ms = None
    if world > 1:
        from niutensor_b200 import shard
        shard.gather_columns(c, N_DIM * world)
        barrier()
        e0.record()
        for _ in range(3):
            shard.gather_columns(c, N_DIM * world)
        e1.record()
        barrier()
        g = torch.tensor([e0.elapsed_time(e1) / 3], device=dev, dtype=torch.float64)
        dist.all_reduce(g, op=dist.ReduceOp.MAX)
        gather_ms = float(g.item())

    # optional: the same gather done by the product's own epilogue (peer stores), for comparison
    fused = None
    if world > 1 and args.fused_gather:
        try:
            from niutensor_b200 import ops as nops
            c_sym, peers = shard.symmetric_matrix(N_DIM, N_DIM * world, torch.float16, dev)
            c_sym.zero_()
            plist = [peers[r] for r in sorted(peers)]
            torch.cuda.synchronize()
            barrier()

            def fused_step():
                nops.MatrixMul2DToPeers(a, capi.X_NOTRANS, b, capi.X_NOTRANS, c_sym, rank * N_DIM, plist, ALPHA, 0.0)

            fused_step()
            barrier()
            e0.record()
            for _ in range(3):
                fused_step()
            e1.record()
            barrier()
            g = torch.tensor([e0.elapsed_time(e1) / 3], device=dev, dtype=torch.float64)
            dist.all_reduce(g, op=dist.ReduceOp.MAX)
            fused = {"ms": float(g.item()),
                     "note": "product (beta = 0) whose epilogue stores its column block into every rank's C; "
                             "compare with ms_per_step + allgather_of_c.ms"}
        except Exception as exc:              # an extra must never sink the benchmark line
            fused = {"ms": None, "note": "failed: %r" % (exc,)}

    if args.kernel_only:
        if rank == 0:
            print(json.dumps({"metric": "MatrixMul TFLOP/s", "value": tflops, "unit": "TFLOP/s",
                              "n_gpus": world, "steps": args.steps, "ms_per_step": ms_per_step,
                              "gpu_launches": int(launches), "kernel_only": True}), flush=True)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return 0

    # end to end: host buffers through the C ABI, copies inside the timed region
    ha = a.cpu().pin_memory()
    hb = b.cpu().pin_memory()
    hc = c0.cpu().pin_memory()
    e2e_steps = max(1, min(args.steps, 5))
    code = capi.X_FLOAT16

    def host_step():
        rc = L.ntb_gemm_host(local, None, ha.data_ptr(), capi.X_NOTRANS, hb.data_ptr(), capi.X_NOTRANS,
                             hc.data_ptr(), code, code, N_DIM, N_DIM, N_DIM, N_DIM, N_DIM, N_DIM,
                             0, 0, 0, 1, ALPHA, BETA)
        if rc != capi.OK:
            raise SystemExit("ntb_gemm_host: " + capi.strerror(rc))

    host_step()
    barrier()
    e0.record()
    for _ in range(e2e_steps):
        host_step()
    e1.record()
    barrier()
    ms2 = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms2, op=dist.ReduceOp.MAX)
    e2e_tflops = FLOPS_PER_RANK * world / (float(ms2.item()) / e2e_steps * 1e-3) / 1e12
    mat_bytes = N_DIM * N_DIM * 2

    if rank == 0:
        peaks = load_peaks()
        # a run of back-to-back launches shorter than a second is a burst measurement
        which = "burst" if total_ms < 1000.0 else "sustained"
        peak = peaks[which]
        line = {
            "metric": "MatrixMul TFLOP/s", "value": tflops, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "M": N_DIM, "N_per_gpu": N_DIM, "K": N_DIM,
                       "l2": "operands (537 MB per GPU) exceed the 126 MB L2; no flush between steps",
                       "parallelism": "column shards of B and C, no collective"},
            "roofline": {"bound": "tensor", "achieved": per_gpu_tflops, "peak": peak, "unit": "TFLOP/s",
                         "frac": per_gpu_tflops / peak,
                         "peak_source": "%s cuBLAS bf16 figure of MEASURED_PEAKS.json (%s)" % (which, peaks["source"]),
                         "frac_of_nominal_2250": per_gpu_tflops / 2250.0,
                         "algorithmic_gb_per_s": BYTES_PER_RANK / (ms_per_step * 1e-3) / 1e9,
                         "traffic": NCU_TRAFFIC_BYTES},
            "e2e": {"value": e2e_tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 3 * mat_bytes * world,
                    "d2h_bytes_per_step": mat_bytes * world, "steps": e2e_steps},
            "gpu_launches": int(launches),
            "clocks": clocks,
        }
        if gather_ms is not None:
            line["allgather_of_c"] = {"ms": gather_ms, "bytes_received_per_gpu": (world - 1) * mat_bytes,
                                      "gb_per_s_per_gpu": (world - 1) * mat_bytes / (gather_ms * 1e-3) / 1e9,
                                      "note": "NCCL all_gather + local re-interleave; only for callers that "
                                              "need the full C on every rank; not part of value"}
        if fused is not None:
            line["fused_gather_of_c"] = fused
        if world == 1:
            try:
                line["cpu_baseline"] = {k: v for k, v in time_cpu(2, 1).items() if k != "ms_per_step"}
            except Exception as exc:          # the baseline must never sink the GPU number
                line["cpu_baseline"] = {"value": None, "unit": "TFLOP/s", "cores": 0, "kind": "port",
                                        "sample": "failed: %r" % (exc,)}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--fused-gather", action="store_true",
                    help="N > 1: also time the product whose epilogue writes its block of C to every rank (symmetric memory)")
    ap.add_argument("--kernel-only", action="store_true",
                    help="skip the end-to-end and CPU-baseline legs (short runs under a profiler)")
    args = ap.parse_args()
    if args.steps < 1:
        args.steps = 1
    if args.impl == "reference":
        return main_reference(args)
    return main_ours(args)


if __name__ == "__main__":
    sys.exit(main())
