#!/usr/bin/env python
"""Benchmark of the MatrixMul hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (`config.workload`): the large square product of the benchmark list,
C = 1.0 * A * B + 0.5 * C0 with A, B 8192 x 8192 ~ U[-1, 1] and C0 ~ N(0, 1), fp16 tensors,
no transposition -- ONE product of fixed size at every N ("strong" scaling). With N ranks it
is N-sharded: A is replicated, rank r owns columns [r * 8192 / N, (r + 1) * 8192 / N) of B,
C0 and C, and the whole C is gathered onto every rank inside the timed region: the
epilogue of each rank's product writes its tiles into every rank's copy of C over NVLink
(symmetric memory): with one multicast store per 128-byte line where an NVLink multicast
object can be bound (`ntb_gemm_multicast`), else, or with `--gather peers`, with one TMA store
per peer and box (`ntb_gemm_peers`). One step = that product; `value` = 2 * 8192^3 flop
divided by the time until every rank holds the whole C. Beside it the line reports
`sharded_only` (C left distributed, no exchange) and `gather` (what the exchange costs, and
the NCCL all-gather + re-interleave kernel as the comparison). Inputs are seeded synthetic
data of the stated distributions.

One JSON line on stdout (rank 0). `value` is TFLOP/s with operands resident in HBM; `e2e` is
the same metric from pinned host buffers, host-to-device and device-to-host copies inside
the timed region: at N = 1 through the host-buffer entry point of the C ABI
(`ntb_gemm_host`, column chunks whose copies overlap the products); at N > 1 rank r copies its
rows of A and its column shards of B and C0 in, an NCCL all-gather over NVLink replicates A
on the devices, `ntb_gemm` multiplies, the shard of C goes back -- every input crosses PCIe
once per job. `roofline_sustained` repeats the headline
step back to back for at least two seconds (clock samples taken meanwhile) against the
sustained peak; `configs` times the other benchmark configurations in the same process,
each beside cuBLAS (torch.matmul) on the same operands.

`--impl reference` times the reference's own CPU MatrixMul (the NiuTensor library built
into oracle/_ref by `make -C oracle ref`: OpenBLAS build with every host thread if
present, else its built-in single-thread loops on a row sample; if neither exists, the
plain-C restatement) on operands of the same shapes and distributions drawn from a host
generator, fp16 values carried in fp32 because the reference has no CPU half arithmetic.
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
WORKLOAD = ("MatrixMul fp16 8192x8192x8192 N/N alpha=1 beta=0.5 (benchmark config 5), one product "
            "column-sharded over n_gpus, whole C gathered on every rank")
FLOPS_TOTAL = 2.0 * N_DIM * N_DIM * N_DIM
MAT_BYTES = N_DIM * N_DIM * 2
# DRAM traffic of one full 8192^3 launch measured by ncu (dram__bytes_read.sum +
# dram__bytes_write.sum) on the CTA-pair kernel with 512 x 256 tiles
NCU_TRAFFIC_BYTES = 1.106e9


def config_dict(world):
    return {"workload": WORKLOAD, "M": N_DIM, "N": N_DIM, "K": N_DIM, "N_per_gpu": N_DIM // max(1, world),
            "l2": "operands (537 MB at N=1) exceed the 126 MB L2; no flush between steps",
            "parallelism": "column shards of B and C; all-gather of C by stores from the epilogue (see gather.method)"
                           if world > 1 else "one GPU"}


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
              "clocks_event_reasons.sw_power_cap,power.draw")

    def __init__(self, index, period_ms=25):
        self.index = index
        self.period_ms = period_ms
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                 "--format=csv,noheader,nounits", "-lms", str(self.period_ms)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def window(self, t0, t1):
        """Summary of the samples taken between the wall-clock times t0 and t1."""
        inside = [l for (t, l) in self.lines if t0 <= t <= t1 + 0.03]
        note = None
        if not inside:
            inside = [l for (_, l) in self.lines]
            note = "no sample fell inside the region; all samples of the run used"
        sm, mx, pw, reasons = [], [], [], set()
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
            try:
                pw.append(float(parts[6]))
            except (IndexError, ValueError):
                pass
        out = {"sm_mhz": float(np.median(sm)) if sm else None,
               "sm_max_mhz": float(max(mx)) if mx else None,
               "reasons": sorted(reasons), "samples": len(sm),
               "power_w_max": max(pw) if pw else None}
        if note:
            out["note"] = note
        return out

    def stop(self):
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()


def pin_to_gpu_numa(index):
    """Binds this process to the CPUs of the NUMA node its GPU hangs off, so that the pinned
    host buffers of the end-to-end leg (first touched afterwards) are local to the GPU's PCIe
    root. Returns the node, or None when the topology cannot be read."""
    try:
        import torch
        p = torch.cuda.get_device_properties(index)
        bdf = "%04x:%02x:%02x.0" % (p.pci_domain_id, p.pci_bus_id, p.pci_device_id)
        with open("/sys/bus/pci/devices/%s/numa_node" % bdf) as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open("/sys/devices/system/node/node%d/cpulist" % node) as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if allowed:
            os.sched_setaffinity(0, allowed)
            return node
    except Exception:
        pass
    return None


# ------------------------------------------------------------------ CPU reference arm

def host_operands(rows=N_DIM):
    """Operands as fp16-valued float32 host arrays (A and C0 cut to `rows` rows)."""
    rng = np.random.default_rng(1005)
    a = rng.uniform(-1, 1, (rows, N_DIM)).astype(np.float16).astype(np.float32)
    b = rng.uniform(-1, 1, (N_DIM, N_DIM)).astype(np.float16).astype(np.float32)
    c0 = rng.normal(size=(rows, N_DIM)).astype(np.float16).astype(np.float32)
    return a, b, c0


def cpu_reference_runner():
    """Returns (kind, cores, description, default rows of A per step, callable(a, b, c0) -> seconds)."""
    from oracle import oracle as orc          # checker / CPU baseline only
    cores = os.cpu_count() or 1
    if orc.ref_available("openblas"):
        try:
            ref = orc.Reference("openblas")
            ref.set_threads(cores)

            def run(a, b, c0):
                t = time.perf_counter()
                ref.run(ref.FORM_GENERAL, a, orc.X_NOTRANS, b, orc.X_NOTRANS, ALPHA, BETA, c0, inplace=True)
                return time.perf_counter() - t
            return ("reference", cores, "reference built with USE_BLAS on OpenBLAS, %d threads, fp16 values in fp32" % cores,
                    N_DIM, run)
        except OSError:
            pass
    if orc.ref_available("builtin"):
        ref = orc.Reference("builtin")

        def run(a, b, c0):
            t = time.perf_counter()
            ref.run(ref.FORM_GENERAL, a, orc.X_NOTRANS, b, orc.X_NOTRANS, ALPHA, BETA, c0, inplace=True)
            return time.perf_counter() - t
        return ("reference", 1, "reference built-in loops, 1 thread", 64, run)
    o = orc.Oracle()
    o.set_threads(cores)

    def run(a, b, c0):
        t = time.perf_counter()
        o.matmul2d(a, orc.X_NOTRANS, b, orc.X_NOTRANS, ALPHA, BETA, c0)
        return time.perf_counter() - t
    return ("port", cores, "C restatement of the built-in loops, %d threads" % cores, 8 * cores, run)


def time_cpu(steps, warmup, budget_s=150.0):
    """Times `steps` steps after `warmup`; a step multiplies the first `rows` rows of A by
    the whole B. `rows` starts at the implementation's default and is cut so that the whole
    run fits the time budget."""
    kind, cores, what, rows, run = cpu_reference_runner()
    a, b, c0 = host_operands(rows)
    first = run(a, b, c0)
    total = (steps + warmup) * first
    if total > budget_s and rows > 256:
        rows = max(256, int(rows * budget_s / total) // 256 * 256)
        a, c0 = a[:rows].copy(), c0[:rows].copy()
    for _ in range(max(0, warmup - 1)):
        run(a, b, c0)
    times = [run(a, b, c0) for _ in range(steps)]
    flops = 2.0 * rows * N_DIM * N_DIM
    tflops = flops / (sum(times) / len(times)) / 1e12
    sample = ("whole 8192^3 product" if rows == N_DIM else "first %d of 8192 rows (%dx8192x8192)" % (rows, rows)) + ", " + what
    return {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": kind, "sample": sample,
            "ms_per_step": 1e3 * sum(times) / len(times)}


def main_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    steps, warm = max(1, args.steps), max(1, args.warmup)
    r = time_cpu(steps, warm)
    cfg = config_dict(world)                        # the same dictionary as the GPU arm prints
    line = {"impl": "reference", "device": "host CPU", "metric": "MatrixMul TFLOP/s", "value": r["value"], "unit": "TFLOP/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": warm, "ms_per_step": r["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic", "config": cfg,
            "cpu_baseline": {"value": r["value"], "unit": "TFLOP/s", "cores": r["cores"], "kind": r["kind"],
                             "sample": r["sample"]},
            "e2e": {"value": r["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)
    return 0


# ------------------------------------------------------------------ GPU arm

def main_ours(args):
    import torch
    import torch.distributed as dist
    from niutensor_b200 import capi, ops, shard

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the MatrixMul path has no CPU implementation")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    numa = pin_to_gpu_numa(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    L = capi.lib()
    warmup = max(3, args.warmup)

    # rank r owns columns [lo, hi) of B, C0 and C; A is replicated
    lo, hi = shard.column_shard(N_DIM, world, rank)
    w = hi - lo
    g = torch.Generator(device=dev)
    g.manual_seed(1005)
    a = (torch.rand(N_DIM, N_DIM, device=dev, generator=g) * 2 - 1).half()
    b_full = (torch.rand(N_DIM, N_DIM, device=dev, generator=g) * 2 - 1).half()
    c0_full = torch.randn(N_DIM, N_DIM, device=dev, generator=g).half()
    b = b_full[:, lo:hi].contiguous()
    c0 = c0_full[:, lo:hi].contiguous()
    del b_full, c0_full
    c_local = c0.clone()                              # packed shard of C ("sharded_only")

    if world > 1:
        # every rank's whole C in symmetric memory; this rank writes its block of each
        want_mc = args.gather != "peers"
        c_all, peers, mc = shard.symmetric_matrix(N_DIM, N_DIM, torch.float16, dev, multicast=want_mc) if want_mc \
            else shard.symmetric_matrix(N_DIM, N_DIM, torch.float16, dev) + (0,)
        # every rank must take the same path
        flag = torch.tensor([1 if mc else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        use_mc = bool(flag.item())
        c_all.zero_()
        c_all[:, lo:hi] = c0
        plist = [peers[r] for r in sorted(peers)]

        def step_peers():
            ops.MatrixMul2DToPeers(a, capi.X_NOTRANS, b, capi.X_NOTRANS, c_all, lo, plist, ALPHA, BETA)

        def step_mc():
            ops.MatrixMul2DToMulticast(a, capi.X_NOTRANS, b, capi.X_NOTRANS, c_all, lo, mc, ALPHA, BETA)

        step = step_mc if use_mc else step_peers
    else:
        def step():
            ops._MatrixMul(a, capi.X_NOTRANS, b, capi.X_NOTRANS, c_local, ALPHA, BETA)

    def step_sharded_only():
        ops._MatrixMul(a, capi.X_NOTRANS, b, capi.X_NOTRANS, c_local, ALPHA, BETA)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)

    def timed(fn, steps):
        """ms per step, max over ranks, of `steps` back-to-back calls between two barriers;
        also wall-clock start and end of the region (for the clock samples)."""
        barrier()
        w0 = time.time()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        w1 = time.time()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()) / steps, w0, w1

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.2)

    # ---- headline: K steps of the (sharded, gathered) product
    for _ in range(warmup):
        step()
    barrier()
    launches0 = L.ntb_launch_count()
    ms_per_step, w0, w1 = timed(step, args.steps)
    launches = L.ntb_launch_count() - launches0
    clocks = sampler.window(w0, w1) if rank == 0 else None
    status = L.ntb_device_status(local)
    if status != capi.OK:
        raise SystemExit("bench.py: device status %d after the timed region" % status)
    tflops = FLOPS_TOTAL / (ms_per_step * 1e-3) / 1e12
    total_ms = ms_per_step * args.steps

    if args.kernel_only:
        if rank == 0:
            sampler.stop()
            print(json.dumps({"metric": "MatrixMul TFLOP/s", "value": tflops, "unit": "TFLOP/s",
                              "n_gpus": world, "steps": args.steps, "ms_per_step": ms_per_step,
                              "gpu_launches": int(launches), "kernel_only": True}), flush=True)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return 0

    # ---- the same step back to back for at least two seconds: the sustained rate
    sus_steps = max(args.steps, int(2200.0 / ms_per_step) + 1)
    sus_ms, s0, s1 = timed(step, sus_steps)
    sus_clocks = sampler.window(s0, s1) if rank == 0 else None
    sus_tflops = FLOPS_TOTAL / (sus_ms * 1e-3) / 1e12

    # ---- N > 1: what the exchange costs
    sharded = gather = None
    sub_steps = max(5, min(args.steps, 20))
    if world > 1:
        for _ in range(3):
            step_sharded_only()
        so_ms, _, _ = timed(step_sharded_only, sub_steps)
        sharded = {"ms_per_step": so_ms, "value": FLOPS_TOTAL / (so_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                   "note": "every rank computes its column block into a packed local buffer; C stays distributed, no exchange"}

        def step_nccl():
            step_sharded_only()
            shard.gather_columns(c_local, N_DIM)

        def gather_only():
            shard.gather_columns(c_local, N_DIM)

        for _ in range(3):
            step_nccl()
        nccl_step_ms, _, _ = timed(step_nccl, sub_steps)
        nccl_gather_ms, _, _ = timed(gather_only, sub_steps)
        peers_ms = None
        if use_mc:
            for _ in range(3):
                step_peers()
            peers_ms, _, _ = timed(step_peers, sub_steps)
        recv = (world - 1) * N_DIM * w * 2
        gather = {"method": ("multimem.st to the NVLink multicast address of C: each block leaves its GPU once, "
                             "the switch replicates it" if use_mc else
                             "TMA stores of every finished box to each peer's C: each block leaves its GPU n_gpus - 1 times"),
                  "bytes_sent_per_gpu": N_DIM * w * 2 * (1 if use_mc else world - 1),
                  "peer_stores_ms_per_step": peers_ms,
                  "bytes_received_per_gpu": recv,
                  "fused_ms_per_step": ms_per_step,
                  "fused_extra_ms": ms_per_step - so_ms,
                  "fused_gb_per_s_per_gpu": recv / (ms_per_step * 1e-3) / 1e9,
                  "nvlink_gb_per_s_per_direction": {"nominal": 900.0, "measured_peer_copy": 770.0},
                  "floor_ms_at_900": recv / 900e9 * 1e3,
                  "nccl_all_gather_ms": nccl_gather_ms,
                  "nccl_gb_per_s_per_gpu": recv / (nccl_gather_ms * 1e-3) / 1e9,
                  "product_then_nccl_ms_per_step": nccl_step_ms,
                  "limited_by": (("NVLink ingress of the replicated blocks" if use_mc else
                                  "NVLink egress of the epilogue's peer stores") if ms_per_step > 1.15 * so_ms
                                 else "the product itself"),
                  "note": "fused = product whose epilogue stores its block into every rank's C (value); nccl = "
                          "all_gather_into_tensor of the packed shards + one re-interleave kernel, after the product"}

    # ---- end to end: host buffers through the C ABI, copies inside the timed region
    ha = a.cpu().pin_memory()
    hb = b.cpu().pin_memory()
    hc = c0.cpu().pin_memory()
    e2e_steps = max(1, min(args.steps, 5))
    code = capi.X_FLOAT16

    def host_step():
        rc = L.ntb_gemm_host(local, None, ha.data_ptr(), capi.X_NOTRANS, hb.data_ptr(), capi.X_NOTRANS,
                             hc.data_ptr(), code, code, N_DIM, N_DIM, N_DIM, w, N_DIM, w,
                             0, 0, 0, 1, ALPHA, BETA)
        if rc != capi.OK:
            raise SystemExit("ntb_gemm_host: " + capi.strerror(rc))

    e2e_note = "one GPU: a, b and C0 in, C out, in column chunks whose copies overlap the products"
    h2d_bytes = 3 * MAT_BYTES
    if world > 1 and N_DIM % world == 0:
        # N ranks: the host's A crosses PCIe once per job, not once per rank. Rank r copies rows
        # [r M/N, (r+1) M/N) of A in, an NCCL all-gather over NVLink replicates them on the
        # devices, then B and C0 shards in, the product, the C shard out.
        rows = N_DIM // world
        a_dev = torch.empty(N_DIM, N_DIM, device=dev, dtype=torch.float16)
        ha_rows = ha[rank * rows:(rank + 1) * rows]

        def host_step():
            mine = a_dev[rank * rows:(rank + 1) * rows]
            mine.copy_(ha_rows, non_blocking=True)
            dist.all_gather_into_tensor(a_dev, mine)
            rc = L.ntb_gemm_host_resident_a(local, ops._stream(a_dev), a_dev.data_ptr(), capi.X_NOTRANS, hb.data_ptr(),
                                            capi.X_NOTRANS, hc.data_ptr(), code, code, N_DIM, N_DIM, N_DIM, w, N_DIM, w,
                                            0, 0, 0, 1, ALPHA, BETA)
            if rc != capi.OK:
                raise SystemExit("ntb_gemm_host_resident_a: " + capi.strerror(rc))

        host_step()
        # the very product from the resident operands (column chunks may take another kernel
        # than the whole shard, hence a bound and not equality)
        check = c0.clone()
        ops._MatrixMul2D(a, capi.X_NOTRANS, b, capi.X_NOTRANS, check, ALPHA, BETA)
        got = hc.to(dev).float()
        if float((got - check.float()).norm() / check.float().norm()) > 1e-3:
            raise SystemExit("bench.py: end-to-end product differs from the resident one")
        del check, got
        e2e_note = ("rank r copies rows r of A in, an NCCL all-gather over NVLink replicates A on the devices; "
                    "then its column shards of B and C0 in, its shard of C out: A, B, C0 cross PCIe once per job")
    else:
        h2d_bytes = world * MAT_BYTES + 2 * MAT_BYTES
        host_step()
    e2e_ms, _, _ = timed(host_step, e2e_steps)
    e2e_tflops = FLOPS_TOTAL / (e2e_ms * 1e-3) / 1e12
    del ha, hb, hc

    # ---- the other benchmark configurations, each beside cuBLAS on the same operands
    configs = None
    if not args.no_configs:
        try:
            from niutensor_b200 import bench_configs
            del c_local
            torch.cuda.empty_cache()
            if world == 1:
                configs = bench_configs.driver_table(dev)
            else:
                configs = bench_configs.sharded_table(dev, world, rank, timed)
        except Exception as exc:                  # an extra must never sink the benchmark line
            configs = {"failed": repr(exc)}

    if rank == 0:
        sampler.stop()
        peaks = load_peaks()
        # a run of back-to-back launches shorter than a second is a burst measurement
        which = "burst" if total_ms < 1000.0 else "sustained"
        peak = peaks[which]
        per_gpu = tflops / world
        line = {
            "metric": "MatrixMul TFLOP/s", "value": tflops, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic", "config": config_dict(world),
            "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": peak, "unit": "TFLOP/s",
                         "frac": per_gpu / peak,
                         "peak_source": "%s cuBLAS bf16 figure of MEASURED_PEAKS.json (%s)" % (which, peaks["source"]),
                         "frac_of_nominal_2250": per_gpu / 2250.0,
                         "algorithmic_gb_per_s": (MAT_BYTES * (1 + 3.0 / world)) / (ms_per_step * 1e-3) / 1e9,
                         "traffic": NCU_TRAFFIC_BYTES if world == 1 else None},
            "roofline_sustained": {"bound": "tensor", "achieved": sus_tflops / world, "peak": peaks["sustained"],
                                   "unit": "TFLOP/s", "frac": sus_tflops / world / peaks["sustained"],
                                   "steps": sus_steps, "seconds": sus_ms * sus_steps * 1e-3, "ms_per_step": sus_ms,
                                   "clocks": sus_clocks},
            "e2e": {"value": e2e_tflops, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": MAT_BYTES,
                    "steps": e2e_steps, "numa_node_of_rank0": numa, "note": e2e_note},
            "gpu_launches": int(launches),
            "clocks": clocks,
        }
        if sharded is not None:
            line["sharded_only"] = sharded
            line["gather"] = gather
        if configs is not None:
            line["configs"] = configs
        if world == 1:
            try:
                line["cpu_baseline"] = {k: v for k, v in time_cpu(2, 1, budget_s=20.0).items() if k != "ms_per_step"}
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
    ap.add_argument("--gather", default="auto", choices=["auto", "peers"],
                    help="N > 1: auto = through the NVLink multicast object where there is one, else stores to each peer")
    ap.add_argument("--no-configs", action="store_true", help="skip the table of the other benchmark configurations")
    ap.add_argument("--kernel-only", action="store_true",
                    help="only the headline region (short runs under a profiler)")
    args = ap.parse_args()
    if args.steps < 1:
        args.steps = 1
    if args.impl == "reference":
        return main_reference(args)
    return main_ours(args)


if __name__ == "__main__":
    sys.exit(main())
