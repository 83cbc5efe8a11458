#!/usr/bin/env python
"""Benchmark of the quantized-contraction hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload decode] [--impl reference]

Prints ONE JSON line (rank 0).  Workloads (seeded synthetic inputs with the
shapes and value distributions of the benchmark configurations):

  decode   W4A16 decode GEMV, M=1: one step = the up projection
           [1,4096]x[4096,14336] and the down projection [1,14336]x[14336,4096];
           metric = weight GB/s (algorithmic bytes / time).  HBM-bound.

`value` is measured with inputs resident in HBM, the K timed steps captured in one
CUDA graph (the kernels are microseconds long; eager launches would measure the
host), weights rotated through more copies than fit in L2 so every pass reads
HBM.  `e2e` is the same metric through `artifact.run` with the step's
activations in pinned host memory (H2D + D2H inside the timed region).  The
weights are model state and stay resident in both.

`--impl reference` times the CPU implementation of the same path (the torch-CPU
restatement of the reference's own CPU code, all host threads) on the same
configuration, on rank 0 only.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

L2_BYTES = 126 * 1024 * 1024
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0

# DRAM traffic per launch of the dominant kernel from an ncu capture
# (dram__bytes_read.sum + dram__bytes_write.sum); see profiles/.  None = not captured yet.
NCU_TRAFFIC_BYTES = {"decode": None}


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]),
                "bf16_tflops_sustained": float(data.get("bf16_tflops_sustained", data["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": FALLBACK_BF16_TFLOPS,
            "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while a region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index = index
        self.process = None
        self.lines: list[str] = []
        self.thread = None

    def start(self) -> None:
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.process = None
            return

        def pump():
            for line in self.process.stdout:
                self.lines.append(line.strip())

        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self) -> dict:
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.process.terminate()
        try:
            self.process.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
        if self.thread is not None:
            self.thread.join(timeout=2)
        clocks, max_clock, power, reasons = [], None, [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            fields = [f.strip() for f in line.split(",")]
            if len(fields) < 7:
                continue
            try:
                clocks.append(float(fields[0]))
                max_clock = float(fields[1])
                power.append(float(fields[2]))
            except ValueError:
                continue
            for name, field in zip(names, fields[3:7]):
                if field.lower().startswith("active"):
                    reasons.add(name)
        # "under load" = the upper half of the power samples
        if clocks:
            threshold = statistics.median(power)
            loaded = [c for c, p in zip(clocks, power) if p >= threshold] or clocks
            median = statistics.median(loaded)
        else:
            median = None
        return {"sm_mhz": median, "sm_max_mhz": max_clock, "reasons": sorted(reasons),
                "samples": len(clocks), "power_w_max": max(power) if power else None}


# ---------------------------------------------------------------------------------------
# decode workload
# ---------------------------------------------------------------------------------------
DECODE_SHAPES = ((4096, 14336), (14336, 4096))      # (K, N): up projection, down projection
GROUP = 128


def decode_bytes(M: int) -> int:
    """Algorithmic bytes of one step (both projections): packed weights + scales + X + Y."""
    total = 0
    for K, N in DECODE_SHAPES:
        total += K * N // 2 + (K // GROUP) * N * 2 + M * K * 2 + M * N * 2
    return total


def decode_inputs(M: int, seed: int = 0):
    import torch

    from intent_b200 import workloads

    return [workloads.w4a16_inputs(M, K, N, dtype=torch.float16, group_size=GROUP, seed=seed + i)
            for i, (K, N) in enumerate(DECODE_SHAPES)]


def run_decode(args, rank: int, world: int, device):
    import torch

    import intent_b200 as ib
    from intent_b200.runtime import native

    M = args.batch
    artifact = ib.compile(ib.programs.weight_only_int4_matmul, target=ib.B200Target(device.index),
                          constexprs={"GROUP_SIZE": GROUP, "ZERO_POINT": 8, "ACT_DTYPE": "f16"})
    host = decode_inputs(M)
    step_bytes = decode_bytes(M)
    weight_bytes = sum(p.numel() * 4 + s.numel() * 2 for _, p, s in host)
    copies = max(2, -(-2 * L2_BYTES // weight_bytes) + 1)          # rotate through > 2x L2 of weights
    sets = []
    for c in range(copies):
        sets.append([(x.to(device), p.to(device), s.to(device))
                     for x, p, s in host])
    calls = [[artifact.prepare(x, p, s) for x, p, s in group] for group in sets]

    def step(i: int) -> None:
        for call in calls[i % copies]:
            call.launch()

    for i in range(max(args.warmup, 3)):
        step(i)
    torch.cuda.synchronize()

    # capture exactly K steps in one graph
    stream = torch.cuda.Stream(device)
    stream.wait_stream(torch.cuda.current_stream())
    before = native.launch_count()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        for i in range(args.steps):
            step(i)
    launches = native.launch_count() - before
    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            graph.replay()
    stream.synchronize()

    sampler = ClockSampler(device.index)
    if rank == 0:
        sampler.start()
    # keep the GPU under the same load for a moment so the clock samples mean something
    with torch.cuda.stream(stream):
        spin_until = time.perf_counter() + args.load_seconds
        while time.perf_counter() < spin_until:
            graph.replay()
            stream.synchronize()
    barrier(world)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        start.record(stream)
        graph.replay()
        stop.record(stream)
    stream.synchronize()
    torch.cuda.synchronize()
    barrier(world)
    elapsed_ms = start.elapsed_time(stop)
    clocks = sampler.stop() if rank == 0 else None
    elapsed_ms = reduce_max(elapsed_ms, world, device)

    # ---- end to end: host activations, artifact.run, result read back ----------------
    pinned_in = [x.pin_memory() for x, _, _ in host]
    pinned_out = [torch.empty((M, N), dtype=torch.float16).pin_memory() for _, N in DECODE_SHAPES]

    def e2e_step(i: int) -> None:
        group = sets[i % copies]
        for j in range(len(DECODE_SHAPES)):
            xd = pinned_in[j].to(device, non_blocking=True)
            y = artifact.run(xd, group[j][1], group[j][2])
            pinned_out[j].copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for i in range(max(args.warmup, 3)):
        e2e_step(i)
    barrier(world)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(args.steps):
        e2e_step(i)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    e2e_s = reduce_max(e2e_s, world, device)

    ms_per_step = elapsed_ms / args.steps
    value = world * step_bytes / (ms_per_step * 1e-3) / 1e9
    peaks = measured_peaks()
    per_launch_bytes = step_bytes / len(DECODE_SHAPES)
    per_launch_s = elapsed_ms * 1e-3 / max(1, launches)
    achieved = per_launch_bytes / per_launch_s / 1e9
    line = {
        "metric": "w4a16_decode_weight_GBps", "value": round(value, 2), "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms_per_step, 6), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"w4a16_decode_gemv M={M} [4096->14336]+[14336->4096] g128 zp8 (configs[1])",
                   "batch": M, "group_size": GROUP, "step": "up+down projection, 2 kernel launches",
                   "l2": f"weights rotated through {copies} resident copies ({copies * weight_bytes >> 20} MiB > L2)",
                   "timing": "K steps in one CUDA graph, CUDA events on the replay stream",
                   "parallelism": "replicas only" if world > 1 else "1 gpu"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4), "traffic": NCU_TRAFFIC_BYTES["decode"],
                     "peak_source": peaks["source"], "algorithmic_bytes_per_launch": per_launch_bytes,
                     "kernel": "w4a16_skinny_kernel", "us_per_launch": round(per_launch_s * 1e6, 3)},
        "e2e": {"value": round(world * step_bytes / (e2e_s / args.steps) / 1e9, 2), "unit": "GB/s",
                "h2d_bytes_per_step": sum(x.numel() * 2 for x in pinned_in),
                "d2h_bytes_per_step": sum(y.numel() * 2 for y in pinned_out),
                "ms_per_step": round(e2e_s / args.steps * 1e3, 6)},
        "gpu_launches": int(launches),
        "clocks": clocks,
    }
    return line


# ---------------------------------------------------------------------------------------
# CPU arm (reference implementation of the path on the host cores)
# ---------------------------------------------------------------------------------------
def cpu_decode(M: int, steps: int, warmup: int, budget_s: float):
    """Time the torch-CPU implementation of the decode step.  Returns
    (GB/s, cores, sample description, ms per step)."""
    import torch

    import oracle

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    host = decode_inputs(M)

    def step(fraction_columns: int) -> None:
        for x, p, s in host:
            n = p.shape[1] // fraction_columns
            oracle.weight_only_int4_matmul(x, p[:, :n].contiguous(), s[:, :n].contiguous(),
                                           group_size=GROUP, zero_point=8)

    divisor = 8
    t0 = time.perf_counter()
    step(divisor)
    probe = time.perf_counter() - t0
    full_estimate = probe * divisor
    divisor = 1
    while full_estimate / divisor * (steps + warmup) > budget_s and divisor < 64:
        divisor *= 2
    for _ in range(warmup):
        step(divisor)
    t0 = time.perf_counter()
    for _ in range(steps):
        step(divisor)
    seconds = (time.perf_counter() - t0) / steps
    step_bytes = decode_bytes(M) / divisor
    sample = (f"{steps} steps of the decode step on the first 1/{divisor} of the output columns "
              f"(M={M}, both projections), torch CPU, {cores} threads")
    return step_bytes / seconds / 1e9, cores, sample, seconds * 1e3


def run_reference(args, rank: int, world: int):
    if rank != 0:
        return None
    value, cores, sample, ms = cpu_decode(args.batch, args.steps, max(args.warmup, 1), budget_s=150.0)
    return {
        "impl": "reference", "metric": "w4a16_decode_weight_GBps", "value": round(value, 4), "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 1), "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"w4a16_decode_gemv M={args.batch} [4096->14336]+[14336->4096] g128 zp8 (configs[1])",
                   "batch": args.batch, "group_size": GROUP},
        "cpu_baseline": {"value": round(value, 4), "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": round(value, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


# ---------------------------------------------------------------------------------------
# distributed plumbing
# ---------------------------------------------------------------------------------------
def barrier(world: int) -> None:
    if world > 1:
        import torch.distributed as dist

        dist.barrier()


def reduce_max(value: float, world: int, device) -> float:
    if world <= 1:
        return value
    import torch
    import torch.distributed as dist

    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--workload", default="decode", choices=["decode"])
    parser.add_argument("--batch", type=int, default=1, help="decode batch M (1, 4, 8)")
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--load-seconds", type=float, default=1.5)
    parser.add_argument("--no-cpu-baseline", action="store_true")
    args = parser.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        line = run_reference(args, rank, world)
        if line is not None:
            print(json.dumps(line), flush=True)
        return 0

    import torch

    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device; this benchmark has no CPU fallback"}), flush=True)
        return 1
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    line = run_decode(args, rank, world, device)
    if rank == 0:
        if args.no_cpu_baseline:
            line["cpu_baseline"] = None
        else:
            value, cores, sample, _ = cpu_decode(args.batch, 5, 1, budget_s=25.0)
            line["cpu_baseline"] = {"value": round(value, 4), "unit": "GB/s", "cores": cores, "kind": "port",
                                    "sample": sample}
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
