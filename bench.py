#!/usr/bin/env python
"""Benchmark of the quantized-contraction hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload W] [--impl reference]

Prints ONE JSON line (rank 0).  Workloads (seeded synthetic inputs with the
shapes and value distributions of the benchmark configurations):

  prefill  (default) W4A16 prefill GEMM 8192^3 bf16, columns of W split over the GPUs;
           metric = TFLOP/s.  Tensor-core bound.  The decode figures are attached to the
           same line under "decode" (the headline metric names both).
  decode   W4A16 decode GEMV, M=1: one step = the up projection
           [1,4096]x[4096,14336] and the down projection [1,14336]x[14336,4096];
           metric = weight GB/s (algorithmic bytes / time).  HBM-bound.  Replicas only.
  w8a8     int8 GEMM 4096x8192x8192 with the scaled bf16 epilogue, columns split.
  moe      16384-token top-2 MoE FFN with int4 experts; expert parallel for N > 1
           (--moe-exchange peer: rows and results move by direct NVLink stores and loads
           between the ranks' buffers; nccl: all-to-all; --moe-graph: the peer step as one
           CUDA graph).
  grouped  the reference's published dense grouped GEMM case (8 groups x 1024 rows,
           K=4096, N=14336, f16), columns split.

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
NCU_TRAFFIC_BYTES = {"decode": 30314496, "prefill": 529902848, "w8a8": 149691136, "grouped": 1231225192}


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
    # decode loop: the packed weights are static model state, so a GEMV may start fetching them while
    # the previous kernel on the stream drains (programmatic dependent launch)
    native.set_gemv_launch_overlap(True)
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

    native.set_gemv_launch_overlap(False)
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
                   "launch": "programmatic dependent launch between consecutive GEMVs (static weights)",
                   "parallelism": "replicas only" if world > 1 else "1 gpu"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4), "traffic": NCU_TRAFFIC_BYTES["decode"],
                     "peak_source": peaks["source"], "algorithmic_bytes_per_launch": per_launch_bytes,
                     "kernel": "w4a16_stream_kernel", "us_per_launch": round(per_launch_s * 1e6, 3)},
        "e2e": {"value": round(world * step_bytes / (e2e_s / args.steps) / 1e9, 2), "unit": "GB/s",
                "h2d_bytes_per_step": sum(x.numel() * 2 for x in pinned_in),
                "d2h_bytes_per_step": sum(y.numel() * 2 for y in pinned_out),
                "ms_per_step": round(e2e_s / args.steps * 1e3, 6)},
        "gpu_launches": int(launches),
        "clocks": clocks,
    }
    return line


# ---------------------------------------------------------------------------------------
# tensor-core workloads: W4A16 prefill (configs[2]), W8A8 (configs[3]), MoE (configs[4])
# ---------------------------------------------------------------------------------------
def timed_steps(step, steps: int, warmup: int, world: int, device, rank: int, load_seconds: float):
    """Warm up, hold the load while clocks are sampled, then time exactly `steps` steps with CUDA
    events on the current stream, bracketed by barriers; returns (ms total, clocks, launches)."""
    import torch

    from intent_b200.runtime import native

    for _ in range(max(warmup, 3)):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(device.index)
    if rank == 0:
        sampler.start()
    # hold the load for about load_seconds; every rank runs the same number of steps (a step may
    # contain collectives, so the count is agreed on, not decided by each rank's own clock)
    load_steps = 0
    if load_seconds > 0:
        t0 = time.perf_counter()
        step()
        torch.cuda.synchronize()
        one = max(time.perf_counter() - t0, 1e-5)
        load_steps = int(reduce_max(min(load_seconds / one, 1e6), world, device))
    for _ in range(load_steps):
        step()
    torch.cuda.synchronize()
    barrier(world)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    before = native.launch_count()
    start.record()
    for _ in range(steps):
        step()
    stop.record()
    torch.cuda.synchronize()
    barrier(world)
    launches = native.launch_count() - before
    elapsed_ms = reduce_max(start.elapsed_time(stop), world, device)
    clocks = sampler.stop() if rank == 0 else None
    return elapsed_ms, clocks, launches


def timed_e2e(step, steps: int, warmup: int, world: int, device):
    import torch

    for _ in range(max(min(warmup, 3), 1)):
        step()
    barrier(world)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    torch.cuda.synchronize()
    return reduce_max(time.perf_counter() - t0, world, device)


PREFILL = dict(M=8192, K=8192, N=8192)
W8A8 = dict(M=4096, K=8192, N=8192)
MOE = dict(tokens=16384, hidden=4096, experts=64, intermediate=1408, top_k=2)


def run_prefill(args, rank: int, world: int, device):
    import torch

    import intent_b200 as ib
    from intent_b200.distributed import column_shard

    M, K, N = PREFILL["M"], PREFILL["K"], PREFILL["N"]
    x, packed, scales = ib.workloads.w4a16_inputs(M, K, N, dtype=torch.bfloat16, group_size=GROUP, seed=0)
    cols = column_shard(N, world, rank)
    artifact = ib.compile(ib.programs.weight_only_int4_matmul, target=ib.B200Target(device.index),
                          constexprs={"GROUP_SIZE": GROUP, "ZERO_POINT": 8, "ACT_DTYPE": "bf16"})
    xd = x.to(device)
    pd, sd = packed[:, cols].contiguous().to(device), scales[:, cols].contiguous().to(device)
    call = artifact.prepare(xd, pd, sd)
    elapsed_ms, clocks, launches = timed_steps(call.launch, args.steps, args.warmup, world, device, rank,
                                               args.load_seconds)
    # end to end: activations from pinned host memory, this rank's block of Y read back
    pinned_x = x.pin_memory()
    n_local = cols.stop - cols.start
    pinned_y = torch.empty((M, n_local), dtype=torch.bfloat16).pin_memory()

    def e2e_step():
        y = artifact.run(pinned_x.to(device, non_blocking=True), pd, sd)
        pinned_y.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_s = timed_e2e(e2e_step, max(1, min(args.steps, 20)), args.warmup, world, device)
    e2e_steps = max(1, min(args.steps, 20))
    flops = 2.0 * M * K * N
    ms = elapsed_ms / args.steps
    peaks = measured_peaks()
    per_launch_flops = flops / world
    achieved = per_launch_flops / (ms * 1e-3) / 1e12
    line = {
        "metric": "w4a16_prefill_TFLOPs", "value": round(flops / (ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 5),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "w4a16_prefill_gemm M=8192 K=8192 N=8192 bf16 g128 zp8 (configs[2])",
                   "group_size": GROUP, "parallelism": f"columns of W split over {world} gpu(s), no collective",
                   "l2": "X (128 MiB) + Y (128 MiB) + W exceed the 126 MB L2 every step",
                   "timing": "CUDA events on the launch stream around K launches"},
        "roofline": {"bound": "tensor", "achieved": round(achieved, 1), "peak": peaks["bf16_tflops"],
                     "unit": "TFLOP/s", "frac": round(achieved / peaks["bf16_tflops"], 4),
                     "traffic": NCU_TRAFFIC_BYTES.get("prefill"), "peak_source": peaks["source"] + " (burst cuBLAS bf16)",
                     "frac_of_sustained": round(achieved / peaks["bf16_tflops_sustained"], 4),
                     "frac_of_nominal_2250": round(achieved / 2250.0, 4),
                     "algorithmic_flops_per_launch": per_launch_flops, "kernel": "w4a16_gemm_pair_kernel",
                     "ms_per_launch": round(ms, 5)},
        "e2e": {"value": round(flops / (e2e_s / e2e_steps) / 1e12, 2), "unit": "TFLOP/s",
                "h2d_bytes_per_step": M * K * 2, "d2h_bytes_per_step": M * n_local * 2,
                "ms_per_step": round(e2e_s / e2e_steps * 1e3, 4), "steps": e2e_steps},
        "gpu_launches": int(launches), "clocks": clocks,
    }
    return line


def run_w8a8(args, rank: int, world: int, device):
    import torch

    import intent_b200 as ib
    from intent_b200.distributed import column_shard

    M, K, N = W8A8["M"], W8A8["K"], W8A8["N"]
    a, b, sa, sb = ib.workloads.w8a8_inputs(M, K, N, seed=0)
    cols = column_shard(N, world, rank)
    artifact = ib.compile(ib.programs.w8a8_gemm, target=ib.B200Target(device.index))
    ad, sad = a.to(device), sa.to(device)
    bd, sbd = b[:, cols].contiguous().to(device), sb[cols].contiguous().to(device)
    call = artifact.prepare(ad, bd, sad, sbd)
    elapsed_ms, clocks, launches = timed_steps(call.launch, args.steps, args.warmup, world, device, rank,
                                               args.load_seconds)
    pinned_a = a.pin_memory()
    n_local = cols.stop - cols.start
    pinned_y = torch.empty((M, n_local), dtype=torch.bfloat16).pin_memory()

    def e2e_step():
        y = artifact.run(pinned_a.to(device, non_blocking=True), bd, sad, sbd)
        pinned_y.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_steps = max(1, min(args.steps, 20))
    e2e_s = timed_e2e(e2e_step, e2e_steps, args.warmup, world, device)
    ops = 2.0 * M * K * N
    ms = elapsed_ms / args.steps
    peaks = measured_peaks()
    achieved = ops / world / (ms * 1e-3) / 1e12
    int8_peak = 2.0 * peaks["bf16_tflops"]   # no measured int8 figure: twice the measured bf16 burst
    return {
        "metric": "w8a8_gemm_TOPs", "value": round(ops / (ms * 1e-3) / 1e12, 2), "unit": "TOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 5),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "w8a8_gemm M=4096 K=8192 N=8192 int8 -> bf16 scaled epilogue (configs[3])",
                   "parallelism": f"columns of B split over {world} gpu(s), no collective",
                   "l2": "A + B + Y = 160 MiB exceed the 126 MB L2 every step"},
        "roofline": {"bound": "tensor", "achieved": round(achieved, 1), "peak": int8_peak, "unit": "TOP/s",
                     "frac": round(achieved / int8_peak, 4), "traffic": NCU_TRAFFIC_BYTES.get("w8a8"),
                     "peak_source": "2 x measured bf16 burst (no int8 peak was measured on this pool)",
                     "frac_of_nominal_4500": round(achieved / 4500.0, 4), "kernel": "i8_gemm_kernel",
                     "ms_per_launch": round(ms, 5)},
        "e2e": {"value": round(ops / (e2e_s / e2e_steps) / 1e12, 2), "unit": "TOP/s",
                "h2d_bytes_per_step": M * K, "d2h_bytes_per_step": M * n_local * 2,
                "ms_per_step": round(e2e_s / e2e_steps * 1e3, 4), "steps": e2e_steps},
        "gpu_launches": int(launches), "clocks": clocks,
    }


GROUPED = dict(groups=8, rows_per_group=1024, K=4096, N=14336)
GROUPED_PUBLISHED_MS = 4.393   # the reference's own number for this case on an RTX 5090D (other hardware)


def run_grouped(args, rank: int, world: int, device):
    """The reference's published dense grouped GEMM case (experiments/gpu/registry.py:7):
    8 groups x 1024 rows, K=4096, N=14336, f16, through the ragged_grouped_gemm program."""
    import torch

    import intent_b200 as ib
    from intent_b200.distributed import column_shard

    G, rows_per_group, K, N = (GROUPED[k] for k in ("groups", "rows_per_group", "K", "N"))
    R = G * rows_per_group
    gen = torch.Generator().manual_seed(0)
    x = (torch.randn((R, K), generator=gen) * 0.5).half()
    cols = column_shard(N, world, rank)
    n_local = cols.stop - cols.start
    wd = torch.empty((G, K, n_local), dtype=torch.float16, device=device)
    for g in range(G):      # weights are drawn group by group so the host never holds all 940 MB at once
        wd[g] = (torch.randn((K, N), generator=gen) / K ** 0.5).half()[:, cols].to(device)
    offsets = (torch.arange(G + 1, dtype=torch.int32) * rows_per_group).to(device)
    artifact = ib.compile(ib.programs.ragged_grouped_gemm, target=ib.B200Target(device.index))
    xd = x.to(device)
    call = artifact.prepare(xd, offsets, wd)
    elapsed_ms, clocks, launches = timed_steps(call.launch, args.steps, args.warmup, world, device, rank,
                                               args.load_seconds)
    pinned_x = x.pin_memory()
    pinned_y = torch.empty((R, n_local), dtype=torch.float16).pin_memory()

    def e2e_step():
        y = artifact.run(pinned_x.to(device, non_blocking=True), offsets, wd)
        pinned_y.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_steps = max(1, min(args.steps, 20))
    e2e_s = timed_e2e(e2e_step, e2e_steps, args.warmup, world, device)
    flops = 2.0 * R * K * N
    ms = elapsed_ms / args.steps
    peaks = measured_peaks()
    achieved = flops / world / (ms * 1e-3) / 1e12
    published_tflops = flops / (GROUPED_PUBLISHED_MS * 1e-3) / 1e12
    return {
        "metric": "ragged_grouped_gemm_TFLOPs", "value": round(flops / (ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 5),
        "higher_is_better": True, "scaling": "strong",
        "vs_baseline": round(flops / (ms * 1e-3) / 1e12 / published_tflops, 3) if world == 1 else None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD_META["grouped"][4],
                   "parallelism": f"columns of W split over {world} gpu(s), no collective",
                   "l2": "W (940 MB) + X + Y exceed the 126 MB L2 every step",
                   "published": f"{GROUPED_PUBLISHED_MS} ms = {published_tflops:.0f} TFLOP/s on an RTX 5090D "
                                "(the reference's generated Triton kernel; other hardware)"},
        "roofline": {"bound": "tensor", "achieved": round(achieved, 1), "peak": peaks["bf16_tflops"],
                     "unit": "TFLOP/s", "frac": round(achieved / peaks["bf16_tflops"], 4),
                     "traffic": NCU_TRAFFIC_BYTES.get("grouped"),
                     "peak_source": peaks["source"] + " (burst cuBLAS bf16)",
                     "frac_of_sustained": round(achieved / peaks["bf16_tflops_sustained"], 4),
                     "algorithmic_flops_per_launch": flops / world, "kernel": "grouped_gemm16_kernel",
                     "ms_per_launch": round(ms, 5)},
        "e2e": {"value": round(flops / (e2e_s / e2e_steps) / 1e12, 2), "unit": "TFLOP/s",
                "h2d_bytes_per_step": R * K * 2, "d2h_bytes_per_step": R * n_local * 2,
                "ms_per_step": round(e2e_s / e2e_steps * 1e3, 4), "steps": e2e_steps},
        "gpu_launches": int(launches), "clocks": clocks,
    }


def run_moe(args, rank: int, world: int, device):
    import torch

    import intent_b200 as ib
    from intent_b200.moe import MoEW4A16FFN

    cfg = MOE
    tokens, hidden, experts, inter = cfg["tokens"], cfg["hidden"], cfg["experts"], cfg["intermediate"]
    if experts % world or tokens % world:
        raise SystemExit("moe workload needs the gpu count to divide 64 experts and 16384 tokens")
    data = ib.workloads.moe_inputs(tokens, hidden, experts, inter, dtype=torch.bfloat16, seed=0)
    t_local, e_local = tokens // world, experts // world
    rows = slice(rank * t_local, (rank + 1) * t_local)
    ex = slice(rank * e_local, (rank + 1) * e_local)
    logits, x = data["logits"][rows].contiguous(), data["x"][rows].contiguous()
    weights = [data[k][ex].contiguous().to(device) for k in ("up_gate_packed", "up_gate_scales", "down_packed",
                                                             "down_scales")]
    if world == 1:
        ffn = MoEW4A16FFN(tokens=tokens, hidden=hidden, intermediate=inter, experts=experts,
                          block_size=args.moe_block, target=ib.B200Target(device.index))

        def forward(lg, xx):
            ids, w = ffn.route(lg)
            return ffn(xx, ids, w, *weights)

        def prepare(lg, xx):
            router = ffn.router.prepare(lg)
            ids, w = router.result()
            y = torch.empty((xx.shape[0], hidden), dtype=torch.float32, device=device)
            chain = ffn.prepare(xx, ids, w, *weights, y)

            def launch():
                router.launch()
                return chain.launch()
            return launch
    elif args.moe_exchange == "peer":
        from intent_b200.peer import PeerExpertParallelMoE

        # rows go straight into the owners' buffers over NVLink and results are read straight back:
        # no collective on the data path, worst-case buffers (no overflow case)
        ep = PeerExpertParallelMoE(tokens=t_local, hidden=hidden, intermediate=inter, experts=experts,
                                   block_rows=args.moe_block, target=ib.B200Target(device.index))
        bound = {}

        def prepare(lg, xx):
            call = ep.prepare(lg, xx, *weights)
            bound.update(logits=lg, x=xx, call=call)
            if not args.moe_graph:
                return call.launch
            # the step holds no collective call (flag posts and bounded flag waits over peer memory),
            # so it can be replayed as one CUDA graph
            for _ in range(3):
                call.launch()
            torch.cuda.synchronize()
            barrier(world)
            from intent_b200.runtime import native

            graph = torch.cuda.CUDAGraph()
            before = native.launch_count()
            with torch.cuda.graph(graph):
                call.launch()
            bound["graph"], bound["launches_per_replay"] = graph, native.launch_count() - before
            return graph.replay

        def forward(lg, xx):      # end to end: the bound input buffers are refilled, the bound step is launched
            bound["logits"].copy_(lg, non_blocking=True)
            bound["x"].copy_(xx, non_blocking=True)
            (bound["graph"].replay if "graph" in bound else bound["call"].launch)()
            return bound["call"].y
    else:
        from intent_b200.distributed import ExpertParallelMoE

        # fixed-capacity exchange (1.5x the mean rows per destination): no device -> host read in the step;
        # an overflow would be recorded on the device and is checked after the timed region
        ep = ExpertParallelMoE(tokens=t_local, hidden=hidden, intermediate=inter, experts=experts,
                               capacity_factor=1.5, block_size=args.moe_block, target=ib.B200Target(device.index))

        def forward(lg, xx):
            return ep(lg, xx, *weights)

        def prepare(lg, xx):
            return ep.prepare(lg, xx, *weights).launch

    # the step is bound once to fixed buffers (prepare), then launched K times
    lgd, xd = logits.to(device), x.to(device)
    elapsed_ms, clocks, launches = timed_steps(prepare(lgd, xd), args.steps, args.warmup, world, device,
                                               rank, args.load_seconds)
    if world > 1 and args.moe_exchange == "peer" and "launches_per_replay" in bound:
        launches = bound["launches_per_replay"] * args.steps      # kernels inside the replayed graph
    pinned_l, pinned_x = logits.pin_memory(), x.pin_memory()
    pinned_y = torch.empty((t_local, hidden), dtype=torch.float32).pin_memory()

    def e2e_step():
        if world > 1 and args.moe_exchange == "peer":
            y = forward(pinned_l, pinned_x)
        else:
            y = forward(pinned_l.to(device, non_blocking=True), pinned_x.to(device, non_blocking=True))
        pinned_y.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_steps = max(1, min(args.steps, 20))
    e2e_s = timed_e2e(e2e_step, e2e_steps, args.warmup, world, device)
    if world > 1 and args.moe_exchange != "peer":
        ep.check_overflow()
    if world > 1 and args.moe_exchange == "peer":
        bound["call"].check()          # a cross-rank wait that gave up would invalidate the run
    flops = tokens * cfg["top_k"] * (2.0 * hidden * 2 * inter + 2.0 * inter * hidden)
    ms = elapsed_ms / args.steps
    peaks = measured_peaks()
    achieved = flops / world / (ms * 1e-3) / 1e12
    return {
        "metric": "moe_w4a16_ffn_TFLOPs", "value": round(flops / (ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 5),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "moe_w4a16_swiglu_ffn 16384 tokens H=4096 E=64 top-2 I=1408 g128 (configs[4])",
                   "parallelism": "all experts local" if world == 1 else
                   (f"expert parallel: {e_local} experts and {t_local} tokens per gpu, rows written into the owners' "
                    "buffers and results read back over NVLink peer memory; three sync points per step as flag "
                    "posts and bounded flag waits over peer memory, no collective call"
                    + (", replayed as one CUDA graph" if args.moe_graph else "") if args.moe_exchange == "peer" else
                    f"expert parallel: {e_local} experts and {t_local} tokens per gpu, NCCL all-to-all each way, "
                    "fixed-capacity exchange (factor 1.5)"),
                   "step": "router + alignment + gather + up|gate GEMM (SiLU) + down GEMM + combine",
                   "expert_block_rows": args.moe_block,
                   "l2": "expert weights (571 MB) and row buffers exceed the 126 MB L2"},
        "roofline": {"bound": "tensor", "achieved": round(achieved, 1), "peak": peaks["bf16_tflops"],
                     "unit": "TFLOP/s", "frac": round(achieved / peaks["bf16_tflops"], 4), "traffic": None,
                     "peak_source": peaks["source"] + " (burst cuBLAS bf16); whole step, not one kernel",
                     "kernel": "w4a16_gemm_kernel (grouped modes)"},
        "e2e": {"value": round(flops / (e2e_s / e2e_steps) / 1e12, 2), "unit": "TFLOP/s",
                "h2d_bytes_per_step": t_local * (64 * 4 + hidden * 2), "d2h_bytes_per_step": t_local * hidden * 4,
                "ms_per_step": round(e2e_s / e2e_steps * 1e3, 4), "steps": e2e_steps},
        "gpu_launches": int(launches), "clocks": clocks,
    }


# ---------------------------------------------------------------------------------------
# CPU arm (the reference's CPU implementation of the path, restated in oracle/)
# ---------------------------------------------------------------------------------------
def cpu_decode(M: int, steps: int, warmup: int, budget_s: float):
    """Time the torch-CPU implementation of the decode step.  Returns
    (GB/s, cores, sample description, ms per step)."""
    import torch

    import oracle

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    host = decode_inputs(M)

    def step(divisor: int) -> None:
        for x, p, s in host:
            n = p.shape[1] // divisor
            oracle.weight_only_int4_matmul(x, p[:, :n].contiguous(), s[:, :n].contiguous(),
                                           group_size=GROUP, zero_point=8)

    t0 = time.perf_counter()
    step(8)
    full_estimate = (time.perf_counter() - t0) * 8
    divisor = 1
    while full_estimate / divisor * (steps + warmup) > budget_s and divisor < 64:
        divisor *= 2
    for _ in range(warmup):
        step(divisor)
    t0 = time.perf_counter()
    for _ in range(steps):
        step(divisor)
    seconds = (time.perf_counter() - t0) / steps
    sample = (f"{steps} steps of the decode step on the first 1/{divisor} of the output columns "
              f"(M={M}, both projections), torch CPU, {cores} threads")
    return decode_bytes(M) / divisor / seconds / 1e9, cores, sample, seconds * 1e3


def cpu_prefill(steps: int, warmup: int, budget_s: float):
    """W4A16 prefill on the CPU: a slice of the rows of X against the whole weight (the dequantisation of
    W is part of every call, as in the reference's torch implementation).  Returns TFLOP/s of the slice."""
    import torch

    import oracle
    from intent_b200 import workloads

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    K, N = PREFILL["K"], PREFILL["N"]
    rows = 64
    x, p, s = workloads.w4a16_inputs(rows, K, N, dtype=torch.bfloat16, group_size=GROUP, seed=0)
    t0 = time.perf_counter()
    oracle.weight_only_int4_matmul(x, p, s, group_size=GROUP, zero_point=8)
    one = time.perf_counter() - t0
    steps = max(1, min(steps, int(budget_s / max(one, 1e-3)) - warmup))
    for _ in range(warmup):
        oracle.weight_only_int4_matmul(x, p, s, group_size=GROUP, zero_point=8)
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle.weight_only_int4_matmul(x, p, s, group_size=GROUP, zero_point=8)
    seconds = (time.perf_counter() - t0) / steps
    sample = (f"{steps} steps of {rows} of the 8192 rows of X against the full 8192x8192 int4 weight "
              f"(dequantisation included), torch CPU, {cores} threads")
    return 2.0 * rows * K * N / seconds / 1e12, cores, sample, seconds * 1e3, steps


def cpu_w8a8(steps: int, warmup: int, budget_s: float):
    import torch

    import oracle
    from intent_b200 import workloads

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    K, N = W8A8["K"], W8A8["N"]
    rows = 512
    a, b, sa, sb = workloads.w8a8_inputs(rows, K, N, seed=0)
    t0 = time.perf_counter()
    oracle.w8a8_scaled_gemm(a, b, sa, sb)
    one = time.perf_counter() - t0
    steps = max(1, min(steps, int(budget_s / max(one, 1e-3)) - warmup))
    for _ in range(warmup):
        oracle.w8a8_scaled_gemm(a, b, sa, sb)
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle.w8a8_scaled_gemm(a, b, sa, sb)
    seconds = (time.perf_counter() - t0) / steps
    sample = f"{steps} steps of {rows} of the 4096 rows of A against the full 8192x8192 B, torch CPU int matmul, {cores} threads"
    return 2.0 * rows * K * N / seconds / 1e12, cores, sample, seconds * 1e3, steps


def cpu_moe(steps: int, warmup: int, budget_s: float):
    import torch

    import oracle
    from intent_b200 import workloads

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    cfg = MOE
    tokens, experts = 256, 8        # bounded sample: 256 tokens over 8 of the 64 experts, same H and I
    data = workloads.moe_inputs(tokens, cfg["hidden"], experts, cfg["intermediate"], dtype=torch.bfloat16, seed=0)

    def step():
        ids, w = oracle.moe_route_top2(data["logits"])
        oracle.moe_w4a16_swiglu_ffn(data["x"], ids, w, data["up_gate_packed"], data["up_gate_scales"],
                                    data["down_packed"], data["down_scales"])

    t0 = time.perf_counter()
    step()
    one = time.perf_counter() - t0
    steps = max(1, min(steps, int(budget_s / max(one, 1e-3)) - warmup))
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    seconds = (time.perf_counter() - t0) / steps
    flops = tokens * 2 * (2.0 * cfg["hidden"] * 2 * cfg["intermediate"] + 2.0 * cfg["intermediate"] * cfg["hidden"])
    sample = (f"{steps} steps of {tokens} tokens over {experts} experts (H=4096, I=1408, top-2; per-expert "
              f"dequantisation included), torch CPU, {cores} threads")
    return flops / seconds / 1e12, cores, sample, seconds * 1e3, steps


def cpu_grouped(steps: int, warmup: int, budget_s: float):
    import torch

    import oracle

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    G, K, N = GROUPED["groups"], GROUPED["K"], GROUPED["N"]
    rows, groups = 128, 2      # bounded sample: 2 of the 8 groups, 128 of the 1024 rows each
    gen = torch.Generator().manual_seed(0)
    x = (torch.randn((rows * groups, K), generator=gen) * 0.5).half()
    w = (torch.randn((groups, K, N), generator=gen) / K ** 0.5).half()
    offsets = torch.arange(groups + 1, dtype=torch.int32) * rows
    t0 = time.perf_counter()
    oracle.ragged_grouped_gemm(x, offsets, w)
    one = time.perf_counter() - t0
    steps = max(1, min(steps, int(budget_s / max(one, 1e-3)) - warmup))
    for _ in range(warmup):
        oracle.ragged_grouped_gemm(x, offsets, w)
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle.ragged_grouped_gemm(x, offsets, w)
    seconds = (time.perf_counter() - t0) / steps
    sample = (f"{steps} steps of {groups} of the {G} groups, {rows} of the 1024 rows each, full K and N, "
              f"torch CPU f32 matmul per group, {cores} threads")
    return 2.0 * rows * groups * K * N / seconds / 1e12, cores, sample, seconds * 1e3, steps


WORKLOAD_META = {
    "prefill": ("w4a16_prefill_TFLOPs", "TFLOP/s", "strong", "bf16",
                "w4a16_prefill_gemm M=8192 K=8192 N=8192 bf16 g128 zp8 (configs[2])"),
    "w8a8": ("w8a8_gemm_TOPs", "TOP/s", "strong", "int8",
             "w8a8_gemm M=4096 K=8192 N=8192 int8 -> bf16 scaled epilogue (configs[3])"),
    "moe": ("moe_w4a16_ffn_TFLOPs", "TFLOP/s", "strong", "bf16",
            "moe_w4a16_swiglu_ffn 16384 tokens H=4096 E=64 top-2 I=1408 g128 (configs[4])"),
    "decode": ("w4a16_decode_weight_GBps", "GB/s", "weak", "f16", None),
    "grouped": ("ragged_grouped_gemm_TFLOPs", "TFLOP/s", "strong", "f16",
                "ragged_grouped_gemm 8 groups x 1024 rows K=4096 N=14336 f16 (the reference's grouped_gemm case)"),
}


def cpu_workload(args, steps: int, warmup: int, budget_s: float):
    """(value, unit, cores, sample, ms per step, steps actually timed) of the CPU implementation."""
    if args.workload == "decode":
        value, cores, sample, ms = cpu_decode(args.batch, steps, warmup, budget_s)
        return value, "GB/s", cores, sample, ms, steps
    fn = {"prefill": cpu_prefill, "w8a8": cpu_w8a8, "moe": cpu_moe, "grouped": cpu_grouped}[args.workload]
    value, cores, sample, ms, done = fn(steps, warmup, budget_s)
    return value, WORKLOAD_META[args.workload][1], cores, sample, ms, done


def run_reference(args, rank: int, world: int):
    if rank != 0:
        return None
    metric, unit, scaling, _, workload = WORKLOAD_META[args.workload]
    if workload is None:
        workload = f"w4a16_decode_gemv M={args.batch} [4096->14336]+[14336->4096] g128 zp8 (configs[1])"
    value, unit, cores, sample, ms, done = cpu_workload(args, args.steps, max(args.warmup, 1), budget_s=150.0)
    return {
        "impl": "reference", "metric": metric, "value": round(value, 5), "unit": unit,
        "n_gpus": world, "steps": done, "warmup": max(args.warmup, 1), "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload, "note": "CPU implementation of the same path on the host cores; each step "
                   "is the bounded sample named in cpu_baseline.sample, throughput is per unit of work"},
        "cpu_baseline": {"value": round(value, 5), "unit": unit, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": round(value, 5), "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
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
    parser.add_argument("--steps", type=int, default=None)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--workload", default="prefill", choices=["prefill", "decode", "w8a8", "moe", "grouped"])
    parser.add_argument("--batch", type=int, default=1, help="decode batch M (1, 4, 8)")
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--load-seconds", type=float, default=1.5)
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--moe-block", type=int, default=128, choices=[128, 256],
                        help="rows every expert span is padded to (= row tile of the grouped contraction)")
    parser.add_argument("--moe-exchange", default="peer", choices=["peer", "nccl"],
                        help="expert-parallel exchange: direct peer-memory stores/loads, or NCCL all-to-all")
    parser.add_argument("--moe-graph", action="store_true",
                        help="replay the expert-parallel step (peer exchange) as one CUDA graph")
    parser.add_argument("--no-decode", action="store_true", help="prefill line without the attached decode figures")
    args = parser.parse_args()
    if args.steps is None:
        args.steps = {"prefill": 50, "decode": 200, "w8a8": 100, "moe": 20, "grouped": 50}[args.workload]
        if args.impl == "reference":
            args.steps = 5

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

    runner = {"prefill": run_prefill, "decode": run_decode, "w8a8": run_w8a8, "moe": run_moe,
              "grouped": run_grouped}[args.workload]
    line = runner(args, rank, world, device)
    if args.workload == "prefill" and not args.no_decode:
        # the headline metric has two halves: attach the decode GEMV (weight GB/s) measured in the same run
        decode_args = argparse.Namespace(**vars(args))
        decode_args.steps, decode_args.load_seconds = 200, 0.5
        decode = run_decode(decode_args, rank, world, device)
        line["decode"] = {k: decode[k] for k in ("metric", "value", "unit", "ms_per_step", "config", "roofline", "e2e",
                                                  "gpu_launches", "scaling")}
    if rank == 0:
        if args.no_cpu_baseline:
            line["cpu_baseline"] = None
        else:
            value, unit, cores, sample, _, _ = cpu_workload(args, 5, 1, budget_s=25.0)
            line["cpu_baseline"] = {"value": round(value, 5), "unit": unit, "cores": cores, "kind": "port",
                                    "sample": sample}
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
