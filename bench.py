#!/usr/bin/env python
"""Benchmark of the quantized-contraction hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload W] [--impl reference|triton]

Prints ONE JSON line (rank 0).  Workloads (seeded synthetic inputs with the
shapes and value distributions of the benchmark configurations):

  prefill  (default) W4A16 prefill GEMM 8192^3 bf16, columns of W split over the GPUs;
           metric = TFLOP/s.  Tensor-core bound.  Unless --attach none is given the same
           line carries one object per other configuration, each with its own roofline,
           e2e and cpu_baseline: "decode" (M=1), "decode_m4", "decode_m8", "w8a8", "moe".
  decode   W4A16 decode GEMV: one step = the up projection [M,4096]x[4096,14336] and the
           down projection [M,14336]x[14336,4096]; metric = weight GB/s (algorithmic
           bytes / time).  HBM-bound.  Replicas only.
  w8a8     int8 GEMM 4096x8192x8192 with the scaled bf16 epilogue, columns split.
  moe      16384-token top-2 MoE FFN with int4 experts; expert parallel for N > 1
           (--moe-exchange peer: rows and results move by direct NVLink stores and loads
           between the ranks' buffers, the bound step replayed as one CUDA graph unless
           --moe-eager; nccl: all-to-all).
  grouped  the reference's published dense grouped GEMM case (8 groups x 1024 rows,
           K=4096, N=14336, f16), columns split.

`value` is measured with inputs resident in HBM (decode: the K timed steps captured in one
CUDA graph, weights rotated through more copies than fit in L2).  `e2e` is the same metric
through the library's public call surface with the step's activations in pinned host memory
(H2D + D2H inside the timed region, overlapped with the contraction where the helper of
intent_b200.distributed does so).  The weights are model state and stay resident in both.

`--impl reference` times the CPU implementation of the same path (the torch-CPU restatement
of the reference's own CPU code, all host threads) on the same configuration, rank 0 only.
`--impl triton` times a hand-restated Triton kernel of the shape the reference's provider
emits for W4A16 (informational; never on the product path).
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

# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) per launch of the dominant kernel, from the ncu
# captures summarised under profiles/, taken on ONE GPU with the full problem.  A rank of a sharded run
# computes a different problem (a column shard against the whole of X), whose traffic was not captured and
# does not scale with the shard: there the line reports null.
NCU_TRAFFIC_BYTES_1GPU = {"decode": 30314496, "prefill": 529902848, "w8a8": 149691136, "grouped": 1231225192,
                          "moe": None}


def ncu_traffic(workload: str, world: int):
    return NCU_TRAFFIC_BYTES_1GPU.get(workload) if world == 1 else None


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
# shapes and the configuration text both arms print
# ---------------------------------------------------------------------------------------
DECODE_SHAPES = ((4096, 14336), (14336, 4096))      # (K, N): up projection, down projection
GROUP = 128
PREFILL = dict(M=8192, K=8192, N=8192)
W8A8 = dict(M=4096, K=8192, N=8192)
MOE = dict(tokens=16384, hidden=4096, experts=64, intermediate=1408, top_k=2)
GROUPED = dict(groups=8, rows_per_group=1024, K=4096, N=14336)
GROUPED_PUBLISHED_MS = 4.393   # the reference's own number for this case on an RTX 5090D (other hardware)

WORKLOAD_META = {     # metric, unit, scaling, dtype
    "prefill": ("w4a16_prefill_TFLOPs", "TFLOP/s", "strong", "bf16"),
    "w8a8": ("w8a8_gemm_TOPs", "TOP/s", "strong", "int8"),
    "moe": ("moe_w4a16_ffn_TFLOPs", "TFLOP/s", "strong", "bf16"),
    "decode": ("w4a16_decode_weight_GBps", "GB/s", "weak", "f16"),
    "grouped": ("ragged_grouped_gemm_TFLOPs", "TFLOP/s", "strong", "f16"),
}


def workload_config(workload: str, world: int, batch: int = 1) -> dict:
    """The `config` object of a line: identical for the B200 arm and the reference arm."""
    if workload == "prefill":
        return {"workload": "w4a16_prefill_gemm M=8192 K=8192 N=8192 bf16 g128 zp8 (configs[2])",
                "group_size": GROUP, "parallelism": f"columns of W split over {world} gpu(s), no collective",
                "l2": "X (128 MiB) + Y (128 MiB) + W exceed the 126 MB L2 every step"}
    if workload == "w8a8":
        return {"workload": "w8a8_gemm M=4096 K=8192 N=8192 int8 -> bf16 scaled epilogue (configs[3])",
                "parallelism": f"columns of B split over {world} gpu(s), no collective",
                "l2": "A + B + Y = 160 MiB exceed the 126 MB L2 every step"}
    if workload == "moe":
        return {"workload": "moe_w4a16_swiglu_ffn 16384 tokens H=4096 E=64 top-2 I=1408 g128 (configs[4])",
                "parallelism": "all experts local" if world == 1 else
                f"expert parallel over {world} gpus: {MOE['experts'] // world} experts and "
                f"{MOE['tokens'] // world} tokens per gpu",
                "step": "router + alignment + gather + up|gate GEMM (SiLU) + down GEMM + combine",
                "l2": "expert weights (571 MB) and row buffers exceed the 126 MB L2"}
    if workload == "decode":
        return {"workload": f"w4a16_decode_gemv M={batch} [4096->14336]+[14336->4096] g128 zp8 (configs[1])",
                "batch": batch, "group_size": GROUP, "step": "up + down projection",
                "parallelism": "replicas only" if world > 1 else "1 gpu"}
    if workload == "grouped":
        return {"workload": "ragged_grouped_gemm 8 groups x 1024 rows K=4096 N=14336 f16 "
                            "(the reference's grouped_gemm case)",
                "parallelism": f"columns of W split over {world} gpu(s), no collective",
                "l2": "W (940 MB) + X + Y exceed the 126 MB L2 every step"}
    raise ValueError(workload)


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


def moe_flops() -> float:
    return MOE["tokens"] * MOE["top_k"] * (2.0 * MOE["hidden"] * 2 * MOE["intermediate"] +
                                           2.0 * MOE["intermediate"] * MOE["hidden"])


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


# ---------------------------------------------------------------------------------------
# decode GEMV (configs[1])
# ---------------------------------------------------------------------------------------
class DecodeWeights:
    """The two projections' packed weights, rotated through more resident copies than fit in L2 (built once
    per run and shared by the batch sizes)."""

    def __init__(self, device):
        host = decode_inputs(1)
        self.host = [(p, s) for _, p, s in host]
        self.bytes = sum(p.numel() * 4 + s.numel() * 2 for p, s in self.host)
        self.copies = max(2, -(-2 * L2_BYTES // self.bytes) + 1)          # rotate through > 2x L2 of weights
        self.sets = [[(p.to(device), s.to(device)) for p, s in self.host] for _ in range(self.copies)]


def run_ring_probe(device) -> dict:
    """Diagnostic, not a benchmark line: what the bare slot ring of the decode kernels streams from HBM
    (``intent_b200_ring_probe_ms``: TMA boxes of 32 x 32 words into a per-SM ring, no arithmetic), for the two
    decode weight shapes, three ring depths, and with a fence or an atomic every 24th unit of a CTA."""
    import ctypes

    import torch

    from intent_b200.runtime import native

    probe = native.library().intent_b200_ring_probe_ms
    probe.restype = ctypes.c_double
    probe.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                      ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p]
    planes = 16                                   # 16 x 29.4 MB: larger than L2
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    scratch = torch.zeros(8192 + sms * 8192, dtype=torch.uint8, device=device)
    stream = torch.cuda.current_stream(device).cuda_stream
    modes = {0: "nothing", 1: "__threadfence()", 2: "stores + atom.acq_rel.gpu", 3: "stores + relaxed atomic",
             4: "stores + atom.release.gpu", 5: "stores + relaxed red"}
    out = {"workload": "tma_ring_probe", "planes": planes, "sync_every": 24, "unit": "GB/s", "results": []}
    for K, N in DECODE_SHAPES:
        rows = K // 8
        matrices = torch.randint(0, 2 ** 31 - 1, (planes, rows, N), dtype=torch.int32, device=device)
        nbytes = matrices.numel() * 4
        cases = [(slots, 0) for slots in (16, 32, 48)] + [(32, mode) for mode in range(1, 6)]
        for slots, mode in cases:
            best = None
            for attempt in range(6):
                ms = float(probe(matrices.data_ptr(), planes, rows, N, slots, mode, 24, scratch.data_ptr(), stream))
                if ms < 0:
                    raise RuntimeError(f"intent_b200_ring_probe_ms failed with status {int(-ms)}")
                if attempt > 0:
                    best = ms if best is None else min(best, ms)
            if int(scratch[:4].view(torch.int32).item()) != 0:
                raise RuntimeError("a bounded wait of the ring probe gave up")
            scratch.zero_()
            out["results"].append({"rows": rows, "cols": N, "slots": slots, "every_24th_unit": modes[mode],
                                   "us_per_launch": round(best * 1e3, 1), "GBps": round(nbytes / (best * 1e-3) / 1e9)})
        del matrices
    return out


def run_decode(args, rank: int, world: int, device, M: int | None = None, weights: DecodeWeights | None = None,
               steps: int | None = None, load_seconds: float | None = None):
    """One decode step = up projection + down projection.  Measured three ways, all with cold weights and
    the K timed steps captured in one CUDA graph:
      table      (headline) one launch per step: both projections as a table of the persistent table kernel;
      long table eight steps' projections (16 problems) per call: what a whole layer stack per launch gives;
      per projection  one launch per projection through the single-problem artifact (the reference's
                 call shape), programmatic dependent launch between consecutive launches."""
    import torch

    import intent_b200 as ib
    from intent_b200 import table as table_module
    from intent_b200.runtime import native

    M = args.batch if M is None else M
    steps = args.steps if steps is None else steps
    steps = max(8, steps // 8 * 8)
    load_seconds = args.load_seconds if load_seconds is None else load_seconds
    weights = weights or DecodeWeights(device)
    table = table_module.W4A16Table(group_size=GROUP, zero_point=8, act_dtype="f16", target=ib.B200Target(device.index))
    tune = native.library().intent_b200_w4a16_gemv_table_tune
    for item in filter(None, args.table_tune.split(",")):
        knob, _, number = item.partition("=")
        native.check(tune(knob.encode(), int(number)), "intent_b200_w4a16_gemv_table_tune")
    artifact = table.artifact
    host_x = [x for x, _, _ in decode_inputs(M)]
    xs = [x.to(device) for x in host_x]
    step_bytes = decode_bytes(M)
    copies = weights.copies
    warm = max(args.warmup, 3)

    def graph_time(step, hold_seconds: float):
        """Capture `steps` steps in one graph, warm it, hold the load, time one replay (ms, launches, clocks)."""
        for i in range(warm):
            step(i)
        torch.cuda.synchronize()
        stream = torch.cuda.Stream(device)
        stream.wait_stream(torch.cuda.current_stream())
        before = native.launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(steps):
                step(i)
        launches = native.launch_count() - before
        with torch.cuda.stream(stream):
            for _ in range(warm):
                graph.replay()
        stream.synchronize()
        sampler = ClockSampler(device.index)
        if rank == 0:
            sampler.start()
        with torch.cuda.stream(stream):       # keep the GPU under the same load so the clock samples mean something
            spin_until = time.perf_counter() + hold_seconds
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
        clocks = sampler.stop() if rank == 0 else None
        return reduce_max(start.elapsed_time(stop), world, device), launches, clocks

    modes = set(args.decode_modes.split(","))
    # ---- one launch per step: the two projections as one table ----------------------------------
    table_module.set_launch_overlap(True)     # static weights: a launch may request them while its predecessor drains
    step_calls = [table.prepare([(xs[j], p, s) for j, (p, s) in enumerate(group)]) for group in weights.sets]
    single_launch = all(call.single_launch for call in step_calls)

    def table_step(i: int) -> None:
        step_calls[i % copies].launch()

    elapsed_ms, launches, clocks = graph_time(table_step, load_seconds)
    for call in step_calls:
        call.check()                          # no bounded wait gave up inside the timed launches

    # ---- eight steps per call ---------------------------------------------------------------------
    long_calls = []
    for first in range(copies if "long" in modes else 0):
        problems = []
        for k in range(8):
            group = weights.sets[(first + k) % copies]
            problems += [(xs[j], p, s) for j, (p, s) in enumerate(group)]
        long_calls.append(table.prepare(problems))

    def long_step(i: int) -> None:
        if i % 8 == 0:
            long_calls[(i // 8) % len(long_calls)].launch()

    long_ms, long_launches = None, 0
    if long_calls:
        long_ms, long_launches, _ = graph_time(long_step, 0.2)
        for call in long_calls:
            call.check()
    # ---- what the slot ring alone can stream: the same long table with every unit's arithmetic skipped -------
    probe_ms, probe_launches = None, 0
    if long_calls and "probe" in modes:
        native.check(tune(b"probe", args.probe_level), "intent_b200_w4a16_gemv_table_tune")
        try:
            probe_ms, probe_launches, _ = graph_time(long_step, 0.2)
        finally:
            native.check(tune(b"probe", 0), "intent_b200_w4a16_gemv_table_tune")
    table_module.set_launch_overlap(False)
    del long_calls

    # ---- one launch per projection (single-problem artifact) ----------------------------------------
    single_ms, single_launches = None, 0
    if "projection" in modes:
        native.set_gemv_launch_overlap(True)
        table_module.set_launch_overlap(True)   # (M = 3 .. 8 run as a table of one problem inside the entry)
        single = ib.compile(ib.programs.weight_only_int4_matmul, target=ib.B200Target(device.index),
                            constexprs={"GROUP_SIZE": GROUP, "ZERO_POINT": 8, "ACT_DTYPE": "f16"})
        calls = [[single.prepare(xs[j], p, s) for j, (p, s) in enumerate(group)] for group in weights.sets]

        def projection_step(i: int) -> None:
            for call in calls[i % copies]:
                call.launch()

        single_ms, single_launches, _ = graph_time(projection_step, 0.2)
        for group in calls:
            for call in group:
                call.check()
        native.set_gemv_launch_overlap(False)
        table_module.set_launch_overlap(False)
        del calls

    # ---- end to end: host activations in, results back, one table launch per step --------------------
    # The step's activations sit in ONE pinned buffer and ONE device buffer (the problems' x are views of it),
    # its results likewise: one host-to-device and one device-to-host copy per step instead of one per projection.
    in_sizes = [x.numel() for x in host_x]
    out_sizes = [M * N for _, N in DECODE_SHAPES]
    pinned_in = torch.cat([x.reshape(-1) for x in host_x]).pin_memory()
    pinned_out = torch.empty((sum(out_sizes),), dtype=torch.float16).pin_memory()
    device_in = torch.empty_like(pinned_in, device=device)
    device_out = torch.empty((sum(out_sizes),), dtype=torch.float16, device=device)
    x_views = [v.view(M, K) for v, (K, _) in zip(device_in.split(in_sizes), DECODE_SHAPES)]
    y_views = [v.view(M, N) for v, (_, N) in zip(device_out.split(out_sizes), DECODE_SHAPES)]
    e2e_calls = [table.prepare([(x_views[j], p, s) for j, (p, s) in enumerate(group)], outputs=y_views)
                 for group in weights.sets]

    def e2e_step(i: int) -> None:
        # (binding the three as one CUDA graph was measured slower: 77 against 64 us per step at M = 8)
        device_in.copy_(pinned_in, non_blocking=True)
        e2e_calls[i % copies].launch()
        pinned_out.copy_(device_out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for i in range(warm):
        e2e_step(i)
    barrier(world)
    torch.cuda.synchronize()
    e2e_steps = max(1, min(steps, 200))
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        e2e_step(i)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    e2e_s = reduce_max(e2e_s, world, device)

    # The headline is a decode step served the fastest way the library offers for it: both projections in one
    # table launch, or one launch per projection; the line says which.
    table_ms, table_launches = elapsed_ms, launches
    best = "table_one_launch_per_step"
    if single_ms is not None and single_ms < elapsed_ms:
        elapsed_ms, launches, best = single_ms, single_launches, "one_launch_per_projection"
        single_launch = False
    ms_per_step = elapsed_ms / steps
    value = world * step_bytes / (ms_per_step * 1e-3) / 1e9
    peaks = measured_peaks()
    per_launch_bytes = step_bytes * steps / max(1, launches)
    per_launch_s = elapsed_ms * 1e-3 / max(1, launches)
    achieved = per_launch_bytes / per_launch_s / 1e9
    config = workload_config("decode", world, M)
    notes = {"l2": f"weights rotated through {copies} resident copies ({copies * weights.bytes >> 20} MiB > L2)",
             "timing": "K steps in one CUDA graph, CUDA events on the replay stream",
             "launch": ("one launch per step: both projections as a table of intent_b200.table.W4A16Table "
                        "(persistent kernel, the second projection's weights stream while the first is reduced)"
                        if single_launch else "one launch per projection through the single-problem artifact") +
                       "; programmatic dependent launch between consecutive launches (static weights)"}

    def mode(ms_total, n_launches):
        if ms_total is None:
            return None
        per_step = ms_total / steps
        return {"ms_per_step": round(per_step, 6), "GBps": round(step_bytes / (per_step * 1e-3) / 1e9, 1),
                "frac_of_hbm_peak": round(step_bytes / (per_step * 1e-3) / 1e9 / peaks["hbm_gbs"], 4),
                "launches_per_step": round(n_launches / steps, 3),
                "us_per_projection": round(per_step * 1e3 / len(DECODE_SHAPES), 3)}

    line = {
        "metric": "w4a16_decode_weight_GBps", "value": round(value, 2), "unit": "GB/s",
        "n_gpus": world, "steps": steps, "warmup": warm,
        "ms_per_step": round(ms_per_step, 6), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic", "config": config, "notes": notes,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4),
                     # ncu capture of the M = 1 step (one table launch of both projections, one GPU):
                     # dram__bytes_read + dram__bytes_write = 60,649,984 + 103,936 (profiles/w4a16_ride_kernel_decode_gemv.md)
                     "traffic": 60753920 if (M == 1 and best == "table_one_launch_per_step") else None,
                     "traffic_note": ("ncu capture of the M = 1 table launch on one GPU (every rank runs the same "
                                      "launch)" if (M == 1 and best == "table_one_launch_per_step")
                                      else "captured for the M = 1 table launch only; see profiles/"),
                     "peak_source": peaks["source"], "frac_of_nominal_8000": round(achieved / 8000.0, 4),
                     "algorithmic_bytes_per_launch": per_launch_bytes,
                     "kernel": "w4a16_ride_kernel" if single_launch or M >= 2 else "w4a16_stream_kernel",
                     "us_per_launch": round(per_launch_s * 1e6, 3),
                     "us_per_projection": round(ms_per_step * 1e3 / len(DECODE_SHAPES), 3)},
        "headline_mode": best,
        "modes": {"table_one_launch_per_step": mode(table_ms, table_launches),
                  "table_eight_steps_per_call": mode(long_ms, long_launches),
                  "stream_only_probe_eight_steps_per_call": mode(probe_ms, probe_launches),
                  "one_launch_per_projection": mode(single_ms, single_launches)},
        "e2e": {"value": round(world * step_bytes / (e2e_s / e2e_steps) / 1e9, 2), "unit": "GB/s",
                "h2d_bytes_per_step": pinned_in.numel() * 2,
                "d2h_bytes_per_step": pinned_out.numel() * 2,
                "ms_per_step": round(e2e_s / e2e_steps * 1e3, 6), "steps": e2e_steps},
        "gpu_launches": int(launches),
        "clocks": clocks,
    }
    # the step's results for the first weight copy (the oracle's weights), for the parity check of the CPU leg
    step_calls[0].launch()
    torch.cuda.synchronize()
    line["_results"] = [y.cpu() for y in step_calls[0].results()]
    return line


# ---------------------------------------------------------------------------------------
# tensor-core workloads: W4A16 prefill (configs[2]), W8A8 (configs[3]), MoE (configs[4])
# ---------------------------------------------------------------------------------------
def run_prefill(args, rank: int, world: int, device):
    import torch

    import intent_b200 as ib
    from intent_b200.distributed import ColumnShardedRows, column_shard

    M, K, N = PREFILL["M"], PREFILL["K"], PREFILL["N"]
    x, packed, scales = ib.workloads.w4a16_inputs(M, K, N, dtype=torch.bfloat16, group_size=GROUP, seed=0)
    cols = column_shard(N, world, rank)
    # --prelayout: the artifact keeps a tiled copy of the static weight (made once, outside the timed region).
    # Measured slower than reading the reference layout directly (about 10 % on this shape), so it is off here.
    artifact = ib.compile(ib.programs.weight_only_int4_matmul, target=ib.B200Target(device.index),
                          constexprs={"GROUP_SIZE": GROUP, "ZERO_POINT": 8, "ACT_DTYPE": "bf16",
                                      "PRELAYOUT": args.prelayout})
    xd = x.to(device)
    pd, sd = packed[:, cols].contiguous().to(device), scales[:, cols].contiguous().to(device)
    call = artifact.prepare(xd, pd, sd)
    elapsed_ms, clocks, launches = timed_steps(call.launch, args.steps, args.warmup, world, device, rank,
                                               args.load_seconds)
    call.check()
    # end to end: rows of X from pinned host memory (each rank uploads its own rows, pieces are all-gathered
    # over NVLink), this rank's block of Y back into pinned host memory, copies overlapped with the GEMM
    pinned_x = x.pin_memory()
    n_local = cols.stop - cols.start
    pinned_y = torch.empty((M, n_local), dtype=torch.bfloat16).pin_memory()
    pipeline = ColumnShardedRows(artifact, (pd, sd), rows=M, width=K, n_local=n_local, in_dtype=torch.bfloat16,
                                 out_dtype=torch.bfloat16, device=device, chunks=args.e2e_chunks)

    def e2e_step():
        pipeline.run(pinned_x, pinned_y)
        torch.cuda.synchronize()

    e2e_steps = max(1, min(args.steps, 20))
    e2e_s = timed_e2e(e2e_step, e2e_steps, args.warmup, world, device)
    artifact.check()
    flops = 2.0 * M * K * N
    ms = elapsed_ms / args.steps
    peaks = measured_peaks()
    per_launch_flops = flops / world
    achieved = per_launch_flops / (ms * 1e-3) / 1e12
    config = workload_config("prefill", world)
    weight_note = ("PRELAYOUT: the artifact keeps a tiled copy of the static weight (made once, before the timed "
                   "region)" if args.prelayout else "reference [K/8, N] layout read directly")
    line = {
        "metric": "w4a16_prefill_TFLOPs", "value": round(flops / (ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 5),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config, "notes": {"timing": "CUDA events on the launch stream around K launches",
                                    "weight": weight_note},
        "roofline": {"bound": "tensor", "achieved": round(achieved, 1), "peak": peaks["bf16_tflops"],
                     "unit": "TFLOP/s", "frac": round(achieved / peaks["bf16_tflops"], 4),
                     "traffic": ncu_traffic("prefill", world),
                     "traffic_note": "ncu capture of the 1-GPU launch" if world == 1 else
                                     "not captured for a column shard (it does not scale with the shard: X is read whole)",
                     "peak_source": peaks["source"] + " (burst cuBLAS bf16)",
                     "frac_of_sustained": round(achieved / peaks["bf16_tflops_sustained"], 4),
                     "frac_of_nominal_2250": round(achieved / 2250.0, 4),
                     "algorithmic_flops_per_launch": per_launch_flops, "kernel": "w4a16_gemm_pair_kernel",
                     "ms_per_launch": round(ms, 5)},
        "e2e": {"value": round(flops / (e2e_s / e2e_steps) / 1e12, 2), "unit": "TFLOP/s",
                "h2d_bytes_per_step": pipeline.h2d_bytes, "d2h_bytes_per_step": pipeline.d2h_bytes,
                "ms_per_step": round(e2e_s / e2e_steps * 1e3, 4), "steps": e2e_steps,
                "path": f"intent_b200.distributed.ColumnShardedRows: pieces of {pipeline.sizes} "
                        "rows per rank, upload / " + ("all-gather over NVLink / " if world > 1 else "") +
                        "GEMM / download overlapped on three streams"},
        "gpu_launches": int(launches), "clocks": clocks,
    }
    return line, {"y": pinned_y, "inputs": (x, packed, scales)}


def measure_int8_peak(device):
    """cuBLASLt int8 GEMM through torch._int_mm at 8192^3, best of 10: the yardstick the int8 roofline is
    reported against (never on the product path).  None when torch cannot run it."""
    import torch

    try:
        a = torch.randint(-127, 128, (8192, 8192), dtype=torch.int8, device=device)
        b = torch.randint(-127, 128, (8192, 8192), dtype=torch.int8, device=device).t().contiguous().t()
        for _ in range(3):
            torch._int_mm(a, b)
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(10):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            torch._int_mm(a, b)
            stop.record()
            torch.cuda.synchronize()
            best = min(best, start.elapsed_time(stop))
        return 2.0 * 8192 ** 3 / (best * 1e-3) / 1e12
    except Exception:
        return None


def run_w8a8(args, rank: int, world: int, device):
    import torch

    import intent_b200 as ib
    from intent_b200.distributed import ColumnShardedRows, RowAligned, column_shard

    M, K, N = W8A8["M"], W8A8["K"], W8A8["N"]
    a, b, sa, sb = ib.workloads.w8a8_inputs(M, K, N, seed=0)
    cols = column_shard(N, world, rank)
    artifact = ib.compile(ib.programs.w8a8_gemm, target=ib.B200Target(device.index))
    ad, sad = a.to(device), sa.to(device)
    bd, sbd = b[:, cols].contiguous().to(device), sb[cols].contiguous().to(device)
    call = artifact.prepare(ad, bd, sad, sbd)
    elapsed_ms, clocks, launches = timed_steps(call.launch, args.steps, args.warmup, world, device, rank,
                                               args.load_seconds)
    call.check()
    pinned_a = a.pin_memory()
    n_local = cols.stop - cols.start
    pinned_y = torch.empty((M, n_local), dtype=torch.bfloat16).pin_memory()
    pipeline = ColumnShardedRows(artifact, (bd, RowAligned(sad), sbd), rows=M, width=K, n_local=n_local,
                                 in_dtype=torch.int8, out_dtype=torch.bfloat16, device=device,
                                 chunks=args.e2e_chunks)

    def e2e_step():
        pipeline.run(pinned_a, pinned_y)
        torch.cuda.synchronize()

    e2e_steps = max(1, min(args.steps, 20))
    e2e_s = timed_e2e(e2e_step, e2e_steps, args.warmup, world, device)
    artifact.check()
    ops = 2.0 * M * K * N
    ms = elapsed_ms / args.steps
    peaks = measured_peaks()
    achieved = ops / world / (ms * 1e-3) / 1e12
    measured = measure_int8_peak(device)
    int8_peak = measured if measured else 2.0 * peaks["bf16_tflops"]
    config = workload_config("w8a8", world)
    line = {
        "metric": "w8a8_gemm_TOPs", "value": round(ops / (ms * 1e-3) / 1e12, 2), "unit": "TOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 5),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": config,
        "roofline": {"bound": "tensor", "achieved": round(achieved, 1), "peak": round(int8_peak, 1), "unit": "TOP/s",
                     "frac": round(achieved / int8_peak, 4), "traffic": ncu_traffic("w8a8", world),
                     "traffic_note": "ncu capture of the 1-GPU launch" if world == 1 else
                                     "not captured for a column shard",
                     "peak_source": "torch._int_mm (cuBLASLt int8) 8192^3, best of 10, measured in this run"
                                    if measured else "2 x measured bf16 burst (torch._int_mm could not run)",
                     "frac_of_2x_bf16_burst": round(achieved / (2.0 * peaks["bf16_tflops"]), 4),
                     "frac_of_nominal_4500": round(achieved / 4500.0, 4), "kernel": "i8_gemm_kernel",
                     "ms_per_launch": round(ms, 5)},
        "e2e": {"value": round(ops / (e2e_s / e2e_steps) / 1e12, 2), "unit": "TOP/s",
                "h2d_bytes_per_step": pipeline.h2d_bytes, "d2h_bytes_per_step": pipeline.d2h_bytes,
                "ms_per_step": round(e2e_s / e2e_steps * 1e3, 4), "steps": e2e_steps,
                "path": f"intent_b200.distributed.ColumnShardedRows, {pipeline.chunks} pieces per rank"},
        "gpu_launches": int(launches), "clocks": clocks,
    }
    return line, {"y": pinned_y, "inputs": (a, b, sa, sb)}


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
    config = workload_config("grouped", world)
    notes = {"published": f"{GROUPED_PUBLISHED_MS} ms = {published_tflops:.0f} TFLOP/s on an RTX 5090D "
                          "(the reference's generated Triton kernel; other hardware)"}
    line = {
        "metric": "ragged_grouped_gemm_TFLOPs", "value": round(flops / (ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 5),
        "higher_is_better": True, "scaling": "strong",
        "vs_baseline": round(flops / (ms * 1e-3) / 1e12 / published_tflops, 3) if world == 1 else None,
        "dtype": "f16", "data": "synthetic", "config": config, "notes": notes,
        "roofline": {"bound": "tensor", "achieved": round(achieved, 1), "peak": peaks["bf16_tflops"],
                     "unit": "TFLOP/s", "frac": round(achieved / peaks["bf16_tflops"], 4),
                     "traffic": ncu_traffic("grouped", world),
                     "peak_source": peaks["source"] + " (burst cuBLAS bf16)",
                     "frac_of_sustained": round(achieved / peaks["bf16_tflops_sustained"], 4),
                     "algorithmic_flops_per_launch": flops / world, "kernel": "grouped_gemm16_kernel",
                     "ms_per_launch": round(ms, 5)},
        "e2e": {"value": round(flops / (e2e_s / e2e_steps) / 1e12, 2), "unit": "TFLOP/s",
                "h2d_bytes_per_step": R * K * 2, "d2h_bytes_per_step": R * n_local * 2,
                "ms_per_step": round(e2e_s / e2e_steps * 1e3, 4), "steps": e2e_steps},
        "gpu_launches": int(launches), "clocks": clocks,
    }
    return line, {}


def phase_times(launch, phases, steps: int, world: int, device):
    """Device time of every phase of a step, averaged over `steps` marked launches (max over ranks)."""
    import torch

    totals = [0.0] * len(phases)
    for _ in range(steps):
        marks = []
        barrier(world)              # the ranks start a marked step together, so a sync phase shows only the wait
        launch(marks=marks)
        torch.cuda.synchronize()
        for i in range(len(phases)):
            totals[i] += marks[i].elapsed_time(marks[i + 1])
    return {name: round(reduce_max(total / steps, world, device) * 1e3, 2) for name, total in zip(phases, totals)}


def run_moe(args, rank: int, world: int, device):
    import torch

    import intent_b200 as ib
    from intent_b200.moe import MoEW4A16FFN

    cfg = MOE
    tokens, hidden, experts, inter = cfg["tokens"], cfg["hidden"], cfg["experts"], cfg["intermediate"]
    if experts % world or tokens % world:
        raise SystemExit("moe workload needs the gpu count to divide 64 experts and 16384 tokens")
    t_local, e_local = tokens // world, experts // world
    all_logits, all_x = ib.workloads.moe_activations(tokens, hidden, experts, dtype=torch.bfloat16, seed=0)
    rows = slice(rank * t_local, (rank + 1) * t_local)
    logits, x = all_logits[rows].contiguous(), all_x[rows].contiguous()
    host_weights = ib.workloads.moe_expert_weights(rank * e_local, e_local, hidden, inter, dtype=torch.bfloat16,
                                                   seed=0)
    weights = [w.to(device) for w in host_weights]
    bound = {}
    if world == 1:
        ffn = MoEW4A16FFN(tokens=tokens, hidden=hidden, intermediate=inter, experts=experts,
                          block_size=args.moe_block, target=ib.B200Target(device.index),
                          prelayout=args.prelayout)

        def forward(lg, xx):
            ids, w = ffn.route(lg)
            return ffn(xx, ids, w, *weights)

        def prepare(lg, xx):
            router = ffn.router.prepare(lg)
            ids, w = router.result()
            y = torch.empty((xx.shape[0], hidden), dtype=torch.float32, device=device)
            chain = ffn.prepare(xx, ids, w, *weights, y)
            bound.update(chain=chain, router=router, phases=("router",) + chain.PHASES)

            def launch(marks=None):
                if marks is not None:
                    event = torch.cuda.Event(enable_timing=True)
                    event.record()
                    marks.append(event)
                router.launch()
                return chain.launch(marks=marks)

            bound["marked"] = launch
            if args.moe_eager:
                return launch
            # the bound step allocates nothing and reads nothing back: replayed as one CUDA graph, which takes
            # the host's launch gaps between its dozen small kernels out of the step
            for _ in range(3):
                launch()
            torch.cuda.synchronize()
            from intent_b200.runtime import native

            graph = torch.cuda.CUDAGraph()
            before = native.launch_count()
            with torch.cuda.graph(graph):
                launch()
            bound["graph"], bound["launches_per_replay"] = graph, native.launch_count() - before
            return graph.replay
    elif args.moe_exchange == "peer":
        from intent_b200.peer import PeerExpertParallelMoE

        # rows go straight into the owners' buffers over NVLink and results are read straight back:
        # no collective on the data path, worst-case buffers (no overflow case)
        ep = PeerExpertParallelMoE(tokens=t_local, hidden=hidden, intermediate=inter, experts=experts,
                                   block_rows=args.moe_block, target=ib.B200Target(device.index))

        def prepare(lg, xx):
            call = ep.prepare(lg, xx, *weights)
            bound.update(logits=lg, x=xx, call=call, phases=call.PHASES, marked=call.launch)
            if args.moe_eager:
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
    launch = prepare(lgd, xd)
    elapsed_ms, clocks, launches = timed_steps(launch, args.steps, args.warmup, world, device,
                                               rank, args.load_seconds)
    if "launches_per_replay" in bound:
        launches = bound["launches_per_replay"] * args.steps      # kernels inside the replayed graph
    phases = None
    if "phases" in bound:
        marked = bound.get("marked", launch)
        phases = phase_times(marked, bound["phases"], 5, world, device)
    pinned_l, pinned_x = logits.pin_memory(), x.pin_memory()
    pinned_y = torch.empty((t_local, hidden), dtype=torch.float32).pin_memory()

    pipelined = None
    if world == 1 and args.moe_e2e_pieces > 1:
        from intent_b200.moe import HostPipelinedFFN

        # host tensors in, host result out: pieces of the batch upload, run and download on three streams
        pipelined = HostPipelinedFFN(tokens=tokens, hidden=hidden, intermediate=inter, experts=experts,
                                     chunks=args.moe_e2e_pieces, block_size=args.moe_block,
                                     target=ib.B200Target(device.index)).bind(*weights)

    def e2e_step():
        if pipelined is not None:
            pipelined.run(pinned_l, pinned_x, pinned_y)
            return
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
    from intent_b200.runtime import native

    if native.library().intent_b200_w4a16_gemm_device_status() != 0:
        raise RuntimeError("a bounded wait of the grouped contraction gave up during the MoE benchmark")
    flops = moe_flops()
    ms = elapsed_ms / args.steps
    peaks = measured_peaks()
    achieved = flops / world / (ms * 1e-3) / 1e12
    config = workload_config("moe", world)
    notes = {"expert_block_rows": args.moe_block}
    if world == 1:
        notes["launch"] = ("eager launches of the bound step" if args.moe_eager else
                           "the bound step (router, alignment, gather, two grouped contractions) replayed as one CUDA graph")
    if world > 1:
        notes["exchange"] = ("rows written into the owners' buffers and results read back over NVLink peer memory; "
                              "three sync points per step as flag posts and bounded flag waits over peer memory, no "
                              "collective call" + ("" if args.moe_eager else ", replayed as one CUDA graph")
                              if args.moe_exchange == "peer" else
                              "NCCL all-to-all each way, fixed-capacity exchange (factor 1.5)")
    split = None
    if phases:
        routes = tokens * cfg["top_k"]
        up_flops = routes * 2.0 * hidden * 2 * inter / world
        down_flops = routes * 2.0 * inter * hidden / world
        down_us = phases.get("down", phases.get("down_combine"))
        split = {"phase_us": phases,
                 "router_align_us": round(sum(v for k, v in phases.items() if k in ("router", "align", "route")), 2),
                 "up_gate_TFLOPs": round(up_flops / (phases["up_gate"] * 1e-6) / 1e12, 1),
                 "down_TFLOPs": round(down_flops / (down_us * 1e-6) / 1e12, 1),
                 "note": "per-phase device times from event marks inside 5 extra steps (max over ranks); the "
                         "sync phases include waiting for the slowest rank"}
        if world > 1 and "dispatch" in phases:
            remote = (world - 1) / world
            sent = routes / world * hidden * 2 * remote            # bf16 rows leaving this GPU
            fetched = routes / world * hidden * 4 * remote         # f32 result rows read from peers
            split["dispatch_GBps"] = round(sent / (phases["dispatch"] * 1e-6) / 1e9, 1)
            split["combine_GBps"] = round(fetched / (phases["combine"] * 1e-6) / 1e9, 1)
            split["nvlink_peak_GBps_per_direction"] = 900.0
    line = {
        "metric": "moe_w4a16_ffn_TFLOPs", "value": round(flops / (ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 5),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config, "notes": notes,
        "roofline": {"bound": "tensor", "achieved": round(achieved, 1), "peak": peaks["bf16_tflops"],
                     "unit": "TFLOP/s", "frac": round(achieved / peaks["bf16_tflops"], 4),
                     "traffic": ncu_traffic("moe", world),
                     "traffic_note": "a step is several kernels; per-kernel DRAM traffic is in "
                                     "profiles/moe_step_launch_list.md, not one figure",
                     "peak_source": peaks["source"] + " (burst cuBLAS bf16); whole step, not one kernel",
                     "frac_of_sustained": round(achieved / peaks["bf16_tflops_sustained"], 4),
                     "kernel": "w4a16_gemm_kernel (grouped modes)"},
        "kernels": split,
        "e2e": {"value": round(flops / (e2e_s / e2e_steps) / 1e12, 2), "unit": "TFLOP/s",
                "h2d_bytes_per_step": t_local * (64 * 4 + hidden * 2), "d2h_bytes_per_step": t_local * hidden * 4,
                "ms_per_step": round(e2e_s / e2e_steps * 1e3, 4), "steps": e2e_steps},
        "gpu_launches": int(launches), "clocks": clocks,
    }
    return line, {"y": pinned_y, "inputs": (all_logits, all_x, host_weights)}


# ---------------------------------------------------------------------------------------
# CPU arm: the reference's CPU implementation of the path (restated in oracle/), all host threads.
# Every function times whole steps of the FULL configuration when one step fits the budget, otherwise the
# largest power-of-two fraction of the rows / tokens that does (never less than 1/8), and says which.
# Returns a dict: value, unit, cores, sample, ms_per_step, steps and (optionally) `result`, the output of
# the last step, which the caller may compare with the GPU's.
# ---------------------------------------------------------------------------------------
def _cpu_threads() -> int:
    import torch

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    return cores


def _bounded(run_fraction, steps: int, warmup: int, budget_s: float):
    """run_fraction(divisor) runs one step on 1/divisor of the rows.  Picks the smallest divisor in
    {1, 2, 4, 8} whose predicted run (warm-up + steps) fits the budget, reducing the step count first."""
    t0 = time.perf_counter()
    result = run_fraction(8)
    eighth = time.perf_counter() - t0
    t0 = time.perf_counter()
    result = run_fraction(4)
    quarter = time.perf_counter() - t0
    # cost model fixed + slope * fraction (the dequantisation of the weight does not shrink with the rows)
    slope = max(0.0, (quarter - eighth) * 8.0)
    fixed = max(0.0, eighth - slope / 8.0)
    predicted = lambda d: fixed + slope / d                          # noqa: E731
    divisor = 1
    while divisor < 8 and predicted(divisor) * 2 > budget_s:         # at least one warm-up and one step
        divisor *= 2
    one = predicted(divisor)
    steps = max(1, min(steps, int(budget_s / max(one, 1e-4)) - warmup))
    warmup = min(warmup, max(0, int(budget_s / max(one, 1e-4)) - steps))
    for _ in range(warmup):
        run_fraction(divisor)
    t0 = time.perf_counter()
    for _ in range(steps):
        result = run_fraction(divisor)
    seconds = (time.perf_counter() - t0) / steps
    return divisor, steps, seconds, result


def cpu_decode(M: int, steps: int, warmup: int, budget_s: float, inputs=None):
    import oracle

    cores = _cpu_threads()
    # the activations of this batch size against the weights the GPU arm streams (those of decode_inputs(1))
    host = [(x, p, s) for (x, _, _), (_, p, s) in zip(decode_inputs(M), decode_inputs(1))]

    def step(divisor: int):
        out = []
        for x, p, s in host:
            n = p.shape[1] // divisor
            out.append(oracle.weight_only_int4_matmul(x, p[:, :n].contiguous(), s[:, :n].contiguous(),
                                                      group_size=GROUP, zero_point=8))
        return out

    divisor, steps, seconds, result = _bounded(step, steps, warmup, budget_s)
    what = "the full decode step" if divisor == 1 else f"the first 1/{divisor} of the output columns of the decode step"
    return {"value": decode_bytes(M) / divisor / seconds / 1e9, "unit": "GB/s", "cores": cores,
            "sample": f"{steps} steps of {what} (M={M}, both projections; the weight is dequantised inside every "
                      f"call, as in the reference's torch implementation), torch CPU, {cores} threads",
            "ms_per_step": seconds * 1e3, "steps": steps, "fraction": 1.0 / divisor,
            "result": result if divisor == 1 else None}


def cpu_prefill(steps: int, warmup: int, budget_s: float, inputs=None):
    import torch

    import oracle
    from intent_b200 import workloads

    cores = _cpu_threads()
    M, K, N = PREFILL["M"], PREFILL["K"], PREFILL["N"]
    x, p, s = inputs or workloads.w4a16_inputs(M, K, N, dtype=torch.bfloat16, group_size=GROUP, seed=0)

    def step(divisor: int):
        return oracle.weight_only_int4_matmul(x[: M // divisor], p, s, group_size=GROUP, zero_point=8)

    divisor, steps, seconds, result = _bounded(step, steps, warmup, budget_s)
    rows = M // divisor
    what = "the full 8192 x 8192 x 8192 problem" if divisor == 1 else \
        f"the first {rows} of the 8192 rows of X (a 1/{divisor} slice; throughput per unit of work)"
    return {"value": 2.0 * rows * K * N / seconds / 1e12, "unit": "TFLOP/s", "cores": cores,
            "sample": f"{steps} steps of {what} against the full int4 weight (dequantised inside every call, as in "
                      f"the reference's torch implementation), torch CPU f32, {cores} threads",
            "ms_per_step": seconds * 1e3, "steps": steps, "fraction": 1.0 / divisor, "result": result}


def cpu_w8a8(steps: int, warmup: int, budget_s: float, inputs=None):
    import oracle
    from intent_b200 import workloads

    cores = _cpu_threads()
    M, K, N = W8A8["M"], W8A8["K"], W8A8["N"]
    a, b, sa, sb = inputs or workloads.w8a8_inputs(M, K, N, seed=0)

    def step(divisor: int):
        return oracle.w8a8_scaled_gemm(a[: M // divisor], b, sa[: M // divisor], sb)[0]

    divisor, steps, seconds, result = _bounded(step, steps, warmup, budget_s)
    rows = M // divisor
    what = "the full 4096 x 8192 x 8192 problem" if divisor == 1 else f"the first {rows} of the 4096 rows of A"
    return {"value": 2.0 * rows * K * N / seconds / 1e12, "unit": "TOP/s", "cores": cores,
            "sample": f"{steps} steps of {what}, torch CPU integer matmul + scaled epilogue, {cores} threads",
            "ms_per_step": seconds * 1e3, "steps": steps, "fraction": 1.0 / divisor, "result": result}


def cpu_moe(steps: int, warmup: int, budget_s: float, inputs=None):
    import torch

    import oracle
    from intent_b200 import workloads

    cores = _cpu_threads()
    cfg = MOE
    tokens, hidden, experts, inter = cfg["tokens"], cfg["hidden"], cfg["experts"], cfg["intermediate"]
    if inputs is None:
        logits, x = workloads.moe_activations(tokens, hidden, experts, dtype=torch.bfloat16, seed=0)
        weights = workloads.moe_expert_weights(0, experts, hidden, inter, dtype=torch.bfloat16, seed=0)
    else:
        logits, x, weights = inputs

    def step(divisor: int):
        n = tokens // divisor
        ids, w = oracle.moe_route_top2(logits[:n])
        return oracle.moe_w4a16_swiglu_ffn(x[:n], ids, w, *weights)

    divisor, steps, seconds, result = _bounded(step, steps, warmup, budget_s)
    n = tokens // divisor
    what = "the full 16384 tokens" if divisor == 1 else \
        f"the first {n} of the 16384 tokens (a 1/{divisor} slice; all 64 experts are still dequantised every step)"
    flops = moe_flops() / divisor
    return {"value": flops / seconds / 1e12, "unit": "TFLOP/s", "cores": cores,
            "sample": f"{steps} steps of {what} over 64 experts (H=4096, I=1408, top-2; router, per-expert "
                      f"dequantisation, SiLU gate, weighted combine), torch CPU f32, {cores} threads",
            "ms_per_step": seconds * 1e3, "steps": steps, "fraction": 1.0 / divisor, "result": result}


def cpu_grouped(steps: int, warmup: int, budget_s: float, inputs=None):
    import torch

    import oracle

    cores = _cpu_threads()
    G, rows_per_group, K, N = (GROUPED[k] for k in ("groups", "rows_per_group", "K", "N"))
    gen = torch.Generator().manual_seed(0)
    x = (torch.randn((G * rows_per_group, K), generator=gen) * 0.5).half()
    w = torch.stack([(torch.randn((K, N), generator=gen) / K ** 0.5).half() for _ in range(G)])

    def step(divisor: int):
        rows = rows_per_group // divisor                 # the same fraction of every group's rows
        index = torch.cat([torch.arange(g * rows_per_group, g * rows_per_group + rows) for g in range(G)])
        offsets = torch.arange(G + 1, dtype=torch.int32) * rows
        return oracle.ragged_grouped_gemm(x[index], offsets, w)

    divisor, steps, seconds, result = _bounded(step, steps, warmup, budget_s)
    rows = rows_per_group // divisor
    what = "the full case" if divisor == 1 else f"{rows} of the 1024 rows of each of the 8 groups"
    return {"value": 2.0 * rows * G * K * N / seconds / 1e12, "unit": "TFLOP/s", "cores": cores,
            "sample": f"{steps} steps of {what}, full K and N, torch CPU f32 matmul per group, {cores} threads",
            "ms_per_step": seconds * 1e3, "steps": steps, "fraction": 1.0 / divisor, "result": None}


CPU_LEGS = {"prefill": cpu_prefill, "w8a8": cpu_w8a8, "moe": cpu_moe, "grouped": cpu_grouped}


def cpu_workload(workload: str, batch: int, steps: int, warmup: int, budget_s: float, inputs=None) -> dict:
    if workload == "decode":
        return cpu_decode(batch, steps, warmup, budget_s)
    return CPU_LEGS[workload](steps, warmup, budget_s, inputs)


def cpu_baseline_object(leg: dict) -> dict:
    return {"value": round(leg["value"], 5), "unit": leg["unit"], "cores": leg["cores"], "kind": "port",
            "sample": leg["sample"], "ms_per_step": round(leg["ms_per_step"], 3)}


def parity_against_cpu(leg: dict, gpu_result) -> dict | None:
    """The CPU leg's last result is the oracle's answer for the rows it covered: compare the GPU's result on
    those rows (max|y - ref| / max|ref|; the benchmark tolerance is 2e-2)."""
    reference = leg.get("result")
    if reference is None or gpu_result is None:
        return None
    if isinstance(reference, (list, tuple)):      # several outputs per step (the decode step's projections)
        parts = [parity_against_cpu({"result": r}, g) for r, g in zip(reference, gpu_result)]
        worst = max(parts, key=lambda part: part["max_abs_rel"])
        return dict(worst, outputs_compared=len(parts), ok=all(part["ok"] for part in parts))
    rows = reference.shape[0]
    got = gpu_result[:rows].float()
    scale = reference.float().abs().max().item() or 1.0
    error = (got - reference.float()).abs().max().item() / scale
    return {"rows_compared": int(rows), "max_abs_rel": float(f"{error:.3e}"), "tolerance": 2e-2,
            "ok": bool(error <= 2e-2)}


def run_reference(args, rank: int, world: int):
    """The reference arm: the CPU implementation on the host cores, same config / metric / unit."""
    if rank != 0:
        return None
    metric, unit, scaling, _ = WORKLOAD_META[args.workload]
    # the driver passes its own --steps; a step of the full configuration takes seconds on the host, so
    # the budget decides how many are timed (the count is in the line)
    leg = cpu_workload(args.workload, args.batch, args.steps, max(min(args.warmup, 1), 1), budget_s=args.cpu_budget)
    value = leg["value"]
    return {
        "impl": "reference", "metric": metric, "value": round(value, 5), "unit": unit,
        "n_gpus": world, "steps": leg["steps"], "warmup": 1, "ms_per_step": round(leg["ms_per_step"], 4),
        "higher_is_better": True, "scaling": scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.workload, world, args.batch),
        "cpu_baseline": cpu_baseline_object(leg),
        "e2e": {"value": round(value, 5), "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


# ---------------------------------------------------------------------------------------
# Same-box Triton column (informational): what a Triton lowering of W4A16 of the shape the reference's
# provider emits does on this GPU.  The reference serialises the contraction as a `tl.dot` of the activation
# tile with a weight tile that is unpacked and scaled per K tile inside the loop
# (lib/Target/Triton/Serialization/Serializer.cpp:393-399), and picks tile rows
# (ownership_m, ownership_n, reduction, NUM_WARPS, NUM_STAGES) from
# lib/Target/Triton/Transforms/Configuration/TuningProfiles.json; unit-M problems use the multiply-and-sum
# expansion instead of tl.dot (lib/Target/Triton/Transforms/Value/Values.cpp:99-108).  The kernels below are
# a hand restatement of that shape, with a few of those tile rows as autotune candidates.  Nothing in
# intent_b200/ imports Triton; this arm exists only to print a comparison line.
# ---------------------------------------------------------------------------------------
def _triton_kernels():
    import triton
    import triton.language as tl

    dense_rows = [(128, 256, 64, 8, 3), (128, 256, 128, 8, 3), (256, 128, 128, 8, 3), (128, 128, 128, 4, 4),
                  (128, 128, 32, 4, 4), (64, 256, 32, 4, 4)]

    @triton.autotune(configs=[triton.Config({"BM": m, "BN": n, "BK": k}, num_warps=w, num_stages=st)
                              for m, n, k, w, st in dense_rows], key=["M", "N", "K"])
    @triton.jit
    def w4a16_dot(x_ptr, p_ptr, s_ptr, y_ptr, M, N, K, GROUP: tl.constexpr, ZP: tl.constexpr,
                  BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr):
        pid_m, pid_n = tl.program_id(0), tl.program_id(1)
        rm = pid_m * BM + tl.arange(0, BM)
        rn = pid_n * BN + tl.arange(0, BN)
        rk = tl.arange(0, BK)
        acc = tl.zeros((BM, BN), dtype=tl.float32)
        for k0 in range(0, K, BK):
            k = k0 + rk
            x = tl.load(x_ptr + rm[:, None] * K + k[None, :], mask=(rm[:, None] < M) & (k[None, :] < K), other=0.0)
            word = tl.load(p_ptr + (k[:, None] // 8) * N + rn[None, :],
                           mask=(k[:, None] < K) & (rn[None, :] < N), other=0)
            q = ((word >> ((k[:, None] % 8) * 4)) & 15) - ZP
            scale = tl.load(s_ptr + (k[:, None] // GROUP) * N + rn[None, :],
                            mask=(k[:, None] < K) & (rn[None, :] < N), other=0.0)
            w = q.to(scale.dtype) * scale                      # rounded to the activation type, as the kernel body does
            acc = tl.dot(x, w, acc)
        tl.store(y_ptr + rm[:, None] * N + rn[None, :], acc.to(y_ptr.dtype.element_ty),
                 mask=(rm[:, None] < M) & (rn[None, :] < N))

    gemv_rows = [(64, 32, 4, 1), (16, 128, 4, 1), (128, 32, 4, 2), (64, 128, 4, 2), (256, 64, 8, 2)]

    @triton.autotune(configs=[triton.Config({"BN": n, "BK": k}, num_warps=w, num_stages=st)
                              for n, k, w, st in gemv_rows], key=["N", "K"])
    @triton.jit
    def w4a16_sum(x_ptr, p_ptr, s_ptr, y_ptr, N, K, GROUP: tl.constexpr, ZP: tl.constexpr,
                  BN: tl.constexpr, BK: tl.constexpr):
        row, pid_n = tl.program_id(0), tl.program_id(1)
        rn = pid_n * BN + tl.arange(0, BN)
        rk = tl.arange(0, BK)
        acc = tl.zeros((BN,), dtype=tl.float32)
        for k0 in range(0, K, BK):
            k = k0 + rk
            x = tl.load(x_ptr + row * K + k, mask=k < K, other=0.0).to(tl.float32)
            word = tl.load(p_ptr + (k[:, None] // 8) * N + rn[None, :],
                           mask=(k[:, None] < K) & (rn[None, :] < N), other=0)
            q = ((word >> ((k[:, None] % 8) * 4)) & 15) - ZP
            scale = tl.load(s_ptr + (k[:, None] // GROUP) * N + rn[None, :],
                            mask=(k[:, None] < K) & (rn[None, :] < N), other=0.0)
            acc += tl.sum(x[:, None] * (q.to(tl.float32) * scale.to(tl.float32)), axis=0)
        tl.store(y_ptr + row * N + rn, acc.to(y_ptr.dtype.element_ty), mask=rn < N)

    return triton, w4a16_dot, w4a16_sum


def run_triton(args) -> dict:
    import torch

    import oracle
    from intent_b200 import workloads

    if args.workload not in ("prefill", "decode"):
        return {"impl": "triton", "unavailable": "the Triton column covers the W4A16 configurations only"}
    try:
        triton, w4a16_dot, w4a16_sum = _triton_kernels()
    except Exception as error:
        return {"impl": "triton", "unavailable": f"triton cannot be imported: {error}"[:200]}
    device = torch.device("cuda", 0)
    peaks = measured_peaks()
    metric, unit, scaling, dtype = WORKLOAD_META[args.workload]

    def timed(launch, steps, flush=None):
        for _ in range(3):
            launch(0)
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(steps):
            launch(i)
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / steps

    if args.workload == "prefill":
        M, K, N = PREFILL["M"], PREFILL["K"], PREFILL["N"]
        x, p, s = (t.to(device) for t in workloads.w4a16_inputs(M, K, N, dtype=torch.bfloat16, seed=0))
        y = torch.empty((M, N), dtype=torch.bfloat16, device=device)
        grid = lambda meta: (triton.cdiv(M, meta["BM"]), triton.cdiv(N, meta["BN"]))      # noqa: E731
        ms = timed(lambda i: w4a16_dot[grid](x, p, s, y, M, N, K, GROUP=GROUP, ZP=8), max(3, min(args.steps, 20)))
        rows = torch.tensor([0, 511, 4096, 8191])
        ref = oracle.weight_only_int4_matmul(x[rows.to(device)].cpu(), p.cpu(), s.cpu(), group_size=GROUP, zero_point=8)
        error = (y[rows.to(device)].cpu().float() - ref.float()).abs().max().item() / ref.float().abs().max().item()
        value = 2.0 * M * K * N / (ms * 1e-3) / 1e12
        roofline = {"bound": "tensor", "achieved": round(value, 1), "peak": peaks["bf16_tflops"], "unit": unit,
                    "frac": round(value / peaks["bf16_tflops"], 4), "traffic": None}
        chosen = str(w4a16_dot.best_config)
    else:
        Mb = args.batch
        sets = [[t.to(device) for t in workloads.w4a16_inputs(Mb, K, N, dtype=torch.float16, seed=i)]
                for i, (K, N) in enumerate(DECODE_SHAPES)]
        copies = 6                                              # rotate the weights through > 2x L2
        rotated = [[(x, p.clone(), s.clone()) for x, p, s in sets] for _ in range(copies)]
        outs = [torch.empty((Mb, N), dtype=torch.float16, device=device) for _, N in DECODE_SHAPES]

        def step(i):
            for j, (K, N) in enumerate(DECODE_SHAPES):
                x, p, s = rotated[i % copies][j]
                w4a16_sum[lambda meta: (Mb, triton.cdiv(N, meta["BN"]))](x, p, s, outs[j], N, K, GROUP=GROUP, ZP=8)

        ms = timed(step, max(10, min(args.steps, 200)))
        x, p, s = sets[0]
        ref = oracle.weight_only_int4_matmul(x.cpu(), p.cpu(), s.cpu(), group_size=GROUP, zero_point=8)
        step(0)
        torch.cuda.synchronize()
        w4a16_sum[lambda meta: (Mb, triton.cdiv(14336, meta["BN"]))](x, p, s, outs[0], 14336, 4096, GROUP=GROUP, ZP=8)
        torch.cuda.synchronize()
        error = (outs[0].cpu().float() - ref.float()).abs().max().item() / ref.float().abs().max().item()
        value = decode_bytes(Mb) / (ms * 1e-3) / 1e9
        per_launch = value
        roofline = {"bound": "hbm", "achieved": round(per_launch, 1), "peak": peaks["hbm_gbs"], "unit": unit,
                    "frac": round(per_launch / peaks["hbm_gbs"], 4), "traffic": None}
        chosen = str(w4a16_sum.best_config)
    return {"impl": "triton", "metric": metric, "value": round(value, 2), "unit": unit, "n_gpus": 1,
            "ms_per_step": round(ms, 5), "higher_is_better": True, "scaling": scaling, "dtype": dtype,
            "data": "synthetic", "config": workload_config(args.workload, 1, args.batch),
            "roofline": roofline, "triton_config": chosen, "max_abs_rel_vs_oracle": float(f"{error:.3e}"),
            "note": "informational: a hand-restated Triton kernel of the shape the reference's provider emits "
                    "(tl.dot / multiply-and-sum with in-loop unpack), eager launches, device-resident inputs"}


ATTACHED_KEYS = ("metric", "value", "unit", "ms_per_step", "steps", "config", "notes", "roofline", "headline_mode", "modes",
                 "kernels", "e2e",
                 "gpu_launches", "scaling", "dtype")


def attach(line: dict, name: str, produce, rank: int) -> None:
    """Run one more configuration and hang its figures under `name`; a failure becomes an error note on
    that object, the primary line still prints."""
    try:
        sub, extra = produce()
    except Exception as error:       # the other configurations must not cost the primary line
        line[name] = {"error": f"{type(error).__name__}: {error}"[:400]}
        return None
    line[name] = {k: sub[k] for k in ATTACHED_KEYS if k in sub}
    return extra


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=None)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--workload", default="prefill", choices=["prefill", "decode", "w8a8", "moe", "grouped", "ring"])
    parser.add_argument("--batch", type=int, default=1, help="decode batch M (1, 4, 8)")
    parser.add_argument("--impl", default="b200", choices=["b200", "reference", "triton"])
    parser.add_argument("--load-seconds", type=float, default=1.5)
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--cpu-budget", type=float, default=150.0,
                        help="seconds of host time the reference arm may spend on its timed steps")
    parser.add_argument("--attach", default="all",
                        help="'all', 'none' or a comma list of decode,decode_m4,decode_m8,w8a8,moe: the other "
                             "configurations measured in the same run and attached to the prefill line")
    parser.add_argument("--moe-e2e-pieces", type=int, default=8,
                        help="MoE end-to-end path on one GPU: pieces of the token batch whose upload, FFN and "
                             "download overlap (intent_b200.moe.HostPipelinedFFN); 1 = the whole batch at once")
    parser.add_argument("--e2e-chunks", type=int, default=8,
                        help="pieces per rank of the pipelined end-to-end path of the dense programs")
    parser.add_argument("--moe-block", type=int, default=128, choices=[128, 256],
                        help="rows every expert span is padded to (= row tile of the grouped contraction)")
    parser.add_argument("--moe-exchange", default="peer", choices=["peer", "nccl"],
                        help="expert-parallel exchange: direct peer-memory stores/loads, or NCCL all-to-all")
    parser.add_argument("--prelayout", action="store_true",
                        help="tensor-core W4A16 kernels read a tiled copy of the weight (intent_b200.prelayout) "
                             "instead of the reference [K/8, N] layout")
    parser.add_argument("--moe-eager", action="store_true",
                        help="launch the bound MoE step eagerly instead of replaying it as one CUDA graph (one GPU, "
                             "and the peer exchange form on several)")
    parser.add_argument("--moe-graph", action="store_true",
                        help="(the default now; kept so that older command lines still parse)")
    parser.add_argument("--no-decode", action="store_true", help="same as --attach none")
    parser.add_argument("--table-tune", default="",
                        help="measurement knobs of the table kernel, e.g. 'slots=24,corr_mma=0' "
                             "(see intent_b200_w4a16_gemv_table_tune)")
    parser.add_argument("--probe-level", type=int, default=1,
                        help="decode 'probe' mode: 1 = arithmetic skipped, 2 = reduction skipped too, 3 = only the packed "
                             "weights are loaded (results are wrong by design; shows where the time goes)")
    parser.add_argument("--decode-modes", default="long,probe,projection",
                        help="extra decode measurements beside the one-launch-per-step table: 'long' (eight steps "
                             "per call), 'probe' (the long table with the arithmetic skipped: the ring's streaming "
                             "ceiling; results are wrong by design and are not read), 'projection' (one launch per "
                             "projection); '' = none (for profiling)")
    args = parser.parse_args()
    if args.steps is None:
        args.steps = {"prefill": 50, "decode": 200, "w8a8": 100, "moe": 20, "grouped": 50, "ring": 1}[args.workload]
        if args.impl == "reference":
            args.steps = 5
    if args.no_decode:
        args.attach = "none"
    names = ("decode", "decode_m4", "decode_m8", "w8a8", "moe")
    attached = names if args.attach == "all" else () if args.attach == "none" else \
        tuple(n for n in args.attach.split(",") if n in names)
    if args.workload != "prefill":
        attached = ()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        line = run_reference(args, rank, world)
        if line is not None:
            print(json.dumps(line), flush=True)
        return 0
    if args.impl == "triton":
        if rank == 0:
            print(json.dumps(run_triton(args)), flush=True)
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

    if args.workload == "ring":
        if rank == 0:
            print(json.dumps(run_ring_probe(device)), flush=True)
        return 0
    cpu_wanted = rank == 0 and world == 1 and not args.no_cpu_baseline
    if args.workload == "decode":
        line = run_decode(args, rank, world, device)
        extra = {"y": line.pop("_results", None)}
    else:
        runner = {"prefill": run_prefill, "w8a8": run_w8a8, "moe": run_moe, "grouped": run_grouped}[args.workload]
        line, extra = runner(args, rank, world, device)
    if rank == 0:
        line["cpu_baseline"] = None
    if cpu_wanted:
        leg = cpu_workload(args.workload, args.batch, 5, 1, budget_s=25.0, inputs=extra.get("inputs"))
        line["cpu_baseline"] = cpu_baseline_object(leg)
        parity = parity_against_cpu(leg, extra.get("y"))
        if parity:
            line["parity_vs_cpu"] = parity
    del extra

    # the other configurations of the headline metric, measured in the same run
    shared = argparse.Namespace(**vars(args))
    weights = None
    for name in attached:
        sub_args = argparse.Namespace(**vars(shared))
        if name.startswith("decode"):
            M = {"decode": 1, "decode_m4": 4, "decode_m8": 8}[name]
            if weights is None:
                weights = DecodeWeights(device)
            def produce(M=M):
                sub = run_decode(sub_args, rank, world, device, M=M, weights=weights, steps=200, load_seconds=0.5)
                return sub, {"y": sub.pop("_results", None)}
            workload, budget = "decode", 6.0
        elif name == "w8a8":
            weights = None
            sub_args.steps, sub_args.load_seconds = 50, 0.5
            produce = lambda: run_w8a8(sub_args, rank, world, device)      # noqa: E731
            workload, budget, M = "w8a8", 10.0, 1
        else:
            weights = None
            sub_args.steps, sub_args.load_seconds = 20, 0.5
            produce = lambda: run_moe(sub_args, rank, world, device)       # noqa: E731
            workload, budget, M = "moe", 30.0, 1
        extra = attach(line, name, produce, rank)
        if cpu_wanted and "error" not in line[name]:
            leg = cpu_workload(workload, M, 3, 1, budget_s=budget, inputs=(extra or {}).get("inputs"))
            line[name]["cpu_baseline"] = cpu_baseline_object(leg)
            parity = parity_against_cpu(leg, (extra or {}).get("y"))
            if parity:
                line[name]["parity_vs_cpu"] = parity
        elif rank == 0 and "error" not in line[name]:
            line[name]["cpu_baseline"] = None
        del extra
        torch.cuda.empty_cache()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
