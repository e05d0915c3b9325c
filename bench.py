#!/usr/bin/env python
"""Benchmark of the packed-GGUF hot path on B200 (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A *step* is one pass of the hot path over one batch of synthetic input. The default workload,
``moe_stack_b64``, is the decode step of the baseline's fifth configuration: 48 packed sparse-MoE
layers (hidden 2048, 512 experts of width 512, top-10 renormalised routing, always-on shared expert,
Q4_K gate/up + Q6_K down, about 50 GB packed and resident in HBM) with per-layer RMSNorm and an FP32
residual stream, 64 tokens per GPU and step; token mixing is the identity. ``value`` is decode
tokens/s with the step captured in a CUDA graph and everything resident in HBM; ``e2e`` is the same
step with its activations copied in from pinned host memory and the result copied back every step.
The 48 distinct layers touch about 22-33 GB per step, far more than L2, so every launch streams its
weights from HBM. ``roofline`` describes the dominant kernel (grouped gate/up + SwiGLU): algorithmic
bytes of one launch over its own CUDA-event duration. ``dense_gemv`` adds a short measurement of the
dense decode GEMVs of the second configuration (the other half of the metric); the ``gemv_*``
workloads run those as the main measurement instead.

With N > 1 (launched by torchrun, one rank per GPU) the MoE workloads run expert-parallel with the
baseline's batch: the experts of every layer AND the 64 (or ``tokens``) rows of a step are split over the
ranks (strong scaling; a rank may hold no row at all), rows and expert terms are exchanged through peer
memory (``--exchange collective`` uses NCCL instead), ``value`` is the step's tokens over the slowest
rank's time, ``parity_checked`` says whether a 2-layer expert-parallel stack reproduced the single-GPU
stack bit for bit on this run's GPUs, and ``ep_breakdown_us_per_layer_rank0`` splits a layer into phases.
The dense GEMV workloads do not shard: N independent replicas, no collective. ``--impl reference``
times the reference's own CPU kernels (oracle/_ref, else the plain-C port) on the host cores instead.
"""

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

L2_BYTES = 126 * 1024 * 1024
BLOCKS = {"Q8_0": (32, 34), "Q4_K": (256, 144), "Q5_K": (256, 176), "Q6_K": (256, 210)}

WORKLOADS = {
    # name: (format, n, k, m, activation dtype)
    "gemv_q4k_8192x2048_m1": ("Q4_K", 8192, 2048, 1, "bfloat16"),
    "gemv_q4k_2048x8192_m1": ("Q4_K", 2048, 8192, 1, "bfloat16"),
    "gemv_q5k_8192x2048_m1": ("Q5_K", 8192, 2048, 1, "bfloat16"),
    "gemv_q6k_8192x2048_m1": ("Q6_K", 8192, 2048, 1, "bfloat16"),
    "gemv_q4k_8192x2048_m8": ("Q4_K", 8192, 2048, 8, "bfloat16"),
    "gemv_q8_0_4096x4096_m1": ("Q8_0", 4096, 4096, 1, "float32"),
    "gemv_q8_0_4096x4096_m8": ("Q8_0", 4096, 4096, 8, "float32"),
    "gemv_q4k_65536x8192_m1": ("Q4_K", 65536, 8192, 1, "bfloat16"),
    # shapes of the third configuration (Q8_0 Llama): LM head and the stacked gate|up projection
    "gemv_q8_0_49152x2048_m1": ("Q8_0", 49152, 2048, 1, "bfloat16"),
    "gemv_q8_0_16384x2048_m1": ("Q8_0", 16384, 2048, 1, "bfloat16"),
    "gemv_q6k_65536x2048_m1": ("Q6_K", 65536, 2048, 1, "bfloat16"),
    "gemv_q8_0_131072x4096_m1": ("Q8_0", 131072, 4096, 1, "bfloat16"),
    "gemv_q8_0_131072x4096_m8": ("Q8_0", 131072, 4096, 8, "bfloat16"),
    # 16 tokens: two 8-token tiles share one pass over the weights
    "gemv_q8_0_131072x4096_m16": ("Q8_0", 131072, 4096, 16, "bfloat16"),
    "gemv_q5k_65536x4096_m1": ("Q5_K", 65536, 4096, 1, "bfloat16"),
    "gemv_q4k_65536x4096_m8": ("Q4_K", 65536, 4096, 8, "bfloat16"),
    "gemv_q4k_65536x4096_m16": ("Q4_K", 65536, 4096, 16, "bfloat16"),
    # integer-dot mode (Q8_1 activations, opt-in): the activation dtype field names the mode
    "gemv_q4k_65536x8192_m1_q8_1": ("Q4_K", 65536, 8192, 1, "q8_1"),
    "gemv_q4k_8192x2048_m1_q8_1": ("Q4_K", 8192, 2048, 1, "q8_1"),
    "gemv_q5k_65536x4096_m1_q8_1": ("Q5_K", 65536, 4096, 1, "q8_1"),
    # prefill / batched sizes of the second configuration: the tcgen05 GEMM (weights in GGUF layout, read once)
    "gemm_q4k_8192x2048_m512": ("Q4_K", 8192, 2048, 512, "bfloat16"),
    "gemm_q4k_2048x8192_m512": ("Q4_K", 2048, 8192, 512, "bfloat16"),
    "gemm_q5k_8192x2048_m512": ("Q5_K", 8192, 2048, 512, "bfloat16"),
    "gemm_q6k_8192x2048_m512": ("Q6_K", 8192, 2048, 512, "bfloat16"),
    "gemm_q4k_8192x2048_m32": ("Q4_K", 8192, 2048, 32, "bfloat16"),
    "gemm_q4k_8192x2048_m2048": ("Q4_K", 8192, 2048, 2048, "bfloat16"),
    "gemm_q8_0_8192x2048_m512": ("Q8_0", 8192, 2048, 512, "bfloat16"),
    "gemm_q8_0_8192x2048_m2048": ("Q8_0", 8192, 2048, 2048, "bfloat16"),
}
# name: (layers, tokens per step, chained)  - the packed MoE layer of the baseline's fourth configuration
# (hidden 2048, 512 experts of width 512, top-10, shared expert, Q4_K gate/up + Q6_K down); "stack" = the
# 48-layer decode step of the fifth configuration (RMSNorm + residual per layer, identity token mixing).
MOE_WORKLOADS = {
    "moe_layer_t1": (8, 1, False), "moe_layer_t16": (8, 16, False), "moe_layer_t64": (4, 64, False),
    "moe_layer_t256": (2, 256, False), "moe_stack_b1": (48, 1, True), "moe_stack_b64": (48, 64, True),
}
DEFAULT_WORKLOAD = "moe_stack_b64"
# dense decode GEMVs timed briefly next to every MoE run (rank 0): second configuration + one large matrix
SIDE_GEMVS = ("gemv_q4k_8192x2048_m1", "gemv_q8_0_4096x4096_m1", "gemv_q4k_65536x8192_m1",
              "gemm_q4k_8192x2048_m512", "gemm_q4k_2048x8192_m512")


def packed_bytes(fmt, n, k):
    qk, qb = BLOCKS[fmt]
    return n * k // qk * qb


def algorithmic_bytes(fmt, n, k, m, act_bytes):
    return packed_bytes(fmt, n, k) + m * k * act_bytes + m * n * act_bytes


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            data = json.loads(path.read_text())
            return float(data["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def measured_tensor_peak():
    """Sustained dense BF16 TFLOP/s (the bench times the kernel inside a long loop), else the stated fallback."""
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["bf16_tflops_sustained"]), "measured"
        except Exception:
            pass
    return 1400.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []
        self.thread = None
        self.first_timed = 0
        self.t_mark = None
        self.held = False

    def mark_timed_region(self):
        """Samples taken from now on belong to the timed region (the sampler is started before the warm-up
        so that nvidia-smi is already running when a short timed region begins)."""
        self.first_timed = len(self.lines)
        self.t_mark = time.perf_counter()

    def hold_load(self, step, step_ms, seconds=0.25, max_steps=100000):
        """A timed region of a few milliseconds ends before nvidia-smi's next sample. Called right after it,
        this keeps the same step running, untimed, until about `seconds` have passed since the region began,
        so that the samples describe the clocks the timed steps ran at. Every rank calls it with the step
        count agreed between the ranks (the step may hold an exchange between them); it does nothing when
        the region was long enough by itself."""
        import torch
        import torch.distributed as dist
        if self.t_mark is None:
            return
        remaining = seconds - (time.perf_counter() - self.t_mark)
        count = min(max_steps, max(0, int(remaining / max(step_ms * 1e-3, 1e-6)) + 1)) if remaining > 0 else 0
        if dist.is_available() and dist.is_initialized():
            agreed = torch.tensor([count], dtype=torch.int64, device="cuda")
            dist.all_reduce(agreed, op=dist.ReduceOp.MAX)
            count = int(agreed.item())
        for _ in range(count):
            step()
        torch.cuda.synchronize()
        self.held = count > 0

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()
        deadline = time.perf_counter() + 3.0          # nvidia-smi takes a moment to print its first line
        while not self.lines and time.perf_counter() < deadline and self.proc.poll() is None:
            time.sleep(0.01)

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        if self.thread is not None:
            self.thread.join(timeout=2)
        clocks, max_clock, reasons = [], None, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        window = "timed region + the same step kept running until 250 ms had passed" if self.held else "timed region"
        lines = self.lines[self.first_timed:]
        if not lines:                       # region shorter than one sampling period: use the warm-up under the same load
            lines, window = self.lines, "warm-up + timed region"
        self.window = window
        for line in lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                clocks.append(float(parts[0]))
                max_clock = float(parts[1])
            except ValueError:
                continue
            for name, flag in zip(names, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max_clock,
                "reasons": sorted(reasons), "samples": len(clocks), "window": window}


# ------------------------------------------------------------------------------ CPU reference arm
def cpu_threads():
    return max(1, len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))


def cpu_gemv_throughput(fmt, n, k, m, act_bytes, seconds):
    """Time the reference's CPU GEMV (row-sliced over all host threads) for about `seconds`."""
    from oracle import build_oracle as bo
    from mylocal_llm_b200.quantize import random_packed
    handle = bo.load_ref()
    kind = "reference"
    if handle is None:
        handle = bo.load_port()
        kind = "port"
    _, gemv, _ = handle
    rows = min(n, 2048)                                   # bounded sample of the weight rows
    w = random_packed(fmt, (rows, k), seed=0, d=0.01, dmin=0.005)
    x = np.random.default_rng(1).normal(0, 1, (m, k)).astype(np.float32)
    threads = cpu_threads()
    rb = w.nbytes // rows
    bounds = np.linspace(0, rows, threads + 1).astype(int)
    outs = [np.empty((m, max(1, b - a)), np.float32) for a, b in zip(bounds[:-1], bounds[1:])]
    fmt_id = bo.FORMAT_ID[fmt]

    def work(i):
        a, b = int(bounds[i]), int(bounds[i + 1])
        if b > a:
            gemv(w.data.ctypes.data + a * rb, fmt_id, b - a, k, x.ctypes.data, m, outs[i].ctypes.data)

    from concurrent.futures import ThreadPoolExecutor
    pool = ThreadPoolExecutor(threads)
    list(pool.map(work, range(threads)))                  # warm-up
    passes, t0 = 0, time.perf_counter()
    while True:
        list(pool.map(work, range(threads)))
        passes += 1
        elapsed = time.perf_counter() - t0
        if elapsed >= seconds:
            break
    pool.shutdown()
    per_pass = algorithmic_bytes(fmt, rows, k, m, act_bytes)
    gbs = per_pass * passes / elapsed / 1e9
    sample = f"{passes} passes over {rows} of {n} rows ({fmt}, K={k}, M={m}) in {elapsed:.1f} s"
    return gbs, kind, threads, sample, elapsed / passes, 2.0 * m * rows * k * passes / elapsed / 1e12


def run_reference_arm(args, name):
    fmt, n, k, m, act = WORKLOADS[name]
    act_bytes = 4 if act == "float32" else 2
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    per_step = max(1.0, 20.0 / max(1, args.steps + args.warmup))
    results = [cpu_gemv_throughput(fmt, n, k, m, act_bytes, per_step) for _ in range(args.warmup + args.steps)]
    timed = results[args.warmup:]
    gbs = statistics.mean(r[0] for r in timed)
    kind, threads, sample = timed[0][1], timed[0][2], timed[0][3]
    line = {
        "impl": "reference", "metric": "quant-GEMV HBM GB/s (algorithmic bytes per launch / time)",
        "value": round(gbs, 3), "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(1e3 * statistics.mean(r[4] for r in timed), 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, "format": fmt, "n": n, "k": k, "m": m, "activation": act,
                   "l2": "CPU run; each step is a bounded sample of the workload"},
        "cpu_baseline": {"value": round(gbs, 3), "unit": "GB/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": round(gbs, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    if m > 16:
        tfl = statistics.mean(r[5] for r in timed)
        line.update({"metric": "quantized GEMM TFLOP/s (2*M*N*K per launch / time)", "value": round(tfl, 6),
                     "unit": "TFLOP/s", "dtype": "bf16"})
        line["cpu_baseline"].update({"value": round(tfl, 6), "unit": "TFLOP/s"})
        line["e2e"].update({"value": round(tfl, 6), "unit": "TFLOP/s"})
    print(json.dumps(line))


# ----------------------------------------------------------------------------------- GPU arm
def run_gpu_arm(args, name):
    import torch
    import torch.distributed as dist
    from mylocal_llm_b200 import packed_to_device, quantized_linear
    from mylocal_llm_b200.quantize import random_packed

    fmt, n, k, m, act = WORKLOADS[name]
    q8_mode = act == "q8_1"                  # FP32 activations, quantised to Q8_1 by a kernel inside the timed step
    if q8_mode:
        act = "float32"
    act_dtype = getattr(torch, act)
    act_bytes = 4 if act == "float32" else 2
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the kernels)")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    wbytes = packed_bytes(fmt, n, k)
    copies = max(2, -(-2 * L2_BYTES // wbytes))
    copies = min(copies, 64)
    base = random_packed(fmt, (n, k), seed=1234 + rank, d=0.01, dmin=0.005)
    weights = []
    for c in range(copies):
        # a distinct HBM allocation per copy; the GEMM workloads read the GGUF layout
        weights.append(packed_to_device(base) if m > 16 else upload(base, act))
    rng = np.random.default_rng(7 + rank)
    host_x = torch.from_numpy(rng.normal(0, 1, (copies, m, k)).astype(np.float32)).to(act_dtype).pin_memory()
    dev_x = host_x.cuda()
    host_y = torch.empty((copies, m, n), dtype=act_dtype).pin_memory()

    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        if q8_mode:
            from mylocal_llm_b200.q8_1 import q8_1_linear, quantize_q8_1
            run = lambda c: q8_1_linear(quantize_q8_1(dev_x[c]), weights[c])     # quantiser + GEMV: two launches
        else:
            run = lambda c: quantized_linear(dev_x[c], weights[c])
        outs = [run(c) for c in range(copies)]   # warm-up, lazy init
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            outs = [run(c) for c in range(copies)]
        out_stack = outs

        def barrier():
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        # ---- device-resident throughput
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        for _ in range(max(3, args.warmup)):
            graph.replay()
        barrier()
        sampler.mark_timed_region()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for _ in range(args.steps):
            graph.replay()
        stop.record(stream)
        barrier()
        dev_ms = start.elapsed_time(stop)
        sampler.hold_load(graph.replay, dev_ms / args.steps)

        # ---- end to end: pinned host activations in, outputs back, every step
        def e2e_step():
            dev_x.copy_(host_x, non_blocking=True)
            graph.replay()
            for c in range(copies):
                host_y[c].copy_(out_stack[c], non_blocking=True)

        for _ in range(max(3, args.warmup)):
            e2e_step()
        barrier()
        start2, stop2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start2.record(stream)
        for _ in range(args.steps):
            e2e_step()
        stop2.record(stream)
        barrier()
        e2e_ms = start2.elapsed_time(stop2)
        clocks = sampler.stop() if rank == 0 else None

    times = torch.tensor([dev_ms, e2e_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = (float(v) for v in times.cpu())

    from mylocal_llm_b200 import _lib
    status = _lib.device_status()
    if status:
        raise SystemExit(f"device status word = {status}: a kernel gave up on a bounded wait")

    if rank == 0:
        per_launch = algorithmic_bytes(fmt, n, k, m, act_bytes)
        launches = copies * args.steps
        job_bytes = per_launch * launches * world
        value = job_bytes / (dev_ms * 1e-3) / 1e9
        e2e_value = job_bytes / (e2e_ms * 1e-3) / 1e9
        peak, peak_kind = measured_peaks()
        per_gpu = per_launch * launches / (dev_ms * 1e-3) / 1e9
        want_cpu = world == 1 and not args.skip_cpu_baseline
        cpu_gbs, cpu_kind, cpu_cores, cpu_sample, _, cpu_tfl = (cpu_gemv_throughput(fmt, n, k, m, act_bytes, 12.0)
                                                                if want_cpu else (None,) * 6)
        line = {
            "metric": "quant-GEMV HBM GB/s (algorithmic bytes per launch / time)",
            "value": round(value, 2), "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(dev_ms / args.steps, 5), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": name, "format": fmt, "n": n, "k": k, "m": m, "activation": act,
                       "copies_per_step": copies, "parallelism": "replicas only" if world > 1 else "single GPU",
                       "l2": f"{copies} distinct weight copies per step = {copies * wbytes / 1e6:.0f} MB > 2x L2",
                       "timing": "CUDA graph of one step, CUDA events on the launch stream"},
            "roofline": {"bound": "hbm", "achieved": round(per_gpu, 2), "peak": peak, "unit": "GB/s",
                         "frac": round(per_gpu / peak, 4), "peak_source": f"of {peak_kind}",
                         "frac_of_nominal_8TBs": round(per_gpu / 8000.0, 4),
                         "traffic": int(per_launch * 1.01) if fmt == "Q4_K" else None,
                         "traffic_source": "dram bytes / algorithmic bytes = 1.01 in the ncu capture "
                                           "profiles/mma_direct_q4k_gemv_65536x8192_m1.md (Q4_K only)",
                         "kernel": "mma_direct_kernel / q6k_tiled_kernel / mma_gemv_kernel by format", "us_per_launch": round(dev_ms * 1e3 / launches, 3),
                         "algorithmic_bytes_per_launch": per_launch},
            "e2e": {"value": round(e2e_value, 2), "unit": "GB/s",
                    "h2d_bytes_per_step": int(host_x.numel() * host_x.element_size()),
                    "d2h_bytes_per_step": int(host_y.numel() * host_y.element_size())},
            "gpu_launches": launches,
            "clocks": clocks,
        }
        if m > 16:
            # a contraction: report FLOP/s against the measured tensor peak instead of bytes against HBM
            tpeak, tkind = measured_tensor_peak()
            flops = 2.0 * m * n * k
            tfl = flops * launches / (dev_ms * 1e-3) / 1e12
            line.update({"metric": "quantized GEMM TFLOP/s (2*M*N*K per launch / time)", "value": round(tfl * world, 2),
                         "unit": "TFLOP/s", "dtype": "bf16"})
            line["e2e"].update({"value": round(flops * launches * world / (e2e_ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s"})
            line["roofline"] = {"bound": "tensor", "achieved": round(tfl, 2), "peak": tpeak, "unit": "TFLOP/s",
                                "frac": round(tfl / tpeak, 4), "peak_source": f"of {tkind} (sustained BF16)",
                                "traffic": None, "kernel": "umma_gemm_kernel (tcgen05.mma, TMEM accumulator, TMA activations)",
                                "us_per_launch": round(dev_ms * 1e3 / launches, 3), "flops_per_launch": flops,
                                "packed_weight_bytes": wbytes}
        if cpu_gbs is not None:
            line["cpu_baseline"] = {"value": round(cpu_gbs, 3), "unit": "GB/s", "cores": cpu_cores,
                                    "kind": cpu_kind, "sample": cpu_sample}
            if m > 16:
                line["cpu_baseline"].update({"value": round(cpu_tfl, 6), "unit": "TFLOP/s"})
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def upload(packed, act):
    """Host packed weight -> HBM, re-ordered into the device tile layout where one exists (the default
    of the MoE layers as well; B200Q_RETILE=0 keeps the GGUF bytes). K > 4096 is tiled only for 16-bit
    activations, the case the tiled kernel's shared-memory budget covers."""
    from mylocal_llm_b200 import packed_to_device
    from mylocal_llm_b200.quantized_linear import retile_enabled, retile_weight
    dev = packed_to_device(packed)
    return retile_weight(dev, force=act != "float32") if retile_enabled() else dev


def gemv_side_numbers(names, replays=20):
    """Short device-resident timing of dense decode GEMVs (same method as run_gpu_arm), reported next to
    the MoE number so one line carries both halves of the metric."""
    import torch
    from mylocal_llm_b200 import packed_to_device, quantized_linear
    from mylocal_llm_b200.quantize import random_packed
    peak, _ = measured_peaks()
    out = {}
    stream = torch.cuda.Stream()
    for name in names:
        fmt, n, k, m, act = WORKLOADS[name]
        act_dtype = getattr(torch, act)
        wbytes = packed_bytes(fmt, n, k)
        copies = min(max(2, -(-2 * L2_BYTES // wbytes)), 64)
        base = random_packed(fmt, (n, k), seed=99, d=0.01, dmin=0.005)
        weights = [packed_to_device(base) if m > 16 else upload(base, act) for _ in range(copies)]
        x = torch.randn((copies, m, k), device="cuda").to(act_dtype)
        with torch.cuda.stream(stream):
            for c in range(copies):
                quantized_linear(x[c], weights[c])
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for c in range(copies):
                    quantized_linear(x[c], weights[c])
            for _ in range(3):
                graph.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(replays):
                graph.replay()
            e1.record(stream)
            stream.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / (replays * copies)
        graph.reset()
        per_launch = algorithmic_bytes(fmt, n, k, m, 4 if act == "float32" else 2)
        gbs = per_launch / (us * 1e-6) / 1e9
        out[name] = {"GB/s": round(gbs, 1), "frac_of_peak": round(gbs / peak, 4), "us_per_launch": round(us, 3),
                     "layout": weights[0].quant_type}
        if m > 16:          # a contraction: FLOP/s against the measured sustained BF16 peak
            tpeak, _ = measured_tensor_peak()
            tfl = 2.0 * m * n * k / (us * 1e-6) / 1e12
            out[name] = {"TFLOP/s": round(tfl, 1), "frac_of_tensor_peak": round(tfl / tpeak, 4),
                         "us_per_launch": round(us, 3), "layout": weights[0].quant_type}
        del weights, graph
    torch.cuda.empty_cache()
    return out


def exit_watchdog(seconds=90):
    """Teardown of a process group whose collectives were captured in a CUDA graph can block; the
    result line is already printed by then, so a stuck teardown ends the process instead of the run."""
    timer = threading.Timer(seconds, lambda: os._exit(0))
    timer.daemon = True
    timer.start()


# ------------------------------------------------------------------------------ MoE workloads
MOE_SHAPE = dict(d_model=2048, d_ff=512, n_experts=512, top_k=10, shared_d_ff=512)
EXPERT_BYTES = 2 * packed_bytes("Q4_K", 512, 2048) + packed_bytes("Q6_K", 2048, 512)
# DRAM traffic of the grouped gate/up kernel over its algorithmic bytes in one ncu capture of the 64-token
# single-GPU layer (448.3 MB moved for 430.2 MB); other token counts and rank counts were not captured.
GATE_UP_TRAFFIC_RATIO = 1.04


def split_rows(tokens, world, rank):
    """Rows of a `tokens`-row batch that rank `rank` is home of, and the slot every rank reserves."""
    base, rem = divmod(tokens, world)
    return base + (1 if rank < rem else 0), base + (1 if rem else 0)


def moe_config(name, world, exchange):
    """Workload description shared by the GPU arm and the CPU reference arm (identical keys and values)."""
    layers, tokens, chained = MOE_WORKLOADS[name]
    touched = (min(512, 10 * tokens) + 1) * EXPERT_BYTES * layers / 1e9
    return {"workload": name, "layers": layers, "tokens_per_step": tokens, "chained": chained, **MOE_SHAPE,
            "formats": "Q4_K gate/up, Q6_K down", "activation": "bfloat16, FP32 residual",
            "parallelism": f"expert-parallel ep{world}: {MOE_SHAPE['n_experts'] // world} experts per rank, the "
                           f"{tokens} tokens of a step split over the ranks" if world > 1 else "single GPU",
            "l2": f"inputs larger than L2: {layers} distinct layers per step, up to {touched:.1f} GB of packed "
                  f"experts touched per step"}


class CpuMoeSample:
    """The reference's CPU path for one token through one MoE layer, on rotating weights.

    Router logits (FP32 NumPy), softmax / top-k / renormalisation and the ascending-expert ordered FP32
    sum are the oracle's restatement of the reference's RouterInference + ExpertsInference; the expert
    FFNs are the reference's own C++ kernel (oracle/_ref, else the plain-C port), top_k + 1 calls per
    token spread over the host threads. `n_rot` distinct experts (> 0.5 GB of packed bytes, more than the
    host's last-level cache) are visited round-robin so the weights stream from DRAM as they would in a
    512-expert layer."""

    def __init__(self, n_rot=288):
        from oracle import build_oracle as bo
        from mylocal_llm_b200.quantize import random_packed
        self.bo = bo
        self.handle, self.kind = bo.load_ref(), "reference"
        if self.handle is None:
            self.handle, self.kind = bo.load_port(), "port"
        self.d, self.f, self.k = MOE_SHAPE["d_model"], MOE_SHAPE["d_ff"], MOE_SHAPE["top_k"]
        d, f = self.d, self.f
        banks = [random_packed(q, (n_rot,) + sh, seed=i, d=1 / 2048, dmin=1 / 4096)
                 for i, (q, sh) in enumerate((("Q4_K", (f, d)), ("Q4_K", (f, d)), ("Q6_K", (d, f))))]
        self.banks = [b.data.reshape(n_rot, -1) for b in banks]
        self.n_rot = n_rot
        rng = np.random.default_rng(0)
        self.router = rng.normal(0, 0.02, (d, MOE_SHAPE["n_experts"])).astype(np.float32)
        self.x = rng.normal(0, 1, (64, d)).astype(np.float32)
        self.threads = cpu_threads()
        from concurrent.futures import ThreadPoolExecutor
        self.pool = ThreadPoolExecutor(self.threads)
        self.cursor = 0

    def token_layer(self, t):
        from oracle import packed_oracle as po
        x = self.x[t % len(self.x)][None]
        weights, ids = po.router_topk_rows_fp32(x @ self.router, self.k, 2.0 ** -14)
        order = np.argsort(ids[0], kind="stable")
        slots = [(self.cursor + j) % self.n_rot for j in range(self.k + 1)]       # k routed + the shared expert
        self.cursor = (self.cursor + self.k + 1) % self.n_rot
        run = lambda e: self.bo.cpu_expert(self.handle, (self.banks[0][e], "Q4_K"), (self.banks[1][e], "Q4_K"),
                                           (self.banks[2][e], "Q6_K"), self.d, self.f, x)
        outs = list(self.pool.map(run, slots))
        y = np.zeros((1, self.d), np.float32)
        for j in order:                                     # ascending expert id, plain FP32 adds
            y = (y + (outs[j] * weights[0, j]).astype(np.float32)).astype(np.float32)
        return (y + outs[self.k]).astype(np.float32)

    def run(self, seconds):
        n, t0 = 0, time.perf_counter()
        while time.perf_counter() - t0 < seconds:
            self.token_layer(n)
            n += 1
        return n, time.perf_counter() - t0

    def close(self):
        self.pool.shutdown()


def cpu_moe_throughput(layers, seconds, sampler=None):
    """Decode tokens/s of a `layers`-deep stack on the host cores, extrapolated from `seconds` of
    token-layer passes (one pass = router + top_k + 1 expert FFNs + ordered sum for one token)."""
    own = sampler is None
    sampler = sampler or CpuMoeSample()
    sampler.run(0.2)                                        # warm-up
    n, elapsed = sampler.run(seconds)
    if own:
        sampler.close()
    sample = (f"{n} token-layer passes (router, top-{sampler.k}, {sampler.k + 1} expert FFNs Q4_K/Q4_K/Q6_K "
              f"D={sampler.d} F={sampler.f} rotating over {sampler.n_rot} distinct experts, ordered sum) in {elapsed:.1f} s; "
              f"a token of the {layers}-layer stack needs {layers} passes")
    return n / elapsed / layers, sampler.kind, sampler.threads, sample, n


def run_moe_reference_arm(args, name):
    layers, tokens, chained = MOE_WORKLOADS[name]
    if int(os.environ.get("RANK", "0")) != 0:
        return
    eff_layers = layers if chained else 1
    per_step = max(1.0, 20.0 / max(1, args.steps + args.warmup))
    sampler = CpuMoeSample()
    runs = [cpu_moe_throughput(eff_layers, per_step, sampler) for _ in range(args.warmup + args.steps)][args.warmup:]
    sampler.close()
    tps = statistics.mean(r[0] for r in runs)
    passes = sum(r[4] for r in runs)
    needed = eff_layers * tokens * args.steps
    line = {
        "impl": "reference", "metric": "MoE decode tokens/s", "value": round(tps, 4), "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(1e3 * tokens / tps, 3),
        "higher_is_better": True, "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": moe_config(name, args.gpus, args.exchange),
        "extrapolated": True,
        "sampled": {"token_layer_passes_timed": passes, "token_layer_passes_in_the_full_steps": needed,
                    "fraction": round(passes / needed, 6),
                    "note": "ms_per_step is tokens_per_step / value, not a timed full step: each step times a "
                            "bounded sample of token-layer passes"},
        "cpu_baseline": {"value": round(tps, 4), "unit": "tokens/s", "cores": runs[0][2], "kind": runs[0][1],
                         "sample": runs[0][3]},
        "e2e": {"value": round(tps, 4), "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def graph_time(torch, stream, fn, replays, warm=3):
    """Capture fn() in a CUDA graph on `stream`; returns (ms per replay, graph, captured result)."""
    fn()
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        out = fn()
    for _ in range(warm):
        graph.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(replays):
        graph.replay()
    e1.record(stream)
    stream.synchronize()
    return e0.elapsed_time(e1) / replays, graph, out


def batch1_side_numbers(torch, stream, stack):
    """Batch-1 decode, the first term of the metric, next to the main number: the 48-layer MoE stack at one
    token (on the resident stack) and the Q8_0 Llama decoder of the third configuration after a 512-token
    prompt. Whole-step HBM fraction = packed bytes a step must read / step time / measured copy peak."""
    from mylocal_llm_b200.llama_model import ExternalLlamaConfig, ExternalLlamaModel
    peak, _ = measured_peaks()
    out = {}
    x1 = torch.randn((1, 1, MOE_SHAPE["d_model"]), device="cuda")
    ms, graph, _ = graph_time(torch, stream, lambda: stack.forward(x1)[0], replays=30)
    graph.reset()
    step_bytes = len(stack.layers) * ((MOE_SHAPE["top_k"] + 1) * EXPERT_BYTES + 4 * 2048 * 512)
    out["moe_stack_b1"] = {"tokens/s": round(1e3 / ms, 1), "ms_per_step": round(ms, 4), "layers": len(stack.layers),
                           "step_bytes": step_bytes, "frac_of_peak": round(step_bytes / (ms * 1e-3) / 1e9 / peak, 4),
                           "step": "one persistent kernel" if getattr(stack, "persistent_step", False) else "chain of launches"}
    if getattr(stack, "persistent_step", False):
        os.environ["B200Q_STAGE_TIMES"] = "1"           # one more step with the kernel's stage stamps switched on
        stack.forward(x1)
        stream.synchronize()
        del os.environ["B200Q_STAGE_TIMES"]
        out["moe_stack_b1"]["last_layer_stage_us"] = stack.stage_times()
        stack.persistent_step = False
        ms_chain, graph, _ = graph_time(torch, stream, lambda: stack.forward(x1)[0], replays=30)
        graph.reset()
        stack.persistent_step = True
        out["moe_stack_b1"]["chain_of_launches_tokens/s"] = round(1e3 / ms_chain, 1)
    model = ExternalLlamaModel.synthetic(ExternalLlamaConfig(**LLAMA_SHAPE), seed=0)
    state = model.create_generation_state(1, LLAMA_PROMPT + 256)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(5)
    prompt = torch.randint(0, LLAMA_SHAPE["vocab_size"], (1, LLAMA_PROMPT), device="cuda", generator=gen)
    token = model.prefill(prompt, state).argmax(dim=-1)
    step = lambda: token.copy_(model.decode_one(token, state).argmax(dim=-1))
    ms, graph, _ = graph_time(torch, stream, step, replays=64)
    graph.reset()
    out["llama_decode_b1"] = {"tokens/s": round(1e3 / ms, 1), "ms_per_step": round(ms, 4),
                              "step_bytes": llama_bytes_per_step(),
                              "frac_of_peak": round(llama_bytes_per_step() / (ms * 1e-3) / 1e9 / peak, 4),
                              "context": f"{LLAMA_PROMPT}-token prompt, positions {LLAMA_PROMPT}..{LLAMA_PROMPT + 70}"}
    del model, state
    torch.cuda.empty_cache()
    return out


def ep_parity_check(torch, dist, comm, tokens, rank, world):
    """Outside the timed region: a 2-layer expert-parallel stack built from the slices of full banks must
    return, for this rank's rows, the bits of the single-GPU stack built from the same banks."""
    from mylocal_llm_b200.expert_parallel import ExpertParallelMoEStack
    from mylocal_llm_b200.moe_stack import PackedMoEStack
    stack = PackedMoEStack.synthetic(2, seed=321, keep_native=True, **MOE_SHAPE)
    twin = ExpertParallelMoEStack.sharded_from(stack, stack.native_banks, comm)
    x = torch.from_numpy(np.random.default_rng(99).normal(0, 1, (1, tokens, MOE_SHAPE["d_model"])).astype(np.float32)).cuda()
    want_res, want_hidden = stack.forward(x)
    rows, slot = split_rows(tokens, world, rank)
    lo = sum(split_rows(tokens, world, r)[0] for r in range(rank))
    mine = x[:, lo:lo + rows].contiguous()
    ok = True
    for _ in range(2):
        res, hidden = twin.forward(mine, slot_rows=slot, total_rows=tokens)
        ok = ok and torch.equal(res, want_res[:, lo:lo + rows]) and torch.equal(hidden, want_hidden[:, lo:lo + rows])
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    del stack, twin
    torch.cuda.empty_cache()
    return bool(flag.item())


def ep_breakdown(torch, stream, step_fn, layers):
    """Eager per-phase CUDA-event times of the expert-parallel layers on this rank, averaged over layers
    (microseconds). "push" and "barrier" include the wait for the slowest rank."""
    from mylocal_llm_b200 import expert_parallel as ep
    marks = []

    def hook(name):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(stream)
        marks.append((name, ev))

    totals = {}
    for rep in range(3):
        marks.clear()
        ep.PHASE_HOOK = hook
        hook("start")
        step_fn()
        ep.PHASE_HOOK = None
        stream.synchronize()
        if rep == 0:
            continue                                        # first eager pass: warm-up
        prev = marks[0][1]
        for name, ev in marks[1:]:
            # "route" closes the stretch since the previous layer's combine: residual add + RMSNorm, then routing
            key = "norm+route" if name == "route" else name
            totals[key] = totals.get(key, 0.0) + prev.elapsed_time(ev) * 1e3
            prev = ev
    return {k: round(v / (2 * layers), 2) for k, v in totals.items()}


def run_moe_gpu_arm(args, name):
    import torch
    import torch.distributed as dist
    from mylocal_llm_b200 import _lib, moe_ops
    from mylocal_llm_b200.moe_stack import PackedMoEStack

    layers, tokens, chained = MOE_WORKLOADS[name]
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the kernels)")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    side = gemv_side_numbers(SIDE_GEMVS) if rank == 0 and not args.skip_side else None
    comm, parity = None, None
    rows, slot = split_rows(tokens, world, rank)
    if world > 1:
        # expert-parallel, strong scaling: the experts AND the `tokens` rows of a step are split over the ranks
        from mylocal_llm_b200.expert_parallel import CollectiveComm, ExpertParallelMoEStack, PeerComm
        if args.exchange == "peer":
            comm = PeerComm(None, max_rows=slot, d_model=MOE_SHAPE["d_model"], k_out=MOE_SHAPE["top_k"] + 1)
        else:
            comm = CollectiveComm()
        parity = ep_parity_check(torch, dist, comm, tokens, rank, world)
        stack = ExpertParallelMoEStack.synthetic(layers, comm, seed=0, **MOE_SHAPE)
    else:
        stack = PackedMoEStack.synthetic(layers, seed=0, **MOE_SHAPE)
    d = MOE_SHAPE["d_model"]
    rng = np.random.default_rng(11 + rank)
    host_x = torch.from_numpy(rng.normal(0, 1, (1, rows, d)).astype(np.float32)).pin_memory()
    dev_x = host_x.cuda()
    host_y = torch.empty((1, rows, d), dtype=torch.float32).pin_memory()

    def step_fn():
        if chained:
            return stack.forward(dev_x, slot, tokens)[0] if world > 1 else stack.forward(dev_x)[0]
        outs = None
        hidden = dev_x.to(torch.bfloat16)
        for layer in stack.layers:                       # independent layers: distinct weights defeat L2
            outs = layer.forward(hidden, slot, tokens) if world > 1 else layer.forward(hidden)
        return outs.float()

    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        # launches per step, counted once through the library's call log
        calls = []
        real_call = _lib.call
        _lib.call = lambda fn, *a: (calls.append(fn), real_call(fn, *a))[1]
        out = step_fn()
        stream.synchronize()
        _lib.call = real_call
        launches_per_step = len(calls)
        step_fn()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            out = step_fn()

        def barrier():
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        for _ in range(max(3, args.warmup)):
            graph.replay()
        barrier()
        sampler.mark_timed_region()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            graph.replay()
        e1.record(stream)
        barrier()
        dev_ms = e0.elapsed_time(e1)
        sampler.hold_load(graph.replay, dev_ms / max(1, args.steps))

        def e2e_step():
            dev_x.copy_(host_x, non_blocking=True)
            graph.replay()
            host_y.copy_(out, non_blocking=True)

        for _ in range(max(3, args.warmup)):
            e2e_step()
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record(stream)
        for _ in range(args.steps):
            e2e_step()
        f1.record(stream)
        barrier()
        e2e_ms = f0.elapsed_time(f1)
        clocks = sampler.stop() if rank == 0 else None

        # dominant kernel (grouped gate/up): its own duration and bytes, eager launches with events
        records = []
        real_gate_up = moe_ops.moe_gate_up

        def timed_gate_up(x2d, plan, *a, **kw):
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record(stream)
            res = real_gate_up(x2d, plan, *a, **kw)
            a1.record(stream)
            records.append((a0, a1, plan.counts))
            return res

        moe_ops.moe_gate_up = timed_gate_up
        # (a one-token step runs as one persistent kernel; its gate/up stage is the same device function as the
        # separate launch timed here)
        persistent = getattr(stack, "persistent_step", False)
        if persistent:
            stack.persistent_step = False
        for _ in range(2):
            records.clear()
            step_fn()
            stream.synchronize()
        moe_ops.moe_gate_up = real_gate_up
        if persistent:
            stack.persistent_step = True
        gate_up_ms = [a0.elapsed_time(a1) for a0, a1, _ in records]
        # expert-parallel plans end with one entry counting the assignments other ranks execute
        executed = [c[:-1] if world > 1 else c for _, _, c in records]
        distinct = [int((c > 0).sum().item()) for c in executed]
        assignments = [int(c.sum().item()) for c in executed]
        breakdown = ep_breakdown(torch, stream, step_fn, layers) if world > 1 else None
        batch1 = None
        if world == 1 and rank == 0 and chained and not args.skip_side:
            batch1 = batch1_side_numbers(torch, stream, stack)

    times = torch.tensor([dev_ms, e2e_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = (float(v) for v in times.cpu())
    if _lib.device_status():
        raise SystemExit("device status word is set: a kernel gave up on a bounded wait")

    if rank == 0:
        tokens_per_step = tokens * (1 if chained else layers)
        value = tokens_per_step * args.steps / (dev_ms * 1e-3)
        e2e_value = tokens_per_step * args.steps / (e2e_ms * 1e-3)
        peak, peak_kind = measured_peaks()
        gu_bytes = statistics.mean(distinct) * 2 * packed_bytes("Q4_K", 512, 2048) + world * slot * d * 2 \
            + statistics.mean(assignments) * 512 * 4
        gu_us = statistics.mean(gate_up_ms) * 1e3
        achieved = gu_bytes / (gu_us * 1e-6) / 1e9
        # bytes this rank's layer must read: its distinct experts, shared expert, router weights, activations
        layer_bytes = statistics.mean(distinct) * EXPERT_BYTES + (EXPERT_BYTES if world > 1 else 0) \
            + 4 * 2048 * 512 + 2 * tokens * d * 2
        single = world == 1 and tokens == 64
        line = {
            "metric": "MoE decode tokens/s", "value": round(value, 2), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dev_ms / args.steps, 5),
            "higher_is_better": True, "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": moe_config(name, world, args.exchange),
            "details": {"packed_bytes_resident_rank0": stack.packed_bytes, "exchange": args.exchange if world > 1 else None,
                        "rows_rank0": rows, "slot_rows": slot,
                        "timing": "CUDA graph of one step, CUDA events on the launch stream, max over ranks",
                        "distinct_experts_per_layer_rank0": round(statistics.mean(distinct), 1),
                        "assignments_per_layer_rank0": round(statistics.mean(assignments), 1),
                        "algorithmic_bytes_per_layer_rank0": int(layer_bytes),
                        "layer_GBs_rank0": round(layer_bytes * layers * args.steps / (dev_ms * 1e-3) / 1e9, 1)},
            "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": peak, "unit": "GB/s",
                         "frac": round(achieved / peak, 4), "peak_source": f"of {peak_kind}",
                         "frac_of_nominal_8TBs": round(achieved / 8000.0, 4),
                         "traffic": int(gu_bytes * GATE_UP_TRAFFIC_RATIO) if single else None,
                         "traffic_source": ("dram bytes read+write / algorithmic bytes = 1.04 in an ncu capture of this "
                                            "kernel on the 64-token single-GPU layer, scaled to this launch") if single
                         else "not captured for this token / rank count",
                         "kernel": "grouped gate/up + SwiGLU (mma_direct_kernel, mode 2)",
                         "us_per_launch": round(gu_us, 3), "algorithmic_bytes_per_launch": int(gu_bytes)},
            "e2e": {"value": round(e2e_value, 2), "unit": "tokens/s",
                    "h2d_bytes_per_step": int(host_x.numel() * 4), "d2h_bytes_per_step": int(host_y.numel() * 4)},
            "gpu_launches": launches_per_step * args.steps, "clocks": clocks,
        }
        if world > 1:
            line["parity_checked"] = parity
            line["parity_check"] = ("2-layer expert-parallel stack vs the single-GPU stack built from the same banks, "
                                    "bit-identical on every rank's rows, outside the timed region")
            line["ep_breakdown_us_per_layer_rank0"] = breakdown
        if side is not None:
            line["dense_gemv"] = side
        if batch1 is not None:
            line["batch1_decode"] = batch1
        if world == 1 and not args.skip_cpu_baseline:
            tps, kind, cores, sample, _ = cpu_moe_throughput(layers if chained else 1, 12.0)
            line["cpu_baseline"] = {"value": round(tps, 4), "unit": "tokens/s", "cores": cores, "kind": kind,
                                    "sample": sample}
        print(json.dumps(line))
    sys.stdout.flush()
    exit_watchdog()
    graph.reset()
    torch.cuda.synchronize()
    if comm is not None:
        comm.close()
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------ Llama decode workloads
# Third configuration: SmolLM2-1.7B shape, random-init Q8_0 weights (embedding and untied LM head included),
# 512-token prompt, then greedy decode; a step = one decode_one() of the whole batch.
LLAMA_SHAPE = dict(vocab_size=49152, hidden_size=2048, intermediate_size=8192, num_hidden_layers=24,
                   num_attention_heads=32, num_key_value_heads=32, head_dim=64, max_position_embeddings=2048,
                   rope_theta=10000.0, rms_norm_eps=1e-5)
LLAMA_WORKLOADS = {"llama_decode_b1": 1, "llama_decode_b16": 16}
LLAMA_PROMPT, LLAMA_NEW = 512, 128
LLAMA_HOLD = 160          # cache positions reserved for the untimed steps that keep the load up for the clock sampler


def llama_bytes_per_step():
    c = LLAMA_SHAPE
    d, f, v = c["hidden_size"], c["intermediate_size"], c["vocab_size"]
    per_layer = 4 * packed_bytes("Q8_0", d, d) + 2 * packed_bytes("Q8_0", f, d) + packed_bytes("Q8_0", d, f)
    return c["num_hidden_layers"] * per_layer + packed_bytes("Q8_0", v, d)          # + LM head, read every step


def run_llama_reference_arm(args, name):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    batch = LLAMA_WORKLOADS[name]
    per_step = max(1.0, 20.0 / max(1, args.steps + args.warmup))
    runs = [cpu_gemv_throughput("Q8_0", 8192, 2048, batch if batch <= 8 else 8, 4, per_step)
            for _ in range(args.warmup + args.steps)][args.warmup:]
    gbs = statistics.mean(r[0] for r in runs)
    passes = -(-batch // 8)                      # the CPU kernel handles the batch in groups like the GPU path
    tps = batch * gbs * 1e9 / (llama_bytes_per_step() * passes)
    line = {
        "impl": "reference", "metric": "decode tokens/s", "value": round(tps, 4), "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(1e3 * batch / tps, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, "batch": batch, **LLAMA_SHAPE, "format": "Q8_0",
                   "l2": "CPU run: the reference's packed GEMV on a bounded row sample, scaled to the bytes of "
                         "one decode step (attention and norms not included)"},
        "cpu_baseline": {"value": round(tps, 4), "unit": "tokens/s", "cores": runs[0][2], "kind": runs[0][1],
                         "sample": runs[0][3]},
        "e2e": {"value": round(tps, 4), "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def run_llama_gpu_arm(args, name):
    import torch
    import torch.distributed as dist
    from mylocal_llm_b200 import _lib
    from mylocal_llm_b200.llama_model import ExternalLlamaConfig, ExternalLlamaModel

    batch = LLAMA_WORKLOADS[name]
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the kernels)")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    model = ExternalLlamaModel.synthetic(ExternalLlamaConfig(**LLAMA_SHAPE), seed=rank)
    state = model.create_generation_state(batch, LLAMA_PROMPT + LLAMA_NEW + 64 + LLAMA_HOLD)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(5 + rank)
    prompt = torch.randint(0, LLAMA_SHAPE["vocab_size"], (batch, LLAMA_PROMPT), device="cuda", generator=gen)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        logits = model.prefill(prompt, state)
        token = logits.argmax(dim=-1)
        host_token = torch.empty(batch, dtype=torch.int64).pin_memory()
        calls = []
        real_call = _lib.call
        _lib.call = lambda fn, *a: (calls.append(fn), real_call(fn, *a))[1]
        token.copy_(model.decode_one(token, state).argmax(dim=-1))            # eager step: warm-up + launch count
        _lib.call = real_call
        launches_per_step = len(calls)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            token.copy_(model.decode_one(token, state).argmax(dim=-1))        # greedy: next token stays on the device

        def barrier():
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        budget = state.horizon - LLAMA_HOLD - LLAMA_PROMPT - 2
        steps = min(args.steps, (budget - 2 * max(3, args.warmup)) // 2)
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        for _ in range(max(3, args.warmup)):
            graph.replay()
        barrier()
        sampler.mark_timed_region()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            graph.replay()
        e1.record(stream)
        barrier()
        dev_ms = e0.elapsed_time(e1)
        sampler.hold_load(graph.replay, dev_ms / max(1, steps), max_steps=LLAMA_HOLD)    # cache room is reserved for it

        def e2e_step():
            graph.replay()
            host_token.copy_(token, non_blocking=True)

        for _ in range(max(3, args.warmup)):
            e2e_step()
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record(stream)
        for _ in range(steps):
            e2e_step()
            stream.synchronize()                  # the sampled token is needed on the host before the next step
        f1.record(stream)
        barrier()
        e2e_ms = f0.elapsed_time(f1)
        clocks = sampler.stop() if rank == 0 else None

    times = torch.tensor([dev_ms, e2e_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = (float(v) for v in times.cpu())
    if _lib.device_status():
        raise SystemExit("device status word is set: a kernel gave up on a bounded wait")
    if rank == 0:
        value = batch * world * steps / (dev_ms * 1e-3)
        e2e_value = batch * world * steps / (e2e_ms * 1e-3)
        peak, peak_kind = measured_peaks()
        step_bytes = llama_bytes_per_step() * (-(-batch // 8))
        achieved = step_bytes * steps / (dev_ms * 1e-3) / 1e9
        line = {
            "metric": "decode tokens/s", "value": round(value, 2), "unit": "tokens/s", "n_gpus": world,
            "steps": steps, "warmup": args.warmup, "ms_per_step": round(dev_ms / steps, 5),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": name, "batch": batch, "prompt_tokens": LLAMA_PROMPT, **LLAMA_SHAPE,
                       "format": "Q8_0 (all linears, embedding, untied LM head)", "activation": "bfloat16, FP32 residual",
                       "packed_bytes_resident": model.packed_bytes,
                       "parallelism": "replicas only" if world > 1 else "single GPU",
                       "l2": f"{llama_bytes_per_step() / 1e6:.0f} MB of packed weights read per step (> L2)",
                       "timing": "CUDA graph of one greedy decode step, CUDA events on the launch stream"},
            "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": peak, "unit": "GB/s",
                         "frac": round(achieved / peak, 4), "peak_source": f"of {peak_kind}", "traffic": None,
                         "kernel": "whole decode step: packed weight bytes per step / step time",
                         "algorithmic_bytes_per_launch": int(step_bytes)},
            "e2e": {"value": round(e2e_value, 2), "unit": "tokens/s", "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": int(host_token.numel() * 8)},
            "gpu_launches": launches_per_step * steps, "clocks": clocks,
        }
        print(json.dumps(line))
    sys.stdout.flush()
    exit_watchdog()
    graph.reset()
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS) + sorted(MOE_WORKLOADS) + sorted(LLAMA_WORKLOADS))
    ap.add_argument("--exchange", default="peer", choices=["peer", "collective"],
                    help="expert-parallel exchange at N > 1: peer-memory stores + device barrier, or NCCL")
    ap.add_argument("--skip-side", action="store_true", help="omit the dense-GEMV side measurements")
    ap.add_argument("--skip-cpu-baseline", action="store_true",
                    help="omit the host-core baseline leg (exploratory runs only)")
    args = ap.parse_args()
    if args.workload in LLAMA_WORKLOADS:
        (run_llama_reference_arm if args.impl == "reference" else run_llama_gpu_arm)(args, args.workload)
        return
    moe = args.workload in MOE_WORKLOADS
    if args.impl == "reference":
        (run_moe_reference_arm if moe else run_reference_arm)(args, args.workload)
    else:
        (run_moe_gpu_arm if moe else run_gpu_arm)(args, args.workload)


if __name__ == "__main__":
    main()
