#!/usr/bin/env python
"""Benchmark of the SDXL UNet quantized-Linear path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A "step" is one pass of the hot path over one batch of synthetic input. The default workload is
the 640-dim transformer-block layer set under W8A8 INT8 ConvRot at 1024^2, CFG batch 2
(to_q/to_k/to_v/to_out [8192,640]x[640,640], ff.net.0.proj+GEGLU [8192,640]x[5120,640],
ff.net.2 [8192,2560]x[640,2560]); the three attention projections share one quantised input.
Other workloads: `layerset1280_fp8` (the 1280-dim set under FP8 E4M3 per-channel, plus the
skinny cross-attention K/V GEMM), `unet743_int8` / `unet743_e5m2` (all 743 rank-2 projections of
one UNet step as one grouped launch), `crossattn_kv_int8` (the 140 cross-attention K/V projections
a per-generation cache removes from every step), `unetstep_int8|e4m3|e5m2` (one denoising step's
projections for this rank's share of 8 images x CFG 2: strong scaling over 1/2/4/8 ranks by
sharding images, projections only).

Rank 0 prints ONE JSON line. `value` is whole-job throughput (all ranks) with inputs resident in
HBM, timed on the device with CUDA events, max over ranks. `e2e` is the same metric through the
public API with host buffers (pinned host -> device copies of the inputs and device -> host reads
of the results inside the timed region). With N > 1 every rank runs the same workload on its own
GPU with replicated weights (weak scaling, no collective on the data path).

`--impl reference` times the reference's own CPU implementation of the path (its threaded AVX2
Linear compiled from the reference sources, else the CPU port) on a bounded sample of the same
workload, on the host cores of the box.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

METRIC = "quantized_linear_tops"
UNIT = "TOPS"
L2_BYTES = 126 * 1024 * 1024
# DRAM bytes (read + write) of one grouped GEMM launch of the default workload, from the ncu
# capture summarised in profiles/ (dram__bytes_read.sum + dram__bytes_write.sum).
TRAFFIC_BYTES = {"layerset640_int8": 88.75e6}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as handle:
            peaks = json.load(handle)
        return {"hbm_gbs": float(peaks["hbm_gbs"]), "bf16_tflops": float(peaks["bf16_tflops"]),
                "bf16_tflops_sustained": float(peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ------------------------------------------------------------------------------------------------
# workloads
# ------------------------------------------------------------------------------------------------
def layer_set(dim: int, tokens: int, batch_rows_context: int):
    """(name, M, N, K, bias, activation, input_key) of one transformer block's projections."""
    c = dim
    rows = [("attn1.to_q", tokens, c, c, False, 0, "norm1"), ("attn1.to_k", tokens, c, c, False, 0, "norm1"),
            ("attn1.to_v", tokens, c, c, False, 0, "norm1"), ("attn1.to_out.0", tokens, c, c, True, 0, "attn1"),
            ("ff.net.0.proj", tokens, 8 * c, c, True, 4, "norm3"), ("ff.net.2", tokens, c, 4 * c, True, 0, "geglu")]
    if batch_rows_context:
        rows.append(("attn2.to_k", batch_rows_context, c, 2048, False, 0, "context"))
        rows.append(("attn2.to_v", batch_rows_context, c, 2048, False, 0, "context"))
    return rows


def workload_rows(name: str):
    if name == "layerset640_int8":
        return layer_set(640, 8192, 0), "int8", ("SDXL UNet 640-dim layer set, W8A8 INT8 ConvRot (group 256 rule: K=2560 rotates), "
                                                "1024^2 CFG batch 2: q,k,v,out [8192,640]x[640,640]; ff.net.0.proj+GEGLU "
                                                "[8192,640]x[5120,640]; ff.net.2 [8192,2560]x[640,2560]")
    if name == "layerset1280_fp8":
        return layer_set(1280, 2048, 154), "e4m3", ("SDXL UNet 1280-dim layer set, FP8 E4M3 per-channel weights, native FP8 activations, "
                                                    "M=2048; plus cross-attention to_k/to_v [154,2048]x[1280,2048]")
    if name == "crossattn_kv_int8":
        # what a cross-attention K/V cache takes out of every denoising step
        shapes = importlib.import_module("sdxl-end2end_b200.unet_shapes")
        rows = [(p.name, p.m, p.n, p.k, p.bias, p.activation, p.input_key) for p in shapes.unet_projections(2)
                if ".attn2.to_k" in p.name or ".attn2.to_v" in p.name]
        return rows, "int8", (f"the {len(rows)} cross-attention to_k/to_v projections [154,2048]x[640|1280,2048] of one SDXL UNet step, "
                              "INT8 ConvRot, one grouped launch (HBM-bound: weights are read once)")
    if name.startswith("unetstep_"):
        # unetstep_<int8|e4m3|e5m2>: every projection of one denoising step for this rank's share of a
        # fixed job of 8 images x CFG 2 (UNet batch 16), images sharded over the ranks with replicated
        # weights (UNet batch 16 / world per rank). Only the projections run: convolutions, norms and
        # attention are not part of this path, so steps/s here bounds the UNet's from above.
        kind = name.split("_", 1)[1]
        if kind not in ("int8", "e4m3", "e5m2"):
            raise SystemExit(f"unknown workload {name}")
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if 16 % world != 0 or 16 // world < 2:
            raise SystemExit("unetstep shards 8 CFG pairs: 1, 2, 4 or 8 ranks")
        local_batch = 16 // world
        shapes = importlib.import_module("sdxl-end2end_b200.unet_shapes")
        rows = [(p.name, p.m, p.n, p.k, p.bias, p.activation, p.input_key) for p in shapes.unet_projections(local_batch)]
        return rows, kind, (f"all 743 rank-2 projections of one SDXL UNet step at 1024^2 for {local_batch // 2} of 8 images x CFG 2 "
                            f"(UNet batch {local_batch} of 16 on this rank), one grouped launch, {kind}; projections only")
    if name in ("unet743_int8", "unet743_e5m2"):
        shapes = importlib.import_module("sdxl-end2end_b200.unet_shapes")
        rows = [(p.name, p.m, p.n, p.k, p.bias, p.activation, p.input_key) for p in shapes.unet_projections(2)]
        kind = "int8" if name.endswith("int8") else "e5m2"
        return rows, kind, f"all 743 rank-2 projections of one SDXL UNet step at 1024^2, CFG batch 2, one grouped launch, {kind}"
    raise SystemExit(f"unknown workload {name}")


def total_ops(rows) -> float:
    return float(sum(2 * m * n * k for (_, m, n, k, _, _, _) in rows))


class DeviceWorkload:
    """Weights (quantised once), and `sets` rotating sets of inputs / outputs with one plan each."""

    def __init__(self, pkg, ops, rows, kind, sets, seed=1234):
        import torch
        import helpers as H
        self.pkg, self.ops, self.rows, self.kind = pkg, ops, rows, kind
        device = torch.device("cuda", torch.cuda.current_device())
        generator = torch.Generator(device=device)
        generator.manual_seed(seed)
        self.weights, self.biases = [], []
        for index, (name, m, n, k, bias, activation, key) in enumerate(rows):
            w = (torch.randn((n, k), generator=generator, device=device, dtype=torch.float32) / (k ** 0.5)).half()
            if kind == "int8":
                options = pkg.INT8WeightLoadOptions(enable_convrot=True, convrot_group_size=256)
                weight = ops.upload_or_quantize_int8_weight(w, None, options)
            elif kind in ("e4m3", "e5m2"):
                fmt = pkg.ScalarType.Float8E4M3 if kind == "e4m3" else pkg.ScalarType.Float8E5M2
                weight = ops.upload_fp8_weight(w, pkg.FP8WeightLoadOptions(format=fmt, scale_mode=pkg.FP8ScaleMode.PerOutputChannel))
            else:
                weight = ops.fp16_weight(w)
            self.weights.append(weight)
            self.biases.append((torch.randn(n, generator=generator, device=device) * 0.1).half() if bias else None)
            del w
        self.inputs, self.outputs, self.plans = [], [], []
        self.input_shapes = {}
        for (name, m, n, k, bias, activation, key) in rows:
            self.input_shapes.setdefault(key, (m, k))
        for s in range(sets):
            inputs = {}
            for key, (m, k) in self.input_shapes.items():
                x = torch.randn((m, k), generator=generator, device=device, dtype=torch.float32)
                if k >= 100:            # 1 % of the channels are x20 outliers
                    channels = torch.randperm(k, generator=generator, device=device)[: max(1, k // 100)]
                    x[:, channels] *= 20.0
                inputs[key] = x.half()
            calls = []
            for index, (name, m, n, k, bias, activation, key) in enumerate(rows):
                calls.append(pkg.LinearCall(inputs[key], self.weights[index], self.biases[index], activation))
            plan = ops.plan(calls)
            self.inputs.append(inputs)
            self.outputs.append([call.y for call in plan.calls])
            self.plans.append(plan)
        self.h2d_bytes = sum(m * k * 2 for (m, k) in self.input_shapes.values())
        self.d2h_bytes = sum(int(y.numel()) * 2 for y in self.outputs[0])
        self.working_set = self.h2d_bytes + self.d2h_bytes + sum(m * k for (m, k) in self.input_shapes.values())

    def launches_per_step(self) -> int:
        return self.plans[0].launches


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.process = None
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--id={gpu_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.process = None
        self.marks = []

    def mark(self, label: str):
        self.marks.append((label, time.time()))

    def stop(self):
        if self.process is not None:
            self.process.terminate()
            try:
                self.process.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.process.kill()
        self.file.flush()
        self.file.seek(0)
        rows = [line.strip().split(", ") for line in self.file.read().splitlines() if line.strip()]
        self.file.close()
        os.unlink(self.file.name)
        clocks, maxima, reasons = [], [], set()
        for row in rows:
            try:
                clock = float(row[1])
                maximum = float(row[2])
            except (ValueError, IndexError):
                continue
            clocks.append(clock)
            maxima.append(maximum)
            for name, value in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), row[5:9]):
                if value.strip().lower().startswith("active"):
                    reasons.add(name)
        loaded = [c for c in clocks if c > 0.5 * max(maxima)] if clocks else []
        return {"sm_mhz": statistics.median(loaded or clocks) if clocks else None,
                "sm_max_mhz": max(maxima) if maxima else None, "reasons": sorted(reasons), "samples": len(clocks),
                "samples_under_load": len(loaded)}


def library_int8_rate(torch, steps: int = 20):
    """INT8 x INT8 -> INT32 rate of the vendor library GEMM (torch._int_mm -> cuBLASLt) on an
    [8192, 8192] x [8192, 8192] product, device-timed: the rate a plain library GEMM without any
    epilogue reaches on this GPU, reported beside the roofline for context (it is not the peak the
    roofline fraction uses)."""
    try:
        a = torch.randint(-127, 128, (8192, 8192), dtype=torch.int8, device="cuda")
        b = torch.randint(-127, 128, (8192, 8192), dtype=torch.int8, device="cuda")
        for _ in range(3):
            torch._int_mm(a, b)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            torch._int_mm(a, b)
        stop.record()
        torch.cuda.synchronize()
        seconds = start.elapsed_time(stop) * 1e-3 / steps
        return {"value": 2.0 * 8192 ** 3 / seconds / 1e12, "unit": "TOPS", "what": "torch._int_mm (cuBLASLt) 8192^3, no epilogue"}
    except Exception as error:  # the library call is context only; the bench does not depend on it
        return {"value": None, "unit": "TOPS", "what": f"torch._int_mm unavailable: {error}"}


# ------------------------------------------------------------------------------------------------
# CPU arms
# ------------------------------------------------------------------------------------------------
def cpu_single_core_baseline(budget_seconds: float = 15.0):
    """The reference's scalar `linear_2d` + `geglu` on a row slice of the FP16 GEGLU projection
    X[rows,640] x W[5120,640]: one host core."""
    from oracle import oracle as O
    import helpers as H
    w = H.make_weight(7, 5120, 640)
    bias = H.make_bias(7, 5120)
    use_reference = O.ref_available()

    def run(rows):
        x = H.make_activations(7, rows, 640).astype(np.float32)
        start = time.perf_counter()
        if use_reference:
            y = O.ref_linear_2d(x, w, bias)
            O.ref_geglu(y)
        else:
            O.lib().orc_set_threads(1)
            y = O.linear_f32(x, w.astype(np.float32), bias.astype(np.float32))
            O.geglu_f32(y)
        return time.perf_counter() - start

    probe_rows = 32
    probe = run(probe_rows)
    rows = int(max(32, min(8192, probe_rows * budget_seconds / max(probe, 1e-6))))
    elapsed = run(rows)
    ops = 2.0 * rows * 5120 * 640
    return {"value": ops / elapsed / 1e12, "unit": UNIT, "cores": 1, "kind": "reference" if use_reference else "port",
            "sample": f"linear_2d+geglu, FP16 weights, X[{rows},640] x W[5120,640] of the [8192,640] GEGLU projection, "
                      f"{elapsed:.1f} s single-threaded"}


def reference_arm(args, rows, description):
    """Times the reference's threaded AVX2 Linear on a bounded row sample of every projection."""
    from oracle import oracle as O
    import helpers as H
    use_reference = O.ref_available()
    threads = O.ref_hardware_threads() if use_reference else O.threads()
    sample_rows = args.reference_rows
    problems = []
    for index, (name, m, n, k, bias, activation, key) in enumerate(rows):
        mm = min(m, sample_rows)
        x = H.make_activations(index, mm, k).astype(np.float32)
        w = H.make_weight(index, n, k)
        b = H.make_bias(index, n) if bias else None
        problems.append((x, w, b, activation, 2.0 * mm * n * k))
    ops_per_step = sum(p[4] for p in problems)

    def step():
        for x, w, b, activation, _ in problems:
            if use_reference:
                y = O.ref_linear_threaded(x, w, b, 0)
                if activation == 4:
                    O.ref_geglu(y)
            else:
                y = O.linear_f32(x, w.astype(np.float32), None if b is None else b.astype(np.float32))
                if activation == 4:
                    O.geglu_f32(y)

    for _ in range(args.warmup):
        step()
    start = time.perf_counter()
    for _ in range(args.steps):
        step()
    elapsed = time.perf_counter() - start
    value = ops_per_step * args.steps / elapsed / 1e12
    sample = (f"threaded AVX2 Linear of the reference (dense FP16 weights; it has no CPU INT8/FP8 arithmetic) on the first "
              f"{sample_rows} rows of every projection, {threads} host threads")
    return {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": elapsed / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": description, "sample_rows": sample_rows},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "reference" if use_reference else "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


# ------------------------------------------------------------------------------------------------
# main
# ------------------------------------------------------------------------------------------------
def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=None)
    parser.add_argument("--warmup", type=int, default=None)
    parser.add_argument("--workload", default="layerset640_int8")
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--reference-rows", type=int, default=256)
    parser.add_argument("--e2e-steps", type=int, default=None)
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--library-rate", action="store_true",
                        help="also time the vendor library's plain INT8 GEMM (context for the roofline; off by default so "
                             "that the default run launches this repository's kernels only)")
    args = parser.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rows, kind, description = workload_rows(args.workload)

    if args.impl == "reference":
        if args.steps is None:
            args.steps = 5
        if args.warmup is None:
            args.warmup = 1
        if rank == 0:
            print(json.dumps(reference_arm(args, rows, description)), flush=True)
        return 0

    import torch
    import torch.distributed as dist

    if args.steps is None:
        args.steps = 2000 if args.workload.startswith("layerset") else (20 if args.workload.startswith("unetstep_") else 200)
    if args.warmup is None:
        args.warmup = 20
    args.warmup = max(args.warmup, 3)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    torch.cuda.set_device(local_rank)
    distributed = world > 1
    if distributed:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    pkg = importlib.import_module("sdxl-end2end_b200")
    peaks = load_peaks()
    sets = 3 if args.workload.startswith("layerset") else 1
    # scratch for the quantised copy of every distinct input of a step (bytes + per-row scales)
    unique_inputs = {key: (m, k) for (_, m, _, k, _, _, key) in rows}
    scratch = sum(m * k + 4 * m + 1024 for (m, k) in unique_inputs.values())
    context = pkg.Context(local_rank, workspace_bytes=max(1 << 30, int(scratch * 1.1)))
    ops = pkg.Ops(context)
    work = DeviceWorkload(pkg, ops, rows, kind, sets)
    ops_per_step = total_ops(rows)
    stream = torch.cuda.current_stream()

    def barrier():
        torch.cuda.synchronize()
        if distributed:
            dist.barrier()

    sampler = ClockSampler(local_rank) if rank == 0 else None

    # ---- device-resident throughput --------------------------------------------------------------
    for step in range(args.warmup):
        work.plans[step % sets].run()
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if sampler:
        sampler.mark("timed_start")
    start.record(stream)
    for step in range(args.steps):
        work.plans[step % sets].run()
    stop.record(stream)
    torch.cuda.synchronize()
    if sampler:
        sampler.mark("timed_stop")
    elapsed_ms = start.elapsed_time(stop)
    barrier()
    if distributed:
        tensor = torch.tensor([elapsed_ms], device="cuda")
        dist.all_reduce(tensor, op=dist.ReduceOp.MAX)
        elapsed_ms = float(tensor.item())
    value = world * ops_per_step * args.steps / (elapsed_ms * 1e-3) / 1e12

    # ---- per-kernel times (second pass over the same steps, event pairs around each launch) --------
    context.profile(True)
    context.kernel_times()
    for step in range(args.steps):
        work.plans[step % sets].run()
    kernel_times = context.kernel_times()
    context.profile(False)
    gemm_ms, gemm_launches = kernel_times["gemm"]
    quant_ms = kernel_times["quant_int8"][0] + kernel_times["quant_fp8"][0]
    quant_launches = kernel_times["quant_int8"][1] + kernel_times["quant_fp8"][1]
    gemm_launches_per_step = max(gemm_launches // max(args.steps, 1), 1)
    gemm_ms_per_launch = gemm_ms / max(args.steps, 1)      # all GEMM launches of one step together
    eight_bit = kind in ("int8", "e4m3", "e5m2")
    tensor_peak = peaks["bf16_tflops"] * (2.0 if eight_bit else 1.0)
    achieved = ops_per_step / (gemm_ms_per_launch * 1e-3) / 1e12 if gemm_ms_per_launch > 0 else 0.0
    quant_bytes = sum((m * k * 3 + (4 * m if kind == "int8" else 0)) for (m, k) in work.input_shapes.values()) if eight_bit else 0
    quant_ms_per_step = quant_ms / max(args.steps, 1)
    quant_gbs = quant_bytes / (quant_ms_per_step * 1e-3) / 1e9 if (quant_bytes and quant_ms_per_step > 0) else 0.0
    roofline = {
        "bound": "tensor", "kernel": "sdxlq_umma_gemm_kernel", "achieved": achieved, "peak": tensor_peak, "unit": "TFLOP/s",
        "frac": achieved / tensor_peak, "traffic": TRAFFIC_BYTES.get(args.workload),
        "peak_source": (f"{peaks['source']} bf16 {peaks['bf16_tflops']} TFLOP/s x2 for 8-bit operands" if eight_bit
                        else f"{peaks['source']} bf16"),
        "launch_ms": gemm_ms_per_launch, "ops_per_launch": ops_per_step, "gemm_launches_per_step": gemm_launches_per_step,
        "quantize_kernel": {"bound": "hbm", "achieved": quant_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                            "bytes_per_step": quant_bytes, "ms_per_step": quant_ms_per_step},
    }
    roofline["quantize_kernel"]["frac"] = roofline["quantize_kernel"]["achieved"] / peaks["hbm_gbs"]
    if rank == 0 and kind == "int8" and args.library_rate:
        roofline["library_int8_gemm"] = library_int8_rate(torch)

    # ---- end to end: pinned host inputs -> device, run, results -> pinned host ----------------------
    # (skipped when one step moves more than 16 GB over PCIe: pinned host copies of that size are not
    # what this measurement is for; only the sharded UNet-step workloads are that large)
    e2e_skipped = work.h2d_bytes + work.d2h_bytes > (16 << 30)
    e2e_value, e2e_seconds, e2e_steps = None, 0.0, 0
    if not e2e_skipped:
        e2e_steps = args.e2e_steps or max(3, min(args.steps, 20))
        host_inputs = [{key: torch.empty(x.shape, dtype=x.dtype).pin_memory().copy_(x) for key, x in work.inputs[s].items()}
                       for s in range(min(sets, 2))]
        host_outputs = [[torch.empty(y.shape, dtype=y.dtype).pin_memory() for y in work.outputs[s]] for s in range(min(sets, 2))]
        copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
        # Per buffer set: inputs uploaded / plan finished / outputs downloaded. The upload of step i + 1
        # waits only for the plan that last read its input buffers, so it overlaps the download of step
        # i (PCIe is full duplex); the plan waits for its inputs and for the download that last read
        # its output buffers.
        uploaded = [torch.cuda.Event() for _ in host_inputs]
        computed = [torch.cuda.Event() for _ in host_inputs]
        downloaded = [torch.cuda.Event() for _ in host_inputs]
        for s in range(len(host_inputs)):
            computed[s].record(stream)
            downloaded[s].record(copy_out)

        def e2e_step(step):
            s = step % len(host_inputs)
            with torch.cuda.stream(copy_in):
                copy_in.wait_event(computed[s])
                for key, host in host_inputs[s].items():
                    work.inputs[s][key].copy_(host, non_blocking=True)
                uploaded[s].record(copy_in)
            stream.wait_event(uploaded[s])
            stream.wait_event(downloaded[s])
            work.plans[s].run()
            computed[s].record(stream)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(computed[s])
                for host, y in zip(host_outputs[s], work.outputs[s]):
                    host.copy_(y, non_blocking=True)
                downloaded[s].record(copy_out)

        for step in range(2):
            e2e_step(step)
        barrier()
        wall = time.perf_counter()
        for step in range(e2e_steps):
            e2e_step(step)
        torch.cuda.synchronize()
        e2e_seconds = time.perf_counter() - wall
        barrier()
        if distributed:
            tensor = torch.tensor([e2e_seconds], device="cuda")
            dist.all_reduce(tensor, op=dist.ReduceOp.MAX)
            e2e_seconds = float(tensor.item())
        e2e_value = world * ops_per_step * e2e_steps / e2e_seconds / 1e12
    context.check()

    clocks = sampler.stop() if sampler else None
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_baseline = cpu_single_core_baseline()

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True,
            "scaling": "strong" if args.workload.startswith("unetstep_") else "weak", "vs_baseline": None,
            "dtype": {"int8": "int8", "e4m3": "fp8_e4m3", "e5m2": "fp8_e5m2"}.get(kind, "f16"), "data": "synthetic",
            "config": {"workload": description, "name": args.workload, "projections": len(rows),
                       "ops_per_step": ops_per_step, "parallelism": f"dp{world} (replicated weights, no collective)",
                       "l2": (f"{sets} rotating input/output sets, {sets * work.working_set / 1e6:.0f} MB touched per cycle "
                              f"(> {L2_BYTES / 1e6:.0f} MB L2)") if sets > 1 else
                             f"working set {work.working_set / 1e6:.0f} MB per step (> {L2_BYTES / 1e6:.0f} MB L2)",
                       "timing": "CUDA events on the launching stream, max over ranks"},
            "clocks": clocks,
            **({"unet_steps_per_s_projections_only": 1e3 / (elapsed_ms / args.steps)} if args.workload.startswith("unetstep_") else {}),
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": work.h2d_bytes, "d2h_bytes_per_step": work.d2h_bytes,
                    "steps": e2e_steps, "ms_per_step": (e2e_seconds / e2e_steps * 1e3) if e2e_steps else None},
            "gpu_launches": work.launches_per_step() * args.steps,
            "launches_per_step": work.launches_per_step(),
            "roofline": roofline,
            "kernel_ms_per_step": {name: times[0] / args.steps for name, times in kernel_times.items()},
            "cpu_baseline": cpu_baseline,
            "library": pkg.load_library().sdxlq_build_info().decode(),
        }
        print(json.dumps(line), flush=True)
    if distributed:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
