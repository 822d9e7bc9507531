#!/usr/bin/env python
"""Benchmark of the SDXL UNet quantized-Linear path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Default workload `unetloop_e4m3`: the synthetic SDXL Base UNet denoising loop at 1024^2 for a fixed
job of 8 images x CFG 2 (UNet batch 16), FP8 E4M3 projections (per-output-channel weight scales,
native FP8 activations), the transformer LayerNorms fused with the quantisers of the projections
they feed, FP16 convolutions / attention from PyTorch and a channels-last GroupNorm kernel around them, Euler
sampler, sigma schedule of 20 steps. A "step" is one denoising step of the whole job: scale the
latents, one UNet forward over [uncond | cond], CFG combine, Euler update; every 20 steps a new
generation starts and the cross-attention K/V projections are recomputed once. With N ranks the
images are sharded (8 / N images, UNet batch 16 / N per rank), weights are replicated and there
is no collective in the step: strong scaling. `value` = denoising steps per second of the job.
Other precisions: `unetloop_e5m2`, `unetloop_int8`, `unetloop_f16`.

Projection-only workloads (`--workload NAME`; the N = 1 default run also times them and reports
them under `other_workloads`): `layerset640_int8` / `layerset640_int8_g64` (640-dim layer set, W8A8
INT8 ConvRot, group 256 rule resp. groups of 64), `layerset1280_fp8` (1280-dim set, FP8 E4M3, plus
the skinny cross-attention K/V GEMM), `unet743_int8` / `unet743_e5m2` (all 743 projections of a UNet
step as one grouped launch), `geglu640_f16` (the single FP16 GEGLU projection [8192,640]x[5120,640]),
`crossattn_kv_int8`, `unetstep_<kind>` (projections of one step, sharded like the loop).

Rank 0 prints ONE JSON line. Device times come from CUDA events on the launching stream, max over
ranks. `e2e` is the same metric through the public API with host buffers: every step copies its
inputs from pinned host memory and reads its result back. `--impl reference` times the reference's
own CPU Linear (compiled from the reference sources, else the CPU port) on a bounded sample of the
same projections with all host threads and converts it to the same metric.
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

L2_BYTES = 126 * 1024 * 1024
JOB_IMAGES = 8                 # images of the fixed job (x CFG 2 = UNet batch 16)
GENERATION_STEPS = 20          # denoising steps per generation (sigma schedule length)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as handle:
            peaks = json.load(handle)
        return {"hbm_gbs": float(peaks["hbm_gbs"]), "bf16_tflops": float(peaks["bf16_tflops"]),
                "bf16_tflops_sustained": float(peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def package():
    return importlib.import_module("sdxl-end2end_b200")


def unet_shapes():
    return importlib.import_module("sdxl-end2end_b200.unet_shapes")


# ------------------------------------------------------------------------------------------------
# projection-only workloads
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


def workload_rows(name: str, world: int = 1):
    """-> (rows, kind, convrot group, description)"""
    if name in ("layerset640_int8", "layerset640_int8_g64"):
        group = 64 if name.endswith("g64") else 256
        rule = "groups of 64: every projection rotates" if group == 64 else "group 256 rule: only K=2560 rotates"
        return layer_set(640, 8192, 0), "int8", group, (
            f"SDXL UNet 640-dim layer set, W8A8 INT8 ConvRot ({rule}), 1024^2 CFG batch 2: q,k,v,out [8192,640]x[640,640]; "
            "ff.net.0.proj+GEGLU [8192,640]x[5120,640]; ff.net.2 [8192,2560]x[640,2560]")
    if name == "layerset1280_fp8":
        return layer_set(1280, 2048, 154), "e4m3", 0, (
            "SDXL UNet 1280-dim layer set, FP8 E4M3 per-channel weights, native FP8 activations, M=2048; plus "
            "cross-attention to_k/to_v [154,2048]x[1280,2048]")
    if name == "geglu640_f16":
        return [("ff.net.0.proj", 8192, 5120, 640, True, 4, "norm3")], "f16", 0, (
            "single SDXL GEGLU ff.net.0.proj Linear, FP16 weights: X [8192,640] x W [5120,640] + bias, GEGLU")
    if name == "crossattn_kv_int8":
        rows = [(p.name, p.m, p.n, p.k, p.bias, p.activation, p.input_key) for p in unet_shapes().unet_projections(2)
                if ".attn2.to_k" in p.name or ".attn2.to_v" in p.name]
        return rows, "int8", 256, (
            f"the {len(rows)} cross-attention to_k/to_v projections [154,2048]x[640|1280,2048] of one SDXL UNet step, INT8 "
            "ConvRot, one grouped launch (HBM-bound: weights are read once)")
    if name.startswith("unetstep_"):
        kind = name.split("_", 1)[1]
        if kind not in ("int8", "e4m3", "e5m2"):
            raise SystemExit(f"unknown workload {name}")
        if 16 % world != 0 or 16 // world < 2:
            raise SystemExit("unetstep shards 8 CFG pairs: 1, 2, 4 or 8 ranks")
        local_batch = 16 // world
        rows = [(p.name, p.m, p.n, p.k, p.bias, p.activation, p.input_key) for p in unet_shapes().unet_projections(local_batch)]
        return rows, kind, 256, (
            f"all 743 rank-2 projections of one SDXL UNet step at 1024^2 for {local_batch // 2} of 8 images x CFG 2 (UNet batch "
            f"{local_batch} of 16 on this rank), one grouped launch, {kind}; projections only")
    if name in ("unet743_int8", "unet743_e5m2"):
        rows = [(p.name, p.m, p.n, p.k, p.bias, p.activation, p.input_key) for p in unet_shapes().unet_projections(2)]
        kind = "int8" if name.endswith("int8") else "e5m2"
        return rows, kind, 256, f"all 743 rank-2 projections of one SDXL UNet step at 1024^2, CFG batch 2, one grouped launch, {kind}"
    raise SystemExit(f"unknown workload {name}")


def total_ops(rows) -> float:
    return float(sum(2 * m * n * k for (_, m, n, k, _, _, _) in rows))


def minimum_bytes(rows, kind) -> float:
    """Bytes a GEMM launch must move at least: each distinct (quantised) input and each weight read
    once, each FP16 output written once."""
    element = 2 if kind == "f16" else 1
    inputs = {key: m * k * element for (_, m, _, k, _, _, key) in rows}
    weights = sum(n * k * element for (_, _, n, k, _, _, _) in rows)
    outputs = sum(m * (n // 2 if act == 4 else n) * 2 for (_, m, n, _, _, act, _) in rows)
    return float(sum(inputs.values()) + weights + outputs)


class DeviceWorkload:
    """Weights (quantised once), and `sets` rotating sets of inputs / outputs with one plan each."""

    def __init__(self, pkg, ops, rows, kind, group, sets, seed=1234):
        import torch
        self.pkg, self.ops, self.rows, self.kind = pkg, ops, rows, kind
        device = torch.device("cuda", torch.cuda.current_device())
        generator = torch.Generator(device=device)
        generator.manual_seed(seed)
        self.weights, self.biases, self.dense = [], [], []
        for index, (name, m, n, k, bias, activation, key) in enumerate(rows):
            w = (torch.randn((n, k), generator=generator, device=device, dtype=torch.float32) / (k ** 0.5)).half()
            if kind == "int8":
                options = pkg.INT8WeightLoadOptions(enable_convrot=True, convrot_group_size=group)
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

    def close(self):
        for plan in self.plans:
            plan.close()


def quantiser_bytes(input_shapes, kind) -> float:
    """Algorithmic bytes of the activation quantisers of one step: FP16 read + 8-bit write (+ one FP32
    scale per row for INT8). The FP8 quantiser needs the tensor-wide maximum before it can write a
    byte, so its input is read twice: 2 + 2 + 1 bytes per element."""
    if kind == "int8":
        return float(sum(m * k * 3 + 4 * m for (m, k) in input_shapes))
    if kind in ("e4m3", "e5m2"):
        return float(sum(m * k * 5 for (m, k) in input_shapes))
    return 0.0


def time_projection_workload(torch, pkg, context, ops, name, peaks, min_seconds=0.4, world=1, library=False):
    """Device-timed grouped plan of a projection-only workload: TOPS, per-kernel times, roofline."""
    rows, kind, group, description = workload_rows(name, world)
    sets = 3 if (name.startswith("layerset") or name.startswith("geglu")) else 1
    work = DeviceWorkload(pkg, ops, rows, kind, group, sets)
    ops_per_step = total_ops(rows)
    stream = torch.cuda.current_stream()
    for step in range(6):
        work.plans[step % sets].run()
    torch.cuda.synchronize()
    # size the timed region: at least `min_seconds`
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for step in range(3):
        work.plans[step % sets].run()
    stop.record(stream)
    torch.cuda.synchronize()
    probe_ms = start.elapsed_time(stop) / 3
    steps = int(max(10, min(20000, min_seconds * 1e3 / max(probe_ms, 1e-3))))
    start.record(stream)
    for step in range(steps):
        work.plans[step % sets].run()
    stop.record(stream)
    torch.cuda.synchronize()
    ms_per_step = start.elapsed_time(stop) / steps
    # per-kernel times: event pairs around every launch, second pass
    profile_steps = max(3, min(steps, 200))
    context.profile(True)
    context.kernel_times()
    for step in range(profile_steps):
        work.plans[step % sets].run()
    kernel_times = context.kernel_times()
    context.profile(False)
    gemm_ms = kernel_times["gemm"][0] / profile_steps
    quant_ms = (kernel_times["quant_int8"][0] + kernel_times["quant_fp8"][0]) / profile_steps
    eight_bit = kind != "f16"
    tensor_peak = peaks["bf16_tflops"] * (2.0 if eight_bit else 1.0)
    achieved = ops_per_step / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
    quant_bytes = quantiser_bytes(work.input_shapes.values(), kind)
    result = {
        "workload": description, "kind": kind, "projections": len(rows), "ops_per_step": ops_per_step,
        "tops": ops_per_step / (ms_per_step * 1e-3) / 1e12, "ms_per_step": ms_per_step, "steps_timed": steps,
        "launches_per_step": work.launches_per_step(),
        "gemm": {"ms": gemm_ms, "tops": achieved, "frac_of_peak": achieved / tensor_peak, "peak_tflops": tensor_peak,
                 "min_bytes": minimum_bytes(rows, kind),
                 "hbm_frac_at_min_bytes": (minimum_bytes(rows, kind) / (gemm_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]) if gemm_ms > 0 else None},
        "quantize": {"ms": quant_ms, "bytes": quant_bytes,
                     "gbs": quant_bytes / (quant_ms * 1e-3) / 1e9 if quant_ms > 0 else None,
                     "frac_of_hbm": (quant_bytes / (quant_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]) if quant_ms > 0 else None},
        "l2": f"{sets} rotating input/output sets, {sets * work.working_set / 1e6:.0f} MB per cycle" if sets > 1
              else f"working set {work.working_set / 1e6:.0f} MB per step",
    }
    if library:
        result["library_same_shapes"] = library_same_shapes(torch, ops, rows, kind, work)
    work.close()
    del work
    torch.cuda.empty_cache()
    return result


def library_same_shapes(torch, ops, rows, kind, work):
    """The vendor library's GEMM in place of this repository's GEMM kernel, on the same shapes and on
    the same quantised activations (produced beforehand by this repository's quantiser, not timed):
    per projection one cuBLASLt GEMM (torch._int_mm = I8 x I8 -> I32 for INT8, as int8_convrot_linear
    calls it, src/cuda/int8_convrot.cu:634-698; torch._scaled_mm = FP8 x FP8 -> FP16 with tensor-wide
    device scales, as native_fp8_linear does, src/cuda/ops_blas.cpp:153-225; a plain FP16 matmul), then
    the separate kernels the reference runs after it: dequantise (int8_convrot.cu:388-402), bias,
    bias + GEGLU (ops_blas.cpp:388-397). Compare `ms_per_step` with this repository's GEMM kernel time
    (`gemm.ms`), which includes all of that in its epilogue. CUDA events, outside the timed region."""
    import torch.nn.functional as F
    try:
        prepared = []
        quantised = {}
        for index, (name, m, n, k, bias, activation, key) in enumerate(rows):
            x = work.inputs[0][key]
            w = work.weights[index]
            b = work.biases[index]
            if kind == "int8":
                tag = (key, w.convrot_group_size)
                if tag not in quantised:
                    quantised[tag] = ops.quantize_int8(x, w.convrot_group_size)
                xq, a_scales = quantised[tag]
                prepared.append((xq, a_scales, w.data, w.scales, b, activation, m))
            elif kind in ("e4m3", "e5m2"):
                dtype = torch.float8_e4m3fn if kind == "e4m3" else torch.float8_e5m2
                if key not in quantised:
                    q = ops.quantize_fp8(x, w.type)
                    quantised[key] = (q.data.view(dtype), q.scales)
                xq, a_scale = quantised[key]
                prepared.append((xq, a_scale, w.data.view(dtype), w.scales, b, activation, m))
            else:
                prepared.append((x, None, w.data, None, b, activation, m))
        torch.cuda.synchronize()
        one = torch.ones((), device="cuda")

        def epilogue(y, b, activation):
            if activation == 4:
                y = y + b
                value, gate = y.chunk(2, dim=-1)
                return value * F.gelu(gate)
            return y + b if b is not None else y

        skipped = []

        def step():
            outs = []
            for xq, a_scale, w, w_scales, b, activation, m in prepared:
                if kind == "int8":
                    if m <= 16:
                        skipped.append(m)                 # _int_mm needs more than 16 rows
                        continue
                    acc = torch._int_mm(xq, w.t())
                    y = (acc.float() * a_scale[:, None] * w_scales[None, :]).half()
                elif kind in ("e4m3", "e5m2"):
                    if m % 16 or w.shape[0] % 16 or w.shape[1] % 16:
                        skipped.append(m)                 # the library's FP8 GEMM wants multiples of 16
                        continue
                    y = torch._scaled_mm(xq, w.t(), scale_a=a_scale.reshape(()), scale_b=one, out_dtype=torch.float16)
                    y = y * w_scales[None, :].half()      # per-output-channel weight scale: one more pass
                else:
                    y = xq @ w.t()
                outs.append(epilogue(y, b, activation))
            return outs

        for _ in range(3):
            step()
        torch.cuda.synchronize()
        skipped.clear()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        repeats = 20
        start.record()
        for _ in range(repeats):
            step()
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / repeats
        return {"ms_per_step": ms, "tops": total_ops(rows) / (ms * 1e-3) / 1e12, "projections_skipped": len(skipped) // repeats,
                "what": "cuBLASLt GEMM (torch._int_mm / torch._scaled_mm / matmul) + separate dequant, bias, GEGLU kernels on "
                        "activations quantised beforehand; to be compared with gemm.ms"}
    except Exception as error:      # context only: the benchmark does not depend on the library arm
        return {"ms_per_step": None, "tops": None, "what": f"library arm unavailable: {type(error).__name__}: {error}"}


def time_norm_quantize(torch, pkg, ops, peaks):
    """The LayerNorm kernels on the row counts of the UNet loop (UNet batch 16 at 1024^2: 65536 tokens x 640,
    16384 tokens x 1280), four rotating inputs per shape so that every launch reads from HBM (4 x 84 MB and
    4 x 42 MB against 132 MB of L2): FP16 LayerNorm, LayerNorm fused with the FP8 / INT8 quantiser, and the
    stand-alone quantisers for comparison. GB/s are algorithmic bytes (FP16 in/out 2 + 2; FP8 2 + 2 + 1: the
    tensor-wide maximum needs a pass of its own; INT8 2 + 1) over the CUDA-event time of replayed graphs of the
    launches (device time without the host's cost per call)."""
    result = {}
    for rows, width in ((65536, 640), (16384, 1280)):
        sets = 4
        xs = [torch.randn(rows, width, device="cuda", dtype=torch.float16) for _ in range(sets)]
        gamma = torch.ones(width, device="cuda", dtype=torch.float16)
        beta = torch.zeros(width, device="cuda", dtype=torch.float16)
        out = torch.empty(rows, width, device="cuda", dtype=torch.float16)
        fp8 = pkg.Weight(torch.zeros((16, width), dtype=torch.uint8, device="cuda"), pkg.ScalarType.Float8E4M3, 16, width,
                         torch.ones(1, device="cuda"), pkg.FP8ScaleMode.TensorWide)
        group = 256 if width % 256 == 0 else 0
        int8 = pkg.Weight(torch.zeros((16, width), dtype=torch.int8, device="cuda"), pkg.ScalarType.Int8, 16, width,
                          torch.ones(16, device="cuda"), pkg.FP8ScaleMode.PerOutputChannel, pkg.FP8StorageLayout.RowMajorNK, group)
        ys = [ops.layer_norm(x, gamma, beta) for x in xs]
        cases = {
            "layer_norm_f16": (4, lambda i: ops.layer_norm(xs[i], gamma, beta, out=out)),
            "layer_norm_to_fp8": (5, lambda i: ops.layer_norm_quantized(xs[i], gamma, beta, fp8)),
            "layer_norm_to_int8": (3, lambda i: ops.layer_norm_quantized(xs[i], gamma, beta, int8)),
            "quantize_fp8": (5, lambda i: ops.quantize_fp8(ys[i], pkg.ScalarType.Float8E4M3)),
            "quantize_int8": (3, lambda i: ops.quantize_int8(ys[i], group)),
        }
        shape = {}
        for name, (bytes_per_element, call) in cases.items():
            for i in range(sets):
                call(i)
            torch.cuda.synchronize()
            # One pass over the rotating inputs captured as a graph and replayed: device time only (a call through
            # the Python mirror allocates its outputs and costs the host 15 to 20 us, more than some of these kernels).
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                ops.ctx.set_stream(torch.cuda.current_stream())
                held = [call(i) for i in range(sets)]
            ops.ctx.set_stream(torch.cuda.current_stream())
            graph.replay()
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            repeats = 10
            start.record()
            for r in range(repeats):
                graph.replay()
            stop.record()
            torch.cuda.synchronize()
            ms = start.elapsed_time(stop) / (repeats * sets)
            del graph, held
            gbs = rows * width * bytes_per_element / (ms * 1e-3) / 1e9
            shape[name] = {"ms": ms, "gbs": gbs, "frac_of_hbm": gbs / peaks["hbm_gbs"], "bytes_per_element": bytes_per_element}
        shape["int8_group"] = group
        result[f"{rows}x{width}"] = shape
        del xs, ys, out
    torch.cuda.empty_cache()
    return result


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
        self.window = [None, None]

    def mark_start(self):
        self.window[0] = time.time()

    def mark_stop(self):
        self.window[1] = time.time()

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


# ------------------------------------------------------------------------------------------------
# CPU arms
# ------------------------------------------------------------------------------------------------
def cpu_single_core_rate(budget_seconds: float = 15.0):
    """The reference's scalar `linear_2d` + `geglu` on a row slice of the FP16 GEGLU projection
    X[rows,640] x W[5120,640]: one host core. Returns (TOPS, kind, description)."""
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
    return ops / elapsed / 1e12, ("reference" if use_reference else "port"), (
        f"linear_2d+geglu, FP16 weights, X[{rows},640] x W[5120,640] of the [8192,640] GEGLU projection, {elapsed:.1f} s single-threaded")


def reference_threaded_rate(rows_table, sample_rows, steps, warmup):
    """The reference's threaded AVX2 Linear on the first `sample_rows` rows of every projection:
    (seconds per sample step, ops per sample step, threads, kind)."""
    from oracle import oracle as O
    import helpers as H
    use_reference = O.ref_available()
    threads = O.ref_hardware_threads() if use_reference else O.threads()
    problems = []
    for index, (name, m, n, k, bias, activation, key) in enumerate(rows_table):
        mm = min(m, sample_rows)
        x = H.make_activations(index, mm, k).astype(np.float32)
        w = H.make_weight(index % 64, n, k)            # 64 distinct weight draws are plenty for a timing
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

    for _ in range(warmup):
        step()
    start = time.perf_counter()
    for _ in range(steps):
        step()
    elapsed = time.perf_counter() - start
    return elapsed / steps, ops_per_step, threads, ("reference" if use_reference else "port")


def reference_device_projections(rows_table, kind):
    """Context for the reference arm, not its value: the reference's own CUDA operators (its Ops class
    compiled unmodified for sm_100, oracle/_ref/libsdxl_ref_cuda.so) timed on this box's GPU for every
    distinct projection shape of the job at full size, operands resident, CUDA events on the reference's
    stream. Each call is what the reference runs per projection: its FP8 quantiser + cuBLASLt FP8 GEMM
    (tensor-wide weight scale) or cuBLASLt FP16 GEMM, then its bias / activation kernel. The INT8
    translation unit of the reference does not compile with this toolchain, so INT8 has no such figure."""
    try:
        from oracle import oracle as O
        if kind == "int8":
            return {"unavailable": "the reference's INT8 translation unit does not compile with nvcc 12.9"}
        if not O.RefCuda.available():
            return {"unavailable": "oracle/_ref/libsdxl_ref_cuda.so was not built"}
        import torch
        if not torch.cuda.is_available():
            return {"unavailable": "no GPU"}
        reference = O.RefCuda()
        shapes = {}
        for (name, m, n, k, bias, activation, key) in rows_table:
            shapes[(m, n, k, bool(bias), int(activation))] = shapes.get((m, n, k, bool(bias), int(activation)), 0) + 1
        total_ms, ops, fallbacks = 0.0, 0.0, 0
        for (m, n, k, bias, activation), count in shapes.items():
            if kind in ("e4m3", "e5m2") and (m % 16 or n % 16 or k % 16):
                fallbacks += count                 # the reference takes its weight-only kernel for these
            ms = reference.time_linear(m, k, n, kind, activation if bias else 0, bias, False, 2, 5)
            total_ms += ms * count
            ops += 2.0 * m * n * k * count
        reference.shutdown()
        return {"projection_ms_per_step": total_ms, "projection_tops": ops / (total_ms * 1e-3) / 1e12,
                "distinct_shapes": len(shapes), "projections": len(rows_table), "weight_only_fallbacks": fallbacks,
                "what": "sum over the job's projections of the reference's CUDA Ops::linear / linear_activation device time "
                        "on this GPU (sm_100 build of the reference's sources), per call: quantise + GEMM + bias/activation kernel"}
    except Exception as error:
        return {"unavailable": f"{type(error).__name__}: {error}"}


def reference_arm(args):
    """`--impl reference`: the reference's CPU Linear on a bounded sample, in this arm's metric."""
    loop = args.workload.startswith("unetloop_")
    if loop:
        rows = [(p.name, p.m, p.n, p.k, p.bias, p.activation, p.input_key) for p in unet_shapes().unet_projections(2 * JOB_IMAGES)]
        description = unetloop_description(args.workload.split("_", 1)[1])
        sample_rows = args.reference_rows or 16
    else:
        rows, _, _, description = workload_rows(args.workload, 1)
        sample_rows = args.reference_rows or 256
    seconds, sample_ops, threads, kind = reference_threaded_rate(rows, sample_rows, args.steps, args.warmup)
    tops = sample_ops / seconds / 1e12
    full_ops = total_ops(rows)
    sample = (f"threaded AVX2 Linear of the reference (dense FP16 weights; it has no CPU INT8/FP8 arithmetic) on the first "
              f"{sample_rows} rows of every projection ({sample_ops / 1e9:.1f} GOP per sample step), {threads} host threads")
    if loop:
        # steps/s of the job if its projections ran at the sampled CPU rate; the CPU reference's
        # convolutions, norms and attention would add to the step time, so this bounds it from above
        value = tops * 1e12 / full_ops
        metric, unit = "sdxl_unet_steps_per_s", "steps/s"
        sample += (f"; converted to denoising steps/s of the 8-image x CFG 2 job by its {full_ops / 1e12:.2f} TOP of projections per step "
                   "(projections only: an upper bound for the CPU reference's full step)")
        ms_per_step = 1e3 / value
    else:
        value, metric, unit = tops, "quantized_linear_tops", "TOPS"
        ms_per_step = seconds * 1e3
    return {
        "impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong" if (loop or args.workload.startswith("unetstep_")) else "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": description, "name": args.workload, "sample_rows": sample_rows, "cpu_tops": tops},
        "cpu_baseline": {"value": value, "unit": unit, "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "reference_device": reference_device_projections(
            rows, next((k for k in ("int8", "e4m3", "e5m2", "f16") if k in args.workload), "e4m3" if "fp8" in args.workload else "f16")),
    }


# ------------------------------------------------------------------------------------------------
# the UNet loop
# ------------------------------------------------------------------------------------------------
def unetloop_description(kind: str) -> str:
    names = {"e4m3": "FP8 E4M3 (per-output-channel weight scales, native FP8 activations)",
             "e5m2": "FP8 E5M2 (per-output-channel weight scales, native FP8 activations)",
             "int8": "W8A8 INT8 ConvRot (group 256 rule)", "f16": "FP16"}
    batch = 2 * JOB_IMAGES
    return (f"synthetic SDXL Base UNet denoising loop, 1024^2, {JOB_IMAGES} images x CFG 2 (latents [{batch},4,128,128], "
            f"context [{batch},77,2048], pooled [{batch},1280]), {GENERATION_STEPS} Euler steps per generation, random-init weights; projections {names[kind]}; "
            "transformer LayerNorms fused with the activation quantisers (library kernel); FP16 convolutions / attention "
            "(PyTorch, channels-last), GroupNorm + SiLU on the channels-last activations (harness kernel of the library)")


def run_unet_loop(args, torch, dist, pkg, rank, local_rank, world, peaks):
    kind = args.workload.split("_", 1)[1]
    if kind not in ("e4m3", "e5m2", "int8", "f16"):
        raise SystemExit(f"unknown workload {args.workload}")
    if JOB_IMAGES % world != 0:
        raise SystemExit("the job has 8 images: 1, 2, 4 or 8 ranks")
    harness = importlib.import_module("sdxl-end2end_b200.unet_harness")
    sharding = importlib.import_module("sdxl-end2end_b200.sharding")
    first, end = sharding.shard_images(JOB_IMAGES, world, rank)
    images = end - first
    local_batch = 2 * images
    device = torch.device("cuda", local_rank)
    distributed = world > 1

    def barrier():
        torch.cuda.synchronize()
        if distributed:
            dist.barrier()

    # scratch: the largest quantised activation of a single call, and the K/V plan's shared input
    largest = max(local_batch * 16384 * 640, local_batch * 4096 * 2560, local_batch * 1024 * 5120)
    context = pkg.Context(local_rank, workspace_bytes=int(largest * 1.05) + (64 << 20))
    ops = pkg.Ops(context)
    # The loop's convolutions are PyTorch / cuDNN scaffolding: let cuDNN time its algorithms per shape once (during
    # the warm-up steps, before the graph capture). Its heuristic choice at one or two images per GPU was a
    # kernel that took 0.5 ms per launch: a fifth of the step.
    torch.backends.cudnn.benchmark = not args.no_cudnn_autotune
    unet = harness.UNetHarness(ops, harness.BASE_1_0, precision=kind, seed=0)
    loop = harness.EulerDenoiser(unet, images, 1024, 1024, GENERATION_STEPS, guidance_scale=5.0, use_graph=not args.no_graph)

    # the job's inputs, seeded per image so that every sharding sees the same job; host copies pinned
    def image_tensor(shape, seed, scale=1.0):
        generator = torch.Generator(device="cpu")
        generator.manual_seed(seed)
        return torch.randn(shape, generator=generator, dtype=torch.float32) * scale

    mine = range(first, first + images)
    noise = torch.stack([image_tensor((4, 128, 128), 1000 + i) for i in mine])
    cond = torch.stack([image_tensor((77, 2048), 2000 + i) for i in mine])
    uncond = torch.stack([image_tensor((77, 2048), 3000) for _ in mine])                 # the empty prompt, shared
    pooled_cond = torch.stack([image_tensor((1280,), 4000 + i) for i in mine])
    pooled_uncond = torch.stack([image_tensor((1280,), 5000) for _ in mine])
    host = {
        "latents": noise.pin_memory(),
        "context": torch.cat([uncond, cond]).half().pin_memory(),
        "pooled": torch.cat([pooled_uncond, pooled_cond]).half().pin_memory(),
        "time_ids": torch.tensor([[1024, 1024, 0, 0, 1024, 1024]] * local_batch, dtype=torch.float16).pin_memory(),
    }
    staged = {name: value.to(device) for name, value in host.items()}
    result_host = torch.empty((images, 4, 128, 128), dtype=torch.float32).pin_memory()
    h2d_bytes = sum(v.numel() * v.element_size() for v in host.values())
    d2h_bytes = result_host.numel() * 4

    def start_generation():
        loop.set_conditioning(staged["context"], staged["pooled"], staged["time_ids"])
        loop.set_latents(staged["latents"])

    stream = torch.cuda.current_stream()
    start_generation()
    for _ in range(max(args.warmup, 3)):
        loop.step()
    barrier()
    # The K steps are repeated until the timed region lasts about a second (clock samples, sustained
    # figure): estimate the step time from two more steps, agree on the count across ranks.
    probe_start, probe_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    probe_start.record(stream)
    loop.step()
    loop.step()
    probe_stop.record(stream)
    torch.cuda.synchronize()
    probe = torch.tensor([probe_start.elapsed_time(probe_stop) / 2], device=device)
    if distributed:
        dist.all_reduce(probe, op=dist.ReduceOp.MAX)
    repeats = int(max(1, min(50, -(-args.min_seconds * 1e3 // (float(probe.item()) * args.steps)))))

    sampler = ClockSampler(local_rank) if rank == 0 else None
    # ---- device-resident: K steps, a new generation every 20 ------------------------------------
    start_generation()
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if sampler:
        sampler.mark_start()
    if args.profiler_range:
        torch.cuda.profiler.start()         # a profiler attached with "--profile-from-start off" sees exactly these launches
    start.record(stream)
    for step in range(args.steps * repeats):
        if step and step % GENERATION_STEPS == 0:
            start_generation()
        loop.step()
    stop.record(stream)
    torch.cuda.synchronize()
    if args.profiler_range:
        torch.cuda.profiler.stop()
    if sampler:
        sampler.mark_stop()
    elapsed_ms = start.elapsed_time(stop) / repeats
    final_latents = loop.latents.clone()
    barrier()
    if distributed:
        tensor = torch.tensor([elapsed_ms], device=device)
        dist.all_reduce(tensor, op=dist.ReduceOp.MAX)
        elapsed_ms = float(tensor.item())
    ms_per_step = elapsed_ms / args.steps
    value = 1e3 / ms_per_step

    # ---- end to end: every step copies its inputs from pinned host memory and reads its result ----
    e2e_steps = args.e2e_steps or max(3, min(args.steps, GENERATION_STEPS))
    def e2e_step(step):
        for name in ("context", "pooled", "time_ids"):
            staged[name].copy_(host[name], non_blocking=True)
        if step % GENERATION_STEPS == 0:
            staged["latents"].copy_(host["latents"], non_blocking=True)     # a new generation starts from noise
            start_generation()
        else:
            loop.latents.copy_(result_host, non_blocking=True)              # the state the caller holds on the host
        loop.step()
        result_host.copy_(loop.latents, non_blocking=True)
        torch.cuda.current_stream().synchronize()       # the caller reads the step's result
    e2e_step(0)
    barrier()
    wall = time.perf_counter()
    for step in range(e2e_steps):
        e2e_step(step)
    torch.cuda.synchronize()
    e2e_seconds = time.perf_counter() - wall
    barrier()
    if distributed:
        tensor = torch.tensor([e2e_seconds], device=device)
        dist.all_reduce(tensor, op=dist.ReduceOp.MAX)
        e2e_seconds = float(tensor.item())
    e2e_value = e2e_steps / e2e_seconds
    clocks = sampler.stop() if sampler else None

    # ---- per-kernel times of the operator inside the loop (eager pass, event pairs per launch) ------
    projections = unet_shapes().unet_projections(local_batch)
    ops_per_forward = float(unet_shapes().total_ops(projections))
    kv_ops = float(sum(2 * p.m * p.n * p.k for p in projections if ".attn2.to_k" in p.name or ".attn2.to_v" in p.name))
    step_ops = ops_per_forward - kv_ops                          # the K/V projections run once per generation
    eager = harness.EulerDenoiser(unet, images, 1024, 1024, GENERATION_STEPS, guidance_scale=5.0, use_graph=False)
    eager.set_conditioning(staged["context"], staged["pooled"], staged["time_ids"])
    eager.set_latents(staged["latents"])
    eager.step()
    torch.cuda.synchronize()
    context.profile(True)
    context.kernel_times()
    profile_steps = 2
    eager_start, eager_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    eager_start.record(stream)
    for _ in range(profile_steps):
        eager.step()
    eager_stop.record(stream)
    kernel_times = context.kernel_times()
    context.profile(False)
    eager_ms = eager_start.elapsed_time(eager_stop) / profile_steps
    gemm_ms = kernel_times["gemm"][0] / profile_steps
    gemm_launches = kernel_times["gemm"][1] // profile_steps
    # the LayerNorm -> quantiser kernels do the quantisers' work for the inputs they feed (same algorithmic
    # bytes: the normalised tensor is read where the stand-alone quantiser would read its input)
    norm_ms = kernel_times["layer_norm"][0] / profile_steps
    norm_launches = kernel_times["layer_norm"][1] // profile_steps
    quant_ms = (kernel_times["quant_int8"][0] + kernel_times["quant_fp8"][0]) / profile_steps + (norm_ms if kind != "f16" else 0.0)
    quant_launches = (kernel_times["quant_int8"][1] + kernel_times["quant_fp8"][1]) // profile_steps + norm_launches
    small_launches = kernel_times["small"][1] // profile_steps
    launches_per_step = int(gemm_launches + quant_launches + small_launches)
    # time of the K/V plan (once per generation)
    context.profile(True)
    context.kernel_times()
    unet.prepare_conditioning(staged["context"])
    kv_times = context.kernel_times()
    context.profile(False)
    kv_gemm_ms = kv_times["gemm"][0]
    kv_launches = sum(v[1] for v in kv_times.values())
    context.check()

    # What an event pair reports around the cheapest launch of the library (a one-row LayerNorm) queued behind a
    # longer kernel on the same stream: the part of every per-launch interval above that is not the kernel's run.
    tiny = torch.zeros((1, 64), dtype=torch.float16, device=device)
    tiny_gamma, tiny_beta = torch.ones(64, dtype=torch.float16, device=device), torch.zeros(64, dtype=torch.float16, device=device)
    filler = torch.zeros(32 << 20, dtype=torch.float16, device=device)
    ops.layer_norm(tiny, tiny_gamma, tiny_beta, 1e-5)
    torch.cuda.synchronize()
    context.profile(True)
    context.kernel_times()
    floor_launches = 64
    for _ in range(floor_launches):
        filler.add_(1.0)
        ops.layer_norm(tiny, tiny_gamma, tiny_beta, 1e-5)
    floor_times = context.kernel_times()
    context.profile(False)
    event_floor_ms = floor_times["layer_norm"][0] / max(floor_times["layer_norm"][1], 1)
    del filler

    eight_bit = kind != "f16"
    tensor_peak = peaks["bf16_tflops"] * (2.0 if eight_bit else 1.0)
    sustained_peak = peaks["bf16_tflops_sustained"] * (2.0 if eight_bit else 1.0)
    achieved = step_ops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
    # quantised inputs of one step: every projection input that is not the text context, once per key
    quant_inputs = {}
    handed_over = {}               # FP8: inputs whose maximum arrives from the producing projection's epilogue
    for p in projections:
        if ".attn2.to_k" in p.name or ".attn2.to_v" in p.name:
            continue
        if kind in ("e4m3", "e5m2") and p.name.endswith(".ff.net.2"):
            handed_over.setdefault(p.input_key, (p.m, p.k))
        else:
            quant_inputs.setdefault(p.input_key, (p.m, p.k))
    # 2 + 1 bytes per element where the maximum pass is skipped, 2 + 2 + 1 otherwise
    quant_bytes = quantiser_bytes(quant_inputs.values(), kind) + float(sum(m * k * 3 for (m, k) in handed_over.values()))
    # the same bytes by kernel family: inputs that come out of a LayerNorm (to_q / to_k / to_v of attn1, attn2.to_q,
    # ff.net.0.proj) are quantised by the fused LayerNorm kernels, the rest by the stand-alone quantisers
    norm_fed = {p.input_key for p in projections
                if p.name.endswith((".attn1.to_q", ".attn1.to_k", ".attn1.to_v", ".attn2.to_q", ".ff.net.0.proj"))}
    norm_bytes = quantiser_bytes([shape for key, shape in quant_inputs.items() if key in norm_fed], kind)
    alone_bytes = quant_bytes - norm_bytes
    alone_ms = quant_ms - (norm_ms if kind != "f16" else 0.0)

    def family(bytes_moved, ms):
        if ms <= 0 or bytes_moved <= 0:
            return None
        return {"bytes_per_step": bytes_moved, "ms_per_step": ms, "achieved": bytes_moved / (ms * 1e-3) / 1e9,
                "frac": bytes_moved / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}
    rows_table = [(p.name, p.m, p.n, p.k, p.bias, p.activation, p.input_key) for p in projections
                  if not (".attn2.to_k" in p.name or ".attn2.to_v" in p.name)]
    roofline = {
        "bound": "tensor", "kernel": "sdxlq_umma_gemm_kernel", "achieved": achieved, "peak": tensor_peak, "unit": "TFLOP/s",
        "frac": achieved / tensor_peak, "frac_of_sustained": achieved / sustained_peak,
        "traffic": None,
        "traffic_note": "not captured on this workload (a step holds several GB); see profiles/ for the ncu captures of the "
                        "640- and 1280-dim sets. Algorithmic minimum per step below.",
        "min_bytes_per_step": minimum_bytes(rows_table, kind),
        "peak_source": (f"{peaks['source']} bf16 burst {peaks['bf16_tflops']} TFLOP/s x2 for 8-bit operands; sustained "
                        f"{peaks['bf16_tflops_sustained']} x2" if eight_bit else f"{peaks['source']} bf16"),
        "launch_ms": gemm_ms / max(gemm_launches, 1), "gemm_ms_per_step": gemm_ms, "gemm_launches_per_step": int(gemm_launches),
        "ops_per_step": step_ops, "ops_per_launch": step_ops / max(gemm_launches, 1),
        "how": "CUDA event pairs around every launch of the operator, eager pass over 2 steps of the same loop on the "
               "launching stream (the timed region replays a captured graph, where single launches cannot be bracketed)",
        "event_pair_floor": {
            "us_per_launch": event_floor_ms * 1e3,
            "what": "interval an event pair reports around a one-row LayerNorm launch queued behind a longer kernel: launch "
                    "gap and event cost that every per-launch interval above contains; gemm_frac_net takes it off the "
                    "GEMM intervals, one launch each (supplementary: `frac` is the plain figure; the ncu launch list "
                    "under profiles/ gives the kernels' own durations)",
            "gemm_frac_net": (step_ops / (max(gemm_ms - gemm_launches * event_floor_ms, 1e-6) * 1e-3) / 1e12 / tensor_peak),
        },
        "quantize_kernel": {"bound": "hbm", "bytes_per_step": quant_bytes, "ms_per_step": quant_ms,
                            "achieved": quant_bytes / (quant_ms * 1e-3) / 1e9 if quant_ms > 0 else None,
                            "peak": peaks["hbm_gbs"], "unit": "GB/s",
                            "frac": (quant_bytes / (quant_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]) if quant_ms > 0 else None,
                            "by_kernel_family": {"layer_norm_fused": family(norm_bytes, norm_ms if kind != "f16" else 0.0),
                                                 "stand_alone": family(alone_bytes, alone_ms)},
                            "per_kernel": "other_workloads.norm_quantize times every LayerNorm / quantiser kernel alone at "
                                          "this job's sizes (replayed graphs: device time)"},
    }
    projection_ms = gemm_ms + quant_ms
    line = {
        "metric": "sdxl_unet_steps_per_s", "value": value, "unit": "steps/s", "n_gpus": world, "steps": args.steps,
        "repeats": repeats, "timed_region_ms": elapsed_ms * repeats,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": {"int8": "int8", "e4m3": "fp8_e4m3", "e5m2": "fp8_e5m2"}.get(kind, "f16"),
        "data": "synthetic",
        "config": {"workload": unetloop_description(kind), "name": args.workload, "projections_per_forward": len(projections),
                   "images_per_rank": images, "unet_batch_per_rank": local_batch,
                   "parallelism": f"dp{world} by image / CFG pair (replicated weights, no collective in the step)",
                   "cuda_graph": not args.no_graph,
                   "l2": "inputs larger than L2: one step streams the 2.2 GB of 8-bit projection weights plus its activations "
                         f"(> {L2_BYTES / 1e6:.0f} MB L2) between repeats of any kernel",
                   "timing": "CUDA events on the launching stream around `repeats` x K steps (region of about a second), "
                             "divided by `repeats`, max over ranks"},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "steps/s", "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes,
                "steps": e2e_steps, "ms_per_step": e2e_seconds / e2e_steps * 1e3},
        "gpu_launches": repeats * (launches_per_step * args.steps + kv_launches * ((args.steps + GENERATION_STEPS - 1) // GENERATION_STEPS)),
        "launches_per_step": launches_per_step,
        "projection_tops_per_gpu": step_ops / (projection_ms * 1e-3) / 1e12 if projection_ms > 0 else None,
        "projection_gemm_tops_per_gpu": achieved,
        "projection_share_of_step": projection_ms / ms_per_step if ms_per_step > 0 else None,
        "projection_ms_per_step": {"gemm": gemm_ms, "quantize": quant_ms, "of_which_layer_norm_fused": norm_ms},
        "eager_ms_per_step": eager_ms,
        "kv_cache": {"gemm_ms_per_generation": kv_gemm_ms, "ops": kv_ops, "launches": int(kv_launches)},
        "roofline": roofline,
        "library": pkg.load_library().sdxlq_build_info().decode(),
    }
    if args.profile_images:
        line["profiling_case"] = f"reduced job of {JOB_IMAGES} images for a profiler capture: not a benchmark value"

    # ---- the final latents of every rank gathered on rank 0 (the only collective; outside the step) ----
    if distributed:
        gathered = [torch.empty_like(final_latents) for _ in range(world)] if rank == 0 else None
        dist.gather(final_latents, gathered, dst=0)
        if rank == 0:
            line["final_latents"] = {"shape": [JOB_IMAGES, 4, 128, 128], "finite": bool(torch.isfinite(torch.cat(gathered)).all()),
                                     "abs_mean": float(torch.cat(gathered).abs().mean())}
    else:
        line["final_latents"] = {"shape": [JOB_IMAGES, 4, 128, 128], "finite": bool(torch.isfinite(final_latents).all()),
                                 "abs_mean": float(final_latents.abs().mean())}
    unet.close()
    return line, context, ops


# ------------------------------------------------------------------------------------------------
# main
# ------------------------------------------------------------------------------------------------
def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=None)
    parser.add_argument("--warmup", type=int, default=None)
    parser.add_argument("--workload", default="unetloop_e4m3")
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--reference-rows", type=int, default=None)
    parser.add_argument("--e2e-steps", type=int, default=None)
    parser.add_argument("--min-seconds", type=float, default=1.0, help="the K steps are repeated until the timed region lasts this long")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-cudnn-autotune", action="store_true", help="UNet loop: leave torch.backends.cudnn.benchmark off")
    parser.add_argument("--no-other-workloads", action="store_true")
    parser.add_argument("--no-graph", action="store_true", help="run the UNet loop eagerly instead of replaying a captured step")
    parser.add_argument("--no-library", action="store_true", help="skip the vendor-library comparison on the same shapes")
    parser.add_argument("--profiler-range", action="store_true",
                        help="bracket the timed region of the UNet loop with cudaProfilerStart/Stop (for profiler captures)")
    parser.add_argument("--profile-images", type=int, default=None,
                        help="profiler captures only: a reduced job of this many images (1, 2 or 4) so that the process holds a "
                             "few GB; the line it prints is marked and is not a benchmark value")
    args = parser.parse_args()
    if args.profile_images:
        global JOB_IMAGES
        JOB_IMAGES = int(args.profile_images)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    loop = args.workload.startswith("unetloop_")

    if args.impl == "reference":
        if args.steps is None:
            args.steps = 5
        if args.warmup is None:
            args.warmup = 1
        args.steps = min(args.steps, 20)
        if rank == 0:
            print(json.dumps(reference_arm(args)), flush=True)
        return 0

    import torch
    import torch.distributed as dist

    if args.steps is None:
        args.steps = GENERATION_STEPS if loop else 0
    if args.warmup is None:
        args.warmup = 3
    args.warmup = max(args.warmup, 3)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    torch.cuda.set_device(local_rank)
    distributed = world > 1
    if distributed:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    pkg = package()
    peaks = load_peaks()

    if loop:
        line, context, ops = run_unet_loop(args, torch, dist, pkg, rank, local_rank, world, peaks)
        if rank == 0 and world == 1 and not args.no_other_workloads:
            others = {}
            # the loop is done with its buffers: give the memory back, and use a context whose scratch holds the
            # quantised copy of every input of a whole-UNet plan
            torch.cuda.empty_cache()
            side_context = pkg.Context(local_rank, workspace_bytes=3 << 30)
            side_ops = pkg.Ops(side_context)
            for name in ("layerset640_int8", "layerset640_int8_g64", "layerset1280_fp8", "geglu640_f16", "unet743_int8", "unet743_e5m2"):
                try:
                    others[name] = time_projection_workload(torch, pkg, side_context, side_ops, name, peaks,
                                                            library=(not args.no_library) and name.startswith(("layerset", "geglu")))
                except Exception as error:       # a side measurement must not lose the headline line
                    others[name] = {"error": f"{type(error).__name__}: {error}"}
            try:
                others["norm_quantize"] = time_norm_quantize(torch, pkg, side_ops, peaks)
            except Exception as error:
                others["norm_quantize"] = {"error": f"{type(error).__name__}: {error}"}
            side_context.check()
            side_context.close()
            line["other_workloads"] = others
        if rank == 0 and world == 1 and not args.no_cpu_baseline:
            tops, kind, sample = cpu_single_core_rate()
            full_ops = float(unet_shapes().total_ops(unet_shapes().unet_projections(2 * JOB_IMAGES)))
            line["cpu_baseline"] = {"value": tops * 1e12 / full_ops, "unit": "steps/s", "cores": 1, "kind": kind,
                                    "cpu_tops": tops,
                                    "sample": sample + f"; converted to steps/s of the job by its {full_ops / 1e12:.2f} TOP of projections "
                                                       "per step (projections only: an upper bound for the CPU reference's step)"}
        else:
            line["cpu_baseline"] = None
        context.check()
        if rank == 0:
            print(json.dumps(line), flush=True)
        if distributed:
            dist.destroy_process_group()
        return 0

    # ---- a projection-only workload as the main line ---------------------------------------------------
    rows, kind, group, description = workload_rows(args.workload, world)
    unique_inputs = {key: (m, k) for (_, m, _, k, _, _, key) in rows}
    scratch = sum(m * k + 4 * m + 1024 for (m, k) in unique_inputs.values())
    context = pkg.Context(local_rank, workspace_bytes=max(1 << 30, int(scratch * 1.1)))
    ops = pkg.Ops(context)

    def barrier():
        torch.cuda.synchronize()
        if distributed:
            dist.barrier()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    barrier()
    if sampler:
        sampler.mark_start()
    result = time_projection_workload(torch, pkg, context, ops, args.workload, peaks, min_seconds=1.0, world=world,
                                      library=(rank == 0 and not args.no_library))
    if sampler:
        sampler.mark_stop()
    barrier()
    ms_per_step = result["ms_per_step"]
    if distributed:
        tensor = torch.tensor([ms_per_step], device="cuda")
        dist.all_reduce(tensor, op=dist.ReduceOp.MAX)
        ms_per_step = float(tensor.item())
    ops_per_step = result["ops_per_step"]
    value = world * ops_per_step / (ms_per_step * 1e-3) / 1e12

    # end to end: pinned host inputs -> device, plan, results -> pinned host
    work = DeviceWorkload(pkg, ops, rows, kind, group, 1)
    e2e_value, e2e_ms, e2e_steps = None, None, 0
    if work.h2d_bytes + work.d2h_bytes <= (8 << 30):
        e2e_steps = args.e2e_steps or 10
        host_inputs = {key: torch.empty(x.shape, dtype=x.dtype).pin_memory().copy_(x) for key, x in work.inputs[0].items()}
        host_outputs = [torch.empty(y.shape, dtype=y.dtype).pin_memory() for y in work.outputs[0]]

        def e2e_step():
            for key, hostbuf in host_inputs.items():
                work.inputs[0][key].copy_(hostbuf, non_blocking=True)
            work.plans[0].run()
            for hostbuf, y in zip(host_outputs, work.outputs[0]):
                hostbuf.copy_(y, non_blocking=True)
            torch.cuda.current_stream().synchronize()
        e2e_step()
        barrier()
        wall = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        e2e_seconds = time.perf_counter() - wall
        barrier()
        if distributed:
            tensor = torch.tensor([e2e_seconds], device="cuda")
            dist.all_reduce(tensor, op=dist.ReduceOp.MAX)
            e2e_seconds = float(tensor.item())
        e2e_value = world * ops_per_step * e2e_steps / e2e_seconds / 1e12
        e2e_ms = e2e_seconds / e2e_steps * 1e3
    context.check()
    clocks = sampler.stop() if sampler else None
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        tops, cpu_kind, sample = cpu_single_core_rate()
        cpu_baseline = {"value": tops, "unit": "TOPS", "cores": 1, "kind": cpu_kind, "sample": sample}
    if rank == 0:
        gemm = result["gemm"]
        line = {
            "metric": "quantized_linear_tops", "value": value, "unit": "TOPS", "n_gpus": world, "steps": result["steps_timed"],
            "warmup": 6, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if args.workload.startswith("unetstep_") else "weak", "vs_baseline": None,
            "dtype": {"int8": "int8", "e4m3": "fp8_e4m3", "e5m2": "fp8_e5m2"}.get(kind, "f16"), "data": "synthetic",
            "config": {"workload": description, "name": args.workload, "projections": len(rows), "ops_per_step": ops_per_step,
                       "parallelism": f"dp{world} (replicated weights, no collective)", "l2": result["l2"],
                       "timing": "CUDA events on the launching stream, max over ranks; steps sized for a timed region of >= 1 s"},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "TOPS", "h2d_bytes_per_step": work.h2d_bytes, "d2h_bytes_per_step": work.d2h_bytes,
                    "steps": e2e_steps, "ms_per_step": e2e_ms},
            "gpu_launches": result["launches_per_step"] * result["steps_timed"], "launches_per_step": result["launches_per_step"],
            "roofline": {"bound": "tensor", "kernel": "sdxlq_umma_gemm_kernel", "achieved": gemm["tops"], "peak": gemm["peak_tflops"],
                         "unit": "TFLOP/s", "frac": gemm["frac_of_peak"], "traffic": None, "min_bytes": gemm["min_bytes"],
                         "launch_ms": gemm["ms"], "ops_per_launch": ops_per_step,
                         "peak_source": f"{peaks['source']} bf16 {peaks['bf16_tflops']} TFLOP/s" + (" x2 for 8-bit operands" if kind != "f16" else ""),
                         "quantize_kernel": result["quantize"]},
            "library_same_shapes": result.get("library_same_shapes"),
            "cpu_baseline": cpu_baseline,
            "library": pkg.load_library().sdxlq_build_info().decode(),
        }
        print(json.dumps(line), flush=True)
    work.close()
    if distributed:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
