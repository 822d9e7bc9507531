"""GPU parity at the full sizes of the benchmark configurations, and of the 743-projection plans.

The oracle is evaluated on a row sample of each projection (rows from every 128-row tile, the
first and last rows included): with per-row activation scales an INT8 row does not depend on the
other rows, and for FP8 the tensor-wide scale comes from the whole input. Every output element is
checked to be written (the fixture poisons outputs with NaN)."""
import importlib

import numpy as np
import pytest
import torch

import helpers as H
from oracle import oracle as O

pytestmark = pytest.mark.gpu

shapes = importlib.import_module("sdxl-end2end_b200.unet_shapes")


def dev(array):
    return torch.from_numpy(np.ascontiguousarray(array)).cuda()


def sample_rows(m, per_tile=3, seed=0):
    rng = np.random.default_rng(seed)
    rows = {0, m - 1}
    for tile in range((m + 127) // 128):
        lo, hi = tile * 128, min(m, tile * 128 + 128)
        rows.update(int(r) for r in rng.integers(lo, hi, size=per_tile))
    return np.array(sorted(rows))


def int8_weight(pkg, n, k, g, seed):
    wq, ws = O.int8_quantize_rows(H.make_weight(seed, n, k).astype(np.float32), g)
    return pkg.Weight(dev(wq), pkg.ScalarType.Int8, n, k, dev(ws), pkg.FP8ScaleMode.PerOutputChannel,
                      pkg.FP8StorageLayout.RowMajorNK, g), wq, ws


@pytest.mark.parametrize("m,n,k,g,activation", [
    (8192, 5120, 640, 0, 4),        # ff.net.0.proj + GEGLU, group-256 rule: K = 640 is not rotated
    (8192, 5120, 640, 64, 4),       # the same with groups of 64 so that it rotates
    (8192, 640, 2560, 256, 0),      # ff.net.2
    (8192, 640, 640, 64, 0),        # attention projections, rotated
    (2048, 10240, 1280, 256, 4),    # 1280-dim ff.net.0.proj + GEGLU
])
def test_int8_full_size_projection(gpu, m, n, k, g, activation):
    pkg, ctx, ops = gpu
    x = H.make_activations(70, m, k)
    weight, wq, ws = int8_weight(pkg, n, k, g, 70)
    bias = H.make_bias(70, n)
    acc = torch.empty((m, n), dtype=torch.int32, device="cuda")
    if activation:
        y = ops.linear_activation(dev(x), weight, dev(bias), activation, acc_out=acc)
    else:
        y = ops.linear(dev(x), weight, dev(bias), acc_out=acc)
    ctx.check()
    assert torch.isfinite(y).all()
    rows = sample_rows(m)
    want = O.int8_convrot_linear(x[rows], wq, ws, g, bias.view(np.uint16), activation)
    assert np.array_equal(acc.cpu().numpy()[rows], want["acc"])               # INT32 accumulators: bit-exact
    got = y.cpu().numpy()[rows]
    if activation == 0:
        assert np.array_equal(got.view(np.uint16), want["out"])               # dequant + bias: bit-exact
    else:
        expected = O.h2f(want["out"])
        assert H.max_rel(got.astype(np.float32), expected) <= 2e-3
        assert np.mean(got.view(np.uint16) == want["out"]) >= 0.9


@pytest.mark.parametrize("m,n,k,activation,fmt", [
    (2048, 10240, 1280, 4, 0), (2048, 1280, 5120, 0, 0), (2048, 1280, 1280, 0, 0), (8192, 5120, 640, 4, 1),
])
def test_fp8_full_size_projection(gpu, m, n, k, activation, fmt):
    pkg, ctx, ops = gpu
    x = H.make_activations(71, m, k, outliers=False)
    wq, ws = O.fp8_quantize_weight(H.make_weight(71, n, k).astype(np.float32), fmt, True)
    kind = pkg.ScalarType.Float8E4M3 if fmt == 0 else pkg.ScalarType.Float8E5M2
    weight = pkg.Weight(dev(wq), kind, n, k, dev(ws), pkg.FP8ScaleMode.PerOutputChannel)
    bias = H.make_bias(71, n)
    y = ops.linear_activation(dev(x), weight, dev(bias), activation) if activation else ops.linear(dev(x), weight, dev(bias))
    ctx.check()
    assert torch.isfinite(y).all()
    rows = sample_rows(m)
    xq, x_scale = O.fp8_quantize_activation(x.view(np.uint16), fmt)             # tensor-wide scale from the whole input
    want = O.fp8_linear(xq[rows], fmt, float(x_scale), wq, fmt, ws, bias.view(np.uint16), activation)
    got = y.cpu().numpy()[rows].astype(np.float32)
    expected = O.h2f(want["out"])
    assert H.max_rel(got, expected, 1e-2) <= 1e-2
    assert H.max_abs_over_max(got, expected) <= 1e-3


def test_fp16_config_one_against_reference_golden_rows(gpu):
    """BASELINE's first configuration at full size, X [8192,640] x W [5120,640] + bias + GEGLU with FP16
    weights, against rows computed by the reference's own linear_2d + geglu (committed fixture made by
    tests/golden/make_golden.py from the reference build)."""
    import os
    pkg, ctx, ops = gpu
    golden = np.load(os.path.join(os.path.dirname(__file__), "golden", "config1_rows.npz"))
    x = H.make_activations(int(golden["seed"]), 8192, 640)
    w = H.make_weight(int(golden["seed"]), 5120, 640)
    bias = H.make_bias(int(golden["seed"]), 5120)
    y = ops.linear_activation(dev(x), ops.fp16_weight(dev(w)), dev(bias), pkg.ACT_GEGLU)
    ctx.check()
    assert torch.isfinite(y).all()
    rows = golden["rows"]
    got = y.cpu().numpy()[rows].astype(np.float32)
    want = golden["out"]
    assert H.max_rel(got, want, 1e-2) <= 2e-3
    assert H.max_abs_over_max(got, want) <= 1e-3


def test_float_paths_against_an_exact_sum(gpu):
    """Separates the kernel's error from the FP32-sequential CPU reference's own: both are compared
    with the FP64 sum of the same FP16 products, with the 1e-3 * max floor. The tensor-core result
    must be no further from the exact value than 4x the reference's CPU arithmetic (both are a few
    1e-6 of the largest output; FP16 output rounding, 4.9e-4, dominates either)."""
    pkg, ctx, ops = gpu
    m, n, k = 256, 1280, 5120
    x = H.make_activations(72, m, k)
    w = H.make_weight(72, n, k)
    y = ops.linear(dev(x), ops.fp16_weight(dev(w))).cpu().numpy().astype(np.float64)
    ctx.check()
    exact = x.astype(np.float64) @ w.astype(np.float64).T
    sequential = O.linear_f32(x.astype(np.float32), w.astype(np.float32)).astype(np.float64)
    scale = float(np.max(np.abs(exact)))
    half_rounded_exact = exact.astype(np.float16).astype(np.float64)
    kernel_error = float(np.max(np.abs(y - half_rounded_exact))) / scale
    reference_error = float(np.max(np.abs(sequential - exact))) / scale
    one_ulp_at_max = 2.0 ** -10
    print(f"kernel vs FP16(exact): {kernel_error:.3e} of max; FP32-sequential CPU vs exact: {reference_error:.3e} of max")
    assert kernel_error <= one_ulp_at_max                        # at most one FP16 step of the largest output
    floor_strict = H.max_rel(y, exact, 1e-3)
    floor_loose = H.max_rel(y, exact, 1e-2)
    print(f"max-rel vs exact: floor 1e-3 -> {floor_strict:.3e}, floor 1e-2 -> {floor_loose:.3e}")
    assert floor_loose <= 2e-3


@pytest.mark.parametrize("kind", ["int8", "e5m2"])
def test_plan_of_all_743_projections(gpu, kind):
    """Builds the plan of every projection of one UNet step (the benchmark's unet743 workloads) with
    seeded inputs, runs it once, and compares one projection of each of the 13 distinct (M, N, K,
    activation) shapes, M = 2 and K = 320 / 2816 included, with the oracle on a row sample."""
    pkg, _, _ = gpu
    # a context of its own: the quantised copy of every distinct input of the step lives in the scratch at once
    ctx = pkg.Context(0, workspace_bytes=3 << 30)
    ops = pkg.Ops(ctx, poison_outputs=True)
    projections = shapes.unet_projections(2)
    assert len(projections) == 743
    distinct = {}
    for index, p in enumerate(projections):
        distinct.setdefault((p.m, p.n, p.k, p.activation), index)
    assert len(distinct) == 13 and (2, 1280, 320, 1) in distinct and (2, 1280, 2816, 1) in distinct
    checked = set(distinct.values())
    generator = torch.Generator(device="cuda")
    generator.manual_seed(77)
    inputs, weights, biases, host = {}, [], [], {}
    for index, p in enumerate(projections):
        if p.input_key not in inputs:
            inputs[p.input_key] = torch.randn((p.m, p.k), generator=generator, device="cuda").half()
        if index in checked:
            w = H.make_weight(index, p.n, p.k)
            b = H.make_bias(index, p.n) if p.bias else None
            if kind == "int8":
                group = 256 if p.k % 256 == 0 else 0
                wq, ws = O.int8_quantize_rows(w.astype(np.float32), group)
                weight = pkg.Weight(dev(wq), pkg.ScalarType.Int8, p.n, p.k, dev(ws), pkg.FP8ScaleMode.PerOutputChannel,
                                    pkg.FP8StorageLayout.RowMajorNK, group)
            else:
                wq, ws = O.fp8_quantize_weight(w.astype(np.float32), 1, True)
                weight = pkg.Weight(dev(wq), pkg.ScalarType.Float8E5M2, p.n, p.k, dev(ws), pkg.FP8ScaleMode.PerOutputChannel)
            host[index] = (wq, ws, b)
            weights.append(weight)
            biases.append(dev(b) if b is not None else None)
        else:
            # the other projections only have to run: cheap device-side random weights
            w = (torch.randn((p.n, p.k), generator=generator, device="cuda") / p.k ** 0.5).half()
            if kind == "int8":
                weights.append(ops.upload_or_quantize_int8_weight(w, None, pkg.INT8WeightLoadOptions()))
            else:
                weights.append(ops.upload_fp8_weight(w, pkg.FP8WeightLoadOptions(format=pkg.ScalarType.Float8E5M2,
                                                                                   scale_mode=pkg.FP8ScaleMode.PerOutputChannel)))
            biases.append((torch.randn(p.n, generator=generator, device="cuda") * 0.1).half() if p.bias else None)
    calls = [pkg.LinearCall(inputs[p.input_key], weights[i], biases[i], p.activation) for i, p in enumerate(projections)]
    plan = ops.plan(calls)
    # quantiser launches (INT8: unrotated + rotated; FP8: maximum + cast) and one GEMM launch
    assert plan.launches == 3
    outputs = plan.run()
    ctx.check()
    for index in sorted(checked):
        p = projections[index]
        wq, ws, b = host[index]
        x = inputs[p.input_key].cpu().numpy()
        rows = sample_rows(p.m, per_tile=1, seed=index)[:48]
        got = outputs[index].cpu().numpy()
        assert np.isfinite(got).all(), p.name
        bias_bits = b.view(np.uint16) if b is not None else None
        if kind == "int8":
            group = 256 if p.k % 256 == 0 else 0
            want = O.int8_convrot_linear(x[rows], wq, ws, group, bias_bits, p.activation)["out"]
            if p.activation == 0:
                assert np.array_equal(got[rows].view(np.uint16), want), p.name
            else:
                assert H.max_rel(got[rows].astype(np.float32), O.h2f(want)) <= 2e-3, p.name
        else:
            xq, x_scale = O.fp8_quantize_activation(x.view(np.uint16), 1)
            want = O.fp8_linear(xq[rows], 1, float(x_scale), wq, 1, ws, bias_bits, p.activation)["out"]
            assert H.max_rel(got[rows].astype(np.float32), O.h2f(want), 1e-2) <= 1e-2, p.name
    plan.close()
    ctx.close()
