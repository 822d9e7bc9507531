"""GPU tests of the synthetic UNet loop: the executor with the real operator behind every
projection against the reference's own CPU UNet (SDXLUNet::forward compiled from the reference
sources into oracle/_ref), graph replay against eager execution, and sharding by image."""
import importlib

import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu

harness = importlib.import_module("sdxl-end2end_b200.unet_harness")

MINIATURE = harness.UNetConfig(channels=(64, 128, 256), heads=(1, 2, 4), transformer_depth=(1, 1, 2),
                               cross_attention_dim=96, time_embed_dim=128, addition_time_embed_dim=8,
                               addition_input_dim=80, layers_per_block=2, norm_groups=32)


def config_tuple(c):
    return (c.channels, c.heads, c.transformer_depth, c.cross_attention_dim, c.time_embed_dim,
            c.addition_time_embed_dim, c.addition_input_dim, c.layers_per_block, c.norm_groups)


def inputs(batch, size=16, seed=5):
    rng = np.random.default_rng(seed)
    h = lambda a: a.astype(np.float16).astype(np.float32)
    latents = h(rng.standard_normal((batch, 4, size, size), dtype=np.float32))
    context = h(rng.standard_normal((batch, 77, MINIATURE.cross_attention_dim), dtype=np.float32))
    pooled = h(rng.standard_normal((batch, MINIATURE.pooled_dim), dtype=np.float32))
    time_ids = np.tile(np.array([[128, 128, 0, 0, 128, 128]], np.float32), (batch, 1))
    return latents, context, pooled, time_ids


def parameters(seed=3):
    values = harness.synthetic_parameters(MINIATURE, torch.device("cuda"), seed=seed)
    return {name: value.to(torch.float16).to(torch.float32) for name, value in values.items()}


def run_forward(ops, precision, params, data, **options):
    latents, context, pooled, time_ids = data
    unet = harness.UNetHarness(ops, MINIATURE, precision=precision, parameters=params, **options)
    unet.prepare_conditioning(torch.from_numpy(context).cuda().half())
    out = unet.forward(torch.from_numpy(latents).cuda().half(), 801.0, torch.from_numpy(pooled).cuda().half(),
                       torch.from_numpy(time_ids).cuda().half())
    ops.ctx.check()
    calls = unet.projection_calls
    unet.close()
    return out.float().cpu().numpy(), calls


@pytest.mark.skipif(not O.ref_available(), reason="oracle/_ref was not built")
@pytest.mark.parametrize("precision,tolerance", [("f16", 2e-2), ("e4m3", 1.5e-1), ("int8", 8e-2)])
def test_forward_matches_the_reference_cpu_unet(gpu, precision, tolerance):
    """All projections on the tensor-core path, everything else PyTorch FP16, against the
    reference's FP32 CPU executor on the same FP16-representable parameters. The FP16 profile differs
    only by FP16 rounding of the activations; the quantised profiles add their quantisation error
    (random weights, so it does not average out over channels the way a trained model's does)."""
    pkg, ctx, ops = gpu
    params = parameters()
    data = inputs(2)
    got, calls = run_forward(ops, precision, params, data)
    reference = O.RefUNet(config_tuple(MINIATURE))
    reference.bind({name: value.cpu().numpy() for name, value in params.items()})
    want = reference.forward(data[0], 801.0, data[1], data[2], data[3])
    reference.close()
    count = sum(1 for name, shape in harness.unet_parameter_shapes(MINIATURE).items() if harness.is_projection_weight(name, shape))
    assert calls == count
    scale = float(np.max(np.abs(want)))
    error = float(np.max(np.abs(got - want))) / scale
    rms = float(np.sqrt(np.mean((got - want) ** 2)) / np.sqrt(np.mean(want ** 2)))
    print(f"{precision}: max|a-b|/max|b| = {error:.3e}, rms rel = {rms:.3e}")
    assert np.isfinite(got).all() and error <= tolerance


@pytest.mark.parametrize("precision", ["int8", "e4m3"])
def test_fused_residual_and_grouping_do_not_change_results(gpu, precision):
    """Residual add in the epilogue and grouped q/k/v against the call-by-call form of the reference
    (separate Linear, then add_in_place): bit-identical."""
    pkg, ctx, ops = gpu
    params = parameters(7)
    data = inputs(2, seed=8)
    fused, _ = run_forward(ops, precision, params, data)
    plain, _ = run_forward(ops, precision, params, data, fuse_residual=False, group_attention_inputs=False)
    assert np.array_equal(fused, plain)


@pytest.mark.parametrize("precision,bound", [("f16", 5e-3), ("e4m3", 3e-2), ("int8", 3e-2)])
def test_fused_layer_norm_stays_within_rounding(gpu, precision, bound):
    """The library's LayerNorm (fused with the quantisers for the quantised profiles) against
    PyTorch's layer_norm in front of self-quantising projections. The two LayerNorms differ in the
    last FP16 bit of a small share of their outputs; behind a quantiser such a flip moves a byte by
    one step, so the UNet outputs agree to the quantisation noise, not bit for bit."""
    pkg, ctx, ops = gpu
    params = parameters(13)
    data = inputs(2, seed=14)
    fused, _ = run_forward(ops, precision, params, data)
    plain, _ = run_forward(ops, precision, params, data, fuse_layer_norm=False)
    rms = float(np.sqrt(np.mean((fused - plain) ** 2)) / np.sqrt(np.mean(plain ** 2)))
    print(f"{precision}: fused vs separate LayerNorm rms rel = {rms:.3e}")
    assert rms <= bound


def test_graph_replay_equals_eager_loop(gpu):
    pkg, ctx, ops = gpu
    params = parameters(9)
    latents, context, pooled, time_ids = inputs(2 * 2, seed=10)
    results = []
    for use_graph in (False, True):
        unet = harness.UNetHarness(ops, MINIATURE, precision="e4m3", parameters=params)
        loop = harness.EulerDenoiser(unet, 2, height=128, width=128, steps=4, use_graph=use_graph)
        loop.set_conditioning(torch.from_numpy(context).cuda().half(), torch.from_numpy(pooled).cuda().half(),
                              torch.from_numpy(time_ids).cuda().half())
        loop.set_latents(torch.from_numpy(latents[:2]).cuda())
        results.append(loop.run().clone())
        # a second generation through the same (captured) step
        loop.set_latents(torch.from_numpy(latents[2:]).cuda())
        results.append(loop.run().clone())
        torch.cuda.synchronize()
        ctx.check()
        unet.close()
    assert torch.isfinite(results[0]).all()
    assert torch.equal(results[0], results[2]) and torch.equal(results[1], results[3])


def test_sharding_by_image_keeps_each_image(gpu):
    """Two images denoised together ([uncond x 2 | cond x 2]) against each image on its own
    ([uncond | cond]), as ranks of a 2-GPU run would hold them. INT8 activations are scaled per token,
    so the projections are bit-identical per image; the PyTorch scaffolding (cuDNN, attention) may
    pick different kernels for different batch sizes, hence a tolerance instead of equality."""
    pkg, ctx, ops = gpu
    params = parameters(11)
    latents, context, pooled, time_ids = inputs(4, seed=12)       # rows 0-1 uncond, 2-3 cond of images 0, 1

    def denoise(image_rows, cond_rows):
        images = len(image_rows)
        unet = harness.UNetHarness(ops, MINIATURE, precision="int8", parameters=params)
        loop = harness.EulerDenoiser(unet, images, height=128, width=128, steps=3, use_graph=False)
        rows = image_rows + cond_rows
        loop.set_conditioning(torch.from_numpy(context[rows]).cuda().half(), torch.from_numpy(pooled[rows]).cuda().half(),
                              torch.from_numpy(time_ids[rows]).cuda().half())
        loop.set_latents(torch.from_numpy(latents[image_rows]).cuda())
        out = loop.run().clone()
        ctx.check()
        unet.close()
        return out

    together = denoise([0, 1], [2, 3])
    alone = torch.cat([denoise([0], [2]), denoise([1], [3])])
    scale = float(together.abs().max())
    assert float((together - alone).abs().max()) <= 2e-2 * scale


@pytest.mark.parametrize("batch,channels,size", [(2, 320, 32), (2, 640, 16), (1, 1280, 8), (2, 960, 16), (2, 1920, 8), (1, 2560, 8), (3, 64, 5)])
@pytest.mark.parametrize("silu,with_bias", [(False, False), (True, False), (True, True)])
def test_group_norm_nhwc_matches_the_fp32_formula(gpu, batch, channels, size, silu, with_bias):
    """The harness's channels-last GroupNorm (+ SiLU, + time-embedding bias) against the FP32 formula of the
    reference's group_norm_kernel (src/cuda/ops_kernels.cu:258-308) evaluated with PyTorch on the NCHW view:
    every output within 2 FP16 steps of the larger of |y| and |beta| (the statistics are FP32 sums in
    another order, the variance one-pass), and two runs bit-identical (no atomics)."""
    pkg, ctx, ops = gpu
    generator = torch.Generator(device="cuda").manual_seed(17 + channels + size)
    x = (torch.randn((batch, channels, size, size), generator=generator, device="cuda") * 1.5 + 0.3).half()
    x = x.contiguous(memory_format=torch.channels_last)
    gamma = (1.0 + 0.2 * torch.randn(channels, generator=generator, device="cuda")).half()
    beta = (0.1 * torch.randn(channels, generator=generator, device="cuda")).half()
    bias = (0.5 * torch.randn((batch, channels), generator=generator, device="cuda")).half() if with_bias else None
    got = ops.group_norm_nhwc(x, gamma, beta, 32, 1e-5, silu, bias)
    again = ops.group_norm_nhwc(x, gamma, beta, 32, 1e-5, silu, bias)
    ctx.check()
    assert got.is_contiguous(memory_format=torch.channels_last) and torch.equal(got, again)
    source = x.float()
    if with_bias:
        source = (source + bias.float()[:, :, None, None]).half().float()
    want = torch.nn.functional.group_norm(source.double(), 32, gamma.double(), beta.double(), 1e-5)
    if silu:
        want = want * torch.sigmoid(want)
    bound = 2.0 ** -9 * torch.maximum(want.abs(), beta.double().abs()[None, :, None, None]) + 1e-6
    assert bool(((got.double() - want).abs() <= bound).all()), float(((got.double() - want).abs() / bound).max())


@pytest.mark.parametrize("precision", ["f16", "e4m3"])
def test_group_norm_kernel_in_the_harness_stays_within_rounding(gpu, precision):
    """The whole forward with the scaffolding GroupNorm kernel against PyTorch's group_norm. FP16: rounding
    level. FP8 E4M3 with random weights: a last-bit difference of a norm output can move a tensor-wide
    maximum, hence the scale and every byte of that tensor by one step; through 70 transformer blocks the
    two runs then differ by the profile's own quantisation noise (the same size as its distance from the
    reference's FP32 UNet, see test_forward_matches_the_reference_cpu_unet)."""
    pkg, ctx, ops = gpu
    params = parameters(15)
    data = inputs(2, seed=16)
    ours, _ = run_forward(ops, precision, params, data)
    torch_norm, _ = run_forward(ops, precision, params, data, fuse_group_norm=False)
    rms = float(np.sqrt(np.mean((ours - torch_norm) ** 2)) / np.sqrt(np.mean(torch_norm ** 2)))
    print(f"{precision}: library GroupNorm vs torch group_norm rms rel = {rms:.3e}")
    assert rms <= (5e-3 if precision == "f16" else 1.5e-1)


def test_bias_residual_add_equals_two_pytorch_adds(gpu):
    pkg, ctx, ops = gpu
    generator = torch.Generator(device="cuda").manual_seed(31)
    x = torch.randn((2, 320, 16, 16), generator=generator, device="cuda").half().contiguous(memory_format=torch.channels_last)
    residual = torch.randn((2, 320, 16, 16), generator=generator, device="cuda").half().contiguous(memory_format=torch.channels_last)
    bias = torch.randn(320, generator=generator, device="cuda").half()
    got = ops.bias_residual_add_nhwc(x, bias, residual)
    ctx.check()
    want = (x + bias[None, :, None, None]) + residual          # two FP16 roundings, like the two kernels it replaces
    assert got.is_contiguous(memory_format=torch.channels_last) and torch.equal(got, want)
