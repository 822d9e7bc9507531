"""Host-side checks of the synthetic UNet loop: parameter inventory and sigma schedule against the
reference's own code (compiled under oracle/_ref), and the executor's wiring against the reference's
CPU UNet on a miniature configuration with a CPU stand-in for the operator."""
import importlib

import numpy as np
import pytest
import torch

from oracle import oracle as O
from fake_ops import FakeOps

harness = importlib.import_module("sdxl-end2end_b200.unet_harness")
shapes = importlib.import_module("sdxl-end2end_b200.unet_shapes")

needs_reference = pytest.mark.skipif(not O.ref_available(), reason="oracle/_ref was not built (no reference tree)")

MINIATURE = harness.UNetConfig(channels=(32, 64, 64), heads=(1, 2, 2), transformer_depth=(1, 1, 2),
                               cross_attention_dim=24, time_embed_dim=64, addition_time_embed_dim=4,
                               addition_input_dim=40, layers_per_block=2, norm_groups=8)


def config_tuple(c):
    return (c.channels, c.heads, c.transformer_depth, c.cross_attention_dim, c.time_embed_dim,
            c.addition_time_embed_dim, c.addition_input_dim, c.layers_per_block, c.norm_groups)


def test_projection_inventory_matches_the_call_site_table():
    """743 rank-2 projections, same names and [N, K] as unet_shapes enumerates for the benchmark plans."""
    inventory = {name[:-len(".weight")]: shape for name, shape in harness.unet_parameter_shapes().items()
                 if harness.is_projection_weight(name, shape)}
    table = {p.name: (p.n, p.k) for p in shapes.unet_projections(2)}
    assert len(table) == 743 and inventory == table
    assert shapes.total_ops(shapes.unet_projections(2)) == 8_708_418_437_120
    assert shapes.weight_bytes_8bit(shapes.unet_projections(2)) == 2_232_647_680


@needs_reference
def test_parameter_inventory_matches_the_reference_graph():
    """Every UNet parameter name and shape of the reference's SDXL Base 1.0 parameter graph
    (add_unet, src/sdxl.cpp:84-238), and of a miniature configuration."""
    for config, ours in ((None, harness.unet_parameter_shapes()), (config_tuple(MINIATURE), harness.unet_parameter_shapes(MINIATURE))):
        reference = O.RefUNet(config)
        theirs = reference.parameters()
        reference.close()
        assert set(theirs) == set(ours)
        assert all(tuple(theirs[name]) == tuple(ours[name]) for name in ours)
    base = O.RefUNet(None)
    projections = {n: s for n, s in base.parameters().items() if harness.is_projection_weight(n, s)}
    base.close()
    assert len(projections) == 743
    assert projections["mid_block.attentions.0.transformer_blocks.9.attn2.to_k.weight"] == (1280, 2048)


@needs_reference
@pytest.mark.parametrize("steps", [1, 4, 20, 30])
def test_sigma_schedule_matches_the_reference(steps):
    timesteps, sigmas = harness.normal_sigma_schedule(steps)
    want_t, want_s = O.ref_normal_sigma_schedule(steps)
    assert np.array_equal(np.asarray(timesteps, np.float32), want_t)
    assert np.allclose(np.asarray(sigmas, np.float32), want_s, rtol=2e-7, atol=0)


def miniature_inputs(batch, seed=5):
    rng = np.random.default_rng(seed)
    latents = rng.standard_normal((batch, 4, 16, 16), dtype=np.float32)
    context = rng.standard_normal((batch, 7, MINIATURE.cross_attention_dim), dtype=np.float32)
    pooled = rng.standard_normal((batch, MINIATURE.pooled_dim), dtype=np.float32)
    time_ids = np.tile(np.array([[128, 128, 0, 0, 128, 128]], np.float32), (batch, 1))
    return latents, context, pooled, time_ids


@needs_reference
def test_forward_wiring_matches_the_reference_cpu_unet():
    """The executor, with a CPU stand-in for the operator, against SDXLUNet::forward
    (src/unet.cpp:699-807) on the same random parameters: same call sites in the same order with the
    same tensors, up to FP16 rounding of the activations (the reference's CPU path is FP32)."""
    cpu = torch.device("cpu")
    parameters = harness.synthetic_parameters(MINIATURE, cpu, seed=3)
    # FP16-representable parameters, so that both sides multiply the same numbers
    parameters = {name: value.to(torch.float16).to(torch.float32) for name, value in parameters.items()}
    ops = FakeOps()
    unet = harness.UNetHarness(ops, MINIATURE, precision="f16", parameters=parameters, device=cpu)
    latents, context, pooled, time_ids = miniature_inputs(2)
    unet.prepare_conditioning(torch.from_numpy(context).to(torch.float16))
    got = unet.forward(torch.from_numpy(latents).to(torch.float16), 801.0, torch.from_numpy(pooled).to(torch.float16),
                       torch.from_numpy(time_ids).to(torch.float16)).float().numpy()
    reference = O.RefUNet(config_tuple(MINIATURE))
    reference.bind({name: value.numpy() for name, value in parameters.items()})
    want = reference.forward(latents.astype(np.float16).astype(np.float32), 801.0, context.astype(np.float16).astype(np.float32),
                             pooled.astype(np.float16).astype(np.float32), time_ids)
    reference.close()
    scale = float(np.max(np.abs(want)))
    assert scale > 0.05
    assert float(np.max(np.abs(got - want))) <= 2e-2 * scale
    # the call inventory: every projection of the configuration exactly once per forward
    count = sum(1 for name, shape in harness.unet_parameter_shapes(MINIATURE).items() if harness.is_projection_weight(name, shape))
    assert unet.projection_calls == count == len([entry for entry in ops.log if entry[0] not in ("layer_norm", "group_norm")])
    fused = [entry for entry in ops.log if entry[6] and entry[0] != "group_norm"]
    blocks = sum(1 for name in unet.projections if name.endswith(".attn1.to_out.0"))
    attention_blocks = sum(1 for name in unet.projections if name.endswith(".proj_out"))
    assert len(fused) == 3 * blocks + attention_blocks          # to_out x2, ff.net.2, proj_out


@needs_reference
def test_euler_loop_matches_a_loop_around_the_reference_unet():
    """Two Euler steps with CFG around the executor against the same arithmetic around the
    reference's CPU UNet (Denoiser::run_loop's Euler branch, src/cuda/denoiser.cpp:297-312)."""
    cpu = torch.device("cpu")
    parameters = {n: v.to(torch.float16).to(torch.float32) for n, v in harness.synthetic_parameters(MINIATURE, cpu, seed=4).items()}
    unet = harness.UNetHarness(FakeOps(), MINIATURE, precision="f16", parameters=parameters, device=cpu)
    images, steps, scale = 1, 2, 5.0
    loop = harness.EulerDenoiser(unet, images, height=128, width=128, steps=steps, guidance_scale=scale, use_graph=False)
    latents, context, pooled, time_ids = miniature_inputs(2 * images, seed=9)
    noise = latents[:images]
    loop.set_conditioning(torch.from_numpy(context).to(torch.float16), torch.from_numpy(pooled).to(torch.float16),
                          torch.from_numpy(time_ids).to(torch.float16))
    loop.set_latents(torch.from_numpy(noise))
    got = loop.run().numpy()

    reference = O.RefUNet(config_tuple(MINIATURE))
    reference.bind({name: value.numpy() for name, value in parameters.items()})
    timesteps, sigmas = O.ref_normal_sigma_schedule(steps)
    x = noise * sigmas[0]
    h = lambda a: a.astype(np.float16).astype(np.float32)
    for step in range(steps):
        sigma, sigma_next = float(sigmas[step]), float(sigmas[step + 1])
        scaled = h(x / np.sqrt(sigma * sigma + 1.0))
        prediction = reference.forward(np.concatenate([scaled, scaled]), float(timesteps[step]), h(context), h(pooled), time_ids)
        prediction = h(prediction)
        guided = h(prediction[:images] + scale * (prediction[images:] - prediction[:images]))
        x = x + ((x - (x - sigma * guided)) / sigma) * (sigma_next - sigma)
    reference.close()
    assert float(np.max(np.abs(got - x))) <= 3e-2 * float(np.max(np.abs(x)))
