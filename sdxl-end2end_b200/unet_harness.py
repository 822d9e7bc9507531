"""A synthetic SDXL UNet denoising loop around the quantized-Linear operator.

The reference's CUDA executor builds the UNet only from `Ops` calls (UNet::forward,
src/cuda/unet.cpp:183-310; transformer_block / transformer2d :98-181; build_time_embedding and the
resnet's time_emb_proj :20-51, 69-72) and drives it from the sampler loop
(Denoiser::run_loop, src/cuda/denoiser.cpp:195-312). This module follows those call sites one to
one. Every rank-2 projection (743 per forward with the SDXL Base configuration) goes through this
package's operator: `Ops.linear`, `Ops.linear_activation`, small grouped calls for projections that
share an input, a per-generation plan for the cross-attention K/V projections. The operators that
are not projections (convolution, GroupNorm, LayerNorm, attention, upsample, the CFG combine and
the Euler update) are plain PyTorch FP16 calls: they are scaffolding around the path, not part of
it. Weights are random-initialised, seeded per tensor name.

Data layout: spatial tensors are NCHW in channels-last memory, so that the token view
[B, H*W, C] the projections read and write is the same storage (the reference's flatten_spatial /
unflatten_spatial copies disappear).
"""
from __future__ import annotations

import math
import zlib
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from .api import (ACT_GEGLU, ACT_NONE, ACT_SILU, CudaError, FP8ScaleMode, FP8WeightLoadOptions,
                  INT8WeightLoadOptions, LinearCall, Ops, ScalarType, Weight)


@dataclass(frozen=True)
class UNetConfig:
    """The UNet fields of sdxl::SDXLConfig (include/sdxl/sdxl.hpp:26-34; base_1_0 at
    src/sdxl.cpp:869-892). Attention blocks exist at every level but the first."""

    channels: Tuple[int, ...] = (320, 640, 1280)
    heads: Tuple[int, ...] = (5, 10, 20)
    transformer_depth: Tuple[int, ...] = (1, 2, 10)
    cross_attention_dim: int = 2048
    time_embed_dim: int = 1280
    addition_time_embed_dim: int = 256
    addition_input_dim: int = 2816
    layers_per_block: int = 2
    norm_groups: int = 32
    latent_channels: int = 4

    @property
    def pooled_dim(self) -> int:
        return self.addition_input_dim - 6 * self.addition_time_embed_dim


BASE_1_0 = UNetConfig()


# --------------------------------------------------------------------------------------------
# parameter inventory
# --------------------------------------------------------------------------------------------
def unet_parameter_shapes(config: UNetConfig = BASE_1_0) -> Dict[str, Tuple[int, ...]]:
    """name -> shape of every UNet parameter, in the diffusers layout the reference's parameter
    graph declares (add_unet, src/sdxl.cpp:84-238). Names carry no `unet.` prefix."""
    c = config
    shapes: Dict[str, Tuple[int, ...]] = {}

    def linear(prefix, n, k, bias=True):
        shapes[f"{prefix}.weight"] = (n, k)
        if bias:
            shapes[f"{prefix}.bias"] = (n,)

    def conv(prefix, out_channels, in_channels, kernel):
        shapes[f"{prefix}.weight"] = (out_channels, in_channels, kernel, kernel)
        shapes[f"{prefix}.bias"] = (out_channels,)

    def norm(prefix, channels):
        shapes[f"{prefix}.weight"] = (channels,)
        shapes[f"{prefix}.bias"] = (channels,)

    def resnet(prefix, in_channels, out_channels):
        norm(f"{prefix}.norm1", in_channels)
        conv(f"{prefix}.conv1", out_channels, in_channels, 3)
        linear(f"{prefix}.time_emb_proj", out_channels, c.time_embed_dim)
        norm(f"{prefix}.norm2", out_channels)
        conv(f"{prefix}.conv2", out_channels, out_channels, 3)
        if in_channels != out_channels:
            conv(f"{prefix}.conv_shortcut", out_channels, in_channels, 1)

    def attention(prefix, channels, depth):
        norm(f"{prefix}.norm", channels)
        linear(f"{prefix}.proj_in", channels, channels)
        for layer in range(depth):
            block = f"{prefix}.transformer_blocks.{layer}"
            for index in (1, 2, 3):
                norm(f"{block}.norm{index}", channels)
            for name in ("to_q", "to_k", "to_v"):
                linear(f"{block}.attn1.{name}", channels, channels, bias=False)
            linear(f"{block}.attn1.to_out.0", channels, channels)
            linear(f"{block}.attn2.to_q", channels, channels, bias=False)
            linear(f"{block}.attn2.to_k", channels, c.cross_attention_dim, bias=False)
            linear(f"{block}.attn2.to_v", channels, c.cross_attention_dim, bias=False)
            linear(f"{block}.attn2.to_out.0", channels, channels)
            linear(f"{block}.ff.net.0.proj", 8 * channels, channels)
            linear(f"{block}.ff.net.2", channels, 4 * channels)
        linear(f"{prefix}.proj_out", channels, channels)

    conv("conv_in", c.channels[0], c.latent_channels, 3)
    linear("time_embedding.linear_1", c.time_embed_dim, c.channels[0])
    linear("time_embedding.linear_2", c.time_embed_dim, c.time_embed_dim)
    linear("add_embedding.linear_1", c.time_embed_dim, c.addition_input_dim)
    linear("add_embedding.linear_2", c.time_embed_dim, c.time_embed_dim)
    levels = len(c.channels)
    previous = c.channels[0]
    skip_channels = [c.channels[0]]
    for level, channels in enumerate(c.channels):
        for layer in range(c.layers_per_block):
            resnet(f"down_blocks.{level}.resnets.{layer}", previous, channels)
            if level > 0:
                attention(f"down_blocks.{level}.attentions.{layer}", channels, c.transformer_depth[level])
            previous = channels
            skip_channels.append(channels)
        if level + 1 < levels:
            conv(f"down_blocks.{level}.downsamplers.0.conv", channels, channels, 3)
            skip_channels.append(channels)
    resnet("mid_block.resnets.0", previous, previous)
    attention("mid_block.attentions.0", previous, c.transformer_depth[-1])
    resnet("mid_block.resnets.1", previous, previous)
    for block in range(levels):
        level = levels - 1 - block
        channels = c.channels[level]
        for layer in range(c.layers_per_block + 1):
            resnet(f"up_blocks.{block}.resnets.{layer}", previous + skip_channels.pop(), channels)
            if level > 0:
                attention(f"up_blocks.{block}.attentions.{layer}", channels, c.transformer_depth[level])
            previous = channels
        if block + 1 < levels:
            conv(f"up_blocks.{block}.upsamplers.0.conv", channels, channels, 3)
    norm("conv_norm_out", previous)
    conv("conv_out", c.latent_channels, previous, 3)
    return shapes


def is_projection_weight(name: str, shape: Sequence[int]) -> bool:
    """The reference's eligibility rule for the quantised loaders: a rank-2 `.weight` that is not
    an embedding table (is_linear_weight, src/cuda/weights.cu:185-193; load_unet_fp8 :484-486)."""
    if len(shape) != 2 or not name.endswith(".weight"):
        return False
    return not ("embeddings." in name or "token_embedding" in name or "position_embedding" in name)


def synthetic_parameters(config: UNetConfig, device, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random-init FP32 parameters, one generator per tensor seeded from the tensor's name (so
    every rank, and every process, draws the same values without communicating). Matrices and
    kernels ~ N(0, 1/fan_in); norm scales ~ 1 + N(0, 0.05^2); every bias ~ N(0, 0.02^2)."""
    out: Dict[str, torch.Tensor] = {}
    for name, shape in unet_parameter_shapes(config).items():
        generator = torch.Generator(device=device)
        generator.manual_seed((zlib.crc32(name.encode()) ^ (seed * 0x9E3779B1)) & 0x7FFFFFFF)
        values = torch.randn(shape, generator=generator, dtype=torch.float32, device=device)
        if name.endswith(".bias"):
            values *= 0.02
        elif len(shape) == 1:
            values = 1.0 + 0.05 * values
        else:
            fan_in = 1
            for dimension in shape[1:]:
                fan_in *= dimension
            values *= 1.0 / math.sqrt(fan_in)
        out[name] = values
    return out


# --------------------------------------------------------------------------------------------
# sigma schedule and sampler arithmetic
# --------------------------------------------------------------------------------------------
def normal_sigma_schedule(steps: int, training_timesteps: int = 1000, beta_start: float = 0.00085,
                          beta_end: float = 0.012) -> Tuple[List[float], List[float]]:
    """SigmaSchedule(steps, Normal) of the reference (src/scheduler.cpp:47-127, 640-668): scaled-linear
    betas, sigma = sqrt((1 - alpha_bar) / alpha_bar), log-linear interpolation at the evenly spaced
    training positions 999 .. 0, the UNet timestep = nearest training index in log-sigma, and a
    final sigma of 0. Returns (timesteps[steps], sigmas[steps + 1])."""
    import numpy as np
    start, end = math.sqrt(float(np.float32(beta_start))), math.sqrt(float(np.float32(beta_end)))
    product = 1.0
    training: List[float] = []
    for index in range(training_timesteps):
        value = start + (end - start) * (index / (training_timesteps - 1))
        beta = float(np.float32(value * value))
        product *= 1.0 - beta
        alpha = float(np.float32(product))
        training.append(float(np.float32(math.sqrt((1.0 - alpha) / alpha))))
    log_training = [math.log(s) for s in training]
    maximum = float(training_timesteps - 1)
    timesteps: List[float] = []
    sigmas: List[float] = []
    for index in range(steps):
        position = maximum if steps == 1 else float(np.float32(maximum) - np.float32(maximum) * np.float32(index) / np.float32(steps - 1))
        position = min(max(position, 0.0), maximum)
        lower = int(math.floor(position))
        upper = min(training_timesteps - 1, lower + 1)
        fraction = float(np.float32(position) - np.float32(lower))
        sigma = float(np.float32(math.exp((1.0 - fraction) * log_training[lower] + fraction * log_training[upper])))
        sigmas.append(sigma)
        if sigma <= training[0]:
            timesteps.append(0.0)
        elif sigma >= training[-1]:
            timesteps.append(maximum)
        else:
            import bisect
            above = bisect.bisect_left(training, sigma)
            below = above - 1
            target = math.log(sigma)
            timesteps.append(float(below if abs(target - log_training[below]) <= abs(log_training[above] - target) else above))
    sigmas.append(0.0)
    return timesteps, sigmas


def sinusoidal_embedding(values: torch.Tensor, dimension: int) -> torch.Tensor:
    """timestep_scalar_kernel / timestep_values_kernel (src/cuda/ops_kernels.cu:632-669): for each
    value v, [cos(v * f_i) | sin(v * f_i)] with f_i = exp(-ln(10000) * i / half), in FP32, rounded to
    FP16. `values` is FP32 [rows]; returns FP16 [rows, dimension]."""
    half = dimension // 2
    index = torch.arange(half, device=values.device, dtype=torch.float32)
    frequencies = torch.exp(index * (-math.log(10000.0) / max(half, 1)))
    angles = values.to(torch.float32)[:, None] * frequencies[None, :]
    return torch.cat([torch.cos(angles), torch.sin(angles)], dim=1).to(torch.float16)


# --------------------------------------------------------------------------------------------
# the executor
# --------------------------------------------------------------------------------------------
class UNetHarness:
    """UNet::forward of the reference's CUDA executor (src/cuda/unet.cpp:183-310) with this
    package's operator behind every projection.

    precision: "e4m3" / "e5m2" (FP8 per-output-channel weights, native FP8 activations), "int8"
    (W8A8 ConvRot, group-256 rule) or "f16" (dense FP16 weights). `fuse_residual` folds the
    add_in_place after to_out / ff.net.2 / proj_out into the projection's epilogue.
    `fuse_layer_norm` runs the three LayerNorms of a transformer block through the library's
    kernel, fused with the activation quantiser of the projections that read them (to_q / to_k /
    to_v, attn2.to_q, ff.net.0.proj) for the quantised profiles; without it they are separate
    PyTorch layer_norm calls and the projections quantise their input themselves.
    `fuse_group_norm` runs GroupNorm (+ SiLU, + the resnet's time-embedding bias in front of norm2) on the
    channels-last activations through the library's scaffolding kernel instead of PyTorch's group_norm,
    which copies a channels-last tensor to NCHW and back around the norm."""

    def __init__(self, ops: Ops, config: UNetConfig = BASE_1_0, precision: str = "e4m3", seed: int = 0,
                 parameters: Optional[Dict[str, torch.Tensor]] = None, fuse_residual: bool = True,
                 group_attention_inputs: bool = True, device: Optional[torch.device] = None,
                 fuse_layer_norm: bool = True, fuse_group_norm: bool = True):
        if precision not in ("e4m3", "e5m2", "int8", "f16"):
            raise CudaError(f"unknown precision profile {precision}")
        self.ops = ops
        self.config = config
        self.precision = precision
        self.fuse_residual = fuse_residual
        self.group_attention_inputs = group_attention_inputs
        self.fuse_layer_norm = fuse_layer_norm
        self.fuse_group_norm = fuse_group_norm
        self.device = device if device is not None else torch.device("cuda", ops.ctx.device)
        source = parameters if parameters is not None else synthetic_parameters(config, self.device, seed)
        self.projections: Dict[str, Weight] = {}
        self.tensors: Dict[str, torch.Tensor] = {}
        for name, shape in unet_parameter_shapes(config).items():
            values = source[name].to(self.device)
            if tuple(values.shape) != tuple(shape):
                raise CudaError(f"parameter {name} has shape {tuple(values.shape)}, expected {tuple(shape)}")
            if is_projection_weight(name, shape):
                self.projections[name[: -len(".weight")]] = self._pack(values)
            elif len(shape) == 4:
                self.tensors[name] = values.to(torch.float16).contiguous(memory_format=torch.channels_last)
            else:
                self.tensors[name] = values.to(torch.float16).contiguous()
        # conv1's bias and the time-embedding projection's bias are both added per (image, channel) in front
        # of norm2: one vector, added once (by the norm kernel's channel bias) instead of twice over the tensor
        self._temb_bias: Dict[str, torch.Tensor] = {}
        for name in self.projections:
            if name.endswith(".time_emb_proj"):
                prefix = name[: -len(".time_emb_proj")]
                folded = self.tensors[f"{name}.bias"].float() + self.tensors[f"{prefix}.conv1.bias"].float()
                self._temb_bias[name] = folded.to(torch.float16).contiguous()
        self._amax_word = torch.zeros(1, dtype=torch.int32, device=self.device)    # zero between uses: the reader clears it
        self.projection_calls = 0          # projections issued by the last forward (K/V cache included)
        self._kv: Dict[str, torch.Tensor] = {}
        self._kv_plan = None
        self._kv_source: Optional[torch.Tensor] = None
        self._temb_plan = None

    # -- weights ----------------------------------------------------------------------------------
    def _pack(self, values: torch.Tensor) -> Weight:
        half = values.to(torch.float16).contiguous()
        if self.precision == "f16":
            return self.ops.fp16_weight(half)
        if self.precision == "int8":
            return self.ops.upload_or_quantize_int8_weight(half, None, INT8WeightLoadOptions())
        fmt = ScalarType.Float8E4M3 if self.precision == "e4m3" else ScalarType.Float8E5M2
        return self.ops.upload_fp8_weight(half, FP8WeightLoadOptions(format=fmt, scale_mode=FP8ScaleMode.PerOutputChannel))

    def projection_names(self) -> List[str]:
        return list(self.projections.keys())

    def _follow_current_stream(self) -> None:
        """The operator launches on PyTorch's current stream (the capture stream inside a graph capture)."""
        if self.device.type == "cuda":
            self.ops.ctx.set_stream(torch.cuda.current_stream(self.device))

    # -- small helpers ------------------------------------------------------------------------------
    def _bias(self, prefix: str) -> torch.Tensor:
        return self.tensors[f"{prefix}.bias"]

    def _linear(self, x, prefix, activation=ACT_NONE, residual=None, out=None, bias=True, y_amax=None, x_amax=None):
        """x is an FP16 tensor, or the (xq, xq_scales) pair of a fused LayerNorm. y_amax / x_amax: the word
        through which a projection hands the maximum of its output to the FP8 quantiser of the next one."""
        self.projection_calls += 1
        b = self._bias(prefix) if bias else None
        quantised = {}
        if y_amax is not None:
            quantised["y_amax"] = y_amax
        if x_amax is not None:
            quantised["x_amax"] = x_amax
        if isinstance(x, tuple):
            quantised.update({"xq": x[0], "xq_scales": x[1]})
            x = None
        if activation != ACT_NONE:
            return self.ops.linear_activation(x, self.projections[prefix], b, activation, **quantised)
        if residual is not None and not self.fuse_residual:
            y = self.ops.linear(x, self.projections[prefix], b, **quantised)
            residual.add_(y)                                   # Ops::add_in_place, FP16
            return residual
        return self.ops.linear(x, self.projections[prefix], b, residual=residual, out=out, **quantised)

    def _group_norm(self, x, prefix, eps=1e-5, silu=False, channel_bias=None):
        """Ops::group_norm_nchw / group_norm_silu_nchw; `channel_bias` [B, C] is the add_spatial_bias in front."""
        gamma, beta = self.tensors[f"{prefix}.weight"], self.tensors[f"{prefix}.bias"]
        if self.fuse_group_norm and x.dim() == 4 and x.shape[1] % 8 == 0 and x.shape[1] <= 3072 and \
                x.is_contiguous(memory_format=torch.channels_last):
            return self.ops.group_norm_nhwc(x, gamma, beta, self.config.norm_groups, eps, silu, channel_bias)
        if channel_bias is not None:
            x = x + channel_bias[:, :, None, None]
        y = F.group_norm(x, self.config.norm_groups, gamma, beta, eps)
        return F.silu(y) if silu else y

    def _conv(self, x, prefix, stride=1, padding=1, bias=True):
        return F.conv2d(x, self.tensors[f"{prefix}.weight"], self.tensors[f"{prefix}.bias"] if bias else None,
                        stride=stride, padding=padding)

    def _layer_norm(self, x, prefix, consumer: str):
        """Ops::layer_norm in front of the projection `consumer`. Returns an FP16 tensor, or with the
        fused quantised form the (xq, xq_scales) pair that projection (and its siblings) take."""
        gamma, beta = self.tensors[f"{prefix}.weight"], self.tensors[f"{prefix}.bias"]
        if not self.fuse_layer_norm:
            return F.layer_norm(x, (x.shape[-1],), gamma, beta, 1e-5)
        if self.precision == "f16":
            return self.ops.layer_norm(x, gamma, beta, 1e-5)
        return self.ops.layer_norm_quantized(x, gamma, beta, self.projections[consumer], 1e-5)

    @staticmethod
    def _attention(query, key, value, heads):
        batch, tokens, channels = query.shape
        head_dim = channels // heads
        q = query.view(batch, tokens, heads, head_dim).transpose(1, 2)
        k = key.view(batch, key.shape[1], heads, head_dim).transpose(1, 2)
        v = value.view(batch, value.shape[1], heads, head_dim).transpose(1, 2)
        out = F.scaled_dot_product_attention(q, k, v)
        return out.transpose(1, 2).reshape(batch, tokens, channels).contiguous()

    # -- per-generation work: cross-attention K/V of every block ----------------------------------------
    def prepare_conditioning(self, encoder_hidden_states: torch.Tensor) -> None:
        """All attn2.to_k / attn2.to_v projections of the UNet in one grouped launch. Their input, the
        text encoder's hidden states, does not change between denoising steps (the reference recomputes
        them in every step, src/cuda/unet.cpp:125-126)."""
        if encoder_hidden_states.dtype != torch.float16 or encoder_hidden_states.dim() != 3 or \
                encoder_hidden_states.shape[2] != self.config.cross_attention_dim:
            raise CudaError("CUDA UNet input shape mismatch")
        source = encoder_hidden_states.contiguous()
        if self._kv_plan is not None and self._kv_source is not None and self._kv_source.shape == source.shape:
            self._kv_source.copy_(source)
            self._kv_plan.run()
            return
        if self._kv_plan is not None:
            self._kv_plan.close()
        self._kv_source = source.clone()
        names = [name for name in self.projections if name.endswith(".attn2.to_k") or name.endswith(".attn2.to_v")]
        calls = [LinearCall(self._kv_source, self.projections[name]) for name in names]
        self._kv_plan = self.ops.plan(calls)
        self._kv = dict(zip(names, self._kv_plan.run()))

    # -- UNet::build_time_embedding + the 17 time_emb_proj ---------------------------------------------
    def _time_embedding(self, timestep: torch.Tensor, batch: int, pooled: torch.Tensor, time_ids: torch.Tensor):
        c = self.config
        time_projection = sinusoidal_embedding(timestep.reshape(1).expand(batch), c.channels[0])
        embedding = self._linear(time_projection, "time_embedding.linear_1", ACT_SILU)
        embedding = self._linear(embedding, "time_embedding.linear_2")
        additional_time = sinusoidal_embedding(time_ids.reshape(-1), c.addition_time_embed_dim).reshape(batch, -1)
        additional_input = torch.cat([pooled, additional_time], dim=1).contiguous()
        additional = self._linear(additional_input, "add_embedding.linear_1", ACT_SILU)
        additional = self._linear(additional, "add_embedding.linear_2")
        activated = F.silu(embedding + additional)            # Ops::add_silu
        # every resnet's time_emb_proj reads this one tensor: one grouped launch for all of them
        names = [name for name in self.projections if name.endswith(".time_emb_proj")]
        if self._temb_plan is None or self._temb_input.shape != activated.shape:
            if self._temb_plan is not None:
                self._temb_plan.close()
            self._temb_input = activated.clone()
            calls = [LinearCall(self._temb_input, self.projections[name], self._temb_bias[name]) for name in names]
            self._temb_plan = self.ops.plan(calls)
            self._temb_outputs = dict(zip(names, [call.y for call in self._temb_plan.calls]))
        self._temb_input.copy_(activated)
        self._temb_plan.run()
        self.projection_calls += len(names)
        return self._temb_outputs

    # -- blocks -------------------------------------------------------------------------------------
    def _resnet(self, prefix, x, projected_temb):
        hidden = self._group_norm(x, f"{prefix}.norm1", silu=True)
        hidden = self._conv(hidden, f"{prefix}.conv1", bias=False)           # its bias travels with the time embedding
        # add_spatial_bias, then group_norm_silu
        hidden = self._group_norm(hidden, f"{prefix}.norm2", silu=True, channel_bias=projected_temb[f"{prefix}.time_emb_proj"])
        residual = x
        if f"{prefix}.conv_shortcut.weight" in self.tensors:
            residual = self._conv(x, f"{prefix}.conv_shortcut", padding=0)
        if self.fuse_group_norm and hidden.shape[1] % 8 == 0 and residual.is_contiguous(memory_format=torch.channels_last):
            hidden = self._conv(hidden, f"{prefix}.conv2", bias=False)
            if hidden.is_contiguous(memory_format=torch.channels_last):
                # conv2's bias add and the residual add in one pass
                return self.ops.bias_residual_add_nhwc(hidden, self.tensors[f"{prefix}.conv2.bias"], residual)
            return (hidden + self.tensors[f"{prefix}.conv2.bias"][None, :, None, None]) + residual
        hidden = self._conv(hidden, f"{prefix}.conv2")
        return hidden + residual

    def _transformer_block(self, prefix, hidden, heads):
        names = [f"{prefix}.attn1.to_q", f"{prefix}.attn1.to_k", f"{prefix}.attn1.to_v"]
        normalized = self._layer_norm(hidden, f"{prefix}.norm1", names[0])
        if self.group_attention_inputs:
            # to_q / to_k / to_v read the same tensor: one quantisation, one GEMM launch
            if isinstance(normalized, tuple):
                calls = [LinearCall(None, self.projections[name], xq=normalized[0], xq_scales=normalized[1]) for name in names]
            else:
                calls = [LinearCall(normalized, self.projections[name]) for name in names]
            query, key, value = self.ops.linear_grouped(calls)
            self.projection_calls += 3
        else:
            query, key, value = (self._linear(normalized, name, bias=False) for name in names)
        attention = self._attention(query, key, value, heads)
        hidden = self._linear(attention, f"{prefix}.attn1.to_out.0", residual=hidden, out=hidden)

        normalized = self._layer_norm(hidden, f"{prefix}.norm2", f"{prefix}.attn2.to_q")
        query = self._linear(normalized, f"{prefix}.attn2.to_q", bias=False)
        key, value = self._kv[f"{prefix}.attn2.to_k"], self._kv[f"{prefix}.attn2.to_v"]
        attention = self._attention(query, key, value, heads)
        hidden = self._linear(attention, f"{prefix}.attn2.to_out.0", residual=hidden, out=hidden)

        normalized = self._layer_norm(hidden, f"{prefix}.norm3", f"{prefix}.ff.net.0.proj")
        # FP8: ff.net.0.proj's epilogue leaves max |GEGLU output| for the quantiser of ff.net.2
        word = self._amax_word if self.precision in ("e4m3", "e5m2") else None
        feed_forward = self._linear(normalized, f"{prefix}.ff.net.0.proj", ACT_GEGLU, y_amax=word)
        hidden = self._linear(feed_forward, f"{prefix}.ff.net.2", residual=hidden, out=hidden, x_amax=word)
        return hidden

    def _transformer2d(self, prefix, x, depth, heads):
        batch, channels, height, width = x.shape
        normalized = self._group_norm(x, f"{prefix}.norm", eps=1e-6)
        tokens = normalized.permute(0, 2, 3, 1).reshape(batch, height * width, channels)     # flatten_spatial
        if not tokens.is_contiguous():
            tokens = tokens.contiguous()
        hidden = self._linear(tokens, f"{prefix}.proj_in")
        for layer in range(depth):
            hidden = self._transformer_block(f"{prefix}.transformer_blocks.{layer}", hidden, heads)
        skip = x.permute(0, 2, 3, 1).reshape(batch, height * width, channels)                # the block's input as tokens
        if not skip.is_contiguous():
            skip = skip.contiguous()
        hidden = self._linear(hidden, f"{prefix}.proj_out", residual=skip)                     # + add_in_place(hidden, input)
        return hidden.view(batch, height, width, channels).permute(0, 3, 1, 2)                 # unflatten_spatial

    # -- UNet::forward --------------------------------------------------------------------------------
    def forward(self, latent_sample: torch.Tensor, timestep, pooled_text_embeds: torch.Tensor,
                time_ids: torch.Tensor) -> torch.Tensor:
        """latent_sample FP16 [B, 4, H, W]; timestep a float or a one-element FP32 device tensor;
        pooled_text_embeds FP16 [B, P]; time_ids FP16 or FP32 [B, 6]. prepare_conditioning() must have
        run for this batch's text states. Returns the FP16 prediction [B, 4, H, W]."""
        c = self.config
        if latent_sample.dim() != 4 or latent_sample.shape[1] != c.latent_channels or \
                pooled_text_embeds.dim() != 2 or time_ids.dim() != 2 or time_ids.shape[1] != 6:
            raise CudaError("CUDA UNet input shape mismatch")
        batch = latent_sample.shape[0]
        if pooled_text_embeds.shape[0] != batch or time_ids.shape[0] != batch or \
                self._kv_source is None or self._kv_source.shape[0] != batch:
            raise CudaError("CUDA UNet conditioning batch mismatch")
        self._follow_current_stream()
        self.projection_calls = len(self._kv)          # the cached K/V projections belong to the forward
        if not torch.is_tensor(timestep):
            timestep = torch.tensor([float(timestep)], dtype=torch.float32, device=self.device)
        projected_temb = self._time_embedding(timestep, batch, pooled_text_embeds.to(torch.float16), time_ids)

        hidden = self._conv(latent_sample.to(torch.float16).contiguous(memory_format=torch.channels_last), "conv_in")
        residuals = [hidden]
        levels = len(c.channels)
        for level in range(levels):
            for layer in range(c.layers_per_block):
                hidden = self._resnet(f"down_blocks.{level}.resnets.{layer}", hidden, projected_temb)
                if level > 0:
                    hidden = self._transformer2d(f"down_blocks.{level}.attentions.{layer}", hidden,
                                                 c.transformer_depth[level], c.heads[level])
                residuals.append(hidden)
            if level + 1 < levels:
                hidden = self._conv(hidden, f"down_blocks.{level}.downsamplers.0.conv", stride=2)
                residuals.append(hidden)
        hidden = self._resnet("mid_block.resnets.0", hidden, projected_temb)
        hidden = self._transformer2d("mid_block.attentions.0", hidden, c.transformer_depth[-1], c.heads[-1])
        hidden = self._resnet("mid_block.resnets.1", hidden, projected_temb)
        for block in range(levels):
            level = levels - 1 - block
            for layer in range(c.layers_per_block + 1):
                skip = residuals.pop()
                hidden = torch.cat([hidden, skip], dim=1)                                     # concat_channels
                hidden = self._resnet(f"up_blocks.{block}.resnets.{layer}", hidden, projected_temb)
                if level > 0:
                    hidden = self._transformer2d(f"up_blocks.{block}.attentions.{layer}", hidden,
                                                 c.transformer_depth[level], c.heads[level])
            if block + 1 < levels:
                target = residuals[-1].shape[2:]
                hidden = F.interpolate(hidden, size=tuple(target), mode="nearest")            # nearest_upsample
                hidden = self._conv(hidden, f"up_blocks.{block}.upsamplers.0.conv")
        if residuals:
            raise CudaError("CUDA UNet left unused residual tensors")
        hidden = self._group_norm(hidden, "conv_norm_out", silu=True)
        hidden = self._conv(hidden, "conv_out")
        if hidden.shape != latent_sample.shape:
            raise CudaError("CUDA UNet output shape differs from latent input")
        return hidden

    def close(self) -> None:
        for plan in (self._kv_plan, self._temb_plan):
            if plan is not None:
                plan.close()
        self._kv_plan = self._temb_plan = None


# --------------------------------------------------------------------------------------------
# the denoising loop
# --------------------------------------------------------------------------------------------
class EulerDenoiser:
    """Denoiser::run_loop with the Euler sampler and classifier-free guidance
    (src/cuda/denoiser.cpp:195-243, 297-312): per step the latents are scaled by 1/sqrt(sigma^2 + 1),
    repeated as [uncond x B | cond x B] (euler_scale_repeat_input), run through the UNet, combined as
    uncond + scale * (cond - uncond) (cfg_kernel, src/cuda/ops_kernels.cu:671-685), and stepped with
    x + ((x - (x - sigma * eps)) / sigma) * (sigma_next - sigma) on FP32 latents
    (euler_step_f16_f32_kernel, :1031-1050, epsilon prediction).

    One step is optionally captured once as a CUDA graph and replayed (the reference captures its
    denoise loop the same way, src/cuda/denoise_graph.cpp); sigma, the next sigma and the timestep are
    read from a small device tensor that is refreshed before each replay."""

    def __init__(self, unet: UNetHarness, images: int, height: int = 1024, width: int = 1024, steps: int = 20,
                 guidance_scale: float = 5.0, use_graph: bool = True):
        self.unet = unet
        self.images = images
        self.steps = steps
        self.guidance_scale = guidance_scale
        self.use_graph = use_graph
        device = unet.device
        c = unet.config
        self.timesteps, self.sigmas = normal_sigma_schedule(steps)
        self.latents = torch.zeros((images, c.latent_channels, height // 8, width // 8), dtype=torch.float32, device=device)
        self.pooled = torch.zeros((2 * images, c.pooled_dim), dtype=torch.float16, device=device)
        self.time_ids = torch.zeros((2 * images, 6), dtype=torch.float16, device=device)
        self.scalars = torch.zeros(3, dtype=torch.float32, device=device)      # sigma, sigma_next, timestep
        table = [[self.sigmas[i], self.sigmas[i + 1], self.timesteps[i]] for i in range(steps)]
        self._scalar_table = torch.tensor(table, dtype=torch.float32)
        if device.type == "cuda":
            self._scalar_table = self._scalar_table.pin_memory()
        self._graph = None
        self.step_index = 0

    def set_conditioning(self, prompt_embeds: torch.Tensor, pooled: torch.Tensor, time_ids: torch.Tensor) -> None:
        """prompt_embeds FP16 [2 * images, 77, cross_dim] laid out [uncond x images | cond x images]."""
        self.unet._follow_current_stream()
        self.unet.prepare_conditioning(prompt_embeds)
        self.pooled.copy_(pooled)
        self.time_ids.copy_(time_ids)

    def set_latents(self, latents: torch.Tensor) -> None:
        """Unit-variance noise; scaled by the first sigma like the reference's initial latents."""
        self.latents.copy_(latents.to(torch.float32) * self.sigmas[0])
        self.step_index = 0

    def _step_body(self) -> None:
        sigma, sigma_next, timestep = self.scalars[0], self.scalars[1], self.scalars[2]
        scaled = (self.latents * torch.rsqrt(sigma * sigma + 1.0)).to(torch.float16)
        model_input = scaled.repeat(2, 1, 1, 1)                                     # [uncond | cond]
        prediction = self.unet.forward(model_input, timestep.reshape(1), self.pooled, self.time_ids)
        prediction = prediction.to(torch.float32)
        unconditional, conditional = prediction[: self.images], prediction[self.images:]
        guided = (unconditional + self.guidance_scale * (conditional - unconditional)).to(torch.float16).to(torch.float32)
        # epsilon prediction: original = x - sigma * eps; derivative = (x - original) / sigma
        original = self.latents - sigma * guided
        derivative = (self.latents - original) / sigma
        self.latents.add_(derivative * (sigma_next - sigma))

    def step(self) -> None:
        """One denoising step (wraps around to the first sigma after the last step)."""
        index = self.step_index % self.steps
        self.scalars.copy_(self._scalar_table[index], non_blocking=True)
        if not self.use_graph:
            self._step_body()
        else:
            if self._graph is None:
                self._capture()
            self._graph.replay()
        self.step_index += 1

    def _capture(self) -> None:
        # Warm up outside the capture (plans, cuDNN algorithm selection, allocator pools), with the
        # latents put back afterwards so that capturing is invisible to the caller.
        saved = self.latents.clone()
        side = torch.cuda.Stream(device=self.unet.device)
        side.wait_stream(torch.cuda.current_stream(self.unet.device))
        with torch.cuda.stream(side):
            for _ in range(2):
                self._step_body()
        torch.cuda.current_stream(self.unet.device).wait_stream(side)
        torch.cuda.synchronize(self.unet.device)
        self.latents.copy_(saved)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self._step_body()
        torch.cuda.synchronize(self.unet.device)
        self.latents.copy_(saved)
        self.unet._follow_current_stream()
        self._graph = graph

    def run(self) -> torch.Tensor:
        for _ in range(self.steps):
            self.step()
        return self.latents
