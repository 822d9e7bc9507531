"""The rank-2 projections of the SDXL Base UNet, enumerated the way the reference's parameter graph
declares them (src/sdxl.cpp:84-238 with the `base_1_0` configuration at :869-892 of the reference)
and the way its CUDA executor calls them (src/cuda/unet.cpp:20-181): 70 transformer blocks x 10
projections, 11 Transformer2D proj_in/proj_out pairs, 4 embedding Linears and 17 resnet
time_emb_proj = 743 calls of Ops::linear / Ops::linear_activation per UNet forward."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

ACT_NONE, ACT_SILU, ACT_GEGLU = 0, 1, 4

BLOCK_CHANNELS = (320, 640, 1280)
TRANSFORMER_DEPTH = (0, 2, 10)          # transformer layers per attention block at each level
CROSS_ATTENTION_DIM = 2048
TIME_EMBED_DIM = 1280
ADD_EMBED_INPUT = 2816                   # pooled text (1280) + 6 x 256 time ids
CONTEXT_TOKENS = 77


@dataclass(frozen=True)
class Projection:
    name: str          # parameter prefix, diffusers layout
    m: int             # rows
    n: int             # output features
    k: int             # input features
    bias: bool
    activation: int
    input_key: str     # projections with the same key read the same activation tensor


def _transformer_block(prefix: str, channels: int, tokens: int, context_rows: int) -> List[Projection]:
    c = channels
    out: List[Projection] = []
    for name in ("to_q", "to_k", "to_v"):
        out.append(Projection(f"{prefix}.attn1.{name}", tokens, c, c, False, ACT_NONE, f"{prefix}.norm1"))
    out.append(Projection(f"{prefix}.attn1.to_out.0", tokens, c, c, True, ACT_NONE, f"{prefix}.attn1"))
    out.append(Projection(f"{prefix}.attn2.to_q", tokens, c, c, False, ACT_NONE, f"{prefix}.norm2"))
    out.append(Projection(f"{prefix}.attn2.to_k", context_rows, c, CROSS_ATTENTION_DIM, False, ACT_NONE, "encoder_hidden_states"))
    out.append(Projection(f"{prefix}.attn2.to_v", context_rows, c, CROSS_ATTENTION_DIM, False, ACT_NONE, "encoder_hidden_states"))
    out.append(Projection(f"{prefix}.attn2.to_out.0", tokens, c, c, True, ACT_NONE, f"{prefix}.attn2"))
    out.append(Projection(f"{prefix}.ff.net.0.proj", tokens, 8 * c, c, True, ACT_GEGLU, f"{prefix}.norm3"))
    out.append(Projection(f"{prefix}.ff.net.2", tokens, c, 4 * c, True, ACT_NONE, f"{prefix}.ff.geglu"))
    return out


def _attention_block(prefix: str, level: int, tokens: int, context_rows: int) -> List[Projection]:
    c = BLOCK_CHANNELS[level]
    out = [Projection(f"{prefix}.proj_in", tokens, c, c, True, ACT_NONE, f"{prefix}.norm")]
    for layer in range(TRANSFORMER_DEPTH[level]):
        out += _transformer_block(f"{prefix}.transformer_blocks.{layer}", c, tokens, context_rows)
    out.append(Projection(f"{prefix}.proj_out", tokens, c, c, True, ACT_NONE, f"{prefix}.blocks_out"))
    return out


def unet_projections(batch: int = 2, height: int = 1024, width: int = 1024) -> List[Projection]:
    """Every projection of one UNet forward at UNet batch `batch` (CFG pair of one image = 2)."""
    latent_tokens = (height // 8) * (width // 8)
    tokens = [batch * latent_tokens // (4 ** level) for level in range(3)]
    context_rows = batch * CONTEXT_TOKENS
    out: List[Projection] = [
        Projection("time_embedding.linear_1", batch, TIME_EMBED_DIM, BLOCK_CHANNELS[0], True, ACT_SILU, "time_proj"),
        Projection("time_embedding.linear_2", batch, TIME_EMBED_DIM, TIME_EMBED_DIM, True, ACT_NONE, "time_embedding.act"),
        Projection("add_embedding.linear_1", batch, TIME_EMBED_DIM, ADD_EMBED_INPUT, True, ACT_SILU, "add_input"),
        Projection("add_embedding.linear_2", batch, TIME_EMBED_DIM, TIME_EMBED_DIM, True, ACT_NONE, "add_embedding.act"),
    ]

    def resnet(prefix: str, channels: int) -> Projection:
        return Projection(f"{prefix}.time_emb_proj", batch, channels, TIME_EMBED_DIM, True, ACT_NONE, "activated_temb")

    for level in range(3):                                     # down blocks: 2 resnets (+ attention) each
        for index in range(2):
            out.append(resnet(f"down_blocks.{level}.resnets.{index}", BLOCK_CHANNELS[level]))
            if TRANSFORMER_DEPTH[level]:
                out += _attention_block(f"down_blocks.{level}.attentions.{index}", level, tokens[level], context_rows)
    out.append(resnet("mid_block.resnets.0", BLOCK_CHANNELS[2]))
    out += _attention_block("mid_block.attentions.0", 2, tokens[2], context_rows)
    out.append(resnet("mid_block.resnets.1", BLOCK_CHANNELS[2]))
    for up_index, level in enumerate((2, 1, 0)):               # up blocks: 3 resnets (+ attention) each
        for index in range(3):
            out.append(resnet(f"up_blocks.{up_index}.resnets.{index}", BLOCK_CHANNELS[level]))
            if TRANSFORMER_DEPTH[level]:
                out += _attention_block(f"up_blocks.{up_index}.attentions.{index}", level, tokens[level], context_rows)
    return out


def total_ops(projections: List[Projection]) -> int:
    """2 * sum(M * N * K): 8.708e12 for the 743 projections at UNet batch 2."""
    return sum(2 * p.m * p.n * p.k for p in projections)


def weight_bytes_8bit(projections: List[Projection]) -> int:
    return sum(p.n * p.k for p in projections)
