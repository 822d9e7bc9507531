"""Data-parallel partition of a generation batch across GPUs.

The reference concatenates the CFG pair and `--batch N` images on the batch axis as
`[uncond x B || cond x B]` (src/cuda/denoiser.cpp:139-148, 225-243) and runs on one GPU. Every
image's CFG pair is independent through the whole UNet step (the guidance combine only mixes
`uncond_i` with `cond_i`, src/cuda/ops_kernels.cu:671-685), so the batch shards by image with
replicated weights and no collective inside the step."""
from __future__ import annotations

from typing import List, Tuple


def shard_images(total_images: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Half-open range [begin, end) of the images rank `rank` owns. Ranges are contiguous, cover
    every image exactly once and differ in size by at most one."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError("invalid rank / world size")
    if total_images < 0:
        raise ValueError("negative image count")
    base, extra = divmod(total_images, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def local_batch_rows(total_images: int, world_size: int, rank: int) -> List[int]:
    """Rows of the global `[uncond x B || cond x B]` batch that form this rank's local batch, in
    local order `[uncond_local || cond_local]`."""
    begin, end = shard_images(total_images, world_size, rank)
    return list(range(begin, end)) + [total_images + i for i in range(begin, end)]


def unet_batch(total_images: int, world_size: int, rank: int) -> int:
    """UNet batch of this rank (2 rows per image: the CFG pair)."""
    begin, end = shard_images(total_images, world_size, rank)
    return 2 * (end - begin)
