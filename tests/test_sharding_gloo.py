"""Host-side logic of the N > 1 path on CPU: the image partition and the max-over-ranks timing /
result gather that bench.py performs, run as two gloo ranks."""
import importlib
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, total_images: int, result_file: str):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sharding = importlib.import_module("sdxl-end2end_b200.sharding")
    begin, end = sharding.shard_images(total_images, world, rank)
    # every rank learns every range: together they partition the images
    ranges = [None] * world
    dist.all_gather_object(ranges, (begin, end))
    covered = sorted(i for (b, e) in ranges for i in range(b, e))
    assert covered == list(range(total_images)), ranges
    # the "step": each rank transforms its local [uncond || cond] rows; rank 0 gathers the images
    torch.manual_seed(0)
    global_batch = torch.randn(2 * total_images, 4, 8, 8)
    rows = sharding.local_batch_rows(total_images, world, rank)
    local = global_batch[rows]
    half = len(rows) // 2
    guided = local[:half] + 7.5 * (local[half:] - local[:half])          # CFG combine per image
    gathered = [None] * world
    dist.gather_object(guided, gathered if rank == 0 else None, dst=0)
    # timing reduction used by bench.py: the slowest rank defines the step time
    elapsed = torch.tensor([1.0 + rank])
    dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    assert elapsed.item() == float(world)
    if rank == 0:
        merged = torch.cat(gathered)
        reference = global_batch[:total_images] + 7.5 * (global_batch[total_images:] - global_batch[:total_images])
        torch.save({"equal": bool(torch.equal(merged, reference)), "unet_batches":
                    [sharding.unet_batch(total_images, world, r) for r in range(world)]}, result_file)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("total_images", [8, 5])
def test_two_rank_partition_and_gather(tmp_path, total_images):
    result_file = str(tmp_path / "result.pt")
    mp.spawn(_worker, args=(2, _free_port(), total_images, result_file), nprocs=2, join=True)
    result = torch.load(result_file)
    assert result["equal"]
    assert sum(result["unet_batches"]) == 2 * total_images


def test_shard_images_properties():
    sharding = importlib.import_module("sdxl-end2end_b200.sharding")
    for total in (0, 1, 7, 8, 16):
        for world in (1, 2, 4, 8):
            ranges = [sharding.shard_images(total, world, r) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
            sizes = [e - b for b, e in ranges]
            assert max(sizes) - min(sizes) <= 1
    assert sharding.local_batch_rows(8, 4, 1) == [2, 3, 10, 11]
    assert sharding.unet_batch(8, 8, 3) == 2
    with pytest.raises(ValueError):
        sharding.shard_images(8, 2, 2)
