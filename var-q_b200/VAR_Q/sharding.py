"""Batch sharding of a generation job across GPUs (one process per GPU, no collective on the
hot path).

Every sample's KV cache and attention are independent, so the work is partitioned by batch.
With classifier-free guidance the model runs each image as a (conditional, unconditional) pair
and combines the two every step (VAR/models/var.py:154-157,175-176;
Infinity/infinity/models/infinity.py:497-513,575-586), so a pair is never split: shards are cut
in units of images and the doubled batch of a shard holds both halves of its images.

Statistics of the reference modes span the batch (VAR_Q/quant.py:78-95), hence a shard's scales
equal those of the reference run on that shard's sub-batch, not on the full batch.
"""
from typing import List, Tuple


def shard_images(n_images: int, world_size: int, rank: int) -> Tuple[int, int]:
    """[begin, end) image indices of `rank`; sizes differ by at most one, larger shards first."""
    if world_size < 1 or not (0 <= rank < world_size) or n_images < 0:
        raise ValueError(f"bad shard request: n_images={n_images}, world_size={world_size}, rank={rank}")
    base, extra = divmod(n_images, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def cfg_rows(begin: int, end: int, n_images: int) -> List[int]:
    """Rows of the CFG-doubled batch [cond(0..n) | uncond(0..n)] that belong to images [begin, end)."""
    return list(range(begin, end)) + list(range(n_images + begin, n_images + end))


def aggregate_throughput(units_per_rank: List[float], seconds_per_rank: List[float]) -> float:
    """Whole-job throughput: all units over the slowest rank's time."""
    if not units_per_rank or len(units_per_rank) != len(seconds_per_rank):
        raise ValueError("need one (units, seconds) pair per rank")
    slowest = max(seconds_per_rank)
    if slowest <= 0:
        raise ValueError("non-positive time")
    return sum(units_per_rank) / slowest
