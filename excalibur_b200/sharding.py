"""Batch sharding of the inference path across the GPUs of one node.

Images are independent, so a batch is cut into contiguous per-rank slices, every rank runs its own
pipeline replica (weights replicated) on its own GPU, and outputs are concatenated by rank.  There
is NO collective on the data path; torch.distributed is only used for the barrier around a timed
region and for the max-over-ranks of the timings.
"""


def shard_bounds(total, world, rank):
    """Contiguous slice [lo, hi) of `total` items for `rank`; the first total % world ranks get one more."""
    if world <= 0 or not (0 <= rank < world) or total < 0:
        raise ValueError("bad shard request total=%r world=%r rank=%r" % (total, world, rank))
    base, extra = divmod(total, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def all_bounds(total, world):
    return [shard_bounds(total, world, r) for r in range(world)]


def max_over_ranks(value, dist=None, device=None):
    """Slowest rank's value (the timing every multi-GPU number is quoted on)."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return float(value)
    import torch
    t = torch.tensor([float(value)], dtype=torch.float64, device=device or "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def aggregate_throughput(units_per_rank, world, elapsed_ms_max):
    """Whole-job units per second: all ranks' units over the slowest rank's time."""
    return units_per_rank * world / (elapsed_ms_max / 1000.0)
