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


def _parse_cpulist(text):
    cpus = set()
    for part in text.strip().split(","):
        if not part:
            continue
        if "-" in part:
            a, b = part.split("-")
            cpus.update(range(int(a), int(b) + 1))
        else:
            cpus.add(int(part))
    return cpus


def gpu_local_cpus(pci_bus_id, sysfs="/sys/bus/pci/devices"):
    """CPUs of the NUMA node a GPU hangs off ("0000:1b:00.0" -> {0..31}), or None when the platform
    does not say (no sysfs entry, node -1, empty list)."""
    import os
    path = os.path.join(sysfs, pci_bus_id.lower(), "local_cpulist")
    try:
        cpus = _parse_cpulist(open(path).read())
    except (OSError, ValueError):
        return None
    return cpus or None


def bind_host_thread_to_gpu(device_index):
    """Pin the calling process to the CPUs next to `device_index`'s PCIe root, so that the pinned host
    buffers it allocates afterwards (first touch) and its copy submissions stay on the GPU's NUMA node:
    with one rank per GPU, host-to-device copies of eight ranks otherwise cross the socket link.
    Best effort: returns the CPU set used, or None when nothing was changed."""
    import os
    try:
        import torch
        p = torch.cuda.get_device_properties(device_index)
        bus = "%04x:%02x:%02x.0" % (p.pci_domain_id, p.pci_bus_id, p.pci_device_id)
    except Exception:
        return None
    cpus = gpu_local_cpus(bus)
    if not cpus:
        return None
    try:
        allowed = os.sched_getaffinity(0)
        target = cpus & allowed
        if not target or target == allowed:
            return None
        os.sched_setaffinity(0, target)
        return target
    except (AttributeError, OSError):
        return None
