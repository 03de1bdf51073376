"""Multi-rank host logic on CPU: two gloo ranks shard a batch, run their slices independently (the
CPU oracle stands in for the GPU kernels) and the concatenation equals the unsharded result; the
timing reduction takes the slowest rank."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from excalibur_b200 import sharding


def test_shard_bounds_cover_exactly():
    for total in (0, 1, 7, 32, 256, 257):
        for world in (1, 2, 3, 4, 8):
            b = sharding.all_bounds(total, world)
            assert b[0][0] == 0 and b[-1][1] == total
            assert all(b[i][1] == b[i + 1][0] for i in range(world - 1))
            sizes = [hi - lo for lo, hi in b]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.shard_bounds(10, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import exb_oracle as O
    r = np.random.default_rng(5)          # same seed on every rank: identical full batch
    x = r.uniform(-1, 1, (6, 8, 9, 9)).astype(np.float32)
    w = (r.standard_normal((16, 8, 3, 3)) * 0.2).astype(np.float32)
    lo, hi = sharding.shard_bounds(x.shape[0], world, rank)
    y = O.pool2d_f32(O.conv2d_f32(x[lo:hi], w, None, 1, 1, act=1), 0, 3, 2, 1)   # this rank's slice only
    np.save(os.path.join(out_dir, "y%d.npy" % rank), y)
    slowest = sharding.max_over_ranks(10.0 + rank, dist)
    np.save(os.path.join(out_dir, "t%d.npy" % rank), np.array([slowest]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_shard_a_batch(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    from oracle import exb_oracle as O
    r = np.random.default_rng(5)
    x = r.uniform(-1, 1, (6, 8, 9, 9)).astype(np.float32)
    w = (r.standard_normal((16, 8, 3, 3)) * 0.2).astype(np.float32)
    full = O.pool2d_f32(O.conv2d_f32(x, w, None, 1, 1, act=1), 0, 3, 2, 1)
    got = np.concatenate([np.load(tmp_path / ("y%d.npy" % k)) for k in range(world)])
    np.testing.assert_array_equal(got, full)
    for k in range(world):
        assert np.load(tmp_path / ("t%d.npy" % k))[0] == 11.0     # the slowest rank's value everywhere
    assert sharding.aggregate_throughput(256, 2, 2.0) == 256000.0


def test_gpu_local_cpus_reads_sysfs(tmp_path):
    from excalibur_b200 import sharding
    d = tmp_path / "0000:1b:00.0"
    d.mkdir()
    (d / "local_cpulist").write_text("0-3,8,10-11\n")
    assert sharding.gpu_local_cpus("0000:1B:00.0", str(tmp_path)) == {0, 1, 2, 3, 8, 10, 11}
    assert sharding.gpu_local_cpus("0000:2c:00.0", str(tmp_path)) is None
    (d / "local_cpulist").write_text("\n")
    assert sharding.gpu_local_cpus("0000:1b:00.0", str(tmp_path)) is None
    assert sharding.bind_host_thread_to_gpu(0) is None or isinstance(sharding.bind_host_thread_to_gpu(0), set)
