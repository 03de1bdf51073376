"""One batch over several replicas (glasssix::excalibur::sharded_pipeline): the host-side scatter / gather
arithmetic on the CPU, and the whole call on however many GPUs are visible against a single pipeline."""
import numpy as np
import pytest

from excalibur_b200 import models, sharding


def _host():
    from excalibur_b200 import host
    return host


def test_shard_bounds_of_the_host_layer_match_the_launcher_rule():
    h = _host()
    for total in (0, 1, 7, 32, 256, 257):
        for world in (1, 2, 3, 4, 8):
            for rank in range(world):
                assert h.shard_bounds(total, world, rank) == sharding.shard_bounds(total, world, rank)
    with pytest.raises(h.HostError):
        h.shard_bounds(10, 2, 2)


def test_scatter_by_offset_then_gather_is_the_identity():
    h = _host()
    r = np.random.default_rng(3)
    for total, world in ((7, 3), (8, 8), (5, 8), (32, 4)):
        x = r.standard_normal((total, 3, 5, 4)).astype(np.float32)
        parts = []
        for rank in range(world):
            lo, hi = h.shard_bounds(total, world, rank)
            parts.append(x[lo:hi] * 2.0)                      # stand-in for a replica's forward
        np.testing.assert_array_equal(h.gather_rows(parts), x * 2.0)


@pytest.mark.gpu
@pytest.mark.parametrize("batch", [8, 5, 1])
def test_sharded_forward_equals_one_pipeline(batch):
    """Replicas on every visible GPU (two replicas on the one GPU where there is only one): the gathered logits equal
    the single pipeline's, image for image - slices are independent, so bit for bit."""
    import torch
    h = _host()
    n_gpu = torch.cuda.device_count()
    devices = list(range(n_gpu)) if n_gpu > 1 else [0, 0]
    devices = devices + [devices[0]]                          # an odd replica count: ragged slices
    g, _ = models.resnet18(2)
    x = np.random.default_rng(41).uniform(0, 1, (batch, 3, 64, 64)).astype(np.float32)
    one = h.Pipeline(g.phai_text(), g.racy_bytes(), 0, fusion=True)
    ref = one.forward(x)["logits"]
    one.close()
    sp = h.ShardedPipeline(g.phai_text(), g.racy_bytes(), devices)
    for _ in range(3):                                        # eager, capture, replay on every replica
        out = sp.forward(x)["logits"]
    assert out.shape == ref.shape
    assert sp.device_ms() > 0
    sp.close()
    # a replica sees a smaller batch than the single pipeline: same kernels, other tile boundaries; the results of
    # an image do not depend on its neighbours
    np.testing.assert_array_equal(out, ref)
