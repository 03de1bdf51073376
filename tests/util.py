"""Helpers shared by the parity tests: seeded data and NCHW/NHWC plumbing."""
import numpy as np


def rng(seed):
    return np.random.default_rng(seed)


def to_nhwc(a, c_stride=None):
    """NCHW numpy -> NHWC numpy, optionally zero-padding the channel dimension."""
    a = np.ascontiguousarray(np.transpose(a, (0, 2, 3, 1)))
    if c_stride and c_stride > a.shape[3]:
        pad = np.zeros(a.shape[:3] + (c_stride - a.shape[3],), a.dtype)
        a = np.concatenate([a, pad], axis=3)
    return np.ascontiguousarray(a)


def to_nchw(a, C=None):
    a = np.transpose(a, (0, 3, 1, 2))
    if C is not None:
        a = a[:, :C]
    return np.ascontiguousarray(a)


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.detach().cpu().numpy()


def f16_round(a):
    """Round fp32 data to fp16 and back, so the oracle sees exactly what the kernel sees."""
    return np.asarray(a, np.float32).astype(np.float16).astype(np.float32)


def assert_close_f16(y, ref, rel=1e-2, what=""):
    """fp16 parity bar: |y - ref| <= rel*|ref| + 1e-3*max|ref| (the 1e-2 relative tolerance
    against the fp32 reference, with an absolute floor for values that cancel to ~0)."""
    y = np.asarray(y, np.float32)
    ref = np.asarray(ref, np.float32)
    assert y.shape == ref.shape, (y.shape, ref.shape)
    tol = rel * np.abs(ref) + 1e-3 * max(float(np.abs(ref).max()), 1e-6)
    bad = np.abs(y - ref) > tol
    assert not bad.any(), "%s: %d of %d elements off, worst abs err %g" % (
        what, int(bad.sum()), bad.size, float(np.abs(y - ref).max()))


def quant_weights(w):
    """Symmetric per-output-channel int8 weights, reference convention ws = 127/max|w|."""
    cout = w.shape[0]
    ws = (127.0 / np.abs(w).reshape(cout, -1).max(axis=1)).astype(np.float32)
    wq = np.clip(np.rint(w * ws[:, None, None, None]), -127, 127).astype(np.int8)
    return wq, ws


# ---- benchmark-size fixtures (tests/golden/fullsize_vectors.npz) -----------------------------------
FULLSIZE_SEEDS = {"resnet_body": 56001, "resnet_body_calib": 56007, "resnet": 224001, "resnet_calib": 224007, "mobilenet": 224101, "mobilenet_calib": 224107, "yolo": 640001}


def fullsize_inputs(tag, n, size):
    """Seeded uniform[0,1] images of one benchmark configuration; the fixture stores only their checksum."""
    return np.random.default_rng(FULLSIZE_SEEDS[tag]).uniform(0, 1, (n, 3, size, size)).astype(np.float32)


def body_inputs(tag, n, channels=64, size=56):
    """Seeded stand-in for the map the first residual block reads (post-ReLU, post-pooling: non-negative, a few
    units large): |N(0, 1.5)| values, about half of them clipped to 0."""
    r = np.random.default_rng(FULLSIZE_SEEDS[tag])
    v = r.standard_normal((n, channels, size, size)).astype(np.float32) * np.float32(1.5) - np.float32(0.2)
    return np.maximum(v, 0).astype(np.float32)


def quantize_half_away(x, scale):
    """The reference's float32_to_int8 (src/Primitives/simd_types.cpp:140-152): x * scale, half away from zero,
    truncate, saturate to [-128, 127]."""
    t = np.asarray(x, np.float32) * np.float32(scale)
    t = np.where(t >= 0, t + np.float32(0.5), t - np.float32(0.5))
    return np.clip(t, -128, 127).astype(np.int32).astype(np.int8)


def sample(a, limit=8192):
    """Every k-th value of a flattened array, at most `limit` values (what a fixture keeps of a large map)."""
    flat = np.ascontiguousarray(a, np.float32).reshape(-1)
    step = max(1, -(-flat.size // limit))
    return flat[::step].copy()
