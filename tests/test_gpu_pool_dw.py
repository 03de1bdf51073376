"""Parity of pooling and depthwise convolution against the CPU oracle."""
import numpy as np
import pytest

from oracle import exb_oracle as O
from tests.util import dev, host, rng, f16_round, to_nhwc, to_nchw

pytestmark = pytest.mark.gpu


def _capi():
    from excalibur_b200 import capi
    return capi


POOL_CASES = [
    # N, C, H, W, type, k, s, pad, pad_mode, cip
    (2, 64, 112, 112, 0, 3, 2, 1, 1, 0),     # ResNet stem pool
    (1, 256, 20, 20, 0, 5, 1, 2, 1, 0),      # SPPF pool
    (3, 16, 7, 9, 0, 2, 2, 0, 0, 0),         # ceil mode, ragged
    (2, 8, 13, 13, 1, 3, 2, 1, 1, 0),        # avg, exclude pad
    (2, 8, 13, 13, 1, 3, 2, 1, 1, 1),        # avg, include pad
    (1, 24, 10, 10, 1, 2, 2, 0, 0, 1),       # avg, ceil
    (1, 8, 5, 5, 1, 3, 1, 1, 0, 1),
]


@pytest.mark.parametrize("case", POOL_CASES)
@pytest.mark.parametrize("dtype", ["f16", "f32"])
def test_pool(ctx, case, dtype):
    capi = _capi()
    N, Cc, H, W, type_, k, s, pad, pad_mode, cip = case
    x = rng(sum(case)).standard_normal((N, Cc, H, W)).astype(np.float32)
    if dtype == "f16":
        x = f16_round(x)
    ref = O.pool2d_f32(x, type_, k, s, pad, False, pad_mode, cip)
    d = capi.make_pool_desc(N, H, W, Cc, type_, k, s, pad, False, pad_mode, cip,
                            capi.EXB_F16 if dtype == "f16" else capi.EXB_F32)
    xd = dev(to_nhwc(x).astype(np.float16 if dtype == "f16" else np.float32))
    y, _ = capi.pool2d(ctx, d, xd)
    ctx.sync_check()
    y = to_nchw(host(y).astype(np.float32))
    assert y.shape == ref.shape
    if type_ == 0:
        np.testing.assert_array_equal(y, ref)
    elif dtype == "f32":
        np.testing.assert_allclose(y, ref, rtol=1e-6, atol=1e-6)
    else:
        np.testing.assert_allclose(y, ref, rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("type_", [0, 1])
@pytest.mark.parametrize("shape", [(4, 512, 7, 7), (2, 1280, 7, 7), (1, 64, 56, 56), (3, 8, 1, 1)])
def test_global_pool(ctx, type_, shape):
    capi = _capi()
    N, Cc, H, W = shape
    x = f16_round(rng(N + Cc).standard_normal(shape))
    ref = O.pool2d_f32(x, type_, global_pool=True)
    d = capi.make_pool_desc(N, H, W, Cc, type_, global_pool=True, dtype=capi.EXB_F16)
    y, _ = capi.pool2d(ctx, d, dev(to_nhwc(x).astype(np.float16)))
    ctx.sync_check()
    y = to_nchw(host(y).astype(np.float32))
    assert y.shape == ref.shape == (N, Cc, 1, 1)
    if type_ == 0:
        np.testing.assert_array_equal(y, ref)
    else:
        np.testing.assert_allclose(y, ref, rtol=2e-3, atol=1e-3)


def test_pool_int8_and_second_output(ctx):
    capi = _capi()
    N, Cc, H, W = 2, 64, 30, 30
    r = rng(77)
    xq = r.integers(-128, 128, (N, Cc, H, W)).astype(np.int8)
    d = capi.make_pool_desc(N, H, W, Cc, 0, 3, 2, 1, dtype=capi.EXB_I8)
    y, _ = capi.pool2d(ctx, d, dev(to_nhwc(xq)))
    ref = O.pool2d_f32(xq.astype(np.float32), 0, 3, 2, 1)
    np.testing.assert_array_equal(to_nchw(host(y)).astype(np.float32), ref)
    # fp16 max pool that also emits the int8 tensor the next int8 conv consumes
    x = f16_round(np.abs(r.standard_normal((N, Cc, H, W))) * 3)
    s = np.float32(127.0 / x.max())
    d = capi.make_pool_desc(N, H, W, Cc, 0, 3, 2, 1, dtype=capi.EXB_F16, out2_dtype=capi.EXB_I8, out2_scale=s)
    y, y2 = capi.pool2d(ctx, d, dev(to_nhwc(x).astype(np.float16)))
    ctx.sync_check()
    ref = O.pool2d_f32(x, 0, 3, 2, 1)
    np.testing.assert_array_equal(to_nchw(host(y).astype(np.float32)), ref)
    np.testing.assert_array_equal(to_nchw(host(y2)), O.requantize_rne(ref, s))


DW_CASES = [
    # N, C, H, W, k, s, pad, bias, act
    (2, 32, 112, 112, 3, 1, 1, True, 103),
    (2, 96, 56, 56, 3, 2, 1, True, 103),
    (1, 144, 57, 31, 3, 1, 1, False, 1),
    (1, 144, 57, 31, 3, 2, 1, True, 0),
    (3, 8, 9, 9, 5, 1, 2, True, 0),
    (1, 16, 4, 4, 4, 1, 0, True, 0),
    (2, 24, 15, 15, 3, 2, 0, True, 104),
]


@pytest.mark.parametrize("case", DW_CASES)
def test_dwconv_f16(ctx, case):
    capi = _capi()
    N, Cc, H, W, k, s, pad, has_bias, act = case
    r = rng(sum(case[:7]))
    x = f16_round(r.standard_normal((N, Cc, H, W)))
    w = (r.standard_normal((Cc, 1, k, k)) * 0.3).astype(np.float32)
    b = (r.standard_normal(Cc) * 0.1).astype(np.float32) if has_bias else None
    ref = O.dwconv2d_f32(x, w, b, s, pad, act)
    d = capi.make_dw_desc(N, H, W, Cc, k, s, pad, act=act)
    wp = capi.DwWeights(ctx, d, w, b)
    y = capi.dwconv2d(ctx, d, dev(to_nhwc(x).astype(np.float16)), wp)
    ctx.sync_check()
    y = to_nchw(host(y).astype(np.float32))
    assert y.shape == ref.shape
    np.testing.assert_allclose(y, ref, rtol=2e-3, atol=2e-3)


def test_dwconv_int8_in_out(ctx):
    capi = _capi()
    N, Cc, H, W = 2, 64, 28, 28
    r = rng(123)
    xq = r.integers(-128, 128, (N, Cc, H, W)).astype(np.int8)
    in_scale = np.float32(1.0 / 31.0)
    w = (r.standard_normal((Cc, 1, 3, 3)) * 0.3).astype(np.float32)
    b = (r.standard_normal(Cc) * 0.1).astype(np.float32)
    v = O.dwconv2d_f32(xq.astype(np.float32) * in_scale, w, b, 1, 1, 103)
    out_scale = np.float32(127.0 / 6.0)
    ref = O.requantize_rne(v, out_scale).astype(np.int32)
    d = capi.make_dw_desc(N, H, W, Cc, 3, 1, 1, capi.EXB_I8, capi.EXB_I8, 103, in_scale, out_scale)
    wp = capi.DwWeights(ctx, d, w, b)
    y = to_nchw(host(capi.dwconv2d(ctx, d, dev(to_nhwc(xq)), wp))).astype(np.int32)
    ctx.sync_check()
    # fp32 summation order differs from the oracle's double accumulation: at most 1 LSB where the
    # pre-rounding value sits on a rounding boundary.
    assert np.abs(y - ref).max() <= 1
    assert (y != ref).mean() < 1e-3
