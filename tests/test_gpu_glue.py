"""Parity of the graph-glue kernels (channel concat, nearest resize, per-channel affine) against the
CPU oracle: copies are bit-exact, the affine map is exact in fp32 (one fma) and within fp16 rounding."""
import numpy as np
import pytest

from oracle import exb_oracle as O
from tests.util import dev, host, rng, f16_round

pytestmark = pytest.mark.gpu


def _capi():
    from excalibur_b200 import capi
    return capi


def _nhwc_padded(x_nchw, cs, dtype):
    n, c, h, w = x_nchw.shape
    out = np.zeros((n, h, w, cs), dtype)
    out[..., :c] = np.transpose(x_nchw, (0, 2, 3, 1)).astype(dtype)
    return out


@pytest.mark.parametrize("channels,strides,y_stride", [
    ((64, 64), (64, 64), 128),            # vector path
    ((32, 128, 128, 128), (32, 128, 128, 128), 416),
    ((3, 16, 21), (16, 16, 32), 64),      # ragged widths: element path, padded output
    ((8, 24), (16, 32), 32),
    ((5,), (8,), 16),
])
@pytest.mark.parametrize("dtype", [np.float16, np.int8])
def test_concat_nhwc(ctx, channels, strides, y_stride, dtype):
    capi = _capi()
    r = rng(sum(channels))
    N, H, W = 2, 5, 7
    xs = [r.integers(-100, 100, (N, c, H, W)).astype(np.float32) for c in channels]
    ref = O.concat_channels(xs)
    y = host(capi.concat_channels(ctx, [dev(_nhwc_padded(x, s, dtype)) for x, s in zip(xs, strides)],
                                  channels, y_stride))
    ctx.sync_check()
    assert y.shape == (N, H, W, y_stride)
    np.testing.assert_array_equal(y[..., :ref.shape[1]].astype(np.float32), O.nchw_to_nhwc(ref))
    assert not y[..., ref.shape[1]:].any()      # the wrapper's zero-filled pad is left alone


def test_concat_nchw_f32_and_empty(ctx):
    capi = _capi()
    r = rng(5)
    xs = [r.standard_normal((3, c, 4, 6)).astype(np.float32) for c in (3, 16, 21, 1)]
    y = host(capi.concat_nchw(ctx, [dev(x) for x in xs]))
    np.testing.assert_array_equal(y, O.concat_channels(xs))
    e = capi.concat_nchw(ctx, [dev(np.zeros((0, 4, 2, 2), np.float32)), dev(np.zeros((0, 1, 2, 2), np.float32))])
    assert tuple(e.shape) == (0, 5, 2, 2)
    ctx.sync_check()


def test_concat_rejects_too_many_inputs(ctx):
    capi = _capi()
    xs = [dev(np.zeros((1, 1, 1, 8), np.float16)) for _ in range(9)]
    with pytest.raises(capi.ExbError):
        capi.concat_channels(ctx, xs)


@pytest.mark.parametrize("shape,out_hw", [((2, 24, 6, 5), (12, 10)), ((2, 24, 6, 5), (7, 11)), ((1, 256, 20, 20), (40, 40)),
                                          ((1, 5, 3, 4), (3, 4)), ((2, 7, 8, 8), (4, 3))])
def test_interp_nearest(ctx, shape, out_hw):
    capi = _capi()
    x = rng(shape[1]).standard_normal(shape).astype(np.float32)
    ref = O.interp_nearest(x, *out_hw)
    y32 = host(capi.interp_nearest(ctx, dev(x), out_hw[0], out_hw[1], channel_last=False))
    np.testing.assert_array_equal(y32, ref)
    cs = (shape[1] + 7) // 8 * 8
    for cs_, dtype in ((cs, np.float16), (shape[1], np.float16), (cs, np.int8)):
        xi = x if dtype == np.float16 else np.clip(np.rint(x * 40), -128, 127)
        xh = _nhwc_padded(xi, cs_, dtype)
        y = host(capi.interp_nearest(ctx, dev(xh), out_hw[0], out_hw[1], channels=shape[1]))
        want = O.nchw_to_nhwc(O.interp_nearest(np.transpose(xh, (0, 3, 1, 2)).astype(np.float32), *out_hw))
        np.testing.assert_array_equal(y.astype(np.float32), want)
    ctx.sync_check()


@pytest.mark.parametrize("shape", [(2, 13, 6, 5), (1, 64, 28, 28), (3, 1, 1, 1)])
def test_channel_affine(ctx, shape):
    capi = _capi()
    r = rng(shape[1] + 100)
    x = r.standard_normal(shape).astype(np.float32)
    mul = r.uniform(0.5, 1.5, shape[1]).astype(np.float32)
    add = r.standard_normal(shape[1]).astype(np.float32)
    y = host(capi.channel_affine(ctx, dev(x), dev(mul), dev(add), channel_last=False))
    ref = O.channel_affine(x, mul, add)
    np.testing.assert_allclose(y, ref, rtol=2e-7, atol=3e-7)      # fma vs mul + add
    cs = (shape[1] + 15) // 16 * 16
    xh = _nhwc_padded(f16_round(x), cs, np.float16)
    xh[..., shape[1]:] = 7.0        # padding channels come out as zeros whatever they held
    yh = host(capi.channel_affine(ctx, dev(xh), dev(mul), dev(add), channels=shape[1]))
    ref16 = O.nchw_to_nhwc(O.channel_affine(f16_round(x), mul, add))
    np.testing.assert_allclose(yh[..., :shape[1]].astype(np.float32), ref16, rtol=1e-3, atol=1e-3)
    assert not yh[..., shape[1]:].any()
    # with a fused ReLU
    yr = host(capi.channel_affine(ctx, dev(x), dev(mul), dev(add), channel_last=False, act=capi.ACT_RELU))
    np.testing.assert_allclose(yr, np.maximum(ref, 0), rtol=2e-7, atol=3e-7)
    ctx.sync_check()


@pytest.mark.parametrize("alpha,beta", [(1.0 / 6.0, 0.5), (0.2, 0.5)])
def test_hardswish(ctx, alpha, beta):
    capi = _capi()
    x = (rng(9).standard_normal(100003) * 4).astype(np.float32)
    y = host(capi.hardswish(ctx, dev(x), alpha, beta))
    np.testing.assert_allclose(y, O.hardswish(x, alpha, beta), rtol=0, atol=5e-7)
    xh = f16_round(x)
    yh = host(capi.hardswish(ctx, dev(xh.astype(np.float16)), alpha, beta)).astype(np.float32)
    np.testing.assert_allclose(yh, O.hardswish(xh, alpha, beta), rtol=1e-3, atol=1e-3)
    if alpha != 0.2:    # the activation code used by fused convolutions
        ya = host(capi.activation(ctx, dev(x), capi.ACT_HARDSWISH))
        np.testing.assert_allclose(ya, O.hardswish(x), rtol=0, atol=5e-7)
    ctx.sync_check()


@pytest.mark.parametrize("shape", [(1, 3, 10, 12), (3, 3, 64, 48), (2, 5, 7, 9)])
def test_focus(ctx, shape):
    capi = _capi()
    x = rng(shape[2]).standard_normal(shape).astype(np.float32)
    ref = O.focus(x)
    np.testing.assert_array_equal(host(capi.focus(ctx, dev(x), channel_last=False)), ref)
    cs_in, cs_out = 8, (4 * shape[1] + 15) // 16 * 16
    xh = _nhwc_padded(f16_round(x), cs_in, np.float16)
    y = host(capi.focus(ctx, dev(xh), channels=shape[1], out_stride=cs_out))
    assert y.shape == (shape[0], shape[2] // 2, shape[3] // 2, cs_out)
    np.testing.assert_array_equal(y[..., :4 * shape[1]].astype(np.float32), O.nchw_to_nhwc(O.focus(f16_round(x))))
    assert not y[..., 4 * shape[1]:].any()
    ctx.sync_check()
