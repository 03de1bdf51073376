"""Parity of the element-wise / quantise / layout kernels against the CPU oracle (bit-exact for
fp32 and integer results, fp16 within rounding of the fp32 result)."""
import numpy as np
import pytest

from oracle import exb_oracle as O
from tests.util import dev, host, rng, f16_round

pytestmark = pytest.mark.gpu

COUNTS = [0, 1, 7, 8, 33, 1000, 4096 + 5, 64 * 56 * 56, 3 * 1000 * 1000 + 3]


def _capi():
    from excalibur_b200 import capi
    return capi


@pytest.mark.parametrize("count", COUNTS)
@pytest.mark.parametrize("dtype", ["f32", "f16"])
def test_relu(ctx, count, dtype):
    capi = _capi()
    x = rng(count + 1).standard_normal(count).astype(np.float32)
    if dtype == "f16":
        x = f16_round(x)
        y = host(capi.relu(ctx, dev(x.astype(np.float16)))).astype(np.float32)
    else:
        y = host(capi.relu(ctx, dev(x)))
    ctx.sync_check()
    np.testing.assert_array_equal(y, O.relu_f32(x.reshape(1, 1, 1, -1)).reshape(-1))


@pytest.mark.parametrize("type_", [0, 1, 2])
@pytest.mark.parametrize("n_in", [2, 3, 5])
@pytest.mark.parametrize("dtype", ["f32", "f16"])
def test_eltwise(ctx, type_, n_in, dtype):
    capi = _capi()
    count = 64 * 28 * 28 + 3
    r = rng(type_ * 10 + n_in)
    xs = [r.standard_normal(count).astype(np.float32) for _ in range(n_in)]
    coeffs = r.uniform(0.5, 1.5, n_in).astype(np.float32) if type_ == 1 else None
    if dtype == "f16":
        xs = [f16_round(x) for x in xs]
        y = host(capi.eltwise(ctx, [dev(x.astype(np.float16)) for x in xs], type_, coeffs)).astype(np.float32)
    else:
        y = host(capi.eltwise(ctx, [dev(x) for x in xs], type_, coeffs))
    ctx.sync_check()
    ref = O.eltwise_f32(xs, type_, coeffs)
    if dtype == "f32" and type_ != 1:
        np.testing.assert_array_equal(y, ref)
    elif dtype == "f32":
        np.testing.assert_allclose(y, ref, rtol=1e-6, atol=1e-6)   # fused vs unfused multiply-add
    else:
        np.testing.assert_allclose(y, ref, rtol=2e-3, atol=1e-3)


@pytest.mark.parametrize("op", [0, 1, 2, 3])
@pytest.mark.parametrize("dtype", ["f32", "f16"])
def test_binaryop(ctx, op, dtype):
    capi = _capi()
    count = 128 * 14 * 14 + 1
    r = rng(op)
    a = r.standard_normal(count).astype(np.float32)
    b = (r.standard_normal(count).astype(np.float32) + 3.0)
    if dtype == "f16":
        a, b = f16_round(a), f16_round(b)
        y = host(capi.binaryop(ctx, dev(a.astype(np.float16)), dev(b.astype(np.float16)), op)).astype(np.float32)
        np.testing.assert_allclose(y, O.binaryop_f32(a, b, op), rtol=1e-3, atol=1e-4)
    else:
        y = host(capi.binaryop(ctx, dev(a), dev(b), op))
        if op == 3:
            np.testing.assert_allclose(y, O.binaryop_f32(a, b, op), rtol=1e-6)
        else:
            np.testing.assert_array_equal(y, O.binaryop_f32(a, b, op))
    ctx.sync_check()


def test_binaryop_scalar(ctx):
    capi = _capi()
    a = rng(5).standard_normal(1001).astype(np.float32)
    for op, f in enumerate([lambda v: v + 1.5, lambda v: v - 1.5, lambda v: v * 1.5, lambda v: v / 1.5]):
        y = host(capi.binaryop_scalar(ctx, dev(a), 1.5, op))
        np.testing.assert_allclose(y, f(a).astype(np.float32), rtol=1e-6)
    ctx.sync_check()


@pytest.mark.parametrize("act", [0, 1, 3, 4, 103, 104])
def test_activation(ctx, act):
    capi = _capi()
    x = (rng(act).standard_normal(5003) * 4).astype(np.float32)
    y = host(capi.activation(ctx, dev(x), act))
    ctx.sync_check()
    ref = O.activation(x, act)
    if act in (0, 1, 3, 103):
        np.testing.assert_array_equal(y, ref)
    else:
        np.testing.assert_allclose(y, ref, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("count", COUNTS)
@pytest.mark.parametrize("rounding", [0, 1])
def test_quantize_f32(ctx, count, rounding):
    capi = _capi()
    x = (rng(count + 3).standard_normal(count) * 2).astype(np.float32)
    if count > 16:
        x[:8] = [0.5 / 37.5, 1.5 / 37.5, 2.5 / 37.5, -0.5 / 37.5, -1.5 / 37.5, 1000, -1000, 0]
    scale = np.float32(37.5)
    q = host(capi.quantize(ctx, dev(x), scale, rounding))
    ctx.sync_check()
    if rounding == 0:
        ref = O.quantize_f32_i8(x.reshape(1, 1, 1, -1), [scale]).reshape(-1)
    else:
        ref = O.requantize_rne(x, scale)
    np.testing.assert_array_equal(q, ref)


def test_quantize_f16_and_dequantize(ctx):
    capi = _capi()
    x = f16_round(rng(9).standard_normal(100003) * 2)
    scale = np.float32(50.0)
    q = host(capi.quantize(ctx, dev(x.astype(np.float16)), scale, 0))
    np.testing.assert_array_equal(q, O.quantize_f32_i8(x.reshape(1, 1, 1, -1), [scale]).reshape(-1))
    qd = dev(q)
    y32 = host(capi.dequantize(ctx, qd, 1.0 / 50.0, capi.EXB_F32))
    np.testing.assert_array_equal(y32, q.astype(np.float32) * np.float32(1.0 / 50.0))
    y16 = host(capi.dequantize(ctx, qd, 1.0 / 50.0, capi.EXB_F16)).astype(np.float32)
    np.testing.assert_array_equal(y16, f16_round(q.astype(np.float32) * np.float32(1.0 / 50.0)))
    ctx.sync_check()


@pytest.mark.parametrize("shape", [(1, 3, 5, 7), (2, 64, 9, 9), (3, 33, 17, 4), (1, 3, 224, 224)])
def test_layout_roundtrip(ctx, shape):
    capi = _capi()
    N, Cc, H, W = shape
    x = rng(N * Cc).standard_normal(shape).astype(np.float32)
    cs = (Cc + 15) // 16 * 16
    xd = dev(x)
    # fp16 NHWC with channel padding
    y = capi.nchw_f32_to_nhwc(ctx, xd, capi.EXB_F16, c_stride=cs)
    yh = host(y).astype(np.float32)
    np.testing.assert_array_equal(yh[..., :Cc], f16_round(np.transpose(x, (0, 2, 3, 1))))
    assert not yh[..., Cc:].any()
    back = host(capi.nhwc_to_nchw_f32(ctx, y, Cc))
    np.testing.assert_array_equal(back, f16_round(x))
    # int8 NHWC, reference rounding
    s = np.float32(20.0)
    q = host(capi.nchw_f32_to_nhwc(ctx, xd, capi.EXB_I8, c_stride=cs, scale=s, rounding=0))
    np.testing.assert_array_equal(q[..., :Cc], np.transpose(O.quantize_f32_i8(x, [s]), (0, 2, 3, 1)))
    ctx.sync_check()


def test_bad_arguments_are_reported_not_fatal(ctx):
    capi = _capi()
    import torch
    x = torch.zeros(16, device="cuda", dtype=torch.int32)
    with pytest.raises(capi.ExbError) as e:
        capi.check(capi.lib().exb_relu_fwd(ctx.handle, capi.ptr(x), capi.ptr(x), 16, 7, None))
    assert e.value.code == capi.EXB_ERR_UNSUPPORTED
    with pytest.raises(capi.ExbError) as e:
        capi.check(capi.lib().exb_relu_fwd(ctx.handle, None, capi.ptr(x), 16, capi.EXB_F32, None))
    assert e.value.code == capi.EXB_ERR_BAD_ARG


def test_bounded_wait_gives_up_with_a_status_and_the_context_stays_usable(ctx):
    """The failure path of the kernels' device-side waits, exercised without a fault: a wait that can
    never be satisfied runs out after a bounded number of tries, the kernel returns, the next
    sync-check reports EXB_ERR_TIMEOUT once, and later launches on the same context are fine."""
    capi = _capi()
    ctx.sync_check()
    capi.check(capi.lib().exb_selftest_bounded_wait(ctx.handle, 64, capi.cur_stream()))
    with pytest.raises(capi.ExbError) as e:
        ctx.sync_check()
    assert e.value.code == -4 and "bounded wait" in str(e.value)
    ctx.sync_check()                                    # the error word was cleared
    x = rng(1).standard_normal(4096).astype(np.float32)
    np.testing.assert_array_equal(host(capi.relu(ctx, dev(x))), np.maximum(x, 0))
    ctx.sync_check()
    with pytest.raises(capi.ExbError):                  # the self-test itself is bounded
        capi.check(capi.lib().exb_selftest_bounded_wait(ctx.handle, 1 << 20, capi.cur_stream()))
