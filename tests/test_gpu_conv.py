"""Parity of the dense convolution (tcgen05 implicit GEMM and the direct kernel) against the CPU
oracle: int32 accumulators bit-exact, dequantised fp32 bit-exact, requantised int8 bit-exact
against the oracle's half-even rule and within 1 LSB of the reference's half-away rule, fp16
within 1e-2 relative of the fp32 result."""
import numpy as np
import pytest

from oracle import exb_oracle as O
from tests.util import dev, host, rng, f16_round, to_nhwc, to_nchw, assert_close_f16, quant_weights

pytestmark = pytest.mark.gpu


def _capi():
    from excalibur_b200 import capi
    return capi


def run_conv_i8(ctx, xq, wq, bias, ws, fs, stride, pad, out_dtype, act=0, impl=0, res=None, out_scale=1.0,
                out2_dtype=-1, out2_scale=1.0, group=1):
    capi = _capi()
    N, Cin, H, W = xq.shape
    Cout, _, kh, kw = wq.shape
    d = capi.make_conv_desc(N, H, W, Cin, Cout, (kh, kw), stride, pad, capi.EXB_I8, out_dtype, out2_dtype,
                            res is not None, act, out_scale, out2_scale, group=group, impl=impl)
    wp = capi.ConvWeights(ctx, d, wq, bias, ws, fs)
    resd = dev(to_nhwc(res).astype(np.float16)) if res is not None else None
    y, y2 = capi.conv2d(ctx, d, dev(to_nhwc(xq)), wp, resd)
    ctx.sync_check()
    return (to_nchw(host(y)), to_nchw(host(y2)) if y2 is not None else None,
            capi.lib().exb_conv2d_uses_tensor_cores(d))


I8_CASES = [
    # N, Cin, H, W, Cout, k, stride, pad
    (1, 64, 8, 8, 64, 3, 1, 1),
    (2, 64, 56, 56, 64, 3, 1, 1),       # ResNet stage 1
    (3, 64, 56, 56, 128, 3, 2, 1),      # stage 2 entry
    (3, 64, 56, 56, 128, 1, 2, 0),      # projection shortcut
    (2, 128, 28, 28, 128, 3, 1, 1),
    (5, 256, 14, 14, 256, 3, 1, 1),
    (20, 512, 7, 7, 512, 3, 1, 1),      # box spans 18 images + ragged tail
    (2, 32, 13, 11, 48, 3, 1, 1),       # odd sizes, 32-byte K blocks, Cout not multiple of 32
    (2, 96, 9, 9, 40, 1, 1, 0),         # 1x1, 32-byte K blocks, ragged Cout
    (1, 128, 15, 15, 64, 3, 2, 1),      # odd input, stride 2
    (1, 64, 12, 12, 320, 3, 1, 1),      # two Cout tiles
    (2, 64, 10, 10, 32, 5, 1, 2),       # 5x5
    (1, 32, 9, 9, 16, 3, 2, 0),         # stride 2 without padding
    (3, 256, 10, 13, 128, 3, 1, 1),     # row-box loop: two channel blocks per kernel row, weights streamed, ragged width
    (5, 128, 6, 5, 64, 3, 1, 1),        # row-box loop: map narrower than the 8-pixel tile, several images per tile
    (1, 192, 12, 12, 64, 2, 1, 0),      # row-box loop with two taps per row (2x2 kernel, no padding), three channel blocks
    (9, 128, 12, 12, 128, 3, 1, 1),     # row-box loop on CTA pairs (resident weights, halves per CTA), odd number of image groups
    (7, 256, 14, 14, 256, 3, 1, 1),     # tap loop on CTA pairs, odd number of image groups (last pair half empty)
]


@pytest.mark.parametrize("impl", [0, 1], ids=["tc", "direct"])
@pytest.mark.parametrize("case", I8_CASES)
def test_conv_i8_accumulators_bit_exact(ctx, case, impl):
    capi = _capi()
    N, Cin, H, W, Cout, k, stride, pad = case
    r = rng(sum(case))
    xq = r.integers(-128, 128, (N, Cin, H, W)).astype(np.int8)
    wq = r.integers(-127, 128, (Cout, Cin, k, k)).astype(np.int8)
    ref = O.conv2d_i8_acc(xq, wq, stride, pad)
    y, _, tc = run_conv_i8(ctx, xq, wq, None, np.ones(Cout, np.float32), 1.0, stride, pad, capi.EXB_I32, impl=impl)
    assert tc == (1 if impl == 0 else 0)
    assert y.shape == ref.shape
    np.testing.assert_array_equal(y, ref)


@pytest.mark.parametrize("case", I8_CASES[:6])
def test_conv_i8_dequant_and_requant(ctx, case):
    """The fused epilogue: fp32 result equals the reference formula acc*1/(ws*fs)+bias bit for bit;
    the int8 result equals the half-even requantisation of it, and is within 1 LSB of quantising
    with the reference's half-away rule."""
    capi = _capi()
    N, Cin, H, W, Cout, k, stride, pad = case
    r = rng(sum(case) + 1)
    x = r.uniform(-1, 1, (N, Cin, H, W)).astype(np.float32)
    w = (r.standard_normal((Cout, Cin, k, k)) * np.sqrt(2.0 / (Cin * k * k))).astype(np.float32)
    b = (r.standard_normal(Cout) * 0.01).astype(np.float32)
    wq, ws = quant_weights(w)
    fs = np.float32(127.0 / np.abs(x).max())
    xq = O.quantize_f32_i8(x, [fs])
    ref = O.conv2d_i8(x, wq, b, ws, fs, stride, pad, act=1)          # the reference's forward_cpu_i8
    y, _, _ = run_conv_i8(ctx, xq, wq, b, ws, fs, stride, pad, capi.EXB_F32, act=1)
    np.testing.assert_array_equal(y, ref)
    nxt = np.float32(127.0 / max(float(ref.max()), 1e-6))
    q, h16, _ = run_conv_i8(ctx, xq, wq, b, ws, fs, stride, pad, capi.EXB_I8, act=1, out_scale=nxt,
                            out2_dtype=capi.EXB_F16)
    np.testing.assert_array_equal(q, O.requantize_rne(ref, nxt))
    assert np.abs(q.astype(np.int32) - O.quantize_f32_i8(ref, [nxt]).astype(np.int32)).max() <= 1
    np.testing.assert_array_equal(h16.astype(np.float32), f16_round(ref))


def test_conv_i8_residual_relu_dual_output(ctx):
    """Second conv of a basic block: conv + skip (fp16) + ReLU, written as fp16 and as int8."""
    capi = _capi()
    N, Cc, H, W = 2, 64, 28, 28
    r = rng(4242)
    x = r.uniform(-1, 1, (N, Cc, H, W)).astype(np.float32)
    w = (r.standard_normal((Cc, Cc, 3, 3)) * np.sqrt(2.0 / (Cc * 9))).astype(np.float32)
    b = (r.standard_normal(Cc) * 0.01).astype(np.float32)
    skip = f16_round(r.uniform(-1, 1, (N, Cc, H, W)))
    wq, ws = quant_weights(w)
    fs = np.float32(127.0 / np.abs(x).max())
    xq = O.quantize_f32_i8(x, [fs])
    v = O.activation(O.conv2d_i8(x, wq, b, ws, fs, 1, 1, act=0) + skip, 1)
    nxt = np.float32(127.0 / v.max())
    y16, q, _ = run_conv_i8(ctx, xq, wq, b, ws, fs, 1, 1, capi.EXB_F16, act=1, res=skip,
                            out2_dtype=capi.EXB_I8, out2_scale=nxt)
    np.testing.assert_array_equal(y16.astype(np.float32), f16_round(v))
    np.testing.assert_array_equal(q, O.requantize_rne(v, nxt))


F16_CASES = [
    (1, 64, 56, 56, 64, 3, 1, 1),       # the single-layer benchmark configuration's shape
    (2, 16, 37, 41, 64, 7, 2, 3),       # stem-like (3 channels padded to 16)
    (2, 64, 28, 28, 128, 3, 2, 1),
    (2, 128, 14, 14, 256, 1, 1, 0),
    (4, 512, 7, 7, 512, 3, 1, 1),
    (1, 32, 40, 40, 255, 1, 1, 0),      # detect head width
    (2, 16, 30, 30, 32, 6, 2, 2),       # 6x6/2 stem
    (2, 32, 21, 19, 32, 3, 1, 1),       # row-box loop on 64-byte K rows, ragged map
    (2, 64, 11, 9, 64, 3, 1, 1),        # row-box loop, weights streamed with two CTAs per SM (73 KB slice)
    (1, 128, 12, 12, 64, 5, 1, 2),      # row-box loop with five taps per row, two channel blocks
    (9, 64, 12, 12, 128, 3, 1, 1),      # row-box loop on CTA pairs, fp16
    (3, 128, 14, 14, 256, 3, 2, 1),     # stride-2 tap loop on CTA pairs, fp16
]


@pytest.mark.parametrize("impl", [0, 1], ids=["tc", "direct"])
@pytest.mark.parametrize("case", F16_CASES)
def test_conv_f16(ctx, case, impl):
    capi = _capi()
    N, Cin, H, W, Cout, k, stride, pad = case
    r = rng(sum(case) + 7)
    x = f16_round(r.uniform(-1, 1, (N, Cin, H, W)))
    w = f16_round(r.standard_normal((Cout, Cin, k, k)) * np.sqrt(2.0 / (Cin * k * k)))
    b = (r.standard_normal(Cout) * 0.01).astype(np.float32)
    ref = O.conv2d_f32(x, w, b, stride, pad, act=1)
    d = capi.make_conv_desc(N, H, W, Cin, Cout, k, stride, pad, capi.EXB_F16, capi.EXB_F32, act=1, impl=impl)
    wp = capi.ConvWeights(ctx, d, w, b)
    y, _ = capi.conv2d(ctx, d, dev(to_nhwc(x).astype(np.float16)), wp)
    ctx.sync_check()
    assert capi.lib().exb_conv2d_uses_tensor_cores(d) == (1 if impl == 0 else 0)
    y = to_nchw(host(y))
    # fp32 accumulation of exactly representable products: only the summation order differs
    np.testing.assert_allclose(y, ref, rtol=1e-4, atol=1e-4)
    d16 = capi.make_conv_desc(N, H, W, Cin, Cout, k, stride, pad, capi.EXB_F16, capi.EXB_F16, act=1, impl=impl)
    y16, _ = capi.conv2d(ctx, d16, dev(to_nhwc(x).astype(np.float16)), wp)
    ctx.sync_check()
    assert_close_f16(to_nchw(host(y16).astype(np.float32)), ref, what="fp16 conv")


def test_conv_f16_config1_against_unrounded_fp32(ctx):
    """The single-layer benchmark configuration: fp32 data, fp16 kernel, 1e-2 relative of the fp32 result."""
    capi = _capi()
    r = rng(1000)
    x = r.uniform(-1, 1, (1, 64, 56, 56)).astype(np.float32)
    w = (r.standard_normal((64, 64, 3, 3)) * np.sqrt(2.0 / 576)).astype(np.float32)
    b = (r.standard_normal(64) * 0.01).astype(np.float32)
    ref = O.conv2d_f32(x, w, b, 1, 1, act=1)
    d = capi.make_conv_desc(1, 56, 56, 64, 64, 3, 1, 1, capi.EXB_F16, capi.EXB_F16, act=1)
    wp = capi.ConvWeights(ctx, d, w, b)
    xh = capi.nchw_f32_to_nhwc(ctx, dev(x), capi.EXB_F16)
    y, _ = capi.conv2d(ctx, d, xh, wp)
    out = host(capi.nhwc_to_nchw_f32(ctx, y))
    ctx.sync_check()
    assert_close_f16(out, ref, what="config 1")


def test_conv_silu_and_padded_channels(ctx):
    capi = _capi()
    N, Cin, H, W, Cout = 2, 24, 20, 20, 40
    cin_s, cout_s = 32, 48
    r = rng(31)
    x = f16_round(r.uniform(-1, 1, (N, Cin, H, W)))
    w = f16_round(r.standard_normal((Cout, Cin, 3, 3)) * 0.1)
    b = (r.standard_normal(Cout) * 0.1).astype(np.float32)
    ref = O.conv2d_f32(x, w, b, 1, 1, act=O.ACT_SILU)
    d = capi.make_conv_desc(N, H, W, Cin, Cout, 3, 1, 1, capi.EXB_F16, capi.EXB_F16, act=capi.ACT_SILU,
                            cin_stride=cin_s, cout_stride=cout_s)
    wp = capi.ConvWeights(ctx, d, w, b)
    y, _ = capi.conv2d(ctx, d, dev(to_nhwc(x, cin_s).astype(np.float16)), wp)
    ctx.sync_check()
    yh = host(y).astype(np.float32)
    assert not yh[..., Cout:].any(), "padding channels must be written as zero"
    assert_close_f16(to_nchw(yh, Cout), ref, what="silu")


def test_conv_grouped_direct(ctx):
    capi = _capi()
    N, Cin, H, W, Cout, g = 2, 16, 9, 9, 24, 4
    r = rng(8)
    x = f16_round(r.uniform(-1, 1, (N, Cin, H, W)))
    w = f16_round(r.standard_normal((Cout, Cin // g, 3, 3)) * 0.2)
    ref = O.conv2d_f32(x, w, None, 1, 1, group=g)
    d = capi.make_conv_desc(N, H, W, Cin, Cout, 3, 1, 1, capi.EXB_F16, capi.EXB_F32, group=g)
    assert capi.lib().exb_conv2d_uses_tensor_cores(d) == 0
    wp = capi.ConvWeights(ctx, d, w, None)
    y, _ = capi.conv2d(ctx, d, dev(to_nhwc(x).astype(np.float16)), wp)
    ctx.sync_check()
    np.testing.assert_allclose(to_nchw(host(y)), ref, rtol=1e-4, atol=1e-4)


def test_conv_full_size_tc_equals_direct(ctx):
    """Batch-256 stage-1 layer: the tensor-core kernel against the direct kernel on the device, bit for bit over the
    whole batch, and two images of that same launch against the CPU oracle."""
    capi = _capi()
    import torch
    N, Cc, H, W = 256, 64, 56, 56
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randint(-128, 128, (N, H, W, Cc), generator=g, device="cuda", dtype=torch.int32).to(torch.int8)
    r = rng(55)
    wq = r.integers(-127, 128, (Cc, Cc, 3, 3)).astype(np.int8)
    outs = []
    for impl in (0, 1):
        d = capi.make_conv_desc(N, H, W, Cc, Cc, 3, 1, 1, capi.EXB_I8, capi.EXB_I32, impl=impl)
        wp = capi.ConvWeights(ctx, d, wq, None, np.ones(Cc, np.float32), 1.0)
        y, _ = capi.conv2d(ctx, d, x, wp)
        ctx.sync_check()
        outs.append(y)
    assert torch.equal(outs[0], outs[1])
    # two images of the same launch (the first and the last) against the CPU oracle's accumulators
    for n in (0, N - 1):
        xn = to_nchw(host(x[n:n + 1]))
        ref = O.conv2d_i8_acc(xn, wq, 1, 1)
        np.testing.assert_array_equal(to_nchw(host(outs[0][n:n + 1])), ref)
    # linearity: conv(2x) == 2*conv(x) on the accumulators
    d = capi.make_conv_desc(N, H, W, Cc, Cc, 3, 1, 1, capi.EXB_I8, capi.EXB_I32)
    wp = capi.ConvWeights(ctx, d, wq, None, np.ones(Cc, np.float32), 1.0)
    xh = (x.to(torch.int32) // 2).to(torch.int8)
    y1, _ = capi.conv2d(ctx, d, xh, wp)
    y2, _ = capi.conv2d(ctx, d, (xh.to(torch.int32) * 2).to(torch.int8), wp)
    ctx.sync_check()
    assert torch.equal(y1 * 2, y2)


def test_conv_empty_batch_and_errors(ctx):
    capi = _capi()
    d = capi.make_conv_desc(0, 8, 8, 64, 64, 3, 1, 1, capi.EXB_I8, capi.EXB_I32)
    wq = np.zeros((64, 64, 3, 3), np.int8)
    wp = capi.ConvWeights(ctx, d, wq, None, np.ones(64, np.float32), 1.0)
    assert capi.lib().exb_conv2d_fwd(ctx.handle, d, None, wp.handle, None, None, None, None) == 0
    bad = capi.make_conv_desc(1, 2, 2, 64, 64, 3, 1, 0, capi.EXB_I8, capi.EXB_I32)   # window > input
    assert capi.lib().exb_conv2d_fwd(ctx.handle, bad, None, wp.handle, None, None, None, None) == capi.EXB_ERR_BAD_ARG
    assert "window" in capi.last_error()


STEM_CASES = [
    # N, H, W, Cout, k, stride, pad, w_pad
    (2, 64, 64, 64, 7, 2, 3, 4),      # ResNet stem
    (3, 37, 41, 32, 3, 2, 1, 4),      # MobileNet stem, odd sizes
    (2, 48, 40, 32, 6, 2, 2, 4),      # YOLOv5 stem
    (1, 224, 224, 64, 7, 2, 3, 4),
]


@pytest.mark.parametrize("impl", [0, 1], ids=["tc", "direct"])
@pytest.mark.parametrize("case", STEM_CASES)
def test_stem_conv_folded_rows(ctx, case, impl):
    """3-channel stem: fp32 NCHW image -> padded NHWC4 fp16 rows -> conv with kw taps folded into K."""
    capi = _capi()
    N, H, W, Cout, k, stride, pad, w_pad = case
    r = rng(sum(case))
    x = r.uniform(0, 1, (N, 3, H, W)).astype(np.float32)
    w = f16_round(r.standard_normal((Cout, 3, k, k)) * np.sqrt(2.0 / (3 * k * k)))
    b = (r.standard_normal(Cout) * 0.01).astype(np.float32)
    ref = O.conv2d_f32(f16_round(x), w, b, stride, pad, act=1)
    w_pitch = (W + w_pad + 8 + 7) // 8 * 8
    xp = capi.nchw_f32_to_nhwc_padded(ctx, dev(x), capi.EXB_F16, 4, w_pad, w_pitch)
    xh = host(xp).astype(np.float32)
    np.testing.assert_array_equal(xh[:, :, w_pad:w_pad + W, :3], f16_round(np.transpose(x, (0, 2, 3, 1))))
    assert not xh[:, :, :w_pad].any() and not xh[:, :, w_pad + W:].any() and not xh[..., 3].any()
    d = capi.make_conv_desc(N, H, W, 3, Cout, k, stride, pad, capi.EXB_F16, capi.EXB_F32, act=1, cin_stride=4,
                            impl=impl, x_w_pitch=w_pitch, x_w_pad=w_pad)
    assert capi.lib().exb_conv2d_uses_tensor_cores(d) == (1 if impl == 0 else 0)
    wp = capi.ConvWeights(ctx, d, w, b)
    y, _ = capi.conv2d(ctx, d, xp, wp)
    ctx.sync_check()
    np.testing.assert_allclose(to_nchw(host(y)), ref, rtol=1e-4, atol=1e-4)


POOL_STEM_CASES = [
    # N, H, W, k, pad
    (2, 64, 64, 7, 3),
    (3, 37, 41, 7, 3),      # odd conv output (19 x 21) -> pooled 10 x 11, ragged last tiles
    (2, 48, 40, 6, 2),      # YOLO-style 6x6/2 stem
    (1, 224, 224, 7, 3),
    (2, 30, 26, 5, 2),
]


@pytest.mark.parametrize("case", POOL_STEM_CASES)
@pytest.mark.parametrize("with_i8", [False, True], ids=["f16", "f16+i8"])
def test_stem_conv_with_fused_max_pool(ctx, case, with_i8):
    """Stem conv + ReLU + 3x3/2 pad-1 max pooling in one kernel equals conv -> fp16 -> pool of the
    oracle (bit-exact given the conv's fp16 result: max of rounded values, then the int8 copy)."""
    capi = _capi()
    N, H, W, k, pad = case
    r = rng(sum(case) + 7)
    x = r.uniform(0, 1, (N, 3, H, W)).astype(np.float32)
    w = f16_round(r.standard_normal((64, 3, k, k)) * np.sqrt(2.0 / (3 * k * k)))
    b = (r.standard_normal(64) * 0.1).astype(np.float32)
    w_pad = 4
    w_pitch = (W + w_pad + 8 + 7) // 8 * 8
    xp = capi.nchw_f32_to_nhwc_padded(ctx, dev(x), capi.EXB_F16, 4, w_pad, w_pitch)
    q = 25.0
    kw = dict(act=1, cin_stride=4, x_w_pitch=w_pitch, x_w_pad=w_pad)
    d0 = capi.make_conv_desc(N, H, W, 3, 64, k, 2, pad, capi.EXB_F16, capi.EXB_F16, **kw)
    d1 = capi.make_conv_desc(N, H, W, 3, 64, k, 2, pad, capi.EXB_F16, capi.EXB_F16,
                             capi.EXB_I8 if with_i8 else -1, out2_scale=q, fuse_pool=1, **kw)
    assert capi.lib().exb_conv2d_pool_fusable(d0) == 1
    wp = capi.ConvWeights(ctx, d0, w, b)
    y0, _ = capi.conv2d(ctx, d0, xp, wp)                     # the plain kernel's fp16 conv output
    y1, y2 = capi.conv2d(ctx, d1, xp, wp)
    ctx.sync_check()
    conv16 = to_nchw(host(y0).astype(np.float32))
    ref_conv = O.conv2d_f32(f16_round(x), w, b, 2, pad, act=1)
    np.testing.assert_allclose(conv16, ref_conv, rtol=2e-3, atol=2e-3)
    ref_pool = O.pool2d_f32(conv16, 0, 3, 2, 1)
    got = to_nchw(host(y1).astype(np.float32))
    assert got.shape == ref_pool.shape
    np.testing.assert_array_equal(got, ref_pool)
    if with_i8:
        np.testing.assert_array_equal(to_nchw(host(y2).astype(np.float32)), O.requantize_rne(ref_pool, q))


def test_fused_max_pool_is_refused_where_it_cannot_run(ctx):
    capi = _capi()
    d = capi.make_conv_desc(1, 16, 16, 32, 64, 3, 1, 1, capi.EXB_I8, capi.EXB_F16, act=1)
    assert capi.lib().exb_conv2d_pool_fusable(d) == 0
    d.fuse_pool = 1
    w = capi.ConvWeights(ctx, d, np.zeros((64, 32, 3, 3), np.int8), np.zeros(64, np.float32), np.ones(64, np.float32), 1.0)
    x = dev(np.zeros((1, 16, 16, 32), np.int8))
    with pytest.raises(capi.ExbError):
        capi.conv2d(ctx, d, x, w)


RES_DUAL_CASES = [
    # N, Cin, H, W, Cout, k, stride, pad
    (2, 64, 56, 56, 64, 3, 1, 1),       # two CTAs per SM, one 64-channel block
    (3, 128, 28, 28, 128, 3, 1, 1),     # two blocks
    (5, 256, 14, 14, 256, 3, 1, 1),     # one CTA per SM, the two halves of a lane quarter on two warps
    (20, 512, 7, 7, 512, 3, 1, 1),      # two Cout tiles of 256, 7x1x18 boxes with a ragged tail
    (3, 64, 56, 56, 128, 1, 2, 0),      # projection shortcut (fp16 output only)
    (2, 32, 13, 11, 48, 3, 1, 1),       # ragged tiles, 48 channels: the thread-per-pixel epilogue
    (1, 64, 12, 12, 320, 3, 1, 1),      # two Cout tiles of 160 channels: thread-per-pixel epilogue
    (2, 64, 9, 7, 192, 3, 1, 1),        # three blocks, tiles ragged in both directions
]


@pytest.mark.parametrize("case", RES_DUAL_CASES)
def test_conv_i8_residual_dual_output_shapes(ctx, case):
    """conv + fp16 skip + ReLU written as fp16 and int8 (the second convolution of a residual block) on every tile /
    channel-block configuration of the tensor-core kernel's two epilogues, against the CPU oracle, bit for bit."""
    capi = _capi()
    N, Cin, H, W, Cout, k, stride, pad = case
    r = rng(sum(case) + 11)
    x = r.uniform(-1, 1, (N, Cin, H, W)).astype(np.float32)
    w = (r.standard_normal((Cout, Cin, k, k)) * np.sqrt(2.0 / (Cin * k * k))).astype(np.float32)
    b = (r.standard_normal(Cout) * 0.01).astype(np.float32)
    wq, ws = quant_weights(w)
    fs = np.float32(127.0 / np.abs(x).max())
    xq = O.quantize_f32_i8(x, [fs])
    pre = O.conv2d_i8(x, wq, b, ws, fs, stride, pad, act=0)
    with_res = k == 3
    skip = f16_round(r.uniform(-1, 1, pre.shape)) if with_res else None
    v = O.activation(pre + skip, 1) if with_res else pre
    nxt = np.float32(127.0 / max(float(np.abs(v).max()), 1e-6))
    if with_res:
        y16, q, tc = run_conv_i8(ctx, xq, wq, b, ws, fs, stride, pad, capi.EXB_F16, act=1, res=skip,
                                 out2_dtype=capi.EXB_I8, out2_scale=nxt)
        np.testing.assert_array_equal(q, O.requantize_rne(v, nxt))
    else:
        y16, _, tc = run_conv_i8(ctx, xq, wq, b, ws, fs, stride, pad, capi.EXB_F16)
    assert tc == 1
    np.testing.assert_array_equal(y16.astype(np.float32), f16_round(v))
    # int8 first, fp16 second (the order the first convolution of the next block's producer uses)
    q2, h2, _ = run_conv_i8(ctx, xq, wq, b, ws, fs, stride, pad, capi.EXB_I8, act=1 if with_res else 0, res=skip,
                            out_scale=nxt, out2_dtype=capi.EXB_F16)
    np.testing.assert_array_equal(q2, O.requantize_rne(v, nxt))
    np.testing.assert_array_equal(h2.astype(np.float32), f16_round(v))
