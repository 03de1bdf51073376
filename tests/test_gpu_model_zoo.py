"""PReLU / LeakyRelu / Deconvolution / Reshape / Transpose kernels and host operations, and the three
networks with the architecture of the reference's shipped descriptions, against outputs of the
reference CPU library (golden vectors) and the CPU oracle."""
import os

import numpy as np
import pytest

from excalibur_b200 import model_zoo
from excalibur_b200.modelfile import GraphBuilder
from oracle import exb_oracle as O
from tests.util import f16_round

pytestmark = pytest.mark.gpu
S = np.load(os.path.join(os.path.dirname(__file__), "golden", "shipped_model_vectors.npz"))


def _host():
    from excalibur_b200 import host
    return host


def _rel(a, b):
    return float(np.abs(a.astype(np.float64) - b).max() / max(np.abs(b).max(), 1e-12))


def _params(g, line=0):
    return g.lines[line].split(" ", 6)[6]


# ---- kernels through the C ABI ----------------------------------------------------------------------
@pytest.mark.parametrize("C,cs", [(13, 16), (64, 64), (5, 5), (40, 48)])
def test_prelu_kernel_nhwc_f16(C, cs):
    import torch
    from excalibur_b200 import capi
    ctx = capi.Context(0)
    r = np.random.default_rng(C)
    x = f16_round(r.standard_normal((2, C, 9, 7)).astype(np.float32) * 3)
    sl = r.uniform(0.01, 0.9, C).astype(np.float32)
    xh = torch.full((2, 9, 7, cs), 7.0, dtype=torch.float16, device="cuda")      # garbage in the padding channels
    xh[..., :C] = torch.from_numpy(O.nchw_to_nhwc(x)).cuda().half()
    for slopes in (sl, sl[:1]):
        y = capi.prelu(ctx, xh, torch.from_numpy(slopes).cuda(), channels=C)
        torch.cuda.synchronize()
        got = O.nhwc_to_nchw(y[..., :C].float().cpu().numpy())
        np.testing.assert_array_equal(got, f16_round(O.prelu(x, slopes)))
        assert float(y[..., C:].abs().sum()) == 0.0
    ctx.close()


def test_prelu_kernel_nchw_f32_and_refusals():
    import torch
    from excalibur_b200 import capi
    ctx = capi.Context(0)
    x = S["act_x"]
    xd = torch.from_numpy(x).cuda()
    y = capi.prelu(ctx, xd, torch.from_numpy(S["prelu_slopes"]).cuda(), channel_last=False)
    np.testing.assert_array_equal(y.cpu().numpy(), S["prelu_out"])
    empty = torch.empty((0, 13, 5, 7), device="cuda")
    assert capi.prelu(ctx, empty, torch.from_numpy(S["prelu_slopes"]).cuda(), channel_last=False).numel() == 0
    with pytest.raises(capi.ExbError):
        capi.prelu(ctx, xd, torch.zeros(4, device="cuda"), channel_last=False)       # 4 slopes, 13 channels
    ctx.close()


@pytest.mark.parametrize("dtype", ["f16", "f32"])
def test_depth_to_space_kernel(dtype):
    import torch
    from excalibur_b200 import capi
    ctx = capi.Context(0)
    r = np.random.default_rng(3)
    N, H, W, rh, rw, C, xs, ys = 2, 5, 6, 2, 3, 7, 48, 8
    x = r.standard_normal((N, H, W, xs)).astype(np.float32)
    td = torch.float16 if dtype == "f16" else torch.float32
    xd = torch.from_numpy(x).cuda().to(td)
    y = capi.depth_to_space(ctx, xd, rh, rw, C, y_stride=ys)
    torch.cuda.synchronize()
    src = xd.float().cpu().numpy()
    want = np.zeros((N, H * rh, W * rw, ys), np.float32)
    for a in range(rh):
        for b in range(rw):
            want[:, a::rh, b::rw, :C] = src[..., (a * rw + b) * C:(a * rw + b + 1) * C]
    np.testing.assert_array_equal(y.float().cpu().numpy(), want)
    ctx.close()


@pytest.mark.parametrize("shape", [(3, 5, 33, 70), (1, 1, 1, 1), (2, 3, 64, 32), (0, 4, 5, 6)])
def test_transpose_kernel(shape):
    import torch
    from excalibur_b200 import capi
    ctx = capi.Context(0)
    x = np.random.default_rng(4).standard_normal(shape).astype(np.float32)
    y = capi.transpose_hw(ctx, torch.from_numpy(x).cuda())
    np.testing.assert_array_equal(y.cpu().numpy(), O.transpose_hw(x))
    ctx.close()


# ---- host operations created through the reflector ----------------------------------------------------
def test_operation_prelu_leakyrelu():
    h = _host()
    x = S["act_x"]
    g = GraphBuilder(); g.prelu("p", "in", "out", S["prelu_slopes"])
    np.testing.assert_array_equal(h.run_op("PReLU", _params(g), [x], g.racy_bytes()), S["prelu_out"])
    g = GraphBuilder(); g.prelu("p", "in", "out", S["prelu_slopes"][:1])
    np.testing.assert_array_equal(h.run_op("PReLU", _params(g), [x], g.racy_bytes()), S["prelu_shared_out"])
    np.testing.assert_array_equal(h.run_op("LeakyRelu", "0=0.1", [x]), S["leaky_out"])
    with pytest.raises(h.HostError):
        h.run_op("LeakyRelu", "7=1", [x])


@pytest.mark.parametrize("tag", ["deconv_k2s2", "deconv_k2s2_c1"])
def test_operation_deconvolution(tag):
    h = _host()
    k, s, p = (int(v) for v in S[tag + "_cfg"])
    g = GraphBuilder(); g.deconv("d", "in", "out", S[tag + "_w"], S[tag + "_b"], s, p)
    y = h.run_op("Deconvolution", _params(g), [S["act_x"]], g.racy_bytes())
    assert y.shape == S[tag + "_out"].shape
    # fp16 operands, fp32 accumulation: exact against the oracle on fp16-rounded operands, 1e-2 against fp32
    want = O.deconv2d_f32(f16_round(S["act_x"]), f16_round(S[tag + "_w"]), S[tag + "_b"], s, p)
    np.testing.assert_allclose(y, want, rtol=0, atol=1e-5)
    assert _rel(y, S[tag + "_out"]) < 1e-2


def test_operation_deconvolution_refuses_overlapping_taps():
    h = _host()
    g = GraphBuilder(); g.deconv("d", "in", "out", S["deconv_k3s2p1_w"], S["deconv_k3s2p1_b"], 2, 1)
    with pytest.raises(h.HostError):
        h.run_op("Deconvolution", _params(g), [S["act_x"]], g.racy_bytes())


def test_operation_reshape_transpose():
    h = _host()
    m = h.run_op("Reshape", "0=20 1=4 2=3", [S["rt_x"]])
    assert m.shape == (2, 3, 4, 20)
    np.testing.assert_array_equal(h.run_op("Transpose", "0=1,0,2", [m]), S["rt_out"])
    np.testing.assert_array_equal(h.run_op("Transpose", "0=0,1,2", [m]), m)
    with pytest.raises(h.HostError):
        h.run_op("Transpose", "0=2,0,1", [m])


# ---- the three networks -------------------------------------------------------------------------------
def _run_net(builder, tag, fusion, tol, inner=(), **kw):
    h = _host()
    g, info = builder(**kw)
    p = h.Pipeline(g.phai_text(), g.racy_bytes(), 0, fusion=fusion)
    x = S[tag + "_x"]
    for _ in range(3):     # eager, capture, replay
        out = p.forward(x)
    assert sorted(out) == sorted(info["outputs"])
    for n in info["outputs"]:
        ref = S["%s_out_%s" % (tag, n)]
        assert out[n].shape == ref.shape, (n, out[n].shape, ref.shape)
        assert np.isfinite(out[n]).all()
        r = _rel(out[n], ref)
        assert r < tol, (n, r)
    if not fusion:
        for n in inner:
            assert _rel(p.get(n), S["%s_map_%s" % (tag, n)]) < tol, n
    stats = p.stats()
    p.close()
    return stats


@pytest.mark.parametrize("fusion", [True, False], ids=["fused", "op_by_op"])
def test_det_db_resnet18(fusion):
    launches, _ = _run_net(model_zoo.det_db_resnet18, "detdb", fusion, 1e-2, ("s2_b2_act", "fuse_out", "head_relu_out"))
    if fusion:
        # 32 convolutions (ReLU / add + ReLU folded), 2 transposed convolutions of 2 launches (BatchNorm + ReLU
        # folded), Input, ingest, 4 poolings, 3 FPN adds not adjacent to their conv, 6 resizes, concat, sigmoid, emit
        assert launches <= 32 + 4 + 2 + 4 + 3 + 6 + 1 + 1 + 1 + 4, launches


@pytest.mark.parametrize("fusion", [True, False], ids=["fused", "op_by_op"])
def test_mobile_unicorn(fusion):
    _run_net(model_zoo.mobile_unicorn, "unicorn", fusion, 2e-2, ("conv2_4_res", "conv5_ex_act"))


@pytest.mark.parametrize("fusion", [True, False], ids=["fused", "op_by_op"])
def test_yolov5s_simp(fusion):
    _run_net(model_zoo.yolov5s_simp, "yolosimp", fusion, 2e-2, ("csp2_cv4_act", "spp_cat_out"), size=128)


def test_yolov5s_simp_batch_is_computed_for_every_image():
    """The reference's Focus only fills image 0; here every image of a batch gives what it gives alone."""
    h = _host()
    g, info = model_zoo.yolov5s_simp(size=128)
    p = h.Pipeline(g.phai_text(), g.racy_bytes(), 0, fusion=True)
    x1 = S["yolosimp_x"]
    x = np.concatenate([x1, x1[:, :, ::-1].copy(), x1], axis=0)
    out = p.forward(x)
    for n in info["outputs"]:
        ref = S["yolosimp_out_" + n]
        assert out[n].shape == (3,) + ref.shape[1:]
        assert _rel(out[n][0:1], ref) < 2e-2
        np.testing.assert_array_equal(out[n][2], out[n][0])
    p.close()


# ---- PReLU in convolution epilogues, fused passes -----------------------------------------------------
@pytest.mark.parametrize("case", [
    # N, Cin, H, W, Cout, k, stride, cin_stride, cout_stride, int8
    (2, 64, 20, 20, 64, 3, 1, 64, 64, False),     # two CTAs per SM variant
    (2, 24, 9, 11, 40, 1, 1, 32, 48, False),      # padded channels, ragged Cout
    (1, 512, 7, 7, 512, 3, 1, 512, 512, False),   # one CTA per SM variant
    (2, 64, 12, 12, 128, 3, 2, 64, 128, True),    # int8 operands
    (2, 16, 9, 9, 24, 3, 1, 16, 24, False),       # ragged output stride: element-wise epilogue
])
def test_conv_prelu_epilogue(case):
    import torch
    from excalibur_b200 import capi
    from tests.util import dev, host, to_nhwc, to_nchw, assert_close_f16, quant_weights
    ctx = capi.Context(0)
    N, Cin, H, W, Cout, k, s, cin_s, cout_s, int8 = case
    r = np.random.default_rng(sum(case[:7]))
    pad = k // 2
    sl = r.uniform(0.05, 0.9, Cout).astype(np.float32)
    b = (r.standard_normal(Cout) * 0.1).astype(np.float32)
    if int8:
        xq = r.integers(-128, 128, (N, Cin, H, W)).astype(np.int8)
        w = (r.standard_normal((Cout, Cin, k, k)) * 0.05).astype(np.float32)
        wq, ws = quant_weights(w)
        fs = np.float32(31.0)
        acc = O.conv2d_i8_acc(xq, wq, s, pad)
        ref = O.prelu(O.dequantize(acc, O.dequant_scales(ws, fs, Cout), b), sl)
        d = capi.make_conv_desc(N, H, W, Cin, Cout, k, s, pad, capi.EXB_I8, capi.EXB_F32, act=capi.ACT_PRELU,
                                cin_stride=cin_s, cout_stride=cout_s)
        wp = capi.ConvWeights(ctx, d, wq, b, ws, fs)
        xin = dev(to_nhwc(xq, cin_s))
    else:
        x = f16_round(r.uniform(-1, 1, (N, Cin, H, W)))
        w = f16_round(r.standard_normal((Cout, Cin, k, k)) * 0.1)
        ref = O.prelu(O.conv2d_f32(x, w, b, s, pad), sl)
        d = capi.make_conv_desc(N, H, W, Cin, Cout, k, s, pad, capi.EXB_F16, capi.EXB_F16, act=capi.ACT_PRELU,
                                cin_stride=cin_s, cout_stride=cout_s)
        wp = capi.ConvWeights(ctx, d, w, b)
        xin = dev(to_nhwc(x, cin_s).astype(np.float16))
    with pytest.raises(capi.ExbError):
        capi.conv2d(ctx, d, xin, wp)                  # no slopes attached yet
    wp.set_slopes(ctx, sl)
    y, _ = capi.conv2d(ctx, d, xin, wp)
    ctx.sync_check()
    yh = host(y).astype(np.float32)
    assert not yh[..., Cout:].any(), "padding channels must be written as zero"
    if int8:
        np.testing.assert_allclose(to_nchw(yh, Cout), ref, rtol=1e-6, atol=1e-6)
    else:
        assert_close_f16(to_nchw(yh, Cout), ref, what="prelu")
    wp.set_slopes(ctx, sl[:1])                         # one shared slope (LeakyRelu)
    y, _ = capi.conv2d(ctx, d, xin, wp)
    ctx.sync_check()
    ref1 = np.where(ref >= 0, ref, 0) + np.where(ref < 0, ref, 0) / sl[None, :, None, None] * sl[0]
    np.testing.assert_allclose(to_nchw(host(y).astype(np.float32), Cout), ref1, rtol=2e-2, atol=2e-2)
    with pytest.raises(capi.ExbError):
        wp.set_slopes(ctx, sl[:3])
    wp.close()
    ctx.close()


@pytest.mark.parametrize("k,s,C", [(3, 1, 64), (3, 2, 40), (5, 1, 16)])
def test_dwconv_prelu_epilogue(k, s, C):
    from excalibur_b200 import capi
    from tests.util import dev, host, to_nhwc, to_nchw
    ctx = capi.Context(0)
    r = np.random.default_rng(k * 100 + C)
    x = f16_round(r.standard_normal((2, C, 15, 17)))
    w = (r.standard_normal((C, 1, k, k)) * 0.3).astype(np.float32)
    b = (r.standard_normal(C) * 0.1).astype(np.float32)
    sl = r.uniform(0.05, 0.9, C).astype(np.float32)
    ref = O.prelu(O.dwconv2d_f32(x, w, b, s, k // 2, 0), sl)
    d = capi.make_dw_desc(2, 15, 17, C, k, s, k // 2, act=capi.ACT_PRELU)
    wp = capi.DwWeights(ctx, d, w, b)
    with pytest.raises(capi.ExbError):
        capi.dwconv2d(ctx, d, dev(to_nhwc(x).astype(np.float16)), wp)
    wp.set_slopes(ctx, sl)
    y = to_nchw(host(capi.dwconv2d(ctx, d, dev(to_nhwc(x).astype(np.float16)), wp)).astype(np.float32))
    ctx.sync_check()
    np.testing.assert_allclose(y, ref, rtol=2e-3, atol=2e-3)
    wp.close()
    ctx.close()


@pytest.mark.parametrize("C,cs", [(13, 16), (64, 64), (5, 5)])
def test_channel_affine_prelu_kernel(C, cs):
    import torch
    from excalibur_b200 import capi
    ctx = capi.Context(0)
    r = np.random.default_rng(C + 1)
    x = f16_round(r.standard_normal((2, C, 6, 5)).astype(np.float32) * 2)
    mul, add = r.uniform(0.5, 1.5, C).astype(np.float32), r.standard_normal(C).astype(np.float32)
    sl = r.uniform(0.01, 0.9, C).astype(np.float32)
    xh = torch.full((2, 6, 5, cs), 3.0, dtype=torch.float16, device="cuda")
    xh[..., :C] = torch.from_numpy(O.nchw_to_nhwc(x)).cuda().half()
    y = capi.channel_affine_prelu(ctx, xh, torch.from_numpy(mul).cuda(), torch.from_numpy(add).cuda(),
                                  torch.from_numpy(sl).cuda(), channels=C)
    torch.cuda.synchronize()
    want = O.prelu(O.channel_affine(x, mul, add), sl)
    got = O.nhwc_to_nchw(y[..., :C].float().cpu().numpy())
    np.testing.assert_allclose(got, want, rtol=2e-3, atol=2e-3)
    assert float(y[..., C:].abs().sum()) == 0.0
    # the plain affine map takes the same vector kernel
    y = capi.channel_affine(ctx, xh, torch.from_numpy(mul).cuda(), torch.from_numpy(add).cuda(), channels=C, act=capi.ACT_RELU)
    got = O.nhwc_to_nchw(y[..., :C].float().cpu().numpy())
    np.testing.assert_allclose(got, np.maximum(O.channel_affine(x, mul, add), 0), rtol=2e-3, atol=2e-3)
    assert float(y[..., C:].abs().sum()) == 0.0
    ctx.close()


@pytest.mark.parametrize("norm", [False, True])
def test_focus_ingest_kernel(norm):
    import torch
    from excalibur_b200 import capi
    ctx = capi.Context(0)
    r = np.random.default_rng(9)
    x = r.uniform(0, 255, (3, 3, 10, 12)).astype(np.float32)
    means, scales = np.array([10.0, 20.0, 30.0], np.float32), np.array([0.01, 0.02, 0.03], np.float32)
    mul = torch.from_numpy(scales).cuda() if norm else None
    add = torch.from_numpy(-means * scales).cuda() if norm else None
    y = capi.focus_ingest(ctx, torch.from_numpy(x).cuda(), 16, mul, add)
    torch.cuda.synchronize()
    src = O.channel_affine(x, scales, -means * scales) if norm else x
    want = O.focus(src)
    got = O.nhwc_to_nchw(y[..., :12].float().cpu().numpy())
    np.testing.assert_allclose(got, want, rtol=1e-3, atol=1e-3 if norm else 0.07)      # fp16 rounding of values up to 255
    assert float(y[..., 12:].abs().sum()) == 0.0
    with pytest.raises(capi.ExbError):
        capi.focus_ingest(ctx, torch.zeros((1, 3, 9, 12), device="cuda"))
    ctx.close()


def test_depth_to_space_kernel_whole_vectors():
    import torch
    from excalibur_b200 import capi
    ctx = capi.Context(0)
    N, H, W, r_, C = 2, 4, 5, 2, 16
    x = np.random.default_rng(5).standard_normal((N, H, W, r_ * r_ * C)).astype(np.float16)
    y = capi.depth_to_space(ctx, torch.from_numpy(x).cuda(), r_, r_, C)
    torch.cuda.synchronize()
    want = np.zeros((N, H * r_, W * r_, C), np.float16)
    for a in range(r_):
        for b in range(r_):
            want[:, a::r_, b::r_] = x[..., (a * r_ + b) * C:(a * r_ + b + 1) * C]
    np.testing.assert_array_equal(y.cpu().numpy(), want)
    ctx.close()


def test_fused_plans_of_the_three_networks_are_short():
    """PReLU / LeakyRelu / BatchNorm fold into their producers and the Focus layer into the ingest kernel."""
    h = _host()
    g, _ = model_zoo.mobile_unicorn()
    p = h.Pipeline(g.phai_text(), g.racy_bytes(), 0, fusion=True)
    p.forward(S["unicorn_x"])
    launches, _ = p.stats()
    p.close()
    # 32 convolutions + 17 depthwise convolutions (every PReLU and residual add folded), Input, ingest, FC
    assert launches <= 32 + 17 + 3, launches
    g, _ = model_zoo.yolov5s_simp(size=128)
    p = h.Pipeline(g.phai_text(), g.racy_bytes(), 0, fusion=True)
    p.forward(S["yolosimp_x"])
    launches, _ = p.stats()
    p.close()
    # 70 convolutions, 8 BatchNorm + LeakyRelu passes, 13 concats, 3 poolings, 2 resizes, 7 adds at most,
    # one ingest + focus kernel, 3 x (emit + transpose)
    assert launches <= 70 + 8 + 13 + 3 + 2 + 7 + 1 + 6, launches


# ---- the shipped int8 description ------------------------------------------------------------------------
@pytest.mark.parametrize("fusion", [True, False], ids=["fused", "op_by_op"])
def test_unicorn_light_fp(fusion):
    h = _host()
    g, _ = model_zoo.unicorn_light()
    p = h.Pipeline(g.phai_text(), g.racy_bytes(), 0, fusion=fusion)
    for _ in range(3):
        out = p.forward(S["ulight_x"])["conv5_dw"]
    assert out.shape == S["ulight_fp_out"].shape
    assert _rel(out, S["ulight_fp_out"]) < 1e-2, _rel(out, S["ulight_fp_out"])
    p.close()


@pytest.mark.parametrize("fusion", [True, False], ids=["fused", "op_by_op"])
def test_unicorn_light_int8(fusion):
    """Every dense convolution int8 (the first one, on the 3-channel image, included), scales from the
    reference's own calibration pass: within 3e-2 of the reference's int8 embedding and no further from
    the fp32 embedding than 1.5 x the reference's own quantisation error (rms; 2 x for the largest deviation)."""
    h = _host()
    scales = {str(n): np.float32(v) for n, v in zip(S["ulight_scale_names"], S["ulight_scales"])}
    g, _ = model_zoo.unicorn_light(act_scales=scales)
    p = h.Pipeline(g.phai_text(), g.racy_bytes(), 0, fusion=fusion)
    for _ in range(3):
        out = p.forward(S["ulight_x"])["conv5_dw"]
    ref8, ref32 = S["ulight_i8_out"], S["ulight_fp_out"]
    assert out.shape == ref8.shape
    assert _rel(out, ref8) < 3e-2, _rel(out, ref8)
    rms = lambda a, b: float(np.sqrt(np.mean((a.astype(np.float64) - b) ** 2)) / np.sqrt(np.mean(b.astype(np.float64) ** 2)))
    print("int8 embedding: rms distance to fp32 %.4g (reference %.4g), max %.4g (reference %.4g)"
          % (rms(out, ref32), rms(ref8, ref32), _rel(out, ref32), _rel(ref8, ref32)))
    assert rms(out, ref32) < 1.5 * rms(ref8, ref32), (rms(out, ref32), rms(ref8, ref32))
    assert _rel(out, ref32) < 2.0 * _rel(ref8, ref32), (_rel(out, ref32), _rel(ref8, ref32))
    if not fusion:
        # op by op the int8 convolutions reproduce the reference's arithmetic: first residual sum within fp32 noise
        m = p.get("res2_2")
        assert _rel(m, S["ulight_i8_map_res2_2"]) < 1e-5, _rel(m, S["ulight_i8_map_res2_2"])
    p.close()
    # a batch: every image is computed (the reference's packed int8 path only computes image 0)
    p = h.Pipeline(g.phai_text(), g.racy_bytes(), 0, fusion=True)
    x = np.concatenate([S["ulight_x"], S["ulight_x"][:, ::-1].copy(), S["ulight_x"]], axis=0)
    out3 = p.forward(x)["conv5_dw"]
    np.testing.assert_array_equal(out3[2], out3[0])
    assert _rel(out3[0:1], ref8) < 3e-2
    assert np.abs(out3[1] - out3[0]).max() > 0
    p.close()


def test_operation_hardsigmoid_softmax_flatten_broadcast_binaryop():
    h = _host()
    x = S["misc_x"]
    np.testing.assert_allclose(h.run_op("HardSigmoid", "0=0.2 1=0.5", [x]), S["hardsigmoid_out"], rtol=0, atol=1e-6)
    np.testing.assert_allclose(h.run_op("Softmax", "0=0 1=1", [x]), S["softmax_out"], rtol=0, atol=1e-6)
    np.testing.assert_array_equal(h.run_op("Flatten", "", [x]), S["flatten_out"])
    np.testing.assert_array_equal(h.run_op("Flatten", "0=0", [x]), S["flatten0_out"])
    gate = h.run_op("Pooling", "0=1 1=1 2=1 3=0 4=1", [x])
    assert gate.shape == (2, 7, 1, 1)
    np.testing.assert_allclose(h.run_op("BinaryOp", "0=2", [x, gate]), S["bcast_mul_out"], rtol=0, atol=1e-6)
    np.testing.assert_allclose(h.run_op("BinaryOp", "0=1", [gate, x]), S["bcast_sub_out"], rtol=0, atol=1e-6)
    np.testing.assert_allclose(h.run_op("BinaryOp", "0=1", [x, gate]), -S["bcast_sub_out"], rtol=0, atol=1e-6)
    with pytest.raises(h.HostError):
        h.run_op("BinaryOp", "0=0", [x, x[:, :, :1]])          # other broadcast shapes are refused
    with pytest.raises(h.HostError):
        h.run_op("Softmax", "0=0 1=1 7=3", [x])


@pytest.mark.parametrize("A,K,cs,hw", [(3, 85, 256, (5, 7)), (3, 8, 32, (9, 4)), (1, 16, 16, (3, 3))])
def test_split_heads_kernel(A, K, cs, hw):
    import torch
    from excalibur_b200 import capi
    ctx = capi.Context(0)
    H, W = hw
    x = np.random.default_rng(A * K).standard_normal((2, H, W, cs)).astype(np.float16)
    y = capi.split_heads(ctx, torch.from_numpy(x).cuda(), A, K)
    torch.cuda.synchronize()
    nchw = O.nhwc_to_nchw(x[..., :A * K].astype(np.float32))
    want = O.transpose_hw(O.reshape_nchw(nchw, w=H * W, h=K, c=A))
    np.testing.assert_array_equal(y.cpu().numpy(), want)
    with pytest.raises(capi.ExbError):
        capi.split_heads(ctx, torch.from_numpy(x).cuda(), A + 1, cs)      # more channels than the tensor has
    ctx.close()


@pytest.mark.parametrize("C,cs,gate_batch", [(64, 64, 3), (13, 16, 3), (40, 48, 1), (5, 5, 3)])
def test_channel_gate_kernel_nhwc_f16(C, cs, gate_batch):
    import torch
    from excalibur_b200 import capi
    ctx = capi.Context(0)
    r = np.random.default_rng(C)
    a = f16_round(r.standard_normal((3, 6, 5, cs)).astype(np.float32))
    g = f16_round(r.uniform(0.5, 1.5, (gate_batch, 1, 1, cs)).astype(np.float32))
    ad, gd = torch.from_numpy(a).cuda().half(), torch.from_numpy(g).cuda().half()
    for op, fn in ((2, lambda x, y: x * y), (1, lambda x, y: x - y), (3, lambda x, y: x / y)):
        for first in (False, True):
            y = capi.binaryop_channel_bcast(ctx, ad, gd, op, first, channels=C).float().cpu().numpy()
            want = fn(g, a) if first else fn(a, g)
            np.testing.assert_allclose(y[..., :C], f16_round(want[..., :C].astype(np.float32)), rtol=1e-3, atol=1e-3)
            assert not y[..., C:].any()
    ctx.close()


@pytest.mark.parametrize("C", [1, 3, 4])
def test_image_ingest_with_normalisation(C):
    import torch
    from excalibur_b200 import capi
    ctx = capi.Context(0)
    r = np.random.default_rng(C)
    x = r.uniform(0, 255, (2, C, 9, 11)).astype(np.float32)
    mul, add = r.uniform(0.005, 0.02, C).astype(np.float32), r.uniform(-2, 0, C).astype(np.float32)
    xd, md, ad = torch.from_numpy(x).cuda(), torch.from_numpy(mul).cuda(), torch.from_numpy(add).cuda()
    norm = capi.channel_affine(ctx, xd, md, ad, channel_last=False)                  # the stand-alone pass
    # fp16, with and without normalisation: equal to normalise + generic ingest, bit for bit
    for cs in (8, 16):
        got = capi.image_ingest(ctx, xd, capi.EXB_F16, cs, md, ad)
        want = capi.nchw_f32_to_nhwc(ctx, norm, capi.EXB_F16, cs)
        assert torch.equal(got, want)
        assert torch.equal(capi.image_ingest(ctx, xd, capi.EXB_F16, cs), capi.nchw_f32_to_nhwc(ctx, xd, capi.EXB_F16, cs))
    # int8 with the quantiser's scale, half-to-even
    for cs in (16, 32):
        got = capi.image_ingest(ctx, xd, capi.EXB_I8, cs, md, ad, scale=37.0, rounding=1)
        want = capi.nchw_f32_to_nhwc(ctx, norm, capi.EXB_I8, cs, 37.0, 1)
        assert torch.equal(got, want)
    with pytest.raises(capi.ExbError):
        capi.image_ingest(ctx, torch.zeros((1, 5, 4, 4), device="cuda"), capi.EXB_F16, 16)
    if C <= 3:
        x4 = r.uniform(0, 255, (2, C, 6, 12)).astype(np.float32)
        x4d = torch.from_numpy(x4).cuda()
        got = capi.padded_ingest_norm(ctx, x4d, md, ad, 4, 24)
        want = capi.nchw_f32_to_nhwc_padded(ctx, capi.channel_affine(ctx, x4d, md, ad, channel_last=False), capi.EXB_F16, 4, 4, 24)
        assert torch.equal(got, want)
    ctx.close()


@pytest.mark.parametrize("int8", [False, True], ids=["fp16", "int8"])
def test_conv_writes_a_channel_slice_of_a_wider_tensor(int8):
    """y_pitch: two convolutions store their channels side by side in one tensor (a Concat without a copy)."""
    import torch
    from excalibur_b200 import capi
    from tests.util import dev, host, to_nhwc, to_nchw, assert_close_f16, quant_weights
    ctx = capi.Context(0)
    r = np.random.default_rng(5)
    N, Cin, H, W, pitch = 2, 32, 11, 9, 96
    outs, refs = [], []
    ybuf = torch.full((N, H, W, pitch), 9.0, dtype=torch.float16, device="cuda")
    off = 0
    for Cout, k in ((32, 3), (48, 1)):
        b = (r.standard_normal(Cout) * 0.1).astype(np.float32)
        if int8:
            xq = r.integers(-128, 128, (N, Cin, H, W)).astype(np.int8)
            wq, ws = quant_weights((r.standard_normal((Cout, Cin, k, k)) * 0.05).astype(np.float32))
            fs = np.float32(25.0)
            ref = O.dequantize(O.conv2d_i8_acc(xq, wq, 1, k // 2), O.dequant_scales(ws, fs, Cout), b)
            d = capi.make_conv_desc(N, H, W, Cin, Cout, k, 1, k // 2, capi.EXB_I8, capi.EXB_F16, cout_stride=Cout, y_pitch=pitch)
            wp = capi.ConvWeights(ctx, d, wq, b, ws, fs)
            xin = dev(to_nhwc(xq))
        else:
            x = f16_round(r.uniform(-1, 1, (N, Cin, H, W)))
            w = f16_round(r.standard_normal((Cout, Cin, k, k)) * 0.1)
            ref = O.conv2d_f32(x, w, b, 1, k // 2)
            d = capi.make_conv_desc(N, H, W, Cin, Cout, k, 1, k // 2, capi.EXB_F16, capi.EXB_F16, cout_stride=Cout, y_pitch=pitch)
            wp = capi.ConvWeights(ctx, d, w, b)
            xin = dev(to_nhwc(x).astype(np.float16))
        capi.conv2d(ctx, d, xin, wp, y=ybuf[..., off:])
        ctx.sync_check()
        refs.append((off, Cout, ref))
        off += Cout
    yh = ybuf.float().cpu().numpy()
    for o, c, ref in refs:
        assert_close_f16(to_nchw(yh[..., o:o + c], c), ref, what="slice at %d" % o)
    assert (yh[..., off:] == 9.0).all(), "channels beyond the slices must be left alone"
    bad = capi.make_conv_desc(N, H, W, Cin, 32, 3, 1, 1, capi.EXB_F16, capi.EXB_F16, res=True, cout_stride=32, y_pitch=pitch)
    with pytest.raises(capi.ExbError):
        capi.conv2d(ctx, bad, xin, capi.ConvWeights(ctx, bad, np.zeros((32, Cin, 3, 3), np.float32), None), ybuf, y=ybuf)
    ctx.close()


def test_concat_of_convolutions_is_written_by_their_epilogues():
    """BottleneckCSP tail conv, conv -> Concat -> BatchNorm -> LeakyRelu: two launches, not five."""
    h = _host()
    r = np.random.default_rng(2)
    g = GraphBuilder()
    g.split("s", "in", ["a", "b"])
    w1 = (r.standard_normal((32, 16, 1, 1)) * 0.2).astype(np.float32)
    w2 = (r.standard_normal((48, 16, 3, 3)) * 0.1).astype(np.float32)
    g.conv("c1", "a", "y1", w1, None, 1, 0)
    g.conv("c2", "b", "y2", w2, None, 1, 1)
    g.concat("cat", ["y1", "y2"], "c")
    bn = [r.uniform(0.5, 1.5, 80), r.standard_normal(80) * 0.1, r.uniform(0.5, 1.5, 80), r.standard_normal(80) * 0.1]
    bn = [v.astype(np.float32) for v in bn]
    g.batchnorm("bn", "c", "n", *bn, eps=1e-5)
    g.leakyrelu("act", "n", "out", 0.1)
    x = f16_round(r.uniform(-1, 1, (2, 16, 9, 10)).astype(np.float32))
    cat = np.concatenate([O.conv2d_f32(x, f16_round(w1), None, 1, 0), O.conv2d_f32(x, f16_round(w2), None, 1, 1)], axis=1)
    mul, add = O.batchnorm_coeffs(*bn, eps=1e-5)
    want = O.leakyrelu(O.channel_affine(cat, mul, add), 0.1)
    for fusion in (True, False):
        p = h.Pipeline(g.phai_text(), g.racy_bytes(), 0, fusion=fusion)
        out = p.forward(x)["out"]
        assert _rel(out, want) < 1e-2, (fusion, _rel(out, want))
        if fusion:
            launches, _ = p.stats()
            assert launches == 4, launches          # ingest, two convolutions, emit
        p.close()
