"""The C++ host layer (operation classes created through the reflector, pipeline<float>) against
the reference's own outputs (golden vectors) and the CPU oracle."""
import os

import numpy as np
import pytest

from excalibur_b200 import models
from excalibur_b200.modelfile import GraphBuilder
from oracle import exb_oracle as O
from tests.util import assert_close_f16, f16_round

pytestmark = pytest.mark.gpu
G = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.npz"))


def _host():
    from excalibur_b200 import host
    return host


def _conv_line_and_blob(w, b, stride, pad, act, int8=None, dw=False):
    g = GraphBuilder()
    if dw:
        g.dwconv("c", "in", "out", w, b, stride, pad, act=act)
    else:
        g.conv("c", "in", "out", w, b, stride, pad, act=act, int8=int8)
    params = g.lines[0].split(" ", 6)[6]
    return params, g.racy_bytes()


@pytest.mark.parametrize("tag", ["conv_i8_wino", "conv_i8_im2col_s2", "conv_i8_im2col_wide", "conv_i8_1x1_s2"])
def test_operation_convolution_int8_matches_reference_bit_for_bit(tag):
    """operation_convolution::forward_gpu_i8 on fp32 NCHW tensors == the reference's forward_cpu_i8."""
    stride, pad, act = [int(v) for v in G[tag + "_cfg"]]
    params, blob = _conv_line_and_blob(G[tag + "_w"], G[tag + "_b"], stride, pad, act,
                                       int8=(G[tag + "_wq"], G[tag + "_ws"], G[tag + "_fs"]))
    y = _host().run_op("Convolution", params, [G[tag + "_x"]], blob)
    np.testing.assert_array_equal(y, G[tag + "_y"])


def test_operation_convolution_int8_batch_is_computed_for_every_image():
    """The reference's packed int8 path only computes image 0 of a batch; this one computes all."""
    tag = "conv_i8_im2col_wide"
    stride, pad, act = [int(v) for v in G[tag + "_cfg"]]
    x = np.concatenate([G[tag + "_x"], G[tag + "_x"][:, ::-1].copy(), G[tag + "_x"] * 0.5])
    params, blob = _conv_line_and_blob(G[tag + "_w"], G[tag + "_b"], stride, pad, act,
                                       int8=(G[tag + "_wq"], G[tag + "_ws"], G[tag + "_fs"]))
    y = _host().run_op("Convolution", params, [x], blob)
    ref = O.conv2d_i8(x, G[tag + "_wq"], G[tag + "_b"], G[tag + "_ws"], G[tag + "_fs"], stride, pad, act=act)
    np.testing.assert_array_equal(y, ref)
    np.testing.assert_array_equal(y[:1], G[tag + "_y"])


@pytest.mark.parametrize("tag", ["conv_f32_wino", "conv_f32_im2col_s2", "conv_f32_stem", "conv_f32_1x1"])
def test_operation_convolution_fp16_compute_within_1e2_of_reference_fp32(tag):
    stride, pad, act = [int(v) for v in G[tag + "_cfg"]]
    params, blob = _conv_line_and_blob(G[tag + "_w"], G[tag + "_b"], stride, pad, act)
    y = _host().run_op("Convolution", params, [G[tag + "_x"]], blob)
    assert_close_f16(y, G[tag + "_y"], what=tag)


@pytest.mark.parametrize("tag,stride", [("dw_s1", 1), ("dw_s2", 2)])
def test_operation_convolutiondepthwise(tag, stride):
    params, blob = _conv_line_and_blob(G[tag + "_w"], G[tag + "_b"], stride, 1, 1, dw=True)
    y = _host().run_op("ConvolutionDepthWise", params, [G[tag + "_x"]], blob)
    assert_close_f16(y, G[tag + "_y"], what=tag)


@pytest.mark.parametrize("tag,params", [
    ("pool_max_3s2p1", "0=0 1=3 2=2 3=1"), ("pool_max_5s1p2", "0=0 1=5 2=1 3=2"),
    ("pool_max_ceil", "0=0 1=2 2=2 3=0 5=0"), ("pool_avg_excl", "0=1 1=3 2=2 3=1 6=0"),
    ("pool_avg_incl", "0=1 1=3 2=2 3=1 6=1"), ("pool_gap", "0=1 4=1"),
])
def test_operation_pooling(tag, params):
    y = _host().run_op("Pooling", params, [G["pool_x"]])
    assert y.shape == G[tag + "_y"].shape
    if params.startswith("0=0"):
        np.testing.assert_array_equal(y, G[tag + "_y"])
    else:
        np.testing.assert_allclose(y, G[tag + "_y"], rtol=1e-6, atol=1e-6)


def test_operation_eltwise_binaryop_relu():
    h = _host()
    x = G["elt_x"]
    np.testing.assert_array_equal(h.run_op("ReLU", "", [x]), G["elt_ra"])
    np.testing.assert_array_equal(h.run_op("BinaryOp", "0=2", [x, x]), G["elt_bb"])
    np.testing.assert_allclose(h.run_op("Eltwise", "0=1 -23301=3,0.5,-1.25", [G["elt_ra"], G["elt_bb"], x]),
                               G["elt_esum"], rtol=1e-6, atol=1e-6)
    np.testing.assert_array_equal(h.run_op("Eltwise", "0=0", [G["elt_ra"], G["elt_bb"]]), G["elt_eprod"])
    np.testing.assert_array_equal(h.run_op("Eltwise", "0=2", [G["elt_ra"], G["elt_bb"], x]), G["elt_emax"])
    np.testing.assert_array_equal(h.run_op("BinaryOp", "0=0", [G["elt_esum"], G["elt_eprod"]]), G["elt_out"])


def test_fatal_errors_become_status_codes():
    h = _host()
    with pytest.raises(h.HostError) as e:
        h.run_op("Pooling", "0=0 1=3 99=1", [G["pool_x"]])
    assert "Un-supported Pooling Attribution" in str(e.value)
    with pytest.raises(h.HostError) as e:
        h.run_op("NoSuchOp", "", [G["pool_x"]])
    assert "Un-suppoted operation type" in str(e.value)
    with pytest.raises(h.HostError):
        h.run_op("Eltwise", "0=1", [G["elt_x"], G["elt_x"][:, :3]])   # shape mismatch CHECK


def _rel(a, b):
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-12))


@pytest.mark.parametrize("fusion", [True, False], ids=["fused", "op_by_op"])
def test_resnet18_fp(fusion):
    h = _host()
    g, _ = models.resnet18(2)
    p = h.Pipeline(g.phai_text(), g.racy_bytes(), 0, fusion=fusion)
    x = G["resnet_x"]
    for _ in range(3):     # eager, capture, replay
        out = p.forward(x)["logits"].reshape(2, -1)
    ref = G["resnet_f32_logits"]
    assert _rel(out, ref) < 1e-2, _rel(out, ref)
    assert (out.argmax(1) == ref.argmax(1)).all()
    s1 = p.get("s1b1_out")
    assert_close_f16(s1, G["resnet_f32_s1b1_out"], rel=2e-2, what="s1b1_out")
    launches, ms = p.stats()
    assert (launches > 0) == fusion
    p.close()


@pytest.mark.parametrize("fusion", [True, False], ids=["fused", "op_by_op"])
def test_resnet18_int8(fusion):
    h = _host()
    scales = {str(n): np.float32(s) for n, s in zip(G["resnet_scale_names"], G["resnet_scales"])}
    g, _ = models.resnet18(2, act_scales=scales)
    p = h.Pipeline(g.phai_text(), g.racy_bytes(), 0, fusion=fusion)
    x = G["resnet_x"]
    for _ in range(3):
        out = p.forward(x)["logits"].reshape(2, -1)
    ref = G["resnet_i8_logits"]
    r = _rel(out, ref)
    assert r < 3e-2, r
    assert (out.argmax(1) == ref.argmax(1)).all()
    # first block output: int8 steps of the reference's own quantisation grid
    s1 = p.get("s1b1_out")
    ref1 = G["resnet_i8_s1b1_out"]
    assert _rel(s1, ref1) < 2e-2, _rel(s1, ref1)
    p.close()


def test_calibration_with_own_pipeline_matches_reference_scales():
    """Max-abs calibration through this library's fp16 pipeline reproduces the scales the fp32
    reference gives (to fp16 accuracy), so a GPU-only deployment can calibrate itself."""
    h = _host()
    g, info = models.resnet18(2)
    p = h.Pipeline(g.phai_text(), g.racy_bytes(), 0, fusion=False)
    calib = np.random.default_rng(2007).uniform(0, 1, (4, 3, 64, 64)).astype(np.float32)
    scales = models.calibrate(p, info["conv_inputs"], calib)
    p.close()
    for n, s in zip(G["resnet_scale_names"], G["resnet_scales"]):
        assert abs(scales[str(n)] / s - 1.0) < 1e-2, (n, scales[str(n)], s)


# ---- MobileNetV2-style network (1x1 expand / 3x3 depthwise / 1x1 project, ReLU6 as Clip) ----------
M = np.load(os.path.join(os.path.dirname(__file__), "golden", "mobilenet_vectors.npz"))


@pytest.mark.parametrize("fusion", [True, False], ids=["fused", "op_by_op"])
def test_mobilenet_v2_fp(fusion):
    """53 layers deep with random weights, the net amplifies rounding noise by ~7 % per layer: every
    conv is within 1e-3 of the fp32 reference on its own (the single-layer tests), the first blocks
    stay within 2e-3 and the logits end up 2 % away.  The bar on the logits is therefore 3e-2."""
    h = _host()
    g, _ = models.mobilenet_v2(3)
    p = h.Pipeline(g.phai_text(), g.racy_bytes(), 0, fusion=fusion)
    x = M["x"]
    for _ in range(3):     # eager, capture, replay
        out = p.forward(x)["logits"].reshape(2, -1)
    ref = M["f32_logits"]
    assert _rel(out, ref) < 3e-2, _rel(out, ref)
    assert (out.argmax(1) == ref.argmax(1)).all()
    if not fusion:         # the fused plan does not materialise maps it folds into a conv epilogue
        for n, bar in (("b1_project_out", 2e-3), ("b3_sum", 2e-3), ("b14_dw_act", 2.5e-2)):
            assert _rel(p.get(n), M["f32_" + n]) < bar, (n, _rel(p.get(n), M["f32_" + n]))
    p.close()


@pytest.mark.parametrize("fusion", [True, False], ids=["fused", "op_by_op"])
def test_mobilenet_v2_int8_pointwise(fusion):
    """35 int8 convs deep, the reference's own int8 logits are 21 % away from its fp32 logits (the
    quantisation noise of this random-weight net), and two int8 realisations whose inputs differ by
    fp16 rounding end up as far from each other.  What can be pinned: each int8 conv is bit-exact
    given the same input (the single-layer tests), the first blocks agree with the reference's int8
    maps to a few int8 steps, and the logits are no further from the fp32 truth than the
    reference's int8 logits are."""
    h = _host()
    scales = {str(n): np.float32(s) for n, s in zip(M["scale_names"], M["scales"])}
    g, _ = models.mobilenet_v2(3, act_scales=scales)
    p = h.Pipeline(g.phai_text(), g.racy_bytes(), 0, fusion=fusion)
    x = M["x"]
    for _ in range(3):
        out = p.forward(x)["logits"].reshape(2, -1)
    noise = _rel(M["i8_logits"], M["f32_logits"])
    assert _rel(out, M["f32_logits"]) < 1.25 * noise, (_rel(out, M["f32_logits"]), noise)
    assert _rel(out, M["i8_logits"]) < 1.5 * noise
    b3 = p.get("b3_sum")
    assert _rel(b3, M["i8_b3_sum"]) < 3e-2, _rel(b3, M["i8_b3_sum"])
    p.close()


# ---- graph glue and the YOLOv5s-style network -------------------------------------------------------
Y = np.load(os.path.join(os.path.dirname(__file__), "golden", "yolo_vectors.npz"))


def test_operation_concat_interp_batchnorm():
    h = _host()
    x = Y["cat_x"]
    a = h.run_op("ReLU", "", [x])
    b = h.run_op("Sigmoid", "", [x])
    y = h.run_op("Concat", "0=-1", [a, b, x])
    assert y.shape == Y["cat_out"].shape
    np.testing.assert_allclose(y, Y["cat_out"], rtol=0, atol=1e-6)      # sigmoid via __expf
    np.testing.assert_array_equal(y[:, 38:], x)
    np.testing.assert_array_equal(h.run_op("Interp", "0=1 1=2.0 2=2.0", [Y["interp2_x"]]), Y["interp2_out"])
    np.testing.assert_array_equal(h.run_op("Interp", "0=1 3=11 4=7", [Y["interp_odd_x"]]), Y["interp_odd_out"])
    g = GraphBuilder()
    g.batchnorm("bn", "in", "out", Y["bn_slope"], Y["bn_mean"], Y["bn_var"], Y["bn_bias"], eps=1e-5)
    params = g.lines[0].split(" ", 6)[6]
    y = h.run_op("BatchNorm", params, [Y["bn_x"]], g.racy_bytes())
    np.testing.assert_allclose(y, Y["bn_out"], rtol=2e-7, atol=3e-7)
    with pytest.raises(h.HostError):
        h.run_op("Concat", "0=0", [x, x])          # only the channel axis is implemented
    with pytest.raises(h.HostError):
        h.run_op("Interp", "0=2 1=2.0 2=2.0", [x])  # bilinear is not


@pytest.mark.parametrize("fusion", [True, False], ids=["fused", "op_by_op"])
def test_yolov5s_fp(fusion):
    h = _host()
    g, info = models.yolov5s(5)
    p = h.Pipeline(g.phai_text(), g.racy_bytes(), 0, fusion=fusion)
    x = Y["yolo_x"]
    for _ in range(3):     # eager, capture, replay
        out = p.forward(x)
    assert sorted(out) == sorted(info["outputs"])
    for n in info["outputs"]:
        ref = Y["yolo_" + n]
        assert out[n].shape == ref.shape
        r = _rel(out[n], ref)
        assert r < 1e-2, (n, r)
    if not fusion:
        for n in ("c3_1_cv3_act", "sppf_cat_out", "neck_up1_out"):
            assert _rel(p.get(n), Y["yolo_" + n]) < 1e-2, n
    else:
        launches, _ = p.stats()
        # every Sigmoid + BinaryOp(mul) pair folds into its conv: 57 SiLU convs + 3 heads, 7 bottleneck
        # adds, 3 pools, 13 concats, 2 resizes, ingest and 3 emits
        assert launches <= 60 + 7 + 3 + 13 + 2 + 1 + 3, launches
    p.close()


def test_chunked_forward_equals_whole_batch_forward():
    """Option h2d_chunks: sub-batches copied and computed in a software pipeline give the logits of
    the whole-batch forward bit for bit (every kernel computes an image independently of its batch)."""
    h = _host()
    scales = {str(n): np.float32(s) for n, s in zip(G["resnet_scale_names"], G["resnet_scales"])}
    g, _ = models.resnet18(2, act_scales=scales)
    p = h.Pipeline(g.phai_text(), g.racy_bytes(), 0, fusion=True)
    x = np.random.default_rng(11).uniform(0, 1, (8, 3, 64, 64)).astype(np.float32)
    whole = p.forward(x)["logits"].copy()
    for k in (2, 4, 8):
        p.set_option("h2d_chunks", k)
        for _ in range(3):      # eager, capture, replay
            out = p.forward(x)["logits"]
        assert out.shape == whole.shape
        np.testing.assert_array_equal(out, whole)
    # the input converted to fp16 by host threads before the copy: the same rounding as the device ingest kernel
    for k, t in ((1, 1), (2, 3), (4, 8)):
        p.set_option("h2d_chunks", k)
        p.set_option("host_f16_threads", t)
        for _ in range(3):
            out = p.forward(x)["logits"]
        np.testing.assert_array_equal(out, whole)
    p.set_option("host_f16_threads", 0)
    p.set_option("h2d_chunks", 3)       # 8 is not divisible by 3: falls back to the whole batch
    np.testing.assert_array_equal(p.forward(x)["logits"], whole)
    p.set_option("h2d_chunks", 1)
    np.testing.assert_array_equal(p.forward(x)["logits"], whole)
    assert p.run_resident(2) > 0
    p.close()


def test_operation_hardswish_input_focus():
    h = _host()
    np.testing.assert_allclose(h.run_op("HardSwish", "0=%r 1=0.5" % (1.0 / 6.0), [Y["hs_x"]]), Y["hs_std_out"], rtol=0, atol=5e-7)
    np.testing.assert_allclose(h.run_op("HardSwish", "0=0.2 1=0.5", [Y["hs_x"]]), Y["hs_02_out"], rtol=0, atol=5e-7)
    g = GraphBuilder()
    g.input_norm("inp", "in", "out", 10, 8, Y["inp_means"], Y["inp_scales"])
    y = h.run_op("Input", g.lines[0].split(" ", 6)[6], [Y["inp_x"]])
    np.testing.assert_allclose(y, Y["inp_out"], rtol=2e-6, atol=2e-6)    # x*v - m*v against (x - m)*v
    np.testing.assert_array_equal(h.run_op("YoloV5Focus", "", [Y["focus_x"]]), Y["focus_out"])
    both = np.concatenate([Y["focus_x"], Y["focus_x"][:, ::-1]])          # every image is converted
    np.testing.assert_array_equal(h.run_op("YoloV5Focus", "", [both]), O.focus(both))


@pytest.mark.parametrize("fusion", [True, False], ids=["fused", "op_by_op"])
def test_focus_net(fusion):
    """Input normalisation -> Focus -> conv + HardSwish x 2 -> conv against the reference's output."""
    h = _host()
    g = models.focus_net(7)
    p = h.Pipeline(g.phai_text(), g.racy_bytes(), 0, fusion=fusion)
    for _ in range(3):
        out = p.forward(Y["fnet_x"])["out"]
    assert out.shape == Y["fnet_out"].shape
    assert _rel(out, Y["fnet_out"]) < 1e-2, _rel(out, Y["fnet_out"])
    if fusion:
        launches, _ = p.stats()
        assert launches == 5       # normalise + ingest + focus in one kernel, 3 convs (HardSwish folded into two), emit
    p.close()


@pytest.mark.parametrize("fusion", [True, False], ids=["fused", "op_by_op"])
def test_batchnorm_after_conv_is_folded(fusion):
    """Conv -> BatchNorm (-> ReLU / Clip) chains: the fused plan folds every BatchNorm into the packed
    weights of the conv in front of it (5 launches: ingest, 3 convs, emit)."""
    h = _host()
    g = models.bn_net(8)
    p = h.Pipeline(g.phai_text(), g.racy_bytes(), 0, fusion=fusion)
    for _ in range(3):
        out = p.forward(Y["bnnet_x"])["out"]
    assert out.shape == Y["bnnet_out"].shape
    assert _rel(out, Y["bnnet_out"]) < 1e-2, _rel(out, Y["bnnet_out"])
    assert_close_f16(out, Y["bnnet_out"], rel=2e-2, what="bn_net out")
    if fusion:
        launches, _ = p.stats()
        assert launches == 5, launches
    p.close()


def test_calibration_tool_reproduces_the_builder_int8_graph():
    """python -m excalibur_b200.calibrate on the floating-point ResNet files gives the weight blob the
    graph builder writes for the same scales, and a pipeline that runs."""
    from excalibur_b200 import calibrate
    g32, info = models.resnet18(2)
    calib = np.random.default_rng(2007).uniform(0, 1, (4, 3, 64, 64)).astype(np.float32)
    text8, blob8, scales = calibrate.convert(g32.phai_text(), g32.racy_bytes(), calib)
    assert sorted(scales) == sorted(info["conv_inputs"])
    g8, _ = models.resnet18(2, act_scales=scales)
    assert blob8 == g8.racy_bytes()
    _, ops_a = calibrate.parse_phai(text8)
    _, ops_b = calibrate.parse_phai(g8.phai_text())
    assert [(o["type"], o["name"], o["ins"], o["outs"], o["params"]) for o in ops_a] == \
           [(o["type"], o["name"], o["ins"], o["outs"], o["params"]) for o in ops_b]
    h = _host()
    p = h.Pipeline(text8, blob8, 0, fusion=True)
    out = p.forward(G["resnet_x"])["logits"].reshape(2, -1)
    p.close()
    for n, s in zip(G["resnet_scale_names"], G["resnet_scales"]):      # the reference's own calibration
        assert abs(scales[str(n)] / s - 1.0) < 1e-2
    assert _rel(out, G["resnet_i8_logits"]) < 5e-2


def test_output_view_is_the_tensor_forward_returned():
    h = _host()
    g, info = models.yolov5s(5)
    p = h.Pipeline(g.phai_text(), g.racy_bytes(), 0)
    out = p.forward(Y["yolo_x"])
    for n in info["outputs"]:
        v = p.output_view(n)
        assert v.shape == out[n].shape
        np.testing.assert_array_equal(v, out[n])
    with pytest.raises(h.HostError):
        p.output_view("stem_act")          # an inner map is not an output
    p.close()


@pytest.mark.parametrize("int8", [False, True], ids=["fp16_net", "int8_net"])
def test_pipeline_f16_runs_the_fused_plan_on_an_fp16_input(int8):
    """pipeline<unsigned short> (the reference's fp16 Dtype): the fp16 image is uploaded as it is and the fused plan
    runs; the logits equal pipeline<float>'s on the same fp16 values, rounded to fp16, bit for bit."""
    h = _host()
    scales = {str(n): np.float32(s) for n, s in zip(G["resnet_scale_names"], G["resnet_scales"])} if int8 else None
    g, _ = models.resnet18(2, act_scales=scales)
    x16 = G["resnet_x"].astype(np.float16)
    pf = h.Pipeline(g.phai_text(), g.racy_bytes(), 0, fusion=True)
    ref = pf.forward(x16.astype(np.float32))["logits"]
    pf.close()
    ph = h.PipelineF16(g.phai_text(), g.racy_bytes(), 0, fusion=True)
    for chunks in (1, 2):
        ph.set_option("h2d_chunks", chunks)
        for _ in range(3):
            ph.forward(x16)
        launches, _ = ph.stats()
        assert launches > 0, "the fused plan did not run"
        out = ph.get("logits")
        assert out.dtype == np.float16 and out.shape == ref.shape
        np.testing.assert_array_equal(out, ref.astype(np.float16))
    ph.close()


def test_pipeline_f16_falls_back_to_op_by_op():
    """A graph whose input is not a 3-channel image (no fp16 ingest step) runs op by op on fp16 tensors."""
    h = _host()
    r = np.random.default_rng(12)
    w = (r.standard_normal((32, 16, 3, 3)) * 0.2).astype(np.float32)
    b = r.standard_normal(32).astype(np.float32)
    g = GraphBuilder()
    g.conv("c", "in", "out", w, b, 1, 1, act=1)
    x = r.uniform(-1, 1, (2, 16, 9, 11)).astype(np.float32)
    ph = h.PipelineF16(g.phai_text(), g.racy_bytes(), 0, fusion=True)
    ph.forward(x.astype(np.float16))
    launches, _ = ph.stats()
    out = ph.get("out").astype(np.float32)
    ph.close()
    assert launches <= 0
    ref = O.conv2d_f32(f16_round(x), f16_round(w), b, 1, 1, act=1)
    assert out.shape == ref.shape
    assert_close_f16(out, ref, what="fp16 pipeline, op by op")
