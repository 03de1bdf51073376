"""Generate tests/golden/reference_vectors.npz from the UNMODIFIED reference CPU library.

Run in a container that has the reference tree (it cannot travel to the GPU box):

    make -C oracle ref            # builds oracle/_ref/libexcalibur_ref.so from the reference sources
    python tests/golden/make_golden.py             # both fixture files
    python tests/golden/make_golden.py mobilenet   # tests/golden/mobilenet_vectors.npz only
    python tests/golden/make_golden.py yolo        # tests/golden/yolo_vectors.npz only
    python tests/golden/make_golden.py shipped     # tests/golden/shipped_model_vectors.npz only
    python tests/golden/make_golden.py architectures   # tests/golden/shipped_architectures.{json,npz} only
    python tests/golden/make_golden.py fullsize    # tests/golden/fullsize_vectors.npz only (minutes of CPU time)
    python tests/golden/make_golden.py boundary    # tests/golden/boundary_vectors.npz only

Every case stores its inputs, weights and the reference's output, so the fixture pins the oracle
(oracle/exb_oracle.c) and, through it, the CUDA kernels, without the reference being present.
"""
import glob
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from excalibur_b200 import model_zoo, models  # noqa: E402
from excalibur_b200.modelfile import GraphBuilder  # noqa: E402
from oracle import ref_lib  # noqa: E402
from tests.util import body_inputs, fullsize_inputs, quantize_half_away  # noqa: E402


def run(g, x, names=("out",)):
    p = ref_lib.RefPipeline(g.phai_text(), g.racy_bytes())
    p.forward(x)
    outs = [p.featmap(n) for n in names]
    p.close()
    return outs


def main():
    assert ref_lib.available(), "build oracle/_ref first: make -C oracle ref"
    r = np.random.default_rng(20240607)
    out = {}

    def conv_case(tag, N, Cin, H, W, Cout, k, stride, pad, act, int8):
        x = r.uniform(-1, 1, (N, Cin, H, W)).astype(np.float32)
        w = (r.standard_normal((Cout, Cin, k, k)) * np.sqrt(2.0 / (Cin * k * k))).astype(np.float32)
        b = (r.standard_normal(Cout) * 0.05).astype(np.float32)
        g = GraphBuilder()
        i8 = None
        if int8:
            wq, ws = models.quantize_weights(w)
            fs = np.float32(127.0 / np.abs(x).max())
            i8 = (wq, ws, fs)
            out[tag + "_wq"], out[tag + "_ws"], out[tag + "_fs"] = wq, ws, fs
        g.conv("c", "in", "out", w, b, stride, pad, act=act, int8=i8)
        (y,) = run(g, x)
        out[tag + "_x"], out[tag + "_w"], out[tag + "_b"], out[tag + "_y"] = x, w, b, y
        out[tag + "_cfg"] = np.array([stride, pad, act], np.int32)

    # fp32: Winograd path (3x3 s1, Cout < 128), packed im2col path (everything else)
    conv_case("conv_f32_wino", 2, 16, 12, 13, 32, 3, 1, 1, 1, False)
    conv_case("conv_f32_im2col_s2", 2, 8, 15, 15, 24, 3, 2, 1, 0, False)
    conv_case("conv_f32_stem", 1, 3, 32, 32, 16, 7, 2, 3, 1, False)
    conv_case("conv_f32_1x1", 2, 32, 7, 7, 136, 1, 1, 0, 0, False)
    # int8: Winograd path handles batches; the im2col path only computes image 0, so batch 1
    conv_case("conv_i8_wino", 2, 32, 10, 10, 64, 3, 1, 1, 1, True)
    conv_case("conv_i8_im2col_s2", 1, 32, 12, 12, 64, 3, 2, 1, 1, True)
    conv_case("conv_i8_im2col_wide", 1, 64, 7, 7, 128, 3, 1, 1, 0, True)
    conv_case("conv_i8_1x1_s2", 1, 32, 8, 8, 64, 1, 2, 0, 0, True)

    # depthwise 3x3 s1 / s2
    for tag, stride in (("dw_s1", 1), ("dw_s2", 2)):
        x = r.uniform(-1, 1, (2, 24, 14, 14)).astype(np.float32)
        w = (r.standard_normal((24, 1, 3, 3)) * 0.3).astype(np.float32)
        b = (r.standard_normal(24) * 0.1).astype(np.float32)
        g = GraphBuilder()
        g.dwconv("d", "in", "out", w, b, stride, 1, act=1)
        (y,) = run(g, x)
        out[tag + "_x"], out[tag + "_w"], out[tag + "_b"], out[tag + "_y"] = x, w, b, y

    # pooling
    x = r.standard_normal((2, 8, 13, 13)).astype(np.float32)
    out["pool_x"] = x
    for tag, kw in (("pool_max_3s2p1", dict(type_=0, kernel=3, stride=2, pad=1)),
                    ("pool_max_5s1p2", dict(type_=0, kernel=5, stride=1, pad=2)),
                    ("pool_max_ceil", dict(type_=0, kernel=2, stride=2, pad=0, pad_mode=0)),
                    ("pool_avg_excl", dict(type_=1, kernel=3, stride=2, pad=1, count_include_pad=0)),
                    ("pool_avg_incl", dict(type_=1, kernel=3, stride=2, pad=1, count_include_pad=1)),
                    ("pool_gap", dict(type_=1, global_pool=True))):
        g = GraphBuilder()
        g.pool("p", "in", "out", **kw)
        (out[tag + "_y"],) = run(g, x)

    # eltwise / binaryop / relu.  The graph input is fanned out through Split and convolutions so
    # that the ops see distinct tensors.
    x = r.standard_normal((2, 6, 9, 9)).astype(np.float32)
    out["elt_x"] = x
    g = GraphBuilder()
    g.split("s", "in", ["a", "b", "c"])
    g.relu("r", "a", "ra")
    g.binaryop("m", "b", "c", "bb", op=2)           # x*x
    g.eltwise("sum", ["ra", "bb", "a"], "esum", 1, coeffs=[0.5, -1.25])   # third coefficient stays 1
    g.eltwise("prod", ["ra", "bb"], "eprod", 0)
    g.eltwise("max", ["ra", "bb", "a"], "emax", 2)
    g.binaryop("add", "esum", "eprod", "out", op=0)
    p = ref_lib.RefPipeline(g.phai_text(), g.racy_bytes())
    p.forward(x)
    for n in ("ra", "bb", "esum", "eprod", "emax", "out"):
        out["elt_" + n] = p.featmap(n)
    p.close()

    # ResNet-18-style net at 64x64, batch 2: fp32 and int8 (image-at-a-time because of the
    # reference's int8 batch quirk), calibration on 4 seeded images through the fp32 reference.
    seed = 2
    x = np.random.default_rng(2000).uniform(0, 1, (2, 3, 64, 64)).astype(np.float32)
    g32, info = models.resnet18(seed)
    p32 = ref_lib.RefPipeline(g32.phai_text(), g32.racy_bytes())
    out["resnet_x"] = x
    out["resnet_f32_logits"] = p32.forward(x)["logits"].reshape(2, -1)
    out["resnet_f32_s1b1_out"] = p32.featmap("s1b1_out")
    calib = np.random.default_rng(2007).uniform(0, 1, (4, 3, 64, 64)).astype(np.float32)
    scales = models.calibrate(_RefAdapter(p32), info["conv_inputs"], calib)
    p32.close()
    names = sorted(scales)
    out["resnet_scale_names"] = np.array(names)
    out["resnet_scales"] = np.array([scales[n] for n in names], np.float32)
    g8, _ = models.resnet18(seed, act_scales=scales)
    p8 = ref_lib.RefPipeline(g8.phai_text(), g8.racy_bytes())
    logits, s1 = [], []
    for i in range(2):
        logits.append(p8.forward(x[i:i + 1])["logits"].reshape(1, -1))
        s1.append(p8.featmap("s1b1_out"))
    p8.close()
    out["resnet_i8_logits"] = np.concatenate(logits)
    out["resnet_i8_s1b1_out"] = np.concatenate(s1)

    path = os.path.join(ROOT, "tests", "golden", "reference_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path) // 1024, "KiB,", len(out), "arrays")
    mobilenet()
    yolo()
    shipped()
    architectures()


def shipped():
    """PReLU, LeakyRelu, Deconvolution, Reshape + Transpose one at a time, and the three networks with the
    architecture of the reference's shipped descriptions (excalibur_b200/model_zoo.py) at small input
    sizes -> tests/golden/shipped_model_vectors.npz."""
    r = np.random.default_rng(20240609)
    out = {}
    x = r.standard_normal((2, 13, 5, 7)).astype(np.float32)
    sl = r.uniform(0.05, 0.5, 13).astype(np.float32)
    out["act_x"], out["prelu_slopes"] = x, sl
    g = GraphBuilder(); g.prelu("p", "in", "out", sl)
    out["prelu_out"], = run(g, x)
    g = GraphBuilder(); g.prelu("p", "in", "out", sl[:1])
    out["prelu_shared_out"], = run(g, x)
    g = GraphBuilder(); g.leakyrelu("p", "in", "out", 0.1)
    out["leaky_out"], = run(g, x)
    # transposed convolutions: kernel == stride (the shipped models' shape), and two overlapping shapes that
    # only pin the CPU restatement
    for tag, cin, cout, k, s, p in (("deconv_k2s2", 13, 6, 2, 2, 0), ("deconv_k2s2_c1", 13, 1, 2, 2, 0),
                                    ("deconv_k3s2p1", 13, 6, 3, 2, 1), ("deconv_k4s2p1", 13, 6, 4, 2, 1)):
        w = (r.standard_normal((cin, cout, k, k)) * 0.2).astype(np.float32)
        b = r.standard_normal(cout).astype(np.float32)
        g = GraphBuilder(); g.deconv("d", "in", "out", w, b, s, p)
        out[tag + "_w"], out[tag + "_b"] = w, b
        out[tag + "_cfg"] = np.array([k, s, p], np.int32)
        out[tag + "_out"], = run(g, x)
    x = r.standard_normal((2, 12, 4, 5)).astype(np.float32)
    g = GraphBuilder()
    g.reshape("r", "in", "m", w=20, h=4, c=3)
    g.transpose("t", "m", "out")
    out["rt_x"] = x
    out["rt_out"], = run(g, x)

    def net(tag, g, info, x, inner=()):
        p = ref_lib.RefPipeline(g.phai_text(), g.racy_bytes())
        res = p.forward(x)
        out[tag + "_x"] = x
        for n in info["outputs"]:
            out["%s_out_%s" % (tag, n)] = res[n]
        for n in inner:
            out["%s_map_%s" % (tag, n)] = p.featmap(n)
        p.close()

    g, info = model_zoo.det_db_resnet18()
    net("detdb", g, info, r.uniform(0, 255, (2, 3, 64, 96)).astype(np.float32), ("s2_b2_act", "fuse_out", "head_relu_out"))
    g, info = model_zoo.mobile_unicorn()
    net("unicorn", g, info, r.uniform(0, 255, (2, 3, 128, 128)).astype(np.float32), ("conv2_4_res", "conv5_ex_act"))
    # batch 1: the reference's YoloV5Focus only fills image 0
    g, info = model_zoo.yolov5s_simp(size=128)
    net("yolosimp", g, info, r.uniform(0, 255, (1, 3, 128, 128)).astype(np.float32), ("csp2_cv4_act", "spp_cat_out"))
    # HardSigmoid, Softmax over channels, Flatten (default axis and axis 0), per-channel broadcast BinaryOp
    x = (r.standard_normal((2, 7, 3, 5)) * 3).astype(np.float32)
    out["misc_x"] = x
    g = GraphBuilder(); g._op("HardSigmoid", "h", ["in"], ["out"], "0=0.2 1=0.5")
    out["hardsigmoid_out"], = run(g, x)
    g = GraphBuilder(); g._op("Softmax", "s", ["in"], ["out"], "0=0 1=1")
    out["softmax_out"], = run(g, x)
    g = GraphBuilder(); g._op("Flatten", "f", ["in"], ["out"], "")
    out["flatten_out"], = run(g, x)
    g = GraphBuilder(); g._op("Flatten", "f", ["in"], ["out"], "0=0")
    out["flatten0_out"], = run(g, x)
    g = GraphBuilder()
    g.split("s", "in", ["a", "b"])
    g.pool("gap", "b", "gate", 1, 1, 1, 0, global_pool=True)
    g.binaryop("mul", "a", "gate", "out", 2)
    out["bcast_mul_out"], = run(g, x)
    g = GraphBuilder()
    g.split("s", "in", ["a", "b"])
    g.pool("gap", "b", "gate", 1, 1, 1, 0, global_pool=True)
    g.binaryop("sub", "gate", "a", "out", 1)          # the reference computes op(larger, smaller) whatever the order
    out["bcast_sub_out"], = run(g, x)

    # the shipped int8 description: max-abs calibration of every dense conv's input through the reference's
    # fp32 pipeline on 8 seeded images, then the reference's int8 forward (batch 1: its packed int8 path only
    # computes image 0)
    g, info = model_zoo.unicorn_light()
    calib = r.uniform(0, 255, (8, 3, 128, 128)).astype(np.float32)
    pf = ref_lib.RefPipeline(g.phai_text(), g.racy_bytes())
    scales = models.calibrate(_RefAdapter(pf), info["conv_inputs"], calib)
    x = r.uniform(0, 255, (1, 3, 128, 128)).astype(np.float32)
    out["ulight_x"] = x
    out["ulight_fp_out"] = pf.forward(x)["conv5_dw"]
    pf.close()
    names = sorted(scales)
    out["ulight_scale_names"] = np.array(names)
    out["ulight_scales"] = np.array([scales[n] for n in names], np.float32)
    g8, info8 = model_zoo.unicorn_light(act_scales=scales)
    p8 = ref_lib.RefPipeline(g8.phai_text(), g8.racy_bytes())
    out["ulight_i8_out"] = p8.forward(x)["conv5_dw"]
    out["ulight_i8_map_res2_2"] = p8.featmap("res2_2")
    p8.close()
    path = os.path.join(ROOT, "tests", "golden", "shipped_model_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path) // 1024, "KiB,", len(out), "arrays")
    for k, v in out.items():
        if "_out" in k:
            print("  %-40s %-18s |max| %.4g finite=%s" % (k, v.shape, np.abs(v).max(), np.isfinite(v).all()))


def yolo():
    """Graph-glue operations (Concat, Interp nearest, BatchNorm) one at a time, and the YOLOv5s-style
    net at 128x128, batch 2 -> tests/golden/yolo_vectors.npz."""
    r = np.random.default_rng(20240608)
    out = {}
    # Concat of three maps with ragged channel counts
    # (the reference driver feeds one input tensor: the three maps derive from it)
    g = GraphBuilder()
    g.split("s", "in", ["i0", "i1", "i2"])
    g.relu("r0", "i0", "a")
    g.sigmoid("r1", "i1", "b")
    g.concat("cat", ["a", "b", "i2"], "out")
    x = r.standard_normal((2, 19, 5, 7)).astype(np.float32)
    out["cat_x"] = x
    out["cat_out"], = run(g, x)
    # nearest resize: 2x, and a non-integer ratio through explicit output sizes
    g = GraphBuilder()
    g.interp_nearest("up", "in", "out", 2.0)
    x = r.standard_normal((2, 10, 6, 5)).astype(np.float32)
    out["interp2_x"] = x
    out["interp2_out"], = run(g, x)
    g = GraphBuilder()
    g._op("Interp", "up", ["in"], ["out"], "0=1 3=11 4=7")
    out["interp_odd_x"] = x
    out["interp_odd_out"], = run(g, x)
    # batch norm
    C = 13
    bn = [r.uniform(0.5, 1.5, C), r.standard_normal(C), r.uniform(0.5, 2.0, C), r.standard_normal(C)]
    bn = [v.astype(np.float32) for v in bn]
    g = GraphBuilder()
    g.batchnorm("bn", "in", "out", *bn, eps=1e-5)
    x = r.standard_normal((2, C, 6, 5)).astype(np.float32)
    out["bn_x"] = x
    for k, n in enumerate(("slope", "mean", "var", "bias")):
        out["bn_" + n] = bn[k]
    out["bn_out"], = run(g, x)

    # HardSwish (standard and ncnn-style constants), Input normalisation, YoloV5Focus (batch 1: the
    # reference only fills image 0), and a small Input -> Focus -> Conv -> HardSwish -> Conv net
    x = (r.standard_normal((2, 5, 6, 7)) * 4).astype(np.float32)
    out["hs_x"] = x
    g = GraphBuilder(); g.hardswish("h", "in", "out")
    out["hs_std_out"], = run(g, x)
    g = GraphBuilder(); g.hardswish("h", "in", "out", 0.2, 0.5)
    out["hs_02_out"], = run(g, x)
    x = r.uniform(0, 255, (2, 3, 8, 10)).astype(np.float32)
    means, scales = [123.675, 116.28, 103.53], [0.0171, 0.0175, 0.0174]
    g = GraphBuilder(); g.input_norm("inp", "in", "out", 10, 8, means, scales)
    out["inp_x"] = x
    out["inp_means"] = np.array(means, np.float32)
    out["inp_scales"] = np.array(scales, np.float32)
    out["inp_out"], = run(g, x)
    x = r.standard_normal((1, 3, 10, 12)).astype(np.float32)
    g = GraphBuilder(); g.focus("f", "in", "out")
    out["focus_x"] = x
    out["focus_out"], = run(g, x)
    x = r.uniform(0, 255, (1, 3, 32, 32)).astype(np.float32)
    g = models.focus_net(7)
    pf = ref_lib.RefPipeline(g.phai_text(), g.racy_bytes())
    out["fnet_x"] = x
    out["fnet_out"] = pf.forward(x)["out"]
    pf.close()

    x = r.uniform(0, 1, (2, 3, 20, 24)).astype(np.float32)
    g = models.bn_net(8)
    pb = ref_lib.RefPipeline(g.phai_text(), g.racy_bytes())
    out["bnnet_x"] = x
    out["bnnet_out"] = pb.forward(x)["out"]
    pb.close()

    x = np.random.default_rng(5000).uniform(0, 1, (2, 3, 128, 128)).astype(np.float32)
    gy, info = models.yolov5s(5)
    py = ref_lib.RefPipeline(gy.phai_text(), gy.racy_bytes())
    res = py.forward(x)
    out["yolo_x"] = x
    for n in info["outputs"]:
        out["yolo_" + n] = res[n]
    for n in ("c3_1_cv3_act", "sppf_cat_out", "neck_up1_out"):
        out["yolo_" + n] = py.featmap(n)
    py.close()
    path = os.path.join(ROOT, "tests", "golden", "yolo_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path) // 1024, "KiB,", len(out), "arrays")


def mobilenet():
    """MobileNetV2-style net at 64x64, batch 2 -> tests/golden/mobilenet_vectors.npz: fp32 logits and
    two inner feature maps, max-abs scales of the 1x1 convs from 4 seeded images, and the int8
    network's logits (one image per forward because of the reference's int8 batch quirk)."""
    seed = 3
    out = {}
    x = np.random.default_rng(3000).uniform(0, 1, (2, 3, 64, 64)).astype(np.float32)
    g32, info = models.mobilenet_v2(seed)
    p32 = ref_lib.RefPipeline(g32.phai_text(), g32.racy_bytes())
    out["x"] = x
    out["f32_logits"] = p32.forward(x)["logits"].reshape(2, -1)
    for n in ("b1_project_out", "b3_sum", "b14_dw_act"):
        out["f32_" + n] = p32.featmap(n)
    calib = np.random.default_rng(3007).uniform(0, 1, (4, 3, 64, 64)).astype(np.float32)
    scales = models.calibrate(_RefAdapter(p32), info["conv_inputs"], calib)
    p32.close()
    names = sorted(scales)
    out["scale_names"] = np.array(names)
    out["scales"] = np.array([scales[n] for n in names], np.float32)
    g8, _ = models.mobilenet_v2(seed, act_scales=scales)
    p8 = ref_lib.RefPipeline(g8.phai_text(), g8.racy_bytes())
    logits, b3 = [], []
    for i in range(2):
        logits.append(p8.forward(x[i:i + 1])["logits"].reshape(1, -1))
        b3.append(p8.featmap("b3_sum"))
    p8.close()
    out["i8_logits"] = np.concatenate(logits)
    out["i8_b3_sum"] = np.concatenate(b3)
    path = os.path.join(ROOT, "tests", "golden", "mobilenet_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path) // 1024, "KiB,", len(out), "arrays")


REF_MODELS = os.path.join(ref_lib.reference_tree(), "models")


def architectures():
    """Every shipped floating-point description whose operation types are all implemented: its name-free
    canonical structure (model_zoo.structure) -> tests/golden/shipped_architectures.json, and the reference's
    outputs for the graph model_zoo.graph_from_structure rebuilds from it (seeded weights, seeded input) ->
    tests/golden/shipped_architectures.npz (outputs and four inner maps, sampled down to 8192 values each).
    Descriptions with identical structures are listed once."""
    from excalibur_b200.calibrate import parse_phai
    archs, out, seen = [], {}, []
    for path in sorted(glob.glob(os.path.join(REF_MODELS, "*.phai"))):
        text = open(path).read()
        name = os.path.basename(path)[:-5]
        if model_zoo.unsupported_types(text) or name.endswith("_int8"):
            continue
        st = model_zoo.structure(text)
        dup = [a["name"] for a, s_ in seen if s_ == st]
        if dup:
            [a for a, s_ in seen if s_ == st][0]["same_as"].append(name)
            continue
        _, ops = parse_phai(text)
        inp = [op for op in ops if op["type"] == "Input"][0]["params"]
        w, h = int(inp[0]), int(inp[1])
        types = {t for t, _, _ in st}
        if not (types & {"innerproduct", "reshape"}):
            h, w = min(h, 64) if h > 0 else 64, 96          # fully convolutional: a small image will do
        elif w < 0:
            w = 160
        arch = {"name": name, "same_as": [], "seed": 31 + len(archs), "input_hw": [h, w], "structure": st}
        picked = None
        # the Input op's width / height keys are nominal (person_attri_simp says 640 x 640 but pools with the
        # 28 x 28 window of a 224 x 224 image): fall back to 224 x 224 when the nominal size gives no finite result
        bad_sizes = set()
        for gain, hw in [(g_, (h, w)) for g_ in (2.0, 1.6, 1.2, 1.0, 0.8, 0.6, 0.5, 0.4, 0.3)] + [(g_, (224, 224)) for g_ in (2.0, 1.6, 1.2, 1.0, 0.8)]:
            if hw in bad_sizes:
                continue
            arch["input_hw"] = list(hw)
            x = model_zoo.architecture_input(arch)
            g, outs = model_zoo.graph_from_structure(st, arch["seed"], gain=gain)
            p = ref_lib.RefPipeline(g.phai_text(), g.racy_bytes())
            try:
                res = p.forward(x)
            except Exception:           # an image size the graph cannot take
                p.close()
                bad_sizes.add(hw)
                continue
            if not all(np.isfinite(v).all() for v in res.values()) and gain == 2.0:
                p.close()
                bad_sizes.add(hw)       # not a matter of weight scale: the size does not fit the graph
                continue
            inner = [i for i in (len(st) // 4, len(st) // 2, 3 * len(st) // 4, len(st) - 2)]
            maps = {i: p.featmap("t%d" % i) for i in inner}
            peak = max(float(np.abs(p.featmap("t%d" % i)).max()) for i in range(len(st)) if st[i][0] != "input")
            logit_peak = max([float(np.abs(p.featmap("t%d" % st[i][2][0][0])).max()) for i in range(len(st))
                              if st[i][0] == "sigmoid" and "t%d" % i in outs] + [0.0])
            p.close()
            # a Sigmoid at the output turns a small relative error of a large logit into a large absolute one:
            # such graphs get weights small enough for logits of a few units
            finite = all(np.isfinite(v).all() for v in res.values())
            if finite and peak < 8000.0 and logit_peak < 12.0:      # fp16 feature maps on the device: stay well below 65504
                picked = gain
                break
        assert picked is not None, name
        arch["gain"] = picked
        arch["outputs"] = outs
        arch["inner"] = inner
        for n in outs:
            out["%s:%s" % (name, n)] = model_zoo.sample(res[n])
            out["%s:%s:shape" % (name, n)] = np.array(res[n].shape, np.int64)
        for i, v in maps.items():
            out["%s:t%d" % (name, i)] = model_zoo.sample(v)
        h, w = arch["input_hw"]
        print("%-40s gain %.1f peak %.3g input %dx%d outputs %s" % (
            name[:40], picked, peak, h, w, " ".join("%s%s" % (n, res[n].shape) for n in outs)), flush=True)
        archs.append(arch)
        seen.append((arch, st))
    jpath = os.path.join(ROOT, "tests", "golden", "shipped_architectures.json")
    with open(jpath, "w") as f:
        json.dump(archs, f, separators=(",", ":"))
    npath = os.path.join(ROOT, "tests", "golden", "shipped_architectures.npz")
    np.savez_compressed(npath, **out)
    print("wrote", jpath, os.path.getsize(jpath) // 1024, "KiB and", npath, os.path.getsize(npath) // 1024, "KiB,", len(archs),
          "architectures")


def boundary():
    """The ReLU6 operation (values above 6 become 0) alone and behind a convolution, and a convolution with the
    Mish suffix activation (key 9=5), fp32 and int8 -> tests/golden/boundary_vectors.npz."""
    r = np.random.default_rng(20240610)
    out = {}
    x = (r.standard_normal((2, 9, 7, 5)) * 4).astype(np.float32)
    x.flat[:6] = [0.0, -0.0, 6.0, np.nextafter(np.float32(6), np.float32(7)), 5.999, -1e-30]
    out["relu6_x"] = x
    g = GraphBuilder(); g.relu6("r", "in", "out")
    out["relu6_out"], = run(g, x)
    g = GraphBuilder(); g._op("ReLU6", "r", ["in"], ["out"], "0=0.0 1=6.0")     # keys 0 / 1 are accepted and ignored
    out["relu6_keys_out"], = run(g, x)
    # convolution -> ReLU6 (fused into the epilogue by the plan)
    xc = r.uniform(-1, 1, (2, 16, 9, 11)).astype(np.float32)
    w = (r.standard_normal((32, 16, 3, 3)) * 0.35).astype(np.float32)
    b = (r.standard_normal(32) * 0.5 + 2.0).astype(np.float32)
    out["conv_x"], out["conv_w"], out["conv_b"] = xc, w, b
    g = GraphBuilder()
    g.conv("c", "in", "m", w, b, 1, 1, act=0)
    g.relu6("r", "m", "out")
    out["conv_relu6_out"], = run(g, xc)
    # Mish suffix activation, fp32 and int8 (batch 2: the 3x3 stride-1 int8 path handles batches)
    g = GraphBuilder(); g.conv("c", "in", "out", w, b, 1, 1, act=5)
    out["conv_mish_out"], = run(g, xc)
    wq, ws = models.quantize_weights(w)
    fs = np.float32(127.0 / np.abs(xc).max())
    out["conv_wq"], out["conv_ws"], out["conv_fs"] = wq, ws, fs
    g = GraphBuilder(); g.conv("c", "in", "out", w, b, 1, 1, act=5, int8=(wq, ws, fs))
    out["conv_mish_i8_out"], = run(g, xc)
    path = os.path.join(ROOT, "tests", "golden", "boundary_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path) // 1024, "KiB,", len(out), "arrays")
    print("relu6: %d of %d values above 6 -> 0" % (int((x > 6).sum()), x.size), float(out["relu6_out"][x > 6].max()))


def fullsize():
    """The benchmark configurations at the image sizes they are benchmarked at -> tests/golden/fullsize_vectors.npz.

    ResNet-18-style at 3x224x224: fp32 logits and sampled block outputs for 3 seeded images; max-abs activation scales
    from 32 seeded calibration images through the reference's fp32 pipeline; the int8 network's logits (one image per
    forward: the reference's packed int8 path only computes image 0) and, for one block output per stage, the int8
    tensor the NEXT int8 convolution sees in the reference: quantize(map, that convolution's scale).
    MobileNetV2-style at 224 (2 images, 8 calibration images) and YOLOv5s-style at 640 (1 image): logits / head outputs
    and inner maps, sampled.  Inputs are regenerated from their seeds (fullsize_inputs); a checksum pins them."""
    out = {}
    # ---- ResNet-18-style -----------------------------------------------------------------------
    seed = 2
    x = fullsize_inputs("resnet", 3, 224)
    out["resnet_x_sum"] = np.float64(x.astype(np.float64).sum())
    g32, info = models.resnet18(seed)
    p32 = ref_lib.RefPipeline(g32.phai_text(), g32.racy_bytes())
    out["resnet_f32_logits"] = p32.forward(x)["logits"].reshape(3, -1)
    maps = ("pool1_out", "s1b1_out", "s1b2_out", "s2b1_out", "s3b1_out", "s4b1_out", "s4b2_out")
    for n in maps:
        out["resnet_f32_" + n] = model_zoo.sample(p32.featmap(n))
    scales = models.calibrate(_RefAdapter(p32), info["conv_inputs"], fullsize_inputs("resnet_calib", 32, 224))
    p32.close()
    names = sorted(scales)
    out["resnet_scale_names"] = np.array(names)
    out["resnet_scales"] = np.array([scales[n] for n in names], np.float32)
    g8, _ = models.resnet18(seed, act_scales=scales)
    p8 = ref_lib.RefPipeline(g8.phai_text(), g8.racy_bytes())
    logits = []
    q = {("pool1_out", "s1b1_conv1"): [], ("s1b1_out", "s1b2_conv1"): [], ("s2b1_out", "s2b2_conv1"): [],
         ("s3b1_out", "s3b2_conv1"): [], ("s4b1_out", "s4b2_conv1"): []}
    smp = {n: [] for n in maps}
    for i in range(3):
        logits.append(p8.forward(x[i:i + 1])["logits"].reshape(1, -1))
        for (m, conv) in q:
            q[(m, conv)].append(quantize_half_away(p8.featmap(m), scales[conv]))
        for n in maps:
            smp[n].append(model_zoo.sample(p8.featmap(n), 4096))
    p8.close()
    out["resnet_i8_logits"] = np.concatenate(logits)
    for (m, conv), v in q.items():
        out["resnet_i8_q_%s_for_%s" % (m, conv)] = np.concatenate(v)
    for n in maps:
        out["resnet_i8_" + n] = np.stack(smp[n])
    print("resnet done", flush=True)

    # ---- the int8 residual trunk alone, from a seeded 64 x 56 x 56 map ----------------------------
    # Both sides then quantise the SAME fp32 input, so the int8 tensors of the first blocks can be compared to the
    # LSB: what differs is only what the plan composes differently (fp16 skip, requantisation in the producer's
    # epilogue with round-half-even where the reference quantises in the consumer with round-half-away).
    seed = 2
    xb = body_inputs("resnet_body", 2)
    out["body_x_sum"] = np.float64(xb.astype(np.float64).sum())
    g32, info = models.resnet18(seed, in_ch=3, stem=False)
    p32 = ref_lib.RefPipeline(g32.phai_text(), g32.racy_bytes())
    out["body_f32_logits"] = p32.forward(xb)["logits"].reshape(2, -1)
    bscales = models.calibrate(_RefAdapter(p32), info["conv_inputs"], body_inputs("resnet_body_calib", 8))
    p32.close()
    names = sorted(bscales)
    out["body_scale_names"] = np.array(names)
    out["body_scales"] = np.array([bscales[n] for n in names], np.float32)
    g8, _ = models.resnet18(seed, act_scales=bscales, stem=False)
    p8 = ref_lib.RefPipeline(g8.phai_text(), g8.racy_bytes())
    logits = []
    qb = {("s1b1_out", "s1b2_conv1"): [], ("s1b2_out", "s2b1_conv1"): [], ("s2b1_out", "s2b2_conv1"): [],
          ("s3b1_out", "s3b2_conv1"): [], ("s4b1_out", "s4b2_conv1"): []}
    for i in range(2):
        logits.append(p8.forward(xb[i:i + 1])["logits"].reshape(1, -1))
        for (m, conv) in qb:
            qb[(m, conv)].append(quantize_half_away(p8.featmap(m), bscales[conv]))
    p8.close()
    out["body_i8_logits"] = np.concatenate(logits)
    for (m, conv), v in qb.items():
        out["body_i8_q_%s_for_%s" % (m, conv)] = np.concatenate(v)
    print("resnet body done", flush=True)

    # ---- MobileNetV2-style ---------------------------------------------------------------------
    seed = 3
    x = fullsize_inputs("mobilenet", 2, 224)
    out["mobilenet_x_sum"] = np.float64(x.astype(np.float64).sum())
    g32, info = models.mobilenet_v2(seed)
    p32 = ref_lib.RefPipeline(g32.phai_text(), g32.racy_bytes())
    out["mobilenet_f32_logits"] = p32.forward(x)["logits"].reshape(2, -1)
    mmaps = ("b1_project_out", "b3_sum", "b7_dw_act", "b14_dw_act")
    for n in mmaps:
        out["mobilenet_f32_" + n] = model_zoo.sample(p32.featmap(n))
    scales = models.calibrate(_RefAdapter(p32), info["conv_inputs"], fullsize_inputs("mobilenet_calib", 8, 224))
    p32.close()
    names = sorted(scales)
    out["mobilenet_scale_names"] = np.array(names)
    out["mobilenet_scales"] = np.array([scales[n] for n in names], np.float32)
    g8, _ = models.mobilenet_v2(seed, act_scales=scales)
    p8 = ref_lib.RefPipeline(g8.phai_text(), g8.racy_bytes())
    logits, b3 = [], []
    for i in range(2):
        logits.append(p8.forward(x[i:i + 1])["logits"].reshape(1, -1))
        b3.append(model_zoo.sample(p8.featmap("b3_sum")))
    p8.close()
    out["mobilenet_i8_logits"] = np.concatenate(logits)
    out["mobilenet_i8_b3_sum"] = np.stack(b3)
    print("mobilenet done", flush=True)

    # ---- YOLOv5s-style -------------------------------------------------------------------------
    x = fullsize_inputs("yolo", 1, 640)
    out["yolo_x_sum"] = np.float64(x.astype(np.float64).sum())
    gy, info = models.yolov5s(5)
    py = ref_lib.RefPipeline(gy.phai_text(), gy.racy_bytes())
    res = py.forward(x)
    out["yolo_outputs"] = np.array(list(info["outputs"]))
    for n in info["outputs"]:
        out["yolo_" + n] = model_zoo.sample(res[n])
        out["yolo_%s_shape" % n] = np.array(res[n].shape, np.int64)
        out["yolo_%s_absmax" % n] = np.float32(np.abs(res[n]).max())
    for n in ("c3_1_cv3_act", "sppf_cat_out", "neck_up1_out"):
        out["yolo_" + n] = model_zoo.sample(py.featmap(n))
        out["yolo_%s_absmax" % n] = np.float32(np.abs(py.featmap(n)).max())
    py.close()
    path = os.path.join(ROOT, "tests", "golden", "fullsize_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path) // 1024, "KiB,", len(out), "arrays")


class _RefAdapter:
    def __init__(self, p):
        self.p = p

    def forward(self, x):
        return self.p.forward(x)

    def get(self, name):
        return self.p.featmap(name)


if __name__ == "__main__":
    if sys.argv[1:] == ["mobilenet"]:
        mobilenet()
    elif sys.argv[1:] == ["yolo"]:
        yolo()
    elif sys.argv[1:] == ["shipped"]:
        shipped()
    elif sys.argv[1:] == ["architectures"]:
        architectures()
    elif sys.argv[1:] == ["fullsize"]:
        fullsize()
    elif sys.argv[1:] == ["boundary"]:
        boundary()
    else:
        main()
