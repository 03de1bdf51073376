"""Seeded synthetic networks of the benchmark configurations, emitted as .phai + .racy so that the
reference CPU library and this package load byte-identical graphs and weights.

ResNet-18-style classifier: 7x7/2 stem (64 ch, folded BN, ReLU), 3x3/2 max pool, four stages of
two basic blocks (two 3x3 convs + residual add + ReLU) at widths 64/128/256/512, stride 2 and a
1x1 projection shortcut at the start of stages 2-4, global average pool, FC 512->1000.  Weights are
Kaiming-normal, BN parameters gamma~U[0.5,1.5], beta~N(0,0.1), mean~N(0,0.1), var~U[0.5,1.5] are
folded into the conv (w*gamma/sqrt(var), beta-gamma*mean/sqrt(var); eps = 0 as in the reference's
BatchNorm default).  The int8 variant quantises every conv except the stem (and leaves the FC in
floating point): symmetric per-output-channel int8 weights with the reference's scale convention
ws[c] = 127/max|w[c]|, one activation scale fs = 127/max|x| per conv from a calibration pass.
"""
import numpy as np

from .modelfile import GraphBuilder

RESNET18_WIDTHS = (64, 128, 256, 512)


def _tensor_rng(seed, index):
    return np.random.default_rng(seed * 100003 + index)


class _Weights:
    def __init__(self, seed):
        self.seed = seed
        self.index = 0

    def conv_bn(self, cout, cin, k):
        r = _tensor_rng(self.seed, self.index)
        self.index += 1
        w = (r.standard_normal((cout, cin, k, k)) * np.sqrt(2.0 / (cin * k * k))).astype(np.float32)
        gamma = r.uniform(0.5, 1.5, cout).astype(np.float32)
        beta = (r.standard_normal(cout) * 0.1).astype(np.float32)
        mean = (r.standard_normal(cout) * 0.1).astype(np.float32)
        var = r.uniform(0.5, 1.5, cout).astype(np.float32)
        s = gamma / np.sqrt(var)
        return (w * s[:, None, None, None]).astype(np.float32), (beta - mean * s).astype(np.float32)

    def fc(self, cout, cin):
        r = _tensor_rng(self.seed, self.index)
        self.index += 1
        return ((r.standard_normal((cout, cin)) * 0.01).astype(np.float32),
                (r.standard_normal(cout) * 0.01).astype(np.float32))


def quantize_weights(w):
    cout = w.shape[0]
    m = np.abs(w).reshape(cout, -1).max(axis=1)
    ws = (127.0 / np.maximum(m, 1e-12)).astype(np.float32)
    wq = np.clip(np.rint(w * ws[:, None, None, None]), -127, 127).astype(np.int8)
    return wq, ws


def resnet18(seed=2, act_scales=None, widths=RESNET18_WIDTHS, num_classes=1000, in_ch=3, stem=True):
    """Returns (GraphBuilder, info).  act_scales: {conv name: fs} turns the named convs into int8
    convs (every conv except the stem must be present); None builds the floating-point graph.
    info["conv_inputs"] maps each quantisable conv to the feature map it reads (for calibration).
    stem=False leaves out the stem convolution and the max pooling: the graph's input "data" is then the
    widths[0]-channel map the first block reads (same weights as the full network's blocks)."""
    g = GraphBuilder("resnet18_style")
    wts = _Weights(seed)
    conv_inputs = {}

    def conv(name, x, y, cout, cin, k, stride, pad, act, quant=True):
        w, b = wts.conv_bn(cout, cin, k)
        int8 = None
        if quant:
            conv_inputs[name] = x
            if act_scales is not None:
                wq, ws = quantize_weights(w)
                int8 = (wq, ws, np.float32(act_scales[name]))
        g.conv(name, x, y, w, b, stride, pad, act=act, int8=int8)
        return y

    if stem:
        x = conv("stem", "data", "stem_out", widths[0], in_ch, 7, 2, 3, 1, quant=False)
        x = g.pool("pool1", x, "pool1_out", 0, 3, 2, 1)
    else:
        wts.conv_bn(widths[0], in_ch, 7)      # keep the weight sequence of the full network
        x = "data"
    cin = widths[0]
    for si, wd in enumerate(widths):
        for bi in range(2):
            stride = 2 if (si > 0 and bi == 0) else 1
            p = "s%db%d" % (si + 1, bi + 1)
            a, b = g.split(p + "_split", x, [p + "_a", p + "_b"])
            h = conv(p + "_conv1", a, p + "_c1", wd, cin, 3, stride, 1, 1)
            h = conv(p + "_conv2", h, p + "_c2", wd, wd, 3, 1, 1, 0)
            if stride != 1 or cin != wd:
                sc = conv(p + "_proj", b, p + "_sc", wd, cin, 1, stride, 0, 0)
            else:
                sc = b
            s = g.eltwise(p + "_add", [h, sc], p + "_sum", 1)
            x = g.relu(p + "_relu", s, p + "_out")
            cin = wd
    x = g.pool("gap", x, "gap_out", 1, global_pool=True)
    fw, fb = wts.fc(num_classes, cin)
    g.innerproduct("fc", x, "logits", fw, fb)
    return g, {"conv_inputs": conv_inputs, "input": "data", "output": "logits"}


MOBILENET_V2_BLOCKS = ((1, 16, 1, 1), (6, 24, 2, 2), (6, 32, 3, 2), (6, 64, 4, 2), (6, 96, 3, 1), (6, 160, 3, 2),
                       (6, 320, 1, 1))


def mobilenet_v2(seed=3, act_scales=None, blocks=MOBILENET_V2_BLOCKS, num_classes=1000, in_ch=3, last=1280):
    """MobileNetV2-style (1.0x) classifier: 3x3/2 stem with 32 channels, 17 inverted-residual blocks
    (1x1 expand t=6, 3x3 depthwise, 1x1 linear project; residual add where stride is 1 and the widths
    match), 1x1 conv to 1280, global average pool, FC.  ReLU6 is written as a Clip(0, 6) operation
    after the conv so that both libraries clamp (the conv's own activation code 3 zeroes values
    above 6 in the reference).  With act_scales the 1x1 convs become int8 convs; the stem, the
    depthwise convs and the FC stay in floating point.  Returns (GraphBuilder, info) like resnet18."""
    g = GraphBuilder("mobilenet_v2_style")
    wts = _Weights(seed)
    conv_inputs = {}

    def relu6(name, x):
        return g.clip(name + "_relu6", x, name + "_act", 0.0, 6.0)

    def pw(name, x, cout, cin, act):
        w, b = wts.conv_bn(cout, cin, 1)
        conv_inputs[name] = x
        int8 = None
        if act_scales is not None:
            wq, ws = quantize_weights(w)
            int8 = (wq, ws, np.float32(act_scales[name]))
        y = g.conv(name, x, name + "_out", w, b, 1, 0, act=0, int8=int8)
        return relu6(name, y) if act else y

    w, b = wts.conv_bn(32, in_ch, 3)
    x = relu6("stem", g.conv("stem", "data", "stem_out", w, b, 2, 1, act=0))
    cin = 32
    bi = 0
    for t, c, n, s in blocks:
        for i in range(n):
            bi += 1
            p = "b%d" % bi
            stride = s if i == 0 else 1
            use_res = stride == 1 and cin == c
            if use_res:
                x, skip = g.split(p + "_split", x, [p + "_a", p + "_b"])
            h = x
            hid = cin * t
            if t != 1:
                h = pw(p + "_expand", h, hid, cin, True)
            wd, bd = wts.conv_bn(hid, 1, 3)
            h = relu6(p + "_dw", g.dwconv(p + "_dw", h, p + "_dw_out", wd, bd, stride, 1, act=0))
            h = pw(p + "_project", h, c, hid, False)
            if use_res:
                h = g.eltwise(p + "_add", [h, skip], p + "_sum", 1)
            x = h
            cin = c
    x = pw("head", x, last, cin, True)
    x = g.pool("gap", x, "gap_out", 1, global_pool=True)
    fw, fb = wts.fc(num_classes, last)
    g.innerproduct("fc", x, "logits", fw, fb)
    return g, {"conv_inputs": conv_inputs, "input": "data", "output": "logits"}


class _Net:
    """Records operations first and emits them afterwards, inserting a Split wherever a feature map
    has more than one consumer (the graph format wants every fan-out spelled out)."""

    def __init__(self, g):
        self.g = g
        self.ops = []

    def add(self, fn, ins, out):
        self.ops.append((fn, list(ins), out))
        return out

    def emit(self, inputs=("data",)):
        uses = {}
        for _, ins, _ in self.ops:
            for t in ins:
                uses[t] = uses.get(t, 0) + 1
        taken = {}

        def take(t):
            if uses.get(t, 0) <= 1:
                return t
            k = taken.get(t, 0)
            taken[t] = k + 1
            return "%s__%d" % (t, k)

        def fan_out(t):
            if uses.get(t, 0) > 1:
                self.g.split(t + "_split", t, ["%s__%d" % (t, k) for k in range(uses[t])])

        for t in inputs:
            fan_out(t)
        for fn, ins, out in self.ops:
            fn([take(t) for t in ins], out)
            fan_out(out)


def yolov5s(seed=5, num_outputs=255, in_ch=3, width=(32, 64, 128, 256, 512), depth=(1, 2, 3, 1)):
    """YOLOv5s-style detector (depth 0.33, width 0.50): 6x6/2 stem with 32 channels, 3x3/2 convs to
    64/128/256/512 each followed by a CSP-C3 block with 1/2/3/1 bottlenecks, SPPF (three chained
    5x5/1 max pools and a concat), PAN neck (nearest 2x upsample + concat on the way up, 3x3/2
    convs + concat on the way down), three 1x1 heads with `num_outputs` channels at strides
    8/16/32.  Every conv except the heads is conv + folded BN + SiLU, with SiLU written as
    Sigmoid + BinaryOp(mul).  Returns (GraphBuilder, info); info["outputs"] names the three heads."""
    g = GraphBuilder("yolov5s_style")
    wts = _Weights(seed)
    net = _Net(g)

    def conv(name, x, cout, cin, k=1, s=1, p=None, act=True):
        w, b = wts.conv_bn(cout, cin, k)
        pad = k // 2 if p is None else p
        y = net.add(lambda ins, out: g.conv(name, ins[0], out, w, b, s, pad, act=0), [x], name + "_out")
        if not act:
            return y
        sg = net.add(lambda ins, out: g.sigmoid(name + "_sig", ins[0], out), [y], name + "_sg")
        return net.add(lambda ins, out: g.binaryop(name + "_mul", ins[0], ins[1], out, 2), [sg, y], name + "_act")

    def concat(name, xs):
        return net.add(lambda ins, out: g.concat(name, ins, out), xs, name + "_out")

    def c3(name, x, c1, c2, n, shortcut):
        c_ = c2 // 2
        a = conv(name + "_cv1", x, c_, c1)
        b = conv(name + "_cv2", x, c_, c1)
        for i in range(n):
            m = "%s_m%d" % (name, i)
            h = conv(m + "_cv1", a, c_, c_)
            h = conv(m + "_cv2", h, c_, c_, 3)
            if shortcut:
                h = net.add(lambda ins, out, m=m: g.binaryop(m + "_add", ins[0], ins[1], out, 0), [a, h], m + "_sum")
            a = h
        return conv(name + "_cv3", concat(name + "_cat", [a, b]), c2, 2 * c_)

    def pool5(name, x):
        return net.add(lambda ins, out: g.pool(name, ins[0], out, 0, 5, 1, 2), [x], name + "_out")

    def up2(name, x):
        return net.add(lambda ins, out: g.interp_nearest(name, ins[0], out, 2.0), [x], name + "_out")

    w0, w1, w2, w3, w4 = width
    x = conv("stem", "data", w0, in_ch, 6, 2, 2)
    x = conv("down1", x, w1, w0, 3, 2)
    x = c3("c3_1", x, w1, w1, depth[0], True)
    x = conv("down2", x, w2, w1, 3, 2)
    p3 = c3("c3_2", x, w2, w2, depth[1], True)
    x = conv("down3", p3, w3, w2, 3, 2)
    p4 = c3("c3_3", x, w3, w3, depth[2], True)
    x = conv("down4", p4, w4, w3, 3, 2)
    x = c3("c3_4", x, w4, w4, depth[3], True)
    h = conv("sppf_cv1", x, w4 // 2, w4)
    y1 = pool5("sppf_p1", h)
    y2 = pool5("sppf_p2", y1)
    y3 = pool5("sppf_p3", y2)
    x = conv("sppf_cv2", concat("sppf_cat", [h, y1, y2, y3]), w4, 2 * w4)
    t5 = conv("neck_cv1", x, w3, w4)
    x = c3("neck_c3_1", concat("neck_cat1", [up2("neck_up1", t5), p4]), 2 * w3, w3, 1, False)
    t4 = conv("neck_cv2", x, w2, w3)
    o3 = c3("neck_c3_2", concat("neck_cat2", [up2("neck_up2", t4), p3]), 2 * w2, w2, 1, False)
    x = conv("neck_down1", o3, w2, w2, 3, 2)
    o4 = c3("neck_c3_3", concat("neck_cat3", [x, t4]), 2 * w2, w3, 1, False)
    x = conv("neck_down2", o4, w3, w3, 3, 2)
    o5 = c3("neck_c3_4", concat("neck_cat4", [x, t5]), 2 * w3, w4, 1, False)
    outs = [conv("head_p3", o3, num_outputs, w2, act=False),
            conv("head_p4", o4, num_outputs, w3, act=False),
            conv("head_p5", o5, num_outputs, w4, act=False)]
    net.emit()
    return g, {"input": "data", "outputs": outs}


def bn_net(seed=8):
    """Convolutions followed by explicit BatchNorm operations (not folded by the exporter): conv 3x3
    3->16 -> BN -> ReLU -> depthwise 3x3 -> BN -> Clip(0,6) -> conv 1x1 16->24 -> BN ("out")."""
    g = GraphBuilder("bn_net")
    r = _tensor_rng(seed, 0)

    def bn(name, x, y, c):
        g.batchnorm(name, x, y, r.uniform(0.5, 1.5, c).astype(np.float32), (r.standard_normal(c) * 0.2).astype(np.float32),
                    r.uniform(0.5, 2.0, c).astype(np.float32), (r.standard_normal(c) * 0.2).astype(np.float32), eps=1e-5)
        return y

    w = (r.standard_normal((16, 3, 3, 3)) * np.sqrt(2.0 / 27)).astype(np.float32)
    g.conv("c1", "data", "c1_out", w, (r.standard_normal(16) * 0.1).astype(np.float32), 1, 1)
    g.relu("r1", bn("bn1", "c1_out", "bn1_out", 16), "r1_out")
    wd = (r.standard_normal((16, 1, 3, 3)) * np.sqrt(2.0 / 9)).astype(np.float32)
    g.dwconv("dw", "r1_out", "dw_out", wd, None, 1, 1)
    g.clip("cl", bn("bn2", "dw_out", "bn2_out", 16), "cl_out", 0.0, 6.0)
    w = (r.standard_normal((24, 16, 1, 1)) * np.sqrt(2.0 / 16)).astype(np.float32)
    g.conv("c3", "cl_out", "c3_out", w, None, 1, 0)
    bn("bn3", "c3_out", "out", 24)
    return g


def focus_net(seed=7):
    """A small YOLOv5-v5-style front end: Input normalisation -> YoloV5Focus (space-to-depth) ->
    3x3 conv 12->32 + HardSwish -> 3x3/2 conv 32->64 + HardSwish -> 1x1 conv 64->16 ("out")."""
    g = GraphBuilder("focus_net")
    wts = _Weights(seed)
    g.input_norm("inp", "data", "data_n", 32, 32, [123.675, 116.28, 103.53], [0.0171, 0.0175, 0.0174])
    g.focus("focus", "data_n", "f0")
    w, b = wts.conv_bn(32, 12, 3)
    g.conv("c1", "f0", "c1_out", w, b, 1, 1)
    g.hardswish("h1", "c1_out", "h1_out")
    w, b = wts.conv_bn(64, 32, 3)
    g.conv("c2", "h1_out", "c2_out", w, b, 2, 1)
    g.hardswish("h2", "c2_out", "h2_out")
    w, b = wts.conv_bn(16, 64, 1)
    g.conv("c3", "h2_out", "out", w, b, 1, 0)
    return g


def calibrate(float_pipeline, conv_inputs, images):
    """fs = 127 / max|x| over the calibration images for every conv input (max-abs calibration).
    `float_pipeline` is any object with forward(x) and get(name) -> NCHW fp32 (the reference
    driver or this package's host.Pipeline)."""
    float_pipeline.forward(images)
    scales = {}
    cache = {}
    for name, fm in conv_inputs.items():
        if fm not in cache:
            cache[fm] = float(np.abs(float_pipeline.get(fm)).max())
        scales[name] = np.float32(127.0 / max(cache[fm], 1e-12))
    return scales


def resnet18_macs(widths=RESNET18_WIDTHS, num_classes=1000, in_ch=3, size=224):
    """Algorithmic multiply-accumulates per image, per layer class."""
    out = {"stem": 0, "conv3x3": 0, "proj": 0, "fc": 0}
    h = size // 2
    out["stem"] = h * h * widths[0] * in_ch * 49
    h //= 2
    cin = widths[0]
    for si, wd in enumerate(widths):
        for bi in range(2):
            if si > 0 and bi == 0:
                h //= 2
                out["proj"] += h * h * wd * cin
            out["conv3x3"] += h * h * wd * cin * 9 + h * h * wd * wd * 9
            cin = wd
    out["fc"] = cin * num_classes
    out["total"] = sum(out.values())
    return out
