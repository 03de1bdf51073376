"""Graphs with the architecture of model descriptions the reference ships, with seeded random weights.

The reference's `models/` folder holds `.phai` descriptions without weights.  These builders emit the
same operation sequences (type, parameters and wiring; feature-map names are this package's own) so the
networks can be run, checked against the reference CPU library and timed wherever the reference tree
is not available:

* `det_db_resnet18()`  - models/det_db_resnet18.phai: DB text detector, ResNet-18-vd trunk (three 3x3
  stem convs, average-pool shortcuts), FPN with nearest upsampling, two 2x2/2 transposed convolutions.
* `mobile_unicorn()`   - models/mobile_unicorn.phai: MobileFaceNet-style embedding net, PReLU
  activations, depthwise 3x3 convs, a global 8x8 depthwise conv and a 128-way InnerProduct.
* `yolov5s_simp()`     - models/yolov5s_simp.phai: YOLOv5s (Focus, BottleneckCSP with BatchNorm +
  LeakyRelu, HardSwish convs, SPP 5/9/13, PAN) with Reshape + Transpose detection heads.
* `unicorn_light()`    - models/unicorn_light_*_usefulpart.phai and its `_int8` sibling, the int8 model
  description the reference ships: every dense convolution quantised, the first one included.

`structure(text)` reduces a description to a name-free canonical form; the test-suite compares the
builders' output with the shipped files through it when the reference tree is present.
"""
import numpy as np

from .modelfile import GraphBuilder
from .models import _Net, _tensor_rng


class _Init:
    """Seeded weights: Kaiming-normal convs, small biases, BatchNorm statistics near identity."""

    def __init__(self, seed):
        self.seed = seed
        self.index = 0

    def _r(self):
        r = _tensor_rng(self.seed, self.index)
        self.index += 1
        return r

    def conv(self, cout, cin, kh, kw=None, gain=2.0):
        r = self._r()
        kw = kh if kw is None else kw
        w = (r.standard_normal((cout, cin, kh, kw)) * np.sqrt(gain / (cin * kh * kw))).astype(np.float32)
        return w, (r.standard_normal(cout) * 0.05).astype(np.float32)

    def deconv(self, cin, cout, k):
        r = self._r()
        w = (r.standard_normal((cin, cout, k, k)) * np.sqrt(2.0 / cin)).astype(np.float32)
        return w, (r.standard_normal(cout) * 0.05).astype(np.float32)

    def bn(self, c):
        r = self._r()
        return (r.uniform(0.5, 1.5, c).astype(np.float32), (r.standard_normal(c) * 0.1).astype(np.float32),
                r.uniform(0.5, 1.5, c).astype(np.float32), (r.standard_normal(c) * 0.1).astype(np.float32))

    def slopes(self, c):
        return self._r().uniform(0.05, 0.3, c).astype(np.float32)


def det_db_resnet18(seed=11, size=800):
    """Returns (GraphBuilder, info); one output, the sigmoid probability map at the input resolution.
    `size` only fills the Input op's nominal width / height keys."""
    g = GraphBuilder()
    net = _Net(g)
    init = _Init(seed)

    def conv(name, x, cout, cin, k, s=1, bias=True, relu=False):
        w, b = init.conv(cout, cin, k)
        y = net.add(lambda ins, out: g.conv(name, ins[0], out, w, b if bias else None, s, k // 2), [x], name + "_out")
        if relu:
            y = net.add(lambda ins, out: g.relu(name + "_relu", ins[0], out), [y], name + "_act")
        return y

    def add_relu(name, a, b):
        y = net.add(lambda ins, out: g.binaryop(name + "_add", ins[0], ins[1], out, 0), [a, b], name + "_sum")
        return net.add(lambda ins, out: g.relu(name + "_relu", ins[0], out), [y], name + "_act")

    def block(name, x, cin, cout, stride, first):
        """Basic block; the shortcut of a stage's first block is (2x2/2 average pool,) 1x1 conv."""
        h = conv(name + "_c1", x, cout, cin, 3, stride, relu=True)
        h = conv(name + "_c2", h, cout, cout, 3)
        if not first:
            return add_relu(name, h, x)
        sc = x
        if stride == 2:
            sc = net.add(lambda ins, out: g._op("Pooling", name + "_avg", ins, [out],
                                                "0=1 1=2 11=2 2=2 12=2 3=0 13=0 14=1 15=1 5=1 4=0"), [x], name + "_pooled")
        sc = conv(name + "_sc", sc, cout, cin, 1)
        return add_relu(name, h, sc)

    x = net.add(lambda ins, out: g.input_norm("input", ins[0], out, size, size, [123.675, 116.28, 103.53],
                                              [0.0171247, 0.017507, 0.0174292]), ["data"], "input")
    x = conv("stem1", x, 32, 3, 3, 2, relu=True)
    x = conv("stem2", x, 32, 32, 3, relu=True)
    x = conv("stem3", x, 64, 32, 3, relu=True)
    x = net.add(lambda ins, out: g._op("Pooling", "maxpool", ins, [out], "0=0 1=3 11=3 2=2 12=2 3=1 13=1 14=1 15=1 5=1 4=0"),
                [x], "pooled")
    feats = []
    cin = 64
    for s, cout in enumerate((64, 128, 256, 512)):
        x = block("s%d_b1" % (s + 1), x, cin, cout, 1 if s == 0 else 2, True)
        x = block("s%d_b2" % (s + 1), x, cout, cout, 1, False)
        feats.append(x)
        cin = cout
    c2, c3, c4, c5 = feats
    in5 = conv("in5", c5, 256, 512, 1, bias=False)
    in4 = conv("in4", c4, 256, 256, 1, bias=False)
    in3 = conv("in3", c3, 256, 128, 1, bias=False)
    in2 = conv("in2", c2, 256, 64, 1, bias=False)

    def up(name, x, scale):
        return net.add(lambda ins, out: g.interp_nearest(name, ins[0], out, float(scale)), [x], name + "_out")

    def plus(name, a, b):
        return net.add(lambda ins, out: g.binaryop(name, ins[0], ins[1], out, 0), [a, b], name + "_out")

    out4 = plus("add4", up("up5", in5, 2), in4)
    out3 = plus("add3", up("up4", out4, 2), in3)
    out2 = plus("add2", up("up3", out3, 2), in2)
    p5 = conv("p5", in5, 64, 256, 3, bias=False)
    p4 = conv("p4", out4, 64, 256, 3, bias=False)
    p3 = conv("p3", out3, 64, 256, 3, bias=False)
    p2 = conv("p2", out2, 64, 256, 3, bias=False)
    p3u = up("p3_up", p3, 2)
    p4u = up("p4_up", p4, 4)
    p5u = up("p5_up", p5, 8)
    fuse = net.add(lambda ins, out: g.concat("fuse", ins, out), [p5u, p4u, p3u, p2], "fuse_out")
    x = conv("head_conv", fuse, 64, 256, 3, relu=True)
    w, b = init.deconv(64, 64, 2)
    x = net.add(lambda ins, out: g.deconv("head_up1", ins[0], out, w, b, 2, 0), [x], "head_up1_out")
    bn = init.bn(64)
    x = net.add(lambda ins, out: g.batchnorm("head_bn", ins[0], out, *bn), [x], "head_bn_out")
    x = net.add(lambda ins, out: g.relu("head_relu", ins[0], out), [x], "head_relu_out")
    w2, b2 = init.deconv(64, 1, 2)
    w2 = (w2 * np.float32(0.02)).astype(np.float32)     # random weights let the maps grow to ~50: keep the logits O(1)
    x = net.add(lambda ins, out: g.deconv("head_up2", ins[0], out, w2, b2, 2, 0), [x], "head_up2_out")
    net.add(lambda ins, out: g.sigmoid("prob", ins[0], out), [x], "output")
    net.emit()
    return g, {"input": "data", "outputs": ["output"]}


def mobile_unicorn(seed=12):
    """Returns (GraphBuilder, info); a 128-value embedding for a 3 x 128 x 128 image (the 8x8 depthwise
    conv at the end is a global one at that resolution)."""
    g = GraphBuilder("Unicorn_Mobile_Net")
    net = _Net(g)
    init = _Init(seed)

    def short(cout, k, s, p, wsize, group=None):
        text = "0=%d 1=%d 2=1 3=%d 4=%d 5=1 6=%d" % (cout, k, s, p, wsize)
        return text + (" 7=%d" % group if group else "")

    def conv(name, x, cout, cin, k, s, p, prelu=True):
        w, b = init.conv(cout, cin, k, gain=1.0)

        def emit(ins, out):
            g._conv_weights(w, b, None)
            g._op("Convolution", name, ins, [out], short(cout, k, s, p, w.size))
        y = net.add(emit, [x], name)
        return act(name, y, cout) if prelu else y

    def dw(name, x, c, k, s, p, prelu=True):
        w, b = init.conv(c, 1, k, gain=2.0)

        def emit(ins, out):
            g._conv_weights(w, b, None)
            g._op("ConvolutionDepthWise", name, ins, [out], short(c, k, s, p, w.size, c))
        y = net.add(emit, [x], name)
        return act(name, y, c) if prelu else y

    def act(name, x, c):
        sl = init.slopes(c)
        return net.add(lambda ins, out: g.prelu(name + "_prelu", ins[0], out, sl), [x], name + "_act")

    def unit(name, x, cin, mid, cout, stride):
        h = conv(name + "_ex", x, mid, cin, 1, 1, 0)
        h = dw(name + "_dw", h, mid, 3, stride, 1)
        return conv(name + "_em", h, cout, mid, 1, 1, 0, prelu=False)

    def res(name, x, c, mid):
        h = unit(name, x, c, mid, c, 1)
        return net.add(lambda ins, out: g._op("Eltwise", name + "_sum", ins, [out], "0=1 -23301=0"), [x, h], name + "_res")

    x = net.add(lambda ins, out: g._op("Input", "data_norm", ins, [out], "0=128 1=128 2=3 3=123.0,117.0,104.0 4=0.0078125"),
                ["data"], "normed")
    x = conv("conv1", x, 64, 3, 3, 2, 1)
    x = dw("conv1_dw", x, 64, 3, 1, 1)
    x = unit("conv2", x, 64, 128, 64, 2)
    for i in range(4):
        x = res("conv2_%d" % (i + 1), x, 64, 128)
    x = unit("conv3", x, 64, 256, 128, 2)
    for i in range(6):
        x = res("conv3_%d" % (i + 1), x, 128, 256)
    x = unit("conv4", x, 128, 512, 128, 2)
    for i in range(2):
        x = res("conv4_%d" % (i + 1), x, 128, 256)
    x = conv("conv5_ex", x, 512, 128, 1, 1, 0)
    x = dw("conv5_dw", x, 512, 8, 1, 0, prelu=False)
    r = init._r()
    fw = (r.standard_normal((128, 512)) * np.sqrt(1.0 / 512)).astype(np.float32)
    net.add(lambda ins, out: g.innerproduct("fc5", ins[0], out, fw, None), [x], "fc5")
    net.emit()
    return g, {"input": "data", "outputs": ["fc5"]}


def yolov5s_simp(seed=13, size=640, num_outputs=255, anchors=3):
    """Returns (GraphBuilder, info); three outputs [N][anchors][(size/s)^2][num_outputs/anchors] for the
    strides s = 8, 16, 32.  The Reshape ops carry the grid size, so the graph is tied to `size`."""
    g = GraphBuilder()
    net = _Net(g)
    init = _Init(seed)

    def conv(name, x, cout, cin, k=1, s=1, bias=True, act=True):
        w, b = init.conv(cout, cin, k)
        y = net.add(lambda ins, out: g.conv(name, ins[0], out, w, b if bias else None, s, k // 2), [x], name + "_out")
        if act:
            y = net.add(lambda ins, out: g.hardswish(name + "_hs", ins[0], out, 1.666667e-01, 0.5), [y], name + "_act")
        return y

    def concat(name, xs):
        return net.add(lambda ins, out: g.concat(name, ins, out), xs, name + "_out")

    def csp(name, x, c1, c2, n, shortcut):
        c_ = c2 // 2
        a = conv(name + "_cv1", x, c_, c1)
        for i in range(n):
            m = "%s_m%d" % (name, i)
            h = conv(m + "_cv1", a, c_, c_)
            h = conv(m + "_cv2", h, c_, c_, 3)
            if shortcut:
                h = net.add(lambda ins, out, m=m: g.binaryop(m + "_add", ins[0], ins[1], out, 0), [a, h], m + "_sum")
            a = h
        y1 = conv(name + "_cv3", a, c_, c_, bias=False, act=False)
        y2 = conv(name + "_cv2", x, c_, c1, bias=False, act=False)
        cat = concat(name + "_cat", [y1, y2])
        bn = init.bn(2 * c_)
        h = net.add(lambda ins, out: g.batchnorm(name + "_bn", ins[0], out, *bn), [cat], name + "_bn_out")
        h = net.add(lambda ins, out: g.leakyrelu(name + "_leaky", ins[0], out, 0.1), [h], name + "_leaky_out")
        return conv(name + "_cv4", h, c2, 2 * c_)

    def pool(name, x, k):
        return net.add(lambda ins, out: g.pool(name, ins[0], out, 0, k, 1, k // 2), [x], name + "_out")

    def up2(name, x):
        return net.add(lambda ins, out: g.interp_nearest(name, ins[0], out, 2.0), [x], name + "_out")

    def head(name, x, cin, stride):
        y = conv(name, x, num_outputs, cin, act=False)
        cells = (size // stride) ** 2
        y = net.add(lambda ins, out: g.reshape(name + "_reshape", ins[0], out, w=cells, h=num_outputs // anchors, c=anchors),
                    [y], name + "_grid")
        return net.add(lambda ins, out: g.transpose(name + "_transpose", ins[0], out, (1, 0, 2)), [y], name + "_boxes")

    x = net.add(lambda ins, out: g.input_norm("images", ins[0], out, size, size, [0, 0, 0], [0.0039215]), ["data"], "images")
    x = net.add(lambda ins, out: g.focus("focus", ins[0], out), [x], "focused")
    x = conv("conv0", x, 32, 12, 3)
    x = conv("down1", x, 64, 32, 3, 2)
    x = csp("csp1", x, 64, 64, 1, True)
    x = conv("down2", x, 128, 64, 3, 2)
    p3 = csp("csp2", x, 128, 128, 3, True)
    x = conv("down3", p3, 256, 128, 3, 2)
    p4 = csp("csp3", x, 256, 256, 3, True)
    x = conv("down4", p4, 512, 256, 3, 2)
    h = conv("spp_cv1", x, 256, 512)
    x = conv("spp_cv2", concat("spp_cat", [h, pool("spp_p5", h, 5), pool("spp_p9", h, 9), pool("spp_p13", h, 13)]), 512, 1024)
    x = csp("csp4", x, 512, 512, 1, False)
    t5 = conv("neck_cv1", x, 256, 512)
    x = csp("neck_csp1", concat("neck_cat1", [up2("neck_up1", t5), p4]), 512, 256, 1, False)
    t4 = conv("neck_cv2", x, 128, 256)
    o3 = csp("neck_csp2", concat("neck_cat2", [up2("neck_up2", t4), p3]), 256, 128, 1, False)
    x = conv("neck_down1", o3, 128, 128, 3, 2)
    o4 = csp("neck_csp3", concat("neck_cat3", [x, t4]), 256, 256, 1, False)
    x = conv("neck_down2", o4, 256, 256, 3, 2)
    o5 = csp("neck_csp4", concat("neck_cat4", [x, t5]), 512, 512, 1, False)
    outs = [head("head_p3", o3, 128, 8), head("head_p4", o4, 256, 16), head("head_p5", o5, 512, 32)]
    net.emit()
    return g, {"input": "data", "outputs": outs}


def unicorn_light(seed=14, act_scales=None):
    """models/unicorn_light_*_usefulpart.phai and its `_int8` sibling: a VGG-like residual embedding net for
    3 x 128 x 128 images - unpadded 3x3 convs + ReLU + 2x2 max pooling between stages, residual pairs of
    padded 3x3 convs whose second ReLU comes BEFORE the addition (Eltwise), and a global 4x4 depthwise conv
    to a 256-value embedding.  act_scales {conv name: fs} turns every dense convolution into an int8 one
    (key 8=2, the first convolution included, as in the shipped int8 description) and the depthwise
    convolution into one with int8 weights (8=1; the reference dequantises those and computes in fp32).
    Returns (GraphBuilder, info); info["conv_inputs"] maps each dense conv to the map it reads."""
    from .models import quantize_weights
    g = GraphBuilder("unicorn_light_int8" if act_scales else "unicorn_light")
    net = _Net(g)
    init = _Init(seed)
    conv_inputs = {}

    def conv(name, x, cout, cin, pad):
        w, b = init.conv(cout, cin, 3)
        conv_inputs[name] = x
        text = "0=%d 1=3 2=1 3=1 4=%d 5=1 6=%d" % (cout, pad, w.size)

        def emit(ins, out):
            conv_inputs[name] = ins[0]
            if act_scales is None:
                g._conv_weights(w, b, None)
                g._op("Convolution", name, ins, [out], text)
            else:
                wq, ws = quantize_weights(w)
                g._conv_weights(w, b, (wq, ws, act_scales[name]))
                g._op("Convolution", name, ins, [out], text + " 8=2")
        y = net.add(emit, [x], name)
        return net.add(lambda ins, out: g.relu(name + "_relu", ins[0], out), [y], name + "_act")

    def pool(name, x):
        return net.add(lambda ins, out: g._op("Pooling", name, ins, [out], "0=0 1=2 2=2 3=0 4=0"), [x], name)

    def res(name, x, c, first):
        h = conv("%s_%d" % (name, first), x, c, c, 1)
        h = conv("%s_%d" % (name, first + 1), h, c, c, 1)
        return net.add(lambda ins, out: g._op("Eltwise", "res%s_%d" % (name[4:], first + 1), ins, [out], "0=1 -23301=0"),
                       [x, h], "res%s_%d" % (name[4:], first + 1))

    x = net.add(lambda ins, out: g._op("Input", "data_norm", ins, [out], "0=128 1=128 2=3 3=104,117,123 4=0.0078125"),
                ["data"], "normed")
    x = conv("conv1a", x, 16, 3, 0)
    x = conv("conv1b", x, 32, 16, 0)
    x = pool("pool1b", x)
    x = res("conv2", x, 32, 1)
    cin = 32
    for stage, (cout, pairs) in enumerate(((64, 2), (128, 5), (256, 3)), start=2):
        x = conv("conv%d" % stage, x, cout, cin, 0)
        x = pool("pool%d" % stage, x)
        for k in range(pairs):
            x = res("conv%d" % (stage + 1), x, cout, 2 * k + 1)
        cin = cout
    x = conv("conv5", x, 256, 256, 0)
    w, b = init.conv(256, 1, 4)

    def emit_dw(ins, out):
        text = "0=256 1=4 2=1 3=1 4=0 5=1 6=4096 7=256"
        if act_scales is None:
            g._conv_weights(w, b, None)
        else:
            wq, ws = quantize_weights(w)
            g._conv_weights(w, b, (wq, ws, 1.0))
            text += " 8=1"
        g._op("ConvolutionDepthWise", "conv5_dw", ins, [out], text)
    net.add(emit_dw, [x], "conv5_dw")
    net.emit()
    return g, {"input": "data", "outputs": ["conv5_dw"], "conv_inputs": conv_inputs}


# ---- canonical, name-free form of a description -----------------------------------------------------
_CONV_TYPES = ("convolution", "convolutiondepthwise", "deconvolution")


def _canon_params(type_, params):
    def nums(v):
        return tuple(round(float(t), 6) for t in v.split(",") if t != "")
    p = {int(k): nums(v) for k, v in params.items()}
    p.pop(-23330, None)
    if type_ in _CONV_TYPES:
        one = lambda k, d: p.get(k, (float(d),))[0]
        kw, dil, sw, pl = one(1, 0), one(2, 1), one(3, 1), one(4, 0)
        return {"cout": one(0, 0), "kw": kw, "kh": one(11, kw), "dw": dil, "dh": one(12, dil), "sw": sw, "sh": one(13, sw),
                "pl": pl, "pt": one(14, pl), "pr": one(15, pl), "pb": one(16, pl), "bias": one(5, 0), "wsize": one(6, 0),
                "group": one(7, 1), "int8": float(one(8, 0) != 0), "act": one(9, 0)}
    if type_ == "pooling":
        one = lambda k, d: p.get(k, (float(d),))[0]
        kw, sw, pl = one(1, 0), one(2, 1), one(3, 0)
        return {"type": one(0, 0), "kw": kw, "kh": one(11, kw), "sw": sw, "sh": one(12, sw), "pl": pl, "pr": one(14, pl),
                "pt": one(13, pl), "pb": one(15, pl), "global": one(4, 0), "pad_mode": one(5, 1), "count_include_pad": one(6, 0)}
    if type_ == "batchnorm":
        p.setdefault(1, (0.0,))
    if type_ == "input":
        p.pop(0, None)      # nominal width / height: not part of the architecture
        p.pop(1, None)
    if type_ == "eltwise" and p.get(-23301) == (0.0,):
        p.pop(-23301)
    return p


def structure(phai_text):
    """[(type, canonical parameters, [(index of the producing op or -1, its output slot), ...])] over the ops
    of a description without its Split ops; indices count non-Split ops."""
    from .calibrate import parse_phai
    _, ops = parse_phai(phai_text)
    where = {}          # feature map -> (producer index, slot)
    out = []
    for op in ops:
        t = op["type"].lower()
        if t == "split":
            src = where.get(op["ins"][0], (-1, 0))
            for o in op["outs"]:
                where[o] = src
            continue
        ins = [where.get(n, (-1, 0)) for n in op["ins"]]
        if not op["ins"]:
            ins = [(-1, 0)]
        idx = len(out)
        for k, o in enumerate(op["outs"]):
            where[o] = (idx, k)
        out.append((t, _canon_params(t, op["params"]), ins))
    return out


# ---- a graph with seeded weights from a canonical structure ------------------------------------------
_CONV_KEYS = (("cout", 0), ("kw", 1), ("kh", 11), ("dw", 2), ("dh", 12), ("sw", 3), ("sh", 13), ("pl", 4), ("pt", 14),
              ("pr", 15), ("pb", 16), ("bias", 5), ("wsize", 6), ("group", 7), ("act", 9))
_POOL_KEYS = (("type", 0), ("kw", 1), ("kh", 11), ("sw", 2), ("sh", 12), ("pl", 3), ("pt", 13), ("pr", 14), ("pb", 15),
              ("global", 4), ("pad_mode", 5), ("count_include_pad", 6))
_TYPE_NAMES = {"convolution": "Convolution", "convolutiondepthwise": "ConvolutionDepthWise", "deconvolution": "Deconvolution",
               "pooling": "Pooling", "innerproduct": "InnerProduct", "batchnorm": "BatchNorm", "prelu": "PReLU",
               "leakyrelu": "LeakyRelu", "relu": "ReLU", "eltwise": "Eltwise", "binaryop": "BinaryOp", "input": "Input",
               "concat": "Concat", "interp": "Interp", "sigmoid": "Sigmoid", "hardswish": "HardSwish", "clip": "Clip",
               "reshape": "Reshape", "transpose": "Transpose", "yolov5focus": "YoloV5Focus", "hardsigmoid": "HardSigmoid",
               "softmax": "Softmax", "flatten": "Flatten"}


def _num(v):
    return repr(int(v)) if float(v) == int(v) else repr(float(v))


def graph_from_structure(struct, seed=21, name="net", gain=1.6):
    """GraphBuilder with the operation sequence of `struct` (the output of structure(), or its JSON round trip)
    and seeded weights: Kaiming-normal convolutions, near-identity BatchNorm statistics, PReLU slopes in
    [0.05, 0.3].  Feature maps are named t<op index>; a Split is inserted wherever a map has several readers.
    int8 flags are dropped (the graph is the floating-point one).  `gain` scales the convolution weights'
    variance (2 keeps the signal level through ReLU layers; residual and gated architectures need less).
    Returns (GraphBuilder, output names)."""
    g = GraphBuilder(name)
    net = _Net(g)
    init = _Init(seed)
    names = {}
    consumed = set()
    for idx, (t, prm, ins) in enumerate(struct):
        t = str(t)
        prm = {(int(k) if str(k).lstrip("-").isdigit() else str(k)): v for k, v in dict(prm).items()}
        srcs = ["data" if int(pi) < 0 else names[int(pi)] for pi, _ in ins]
        consumed.update(srcs)
        out = "t%d" % idx
        names[idx] = out
        opname = "%s_%d" % (t, idx)
        tname = _TYPE_NAMES[t]
        if t in _CONV_TYPES:
            text = " ".join("%d=%s" % (k, _num(prm[key])) for key, k in _CONV_KEYS)
            cout, kh, kw, group = int(prm["cout"]), int(prm["kh"]), int(prm["kw"]), int(prm["group"])
            wsize = int(prm["wsize"])
            per = wsize // (cout * kh * kw // group * group) * group if t != "convolutiondepthwise" else 1
            cin_g = wsize // (cout * kh * kw)
            if t == "deconvolution":
                w, b = init.deconv(wsize // (cout * kh * kw), cout, kh) if kh == kw else (None, None)
            else:
                w, b = init.conv(cout, cin_g, kh, kw, gain=gain)
            bias = b if int(prm["bias"]) else None

            def emit(ins_, out_, tname=tname, opname=opname, text=text, w=w, bias=bias):
                g._conv_weights(w, bias, None)
                g._op(tname, opname, ins_, [out_], text)
        elif t == "pooling":
            text = " ".join("%d=%s" % (k, _num(prm[key])) for key, k in _POOL_KEYS)

            def emit(ins_, out_, opname=opname, text=text):
                g._op("Pooling", opname, ins_, [out_], text)
        elif t == "innerproduct":
            nout, wsize = int(prm[0][0]), int(prm[2][0])
            r = init._r()
            w = (r.standard_normal((nout, wsize // nout)) * np.sqrt(1.0 / (wsize // nout))).astype(np.float32)
            bias = (r.standard_normal(nout) * 0.05).astype(np.float32) if int(prm.get(1, (0,))[0]) else None

            def emit(ins_, out_, opname=opname, w=w, bias=bias):
                g.innerproduct(opname, ins_[0], out_, w, bias)
        elif t == "batchnorm":
            bn = init.bn(int(prm[0][0]))
            eps = float(prm.get(1, (0.0,))[0])

            def emit(ins_, out_, opname=opname, bn=bn, eps=eps):
                g.batchnorm(opname, ins_[0], out_, *bn, eps=eps)
        elif t == "prelu":
            sl = init.slopes(int(prm[0][0]))

            def emit(ins_, out_, opname=opname, sl=sl):
                g.prelu(opname, ins_[0], out_, sl)
        else:
            text = " ".join("%d=%s" % (k, ",".join(_num(x) for x in v)) for k, v in prm.items())
            if t == "input":
                text = "0=%d 1=%d %s" % (int(prm.get("w", 0)), int(prm.get("h", 0)),
                                         " ".join("%d=%s" % (k, ",".join(_num(x) for x in v)) for k, v in prm.items()
                                                  if not isinstance(k, str)))

            def emit(ins_, out_, tname=tname, opname=opname, text=text):
                g._op(tname, opname, ins_, [out_], text)
        net.add(emit, srcs, out)
    net.emit()
    outs = [n for i, n in names.items() if n not in consumed]
    return g, outs


def architecture_input(arch, batch=1):
    """The seeded image batch (values 0..255) for one entry of the shipped-architecture fixture list."""
    h, w = arch["input_hw"]
    return np.random.default_rng(arch["seed"] + 1000).uniform(0, 255, (batch, 3, h, w)).astype(np.float32)


def sample(a, limit=8192):
    """Every k-th value of a flattened array, at most `limit` values (what the fixture keeps of a large map)."""
    flat = np.ascontiguousarray(a, np.float32).reshape(-1)
    step = max(1, -(-flat.size // limit))
    return flat[::step].copy()


def unsupported_types(phai_text):
    """Operation types of a description that this library has no implementation for (empty = every operation of
    the file can be created; shape-dependent refusals, e.g. a transposed convolution with overlapping taps,
    only show when the graph is built).  Needs no GPU."""
    from . import host
    from .calibrate import parse_phai
    _, ops = parse_phai(phai_text)
    return sorted({op["type"] for op in ops if not host.registered("operation_" + op["type"].lower())})


def main(argv=None):
    """python -m excalibur_b200.model_zoo file.phai ...: which operation types of each description are missing."""
    import sys
    for path in (argv if argv is not None else sys.argv[1:]):
        with open(path) as f:
            missing = unsupported_types(f.read())
        print("%-70s %s" % (path, "all operation types implemented" if not missing else "missing: " + ", ".join(missing)))


if __name__ == "__main__":
    main()
