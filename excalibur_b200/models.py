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


def resnet18(seed=2, act_scales=None, widths=RESNET18_WIDTHS, num_classes=1000, in_ch=3):
    """Returns (GraphBuilder, info).  act_scales: {conv name: fs} turns the named convs into int8
    convs (every conv except the stem must be present); None builds the floating-point graph.
    info["conv_inputs"] maps each quantisable conv to the feature map it reads (for calibration)."""
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

    x = conv("stem", "data", "stem_out", widths[0], in_ch, 7, 2, 3, 1, quant=False)
    x = g.pool("pool1", x, "pool1_out", 0, 3, 2, 1)
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
