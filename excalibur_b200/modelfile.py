"""Writers for the two model-file formats of the reference library.

* ``.phai``: text network description, one op per line,
  ``<Type> <name> <n_in> <n_out> <in names...> <out names...> <k=v ...>``
  (reference src/Excalibur/pipeline.cpp:54-116).
* ``.racy``: headerless little-endian weight blob read sequentially by every op's
  ``init_weights(FILE*)`` in file order (reference src/Excalibur/operation_convolution.cpp:71-152,
  src/Excalibur/operation_innerproduct.cpp:77-120).

`GraphBuilder` emits both at once so that the reference CPU library and this package's C++
pipeline load byte-identical graphs and weights.
"""
import struct

import numpy as np

RACY_TAG_F32 = 0
RACY_TAG_I8 = 871224


class GraphBuilder:
    def __init__(self, name="net"):
        self.name = name
        self.lines = []
        self.blob = bytearray()
        self.featmaps = set()

    # -- plumbing -----------------------------------------------------------------------
    def _op(self, type_, name, ins, outs, params=""):
        self.featmaps.update(ins)
        self.featmaps.update(outs)
        toks = [type_, name, str(len(ins)), str(len(outs))] + list(ins) + list(outs)
        if params:
            toks.append(params)
        self.lines.append(" ".join(toks))
        return outs[0] if len(outs) == 1 else outs

    def phai_text(self):
        head = ["glsv1 " + self.name, "%d %d" % (len(self.lines), len(self.featmaps))]
        return "\n".join(head + self.lines) + "\n"

    def racy_bytes(self):
        return bytes(self.blob)

    def save(self, phai_path, racy_path):
        with open(phai_path, "w") as f:
            f.write(self.phai_text())
        with open(racy_path, "wb") as f:
            f.write(self.racy_bytes())

    # -- ops ----------------------------------------------------------------------------
    def _conv_params(self, cout, kh, kw, stride, pad, bias, wsize, group, act, int8):
        sh, sw = (stride, stride) if isinstance(stride, int) else stride
        pt, pb, pl, pr = (pad,) * 4 if isinstance(pad, int) else pad
        p = "0=%d 1=%d 11=%d 2=1 12=1 3=%d 13=%d 4=%d 14=%d 15=%d 16=%d 5=%d 6=%d" % (
            cout, kw, kh, sw, sh, pl, pt, pr, pb, int(bias), wsize)
        if group != 1:
            p += " 7=%d" % group
        if int8:
            p += " 8=1"
        if act:
            p += " 9=%d" % act
        return p

    def _conv_weights(self, w, bias, int8):
        if int8 is None:
            self.blob += struct.pack("<i", RACY_TAG_F32)
            self.blob += np.ascontiguousarray(w, "<f4").tobytes()
            if bias is not None:
                self.blob += np.ascontiguousarray(bias, "<f4").tobytes()
        else:
            wq, ws, fs = int8
            raw = np.ascontiguousarray(wq, np.int8).tobytes()
            raw += b"\0" * ((-len(raw)) % 4)
            self.blob += struct.pack("<i", RACY_TAG_I8) + raw
            if bias is not None:
                self.blob += np.ascontiguousarray(bias, "<f4").tobytes()
            self.blob += np.ascontiguousarray(ws, "<f4").tobytes()
            self.blob += struct.pack("<f", float(fs))

    def conv(self, name, x, y, w, bias=None, stride=1, pad=0, act=0, group=1, int8=None,
             type_="Convolution"):
        """w: OIHW fp32 (ignored for the blob when int8=(wq, weight_scales[Cout], act_scale))."""
        cout, _, kh, kw = (w if int8 is None else int8[0]).shape
        wsize = int(np.prod((w if int8 is None else int8[0]).shape))
        self._conv_weights(w, bias, int8)
        return self._op(type_, name, [x], [y],
                        self._conv_params(cout, kh, kw, stride, pad, bias is not None, wsize,
                                          group, act, int8 is not None))

    def dwconv(self, name, x, y, w, bias=None, stride=1, pad=0, act=0):
        return self.conv(name, x, y, w, bias, stride, pad, act, group=w.shape[0],
                         type_="ConvolutionDepthWise")

    def pool(self, name, x, y, type_=0, kernel=2, stride=2, pad=0, global_pool=False,
             pad_mode=1, count_include_pad=None):
        p = "0=%d 1=%d 2=%d 3=%d 4=%d 5=%d" % (type_, kernel, stride, pad, int(global_pool), pad_mode)
        if count_include_pad is not None:
            p += " 6=%d" % count_include_pad
        return self._op("Pooling", name, [x], [y], p)

    def eltwise(self, name, xs, y, type_=1, coeffs=None):
        p = "0=%d" % type_
        if coeffs is not None:
            p += " -23301=%d,%s" % (len(coeffs) + 1, ",".join(repr(float(c)) for c in coeffs))
        return self._op("Eltwise", name, list(xs), [y], p)

    def binaryop(self, name, a, b, y, op=0):
        return self._op("BinaryOp", name, [a, b], [y], "0=%d" % op)

    def relu(self, name, x, y):
        return self._op("ReLU", name, [x], [y])

    def relu6(self, name, x, y):
        """The reference's ReLU6 operation: 0 outside [0, 6] (values above 6 become 0, not 6)."""
        return self._op("ReLU6", name, [x], [y])

    def clip(self, name, x, y, lo, hi):
        return self._op("Clip", name, [x], [y], "0=%r 1=%r" % (float(lo), float(hi)))

    def sigmoid(self, name, x, y):
        return self._op("Sigmoid", name, [x], [y])

    def hardswish(self, name, x, y, alpha=1.0 / 6.0, beta=0.5):
        return self._op("HardSwish", name, [x], [y], "0=%r 1=%r" % (float(alpha), float(beta)))

    def input_norm(self, name, x, y, w, h, means, scales):
        """y = (x - means[c]) * scales[c] (the reference calls the multipliers 'vars')."""
        return self._op("Input", name, [x], [y], "0=%d 1=%d 2=%d 3=%s 4=%s" % (
            w, h, len(means), ",".join(repr(float(m)) for m in means), ",".join(repr(float(v)) for v in scales)))

    def focus(self, name, x, y):
        return self._op("YoloV5Focus", name, [x], [y])

    def split(self, name, x, outs):
        return self._op("Split", name, [x], list(outs))

    def concat(self, name, xs, y, axis=-1):
        return self._op("Concat", name, list(xs), [y], "0=%d" % axis)

    def interp_nearest(self, name, x, y, scale=2.0):
        return self._op("Interp", name, [x], [y], "0=1 1=%r 2=%r" % (float(scale), float(scale)))

    def batchnorm(self, name, x, y, slope, mean, var, bias, eps=0.0):
        """Weights in file order slope, mean, var, bias, no quantize tag."""
        for v in (slope, mean, var, bias):
            self.blob += np.ascontiguousarray(v, "<f4").tobytes()
        return self._op("BatchNorm", name, [x], [y], "0=%d 1=%r" % (len(slope), float(eps)))

    def prelu(self, name, x, y, slopes):
        """Weights: the slopes, no quantize tag (1 slope = shared by every channel)."""
        self.blob += np.ascontiguousarray(slopes, "<f4").tobytes()
        return self._op("PReLU", name, [x], [y], "0=%d" % len(slopes))

    def leakyrelu(self, name, x, y, alpha):
        return self._op("LeakyRelu", name, [x], [y], "0=%r" % float(alpha))

    def deconv(self, name, x, y, w, bias=None, stride=1, pad=0):
        """w: [Cin][Cout][kh][kw] fp32 (the transposed-convolution layout of the reference)."""
        _, cout, kh, kw = w.shape
        self._conv_weights(w, bias, None)
        return self._op("Deconvolution", name, [x], [y],
                        self._conv_params(cout, kh, kw, stride, pad, bias is not None, int(w.size), 1, 0, False) + " 7=1")

    def reshape(self, name, x, y, w=0, h=0, c=0):
        return self._op("Reshape", name, [x], [y], "0=%d 1=%d 2=%d" % (w, h, c))

    def transpose(self, name, x, y, perm=(1, 0, 2)):
        return self._op("Transpose", name, [x], [y], "0=" + ",".join(str(int(v)) for v in perm))

    def innerproduct(self, name, x, y, w, bias=None):
        """w: [out][in] fp32."""
        self.blob += struct.pack("<i", RACY_TAG_F32)
        self.blob += np.ascontiguousarray(w, "<f4").tobytes()
        if bias is not None:
            self.blob += np.ascontiguousarray(bias, "<f4").tobytes()
        return self._op("InnerProduct", name, [x], [y],
                        "0=%d 1=%d 2=%d" % (w.shape[0], int(bias is not None), w.size))
