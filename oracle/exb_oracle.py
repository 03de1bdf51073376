"""TEST INFRASTRUCTURE - NOT PRODUCT CODE.

numpy front-end of the plain-C oracle (oracle/exb_oracle.c).  Every function takes and
returns dense NCHW arrays like the reference's tensors; helpers at the bottom convert to
the NHWC layouts the CUDA kernels use.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

ACT_NONE, ACT_RELU, ACT_RELU6_QUIRK, ACT_SIGMOID, ACT_MISH = 0, 1, 3, 4, 5
ACT_RELU6, ACT_SILU = 103, 104


def build(force=False):
    """Compile oracle/exb_oracle.c into oracle/libexb_oracle.so (gcc, a second or two)."""
    so = os.path.join(_HERE, "libexb_oracle.so")
    src = os.path.join(_HERE, "exb_oracle.c")
    hdr = os.path.join(_HERE, "exb_oracle.h")
    if force or not os.path.exists(so) or os.path.getmtime(so) < max(os.path.getmtime(src), os.path.getmtime(hdr)):
        subprocess.check_call(["make", "-s", "-C", _HERE, "oracle"])
    return so


def lib():
    global _LIB
    if _LIB is None:
        _LIB = C.CDLL(build())
        _LIB.exbo_float32_to_int8.restype = C.c_int8
        _LIB.exbo_float32_to_int8.argtypes = [C.c_float]
        _LIB.exbo_conv_out_dim.restype = C.c_int
        _LIB.exbo_pool_out_dim.restype = C.c_int
    return _LIB


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _pads(pad):
    """pad: int or (top, bottom, left, right)."""
    if isinstance(pad, int):
        return pad, pad, pad, pad
    return tuple(pad)


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


def conv_out_dim(i, pa, pb, k, s):
    return (i + pa + pb - k) // s + 1


def conv2d_f32(x, w, bias=None, stride=1, pad=0, group=1, act=0):
    x, w = _f32(x), _f32(w)
    N, Cc, H, W = x.shape
    Cout, _, kh, kw = w.shape
    sh, sw = _pair(stride)
    pt, pb, pl, pr = _pads(pad)
    OH, OW = conv_out_dim(H, pt, pb, kh, sh), conv_out_dim(W, pl, pr, kw, sw)
    y = np.empty((N, Cout, OH, OW), np.float32)
    b = _f32(bias) if bias is not None else None
    lib().exbo_conv2d_f32(_p(x), _p(w), _p(b), _p(y), N, Cc, H, W, Cout, kh, kw, sh, sw,
                          pt, pb, pl, pr, group, act)
    return y


def float32_to_int8(v):
    return int(lib().exbo_float32_to_int8(float(v)))


def quantize_f32_i8(x, scales):
    x = _f32(x)
    N, Cc, H, W = x.shape
    s = _f32(np.atleast_1d(scales))
    q = np.empty(x.shape, np.int8)
    lib().exbo_quantize_f32_i8(_p(x), _p(q), N, Cc, H * W, _p(s), int(s.size))
    return q


def requantize_rne(v, scale):
    v = _f32(v)
    q = np.empty(v.shape, np.int8)
    lib().exbo_requantize_rne_f32_i8(_p(v), _p(q), C.c_int64(v.size), C.c_float(scale))
    return q


def conv2d_i8_acc(xq, wq, stride=1, pad=0, group=1):
    xq = np.ascontiguousarray(xq, np.int8)
    wq = np.ascontiguousarray(wq, np.int8)
    N, Cc, H, W = xq.shape
    Cout, _, kh, kw = wq.shape
    sh, sw = _pair(stride)
    pt, pb, pl, pr = _pads(pad)
    OH, OW = conv_out_dim(H, pt, pb, kh, sh), conv_out_dim(W, pl, pr, kw, sw)
    acc = np.empty((N, Cout, OH, OW), np.int32)
    lib().exbo_conv2d_i8_acc(_p(xq), _p(wq), _p(acc), N, Cc, H, W, Cout, kh, kw, sh, sw,
                             pt, pb, pl, pr, group)
    return acc


def dequant_scales(ws, fs, cout):
    ws, fs = _f32(np.atleast_1d(ws)), _f32(np.atleast_1d(fs))
    out = np.empty(cout, np.float32)
    lib().exbo_dequant_scales(_p(ws), int(ws.size), _p(fs), int(fs.size), _p(out), cout)
    return out


def dequantize(acc, scale, bias=None):
    acc = np.ascontiguousarray(acc, np.int32)
    N, Cc, H, W = acc.shape
    y = np.empty(acc.shape, np.float32)
    b = _f32(bias) if bias is not None else None
    lib().exbo_dequantize_i32_f32(_p(acc), _p(_f32(scale)), _p(b), _p(y), N, Cc, H * W)
    return y


def activation(y, act):
    y = _f32(y).copy()
    lib().exbo_activation_f32(_p(y), C.c_int64(y.size), act)
    return y


def conv2d_i8(x, wq, bias, ws, fs, stride=1, pad=0, group=1, act=0):
    x = _f32(x)
    wq = np.ascontiguousarray(wq, np.int8)
    N, Cc, H, W = x.shape
    Cout, _, kh, kw = wq.shape
    sh, sw = _pair(stride)
    pt, pb, pl, pr = _pads(pad)
    OH, OW = conv_out_dim(H, pt, pb, kh, sh), conv_out_dim(W, pl, pr, kw, sw)
    y = np.empty((N, Cout, OH, OW), np.float32)
    ws, fs = _f32(np.atleast_1d(ws)), _f32(np.atleast_1d(fs))
    b = _f32(bias) if bias is not None else None
    lib().exbo_conv2d_i8(_p(x), _p(wq), _p(b), _p(ws), int(ws.size), _p(fs), int(fs.size), _p(y),
                         N, Cc, H, W, Cout, kh, kw, sh, sw, pt, pb, pl, pr, group, act)
    return y


def dwconv2d_f32(x, w, bias=None, stride=1, pad=0, act=0):
    x, w = _f32(x), _f32(w)
    N, Cc, H, W = x.shape
    kh, kw = w.shape[-2:]
    sh, sw = _pair(stride)
    pt, pb, pl, pr = _pads(pad)
    OH, OW = conv_out_dim(H, pt, pb, kh, sh), conv_out_dim(W, pl, pr, kw, sw)
    y = np.empty((N, Cc, OH, OW), np.float32)
    b = _f32(bias) if bias is not None else None
    lib().exbo_dwconv2d_f32(_p(x), _p(w), _p(b), _p(y), N, Cc, H, W, kh, kw, sh, sw,
                            pt, pb, pl, pr, act)
    return y


def pool2d_f32(x, type=0, kernel=2, stride=2, pad=0, global_pool=False, pad_mode=1,
               count_include_pad=0):
    x = _f32(x)
    N, Cc, H, W = x.shape
    kh, kw = _pair(kernel)
    sh, sw = _pair(stride)
    pt, pb, pl, pr = _pads(pad)
    if global_pool:
        kh, kw, sh, sw, pt, pb, pl, pr = H, W, 1, 1, 0, 0, 0, 0
    PH = lib().exbo_pool_out_dim(H, pt, pb, kh, sh, pad_mode)
    PW = lib().exbo_pool_out_dim(W, pl, pr, kw, sw, pad_mode)
    y = np.empty((N, Cc, PH, PW), np.float32)
    lib().exbo_pool2d_f32(_p(x), _p(y), N, Cc, H, W, type, kh, kw, sh, sw, pt, pb, pl, pr,
                          int(global_pool), pad_mode, count_include_pad)
    return y


def eltwise_f32(xs, type=1, coeffs=None):
    xs = [_f32(a) for a in xs]
    arr = (C.c_void_p * len(xs))(*[a.ctypes.data for a in xs])
    cf = _f32(coeffs) if coeffs is not None else None
    y = np.empty(xs[0].shape, np.float32)
    lib().exbo_eltwise_f32(arr, len(xs), _p(cf), type, _p(y), C.c_int64(y.size))
    return y


def binaryop_f32(a, b, op=0):
    a, b = _f32(a), _f32(b)
    y = np.empty(a.shape, np.float32)
    lib().exbo_binaryop_f32(_p(a), _p(b), _p(y), C.c_int64(y.size), op)
    return y


def relu_f32(x):
    x = _f32(x)
    y = np.empty(x.shape, np.float32)
    lib().exbo_relu_f32(_p(x), _p(y), C.c_int64(y.size))
    return y


# ---- graph glue (pure index arithmetic, restated in numpy) -----------------------------
def concat_channels(xs):
    """Channel concat of NCHW arrays: src/Excalibur/operation_concat.cpp:84-110 (axis key -1)."""
    return np.concatenate([_f32(x) for x in xs], axis=1)


def interp_nearest(x, out_h, out_w):
    """Nearest resize, src/Excalibur/operation_interp.cpp:247-268: source index
    min((int)(o * (in / (float)out)), in - 1) with the ratio and the product in fp32."""
    x = _f32(x)
    H, W = x.shape[2], x.shape[3]
    hs = np.float32(H) / np.float32(out_h)
    ws = np.float32(W) / np.float32(out_w)
    iy = np.minimum((np.arange(out_h, dtype=np.float32) * hs).astype(np.int32), H - 1)
    ix = np.minimum((np.arange(out_w, dtype=np.float32) * ws).astype(np.int32), W - 1)
    return np.ascontiguousarray(x[:, :, iy][:, :, :, ix])


def batchnorm_coeffs(slope, mean, var, bias, eps=0.0):
    """(b, a) of y = b*x + a, src/Excalibur/operation_batchnorm.cpp:56-66: fp32 throughout,
    sqrt of (var + eps) rounded to fp32 before the divisions."""
    slope, mean, var, bias = (_f32(v) for v in (slope, mean, var, bias))
    sq = np.sqrt((var + np.float32(eps)).astype(np.float64)).astype(np.float32)
    return (slope / sq).astype(np.float32), (bias - slope * mean / sq).astype(np.float32)


def channel_affine(x, mul, add):
    """y[n][c] = x[n][c] * mul[c] + add[c] (src/Excalibur/operation_batchnorm.cpp:123-160)."""
    x = _f32(x)
    return (x * _f32(mul)[None, :, None, None] + _f32(add)[None, :, None, None]).astype(np.float32)


def hardswish(x, alpha=1.0 / 6.0, beta=0.5):
    """y = x * min(max(0, alpha*x + beta), 1): src/Excalibur/operation_hardswish.cpp:58-62 (the AVX
    body fuses alpha*x + beta into one fma; both forms are within 1 ulp of each other)."""
    x = _f32(x)
    t = (np.float32(alpha) * x + np.float32(beta)).astype(np.float32)
    return (x * np.minimum(np.maximum(t, np.float32(0)), np.float32(1))).astype(np.float32)


def input_norm(x, means, scales):
    """y = (x - means[c]) * scales[c]: src/Excalibur/operation_input.cpp:92-96."""
    x = _f32(x)
    m = _f32(means)[None, :, None, None]
    v = _f32(scales)[None, :, None, None]
    return ((x - m) * v).astype(np.float32)


def focus(x):
    """out[n][g*C + c][i][j] = in[n][c][2i + g%2][2j + g/2]: src/Excalibur/operation_yolov5focus.cpp:27-41
    (applied to every image; the reference only fills image 0)."""
    x = _f32(x)
    n, c, h, w = x.shape
    out = np.empty((n, 4 * c, h // 2, w // 2), np.float32)
    for g in range(4):
        out[:, g * c:(g + 1) * c] = x[:, :, (g % 2):(h // 2) * 2:2, (g // 2):(w // 2) * 2:2]
    return out


def prelu(x, slopes):
    """y = x >= 0 ? x : slope[c] * x, one shared slope when len(slopes) == 1
    (src/Excalibur/operation_prelu.cpp:58-147)."""
    x = _f32(x)
    sl = _f32(slopes).reshape(-1)
    sl = np.float32(sl[0]) if sl.size == 1 else sl[None, :, None, None]
    return np.where(x >= 0, x, (x * sl).astype(np.float32)).astype(np.float32)


def leakyrelu(x, alpha):
    """y = x < 0 ? alpha * x : x (src/Excalibur/operation_leakyrelu.cpp:31-58)."""
    x = _f32(x)
    return np.where(x < 0, (x * np.float32(alpha)).astype(np.float32), x).astype(np.float32)


def deconv2d_f32(x, w, bias=None, stride=1, pad=0):
    """Transposed convolution, weights [Cin][Cout][kh][kw], one group:
    out[n][co][ih*s + a - pad][iw*s + b - pad] += sum_ci w[ci][co][a][b] * x[n][ci][ih][iw], output
    (H - 1)*s + k - 2*pad (src/Excalibur/operation_deconvolution.cpp:83-150: GEMM into a column buffer, col2im
    scatter-add, bias GEMM).  Accumulated in fp32 per tap, then scattered."""
    x = _f32(x)
    w = _f32(w)
    n, cin, h, wd = x.shape
    _, cout, kh, kw = w.shape
    sh, sw = _pair(stride)
    ph, pw = _pair(pad)
    oh, ow = (h - 1) * sh + kh - 2 * ph, (wd - 1) * sw + kw - 2 * pw
    full = np.zeros((n, cout, (h - 1) * sh + kh, (wd - 1) * sw + kw), np.float32)
    for a in range(kh):
        for b in range(kw):
            col = np.einsum("nchw,cd->ndhw", x, w[:, :, a, b]).astype(np.float32)
            full[:, :, a:a + (h - 1) * sh + 1:sh, b:b + (wd - 1) * sw + 1:sw] += col
    out = full[:, :, ph:ph + oh, pw:pw + ow]
    if bias is not None:
        out = out + _f32(bias)[None, :, None, None]
    return np.ascontiguousarray(out, np.float32)


def hardsigmoid(x, alpha, beta):
    """y = max(0, min(1, alpha*x + beta)) (src/Excalibur/operation_hardsigmoid.cpp:42-45)."""
    x = _f32(x)
    t = (np.float32(alpha) * x + np.float32(beta)).astype(np.float32)
    return np.maximum(np.float32(0), np.minimum(np.float32(1), t)).astype(np.float32)


def softmax_channels(x):
    """Softmax over the channels of every position of an NCHW tensor: subtract the channel maximum, exp,
    divide by the channel sum (src/Excalibur/operation_softmax.cpp:62-96)."""
    x = _f32(x)
    e = np.exp((x - x.max(axis=1, keepdims=True)).astype(np.float32)).astype(np.float32)
    return (e / e.sum(axis=1, keepdims=True, dtype=np.float32)).astype(np.float32)


def flatten_nchw(x, axis=1):
    """Same values, shape {n, 1, h, w} with (h, w) = (chw, 1), (ch, w), (c, hw), (1, chw) for axis 0..3
    (src/Excalibur/operation_flatten.cpp:33-63)."""
    x = _f32(x)
    n, c, h, w = x.shape
    hw = {0: (c * h * w, 1), 1: (c * h, w), 2: (c, h * w), 3: (1, c * h * w)}[axis]
    return np.ascontiguousarray(x).reshape((n, 1) + hw)


def reshape_nchw(x, w=0, h=0, c=0):
    """New shape over the same NCHW bytes: a positive key replaces the axis, 0 keeps it, -1 deduces it; n is
    kept (src/Excalibur/operation_reshape.cpp:48-84)."""
    x = _f32(x)
    s = list(x.shape)
    for axis, v in ((1, c), (2, h), (3, w)):
        if v > 0:
            s[axis] = v
    for axis, v in ((1, c), (2, h), (3, w)):
        if v < 0:
            rest = int(np.prod([s[a] for a in range(4) if a != axis]))
            s[axis] = x.size // rest
    return np.ascontiguousarray(x).reshape(s)


def transpose_hw(x):
    """out[n][c][w][h] = in[n][c][h][w]: Transpose with permutation 1,0,2
    (src/Excalibur/operation_transpose.cpp:47-66)."""
    return np.ascontiguousarray(np.swapaxes(_f32(x), 2, 3))


# ---- layout helpers -------------------------------------------------------------------
def nchw_to_nhwc(a):
    return np.ascontiguousarray(np.transpose(a, (0, 2, 3, 1)))


def nhwc_to_nchw(a):
    return np.ascontiguousarray(np.transpose(a, (0, 3, 1, 2)))
