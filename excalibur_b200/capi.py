"""ctypes binding of the C ABI (include/excalibur_b200.h) plus thin helpers that take torch
tensors for device memory.  torch is plumbing here (allocation, streams); every computation
goes through libexcalibur_b200.so, and importing this module fails loudly if the library has
not been built.
"""
import ctypes as C
import os

import numpy as np

_PKG = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.path.join(_PKG, "lib", "libexcalibur_b200.so")

EXB_OK, EXB_ERR_BAD_ARG, EXB_ERR_UNSUPPORTED, EXB_ERR_CUDA, EXB_ERR_TIMEOUT, EXB_ERR_NOMEM = 0, -1, -2, -3, -4, -5
EXB_F16, EXB_I8, EXB_F32, EXB_I32 = 0, 1, 2, 3
ACT_NONE, ACT_RELU, ACT_RELU6_QUIRK, ACT_SIGMOID, ACT_MISH, ACT_RELU6, ACT_SILU, ACT_HARDSWISH, ACT_PRELU = 0, 1, 3, 4, 5, 103, 104, 105, 106

EXPORTED_SYMBOLS = [
    "exb_ctx_create", "exb_ctx_destroy", "exb_last_error_string", "exb_version", "exb_ctx_sm_count",
    "exb_ctx_sync_check", "exb_selftest_bounded_wait", "exb_tensor_peak_probe", "exb_tensor_peak_probe_layout", "exb_nchw_f32_to_nhwc", "exb_nchw_f32_to_nhwc_padded", "exb_nhwc_to_nchw_f32", "exb_conv_out_dims",
    "exb_conv_weights_pack_f16", "exb_conv_weights_pack_i8", "exb_conv_weights_destroy",
    "exb_conv2d_fwd", "exb_conv2d_uses_tensor_cores", "exb_conv2d_pool_fusable", "exb_dw_weights_pack", "exb_dw_weights_destroy",
    "exb_dwconv2d_fwd", "exb_pool_out_dims", "exb_pool2d_fwd", "exb_pool2d_nchw_f32_static", "exb_eltwise_fwd", "exb_binaryop_fwd",
    "exb_binaryop_scalar_fwd", "exb_relu_fwd", "exb_activation_fwd", "exb_quantize_fwd",
    "exb_dequantize_fwd", "exb_concat_fwd", "exb_interp_nearest_fwd", "exb_channel_affine_fwd",
    "exb_conv_weights_set_slopes", "exb_dw_weights_set_slopes", "exb_depth_to_space_nchw_f32", "exb_image_f32_to_nhwc_norm", "exb_nchw_f32_to_nhwc4_padded_norm", "exb_nhwc_f16_split_heads_f32", "exb_hardsigmoid_fwd", "exb_softmax_channels_f32", "exb_binaryop_channel_bcast_fwd", "exb_nchw_f16_to_nhwc4_padded", "exb_nchw_f32_focus_to_nhwc_f16", "exb_channel_affine_prelu_fwd", "exb_hardswish_fwd", "exb_focus_fwd", "exb_prelu_fwd", "exb_depth_to_space_fwd", "exb_transpose_hw_f32",
]


class ConvDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "N", "H", "W", "Cin", "Cout", "cin_stride", "cout_stride", "kh", "kw", "stride_h", "stride_w",
        "pad_t", "pad_b", "pad_l", "pad_r", "dilation", "group", "in_dtype", "out_dtype", "out2_dtype",
        "res_dtype", "act")] + [("out_scale", C.c_float), ("out2_scale", C.c_float), ("impl", C.c_int32),
                                      ("x_w_pitch", C.c_int32), ("x_w_pad", C.c_int32), ("fuse_pool", C.c_int32),
                                      ("y_pitch", C.c_int32)]


class DwConvDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "N", "H", "W", "C", "c_stride", "kh", "kw", "stride_h", "stride_w", "pad_t", "pad_b", "pad_l",
        "pad_r", "in_dtype", "out_dtype", "act")] + [("in_scale", C.c_float), ("out_scale", C.c_float)]


class PoolDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "N", "H", "W", "C", "c_stride", "type", "kh", "kw", "stride_h", "stride_w", "pad_t", "pad_b",
        "pad_l", "pad_r", "global_pool", "pad_mode", "count_include_pad", "dtype", "out2_dtype")] + \
        [("out2_scale", C.c_float)]


class ExbError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__("excalibur_b200 error %d: %s" % (code, msg))
        self.code = code


_LIB = None


def lib():
    """Load the shared library (raises if it has not been built: there is no fallback)."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(SO_PATH):
            raise ImportError("%s is missing: run `python -m excalibur_b200.build`" % SO_PATH)
        L = C.CDLL(SO_PATH)
        L.exb_last_error_string.restype = C.c_char_p
        L.exb_version.restype = C.c_char_p
        vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_int64, C.c_float
        L.exb_ctx_create.argtypes = [i32, C.POINTER(vp)]
        L.exb_ctx_destroy.argtypes = [vp]
        L.exb_ctx_sm_count.argtypes = [vp, C.POINTER(i32)]
        L.exb_ctx_sync_check.argtypes = [vp, vp]
        L.exb_selftest_bounded_wait.argtypes = [vp, i32, vp]
        L.exb_tensor_peak_probe.argtypes = [vp, i32, i32, i32, i32, i32, C.POINTER(C.c_double), vp, vp]
        L.exb_tensor_peak_probe_layout.argtypes = [vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, C.POINTER(C.c_double), vp, vp]
        L.exb_nchw_f32_to_nhwc.argtypes = [vp, vp, vp, i32, i32, i32, i32, i32, i32, f32, i32, vp]
        L.exb_nchw_f32_to_nhwc_padded.argtypes = [vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, f32, i32, vp]
        L.exb_nhwc_to_nchw_f32.argtypes = [vp, vp, i32, vp, i32, i32, i32, i32, i32, f32, vp]
        L.exb_conv_out_dims.argtypes = [C.POINTER(ConvDesc), C.POINTER(i32), C.POINTER(i32)]
        L.exb_conv2d_uses_tensor_cores.argtypes = [C.POINTER(ConvDesc)]
        L.exb_conv2d_pool_fusable.argtypes = [C.POINTER(ConvDesc)]
        L.exb_conv_weights_pack_f16.argtypes = [vp, C.POINTER(ConvDesc), vp, vp, C.POINTER(vp)]
        L.exb_conv_weights_pack_i8.argtypes = [vp, C.POINTER(ConvDesc), vp, vp, vp, i32, f32, C.POINTER(vp)]
        L.exb_conv_weights_destroy.argtypes = [vp]
        L.exb_conv2d_fwd.argtypes = [vp, C.POINTER(ConvDesc), vp, vp, vp, vp, vp, vp]
        L.exb_dw_weights_pack.argtypes = [vp, C.POINTER(DwConvDesc), vp, vp, C.POINTER(vp)]
        L.exb_dw_weights_destroy.argtypes = [vp]
        L.exb_dwconv2d_fwd.argtypes = [vp, C.POINTER(DwConvDesc), vp, vp, vp, vp]
        L.exb_pool_out_dims.argtypes = [C.POINTER(PoolDesc), C.POINTER(i32), C.POINTER(i32)]
        L.exb_pool2d_fwd.argtypes = [vp, C.POINTER(PoolDesc), vp, vp, vp, vp]
        L.exb_pool2d_nchw_f32_static.argtypes = [i32, C.POINTER(PoolDesc), vp, vp, vp]
        L.exb_eltwise_fwd.argtypes = [vp, i32, i32, C.POINTER(vp), C.POINTER(f32), vp, i64, i32, vp]
        L.exb_binaryop_fwd.argtypes = [vp, i32, vp, vp, vp, i64, i32, vp]
        L.exb_binaryop_scalar_fwd.argtypes = [vp, i32, vp, f32, vp, i64, i32, vp]
        L.exb_relu_fwd.argtypes = [vp, vp, vp, i64, i32, vp]
        L.exb_activation_fwd.argtypes = [vp, i32, vp, vp, i64, i32, vp]
        L.exb_quantize_fwd.argtypes = [vp, vp, i32, vp, i64, f32, i32, vp]
        L.exb_dequantize_fwd.argtypes = [vp, vp, vp, i32, i64, f32, vp]
        L.exb_concat_fwd.argtypes = [vp, i32, C.POINTER(vp), C.POINTER(i64), C.POINTER(i64), vp, i64, i64, i32, vp]
        L.exb_interp_nearest_fwd.argtypes = [vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp]
        L.exb_channel_affine_fwd.argtypes = [vp, vp, vp, vp, vp, i64, i32, i32, i64, i32, i32, i32, vp]
        L.exb_hardswish_fwd.argtypes = [vp, vp, vp, i64, i32, f32, f32, vp]
        L.exb_focus_fwd.argtypes = [vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, vp]
        L.exb_conv_weights_set_slopes.argtypes = [vp, vp, vp, i32]
        L.exb_dw_weights_set_slopes.argtypes = [vp, vp, vp, i32]
        L.exb_channel_affine_prelu_fwd.argtypes = [vp, vp, vp, vp, vp, vp, i32, i64, i32, i32, i64, i32, i32, vp]
        L.exb_nchw_f32_focus_to_nhwc_f16.argtypes = [vp, vp, vp, i32, i32, i32, i32, i32, vp, vp, vp]
        L.exb_binaryop_channel_bcast_fwd.argtypes = [vp, i32, vp, vp, i32, vp, i32, i32, i32, i32, i64, i32, i32, vp]
        L.exb_hardsigmoid_fwd.argtypes = [vp, vp, vp, i64, i32, f32, f32, vp]
        L.exb_softmax_channels_f32.argtypes = [vp, vp, vp, i32, i32, i64, i64, vp]
        L.exb_nchw_f16_to_nhwc4_padded.argtypes = [vp, vp, vp, i32, i32, i32, i32, i32, i32, vp]
        L.exb_nhwc_f16_split_heads_f32.argtypes = [vp, vp, vp, i32, i32, i32, i32, i32, vp]
        L.exb_image_f32_to_nhwc_norm.argtypes = [vp, vp, vp, i32, i32, i32, i32, i32, i32, vp, vp, f32, i32, vp]
        L.exb_nchw_f32_to_nhwc4_padded_norm.argtypes = [vp, vp, vp, i32, i32, i32, i32, i32, i32, vp, vp, vp]
        L.exb_prelu_fwd.argtypes = [vp, vp, vp, vp, i32, i64, i32, i32, i64, i32, i32, vp]
        L.exb_depth_to_space_fwd.argtypes = [vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp]
        L.exb_transpose_hw_f32.argtypes = [vp, vp, vp, i64, i32, i32, vp]
        _LIB = L
    return _LIB


def check(rc):
    if rc != 0:
        raise ExbError(rc, lib().exb_last_error_string().decode())


def last_error():
    return lib().exb_last_error_string().decode()


# ---- torch plumbing ---------------------------------------------------------------------------
def _torch():
    import torch
    return torch


def torch_dtype(dt):
    t = _torch()
    return {EXB_F16: t.float16, EXB_I8: t.int8, EXB_F32: t.float32, EXB_I32: t.int32}[dt]


def exb_dtype_of(tensor):
    t = _torch()
    return {t.float16: EXB_F16, t.int8: EXB_I8, t.float32: EXB_F32, t.int32: EXB_I32}[tensor.dtype]


def ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def cur_stream():
    return C.c_void_p(_torch().cuda.current_stream().cuda_stream)


def _np_ptr(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


class Context:
    """exb_ctx for one device."""

    def __init__(self, device=0):
        self._h = C.c_void_p()
        self.device = device
        check(lib().exb_ctx_create(device, C.byref(self._h)))

    @property
    def handle(self):
        return self._h

    def sm_count(self):
        n = C.c_int()
        check(lib().exb_ctx_sm_count(self._h, C.byref(n)))
        return n.value

    def sync_check(self):
        check(lib().exb_ctx_sync_check(self._h, cur_stream()))

    def close(self):
        if self._h:
            lib().exb_ctx_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def make_conv_desc(N, H, W, Cin, Cout, k, stride=1, pad=0, in_dtype=EXB_F16, out_dtype=EXB_F16,
                   out2_dtype=-1, res=False, act=ACT_NONE, out_scale=1.0, out2_scale=1.0,
                   cin_stride=0, cout_stride=0, group=1, impl=0, x_w_pitch=0, x_w_pad=0, fuse_pool=0,
                   y_pitch=0):
    kh, kw = (k, k) if isinstance(k, int) else k
    sh, sw = (stride, stride) if isinstance(stride, int) else stride
    pt, pb, pl, pr = (pad,) * 4 if isinstance(pad, int) else pad
    return ConvDesc(N, H, W, Cin, Cout, cin_stride, cout_stride, kh, kw, sh, sw, pt, pb, pl, pr, 1, group,
                    in_dtype, out_dtype, out2_dtype, EXB_F16 if res else -1, act, out_scale, out2_scale, impl, x_w_pitch, x_w_pad, fuse_pool,
                    y_pitch)


class ConvWeights:
    """Packed device-resident convolution weights (exb_conv_weights)."""

    def __init__(self, ctx, desc, w_oihw, bias=None, wscale=None, act_scale=None):
        self._h = C.c_void_p()
        bias = None if bias is None else np.ascontiguousarray(bias, np.float32)
        if desc.in_dtype == EXB_I8:
            w = np.ascontiguousarray(w_oihw, np.int8)
            ws = np.ascontiguousarray(np.atleast_1d(wscale), np.float32)
            check(lib().exb_conv_weights_pack_i8(ctx.handle, C.byref(desc), _np_ptr(w), _np_ptr(bias),
                                                 _np_ptr(ws), int(ws.size), float(act_scale), C.byref(self._h)))
        else:
            w = np.ascontiguousarray(w_oihw, np.float32)
            check(lib().exb_conv_weights_pack_f16(ctx.handle, C.byref(desc), _np_ptr(w), _np_ptr(bias),
                                                  C.byref(self._h)))

    @property
    def handle(self):
        return self._h

    def set_slopes(self, ctx, slopes):
        """Per-output-channel (or one shared) PReLU slope for act == ACT_PRELU."""
        sl = np.ascontiguousarray(np.atleast_1d(slopes), np.float32)
        check(lib().exb_conv_weights_set_slopes(ctx.handle, self._h, _np_ptr(sl), int(sl.size)))

    def close(self):
        if self._h:
            lib().exb_conv_weights_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def conv_out_dims(desc):
    oh, ow = C.c_int(), C.c_int()
    check(lib().exb_conv_out_dims(C.byref(desc), C.byref(oh), C.byref(ow)))
    return oh.value, ow.value


def conv2d(ctx, desc, x, weights, residual=None, y=None, y2=None):
    """x: NHWC torch tensor on the context's device.  Returns (y, y2)."""
    t = _torch()
    oh, ow = conv_out_dims(desc)
    cs = desc.cout_stride or desc.Cout
    if y is None:
        y = t.empty((desc.N, oh, ow, cs), dtype=torch_dtype(desc.out_dtype), device=x.device)
    if desc.out2_dtype != -1 and y2 is None:
        y2 = t.empty((desc.N, oh, ow, cs), dtype=torch_dtype(desc.out2_dtype), device=x.device)
    check(lib().exb_conv2d_fwd(ctx.handle, C.byref(desc), ptr(x), weights.handle, ptr(residual), ptr(y),
                               ptr(y2), cur_stream()))
    return y, y2


class DwWeights:
    def __init__(self, ctx, desc, w, bias=None):
        self._h = C.c_void_p()
        w = np.ascontiguousarray(w, np.float32)
        bias = None if bias is None else np.ascontiguousarray(bias, np.float32)
        check(lib().exb_dw_weights_pack(ctx.handle, C.byref(desc), _np_ptr(w), _np_ptr(bias), C.byref(self._h)))

    @property
    def handle(self):
        return self._h

    def set_slopes(self, ctx, slopes):
        sl = np.ascontiguousarray(np.atleast_1d(slopes), np.float32)
        check(lib().exb_dw_weights_set_slopes(ctx.handle, self._h, _np_ptr(sl), int(sl.size)))

    def close(self):
        if self._h:
            lib().exb_dw_weights_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def make_dw_desc(N, H, W, Cc, k=3, stride=1, pad=1, in_dtype=EXB_F16, out_dtype=EXB_F16, act=ACT_NONE,
                 in_scale=1.0, out_scale=1.0, c_stride=0):
    kh, kw = (k, k) if isinstance(k, int) else k
    sh, sw = (stride, stride) if isinstance(stride, int) else stride
    pt, pb, pl, pr = (pad,) * 4 if isinstance(pad, int) else pad
    return DwConvDesc(N, H, W, Cc, c_stride, kh, kw, sh, sw, pt, pb, pl, pr, in_dtype, out_dtype, act,
                      in_scale, out_scale)


def dwconv2d(ctx, desc, x, weights, y=None):
    t = _torch()
    oh = (desc.H + desc.pad_t + desc.pad_b - desc.kh) // desc.stride_h + 1
    ow = (desc.W + desc.pad_l + desc.pad_r - desc.kw) // desc.stride_w + 1
    cs = desc.c_stride or desc.C
    if y is None:
        y = t.empty((desc.N, oh, ow, cs), dtype=torch_dtype(desc.out_dtype), device=x.device)
    check(lib().exb_dwconv2d_fwd(ctx.handle, C.byref(desc), ptr(x), weights.handle, ptr(y), cur_stream()))
    return y


def make_pool_desc(N, H, W, Cc, type=0, k=2, stride=2, pad=0, global_pool=False, pad_mode=1,
                   count_include_pad=0, dtype=EXB_F16, out2_dtype=-1, out2_scale=1.0, c_stride=0):
    kh, kw = (k, k) if isinstance(k, int) else k
    sh, sw = (stride, stride) if isinstance(stride, int) else stride
    pt, pb, pl, pr = (pad,) * 4 if isinstance(pad, int) else pad
    return PoolDesc(N, H, W, Cc, c_stride, type, kh, kw, sh, sw, pt, pb, pl, pr, int(global_pool), pad_mode,
                    count_include_pad, dtype, out2_dtype, out2_scale)


def pool_out_dims(desc):
    ph, pw = C.c_int(), C.c_int()
    check(lib().exb_pool_out_dims(C.byref(desc), C.byref(ph), C.byref(pw)))
    return ph.value, pw.value


def pool2d(ctx, desc, x, y=None, y2=None):
    t = _torch()
    ph, pw = pool_out_dims(desc)
    cs = desc.c_stride or desc.C
    if y is None:
        y = t.empty((desc.N, ph, pw, cs), dtype=x.dtype, device=x.device)
    if desc.out2_dtype != -1 and y2 is None:
        y2 = t.empty((desc.N, ph, pw, cs), dtype=t.int8, device=x.device)
    check(lib().exb_pool2d_fwd(ctx.handle, C.byref(desc), ptr(x), ptr(y), ptr(y2), cur_stream()))
    return y, y2


def eltwise(ctx, xs, type=1, coeffs=None, y=None):
    t = _torch()
    if y is None:
        y = t.empty_like(xs[0])
    arr = (C.c_void_p * len(xs))(*[x.data_ptr() for x in xs])
    cf = None if coeffs is None else (C.c_float * len(xs))(*[float(c) for c in coeffs])
    check(lib().exb_eltwise_fwd(ctx.handle, type, len(xs), arr, cf, ptr(y), xs[0].numel(), exb_dtype_of(xs[0]),
                                cur_stream()))
    return y


def binaryop(ctx, a, b, op=0, y=None):
    t = _torch()
    if y is None:
        y = t.empty_like(a)
    check(lib().exb_binaryop_fwd(ctx.handle, op, ptr(a), ptr(b), ptr(y), a.numel(), exb_dtype_of(a), cur_stream()))
    return y


def binaryop_scalar(ctx, a, scalar, op=0, y=None):
    t = _torch()
    if y is None:
        y = t.empty_like(a)
    check(lib().exb_binaryop_scalar_fwd(ctx.handle, op, ptr(a), float(scalar), ptr(y), a.numel(), exb_dtype_of(a),
                                        cur_stream()))
    return y


def relu(ctx, x, y=None):
    t = _torch()
    if y is None:
        y = t.empty_like(x)
    check(lib().exb_relu_fwd(ctx.handle, ptr(x), ptr(y), x.numel(), exb_dtype_of(x), cur_stream()))
    return y


def activation(ctx, x, act, y=None):
    t = _torch()
    if y is None:
        y = t.empty_like(x)
    check(lib().exb_activation_fwd(ctx.handle, act, ptr(x), ptr(y), x.numel(), exb_dtype_of(x), cur_stream()))
    return y


def concat_channels(ctx, xs, channels=None, y_stride=None, y=None):
    """Channel concat of NHWC tensors [N][H][W][cs_i] holding channels[i] valid channels each
    (default: all of them); the result has y_stride physical channels (default: the sum)."""
    t = _torch()
    n = len(xs)
    widths = [int(c) for c in (channels if channels is not None else [x.shape[-1] for x in xs])]
    total = sum(widths)
    ys = int(y_stride) if y_stride else total
    rows = xs[0].numel() // xs[0].shape[-1]
    if y is None:
        y = t.zeros(tuple(xs[0].shape[:-1]) + (ys,), device=xs[0].device, dtype=xs[0].dtype)
    px = (C.c_void_p * n)(*[x.data_ptr() for x in xs])
    pw = (C.c_int64 * n)(*widths)
    ps = (C.c_int64 * n)(*[int(x.shape[-1]) for x in xs])
    check(lib().exb_concat_fwd(ctx.handle, n, px, pw, ps, ptr(y), ys, rows, exb_dtype_of(xs[0]), cur_stream()))
    return y


def concat_nchw(ctx, xs, y=None):
    """Channel concat of dense NCHW tensors."""
    t = _torch()
    n = len(xs)
    N = xs[0].shape[0]
    widths = [x.numel() // max(N, 1) for x in xs]
    if y is None:
        y = t.empty((N, sum(x.shape[1] for x in xs)) + tuple(xs[0].shape[2:]), device=xs[0].device, dtype=xs[0].dtype)
    px = (C.c_void_p * n)(*[x.data_ptr() for x in xs])
    pw = (C.c_int64 * n)(*widths)
    check(lib().exb_concat_fwd(ctx.handle, n, px, pw, pw, ptr(y), sum(widths), N, exb_dtype_of(xs[0]), cur_stream()))
    return y


def interp_nearest(ctx, x, OH, OW, channels=None, channel_last=True, y=None):
    """Nearest resize of NHWC [N][H][W][cs] (channel_last) or NCHW fp32 [N][C][H][W]."""
    t = _torch()
    if channel_last:
        N, H, W, cs = x.shape
        Cc = channels or cs
        if y is None:
            y = t.empty((N, OH, OW, cs), device=x.device, dtype=x.dtype)
    else:
        N, Cc, H, W = x.shape
        cs = 0
        if y is None:
            y = t.empty((N, Cc, OH, OW), device=x.device, dtype=x.dtype)
    check(lib().exb_interp_nearest_fwd(ctx.handle, ptr(x), ptr(y), N, H, W, Cc, cs, OH, OW, exb_dtype_of(x),
                                       1 if channel_last else 0, cur_stream()))
    return y


def channel_affine(ctx, x, mul, add, channels=None, channel_last=True, act=ACT_NONE, y=None):
    """y = act(x * mul[c] + add[c]); mul / add: fp32 device tensors with one entry per channel."""
    t = _torch()
    if y is None:
        y = t.empty_like(x)
    if channel_last:
        cs = x.shape[-1]
        Cc = channels or cs
        outer, inner = x.numel() // cs, 1
    else:
        Cc, cs = x.shape[1], 0
        outer, inner = x.shape[0], x.numel() // max(x.shape[0] * x.shape[1], 1)
    check(lib().exb_channel_affine_fwd(ctx.handle, ptr(x), ptr(y), ptr(mul), ptr(add), outer, Cc, cs, inner,
                                       exb_dtype_of(x), 1 if channel_last else 0, act, cur_stream()))
    return y


def hardswish(ctx, x, alpha=1.0 / 6.0, beta=0.5, y=None):
    t = _torch()
    if y is None:
        y = t.empty_like(x)
    check(lib().exb_hardswish_fwd(ctx.handle, ptr(x), ptr(y), x.numel(), exb_dtype_of(x), float(alpha), float(beta),
                                  cur_stream()))
    return y


def focus(ctx, x, channels=None, out_stride=0, channel_last=True, y=None):
    """Space-to-depth 2x2 of NHWC [N][H][W][cs] (channel_last) or fp32 NCHW."""
    t = _torch()
    if channel_last:
        N, H, W, cs = x.shape
        Cc = channels or cs
        ocs = out_stride or 4 * Cc
        if y is None:
            y = t.empty((N, H // 2, W // 2, ocs), device=x.device, dtype=x.dtype)
        check(lib().exb_focus_fwd(ctx.handle, ptr(x), ptr(y), N, Cc, H, W, cs, ocs, exb_dtype_of(x), 1, cur_stream()))
    else:
        N, Cc, H, W = x.shape
        if y is None:
            y = t.empty((N, 4 * Cc, H // 2, W // 2), device=x.device, dtype=x.dtype)
        check(lib().exb_focus_fwd(ctx.handle, ptr(x), ptr(y), N, Cc, H, W, 0, 0, exb_dtype_of(x), 0, cur_stream()))
    return y


def prelu(ctx, x, slopes, channels=None, channel_last=True, y=None):
    """y = x >= 0 ? x : x * slopes[c]; slopes: fp32 device tensor with one entry per channel, or one entry."""
    t = _torch()
    if y is None:
        y = t.empty_like(x)
    if channel_last:
        cs = x.shape[-1]
        Cc = channels or cs
        outer, inner = x.numel() // cs, 1
    else:
        Cc, cs = x.shape[1], 0
        outer, inner = x.shape[0], max(int(np.prod(x.shape[2:])), 1)
    check(lib().exb_prelu_fwd(ctx.handle, ptr(x), ptr(y), ptr(slopes), slopes.numel(), outer, Cc, cs, inner,
                              exb_dtype_of(x), 1 if channel_last else 0, cur_stream()))
    return y


def channel_affine_prelu(ctx, x, mul, add, slopes, channels=None, channel_last=True, y=None):
    """y = prelu(x * mul[c] + add[c], slopes); mul / add / slopes: fp32 device tensors."""
    t = _torch()
    if y is None:
        y = t.empty_like(x)
    if channel_last:
        cs = x.shape[-1]
        Cc = channels or cs
        outer, inner = x.numel() // cs, 1
    else:
        Cc, cs = x.shape[1], 0
        outer, inner = x.shape[0], max(int(np.prod(x.shape[2:])), 1)
    check(lib().exb_channel_affine_prelu_fwd(ctx.handle, ptr(x), ptr(y), ptr(mul), ptr(add), ptr(slopes), slopes.numel(),
                                             outer, Cc, cs, inner, exb_dtype_of(x), 1 if channel_last else 0, cur_stream()))
    return y


def image_ingest(ctx, x, dtype=EXB_F16, c_stride=16, mul=None, add=None, scale=1.0, rounding=1, y=None):
    """fp32 NCHW image (<= 4 channels) -> optional x * mul[c] + add[c] -> NHWC fp16 / int8 with c_stride channels."""
    t = _torch()
    N, Cc, H, W = x.shape
    if y is None:
        y = t.empty((N, H, W, c_stride), dtype=torch_dtype(dtype), device=x.device)
    check(lib().exb_image_f32_to_nhwc_norm(ctx.handle, ptr(x), ptr(y), dtype, N, Cc, H, W, c_stride,
                                           None if mul is None else ptr(mul), None if add is None else ptr(add),
                                           float(scale), int(rounding), cur_stream()))
    return y


def padded_ingest_norm(ctx, x, mul, add, w_pad=4, w_pitch=0, y=None):
    """fp32 NCHW image (<= 3 channels) -> x * mul[c] + add[c] -> fp16 NHWC4 rows padded along W."""
    t = _torch()
    N, Cc, H, W = x.shape
    w_pitch = w_pitch or (W + w_pad + 8 + 7) // 8 * 8
    if y is None:
        y = t.empty((N, H, w_pitch, 4), dtype=t.float16, device=x.device)
    check(lib().exb_nchw_f32_to_nhwc4_padded_norm(ctx.handle, ptr(x), ptr(y), N, Cc, H, W, w_pad, w_pitch, ptr(mul), ptr(add),
                                                  cur_stream()))
    return y


def focus_ingest(ctx, x, c_stride=16, mul=None, add=None, y=None):
    """fp32 NCHW image -> optional per-channel affine -> Focus -> NHWC fp16 [N][H/2][W/2][c_stride]."""
    t = _torch()
    N, Cc, H, W = x.shape
    if y is None:
        y = t.empty((N, H // 2, W // 2, c_stride), dtype=t.float16, device=x.device)
    check(lib().exb_nchw_f32_focus_to_nhwc_f16(ctx.handle, ptr(x), ptr(y), N, Cc, H, W, c_stride,
                                               None if mul is None else ptr(mul), None if add is None else ptr(add),
                                               cur_stream()))
    return y


def binaryop_channel_bcast(ctx, a, gate, op=2, gate_first=False, channels=None, y=None):
    """y = a op gate[n][c] (or gate op a): a NHWC [N][H][W][cs], gate [N or 1][1][1][cs], same dtype."""
    t = _torch()
    N, H, W, cs = a.shape
    if y is None:
        y = t.empty_like(a)
    check(lib().exb_binaryop_channel_bcast_fwd(ctx.handle, op, ptr(a), ptr(gate), 1 if gate_first else 0, ptr(y), N, gate.shape[0],
                                               channels or cs, cs, H * W, exb_dtype_of(a), 1, cur_stream()))
    return y


def split_heads(ctx, x, anchors, values, y=None):
    """NHWC fp16 [N][H][W][cs] detection head -> fp32 [N][anchors][H*W][values] (Reshape + Transpose in one pass)."""
    t = _torch()
    N, H, W, cs = x.shape
    if y is None:
        y = t.empty((N, anchors, H * W, values), device=x.device, dtype=t.float32)
    check(lib().exb_nhwc_f16_split_heads_f32(ctx.handle, ptr(x), ptr(y), N, H * W, cs, anchors, values, cur_stream()))
    return y


def depth_to_space(ctx, x, rh, rw, channels, y_stride=0, y=None):
    """NHWC [N][H][W][xs] with channel (a*rw + b)*channels + c -> [N][H*rh][W*rw][y_stride or channels]."""
    t = _torch()
    N, H, W, xs = x.shape
    ys = y_stride or channels
    if y is None:
        y = t.empty((N, H * rh, W * rw, ys), device=x.device, dtype=x.dtype)
    check(lib().exb_depth_to_space_fwd(ctx.handle, ptr(x), ptr(y), N, H, W, rh, rw, channels, xs, ys,
                                       exb_dtype_of(x), cur_stream()))
    return y


def transpose_hw(ctx, x, y=None):
    """fp32 [..., H, W] -> [..., W, H]."""
    t = _torch()
    H, W = x.shape[-2], x.shape[-1]
    if y is None:
        y = t.empty(tuple(x.shape[:-2]) + (W, H), device=x.device, dtype=x.dtype)
    check(lib().exb_transpose_hw_f32(ctx.handle, ptr(x), ptr(y), x.numel() // max(H * W, 1), H, W, cur_stream()))
    return y


def quantize(ctx, x, scale, rounding=0, q=None):
    t = _torch()
    if q is None:
        q = t.empty(x.shape, dtype=t.int8, device=x.device)
    check(lib().exb_quantize_fwd(ctx.handle, ptr(x), exb_dtype_of(x), ptr(q), x.numel(), float(scale), rounding,
                                 cur_stream()))
    return q


def dequantize(ctx, q, scale, out_dtype=EXB_F16, y=None):
    t = _torch()
    if y is None:
        y = t.empty(q.shape, dtype=torch_dtype(out_dtype), device=q.device)
    check(lib().exb_dequantize_fwd(ctx.handle, ptr(q), ptr(y), out_dtype, q.numel(), float(scale), cur_stream()))
    return y


def nchw_f32_to_nhwc(ctx, x, dtype=EXB_F16, c_stride=0, scale=1.0, rounding=0, y=None):
    t = _torch()
    N, Cc, H, W = x.shape
    cs = c_stride or Cc
    if y is None:
        y = t.empty((N, H, W, cs), dtype=torch_dtype(dtype), device=x.device)
    check(lib().exb_nchw_f32_to_nhwc(ctx.handle, ptr(x), ptr(y), dtype, N, Cc, H, W, cs, float(scale), rounding,
                                     cur_stream()))
    return y


def nchw_f32_to_nhwc_padded(ctx, x, dtype=EXB_F16, c_stride=4, w_pad=4, w_pitch=0, scale=1.0, rounding=0, y=None):
    t = _torch()
    N, Cc, H, W = x.shape
    w_pitch = w_pitch or (W + 2 * w_pad)
    if y is None:
        y = t.empty((N, H, w_pitch, c_stride), dtype=torch_dtype(dtype), device=x.device)
    check(lib().exb_nchw_f32_to_nhwc_padded(ctx.handle, ptr(x), ptr(y), dtype, N, Cc, H, W, c_stride, w_pad, w_pitch,
                                            float(scale), rounding, cur_stream()))
    return y


def nhwc_to_nchw_f32(ctx, x, Cc=None, scale=1.0, y=None):
    t = _torch()
    N, H, W, cs = x.shape
    Cc = Cc or cs
    if y is None:
        y = t.empty((N, Cc, H, W), dtype=t.float32, device=x.device)
    check(lib().exb_nhwc_to_nchw_f32(ctx.handle, ptr(x), exb_dtype_of(x), ptr(y), N, Cc, H, W, cs, float(scale),
                                     cur_stream()))
    return y
