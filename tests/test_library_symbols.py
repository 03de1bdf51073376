"""The C-ABI shared library builds without a GPU (nvcc cross-compiles), loads, and exports every
entry point the public headers declare.  No compute call is made here."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    return sorted(set(re.findall(r"EXB_API\s+[\w\s\*]+?\b(exb_\w+)\s*\(", text)))


@pytest.fixture(scope="module")
def so_path():
    from excalibur_b200 import build
    return build.build()


def test_headers_declare_entry_points():
    names = _declared("excalibur_b200.h")
    assert "exb_conv2d_fwd" in names and "exb_pool2d_fwd" in names and len(names) >= 25
    assert "exb_host_pipeline_forward" in _declared("excalibur_b200_host.h")


def test_library_exports_every_declared_symbol(so_path):
    lib = ctypes.CDLL(so_path)
    missing = [n for h in ("excalibur_b200.h", "excalibur_b200_host.h") for n in _declared(h) if not hasattr(lib, n)]
    assert not missing, missing


def test_python_binding_lists_match_headers():
    from excalibur_b200 import capi, host
    assert sorted(capi.EXPORTED_SYMBOLS) == _declared("excalibur_b200.h")
    assert sorted(host.HOST_SYMBOLS) == _declared("excalibur_b200_host.h")


def test_pure_host_calls_work_without_a_gpu(so_path):
    from excalibur_b200 import capi, host
    assert capi.lib().exb_version().decode().count(".") == 2
    d = capi.make_conv_desc(4, 56, 56, 64, 128, 3, 2, 1, capi.EXB_I8, capi.EXB_I8)
    assert capi.conv_out_dims(d) == (28, 28)
    assert capi.lib().exb_conv2d_uses_tensor_cores(d) == 1
    d = capi.make_conv_desc(4, 56, 56, 30, 128, 3, 1, 1, capi.EXB_F16, capi.EXB_F16)   # 60-byte rows
    assert capi.lib().exb_conv2d_uses_tensor_cores(d) == 0
    p = capi.make_pool_desc(1, 112, 112, 64, 0, 3, 2, 1)
    assert capi.pool_out_dims(p) == (56, 56)
    p = capi.make_pool_desc(1, 7, 9, 16, 0, 2, 2, 0, pad_mode=0)
    assert capi.pool_out_dims(p) == (5, 6) or capi.pool_out_dims(p) == (4, 5)
    bad = capi.make_conv_desc(1, 2, 2, 64, 64, 3, 1, 0)
    with pytest.raises(capi.ExbError):
        capi.conv_out_dims(bad)
    # operation classes are registered under the reference's keys
    for key in ("operation_convolution", "operation_convolutiondepthwise", "operation_pooling", "operation_eltwise",
                "operation_binaryop", "operation_relu", "operation_split", "operation_innerproduct", "operation_clip",
                "operation_sigmoid", "operation_concat", "operation_interp", "operation_batchnorm", "operation_hardswish",
                "operation_input", "operation_yolov5focus", "operation_prelu", "operation_leakyrelu", "operation_deconvolution",
                "operation_reshape", "operation_transpose", "operation_hardsigmoid", "operation_softmax", "operation_flatten"):
        assert host.registered(key), key
    assert not host.registered("operation_nonexistent")
    # capability queries are pure host arithmetic
    stem = capi.make_conv_desc(8, 224, 224, 3, 64, 7, 2, 3, capi.EXB_F16, capi.EXB_F16, act=capi.ACT_RELU, cin_stride=4,
                               x_w_pitch=240, x_w_pad=4)
    assert capi.lib().exb_conv2d_pool_fusable(stem) == 1
    stem.fuse_pool = 1
    assert capi.conv_out_dims(stem) == (56, 56)
    body = capi.make_conv_desc(8, 56, 56, 64, 64, 3, 1, 1, capi.EXB_I8, capi.EXB_I8)
    assert capi.lib().exb_conv2d_pool_fusable(body) == 0


def test_no_cpu_fallback_in_the_product(so_path):
    """Without a GPU a context cannot be created and the host layer reports it; nothing computes."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    from excalibur_b200 import capi
    with pytest.raises(capi.ExbError):
        capi.Context(0)
