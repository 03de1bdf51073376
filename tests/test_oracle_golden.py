"""Pins the CPU oracle (oracle/exb_oracle.c) against vectors produced by the UNMODIFIED reference
library (tests/golden/reference_vectors.npz, written by tests/golden/make_golden.py).
Runs without a GPU and without the reference tree."""
import os

import numpy as np
import pytest

from oracle import exb_oracle as O

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.npz"))


@pytest.mark.parametrize("tag", ["conv_f32_wino", "conv_f32_im2col_s2", "conv_f32_stem", "conv_f32_1x1"])
def test_conv_f32(tag):
    stride, pad, act = [int(v) for v in G[tag + "_cfg"]]
    y = O.conv2d_f32(G[tag + "_x"], G[tag + "_w"], G[tag + "_b"], stride, pad, act=act)
    # Winograd / packed-GEMM fp32 summation order vs the oracle's double accumulation
    np.testing.assert_allclose(y, G[tag + "_y"], rtol=1e-5, atol=2e-6)


@pytest.mark.parametrize("tag", ["conv_i8_wino", "conv_i8_im2col_s2", "conv_i8_im2col_wide", "conv_i8_1x1_s2"])
def test_conv_i8_bit_exact(tag):
    stride, pad, act = [int(v) for v in G[tag + "_cfg"]]
    y = O.conv2d_i8(G[tag + "_x"], G[tag + "_wq"], G[tag + "_b"], G[tag + "_ws"], G[tag + "_fs"], stride, pad, act=act)
    np.testing.assert_array_equal(y, G[tag + "_y"])


@pytest.mark.parametrize("tag,stride", [("dw_s1", 1), ("dw_s2", 2)])
def test_dwconv(tag, stride):
    y = O.dwconv2d_f32(G[tag + "_x"], G[tag + "_w"], G[tag + "_b"], stride, 1, act=1)
    np.testing.assert_allclose(y, G[tag + "_y"], rtol=1e-5, atol=2e-6)


@pytest.mark.parametrize("tag,kw", [
    ("pool_max_3s2p1", dict(type=0, kernel=3, stride=2, pad=1)),
    ("pool_max_5s1p2", dict(type=0, kernel=5, stride=1, pad=2)),
    ("pool_max_ceil", dict(type=0, kernel=2, stride=2, pad=0, pad_mode=0)),
    ("pool_avg_excl", dict(type=1, kernel=3, stride=2, pad=1, count_include_pad=0)),
    ("pool_avg_incl", dict(type=1, kernel=3, stride=2, pad=1, count_include_pad=1)),
    ("pool_gap", dict(type=1, global_pool=True)),
])
def test_pool(tag, kw):
    y = O.pool2d_f32(G["pool_x"], **kw)
    assert y.shape == G[tag + "_y"].shape
    np.testing.assert_array_equal(y, G[tag + "_y"])


def test_eltwise_binaryop_relu():
    x = G["elt_x"]
    ra = O.relu_f32(x)
    np.testing.assert_array_equal(ra, G["elt_ra"])
    bb = O.binaryop_f32(x, x, 2)
    np.testing.assert_array_equal(bb, G["elt_bb"])
    # "-23301=3,0.5,-1.25": the reference reads n-1 = 2 coefficients, the third stays 1
    esum = O.eltwise_f32([ra, bb, x], 1, [0.5, -1.25, 1.0])
    np.testing.assert_allclose(esum, G["elt_esum"], rtol=1e-6, atol=1e-6)
    np.testing.assert_array_equal(O.eltwise_f32([ra, bb], 0), G["elt_eprod"])
    np.testing.assert_array_equal(O.eltwise_f32([ra, bb, x], 2), G["elt_emax"])
    np.testing.assert_array_equal(O.binaryop_f32(G["elt_esum"], G["elt_eprod"], 0), G["elt_out"])


def test_float32_to_int8_rule():
    # half away from zero, truncation, saturation (reference src/Primitives/simd_types.cpp:140-152)
    for v, q in [(0.5, 1), (-0.5, -1), (1.5, 2), (2.5, 3), (-2.5, -3), (0.49, 0), (126.6, 127), (127.5, 127),
                 (-128.4, -128), (-500.0, -128), (500.0, 127)]:
        assert O.float32_to_int8(v) == q
    assert list(O.requantize_rne(np.array([0.5, 1.5, 2.5, -0.5, -1.5, 300, -300], np.float32), 1.0)) == \
        [0, 2, 2, 0, -2, 127, -128]


def test_dequant_scale_rule():
    s = O.dequant_scales(np.array([2.0, 1e-7, 4.0], np.float32), np.array([8.0], np.float32), 3)
    np.testing.assert_array_equal(s, np.array([1.0 / 16.0, 0.0, 1.0 / 32.0], np.float32))


# ---- graph glue (Concat, Interp nearest, BatchNorm) against tests/golden/yolo_vectors.npz ---------
Y = np.load(os.path.join(os.path.dirname(__file__), "golden", "yolo_vectors.npz"))


def test_concat_channels():
    x = Y["cat_x"]
    relu = O.relu_f32(x)
    sig = (1.0 / (1.0 + np.exp(-x.astype(np.float64)))).astype(np.float32)
    y = O.concat_channels([relu, sig, x])
    assert y.shape == Y["cat_out"].shape
    np.testing.assert_array_equal(y[:, :19], Y["cat_out"][:, :19])
    np.testing.assert_array_equal(y[:, 38:], Y["cat_out"][:, 38:])
    np.testing.assert_allclose(y[:, 19:38], Y["cat_out"][:, 19:38], rtol=0, atol=2e-7)   # expf vs exp


def test_interp_nearest():
    np.testing.assert_array_equal(O.interp_nearest(Y["interp2_x"], 12, 10), Y["interp2_out"])
    np.testing.assert_array_equal(O.interp_nearest(Y["interp_odd_x"], 7, 11), Y["interp_odd_out"])


def test_batchnorm():
    b, a = O.batchnorm_coeffs(Y["bn_slope"], Y["bn_mean"], Y["bn_var"], Y["bn_bias"], 1e-5)
    # the reference's loop may or may not contract b*x + a into one fma
    np.testing.assert_allclose(O.channel_affine(Y["bn_x"], b, a), Y["bn_out"], rtol=2e-7, atol=3e-7)


def test_hardswish_input_focus():
    np.testing.assert_allclose(O.hardswish(Y["hs_x"]), Y["hs_std_out"], rtol=0, atol=5e-7)
    np.testing.assert_allclose(O.hardswish(Y["hs_x"], 0.2, 0.5), Y["hs_02_out"], rtol=0, atol=5e-7)
    np.testing.assert_array_equal(O.input_norm(Y["inp_x"], Y["inp_means"], Y["inp_scales"]), Y["inp_out"])
    np.testing.assert_array_equal(O.focus(Y["focus_x"]), Y["focus_out"])
