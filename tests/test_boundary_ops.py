"""The ReLU6 operation and the Mish suffix activation of a convolution, against outputs of the reference CPU
library (tests/golden/boundary_vectors.npz): the oracle on the CPU, the host layer's operations and the fused plan on
the GPU."""
import os

import numpy as np
import pytest

from excalibur_b200.modelfile import GraphBuilder
from oracle import exb_oracle as O
from tests.util import assert_close_f16

B = np.load(os.path.join(os.path.dirname(__file__), "golden", "boundary_vectors.npz"))


def test_oracle_relu6_writes_zero_above_six():
    x = B["relu6_x"]
    y = O.activation(x, O.ACT_RELU6_QUIRK)
    np.testing.assert_array_equal(y, B["relu6_out"])
    np.testing.assert_array_equal(y, B["relu6_keys_out"])
    assert (x > 6).any() and (y[x > 6] == 0).all()


def test_oracle_conv_relu6_and_mish():
    x, w, b = B["conv_x"], B["conv_w"], B["conv_b"]
    y = O.activation(O.conv2d_f32(x, w, b, 1, 1), O.ACT_RELU6_QUIRK)
    ref = B["conv_relu6_out"]
    # an output within rounding of 6 may fall on the other side of the cut in another summation order
    edge = np.abs(O.conv2d_f32(x, w, b, 1, 1) - 6.0) < 1e-4
    np.testing.assert_allclose(y[~edge], ref[~edge], rtol=1e-5, atol=2e-6)
    np.testing.assert_allclose(O.conv2d_f32(x, w, b, 1, 1, act=O.ACT_MISH), B["conv_mish_out"], rtol=1e-5, atol=2e-6)
    y8 = O.conv2d_i8(x, B["conv_wq"], b, B["conv_ws"], B["conv_fs"], 1, 1, act=O.ACT_MISH)
    np.testing.assert_allclose(y8, B["conv_mish_i8_out"], rtol=1e-6, atol=1e-6)


def _host():
    from excalibur_b200 import host
    return host


@pytest.mark.gpu
def test_operation_relu6_matches_the_reference_exactly():
    h = _host()
    assert h.registered("operation_relu6")
    np.testing.assert_array_equal(h.run_op("ReLU6", "", [B["relu6_x"]]), B["relu6_out"])
    np.testing.assert_array_equal(h.run_op("ReLU6", "0=0.0 1=6.0", [B["relu6_x"]]), B["relu6_keys_out"])
    with pytest.raises(h.HostError) as e:
        h.run_op("ReLU6", "2=1", [B["relu6_x"]])
    assert "Un-supported ReLU6 Attribution" in str(e.value)


@pytest.mark.gpu
@pytest.mark.parametrize("fusion", [True, False], ids=["fused", "op_by_op"])
def test_conv_then_relu6_in_a_pipeline(fusion):
    x, w, b = B["conv_x"], B["conv_w"], B["conv_b"]
    g = GraphBuilder()
    g.conv("c", "in", "m", w, b, 1, 1, act=0)
    g.relu6("r", "m", "out")
    p = _host().Pipeline(g.phai_text(), g.racy_bytes(), 0, fusion=fusion)
    for _ in range(3):
        y = p.forward(x)["out"]
    p.close()
    ref = B["conv_relu6_out"]
    pre = O.conv2d_f32(x, w, b, 1, 1)
    edge = np.abs(pre - 6.0) < 0.08          # fp16 rounding of a value next to the cut decides which side it falls on
    assert edge.mean() < 0.05
    assert_close_f16(np.where(edge, ref, y), ref, what="conv + ReLU6")
    assert (y[pre > 6.1] == 0).all() and (pre > 6.1).any()


@pytest.mark.gpu
def test_convolution_with_mish_suffix_activation():
    h = _host()
    x, w, b = B["conv_x"], B["conv_w"], B["conv_b"]
    g = GraphBuilder()
    g.conv("c", "in", "out", w, b, 1, 1, act=5)
    params = g.lines[0].split(" ", 6)[6]
    y = h.run_op("Convolution", params, [x], g.racy_bytes())
    assert_close_f16(y, B["conv_mish_out"], what="conv + Mish fp16")
    g = GraphBuilder()
    g.conv("c", "in", "out", w, b, 1, 1, act=5, int8=(B["conv_wq"], B["conv_ws"], B["conv_fs"]))
    params = g.lines[0].split(" ", 6)[6]
    y = h.run_op("Convolution", params, [x], g.racy_bytes())
    # int32 accumulators are exact; the activation is evaluated in fp32 here and in double by the reference
    np.testing.assert_allclose(y, B["conv_mish_i8_out"], rtol=2e-6, atol=2e-6)
    p = h.Pipeline(g.phai_text(), g.racy_bytes(), 0, fusion=True)
    for _ in range(3):
        yf = p.forward(x)["out"]
    p.close()
    assert_close_f16(yf, B["conv_mish_i8_out"], what="conv + Mish int8, fused plan")
