"""Live check of the CPU oracle against the reference library where oracle/_ref has been built
(`make -C oracle ref`, which needs the reference source tree).  Skipped elsewhere; the committed
golden vectors cover the same ground."""
import numpy as np
import pytest

from excalibur_b200 import models
from excalibur_b200.modelfile import GraphBuilder
from oracle import exb_oracle as O
from oracle import ref_lib

pytestmark = pytest.mark.skipif(not ref_lib.available(), reason="oracle/_ref not built")


def _ref(g, x, name="out"):
    p = ref_lib.RefPipeline(g.phai_text(), g.racy_bytes())
    p.forward(x)
    y = p.featmap(name)
    p.close()
    return y


@pytest.mark.parametrize("cout,k,stride,pad,n", [(64, 3, 1, 1, 2), (128, 3, 1, 1, 1), (64, 3, 2, 1, 1), (96, 1, 1, 0, 1)])
def test_int8_conv_bit_exact(cout, k, stride, pad, n):
    r = np.random.default_rng(cout + k + stride)
    x = r.uniform(-1, 1, (n, 32, 14, 14)).astype(np.float32)
    w = (r.standard_normal((cout, 32, k, k)) * 0.1).astype(np.float32)
    b = (r.standard_normal(cout) * 0.01).astype(np.float32)
    wq, ws = models.quantize_weights(w)
    fs = np.float32(127.0 / np.abs(x).max())
    g = GraphBuilder()
    g.conv("c", "in", "out", w, b, stride, pad, act=1, int8=(wq, ws, fs))
    np.testing.assert_array_equal(O.conv2d_i8(x, wq, b, ws, fs, stride, pad, act=1), _ref(g, x))


def test_config1_conv_fp32():
    r = np.random.default_rng(1000)
    x = r.uniform(-1, 1, (1, 64, 56, 56)).astype(np.float32)
    w = (r.standard_normal((64, 64, 3, 3)) * np.sqrt(2.0 / 576)).astype(np.float32)
    b = (r.standard_normal(64) * 0.01).astype(np.float32)
    g = GraphBuilder()
    g.conv("c", "in", "out", w, b, 1, 1, act=1)
    np.testing.assert_allclose(O.conv2d_f32(x, w, b, 1, 1, act=1), _ref(g, x), rtol=1e-5, atol=3e-6)
