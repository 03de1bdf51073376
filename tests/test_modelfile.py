"""The .phai / .racy writers produce what the reference's parser and init_weights expect."""
import struct

import numpy as np

from excalibur_b200 import models
from excalibur_b200.modelfile import GraphBuilder, RACY_TAG_F32, RACY_TAG_I8


def test_phai_lines_and_racy_records():
    g = GraphBuilder("t")
    w = np.arange(2 * 3 * 3 * 3, dtype=np.float32).reshape(2, 3, 3, 3)
    b = np.array([1.0, 2.0], np.float32)
    g.conv("c1", "in", "a", w, b, 2, 1, act=1)
    wq = np.ones((4, 2, 1, 1), np.int8)
    g.conv("c2", "a", "b", None, None, 1, 0, int8=(wq, np.full(4, 3.0, np.float32), 5.0))
    g.pool("p", "b", "c", 0, 3, 2, 1)
    text = g.phai_text().splitlines()
    assert text[0].startswith("glsv1") and text[1] == "3 4"
    assert text[2] == "Convolution c1 1 1 in a 0=2 1=3 11=3 2=1 12=1 3=2 13=2 4=1 14=1 15=1 16=1 5=1 6=54 9=1"
    assert "8=1" in text[3] and "5=0" in text[3] and "6=8" in text[3]
    blob = g.racy_bytes()
    assert struct.unpack_from("<i", blob, 0)[0] == RACY_TAG_F32
    off = 4 + 54 * 4 + 2 * 4
    assert struct.unpack_from("<i", blob, off)[0] == RACY_TAG_I8
    off += 4 + 8            # 8 int8 weights, already a multiple of 4
    assert struct.unpack_from("<4f", blob, off) == (3.0, 3.0, 3.0, 3.0)
    assert struct.unpack_from("<f", blob, off + 16)[0] == 5.0
    assert len(blob) == off + 20


def test_int8_weight_padding_to_four_bytes():
    g = GraphBuilder()
    wq = np.ones((1, 3, 1, 1), np.int8)
    g.conv("c", "in", "out", None, None, int8=(wq, np.ones(1, np.float32), 1.0))
    assert len(g.racy_bytes()) == 4 + 4 + 4 + 4   # tag, 3 weights + 1 pad, 1 weight scale, 1 act scale


def test_resnet18_builder_counts():
    g, info = models.resnet18(2)
    convs = [l for l in g.lines if l.startswith("Convolution")]
    assert len(convs) == 1 + 16 + 3
    assert len(info["conv_inputs"]) == 19
    macs = models.resnet18_macs()
    assert macs["total"] == 1814073344 and macs["conv3x3"] == 1676279808
    wq, ws = models.quantize_weights(np.array([[[[0.5]], [[-2.0]]]], np.float32))
    assert ws[0] == np.float32(63.5) and list(wq.reshape(-1)) == [32, -127]


def test_calibrate_reader_walks_every_weight_record():
    """The .phai / .racy reader of the calibration tool accounts for every byte of the weight blob of
    the floating-point and int8 benchmark graphs and reproduces the op lines it parsed."""
    from excalibur_b200 import calibrate, models
    scales = None
    g32, info = models.resnet18(2)
    graphs = [g32, models.mobilenet_v2(3)[0], models.yolov5s(5)[0], models.bn_net(8), models.focus_net(7),
              models.resnet18(2, act_scales={k: 30.0 for k in info["conv_inputs"]})[0]]
    for g in graphs:
        head, ops = calibrate.parse_phai(g.phai_text())
        assert [calibrate.op_line(op) for op in ops] == g.lines
        pos = 0
        blob = g.racy_bytes()
        for op in ops:
            pos += calibrate.racy_record_size(op, blob, pos)
        assert pos == len(blob)


def test_host_f32_to_f16_conversion_rounds_to_nearest_even():
    """The conversion the host_f16_threads option runs before the copy: F16C, bit-level and pooled variants all
    equal numpy's round-to-nearest-even (which is also the device's __float2half_rn)."""
    from excalibur_b200 import host
    r = np.random.default_rng(3)
    x = np.concatenate([
        r.standard_normal(100003).astype(np.float32),
        (r.standard_normal(50000) * 1e-6).astype(np.float32),         # half subnormals and underflow
        (r.standard_normal(50000) * 3e4).astype(np.float32),          # around the overflow threshold
        np.array([0.0, -0.0, 65504.0, 65519.99, 65520.0, 65536.0, 1e9, -1e9, np.inf, -np.inf, 2.0 ** -24, 2.0 ** -25,
                  1.5 * 2.0 ** -25, 2.0 ** -14, 2.0 ** -14 - 2.0 ** -26, 1.0 + 2.0 ** -11, 1.0 + 3 * 2.0 ** -11,
                  0.1, 255.0, 1e-8], np.float32),
    ])
    with np.errstate(over="ignore"):
        want = x.astype(np.float16)
    for threads, scalar in ((1, False), (1, True), (5, False)):
        got = host.convert_f32_to_f16(x, threads, scalar)
        np.testing.assert_array_equal(got.view(np.uint16), want.view(np.uint16), err_msg="threads %d scalar %s" % (threads, scalar))
    nan = host.convert_f32_to_f16(np.array([np.nan], np.float32), 1, True)
    assert np.isnan(nan[0])
    assert host.convert_f32_to_f16(np.zeros((0,), np.float32)).size == 0
