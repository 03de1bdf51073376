"""CPU checks for the operations and graphs added for the reference's shipped model descriptions: the
oracle's PReLU / LeakyRelu / Deconvolution / Reshape / Transpose against outputs of the reference CPU
library (golden vectors), and the model builders against the shipped `.phai` files themselves where the
reference tree is present."""
import os

import numpy as np
import pytest

from excalibur_b200 import model_zoo
from oracle import exb_oracle as O
from oracle import ref_lib

S = np.load(os.path.join(os.path.dirname(__file__), "golden", "shipped_model_vectors.npz"))
REF_MODELS = os.path.join(ref_lib.reference_tree(), "models")


def test_oracle_prelu_leakyrelu_match_the_reference():
    x = S["act_x"]
    np.testing.assert_array_equal(O.prelu(x, S["prelu_slopes"]), S["prelu_out"])
    np.testing.assert_array_equal(O.prelu(x, S["prelu_slopes"][:1]), S["prelu_shared_out"])
    np.testing.assert_array_equal(O.leakyrelu(x, 0.1), S["leaky_out"])


@pytest.mark.parametrize("tag", ["deconv_k2s2", "deconv_k2s2_c1", "deconv_k3s2p1", "deconv_k4s2p1"])
def test_oracle_deconvolution_matches_the_reference(tag):
    k, s, p = (int(v) for v in S[tag + "_cfg"])
    y = O.deconv2d_f32(S["act_x"], S[tag + "_w"], S[tag + "_b"], s, p)
    assert y.shape == S[tag + "_out"].shape
    np.testing.assert_allclose(y, S[tag + "_out"], rtol=0, atol=2e-6)      # fp32 summation order differs


def test_oracle_reshape_transpose_match_the_reference():
    y = O.transpose_hw(O.reshape_nchw(S["rt_x"], w=20, h=4, c=3))
    np.testing.assert_array_equal(y, S["rt_out"])
    assert O.reshape_nchw(S["rt_x"], w=-1, h=2, c=6).shape == (2, 6, 2, 20)


def test_oracle_hardsigmoid_softmax_flatten_match_the_reference():
    x = S["misc_x"]
    np.testing.assert_allclose(O.hardsigmoid(x, 0.2, 0.5), S["hardsigmoid_out"], rtol=0, atol=1e-7)
    np.testing.assert_allclose(O.softmax_channels(x), S["softmax_out"], rtol=0, atol=2e-7)
    np.testing.assert_array_equal(O.flatten_nchw(x), S["flatten_out"])
    np.testing.assert_array_equal(O.flatten_nchw(x, 0), S["flatten0_out"])
    gate = O.pool2d_f32(x, 1, global_pool=True)
    np.testing.assert_allclose(x * gate, S["bcast_mul_out"], rtol=0, atol=1e-6)
    np.testing.assert_allclose(gate - x, S["bcast_sub_out"], rtol=0, atol=1e-6)     # operand order is kept


@pytest.mark.parametrize("name,ops", [("det_db_resnet18", 80), ("mobile_unicorn", 96), ("yolov5s_simp", 170)])
def test_builders_have_the_shipped_architecture(name, ops):
    g, info = getattr(model_zoo, name)()
    mine = model_zoo.structure(g.phai_text())
    assert len(mine) == ops
    path = os.path.join(REF_MODELS, name + ".phai")
    if not os.path.exists(path):
        pytest.skip("reference tree not present: only the op count is checked")
    with open(path) as f:
        shipped = model_zoo.structure(f.read())
    assert mine == shipped


def test_unicorn_light_builder_matches_the_shipped_fp_and_int8_descriptions():
    g, info = model_zoo.unicorn_light()
    fp = model_zoo.structure(g.phai_text())
    g8, _ = model_zoo.unicorn_light(act_scales={n: 1.0 for n in info["conv_inputs"]})
    i8 = model_zoo.structure(g8.phai_text())
    assert len(fp) == len(i8) == 73
    assert sum(1 for t, p, _ in i8 if t == "convolution" and p["int8"]) == 28
    base = os.path.join(REF_MODELS, "unicorn_light_806204_m1x3x2+120k_universial_noised_usefulpart")
    if not os.path.exists(base + ".phai"):
        pytest.skip("reference tree not present: only the op counts are checked")
    assert fp == model_zoo.structure(open(base + ".phai").read())
    assert i8 == model_zoo.structure(open(base + "_int8.phai").read())


def test_weight_file_covers_every_record_of_the_builders():
    from excalibur_b200.calibrate import parse_phai, racy_record_size
    int8 = lambda: model_zoo.unicorn_light(act_scales={n: 2.0 for n in model_zoo.unicorn_light()[1]["conv_inputs"]})
    int8.__name__ = "unicorn_light_int8"
    for fn in (model_zoo.det_db_resnet18, model_zoo.mobile_unicorn, model_zoo.yolov5s_simp, model_zoo.unicorn_light, int8):
        g, _ = fn()
        _, ops = parse_phai(g.phai_text())
        blob = g.racy_bytes()
        pos = 0
        for op in ops:
            pos += racy_record_size(op, blob, pos)
        assert pos == len(blob), fn.__name__


def test_structure_fixture_round_trips_through_the_graph_generator():
    """tests/golden/shipped_architectures.json -> graph_from_structure -> structure gives the fixture back, and
    the generated weight file holds exactly the records the graph consumes."""
    import json
    from excalibur_b200.calibrate import parse_phai, racy_record_size
    with open(os.path.join(os.path.dirname(__file__), "golden", "shipped_architectures.json")) as f:
        archs = json.load(f)
    assert len(archs) == 15
    for a in archs:
        g, outs = model_zoo.graph_from_structure(a["structure"], a["seed"], gain=a["gain"])
        assert outs == a["outputs"], a["name"]
        again = json.loads(json.dumps(model_zoo.structure(g.phai_text())))
        assert again == json.loads(json.dumps(a["structure"])), a["name"]
        _, ops = parse_phai(g.phai_text())
        blob, pos = g.racy_bytes(), 0
        for op in ops:
            pos += racy_record_size(op, blob, pos)
        assert pos == len(blob), a["name"]
