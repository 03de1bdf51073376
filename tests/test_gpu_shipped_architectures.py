"""Every floating-point model description the reference ships whose operation types are implemented, rebuilt
from its name-free structure with seeded weights (tests/golden/shipped_architectures.json, written by
tests/golden/make_golden.py from the shipped files), against what the reference CPU library computes for the
same graph and input (tests/golden/shipped_architectures.npz: outputs and four inner maps, sampled)."""
import json
import os

import numpy as np
import pytest

from excalibur_b200 import model_zoo

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(__file__)
with open(os.path.join(HERE, "golden", "shipped_architectures.json")) as f:
    ARCHS = json.load(f)
GOLD = np.load(os.path.join(HERE, "golden", "shipped_architectures.npz"))


def _rel(a, b):
    return float(np.abs(a.astype(np.float64) - b).max() / max(np.abs(b).max(), 1e-12))


@pytest.mark.parametrize("fusion", [False, True], ids=["op_by_op", "fused"])
@pytest.mark.parametrize("arch", ARCHS, ids=[a["name"][:28] for a in ARCHS])
def test_shipped_architecture(arch, fusion):
    from excalibur_b200 import host
    g, outs = model_zoo.graph_from_structure(arch["structure"], arch["seed"], gain=arch["gain"])
    assert outs == arch["outputs"]
    p = host.Pipeline(g.phai_text(), g.racy_bytes(), 0, fusion=fusion)
    x = model_zoo.architecture_input(arch)
    for _ in range(2 if fusion else 1):
        res = p.forward(x)
    assert sorted(res) == sorted(outs)
    name = arch["name"]
    for n in outs:
        assert tuple(res[n].shape) == tuple(GOLD["%s:%s:shape" % (name, n)]), n
        got, want = model_zoo.sample(res[n]), GOLD["%s:%s" % (name, n)]
        assert np.isfinite(got).all()
        assert _rel(got, want) < 2e-2, (n, _rel(got, want))
    if not fusion:
        for i in arch["inner"]:
            got, want = model_zoo.sample(p.get("t%d" % i)), GOLD["%s:t%d" % (name, i)]
            assert _rel(got, want) < 2e-2, ("t%d" % i, arch["structure"][i][0], _rel(got, want))
    if fusion:
        # all but two run on the fused plan; those two flatten a convolution map in front of an InnerProduct /
        # Concat (a Reshape in the middle of the graph), which the plan refuses, and run op by op instead
        launches, _ = p.stats()
        print("%s: %d launches" % (name, launches))
        assert (launches > 0) == (name not in ("pfld11_landmark65_simp", "singel_char_classfi_simp")), launches
    p.close()
