"""dump_profile: the chrome://tracing writer on the CPU, and a profiled forward on the GPU."""
import json

import numpy as np
import pytest

from excalibur_b200 import models


def _host():
    from excalibur_b200 import host
    return host


def _check_trace(path, names):
    doc = json.load(open(path))
    ev = doc["traceEvents"]
    assert len(ev) == 2 * len(names)
    for i, n in enumerate(names):
        b, e = ev[2 * i], ev[2 * i + 1]
        assert b["name"] == n and e["name"] == n
        assert b["ph"] == "B" and e["ph"] == "E" and b["cat"] == "op"
        assert e["ts"] >= b["ts"] >= 0
    return ev


def test_chrome_trace_writer_emits_one_pair_per_entry(tmp_path):
    h = _host()
    entries = [("stem", 0.0, 0.25), ('odd "name" \\ with\ttab', 0.25, 0.26), ("fc", 0.26, 1.5)]
    path = str(tmp_path / "trace.json")
    h.write_chrome_trace(path, entries)
    ev = _check_trace(path, [e[0] for e in entries])
    assert ev[1]["ts"] == pytest.approx(250.0) and ev[5]["ts"] == pytest.approx(1500.0)    # microseconds
    h.write_chrome_trace(path, [])
    assert json.load(open(path)) == {"traceEvents": []}
    with pytest.raises(h.HostError):
        h.write_chrome_trace(str(tmp_path / "no_such_dir" / "t.json"), entries)


@pytest.mark.gpu
@pytest.mark.parametrize("fusion", [True, False], ids=["fused", "op_by_op"])
def test_dump_profile_of_a_forward(tmp_path, fusion):
    h = _host()
    g, _ = models.resnet18(2)
    p = h.Pipeline(g.phai_text(), g.racy_bytes(), 0, fusion=fusion)
    x = np.random.default_rng(1).uniform(0, 1, (2, 3, 64, 64)).astype(np.float32)
    p.forward(x)
    p.set_option("profile", 1)
    p.forward(x)
    names = [n for n, _, _ in p.trace()]
    assert len(names) >= 20
    path = str(tmp_path / "profile.json")
    p.dump_profile(path)
    p.close()
    _check_trace(path, names)
