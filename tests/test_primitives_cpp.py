"""C++ host primitives tested as C++ (no GPU): small programs under tests/cpp/ are compiled with g++ against the
host layer's headers, linked to the built library and run."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _build_and_run(name, tmp_path):
    from excalibur_b200 import build
    so = build.build()
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("g++ not found")
    exe = str(tmp_path / name)
    cmd = [gxx, "-std=c++17", "-O1", "-pthread", "-I", os.path.join(CUDA, "include"),
           "-I", os.path.join(ROOT, "excalibur_b200", "csrc", "host"), "-I", os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tests", "cpp", name + ".cpp"), "-o", exe, so, "-Wl,-rpath," + os.path.dirname(so),
           "-L", os.path.join(CUDA, "lib64"), "-lcudart_static", "-ldl", "-lrt"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-4000:]
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, (r.stdout[-2000:], r.stderr[-2000:])
    return r.stdout


def test_pool_allocator_reuse_rule_and_two_thread_stress(tmp_path):
    out = _build_and_run("pool_allocator_test", tmp_path)
    assert out.strip().endswith("ok"), out
