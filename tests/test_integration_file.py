"""The reference-side binding shown in the integration notes (include/reference_side/operation_convolution_b200.cpp)
is real code: where the reference's source tree is present it is compiled (syntax and types, no code generation)
against the reference's own headers with USE_CUDA and against this library's C header."""
import os
import shutil
import subprocess

import pytest

from oracle import ref_lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def test_reference_side_binding_compiles_against_the_reference_headers():
    tree = ref_lib.reference_tree()
    inc = os.path.join(tree, "include")
    if not os.path.isdir(os.path.join(inc, "Excalibur")):
        pytest.skip("reference source tree not present")
    gxx = shutil.which("g++")
    if gxx is None or not os.path.exists(os.path.join(CUDA, "include", "cublas_v2.h")):
        pytest.skip("g++ or the CUDA headers are missing")
    src = os.path.join(ROOT, "include", "reference_side", "operation_convolution_b200.cpp")
    cmd = [gxx, "-std=c++17", "-fsyntax-only", "-w", "-DUSE_CUDA", "-mavx2", "-mfma", "-mf16c",
           "-I", inc, "-I", os.path.join(inc, "Primitives"), "-I", os.path.join(inc, "Excalibur"),
           "-I", os.path.join(CUDA, "include"), "-I", os.path.join(ROOT, "include"), src]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-6000:]
