"""TEST INFRASTRUCTURE - NOT PRODUCT CODE.

ctypes driver for the UNMODIFIED reference CPU library (oracle/_ref/libexcalibur_ref.so, built
from the reference's own sources by `make -C oracle ref`).  Runs a .phai graph + .racy weights
through glasssix::excalibur::pipeline<float> on the host and returns feature maps as numpy.
"""
import ctypes as C
import os
import tempfile

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))


def reference_tree():
    """Where the reference project's source tree is expected: $EXB_REFERENCE_TREE, else a directory named
    `reference` beside this repository.  The tree is only ever read (build recipe, fixture generator)."""
    return os.environ.get("EXB_REFERENCE_TREE") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")

SO_PATH = os.path.join(_HERE, "_ref", "libexcalibur_ref.so")
_LIB = None


def available():
    return os.path.exists(SO_PATH)


def lib():
    global _LIB
    if _LIB is None:
        _LIB = C.CDLL(SO_PATH)
        _LIB.ref_pipeline_create.restype = C.c_void_p
        _LIB.ref_pipeline_create.argtypes = [C.c_char_p, C.c_char_p]
        _LIB.ref_pipeline_destroy.argtypes = [C.c_void_p]
        _LIB.ref_pipeline_forward.argtypes = [C.c_void_p, C.c_void_p] + [C.c_int] * 5
        _LIB.ref_pipeline_output_name.argtypes = [C.c_void_p, C.c_int, C.c_char_p, C.c_int]
        _LIB.ref_pipeline_get_featmap.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p,
                                                  C.c_longlong, C.c_void_p]
    return _LIB


class RefPipeline:
    """pipeline<float>(lines, racy_path, device=-1) of the reference."""

    def __init__(self, phai_text, racy_bytes=b""):
        self._tmp = None
        path = b""
        if racy_bytes:
            self._tmp = tempfile.NamedTemporaryFile(suffix=".racy", delete=False)
            self._tmp.write(racy_bytes)
            self._tmp.close()
            path = self._tmp.name.encode()
        self._h = lib().ref_pipeline_create(phai_text.encode(), path)

    def forward(self, x_nchw):
        x = np.ascontiguousarray(x_nchw, np.float32)
        n, c, h, w = x.shape
        k = lib().ref_pipeline_forward(self._h, x.ctypes.data, n, c, h, w, 0)
        names = []
        buf = C.create_string_buffer(256)
        for i in range(k):
            lib().ref_pipeline_output_name(self._h, i, buf, 256)
            names.append(buf.value.decode())
        return {nm: self.featmap(nm) for nm in names}

    def featmap(self, name):
        shp = (C.c_int * 4)()
        rc = lib().ref_pipeline_get_featmap(self._h, name.encode(), None, 0, shp)
        if rc != 0:
            raise KeyError(name)
        out = np.empty(tuple(shp), np.float32)
        rc = lib().ref_pipeline_get_featmap(self._h, name.encode(), out.ctypes.data, out.size, shp)
        assert rc == 0
        return out

    def close(self):
        if self._h:
            lib().ref_pipeline_destroy(self._h)
            self._h = None
        if self._tmp is not None:
            os.unlink(self._tmp.name)
            self._tmp = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
