"""ctypes binding of the C++ host layer (include/excalibur_b200_host.h): pipeline<float> and single
operations created through the operation reflector, driven with numpy / pinned torch buffers."""
import ctypes as C
import os
import tempfile

import numpy as np

from . import capi

EXB_HOST_FATAL = -100
HOST_SYMBOLS = [
    "exb_host_last_error", "exb_host_registered", "exb_host_pipeline_create", "exb_host_pipeline_destroy",
    "exb_host_pipeline_set_option", "exb_host_pipeline_forward", "exb_host_pipeline_num_outputs",
    "exb_host_pipeline_output_name", "exb_host_pipeline_get", "exb_host_pipeline_output_ptr", "exb_host_pipeline_stats",
    "exb_host_pipeline_dump_profile", "exb_host_write_chrome_trace", "exb_host_pipeline_run_resident", "exb_host_pipeline_trace_size",
    "exb_host_pipeline_trace_entry", "exb_host_op_run", "exb_host_convert_f32_to_f16",
    "exb_host_pipeline_f16_create", "exb_host_pipeline_f16_destroy", "exb_host_pipeline_f16_set_option",
    "exb_host_pipeline_f16_forward", "exb_host_pipeline_f16_get", "exb_host_pipeline_f16_stats",
    "exb_host_shard_bounds", "exb_host_gather_rows", "exb_host_sharded_create", "exb_host_sharded_destroy",
    "exb_host_sharded_set_option", "exb_host_sharded_forward", "exb_host_sharded_num_outputs",
    "exb_host_sharded_output_name", "exb_host_sharded_get", "exb_host_sharded_device_ms",
]
_READY = False


class HostError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__("excalibur_b200 host error %d: %s" % (code, msg))
        self.code = code


def lib():
    global _READY
    L = capi.lib()
    if not _READY:
        vp, i32 = C.c_void_p, C.c_int
        L.exb_host_last_error.restype = C.c_char_p
        L.exb_host_registered.argtypes = [C.c_char_p]
        L.exb_host_pipeline_create.argtypes = [C.c_char_p, C.c_char_p, i32, C.POINTER(vp)]
        L.exb_host_pipeline_destroy.argtypes = [vp]
        L.exb_host_pipeline_set_option.argtypes = [vp, C.c_char_p, i32]
        L.exb_host_pipeline_forward.argtypes = [vp, vp, i32, i32, i32, i32]
        L.exb_host_pipeline_num_outputs.argtypes = [vp]
        L.exb_host_pipeline_output_name.argtypes = [vp, i32, C.c_char_p, i32]
        L.exb_host_pipeline_get.argtypes = [vp, C.c_char_p, vp, C.c_int64, vp]
        L.exb_host_pipeline_output_ptr.argtypes = [vp, C.c_char_p, C.POINTER(C.POINTER(C.c_float)), vp]
        L.exb_host_pipeline_stats.argtypes = [vp, C.POINTER(i32), C.POINTER(C.c_double)]
        L.exb_host_pipeline_dump_profile.argtypes = [vp, C.c_char_p]
        L.exb_host_write_chrome_trace.argtypes = [C.c_char_p, i32, C.POINTER(C.c_char_p), vp, vp]
        L.exb_host_pipeline_run_resident.argtypes = [vp, i32, C.POINTER(C.c_double)]
        L.exb_host_pipeline_trace_size.argtypes = [vp]
        L.exb_host_pipeline_trace_entry.argtypes = [vp, i32, C.c_char_p, i32, C.POINTER(C.c_double),
                                                    C.POINTER(C.c_double)]
        L.exb_host_op_run.argtypes = [C.c_char_p, C.c_char_p, C.c_char_p, i32, i32, C.POINTER(vp), vp, vp,
                                      C.c_int64, vp]
        L.exb_host_convert_f32_to_f16.argtypes = [vp, vp, C.c_int64, i32, i32]
        L.exb_host_pipeline_f16_create.argtypes = [C.c_char_p, C.c_char_p, i32, C.POINTER(vp)]
        L.exb_host_pipeline_f16_destroy.argtypes = [vp]
        L.exb_host_pipeline_f16_set_option.argtypes = [vp, C.c_char_p, i32]
        L.exb_host_pipeline_f16_forward.argtypes = [vp, vp, i32, i32, i32, i32]
        L.exb_host_pipeline_f16_get.argtypes = [vp, C.c_char_p, vp, C.c_int64, vp]
        L.exb_host_pipeline_f16_stats.argtypes = [vp, C.POINTER(i32), C.POINTER(C.c_double)]
        L.exb_host_shard_bounds.argtypes = [i32, i32, i32, C.POINTER(i32), C.POINTER(i32)]
        L.exb_host_gather_rows.argtypes = [C.POINTER(vp), vp, i32, C.c_int64, vp]
        L.exb_host_sharded_create.argtypes = [C.c_char_p, C.c_char_p, vp, i32, C.POINTER(vp)]
        L.exb_host_sharded_destroy.argtypes = [vp]
        L.exb_host_sharded_set_option.argtypes = [vp, C.c_char_p, i32]
        L.exb_host_sharded_forward.argtypes = [vp, vp, i32, i32, i32, i32]
        L.exb_host_sharded_num_outputs.argtypes = [vp]
        L.exb_host_sharded_output_name.argtypes = [vp, i32, C.c_char_p, i32]
        L.exb_host_sharded_get.argtypes = [vp, C.c_char_p, vp, C.c_int64, vp]
        L.exb_host_sharded_device_ms.argtypes = [vp, C.POINTER(C.c_double)]
        _READY = True
    return L


def _check(rc):
    if rc == EXB_HOST_FATAL:
        raise HostError(rc, lib().exb_host_last_error().decode())
    if rc != 0:
        msg = lib().exb_host_last_error().decode()
        raise HostError(rc, msg if msg != "no error" else capi.last_error())


def registered(class_name):
    return bool(lib().exb_host_registered(class_name.encode()))


class Pipeline:
    """glasssix::excalibur::pipeline<float> on a GPU device."""

    def __init__(self, phai_text, racy_bytes=b"", device=0, fusion=True, cuda_graph=True):
        self._h = C.c_void_p()
        self._tmp = None
        path = b""
        if racy_bytes:
            self._tmp = tempfile.NamedTemporaryFile(suffix=".racy", delete=False)
            self._tmp.write(racy_bytes)
            self._tmp.close()
            path = self._tmp.name.encode()
        _check(lib().exb_host_pipeline_create(phai_text.encode(), path, device, C.byref(self._h)))
        self.set_option("fusion", int(fusion))
        self.set_option("cuda_graph", int(cuda_graph))

    def set_option(self, key, value):
        _check(lib().exb_host_pipeline_set_option(self._h, key.encode(), int(value)))

    def forward_ptr(self, host_ptr, N, Cc, H, W):
        """forward() on caller-owned host memory (fp32 NCHW); returns nothing, see get()."""
        _check(lib().exb_host_pipeline_forward(self._h, C.c_void_p(host_ptr), N, Cc, H, W))

    def forward(self, x_nchw):
        x = np.ascontiguousarray(x_nchw, np.float32)
        self._keep = x
        self.forward_ptr(x.ctypes.data, *x.shape)
        return {n: self.get(n) for n in self.output_names()}

    def output_names(self):
        buf = C.create_string_buffer(256)
        names = []
        for i in range(lib().exb_host_pipeline_num_outputs(self._h)):
            _check(lib().exb_host_pipeline_output_name(self._h, i, buf, 256))
            names.append(buf.value.decode())
        return names

    def get(self, name, out=None):
        shp = (C.c_int * 4)()
        _check(lib().exb_host_pipeline_get(self._h, name.encode(), None, 0, shp))
        if out is None:
            out = np.empty(tuple(shp), np.float32)
        _check(lib().exb_host_pipeline_get(self._h, name.encode(), out.ctypes.data, out.size, shp))
        return out

    def output_view(self, name):
        """Zero-copy numpy view of an output of the last forward (valid until the next forward)."""
        shp = (C.c_int * 4)()
        ptr = C.POINTER(C.c_float)()
        _check(lib().exb_host_pipeline_output_ptr(self._h, name.encode(), C.byref(ptr), shp))
        return np.ctypeslib.as_array(ptr, shape=tuple(shp))

    def stats(self):
        n, ms = C.c_int(), C.c_double()
        lib().exb_host_pipeline_stats(self._h, C.byref(n), C.byref(ms))
        return n.value, ms.value

    def run_resident(self, iters):
        """Device time (ms) of `iters` back-to-back runs of the fused plan on the resident input."""
        ms = C.c_double()
        _check(lib().exb_host_pipeline_run_resident(self._h, iters, C.byref(ms)))
        return ms.value

    def trace(self):
        """[(kernel/op name, begin_ms, end_ms)] of the last forward run with option profile=1."""
        out = []
        buf = C.create_string_buffer(256)
        b, e = C.c_double(), C.c_double()
        for i in range(lib().exb_host_pipeline_trace_size(self._h)):
            _check(lib().exb_host_pipeline_trace_entry(self._h, i, buf, 256, C.byref(b), C.byref(e)))
            out.append((buf.value.decode(), b.value, e.value))
        return out

    def dump_profile(self, path):
        _check(lib().exb_host_pipeline_dump_profile(self._h, path.encode()))

    def close(self):
        if self._h:
            lib().exb_host_pipeline_destroy(self._h)
            self._h = C.c_void_p()
        if self._tmp is not None:
            os.unlink(self._tmp.name)
            self._tmp = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class PipelineF16:
    """glasssix::excalibur::pipeline<unsigned short>: fp16 NCHW host tensors in and out (numpy float16)."""

    def __init__(self, phai_text, racy_bytes=b"", device=0, fusion=True):
        self._h = C.c_void_p()
        self._tmp = None
        path = b""
        if racy_bytes:
            self._tmp = tempfile.NamedTemporaryFile(suffix=".racy", delete=False)
            self._tmp.write(racy_bytes)
            self._tmp.close()
            path = self._tmp.name.encode()
        _check(lib().exb_host_pipeline_f16_create(phai_text.encode(), path, device, C.byref(self._h)))
        self.set_option("fusion", int(fusion))

    def set_option(self, key, value):
        _check(lib().exb_host_pipeline_f16_set_option(self._h, key.encode(), int(value)))

    def forward_ptr(self, host_ptr, N, Cc, H, W):
        _check(lib().exb_host_pipeline_f16_forward(self._h, C.c_void_p(host_ptr), N, Cc, H, W))

    def forward(self, x_nchw_f16):
        x = np.ascontiguousarray(x_nchw_f16, np.float16)
        self._keep = x
        self.forward_ptr(x.ctypes.data, *x.shape)

    def get(self, name, out=None):
        shp = (C.c_int * 4)()
        _check(lib().exb_host_pipeline_f16_get(self._h, name.encode(), None, 0, shp))
        if out is None:
            out = np.empty(tuple(shp), np.float16)
        _check(lib().exb_host_pipeline_f16_get(self._h, name.encode(), out.ctypes.data, out.size, shp))
        return out

    def stats(self):
        n, ms = C.c_int(), C.c_double()
        lib().exb_host_pipeline_f16_stats(self._h, C.byref(n), C.byref(ms))
        return n.value, ms.value

    def close(self):
        if self._h:
            lib().exb_host_pipeline_f16_destroy(self._h)
            self._h = C.c_void_p()
        if self._tmp is not None:
            os.unlink(self._tmp.name)
            self._tmp = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def write_chrome_trace(path, entries):
    """entries: [(name, begin_ms, end_ms)] -> chrome://tracing JSON (the writer behind Pipeline.dump_profile).  No GPU."""
    names = (C.c_char_p * len(entries))(*[e[0].encode() for e in entries])
    b = np.array([e[1] for e in entries], np.float64)
    e_ = np.array([e[2] for e in entries], np.float64)
    _check(lib().exb_host_write_chrome_trace(path.encode(), len(entries), names, b.ctypes.data, e_.ctypes.data))


def shard_bounds(total, world, rank):
    """[lo, hi) of shard `rank`: the host layer's rule (same as sharding.shard_bounds).  Needs no GPU."""
    lo, hi = C.c_int(), C.c_int()
    _check(lib().exb_host_shard_bounds(total, world, rank, C.byref(lo), C.byref(hi)))
    return lo.value, hi.value


def gather_rows(parts):
    """Concatenate float32 arrays along axis 0 with the host layer's gather.  Needs no GPU."""
    parts = [np.ascontiguousarray(a, np.float32) for a in parts]
    row = int(np.prod(parts[0].shape[1:])) if parts[0].ndim > 1 else 1
    out = np.empty((sum(a.shape[0] for a in parts),) + parts[0].shape[1:], np.float32)
    ptrs = (C.c_void_p * len(parts))(*[a.ctypes.data for a in parts])
    rows = np.array([a.shape[0] for a in parts], np.int32)
    _check(lib().exb_host_gather_rows(ptrs, rows.ctypes.data, len(parts), row, out.ctypes.data))
    return out


class ShardedPipeline:
    """glasssix::excalibur::sharded_pipeline: one batch cut into contiguous slices over several replicas
    (one pipeline<float> per entry of `devices`), outputs gathered by offset."""

    def __init__(self, phai_text, racy_bytes=b"", devices=(0,), fusion=True):
        self._h = C.c_void_p()
        self._tmp = None
        path = b""
        if racy_bytes:
            self._tmp = tempfile.NamedTemporaryFile(suffix=".racy", delete=False)
            self._tmp.write(racy_bytes)
            self._tmp.close()
            path = self._tmp.name.encode()
        dev = np.array(list(devices), np.int32)
        _check(lib().exb_host_sharded_create(phai_text.encode(), path, dev.ctypes.data, len(dev), C.byref(self._h)))
        self.set_option("fusion", int(fusion))

    def set_option(self, key, value):
        _check(lib().exb_host_sharded_set_option(self._h, key.encode(), int(value)))

    def forward_ptr(self, host_ptr, N, Cc, H, W):
        _check(lib().exb_host_sharded_forward(self._h, C.c_void_p(host_ptr), N, Cc, H, W))

    def forward(self, x_nchw):
        x = np.ascontiguousarray(x_nchw, np.float32)
        self._keep = x
        self.forward_ptr(x.ctypes.data, *x.shape)
        buf = C.create_string_buffer(256)
        out = {}
        for i in range(lib().exb_host_sharded_num_outputs(self._h)):
            _check(lib().exb_host_sharded_output_name(self._h, i, buf, 256))
            out[buf.value.decode()] = self.get(buf.value.decode())
        return out

    def get(self, name, out=None):
        shp = (C.c_int * 4)()
        _check(lib().exb_host_sharded_get(self._h, name.encode(), None, 0, shp))
        if out is None:
            out = np.empty(tuple(shp), np.float32)
        _check(lib().exb_host_sharded_get(self._h, name.encode(), out.ctypes.data, out.size, shp))
        return out

    def device_ms(self):
        ms = C.c_double()
        _check(lib().exb_host_sharded_device_ms(self._h, C.byref(ms)))
        return ms.value

    def close(self):
        if self._h:
            lib().exb_host_sharded_destroy(self._h)
            self._h = C.c_void_p()
        if self._tmp is not None:
            os.unlink(self._tmp.name)
            self._tmp = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def run_op(type_, params, inputs, racy_bytes=None, device=0):
    """Create one operation through the reflector and run its forward_gpu on fp32 NCHW arrays."""
    ins = [np.ascontiguousarray(a, np.float32) for a in inputs]
    ptrs = (C.c_void_p * len(ins))(*[a.ctypes.data for a in ins])
    shapes = np.array([list(a.shape) for a in ins], np.int32)
    tmp = None
    path = b""
    if racy_bytes:
        tmp = tempfile.NamedTemporaryFile(suffix=".racy", delete=False)
        tmp.write(racy_bytes)
        tmp.close()
        path = tmp.name.encode()
    try:
        shp = (C.c_int * 4)()
        # the output shape is only known after running, so run into a generous buffer
        cap = max(int(a.size) for a in ins) * 64 + 1024
        out = np.empty(cap, np.float32)
        _check(lib().exb_host_op_run(type_.encode(), params.encode(), path, device, len(ins), ptrs,
                                     shapes.ctypes.data, out.ctypes.data, cap, shp))
        n = int(np.prod(tuple(shp)))
        return out[:n].reshape(tuple(shp)).copy()
    finally:
        if tmp is not None:
            os.unlink(tmp.name)


def convert_f32_to_f16(x, threads=1, force_scalar=False):
    """The host-side conversion the "host_f16_threads" option uses; returns a float16 array.  No GPU needed."""
    src = np.ascontiguousarray(x, np.float32)
    dst = np.empty(src.shape, np.float16)
    _check(lib().exb_host_convert_f32_to_f16(src.ctypes.data_as(C.c_void_p), dst.ctypes.data_as(C.c_void_p),
                                             C.c_int64(src.size), int(threads), int(bool(force_scalar))))
    return dst
