"""The allocation-free pooling entry point (exb_pool2d_nchw_f32_static) against the regular entry
points and against the CPU oracle's pooling (the restatement of the reference's
operation_pooling.cpp:128-210).  Who needs it: code that may not allocate while it runs inference - a
host that handed out all device memory at start-up, a real-time loop under a no-malloc rule, a plug-in that must
not enter the application's allocator - so the NHWC intermediates come from a buffer built into
the library instead of from the caller.

Collected last on purpose: a run that stops at the first failure has then already run every other
test.  The test is self-contained (own context, own tensors), so it also passes alone in a fresh
process.
"""
import ctypes as C

import numpy as np
import pytest

from oracle import exb_oracle as O

pytestmark = pytest.mark.gpu

SCRATCH_BYTES = 16 << 20      # size of the buffer built into the library


def _oracle_kw(kw):
    """make_pool_desc keywords -> oracle keywords."""
    o = dict(type=kw.get("type", 0), global_pool=kw.get("global_pool", False))
    if not o["global_pool"]:
        o.update(kernel=kw["k"], stride=kw["stride"], pad=kw.get("pad", 0))
    for k in ("pad_mode", "count_include_pad"):
        if k in kw:
            o[k] = kw[k]
    return o


def _regular_path(capi, ctx, x, desc_kw):
    """NCHW fp32 -> NHWC, exb_pool2d_fwd, NHWC -> NCHW fp32 with caller-allocated intermediates."""
    N, Cc, H, W = x.shape
    cs = (Cc + 3) // 4 * 4
    xh = capi.nchw_f32_to_nhwc(ctx, x, capi.EXB_F32, c_stride=cs)
    d = capi.make_pool_desc(N, H, W, Cc, dtype=capi.EXB_F32, c_stride=cs, **desc_kw)
    yh, _ = capi.pool2d(ctx, d, xh)
    return capi.nhwc_to_nchw_f32(ctx, yh, Cc)


def test_static_pooling_matches_regular_entry_points_twice_in_a_row():
    import torch
    from excalibur_b200 import capi
    torch.cuda.set_device(0)
    ctx = capi.Context(0)
    try:
        g = torch.Generator(device="cuda").manual_seed(11)
        calls = [
            ((2, 64, 56, 56), dict(type=0, k=3, stride=2, pad=1)),                          # ResNet stem pool
            ((3, 10, 17, 23), dict(type=1, k=3, stride=2, pad=1, count_include_pad=1)),     # ragged, channels not x4
            ((4, 96, 7, 7), dict(type=1, global_pool=True)),
            ((2, 5, 9, 11), dict(type=0, k=2, stride=2, pad=0, pad_mode=0)),               # ceil mode: last window overhangs
            ((3, 7, 10, 13), dict(type=1, k=3, stride=2, pad=0, pad_mode=0, count_include_pad=0)),
        ]
        for shape, kw in calls:      # consecutive calls share the built-in buffer
            x = torch.randn(shape, generator=g, device="cuda", dtype=torch.float32)
            ref = _regular_path(capi, ctx, x, kw)
            d = capi.make_pool_desc(shape[0], shape[2], shape[3], shape[1], dtype=capi.EXB_F32, **kw)
            y = torch.full_like(ref, float("nan"))
            stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
            capi.check(capi.lib().exb_pool2d_nchw_f32_static(0, C.byref(d), capi.ptr(x), capi.ptr(y), stream))
            torch.cuda.synchronize()
            assert y.shape == ref.shape
            assert torch.equal(y, ref), "static pooling differs from the regular entry points for %r" % (shape,)
            cpu = O.pool2d_f32(x.cpu().numpy(), **_oracle_kw(kw))
            assert cpu.shape == tuple(y.shape), (cpu.shape, tuple(y.shape))
            if kw.get("type", 0) == 0:
                np.testing.assert_array_equal(y.cpu().numpy(), cpu)                 # max pooling: exact
            else:
                np.testing.assert_allclose(y.cpu().numpy(), cpu, rtol=1e-6, atol=1e-6)   # fp32 summation order
        # exactly at the limit: 1x1 "pooling" of C=4 channels, in + out = 2 * N*H*W*16 bytes = 16 MiB
        n_px = SCRATCH_BYTES // 2 // 16
        x = torch.randn((1, 4, 512, n_px // 512), generator=g, device="cuda", dtype=torch.float32)
        assert x.numel() * 4 * 2 == SCRATCH_BYTES
        d = capi.make_pool_desc(1, 512, n_px // 512, 4, type=0, k=1, stride=1, pad=0, dtype=capi.EXB_F32)
        y = torch.full_like(x, float("nan"))
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        capi.check(capi.lib().exb_pool2d_nchw_f32_static(0, C.byref(d), capi.ptr(x), capi.ptr(y), stream))
        torch.cuda.synchronize()
        assert torch.equal(y, x)
        # one more row (more than 256 bytes over): refused
        d = capi.make_pool_desc(1, 513, n_px // 512, 4, type=0, k=1, stride=1, pad=0, dtype=capi.EXB_F32)
        assert capi.lib().exb_pool2d_nchw_f32_static(0, C.byref(d), capi.ptr(x), capi.ptr(y), stream) == capi.EXB_ERR_NOMEM
        # beyond the built-in buffer: refused with a clear message, nothing launched
        big = capi.make_pool_desc(64, 224, 224, 64, type=0, k=3, stride=2, pad=1, dtype=capi.EXB_F32)
        rc = capi.lib().exb_pool2d_nchw_f32_static(0, C.byref(big), None, None, None)
        assert rc == capi.EXB_ERR_NOMEM
        assert "built-in" in capi.last_error()
        # unsupported element types are refused too
        half = capi.make_pool_desc(1, 8, 8, 8, type=0, k=2, stride=2, dtype=capi.EXB_F16)
        assert capi.lib().exb_pool2d_nchw_f32_static(0, C.byref(half), None, None, None) == capi.EXB_ERR_UNSUPPORTED
        # a device index below the entry point's own limit that does not exist: a host-side CUDA error, reported once;
        # the caller's current device is untouched and the library keeps working afterwards
        small = capi.make_pool_desc(1, 8, 8, 8, type=0, k=2, stride=2, dtype=capi.EXB_F32)
        xs = torch.randn((1, 8, 8, 8), generator=g, device="cuda", dtype=torch.float32)
        ys = torch.empty((1, 8, 4, 4), device="cuda", dtype=torch.float32)
        rc = capi.lib().exb_pool2d_nchw_f32_static(63, C.byref(small), capi.ptr(xs), capi.ptr(ys), None)
        assert rc == capi.EXB_ERR_CUDA, rc
        assert torch.cuda.current_device() == 0
        ref = _regular_path(capi, ctx, xs, dict(type=0, k=2, stride=2))      # launches after the error still succeed
        capi.check(capi.lib().exb_pool2d_nchw_f32_static(0, C.byref(small), capi.ptr(xs), capi.ptr(ys), None))
        torch.cuda.synchronize()
        assert torch.equal(ys, ref)
    finally:
        ctx.close()
