"""The allocation-free pooling entry point (exb_pool2d_nchw_f32_static) against the regular entry
points.  Who needs it: code that may not allocate while it runs inference - a host that handed
out all device memory at start-up, a real-time loop under a no-malloc rule, a plug-in that must
not enter the application's allocator - so the NHWC intermediates come from a buffer built into
the library instead of from the caller.

Collected last on purpose: a run that stops at the first failure has then already run every other
test.  The test is self-contained (own context, own tensors), so it also passes alone in a fresh
process.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


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
        # beyond the built-in buffer: refused with a clear message, nothing launched
        big = capi.make_pool_desc(64, 224, 224, 64, type=0, k=3, stride=2, pad=1, dtype=capi.EXB_F32)
        rc = capi.lib().exb_pool2d_nchw_f32_static(0, C.byref(big), None, None, None)
        assert rc == capi.EXB_ERR_NOMEM
        assert "built-in" in capi.last_error()
        # unsupported element types are refused too
        half = capi.make_pool_desc(1, 8, 8, 8, type=0, k=2, stride=2, dtype=capi.EXB_F16)
        assert capi.lib().exb_pool2d_nchw_f32_static(0, C.byref(half), None, None, None) == capi.EXB_ERR_UNSUPPORTED
    finally:
        ctx.close()
