"""The tensor-peak probe (tcgen05.mma back to back on operands resident in shared memory): every shape / layout the
benchmark tools ask for runs to completion, reports the operation count it issued, and leaves the context usable."""
import ctypes as C

import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype_name", ["i8", "f16"])
@pytest.mark.parametrize("m,n,ctas", [(128, 64, 2), (128, 256, 1), (64, 128, 2)])
def test_probe_runs_and_counts_its_work(ctx, dtype_name, m, n, ctas):
    import torch
    from excalibur_b200 import capi
    L = capi.lib()
    dt = capi.EXB_I8 if dtype_name == "i8" else capi.EXB_F16
    ops = C.c_double()
    cyc = torch.zeros(1, dtype=torch.int64, device="cuda")
    kblk, iters = 2, 64
    capi.check(L.exb_tensor_peak_probe_layout(ctx.handle, dt, m, n, ctas, kblk, iters, 128, 1024, 0, C.byref(ops),
                                              cyc.data_ptr(), capi.cur_stream()))
    ctx.sync_check()
    k_per_mma = 32 if dtype_name == "i8" else 16
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    assert ops.value == 2.0 * m * n * k_per_mma * 4 * kblk * iters * sms * ctas
    assert int(cyc.item()) > 0


def test_probe_layout_of_a_row_box_and_bad_arguments(ctx):
    import torch
    from excalibur_b200 import capi
    L = capi.lib()
    ops = C.c_double()
    # 64-byte K rows, groups a 10-pixel box row apart, descriptor two pixels into the box: the row-box loop's A operand
    capi.check(L.exb_tensor_peak_probe_layout(ctx.handle, capi.EXB_I8, 128, 64, 2, 2, 32, 64, 640, 128, C.byref(ops), None,
                                              capi.cur_stream()))
    ctx.sync_check()
    assert ops.value > 0
    assert L.exb_tensor_peak_probe_layout(ctx.handle, capi.EXB_I8, 96, 64, 2, 2, 32, 64, 640, 128, C.byref(ops), None,
                                          capi.cur_stream()) != 0      # M must be 64 or 128
    assert L.exb_tensor_peak_probe(ctx.handle, capi.EXB_F32, 64, 1, 2, 32, C.byref(ops), None, capi.cur_stream()) != 0
    ctx.sync_check()
