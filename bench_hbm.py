"""Bandwidth-bound kernels against the HBM roofline, on the shapes the benchmark networks use.

    python bench_hbm.py [--batch 256] [--iters 20]

Per kernel: CUDA-event time of one launch, algorithmic bytes (every operand once at its storage
width) and the resulting GB/s, as a fraction of the measured HBM copy bandwidth in
MEASURED_PEAKS.json (6650 GB/s when the file is absent).  Tensors are larger than the 126 MB L2 at
the default batch, so no L2 flush is needed between launches.
"""
import argparse
import json
import os

import numpy as np

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from excalibur_b200 import capi  # noqa: E402

ROOT = os.path.dirname(os.path.abspath(__file__))


def _time(torch, fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main(argv=None):
    import torch
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args(argv)
    N = args.batch
    try:
        peak = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]
        src = "measured"
    except Exception:
        peak, src = 6650.0, "fallback"
    torch.cuda.set_device(0)
    ctx = capi.Context(0)
    rng = np.random.default_rng(0)
    rows = []

    def report(name, ms, byts):
        gbs = byts / ms / 1e6
        rows.append((name, ms, gbs, gbs / peak))
        print("%-44s %8.3f ms  %8.1f GB/s  %5.1f %% of %s HBM peak" % (name, ms, gbs, 100 * gbs / peak, src), flush=True)

    def f16(*shape):
        return torch.randn(shape, device="cuda", dtype=torch.float16)

    # depthwise 3x3 (MobileNetV2-style layers), fp16 NHWC
    for name, C, hw, s in (("dw3x3 s1 32ch @112", 32, 112, 1), ("dw3x3 s2 96ch @112", 96, 112, 2),
                           ("dw3x3 s1 144ch @56", 144, 56, 1), ("dw3x3 s2 144ch @56", 144, 56, 2),
                           ("dw3x3 s1 384ch @14", 384, 14, 1), ("dw3x3 s1 960ch @7", 960, 7, 1)):
        cs = (C + 31) // 32 * 32
        d = capi.make_dw_desc(N, hw, hw, C, 3, s, 1, act=capi.ACT_RELU6, c_stride=cs)
        w = capi.DwWeights(ctx, d, rng.standard_normal((C, 3, 3)).astype(np.float32), np.zeros(C, np.float32))
        x = f16(N, hw, hw, cs)
        oh = (hw + 2 - 3) // s + 1
        y = torch.empty((N, oh, oh, cs), device="cuda", dtype=torch.float16)
        ms = _time(torch, lambda: capi.dwconv2d(ctx, d, x, w, y), args.iters)
        report(name, ms, (x.numel() + y.numel()) * 2 + C * 9 * 4)
    # pooling
    x = f16(N, 112, 112, 64)
    d = capi.make_pool_desc(N, 112, 112, 64, 0, 3, 2, 1, dtype=capi.EXB_F16, out2_dtype=capi.EXB_I8, out2_scale=10.0)
    y = torch.empty((N, 56, 56, 64), device="cuda", dtype=torch.float16)
    y2 = torch.empty((N, 56, 56, 64), device="cuda", dtype=torch.int8)
    report("max pool 3x3/2 64ch @112 -> fp16 + int8", _time(torch, lambda: capi.pool2d(ctx, d, x, y, y2), args.iters),
           x.numel() * 2 + y.numel() * 3)
    x = f16(max(N // 8, 1), 20, 20, 256)
    d = capi.make_pool_desc(x.shape[0], 20, 20, 256, 0, 5, 1, 2, dtype=capi.EXB_F16)
    y = torch.empty_like(x)
    report("max pool 5x5/1 256ch @20 (batch/8)", _time(torch, lambda: capi.pool2d(ctx, d, x, y), args.iters), x.numel() * 4)
    x = f16(N, 7, 7, 512)
    d = capi.make_pool_desc(N, 7, 7, 512, 1, 7, 1, 0, global_pool=True, dtype=capi.EXB_F16)
    y = torch.empty((N, 1, 1, 512), device="cuda", dtype=torch.float16)
    report("global average pool 512ch @7", _time(torch, lambda: capi.pool2d(ctx, d, x, y), args.iters),
           (x.numel() + y.numel()) * 2)
    # element-wise
    a, b = f16(N, 56, 56, 64), f16(N, 56, 56, 64)
    y = torch.empty_like(a)
    report("eltwise sum, 2 inputs, 64ch @56 fp16", _time(torch, lambda: capi.eltwise(ctx, [a, b], 1, None, y), args.iters),
           a.numel() * 6)
    report("binary add 64ch @56 fp16", _time(torch, lambda: capi.binaryop(ctx, a, b, 0, y), args.iters), a.numel() * 6)
    report("ReLU 64ch @56 fp16", _time(torch, lambda: capi.relu(ctx, a, y), args.iters), a.numel() * 4)
    q = torch.empty(a.shape, device="cuda", dtype=torch.int8)
    report("quantise fp16 -> int8 64ch @56", _time(torch, lambda: capi.quantize(ctx, a, 20.0, 1, q), args.iters), a.numel() * 3)
    # layout edge and glue
    x32 = torch.rand((N, 3, 224, 224), device="cuda", dtype=torch.float32)
    pitch = (224 + 4 + 8 + 7) // 8 * 8
    yp = torch.empty((N, 224, pitch, 4), device="cuda", dtype=torch.float16)
    report("ingest fp32 NCHW -> NHWC4 fp16 rows @224",
           _time(torch, lambda: capi.nchw_f32_to_nhwc_padded(ctx, x32, capi.EXB_F16, 4, 4, pitch, y=yp), args.iters),
           x32.numel() * 4 + yp.numel() * 2)
    xs = [f16(max(N // 8, 1), 40, 40, 128) for _ in range(2)]
    yc = torch.empty((xs[0].shape[0], 40, 40, 256), device="cuda", dtype=torch.float16)
    report("concat 2 x 128ch @40 (batch/8)", _time(torch, lambda: capi.concat_channels(ctx, xs, y=yc), args.iters),
           yc.numel() * 4)
    xi = f16(max(N // 8, 1), 20, 20, 256)
    yi = torch.empty((xi.shape[0], 40, 40, 256), device="cuda", dtype=torch.float16)
    report("nearest 2x resize 256ch @20 (batch/8)", _time(torch, lambda: capi.interp_nearest(ctx, xi, 40, 40, y=yi), args.iters),
           (xi.numel() + yi.numel()) * 2)
    # the kernels added for the shipped model descriptions
    a = f16(N, 64, 64, 64)
    y = torch.empty_like(a)
    sl = torch.rand(64, device="cuda") * 0.3
    mul, add = torch.rand(64, device="cuda") + 0.5, torch.randn(64, device="cuda")
    report("PReLU 64ch @64 fp16", _time(torch, lambda: capi.prelu(ctx, a, sl, y=y), args.iters), a.numel() * 4)
    report("BatchNorm + LeakyRelu 64ch @64 fp16, one pass",
           _time(torch, lambda: capi.channel_affine_prelu(ctx, a, mul, add, sl[:1], y=y), args.iters), a.numel() * 4)
    gate = f16(N, 1, 1, 64)
    check = capi.check
    report("per-channel gate (N,C,H,W) x (N,C,1,1) 64ch @64",
           _time(torch, lambda: check(capi.lib().exb_binaryop_channel_bcast_fwd(
               ctx.handle, 2, capi.ptr(a), capi.ptr(gate), 0, capi.ptr(y), N, N, 64, 64, 64 * 64, capi.EXB_F16, 1,
               capi.cur_stream())), args.iters), a.numel() * 4)
    xd = f16(max(N // 4, 1), 80, 80, 256)
    yd = torch.empty((xd.shape[0], 160, 160, 64), device="cuda", dtype=torch.float16)
    report("depth-to-space 2x2 64ch @80 (batch/4)", _time(torch, lambda: capi.depth_to_space(ctx, xd, 2, 2, 64, y=yd), args.iters),
           xd.numel() * 4)
    x640 = torch.rand((max(N // 8, 1), 3, 640, 640), device="cuda", dtype=torch.float32)
    yf = torch.empty((x640.shape[0], 320, 320, 16), device="cuda", dtype=torch.float16)
    report("normalise + Focus + ingest fp32 @640 (batch/8)",
           _time(torch, lambda: capi.focus_ingest(ctx, x640, 16, mul[:3], add[:3], y=yf), args.iters),
           x640.numel() * 4 + yf.numel() * 2)
    xt = torch.rand((max(N // 8, 1) * 3, 85, 6400), device="cuda", dtype=torch.float32)
    yt = torch.empty((xt.shape[0], 6400, 85), device="cuda", dtype=torch.float32)
    report("transpose 85 x 6400 planes fp32 (batch/8 x 3)", _time(torch, lambda: capi.transpose_hw(ctx, xt, y=yt), args.iters),
           xt.numel() * 8)
    ctx.sync_check()
    ctx.close()
    return rows


if __name__ == "__main__":
    main()
