"""Per-layer timing of the hot-path kernels on the shapes of the ResNet-18-style network.

    python bench_layers.py [--batch 256] [--layers s1_conv1,s1_conv2,...] [--iters 20]

Prints, per layer, the CUDA-event time of one launch and the algorithmic TFLOP/s and GB/s
(FLOP = 2*N*OH*OW*Cout*Cin*kh*kw; bytes = every operand once at its storage width).  With
--iters 1 --warmup 0 it launches each selected kernel exactly once, which is the form used for
profiler captures.
"""
import argparse
import sys

import numpy as np

import os

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from excalibur_b200 import capi  # noqa: E402

# name: (Cin, H=W, Cout, k, stride, pad, kind)   kind: conv1 = int8 -> int8 + ReLU,
# conv2 = int8 + fp16 residual -> fp16 + int8 + ReLU, proj = int8 -> fp16
LAYERS = {
    "s1_conv1": (64, 56, 64, 3, 1, 1, "conv1"), "s1_conv2": (64, 56, 64, 3, 1, 1, "conv2"),
    "s2_conv1a": (64, 56, 128, 3, 2, 1, "conv1"), "s2_proj": (64, 56, 128, 1, 2, 0, "proj"),
    "s2_conv1": (128, 28, 128, 3, 1, 1, "conv1"), "s2_conv2": (128, 28, 128, 3, 1, 1, "conv2"),
    "s3_conv1a": (128, 28, 256, 3, 2, 1, "conv1"), "s3_proj": (128, 28, 256, 1, 2, 0, "proj"),
    "s3_conv1": (256, 14, 256, 3, 1, 1, "conv1"), "s3_conv2": (256, 14, 256, 3, 1, 1, "conv2"),
    "s4_conv1a": (256, 14, 512, 3, 2, 1, "conv1"), "s4_proj": (256, 14, 512, 1, 2, 0, "proj"),
    "s4_conv1": (512, 7, 512, 3, 1, 1, "conv1"), "s4_conv2": (512, 7, 512, 3, 1, 1, "conv2"),
}
EXTRA = ("stem", "pool1", "stem_pool")


def _timeit(torch, fn, iters, warmup):
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
    ap.add_argument("--layers", default=",".join(list(LAYERS) + list(EXTRA)))
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--sets", type=int, default=1,
                    help="conv layers: rotate through this many copies of the activations (input, residual, outputs); with "
                         "one copy a narrow layer's tensors stay in the 126 MB L2 between launches, with enough copies to "
                         "exceed it every launch reads from HBM as it does inside a network")
    args = ap.parse_args(argv)
    N = args.batch
    torch.cuda.set_device(0)
    ctx = capi.Context(0)
    rng = np.random.default_rng(0)
    for name in args.layers.split(","):
        if name in LAYERS:
            cin, hw, cout, k, s, p, kind = LAYERS[name]
            res = kind == "conv2"
            out = capi.EXB_I8 if kind == "conv1" else capi.EXB_F16
            out2 = capi.EXB_I8 if res else -1
            d = capi.make_conv_desc(N, hw, hw, cin, cout, k, s, p, capi.EXB_I8, out, out2, res,
                                    capi.ACT_NONE if kind == "proj" else capi.ACT_RELU, 0.05, 0.05)
            oh, ow = capi.conv_out_dims(d)
            wq = rng.integers(-127, 128, (cout, cin, k, k)).astype(np.int8)
            wp = capi.ConvWeights(ctx, d, wq, np.zeros(cout, np.float32), np.full(cout, 40.0, np.float32), 30.0)
            sets = []
            for _ in range(max(1, args.sets)):
                x = torch.randint(-128, 128, (N, hw, hw, cin), device="cuda", dtype=torch.int32).to(torch.int8)
                r = torch.randn((N, oh, ow, cout), device="cuda", dtype=torch.float16) if res else None
                y = torch.empty((N, oh, ow, cout), device="cuda", dtype=capi.torch_dtype(out))
                y2 = torch.empty((N, oh, ow, cout), device="cuda", dtype=torch.int8) if res else None
                sets.append((x, r, y, y2))
            turn = [0]

            def launch():
                xs, rs, ys, y2s = sets[turn[0] % len(sets)]
                turn[0] += 1
                capi.conv2d(ctx, d, xs, wp, rs, ys, y2s)

            ms = _timeit(torch, launch, args.iters, args.warmup)
            flop = 2.0 * N * oh * ow * cout * cin * k * k
            byts = x.numel() + y.numel() * y.element_size() + (r.numel() * 2 + y2.numel() if res else 0) + wq.size
        elif name == "stem":
            pitch = (224 + 4 + 8 + 7) // 8 * 8
            d = capi.make_conv_desc(N, 224, 224, 3, 64, 7, 2, 3, capi.EXB_F16, capi.EXB_F16, act=capi.ACT_RELU,
                                    cin_stride=4, x_w_pitch=pitch, x_w_pad=4)
            wp = capi.ConvWeights(ctx, d, rng.standard_normal((64, 3, 7, 7)).astype(np.float32), np.zeros(64, np.float32))
            x = torch.zeros((N, 224, pitch, 4), device="cuda", dtype=torch.float16)
            x[:, :, 4:228, :3] = torch.rand((N, 224, 224, 3), device="cuda").to(torch.float16)
            y = torch.empty((N, 112, 112, 64), device="cuda", dtype=torch.float16)
            ms = _timeit(torch, lambda: capi.conv2d(ctx, d, x, wp, None, y, None), args.iters, args.warmup)
            flop = 2.0 * N * 112 * 112 * 64 * 147
            byts = x.numel() * 2 + y.numel() * 2
        elif name == "stem_pool":     # stem + ReLU + 3x3/2 max pool in one kernel, fp16 + int8 pooled outputs
            pitch = (224 + 4 + 8 + 7) // 8 * 8
            d = capi.make_conv_desc(N, 224, 224, 3, 64, 7, 2, 3, capi.EXB_F16, capi.EXB_F16, capi.EXB_I8, act=capi.ACT_RELU,
                                    out2_scale=10.0, cin_stride=4, x_w_pitch=pitch, x_w_pad=4, fuse_pool=1)
            wp = capi.ConvWeights(ctx, d, rng.standard_normal((64, 3, 7, 7)).astype(np.float32), np.zeros(64, np.float32))
            x = torch.zeros((N, 224, pitch, 4), device="cuda", dtype=torch.float16)
            x[:, :, 4:228, :3] = torch.rand((N, 224, 224, 3), device="cuda").to(torch.float16)
            y = torch.empty((N, 56, 56, 64), device="cuda", dtype=torch.float16)
            y2 = torch.empty((N, 56, 56, 64), device="cuda", dtype=torch.int8)
            ms = _timeit(torch, lambda: capi.conv2d(ctx, d, x, wp, None, y, y2), args.iters, args.warmup)
            flop = 2.0 * N * 112 * 112 * 64 * 147
            byts = x.numel() * 2 + y.numel() * 3
        elif name == "pool1":
            x = torch.randn((N, 112, 112, 64), device="cuda", dtype=torch.float16)
            d = capi.make_pool_desc(N, 112, 112, 64, 0, 3, 2, 1, dtype=capi.EXB_F16, out2_dtype=capi.EXB_I8, out2_scale=10.0)
            y = torch.empty((N, 56, 56, 64), device="cuda", dtype=torch.float16)
            y2 = torch.empty((N, 56, 56, 64), device="cuda", dtype=torch.int8)
            ms = _timeit(torch, lambda: capi.pool2d(ctx, d, x, y, y2), args.iters, args.warmup)
            flop = 0.0
            byts = x.numel() * 2 + y.numel() * 3
        else:
            print("unknown layer", name, file=sys.stderr)
            continue
        ctx.sync_check()
        print("%-10s %8.3f ms  %8.1f TFLOP/s  %8.1f GB/s" % (name, ms, flop / ms / 1e9, byts / ms / 1e6), flush=True)
    ctx.close()


if __name__ == "__main__":
    main()
