"""Whole-network throughput of the benchmark configurations other than the headline one.

    python bench_nets.py [--net resnet18_fp16,resnet18_int8,mobilenetv2_fp16,mobilenetv2_int8,yolov5s_fp16,
                                              det_db_resnet18_fp16,mobile_unicorn_fp16,yolov5s_simp_fp16,unicorn_light_fp16,unicorn_light_int8]
                                       [--batch B] [--size S] [--iters K] [--trace | --trace-all]

Per network: images/s with the input resident on the device (CUDA-graph replays, CUDA events on the
plan's stream) and end to end (pinned host input, H2D and D2H inside the timed region).  Defaults
follow the benchmark configurations: ResNet-18-style fp16 batch 64 / int8 batch 256 at 224x224,
MobileNetV2-style batch 256 at 224x224, YOLOv5s-style batch 32 at 640x640; the DB text detector batch 8 at
640x640, the MobileFaceNet-style embedding net batch 256 at 128x128 (its fixed size) and the shipped
YOLOv5s variant batch 32 at 640x640 (--size does not apply to the last two).  Weights are seeded
random tensors; int8 scales come from a max-abs calibration pass of 8 seeded images through this
library's own floating-point pipeline.  --trace prints the ten slowest steps of the plan.
"""
import argparse
import time

import numpy as np

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from excalibur_b200 import host, model_zoo, models  # noqa: E402

NETS = {
    # name: (builder, int8, batch, size)
    "resnet18_fp16": (models.resnet18, False, 64, 224),
    "resnet18_int8": (models.resnet18, True, 256, 224),
    "mobilenetv2_fp16": (models.mobilenet_v2, False, 256, 224),
    "mobilenetv2_int8": (models.mobilenet_v2, True, 256, 224),
    "yolov5s_fp16": (models.yolov5s, False, 32, 640),
    # the architectures of three model descriptions the reference ships (model_zoo), seeded random weights
    "det_db_resnet18_fp16": (model_zoo.det_db_resnet18, False, 8, 640),
    "mobile_unicorn_fp16": (model_zoo.mobile_unicorn, False, 256, 128),
    "yolov5s_simp_fp16": (lambda **kw: model_zoo.yolov5s_simp(size=640, **kw), False, 32, 640),
    "unicorn_light_fp16": (model_zoo.unicorn_light, False, 256, 128),
    "unicorn_light_int8": (model_zoo.unicorn_light, True, 256, 128),
}


def build(name, device, size):
    builder, int8, _, _ = NETS[name]
    g, info = builder()
    if int8:
        p = host.Pipeline(g.phai_text(), g.racy_bytes(), device, fusion=False)
        hi = 255 if "Input" in g.phai_text() else 1
        calib = np.random.default_rng(77).uniform(0, hi, (8, 3, size, size)).astype(np.float32)
        scales = models.calibrate(p, info["conv_inputs"], calib)
        p.close()
        g, info = builder(act_scales=scales)
    return g, info


def main(argv=None):
    import torch
    ap = argparse.ArgumentParser()
    ap.add_argument("--net", default=",".join(NETS))
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--size", type=int, default=0)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--trace", action="store_true")
    ap.add_argument("--trace-all", action="store_true", help="every step of the plan in execution order")
    args = ap.parse_args(argv)
    torch.cuda.set_device(0)
    for name in args.net.split(","):
        _, _, batch, size = NETS[name]
        batch = args.batch or batch
        size = args.size or size
        g, info = build(name, 0, size)
        pipe = host.Pipeline(g.phai_text(), g.racy_bytes(), 0, fusion=True)
        x = torch.empty((batch, 3, size, size), dtype=torch.float32).pin_memory()
        x.uniform_(0, 255 if "Input" in g.phai_text() else 1, generator=torch.Generator().manual_seed(1))
        outs = None
        for _ in range(3):      # eager, capture, replay
            pipe.forward_ptr(x.data_ptr(), batch, 3, size, size)
            outs = {n: pipe.get(n) for n in pipe.output_names()}
        launches, _ = pipe.stats()
        pipe.run_resident(3)
        ms = pipe.run_resident(args.iters) / args.iters
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(args.iters):
            pipe.forward_ptr(x.data_ptr(), batch, 3, size, size)
            for n in outs:
                pipe.output_view(n)      # the host tensors forward() returns, no second copy
        e2e = (time.perf_counter() - t0) / args.iters
        finite = all(np.isfinite(v).all() for v in outs.values())
        print("%-18s batch %3d @%d  %4d launches  %8.3f ms/step  %9.0f images/s resident  %9.0f images/s end-to-end  finite=%s"
              % (name, batch, size, launches, ms, batch / ms * 1e3, batch / e2e, finite), flush=True)
        if args.trace or args.trace_all:
            pipe.set_option("profile", 1)
            pipe.forward_ptr(x.data_ptr(), batch, 3, size, size)
            tr = pipe.trace() if args.trace_all else sorted(pipe.trace(), key=lambda t: t[1] - t[2])[:10]
            pipe.set_option("profile", 0)
            for n, b, e in tr:
                print("    %-28s %8.3f ms" % (n, e - b))
        pipe.close()


if __name__ == "__main__":
    main()
