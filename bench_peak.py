#!/usr/bin/env python
"""Measured tensor-core peaks of this GPU with the library's own tcgen05.mma stream (no TMA, no epilogue,
operands resident in shared memory): the denominator of the convolution kernel's tensor roofline.

    python bench_peak.py [--seconds 2.0] [--m64] [--json out.json]

For int8 (s8 x s8 -> s32) and fp16 (-> fp32), M = 128, N in 64 / 128 / 256, one and two CTAs per SM:
  burst     best single launch (~0.3 ms) after warm-up, CUDA events
  sustained launches back to back for --seconds, total work / total device time, with the SM clock
            sampled by nvidia-smi during that loop
Prints one JSON object; `int8_peak_tops` / `f16_peak_tflops` are the best burst figures over all shapes,
`*_sustained` the best sustained ones.
"""
import argparse
import ctypes as C
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def probe(ctx, dtype, n, ctas, seconds, sampler_cls=None, device=0, m=128):
    import torch
    from excalibur_b200 import capi
    L = capi.lib()
    kblk = 2 if ctas == 2 else 4
    ops = C.c_double()
    cyc = torch.zeros(1, dtype=torch.int64, device="cuda")

    def launch(iters):
        # dense 128-byte K blocks: 1024 bytes between 8-row groups, descriptor at the start of its region
        capi.check(L.exb_tensor_peak_probe_layout(ctx.handle, dtype, m, n, ctas, kblk, iters, 128, 1024, 0, C.byref(ops),
                                                  cyc.data_ptr(), capi.cur_stream()))

    # size a launch to about 0.3 ms from a first guess
    iters = 256
    launch(iters)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    launch(iters)
    e1.record()
    torch.cuda.synchronize()
    ms = max(e0.elapsed_time(e1), 1e-3)
    iters = int(max(16, min(1 << 18, iters * 0.3 / ms)))
    best = 0.0
    cycles_per_mma = None
    for _ in range(5):
        e0.record()
        launch(iters)
        e1.record()
        torch.cuda.synchronize()
        rate = ops.value / (e0.elapsed_time(e1) * 1e-3) / 1e12
        if rate > best:
            best = rate
            cycles_per_mma = float(cyc.item()) / (iters * kblk * 4)
    ctx.sync_check()
    out = {"m": m, "n": n, "ctas_per_sm": ctas, "burst": round(best, 1), "sm_cycles_per_mma": round(cycles_per_mma, 1)}
    if seconds > 0:
        sampler = sampler_cls(device) if sampler_cls else None
        if sampler:
            sampler.start()
            time.sleep(0.25)
        t0 = time.time()
        e0.record()
        launches = 0
        while time.time() - t0 < seconds:
            for _ in range(50):
                launch(iters)
            launches += 50
            torch.cuda.current_stream().synchronize() if launches % 500 == 0 else None
        e1.record()
        torch.cuda.synchronize()
        t1 = time.time()
        out["sustained"] = round(ops.value * launches / (e0.elapsed_time(e1) * 1e-3) / 1e12, 1)
        out["sustained_seconds"] = round(e0.elapsed_time(e1) * 1e-3, 2)
        if sampler:
            out["clocks"] = sampler.stop(t0, t1)
        ctx.sync_check()
    return out


def measure(seconds=2.0, device=0, shapes=((64, 1), (64, 2), (128, 1), (128, 2), (256, 1)), dtypes=("int8", "f16"),
            m64_shapes=()):
    import torch
    from bench import ClockSampler
    from excalibur_b200 import capi
    torch.cuda.set_device(device)
    ctx = capi.Context(device)
    res = {"int8": [], "f16": []}
    for name, dt in (("int8", capi.EXB_I8), ("f16", capi.EXB_F16)):
        if name not in dtypes:
            continue
        for n, ctas in shapes:
            # the long loop only on the widest shape of each type: it is the one that reaches the peak
            res[name].append(probe(ctx, dt, n, ctas, seconds if (n, ctas) == (256, 1) else 0.0, ClockSampler, device))
        # M = 64: what a GEMM with a narrow layer's output channels on M would issue (never counted into the peaks)
        for n, ctas in m64_shapes:
            res[name].append(probe(ctx, dt, n, ctas, 0.0, ClockSampler, device, m=64))
    ctx.close()
    out = {
        "how": "tcgen05.mma cta_group::1 M=128 K=32B back to back from one thread per CTA, operands resident in shared "
               "memory, no TMA / epilogue; burst = best ~0.3 ms launch, sustained = launches back to back for %.1f s" % seconds,
        "int8_peak_tops": max([r["burst"] for r in res["int8"] if r["m"] == 128] or [0.0]),
        "f16_peak_tflops": max([r["burst"] for r in res["f16"] if r["m"] == 128] or [0.0]),
        "int8_peak_tops_sustained": max([r.get("sustained", 0.0) for r in res["int8"]] or [0.0]),
        "f16_peak_tflops_sustained": max([r.get("sustained", 0.0) for r in res["f16"]] or [0.0]),
        "shapes": res,
    }
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--seconds", type=float, default=2.0)
    ap.add_argument("--json", default=None)
    ap.add_argument("--m64", action="store_true", help="also time M = 64 MMAs (N = 64 and 128 on two CTAs per SM, N = 256 on one)")
    a = ap.parse_args()
    r = measure(a.seconds, m64_shapes=((64, 2), (128, 2), (256, 1)) if a.m64 else ())
    s = json.dumps(r)
    if a.json:
        open(a.json, "w").write(s + "\n")
    print(s)
