#!/usr/bin/env python
"""Benchmark of the CNN forward hot path: ResNet-18-style int8 classifier, batch 256 per GPU,
3x224x224 synthetic images (BASELINE configs[2]), through pipeline<float>'s fused plan.

    python bench.py [--gpus N] [--steps K] [--warmup W]        # this library (one rank per GPU)
    python bench.py --impl reference [...]                     # the reference's CPU path, host cores

Prints ONE JSON line (rank 0).  `value` is images/s over all GPUs with the input resident in HBM
(CUDA-graph replay of the fused plan, device-timed); `e2e` is the same metric through
pipeline<float>::forward with pinned HOST buffers, upload and download inside the timed region.
`roofline` describes the dominant kernel (the int8 tcgen05 implicit-GEMM conv) from per-kernel CUDA
event times; `cpu_baseline` is the reference CPU library (oracle/_ref, when it was built) or the
plain-C oracle timed on the host cores on a bounded sample.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BATCH = 256
IMG = 224
SEED = 2
METRIC = "images/s/GPU, ResNet-18-style int8 conv net, bs256; % of tensor/HBM roofline"


# ----------------------------------------------------------------------------------------------
# clocks
# ----------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, smax, reasons = [], None, set()
        for ts, line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                mhz = float(parts[0])
                smax = float(parts[1])
            except ValueError:
                continue
            if t0 - 0.05 <= ts <= t1 + 0.15:
                sm.append(mhz)
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
        if not sm:   # timed region shorter than the sampling period: use every sample taken
            for ts, line in self.lines:
                try:
                    sm.append(float(line.split(",")[0]))
                except ValueError:
                    pass
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm)}


# ----------------------------------------------------------------------------------------------
# workload description (algorithmic work per kernel, for the roofline)
# ----------------------------------------------------------------------------------------------
def resnet_layers(batch):
    """name -> dict(kind, flops, bytes) for every kernel of the fused plan, algorithmic figures:
    conv FLOP = 2*N*OH*OW*Cout*Cin*kh*kw; bytes = each operand once at its storage type."""
    L = {}
    widths = (64, 128, 256, 512)
    h = IMG // 2
    pitch = (IMG + 4 + 8 + 7) // 8 * 8      # NHWC4 fp16 rows, zero-padded along W for the folded-K stem
    L["ingest data"] = dict(kind="layout", flops=0, bytes=batch * 3 * IMG * IMG * 4 + batch * IMG * pitch * 4 * 2)
    L["stem"] = dict(kind="conv_f16", flops=2 * batch * h * h * 64 * 3 * 49,
                     bytes=batch * IMG * pitch * 4 * 2 + batch * h * h * 64 * 2 + 64 * 7 * 8 * 4 * 2)
    L["pool1"] = dict(kind="pool", flops=0, bytes=batch * h * h * 64 * 2 + batch * (h // 2) ** 2 * 64 * 3)
    h //= 2
    cin = 64
    for si, wd in enumerate(widths):
        for bi in range(2):
            p = "s%db%d" % (si + 1, bi + 1)
            hin = h
            if si > 0 and bi == 0:
                h //= 2
                # projection: int8 in, fp16 out
                L[p + "_proj"] = dict(kind="conv_i8", flops=2 * batch * h * h * wd * cin,
                                      bytes=batch * hin * hin * cin + batch * h * h * wd * 2 + wd * cin)
            # conv1: int8 in, int8 out
            L[p + "_conv1"] = dict(kind="conv_i8", flops=2 * batch * h * h * wd * cin * 9,
                                   bytes=batch * hin * hin * cin + batch * h * h * wd + wd * cin * 9)
            # conv2 + add + relu: int8 in, fp16 skip in, fp16 + int8 out (last block: fp16 only)
            last = si == 3 and bi == 1
            L[p + "_conv2"] = dict(kind="conv_i8", flops=2 * batch * h * h * wd * wd * 9,
                                   bytes=batch * h * h * wd * (1 + 2 + 2 + (0 if last else 1)) + wd * wd * 9)
            cin = wd
    L["gap"] = dict(kind="pool", flops=0, bytes=batch * h * h * 512 * 2 + batch * 512 * 2)
    L["fc"] = dict(kind="conv_f16", flops=2 * batch * 512 * 1000, bytes=batch * 512 * 2 + 512 * 1000 * 2 + batch * 1000 * 4)
    L["emit logits"] = dict(kind="layout", flops=0, bytes=0)
    return L


def group_name(step):
    # fused groups are named after the op that leads them: "<block>_conv2" absorbs add + relu
    return step


# ----------------------------------------------------------------------------------------------
# CPU baseline (reference library when built, else the plain-C oracle)
# ----------------------------------------------------------------------------------------------
def _cpu_worker(phai_path, racy_path, budget_s):
    """Child process: time int8 ResNet-18 forwards, one image per call (the reference's packed int8
    path only computes image 0 of a batch), for about budget_s seconds.  Prints 'images seconds'."""
    from oracle import ref_lib
    r = np.random.default_rng(os.getpid())
    x = r.uniform(0, 1, (1, 3, IMG, IMG)).astype(np.float32)
    if ref_lib.available():
        p = ref_lib.RefPipeline(open(phai_path).read(), open(racy_path, "rb").read())
        fwd = lambda: p.forward(x)
    else:
        fwd = _oracle_forward_factory(phai_path, racy_path, x)
    fwd()   # warm-up (page-in, weight transforms)
    n, t0 = 0, time.perf_counter()
    while True:
        fwd()
        n += 1
        el = time.perf_counter() - t0
        if el >= budget_s or n >= 256:
            break
    print(n, el)


def _oracle_forward_factory(phai_path, racy_path, x):
    """ResNet-18 int8 forward on the plain-C oracle (used only where oracle/_ref is absent)."""
    from excalibur_b200 import models
    from oracle import exb_oracle as O
    meta = json.load(open(phai_path + ".json"))
    scales = {k: np.float32(v) for k, v in meta["scales"].items()}
    wts = models._Weights(SEED)

    def fwd():
        wts.index = 0
        w, b = wts.conv_bn(64, 3, 7)
        h = O.conv2d_f32(x, w, b, 2, 3, act=1)
        h = O.pool2d_f32(h, 0, 3, 2, 1)
        cin = 64
        for si, wd in enumerate((64, 128, 256, 512)):
            for bi in range(2):
                stride = 2 if (si > 0 and bi == 0) else 1
                p = "s%db%d" % (si + 1, bi + 1)
                w1, b1 = wts.conv_bn(wd, cin, 3)
                q1, s1 = models.quantize_weights(w1)
                a = O.conv2d_i8(h, q1, b1, s1, scales[p + "_conv1"], stride, 1, act=1)
                w2, b2 = wts.conv_bn(wd, wd, 3)
                q2, s2 = models.quantize_weights(w2)
                a = O.conv2d_i8(a, q2, b2, s2, scales[p + "_conv2"], 1, 1)
                if stride != 1 or cin != wd:
                    w3, b3 = wts.conv_bn(wd, cin, 1)
                    q3, s3 = models.quantize_weights(w3)
                    h = O.conv2d_i8(h, q3, b3, s3, scales[p + "_proj"], stride, 0)
                h = O.relu_f32(O.eltwise_f32([a, h], 1))
                cin = wd
        h = O.pool2d_f32(h, 1, global_pool=True)
        fw, fb = wts.fc(1000, 512)
        return h.reshape(1, -1) @ fw.T + fb
    return fwd


def cpu_baseline(g8, scales, budget_s=12.0, max_workers=None):
    from oracle import ref_lib
    cores = len(os.sched_getaffinity(0))
    workers = max(1, min(cores, max_workers or cores))
    tmp = tempfile.mkdtemp(prefix="exb_cpu_")
    phai, racy = os.path.join(tmp, "net.phai"), os.path.join(tmp, "net.racy")
    g8.save(phai, racy)
    json.dump({"scales": {k: float(v) for k, v in scales.items()}}, open(phai + ".json", "w"))
    kind = "reference" if ref_lib.available() else "port"
    if kind == "port":
        budget_s = min(budget_s, 8.0)
    t0 = time.perf_counter()
    procs = [subprocess.Popen([sys.executable, os.path.abspath(__file__), "--_cpu_worker", phai, racy, str(budget_s)],
                              stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
                              env=dict(os.environ, OMP_NUM_THREADS="1")) for _ in range(workers)]
    imgs, slowest = 0, 0.0
    for p in procs:
        out = p.communicate()[0].strip().split()
        if len(out) == 2:
            imgs += int(out[0])
            slowest = max(slowest, float(out[1]))
    wall = time.perf_counter() - t0
    value = imgs / slowest if slowest > 0 else 0.0
    return {"value": value, "unit": "images/s", "cores": workers, "kind": kind,
            "sample": "%d single-image int8 ResNet-18 forwards over %d processes (1 thread each), %.1f s of "
                      "timed work per process, %.1f s wall including start-up" % (imgs, workers, slowest, wall)}


# ----------------------------------------------------------------------------------------------
# network construction
# ----------------------------------------------------------------------------------------------
def build_int8_net_gpu(device):
    """fp graph -> max-abs calibration on 32 seeded images through this library's own pipeline ->
    int8 graph (stem and FC stay floating point)."""
    from excalibur_b200 import host, models
    g32, info = models.resnet18(SEED)
    p = host.Pipeline(g32.phai_text(), g32.racy_bytes(), device, fusion=False)
    calib = np.random.default_rng(SEED * 1000 + 7).uniform(0, 1, (32, 3, IMG, IMG)).astype(np.float32)
    scales = models.calibrate(p, info["conv_inputs"], calib)
    p.close()
    g8, _ = models.resnet18(SEED, act_scales=scales)
    return g8, scales


def build_int8_net_cpu():
    """Reference arm: calibrate through the reference CPU library itself (4 images)."""
    from excalibur_b200 import models
    from oracle import ref_lib
    g32, info = models.resnet18(SEED)
    if ref_lib.available():
        class A:
            def __init__(self):
                self.p = ref_lib.RefPipeline(g32.phai_text(), g32.racy_bytes())

            def forward(self, x):
                return self.p.forward(x)

            def get(self, n):
                return self.p.featmap(n)
        a = A()
        calib = np.random.default_rng(SEED * 1000 + 7).uniform(0, 1, (4, 3, IMG, IMG)).astype(np.float32)
        scales = models.calibrate(a, info["conv_inputs"], calib)
        a.p.close()
    else:
        scales = {k: np.float32(30.0) for k in info["conv_inputs"]}
    g8, _ = models.resnet18(SEED, act_scales=scales)
    return g8, scales


# ----------------------------------------------------------------------------------------------
# arms
# ----------------------------------------------------------------------------------------------
def run_reference_arm(args, rank):
    if rank != 0:
        return
    g8, scales = build_int8_net_cpu()
    # warm-up and steps are folded into one bounded sample: every process runs a warm-up forward,
    # then forwards for a time budget; a "step" of batch 256 would take minutes on the host.
    budget = max(4.0, min(20.0, 4.0 * args.steps))
    cb = cpu_baseline(g8, scales, budget_s=budget)
    v = cb["value"]
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": "images/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": (BATCH / v * 1000.0) if v > 0 else None, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "configs[2]: ResNet-18-style int8 classifier, 3x224x224; the reference CPU path runs "
                               "one image per forward (its packed int8 conv only computes image 0 of a batch)",
                   "batch_per_gpu": BATCH},
        "cpu_baseline": cb,
        "e2e": {"value": v, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_gpu_arm(args, rank, world, local_rank):
    import torch
    from excalibur_b200 import host
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if dist is not None:
            t = torch.zeros(1, device="cuda")
            dist.all_reduce(t)
        torch.cuda.synchronize()

    def max_over_ranks(v):
        from excalibur_b200 import sharding
        return sharding.max_over_ranks(v, dist, "cuda")

    g8, scales = build_int8_net_gpu(local_rank)
    # one rank per GPU: keep this rank's pinned input and its copy submissions on the GPU's NUMA node
    numa_cpus = None
    if world > 1:
        from excalibur_b200 import sharding
        numa_cpus = sharding.bind_host_thread_to_gpu(local_rank)
    pipe = host.Pipeline(g8.phai_text(), g8.racy_bytes(), local_rank, fusion=True, cuda_graph=not args.no_graph)
    x = torch.empty((BATCH, 3, IMG, IMG), dtype=torch.float32).pin_memory()
    gen = torch.Generator().manual_seed(SEED * 1000 + 100 + rank)
    x.uniform_(0, 1, generator=gen)
    logits = np.empty((BATCH, 1000, 1, 1), np.float32)

    def e2e_step():
        pipe.forward_ptr(x.data_ptr(), BATCH, 3, IMG, IMG)
        pipe.get("logits", logits)

    # ---- warm-up: eager, capture, replay; then W resident steps --------------------------------
    for _ in range(max(3, args.warmup)):
        e2e_step()
    pipe.run_resident(max(3, args.warmup))
    launches_per_step, _ = pipe.stats()

    # ---- timed region: K steps, input resident in HBM ------------------------------------------
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.3)
    barrier()
    t0 = time.time()
    ms = pipe.run_resident(args.steps)
    torch.cuda.synchronize()
    barrier()
    t1 = time.time()
    ms = max_over_ranks(ms)
    clocks = sampler.stop(t0, t1) if sampler else None

    # ---- end-to-end: host buffers, H2D + D2H inside the timed region ---------------------------
    # pipeline<float>::forward on the whole pinned batch; the pipeline copies sub-batch c+1 to the
    # device while it computes sub-batch c (option h2d_chunks), logits come back per sub-batch
    # (--e2e-host-threads T: after T host threads have converted it to fp16 - half the PCIe bytes, identical
    # logits; off by default)
    host_threads = args.e2e_host_threads
    if host_threads < 0:
        per_rank = (os.cpu_count() or 1) // max(world, 1)
        host_threads = min(16, per_rank) if per_rank >= 4 else 0
    pipe.set_option("h2d_chunks", args.e2e_chunks)
    pipe.set_option("host_f16_threads", host_threads)
    for _ in range(3):
        e2e_step()
    barrier()
    te0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_s = max_over_ranks(time.perf_counter() - te0)
    barrier()
    pipe.set_option("h2d_chunks", 1)
    pipe.set_option("host_f16_threads", 0)

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    # ---- per-kernel device times (CUDA events on the plan's stream) for the roofline -----------
    pipe.set_option("profile", 1)
    acc = {}
    PROF = 3
    for _ in range(PROF):
        e2e_step()
        for name, b, e in pipe.trace():
            acc[name] = acc.get(name, 0.0) + (e - b) / PROF
    pipe.set_option("profile", 0)
    layers = resnet_layers(BATCH)
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    hbm_peak = peaks.get("hbm_gbs", 6650.0)
    bf16_peak = peaks.get("bf16_tflops_sustained", 1400.0)
    peak_src = "measured" if peaks else "fallback"
    kinds = {}
    for name, t_ms in acc.items():
        info = layers.get(name)
        if info is None:
            info = dict(kind="other", flops=0, bytes=0)
        k = kinds.setdefault(info["kind"], dict(ms=0.0, flops=0.0, bytes=0.0, launches=0))
        k["ms"] += t_ms
        k["flops"] += info["flops"]
        k["bytes"] += info["bytes"]
        k["launches"] += 1
    total_ms = sum(k["ms"] for k in kinds.values())
    per_kernel = {}
    for kind, k in kinds.items():
        e = {"launches_per_step": k["launches"], "ms_per_step": round(k["ms"], 4), "share": round(k["ms"] / total_ms, 4)}
        if k["flops"]:
            e["tflops"] = round(k["flops"] / k["ms"] / 1e9, 1)
        if k["bytes"]:
            e["gbs"] = round(k["bytes"] / k["ms"] / 1e6, 1)
        per_kernel[kind] = e
    ci = kinds.get("conv_i8", dict(ms=1.0, flops=0.0, launches=1))
    i8_peak = 2.0 * bf16_peak
    achieved = ci["flops"] / ci["ms"] / 1e9
    roofline = {
        "kernel": "conv_tc_kernel<int8> (tcgen05 implicit GEMM, 19 launches per step: 16 3x3 + 3 1x1)",
        "bound": "tensor", "achieved": round(achieved, 1), "peak": round(i8_peak, 1), "unit": "TFLOP/s",
        "frac": round(achieved / i8_peak, 4),
        "peak_source": "2 x the %s sustained bf16 figure (MEASURED_PEAKS.json holds no int8 peak)" % peak_src,
        "share_of_step": round(ci["ms"] / total_ms, 4),
        "traffic": TRAFFIC_FROM_NCU,
        "per_kernel": per_kernel,
        "hbm_peak_gbs": hbm_peak,
    }

    g_cpu, s_cpu = g8, scales
    cb = cpu_baseline(g_cpu, s_cpu) if world == 1 else None

    images = BATCH * world * args.steps
    value = images / (ms / 1000.0)
    line = {
        "metric": METRIC, "value": value, "unit": "images/s", "per_gpu": value / world, "n_gpus": world,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "configs[2]: ResNet-18-style int8 classifier (stem and FC fp16), batch 256 per GPU, "
                               "3x224x224 uniform[0,1], max-abs calibration on 32 seeded images",
                   "batch_per_gpu": BATCH, "global_batch": BATCH * world,
                   "parallelism": "batch-sharded replicas, one process per GPU, no collective",
                   "l2": "no flush: every step streams a 154 MB input and >1 GB of activations, larger than the 126 MB L2",
                   "timing": "CUDA events on the plan's stream around K %s, max over ranks"
                             % ("eager launches of the plan (--no-graph)" if args.no_graph else "CUDA-graph replays")},
        "clocks": clocks,
        "e2e": {"value": images / e2e_s, "unit": "images/s",
                "h2d_bytes_per_step": BATCH * 3 * IMG * IMG * (2 if host_threads > 0 else 4),
                "host_convert_threads": host_threads,
                "d2h_bytes_per_step": BATCH * 1000 * 4, "ms_per_step": e2e_s * 1000.0 / args.steps,
                "h2d_chunks": args.e2e_chunks,
                "host_binding": ("rank 0 bound to %d CPUs next to its GPU" % len(numa_cpus)) if numa_cpus else "none"},
        "gpu_launches": int(launches_per_step) * args.steps,
        "roofline": roofline,
    }
    if cb is not None:
        line["cpu_baseline"] = cb
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel (bytes): the ncu
# capture of one launch per layer shape at batch 256 (profiles/conv_tc_dram_traffic_resnet18_layers_
# batch256.md), weighted by how often each shape occurs among the 19 int8 conv launches of a step
# (1163 MB per step).  Lower than the algorithmic 93 MB per launch because small outputs stay in L2.
TRAFFIC_FROM_NCU = 61.2e6


def main():
    if len(sys.argv) >= 5 and sys.argv[1] == "--_cpu_worker":
        _cpu_worker(sys.argv[2], sys.argv[3], float(sys.argv[4]))
        return
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-chunks", type=int, default=4,
                    help="sub-batches of one end-to-end forward (copy of c+1 overlaps compute of c)")
    ap.add_argument("--e2e-host-threads", type=int, default=0,
                    help="host threads converting the fp32 input to fp16 before the copy in the end-to-end measurement "
                         "(0 = copy fp32 as it is, the default: on this pool's 16-vCPU hosts the conversion costs more "
                         "than the PCIe bytes it saves; -1 = min(16, host CPUs per rank), off below 4)")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch the plan's kernels one by one instead of replaying a CUDA graph (profilers "
                         "cannot attach to launches made during stream capture); not a bench configuration")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if world == 1 and args.gpus > 1:
        # launched without torchrun: re-launch one rank per GPU
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(args.gpus),
               "--master-addr", "127.0.0.1", "--master-port", "29517", os.path.abspath(__file__), "--gpus", str(args.gpus),
               "--steps", str(args.steps), "--warmup", str(args.warmup)]
        sys.exit(subprocess.call(cmd))
    run_gpu_arm(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
