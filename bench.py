#!/usr/bin/env python
"""Benchmark of the CNN forward hot path: ResNet-18-style int8 classifier, batch 256 per GPU,
3x224x224 synthetic images (the third benchmark configuration), through pipeline<float>'s fused plan.

    python bench.py [--gpus N] [--steps K] [--warmup W]        # this library (one rank per GPU)
    python bench.py --impl reference [...]                     # the reference's CPU path, host cores

Prints ONE JSON line (rank 0).  `value` is images/s over all GPUs with the input resident in HBM
(CUDA-graph replay of the fused plan, device-timed: the median of K-step blocks run back to back for
--min-seconds, so it is a sustained figure; the first block is reported too); `e2e` is the same metric through
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


def _median(v):
    v = sorted(v)
    return v[len(v) // 2] if v else 0.0


def run_gpu_arm(args, rank, world, local_rank):
    import torch
    from excalibur_b200 import host, sharding
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
        return sharding.max_over_ranks(v, dist, "cuda")

    def max_vec(vals):
        """element-wise max over ranks of a list of floats"""
        if dist is None:
            return list(vals)
        t = torch.tensor(vals, dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(v) for v in t.tolist()]

    g8, scales = build_int8_net_gpu(local_rank)
    # one rank per GPU: keep this rank's pinned input and its copy submissions on the GPU's NUMA node
    numa_cpus = None
    if world > 1:
        numa_cpus = sharding.bind_host_thread_to_gpu(local_rank)
    pipe = host.Pipeline(g8.phai_text(), g8.racy_bytes(), local_rank, fusion=True, cuda_graph=not args.no_graph)
    x = torch.empty((BATCH, 3, IMG, IMG), dtype=torch.float32).pin_memory()
    gen = torch.Generator().manual_seed(SEED * 1000 + 100 + rank)
    x.uniform_(0, 1, generator=gen)
    logits = np.empty((BATCH, 1000, 1, 1), np.float32)
    K = args.steps

    def e2e_step():
        pipe.forward_ptr(x.data_ptr(), BATCH, 3, IMG, IMG)
        pipe.get("logits", logits)

    # ---- warm-up: eager, capture, replay; then W resident steps --------------------------------
    warm = max(3, args.warmup)
    for _ in range(warm):
        e2e_step()
    pipe.run_resident(warm)
    launches_per_step, _ = pipe.stats()

    # ---- timed region, input resident in HBM: blocks of exactly K steps, back to back, until at least
    # `--min-seconds` of device time have passed.  `value` is the median block (what the part sustains: the first
    # blocks run at the boost clock, later ones under the power limit), the first block is reported as the burst.
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.3)
    barrier()
    t0 = time.time()
    first = max_over_ranks(pipe.run_resident(K))
    n_blocks = max(1, min(2000, int(np.ceil(args.min_seconds * 1000.0 / max(first, 1e-3)))))
    blocks = [pipe.run_resident(K) for _ in range(n_blocks)]
    torch.cuda.synchronize()
    barrier()
    t1 = time.time()
    blocks = [first] + max_vec(blocks)
    clocks = sampler.stop(t0, t1) if sampler else None
    ms = _median(blocks)
    total_ms = sum(blocks)

    # ---- end to end: host buffers, H2D + D2H inside the timed region -----------------------------
    # pipeline<float>::forward on the whole pinned batch; the pipeline copies sub-batch c+1 to the
    # device while it computes sub-batch c (option h2d_chunks), logits come back per sub-batch
    host_threads = args.e2e_host_threads
    if host_threads < 0:
        per_rank = (os.cpu_count() or 1) // max(world, 1)
        host_threads = min(16, per_rank) if per_rank >= 4 else 0
    pipe.set_option("h2d_chunks", args.e2e_chunks)
    pipe.set_option("host_f16_threads", host_threads)
    for _ in range(3):
        e2e_step()
    barrier()
    e2e_blocks = []
    e2e_total = 0.0
    while e2e_total < min(1.0, args.min_seconds) or not e2e_blocks:
        te0 = time.perf_counter()
        for _ in range(K):
            e2e_step()
        torch.cuda.synchronize()
        dt = max_over_ranks(time.perf_counter() - te0)       # every rank sees the same value: same loop count
        e2e_blocks.append(dt)
        e2e_total += dt
    barrier()
    e2e_s = _median(e2e_blocks)

    # ---- the same call from two callers: a second pipeline object on the same GPU, one host thread each, every
    # forward still synchronous (input from pinned host memory, logits back on the host when it returns).  One
    # caller's copy runs while the other's last sub-batch computes, so the copy engine does not idle between steps.
    pipe_b = host.Pipeline(g8.phai_text(), g8.racy_bytes(), local_rank, fusion=True, cuda_graph=not args.no_graph)
    pipe_b.set_option("h2d_chunks", args.e2e_chunks)
    pipe_b.set_option("host_f16_threads", host_threads)
    x_b = torch.empty((BATCH, 3, IMG, IMG), dtype=torch.float32).pin_memory()
    x_b.uniform_(0, 1, generator=gen)
    logits_b = np.empty((BATCH, 1000, 1, 1), np.float32)

    caller_errors = []

    def caller(pl, xin, out, n):
        try:
            torch.cuda.set_device(local_rank)
            for _ in range(n):
                pl.forward_ptr(xin.data_ptr(), BATCH, 3, IMG, IMG)
                pl.get("logits", out)
        except BaseException as exc:      # a failed caller must fail the run, not shorten the timed work
            caller_errors.append(exc)

    def two_callers(n_total):
        ta = threading.Thread(target=caller, args=(pipe, x, logits, n_total - n_total // 2))
        tb = threading.Thread(target=caller, args=(pipe_b, x_b, logits_b, n_total // 2))
        ta.start()
        tb.start()
        ta.join()
        tb.join()
        if caller_errors:
            raise caller_errors[0]

    two_callers(6)
    barrier()
    e2e2_blocks, e2e2_total = [], 0.0
    while e2e2_total < min(1.0, args.min_seconds) or not e2e2_blocks:
        te0 = time.perf_counter()
        two_callers(K)
        torch.cuda.synchronize()
        dt = max_over_ranks(time.perf_counter() - te0)
        e2e2_blocks.append(dt)
        e2e2_total += dt
    barrier()
    e2e2_s = _median(e2e2_blocks)
    pipe_b.close()
    del x_b
    pipe.set_option("h2d_chunks", 1)
    pipe.set_option("host_f16_threads", 0)

    # ---- the same through pipeline<unsigned short>: a caller that holds fp16 images moves half the bytes ------
    pipe16 = host.PipelineF16(g8.phai_text(), g8.racy_bytes(), local_rank, fusion=True)
    pipe16.set_option("h2d_chunks", args.e2e_f16_chunks)
    x16 = x.to(torch.float16).pin_memory()
    logits16 = np.empty((BATCH, 1000, 1, 1), np.float16)

    def e2e16_step():
        pipe16.forward_ptr(x16.data_ptr(), BATCH, 3, IMG, IMG)
        pipe16.get("logits", logits16)

    for _ in range(3):
        e2e16_step()
    f16_fused = pipe16.stats()[0] > 0
    barrier()
    e16_blocks, e16_total = [], 0.0
    while e16_total < min(1.0, args.min_seconds) or not e16_blocks:
        te0 = time.perf_counter()
        for _ in range(K):
            e2e16_step()
        torch.cuda.synchronize()
        dt = max_over_ranks(time.perf_counter() - te0)
        e16_blocks.append(dt)
        e16_total += dt
    barrier()
    e2e16_s = _median(e16_blocks)
    # two callers, as for the fp32 call
    pipe16_b = host.PipelineF16(g8.phai_text(), g8.racy_bytes(), local_rank, fusion=True)
    pipe16_b.set_option("h2d_chunks", args.e2e_f16_chunks)
    x16_b = x16.clone().pin_memory()
    logits16_b = np.empty((BATCH, 1000, 1, 1), np.float16)

    def two_callers16(n_total):
        ta = threading.Thread(target=caller, args=(pipe16, x16, logits16, n_total - n_total // 2))
        tb = threading.Thread(target=caller, args=(pipe16_b, x16_b, logits16_b, n_total // 2))
        ta.start()
        tb.start()
        ta.join()
        tb.join()
        if caller_errors:
            raise caller_errors[0]

    two_callers16(6)
    barrier()
    e16b_blocks, e16b_total = [], 0.0
    while e16b_total < min(1.0, args.min_seconds) or not e16b_blocks:
        te0 = time.perf_counter()
        two_callers16(K)
        torch.cuda.synchronize()
        dt = max_over_ranks(time.perf_counter() - te0)
        e16b_blocks.append(dt)
        e16b_total += dt
    barrier()
    e2e16b_s = _median(e16b_blocks)
    pipe16_b.close()
    pipe16.close()
    del x16, x16_b

    # ---- the bare copy the end-to-end number is made of: pinned host -> device, every rank at once ---------
    xd = torch.empty((BATCH, 3, IMG, IMG), dtype=torch.float32, device="cuda")
    for _ in range(2):
        xd.copy_(x, non_blocking=True)
    barrier()
    ce0, ce1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ce0.record()
    n_copies = 10
    for _ in range(n_copies):
        xd.copy_(x, non_blocking=True)
    ce1.record()
    torch.cuda.synchronize()
    copy_ms = max_over_ranks(ce0.elapsed_time(ce1))
    barrier()
    h2d_bare_gbs = x.numel() * 4 * n_copies / (copy_ms * 1e-3) / 1e9
    del xd

    # ---- second configuration, strong scaling: YOLOv5s-style fp16, batch 32 over all ranks -----------------
    secondary = None
    if not args.no_secondary:
        secondary = yolo_strong_scaling(host, torch, local_rank, rank, world, barrier, max_over_ranks)

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
    prof_total_ms = sum(k["ms"] for k in kinds.values())
    per_kernel = {}
    for kind, k in kinds.items():
        e = {"launches_per_step": k["launches"], "ms_per_step": round(k["ms"], 4), "share": round(k["ms"] / prof_total_ms, 4)}
        if k["flops"]:
            e["tflops"] = round(k["flops"] / k["ms"] / 1e9, 1)
        if k["bytes"]:
            e["gbs"] = round(k["bytes"] / k["ms"] / 1e6, 1)
        per_kernel[kind] = e
    ci = kinds.get("conv_i8", dict(ms=1.0, flops=0.0, bytes=0.0, launches=1))
    # the denominator: this GPU's int8 tensor rate, measured now with the library's own MMA stream
    import bench_peak
    pk = bench_peak.measure(seconds=1.0, device=local_rank, shapes=((128, 2), (256, 1)), dtypes=("int8",))
    i8_burst, i8_sustained = pk["int8_peak_tops"], pk["int8_peak_tops_sustained"]
    achieved = ci["flops"] / ci["ms"] / 1e9
    roofline = {
        "kernel": "conv_tc_kernel<int8> (tcgen05 implicit GEMM, %d launches per step: 16 3x3 + 3 1x1)" % ci["launches"],
        "bound": "tensor", "achieved": round(achieved, 1), "peak": round(i8_burst, 1), "unit": "TFLOP/s",
        "frac": round(achieved / i8_burst, 4),
        "peak_source": "measured in this run: tcgen05.mma kind::i8 M=128 N=128/256 back to back from shared memory, best "
                       "0.3 ms launch (bench_peak.py); the same loop held for 1 s under the power limit gives "
                       "peak_sustained",
        "peak_sustained": round(i8_sustained, 1), "frac_of_peak_sustained": round(achieved / max(i8_sustained, 1e-9), 4),
        "achieved_note": "algorithmic FLOP of the int8 conv launches / their summed CUDA-event times in profiled forwards "
                         "(an event between kernels switches programmatic dependent launch overlap off: the sum of all "
                         "kernels is %.3f ms against %.3f ms per step in the timed region, so achieved is understated by "
                         "up to that ratio)" % (prof_total_ms, ms / K),
        "share_of_step": round(ci["ms"] / prof_total_ms, 4),
        "traffic": TRAFFIC_FROM_NCU, "traffic_source": TRAFFIC_SOURCE,
        "algorithmic_bytes": round(ci["bytes"] / max(ci["launches"], 1)),
        "per_kernel": per_kernel,
        "hbm_peak_gbs": hbm_peak,
    }

    cb = cpu_baseline(g8, scales) if world == 1 else None

    images_block = BATCH * world * K
    value = images_block / (ms / 1000.0)
    sm_mhz = (clocks or {}).get("sm_mhz")
    line = {
        "metric": METRIC, "value": value, "unit": "images/s", "per_gpu": value / world, "n_gpus": world,
        "steps": K, "warmup": warm, "ms_per_step": ms / K, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "value_sustained": BATCH * world * K * len(blocks) / (total_ms / 1000.0),
        "value_first_block": images_block / (blocks[0] / 1000.0),
        "timed_region": {"blocks": len(blocks), "steps_per_block": K, "device_seconds": round(total_ms / 1000.0, 3),
                         "value_is": "median block of K steps", "sm_mhz_median": sm_mhz,
                         "ms_per_step_x_sm_mhz": round(ms / K * sm_mhz, 1) if sm_mhz else None,
                         "first_block_ms_per_step": blocks[0] / K, "last_block_ms_per_step": blocks[-1] / K},
        "config": {"workload": "configs[2]: ResNet-18-style int8 classifier (stem and FC fp16), batch 256 per GPU, "
                               "3x224x224 uniform[0,1], max-abs calibration on 32 seeded images",
                   "batch_per_gpu": BATCH, "global_batch": BATCH * world,
                   "parallelism": "batch-sharded replicas, one process per GPU, no collective",
                   "l2": "no flush: every step streams a 154 MB input and >1 GB of activations, larger than the 126 MB L2",
                   "timing": "CUDA events on the plan's stream around blocks of K %s, max over ranks per block"
                             % ("eager launches of the plan (--no-graph)" if args.no_graph else "CUDA-graph replays")},
        "clocks": clocks,
        "e2e": {"value": images_block / min(e2e_s, e2e2_s), "unit": "images/s",
                "h2d_bytes_per_step": BATCH * 3 * IMG * IMG * (2 if host_threads > 0 else 4),
                "host_convert_threads": host_threads,
                "d2h_bytes_per_step": BATCH * 1000 * 4, "ms_per_step": min(e2e_s, e2e2_s) * 1000.0 / K,
                "callers": 2 if e2e2_s < e2e_s else 1,
                "callers_note": "K synchronous pipeline<float>::forward calls on pinned host batches, issued by two host "
                                "threads with a pipeline object each (K/2 calls per thread) or by one thread; value is "
                                "the faster arrangement, both are listed",
                "two_callers": {"value": images_block / e2e2_s, "ms_per_step": e2e2_s * 1000.0 / K, "blocks": len(e2e2_blocks)},
                "one_caller": {"value": images_block / e2e_s, "ms_per_step": e2e_s * 1000.0 / K, "blocks": len(e2e_blocks)},
                "blocks": len(e2e_blocks), "h2d_chunks": args.e2e_chunks,
                "h2d_bare_gbs": round(h2d_bare_gbs, 2),
                "h2d_bare_note": "cudaMemcpyAsync of the same pinned 154 MB input, %d copies back to back, every rank at "
                                 "once, slowest rank; %.2f ms per copy is the floor of an end-to-end step"
                                 % (n_copies, copy_ms / n_copies),
                "host_binding": ("rank 0 bound to %d CPUs next to its GPU" % len(numa_cpus)) if numa_cpus else "none"},
        "e2e_f16_input": {"value": images_block / min(e2e16_s, e2e16b_s), "unit": "images/s",
                          "ms_per_step": min(e2e16_s, e2e16b_s) * 1000.0 / K,
                          "callers": 2 if e2e16b_s < e2e16_s else 1,
                          "two_callers": {"value": images_block / e2e16b_s, "ms_per_step": e2e16b_s * 1000.0 / K},
                          "one_caller": {"value": images_block / e2e16_s, "ms_per_step": e2e16_s * 1000.0 / K},
                          "h2d_bytes_per_step": BATCH * 3 * IMG * IMG * 2, "d2h_bytes_per_step": BATCH * 1000 * 2,
                          "h2d_chunks": args.e2e_f16_chunks, "fused_plan": bool(f16_fused),
                          "api": "pipeline<unsigned short>::forward on pinned fp16 NCHW host tensors (the reference's fp16 "
                                 "Dtype); a second number beside e2e, which stays the fp32 call"},
        "gpu_launches": int(launches_per_step) * K,
        "roofline": roofline,
    }
    if secondary is not None:
        line["secondary"] = secondary
    if cb is not None:
        line["cpu_baseline"] = cb
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def yolo_strong_scaling(host, torch, local_rank, rank, world, barrier, max_over_ranks, total=32, size=640, steps=10):
    """The fifth benchmark configuration: YOLOv5s-style fp16 detector, batch 32 at 3x640x640, the batch split over the ranks
    (32 / 16 / 8 / 4 images per GPU at 1 / 2 / 4 / 8 GPUs): total work fixed, so this one is strong scaling."""
    from excalibur_b200 import models, sharding
    lo, hi = sharding.shard_bounds(total, world, rank)
    n = hi - lo
    g, info = models.yolov5s(5)
    p = host.Pipeline(g.phai_text(), g.racy_bytes(), local_rank, fusion=True)
    x = torch.empty((max(n, 1), 3, size, size), dtype=torch.float32).pin_memory()
    x.uniform_(0, 1, generator=torch.Generator().manual_seed(5000 + rank))
    ms = 0.0
    if n > 0:
        for _ in range(3):
            p.forward_ptr(x.data_ptr(), n, 3, size, size)
        p.run_resident(3)
    barrier()
    if n > 0:
        ms = p.run_resident(steps)
    torch.cuda.synchronize()
    ms = max_over_ranks(ms)
    barrier()
    launches, _ = p.stats()
    p.close()
    return {"workload": "configs[4]: YOLOv5s-style fp16 detector, global batch %d at 3x%dx%d, %d images per GPU" % (
                total, size, size, (total + world - 1) // world),
            "scaling": "strong", "metric": "images/s, whole job", "value": total * steps / (ms / 1000.0),
            "ms_per_step": ms / steps, "steps": steps, "n_gpus": world, "launches_per_step": int(launches),
            "timing": "CUDA-graph replays of the fused plan, input resident, max over ranks"}


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel (bytes), from ncu captures of one
# launch per layer shape at batch 256, weighted by how often each shape occurs among the int8 conv launches of a step.
# It is a constant of the kernel version named in TRAFFIC_SOURCE, not re-measured by this script (ncu cannot run
# inside the timed program); lower than the algorithmic bytes because small outputs stay in L2.
TRAFFIC_FROM_NCU = 62.4e6
TRAFFIC_SOURCE = ("ncu dram__bytes_read.sum + dram__bytes_write.sum, one launch per layer shape at batch 256 (bench_layers.py "
                  "--iters 1 --warmup 0), weighted over the 19 int8 conv launches of a step; captured on the kernel with the "
                  "row-box main loop, the quad epilogue and CTA pairs")


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
    ap.add_argument("--e2e-f16-chunks", type=int, default=2,
                    help="the same for the fp16-input forward (half the bytes per image: fewer, larger sub-batches)")
    ap.add_argument("--e2e-host-threads", type=int, default=0,
                    help="host threads converting the fp32 input to fp16 before the copy in the end-to-end measurement "
                         "(0 = copy fp32 as it is, the default: with 16 host cores the conversion costs more "
                         "than the PCIe bytes it saves; -1 = min(16, host CPUs per rank), off below 4)")
    ap.add_argument("--min-seconds", type=float, default=2.0,
                    help="the K-step block is repeated until this much device time has passed; value = median block")
    ap.add_argument("--no-secondary", action="store_true", help="skip the YOLOv5s-style strong-scaling measurement")
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
