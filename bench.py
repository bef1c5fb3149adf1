#!/usr/bin/env python
"""Benchmark of the dense-contraction path.

One "step" = forward + input-gradient + weight-gradient (with bias gradient) of every layer of
the workload, inputs resident in HBM.  The default workload is the Linear projection sweep
(X[B*T, d] @ W^T[d, 4d] + b for d in {512, 1024, 2048}, B*T in {4096, 16384}; fp16 storage, fp32
accumulation; synthetic N(0,1) activations, Xavier-uniform weights).  Prints ONE JSON line.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload linear|resnet]

N > 1 is launched with torch.distributed.run; every rank owns its own shard of the rows (weak
scaling: per-GPU work fixed), the weight and bias gradients are all-reduced over NCCL each step.
`--impl reference` times the reference's own CPU arithmetic for the path (NumPy matmul, all host
threads) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LINEAR_SWEEP = [(rows, d) for d in (512, 1024, 2048) for rows in (4096, 16384)]
# ResNet-style conv shapes at batch 256 (7x7 s2 p3 3->64 @224 is left to the parity tests until
# its small-channel path exists): (c_in, hw, c_out, k, stride, pad)
# (c_in, input h = w, c_out, kernel, stride, padding, transposed)
RESNET_SWEEP = [(3, 224, 64, 7, 2, 3, False), (64, 56, 64, 3, 1, 1, False), (256, 56, 64, 1, 1, 0, False),
                (128, 28, 128, 3, 2, 1, False), (1024, 14, 2048, 1, 2, 0, False)]
RESNET_BATCH = 256
# the 16 convolutions of the Pix2Pix U-Net generator (4x4, stride 2, padding 1; decoder inputs carry the skip concat)
PIX2PIX_SWEEP = ([(ci, hw, co, 4, 2, 1, False) for ci, hw, co in
                  ((3, 256, 64), (64, 128, 128), (128, 64, 256), (256, 32, 512), (512, 16, 512), (512, 8, 512),
                   (512, 4, 512), (512, 2, 512))] +
                 [(ci, hw, co, 4, 2, 1, True) for ci, hw, co in
                  ((512, 1, 512), (1024, 2, 512), (1024, 4, 512), (1024, 8, 512), (1024, 16, 256), (512, 32, 128),
                   (256, 64, 64), (128, 128, 3))])
PIX2PIX_BATCH = 64
LINEAR_NAME = ("Linear sweep X[B*T,d]@W^T[d,4d]+b, d in {512,1024,2048} x B*T in {4096,16384}, "
               "forward+dgrad+wgrad+db, fp16 storage / fp32 accumulate")
RESNET_NAME = ("ResNet-style conv shapes, batch 256 per GPU, NHWC fp16: 7x7 s2 3->64 @224, 3x3 64->64 @56, 1x1 256->64 @56, "
               "3x3 s2 128->128 @28, 1x1 s2 1024->2048 @14; forward+dgrad+wgrad+db")
PIX2PIX_NAME = ("Pix2Pix U-Net generator convolutions, batch 64 per GPU, NHWC fp16: 8 Conv2d 4x4 s2 p1 "
                "(3-64-128-256-512-512-512-512-512) + 8 ConvTranspose2d 4x4 s2 p1 with skip-concat inputs; "
                "forward+dgrad+wgrad+db of every layer (normalisation and activations not included)")


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"tflops": float(p["bf16_tflops"]), "hbm_gbs": float(p["hbm_gbs"]), "source": "measured"}
    return {"tflops": 1590.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "25"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0: float, t1: float):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ts, line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6 or not (t0 - 0.05 <= ts <= t1 + 0.15):
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:  # timed region shorter than one sample: fall back to every sample taken
            for _, line in self.lines:
                parts = [p.strip() for p in line.split(",")]
                try:
                    sm.append(float(parts[0]))
                    mx.append(float(parts[1]))
                except (ValueError, IndexError):
                    pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------ workloads --
def linear_flops(rows, d):
    return 3 * 2.0 * rows * d * 4 * d  # forward + dgrad + wgrad


def conv_flops(batch, c_in, hw, c_out, k, s, p, transposed=False):
    ho = hw if transposed else (hw + 2 * p - k) // s + 1  # a transposed layer does its multiplies per INPUT pixel
    return 3 * 2.0 * batch * ho * ho * c_out * c_in * k * k


def make_linear_host(seed, sweep):
    """Pinned host buffers of one step's inputs, and the parameters."""
    import torch
    rng = np.random.default_rng(seed)
    layers = []
    for rows, d in sweep:
        bound = np.sqrt(6.0 / (d + 4 * d))
        layers.append({
            "rows": rows, "d": d,
            "x": torch.from_numpy(rng.standard_normal((rows, d), dtype=np.float32)).half().pin_memory(),
            "dy": torch.from_numpy(rng.standard_normal((rows, 4 * d), dtype=np.float32)).half().pin_memory(),
            "w": torch.from_numpy(rng.uniform(-bound, bound, (4 * d, d)).astype(np.float32)).half(),
            "b": torch.zeros(4 * d, dtype=torch.float16),
        })
    return layers


def run_gpu(args):
    import torch
    import torch.distributed as dist
    from nectarml_b200 import build, ops
    from nectarml_b200.ops import ConvGeometry

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    build.build()

    peaks = measured_peaks()
    flops_per_launch = []  # algorithmic FLOPs of each contraction launch of one step, in launch order

    if args.workload == "linear":
        # under data parallelism the largest shapes go first, so that their gradient all-reduce overlaps the
        # smaller shapes' kernels (on one GPU the listed order measured 1-2 % faster)
        sweep = sorted(LINEAR_SWEEP, key=lambda s_: -s_[0] * s_[1] * s_[1]) if world > 1 else list(LINEAR_SWEEP)
        if args.only:  # profiling aid: one shape of the sweep, e.g. --only 16384x1024
            r_, d_ = (int(v) for v in args.only.lower().split("x"))
            sweep = [(r_, d_)]
        host = make_linear_host(1235 + rank, sweep)
        layers = []
        for h in host:
            rows, d = h["rows"], h["d"]
            layers.append({
                **h,
                "xd": h["x"].to(dev), "dyd": h["dy"].to(dev), "wd": h["w"].to(dev), "bd": h["b"].to(dev),
                "y": torch.empty(rows, 4 * d, dtype=torch.float16, device=dev),
                "dx": torch.empty(rows, d, dtype=torch.float16, device=dev),
                "dw": torch.empty(4 * d, d, dtype=torch.float32, device=dev),
                "db": torch.empty(4 * d, dtype=torch.float32, device=dev),
                "dw_host": torch.empty(4 * d, d, dtype=torch.float32).pin_memory(),
                "db_host": torch.empty(4 * d, dtype=torch.float32).pin_memory(),
            })
            flops_per_launch += [2.0 * rows * d * 4 * d] * 3
        step_flops = sum(linear_flops(l["rows"], l["d"]) for l in layers)
        bytes_resident = sum(t.numel() * t.element_size() for l in layers for t in
                             (l["xd"], l["dyd"], l["wd"], l["y"], l["dx"], l["dw"]))

        def step():
            pending = []
            for l in layers:
                ops.linear_forward(l["xd"], l["wd"], l["bd"], out=l["y"])
                ops.linear_backward_data(l["dyd"], l["wd"], out=l["dx"])
                ops.linear_backward_weight(l["xd"], l["dyd"], dw=l["dw"], db=l["db"])
                if world > 1:
                    pending.append(dist.all_reduce(l["dw"], async_op=True))
                    pending.append(dist.all_reduce(l["db"], async_op=True))
            for p in pending:
                p.wait()

        # End-to-end step: the same calls, with each layer's inputs coming from pinned host memory and its
        # gradients going back to it.  Copies run on their own streams, ordered against the compute stream
        # by events, so a layer's transfers overlap the other layers' kernels inside the step; every step
        # ends with the compute stream waiting for that step's last device-to-host copy.
        s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        ev_in = [torch.cuda.Event() for _ in layers]
        ev_done = [torch.cuda.Event() for _ in layers]
        ev_out = [torch.cuda.Event() for _ in layers]

        def step_e2e():
            cur = torch.cuda.current_stream()
            with torch.cuda.stream(s_in):
                for i, l in enumerate(layers):
                    s_in.wait_event(ev_done[i])  # the previous step's kernels have finished reading xd / dyd
                    l["xd"].copy_(l["x"], non_blocking=True)
                    l["dyd"].copy_(l["dy"], non_blocking=True)
                    ev_in[i].record(s_in)
            for i, l in enumerate(layers):
                cur.wait_event(ev_in[i])
                cur.wait_event(ev_out[i])  # the previous step's copy of dw / db has left the device
                ops.linear_forward(l["xd"], l["wd"], l["bd"], out=l["y"])
                ops.linear_backward_data(l["dyd"], l["wd"], out=l["dx"])
                ops.linear_backward_weight(l["xd"], l["dyd"], dw=l["dw"], db=l["db"])
                if world > 1:
                    dist.all_reduce(l["dw"])
                    dist.all_reduce(l["db"])
                ev_done[i].record(cur)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_done[i])
                    l["dw_host"].copy_(l["dw"], non_blocking=True)
                    l["db_host"].copy_(l["db"], non_blocking=True)
                    ev_out[i].record(s_out)
            cur.wait_event(ev_out[-1])

        h2d = sum(l["x"].numel() * 2 + l["dy"].numel() * 2 for l in layers)
        d2h = sum(l["dw"].numel() * 4 + l["db"].numel() * 4 for l in layers)
        workload = {"workload": LINEAR_NAME,
                    "layers": len(layers), "rows_per_gpu": sum(l["rows"] for l in layers)}
    else:
        torch.manual_seed(1237 + rank)
        sweep, batch = (RESNET_SWEEP, RESNET_BATCH) if args.workload == "resnet" else (PIX2PIX_SWEEP, PIX2PIX_BATCH)
        if args.only:  # profiling aid: one layer of the sweep by index, e.g. --workload resnet --only 1
            sweep = [sweep[int(args.only)]]
        layers = []
        for (ci, hw, co, k, s, p, tr) in sweep:
            g = ConvGeometry(batch, ci, hw, hw, co, k, k, (s, s), (p, p), transposed=tr)
            ho, wo = g.out_hw()
            std = np.sqrt(2.0 / (ci * k * k)) if args.workload == "resnet" else 0.02
            layers.append({
                "g": g, "name": f"{'convT' if tr else 'conv'} {k}x{k} s{s} {ci}->{co} @{hw}",
                "xd": torch.randn(batch, hw, hw, ci, device=dev).half(),
                "dyd": torch.randn(batch, ho, wo, co, device=dev).half(),
                "wd": (torch.randn(*g.weight_shape(), device=dev) * std).half(),
                "y": torch.empty(batch, ho, wo, co, dtype=torch.float16, device=dev),
                "dx": torch.empty(batch, hw, hw, ci, dtype=torch.float16, device=dev),
            })
            flops_per_launch += [conv_flops(batch, ci, hw, co, k, s, p, tr) / 3] * 3
        step_flops = sum(flops_per_launch)
        bytes_resident = sum(t.numel() * t.element_size() for l in layers for t in (l["xd"], l["dyd"], l["y"], l["dx"]))
        grads = {}

        def step():
            pending = []
            for i, l in enumerate(layers):
                ops.conv_forward(l["g"], l["xd"], l["wd"], None, layout="nhwc", out=l["y"])
                ops.conv_backward_data(l["g"], l["dyd"], l["wd"], layout="nhwc", out=l["dx"])
                grads[i] = ops.conv_backward_weight(l["g"], l["xd"], l["dyd"], layout="nhwc")
                if world > 1:
                    pending.append(dist.all_reduce(grads[i][0], async_op=True))
                    pending.append(dist.all_reduce(grads[i][1], async_op=True))
            for p in pending:
                p.wait()

        h2d = d2h = 0
        workload = {"workload": RESNET_NAME if args.workload == "resnet" else PIX2PIX_NAME,
                    "layers": len(layers)}

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        """Times `steps` calls on the device; returns max-over-ranks milliseconds."""
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(max(args.warmup, 3)):
        step()
    ops.device_status()

    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.25)
    launches0 = ops.launch_count()
    t0 = time.time()
    ms_total = timed(lambda: step(), args.steps)
    t1 = time.time()
    launches = ops.launch_count() - launches0
    clocks = sampler.stop(t0, t1) if sampler else None
    ops.device_status()

    # per-launch durations of the contraction kernel, CUDA events on the launching stream
    n_rec = len(flops_per_launch) * args.steps
    barrier()
    ops.profile_begin(n_rec)
    for _ in range(args.steps):
        step()
    per_launch_ms = ops.profile_end(n_rec)
    kern_ms = sum(per_launch_ms)
    per_layer = None
    if args.per_layer and per_launch_ms:
        n1 = len(flops_per_launch)
        mean = [sum(per_launch_ms[i::n1]) / len(per_launch_ms[i::n1]) for i in range(n1)]
        names = [l["name"] if "name" in l else f"linear {l['rows']}x{l['d']}->{4 * l['d']}" for l in layers]
        per_layer = [{"layer": names[i // 3], "pass": ("fwd", "dgrad", "wgrad")[i % 3], "us": round(mean[i] * 1e3, 1),
                      "tflops": round(flops_per_launch[i] / (mean[i] * 1e-3) / 1e12, 1)} for i in range(n1)]
    kern_flops = sum(flops_per_launch) * (len(per_launch_ms) / max(len(flops_per_launch), 1))
    achieved = kern_flops / (kern_ms * 1e-3) / 1e12 if kern_ms > 0 else None

    # end to end through the public API with host buffers (pinned), copies inside the timed region
    e2e = None
    if args.workload == "linear":
        for _ in range(2):
            step_e2e()
        e2e_steps = max(2, min(args.steps, 5))
        e2e_ms = timed(step_e2e, e2e_steps)
        for l in layers:  # the gradients that reached the host are the ones on the device
            if not torch.equal(l["db_host"], l["db"].cpu()):
                raise SystemExit("bench.py: end-to-end leg returned stale gradients")
        e2e = {"value": step_flops * world * e2e_steps / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)}

    out = None
    if rank == 0:
        value = step_flops * world * args.steps / (ms_total * 1e-3) / 1e12
        out = {
            "metric": "conv/linear fwd+bwd TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_total / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16 (fp32 accumulate)",
            "data": "synthetic", "impl": "nectarml_b200",
            "config": {**workload, "parallelism": f"dp{world} (rows sharded, NCCL all-reduce of dW/db)" if world > 1 else "1 GPU",
                       "l2": f"working set {bytes_resident / 1e6:.0f} MB per GPU cycles through the 126 MB L2 every step"},
            "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["tflops"], "unit": "TFLOP/s",
                         "frac": (achieved / peaks["tflops"]) if achieved else None,
                         "peak_source": f"{peaks['source']} burst bf16 (MEASURED_PEAKS.json)" if peaks["source"] == "measured" else "fallback",
                         "kernel": "umma_conv_kernel", "launches_timed": len(per_launch_ms),
                         "traffic": TRAFFIC_BYTES_PER_LAUNCH.get(args.workload)},
        }
        if per_layer:
            out["per_layer"] = per_layer
        if world == 1 and not args.no_cpu_baseline:
            out["cpu_baseline"] = cpu_baseline(args.workload, budget_s=12.0)
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return out


# dram__bytes_read.sum + dram__bytes_write.sum per contraction launch, averaged over one step of the
# workload, from the ncu capture summarised under profiles/ (None until a capture exists).
TRAFFIC_BYTES_PER_LAUNCH = {"linear": 164.5e6, "resnet": None, "pix2pix": None}


# ------------------------------------------------------------ CPU reference arm --
def cpu_linear_sample(budget_s: float):
    """The reference's CPU arithmetic for Linear (np.matmul, fp32 as its CPU tensors are) on as
    many layers of the sweep as fit the budget.  Returns (flops, seconds, description)."""
    from oracle import nectar_oracle as orc
    rng = np.random.default_rng(1235)
    done_flops, t_used, names = 0.0, 0.0, []
    for rows, d in sorted(LINEAR_SWEEP, key=lambda s: s[0] * s[1] * s[1]):
        est = linear_flops(rows, d) / max(done_flops / t_used, 2e11) if t_used > 0 else 0.0
        if t_used > 0 and t_used + est > budget_s:
            continue
        x = rng.standard_normal((rows, d), dtype=np.float32)
        w = rng.standard_normal((4 * d, d), dtype=np.float32)
        b = np.zeros(4 * d, np.float32)
        dy = rng.standard_normal((rows, 4 * d), dtype=np.float32)
        t0 = time.perf_counter()
        orc.linear_forward(x, w, b)
        orc.linear_backward(x, w, dy)
        t_used += time.perf_counter() - t0
        done_flops += linear_flops(rows, d)
        names.append(f"{rows}x{d}")
    return done_flops, t_used, "Linear layers " + ",".join(names) + " of the sweep, fp32 np.matmul"


def cpu_conv_sample(budget_s: float):
    from oracle import nectar_oracle as orc
    rng = np.random.default_rng(1237)
    ci, hw, co, k, s, p, _ = RESNET_SWEEP[1]
    x = rng.standard_normal((1, ci, hw, hw), dtype=np.float32)
    w = rng.standard_normal((co, ci, k, k), dtype=np.float32)
    dy = rng.standard_normal((1, co, hw, hw), dtype=np.float32)
    t0 = time.perf_counter()
    n = 0
    while time.perf_counter() - t0 < budget_s / 3 or n == 0:
        orc.conv2d(x, w, None, (s, s), (p, p))
        orc.conv2d_backward_input(dy, w, x.shape, (s, s), (p, p))
        orc.conv2d_backward_weight(dy, x, w.shape, (s, s), (p, p))
        n += 1
    return n * conv_flops(1, ci, hw, co, k, s, p), time.perf_counter() - t0, \
        "3x3 64->64 @56 at batch 1 (measured at reduced batch), C port of the reference's NumPy loops, 1 thread"


def cpu_threads():
    """Lets the BLAS behind np.matmul use every core this process may run on (launchers such as
    torchrun export OMP_NUM_THREADS=1) and returns the thread count it ends up with."""
    try:
        usable = len(os.sched_getaffinity(0))
    except AttributeError:
        usable = os.cpu_count() or 1
    try:
        from threadpoolctl import threadpool_info, threadpool_limits
        threadpool_limits(limits=usable)
        n = max([p.get("num_threads", 1) for p in threadpool_info()] or [1])
        return int(n)
    except Exception:
        return 1


def cpu_baseline(workload: str, budget_s: float):
    if workload == "linear":
        cores = cpu_threads()
        flops, secs, what = cpu_linear_sample(budget_s)
    else:
        flops, secs, what = cpu_conv_sample(budget_s)
        cores = 1
    return {"value": flops / secs / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": what,
            "seconds": secs}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    warm = max(args.warmup, 1)
    per_step_budget = args.cpu_budget if args.cpu_budget > 0 else max(0.5, min(6.0, 150.0 / (args.steps + warm)))
    for _ in range(warm):
        cpu_baseline(args.workload, per_step_budget)
    flops = secs = 0.0
    base = None
    for _ in range(args.steps):
        base = cpu_baseline(args.workload, per_step_budget)
        secs += base["seconds"]
        flops += base["value"] * 1e12 * base["seconds"]
    value = flops / secs / 1e12
    base = {k: base[k] for k in ("unit", "cores", "kind", "sample")}
    base["value"] = value
    name = {"linear": LINEAR_NAME, "resnet": RESNET_NAME, "pix2pix": PIX2PIX_NAME}[args.workload]
    print(json.dumps({
        "metric": "conv/linear fwd+bwd TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": warm, "ms_per_step": secs / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32 (CPU)", "data": "synthetic", "impl": "reference",
        "config": {"workload": name, "parallelism": "host cores of rank 0",
                   "note": "the reference's CPU arithmetic (NumPy, fp32) on a bounded sample of the workload per step"},
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="nectarml_b200", choices=["nectarml_b200", "reference"])
    ap.add_argument("--workload", default="linear", choices=["linear", "resnet", "pix2pix"])
    ap.add_argument("--per-layer", action="store_true",
                    help="add the contraction kernel's mean time per layer and pass to the JSON line")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-budget", type=float, default=0.0,
                    help="seconds of CPU work per step of the reference arm (default: sized from --steps)")
    ap.add_argument("--only", default="", help="profiling aid: restrict the linear sweep to ROWSxD, or a conv sweep to the layer with this index")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
