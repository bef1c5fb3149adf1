#!/usr/bin/env python
"""Benchmark of the dense-contraction path.

One "step" = forward + input-gradient + weight-gradient (with bias gradient) of every layer of a
workload, inputs resident in HBM.  The headline workload (`value`) is the Linear projection sweep
(X[B*T, d] @ W^T[d, 4d] + b for d in {512, 1024, 2048}, B*T in {4096, 16384}; fp16 storage, fp32
accumulation; synthetic N(0,1) activations, Xavier-uniform weights).  The same JSON line carries,
under `workloads`, the ResNet-style conv shapes at batch 256, the 16 convolutions of the Pix2Pix
U-Net generator at batch 64 and the fp32 (3xTF32) Conv2d of configuration 1, each with its own
roofline block, per-layer table and CPU baseline.  Prints ONE JSON line.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload linear|resnet|pix2pix|config1]

N > 1 is launched with torch.distributed.run; every rank owns its own shard of the rows / batch (weak
scaling: per-GPU work fixed); the weight and bias gradients are written straight into flat fp32
buckets that are all-reduced over NCCL, a bucket as soon as its layers are done.
`--impl reference` times the reference's own CPU arithmetic for the path (NumPy matmul, all host
threads) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import re
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LINEAR_SWEEP = [(rows, d) for d in (512, 1024, 2048) for rows in (4096, 16384)]
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
CONFIG1_LAYER = (64, 56, 64, 3, 1, 1, False)
CONFIG1_BATCH = 8
LINEAR_NAME = ("Linear sweep X[B*T,d]@W^T[d,4d]+b, d in {512,1024,2048} x B*T in {4096,16384}, "
               "forward+dgrad+wgrad+db, fp16 storage / fp32 accumulate")
RESNET_NAME = ("ResNet-style conv shapes, batch 256 per GPU, NHWC fp16: 7x7 s2 3->64 @224, 3x3 64->64 @56, 1x1 256->64 @56, "
               "3x3 s2 128->128 @28, 1x1 s2 1024->2048 @14; forward+dgrad+wgrad+db")
PIX2PIX_NAME = ("Pix2Pix U-Net generator convolutions, batch 64 per GPU, NHWC fp16: 8 Conv2d 4x4 s2 p1 "
                "(3-64-128-256-512-512-512-512-512) + 8 ConvTranspose2d 4x4 s2 p1 with skip-concat inputs; "
                "forward+dgrad+wgrad+db of every layer (normalisation and activations not included)")
CONFIG1_NAME = ("Conv2d fp32 NCHW N=8 64->64 56x56 3x3 s1 p1 with bias, 3xTF32 arithmetic (three tf32 tensor-core "
                "products per fp32 product), forward+dgrad+wgrad+db through the reference-shaped tensors")
WORKLOAD_NAMES = {"linear": LINEAR_NAME, "resnet": RESNET_NAME, "pix2pix": PIX2PIX_NAME, "config1": CONFIG1_NAME}

# NVIDIA's B200 datasheet figures for dense (no 2:4 sparsity) tensor throughput, TFLOP/s
NOMINAL_F16_TFLOPS = 2250.0
NOMINAL_TF32_TFLOPS = 1100.0


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"tflops": float(p["bf16_tflops"]), "tflops_sustained": float(p.get("bf16_tflops_sustained", 0)) or None,
                "hbm_gbs": float(p["hbm_gbs"]), "source": "measured"}
    return {"tflops": 1590.0, "tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


def profiled_traffic(workload: str):
    """dram__bytes_read.sum + dram__bytes_write.sum per contraction launch, averaged over one step, read from
    the ncu summary under profiles/ (a line `traffic_bytes_per_launch: <number>`); None without a capture."""
    path = os.path.join(ROOT, "profiles", f"launch_list_{workload}.md")
    try:
        m = re.search(r"traffic_bytes_per_launch:\s*([0-9.eE+]+)", open(path).read())
        return float(m.group(1)) if m else None
    except OSError:
        return None


class ClockSampler:
    """Samples SM clocks and throttle reasons while a timed region runs: NVML read-only queries every few
    milliseconds from a thread of this process (a 50 ms burst then holds ten samples), or `nvidia-smi -lms`
    when the NVML binding is missing.  Nothing is ever set."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    # nvmlClocksEventReason* bits (nvml.h)
    REASON_BITS = (("sw_power_cap", 0x4), ("hw_slowdown", 0x8), ("sw_thermal_slowdown", 0x20), ("hw_thermal_slowdown", 0x40))

    def __init__(self, index: int, uuid: str = ""):
        self.index, self.uuid, self.proc, self.samples = index, uuid, None, []  # samples: (time, sm MHz, max MHz, reasons)
        self.nvml, self.handle, self.running, self.source = None, None, False, None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            if self.uuid:
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(self.uuid if self.uuid.startswith("GPU-") else "GPU-" + self.uuid)
            else:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.nvml, self.running, self.source = pynvml, True, "nvml"
            self.thread = threading.Thread(target=self._poll_nvml, daemon=True)
            self.thread.start()
            return
        except Exception:  # no binding, no library, or the device is not visible to NVML under this id
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "25"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.source = "nvidia-smi"
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _poll_nvml(self):
        nv = self.nvml
        reasons_fn = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
        while self.running:
            try:
                mhz = float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                mask = int(reasons_fn(self.handle))
                self.samples.append((time.time(), mhz, self.max_mhz, tuple(n for n, b in self.REASON_BITS if mask & b)))
            except Exception:
                pass
            time.sleep(0.004)

    def _pump(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                mhz, mx = float(parts[0]), float(parts[1])
            except ValueError:
                continue
            names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
            self.samples.append((time.time(), mhz, mx, tuple(n for n, v in zip(names, parts[2:6]) if v.lower().startswith("active"))))

    def window(self, t0: float, t1: float):
        """Clock summary of the samples taken between t0 and t1 (the sampler keeps running)."""
        if self.source is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no clock source (NVML binding and nvidia-smi unavailable)"]}
        slack = (0.0, 0.0) if self.source == "nvml" else (0.05, 0.15)
        inside = [x for x in list(self.samples) if t0 - slack[0] <= x[0] <= t1 + slack[1]]
        if not inside:  # timed region shorter than one sample: the samples nearest to it
            inside = sorted(list(self.samples), key=lambda x: abs(x[0] - 0.5 * (t0 + t1)))[:3]
        reasons = sorted({r for x in inside for r in x[3]})
        return {"sm_mhz": statistics.median(x[1] for x in inside) if inside else None,
                "sm_max_mhz": max(x[2] for x in inside) if inside else None,
                "reasons": reasons, "samples": len(inside), "source": self.source}

    def stop(self):
        self.running = False
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()


# ------------------------------------------------------------------ accounting --
def linear_flops(rows, d):
    return 3 * 2.0 * rows * d * 4 * d  # forward + dgrad + wgrad


def conv_flops(batch, c_in, hw, c_out, k, s, p, transposed=False):
    ho = hw if transposed else (hw + 2 * p - k) // s + 1  # a transposed layer does its multiplies per INPUT pixel
    return 3 * 2.0 * batch * ho * ho * c_out * c_in * k * k


def conv_out_hw(hw, k, s, p, transposed):
    return (hw - 1) * s - 2 * p + k if transposed else (hw + 2 * p - k) // s + 1


def pass_bytes(n_x, n_w, n_y, es):
    """Algorithmic minimum traffic of the three passes: each operand and result once at storage width, the weight
    gradient in fp32."""
    return [(n_x + n_w + n_y) * es, (n_y + n_w + n_x) * es, (n_x + n_y) * es + n_w * 4]


# ------------------------------------------------------------------ workloads --
def bucket_groups(numel, ratio=0.5, min_bytes=8 << 20):
    """Cuts layers (fp32 gradient elements per layer, in execution order) into consecutive buckets: a bucket is
    closed once it holds at least `ratio` times what is still to come and `min_bytes`, so the early buckets are
    large (their all-reduce overlaps the remaining layers) and the last, exposed one is small."""
    groups, cur, acc = [], [], 0
    for i, n_ in enumerate(numel):
        cur.append(i)
        acc += n_
        rest = sum(numel[i + 1:])
        if rest and acc >= ratio * rest and acc * 4 >= min_bytes:
            groups.append(cur)
            cur, acc = [], 0
    if cur:
        groups.append(cur)
    return groups


class Workload:
    """Tensors of one workload on one GPU, its step, and the algorithmic work of every contraction launch."""

    def __init__(self, key, dev, rank, world, only=""):
        import torch
        from nectarml_b200 import ops
        from nectarml_b200.ops import ConvGeometry
        from nectarml_b200.parallel import GradientBucket
        self.key, self.dev, self.world = key, dev, world
        self.ops, self.torch = ops, torch
        self.launches = []  # one dict per contraction launch of a step, in launch order
        self.layers = []
        self.math = "3xtf32" if key == "config1" else "f16"
        self.es = 4 if key == "config1" else 2
        if key == "linear":
            # under data parallelism the layers with the largest gradients go first, so that their all-reduce
            # overlaps the other layers' kernels (on one GPU the listed order measured 1-2 % faster)
            sweep = sorted(LINEAR_SWEEP, key=lambda s_: (-s_[1], -s_[0])) if world > 1 else list(LINEAR_SWEEP)
            if only:  # profiling aid: one shape of the sweep, e.g. --only 16384x1024
                r_, d_ = (int(v) for v in only.lower().split("x"))
                sweep = [(r_, d_)]
            rng = np.random.default_rng(1235 + rank)
            for rows, d in sweep:
                bound = np.sqrt(6.0 / (d + 4 * d))
                l = {"name": f"linear {rows}x{d}->{4 * d}", "rows": rows, "d": d,
                     "x": torch.from_numpy(rng.standard_normal((rows, d), dtype=np.float32)).half().pin_memory(),
                     "dy": torch.from_numpy(rng.standard_normal((rows, 4 * d), dtype=np.float32)).half().pin_memory(),
                     "w": torch.from_numpy(rng.uniform(-bound, bound, (4 * d, d)).astype(np.float32)).half(),
                     "b": torch.zeros(4 * d, dtype=torch.float16)}
                l.update(xd=l["x"].to(dev), dyd=l["dy"].to(dev), wd=l["w"].to(dev), bd=l["b"].to(dev),
                         y=torch.empty(rows, 4 * d, dtype=torch.float16, device=dev),
                         dx=torch.empty(rows, d, dtype=torch.float16, device=dev))
                self.layers.append(l)
                by = pass_bytes(rows * d, 4 * d * d, rows * 4 * d, 2)
                for i, ps in enumerate(("fwd", "dgrad", "wgrad")):
                    self.launches.append({"layer": l["name"], "pass": ps, "flops": 2.0 * rows * d * 4 * d, "bytes": by[i]})
            shapes = []
            for l in self.layers:
                shapes += [(4 * l["d"], l["d"]), (4 * l["d"],)]
        else:
            sweep, batch = {"resnet": (RESNET_SWEEP, RESNET_BATCH), "pix2pix": (PIX2PIX_SWEEP, PIX2PIX_BATCH),
                            "config1": ([CONFIG1_LAYER], CONFIG1_BATCH)}[key]
            if only:  # profiling aid: one layer of the sweep by index
                sweep = [sweep[int(only)]]
            torch.manual_seed(1237 + rank)
            nchw = key == "config1"
            dt = torch.float32 if nchw else torch.float16
            self.layout = "nchw" if nchw else "nhwc"
            for (ci, hw, co, k, s, p, tr) in sweep:
                g = ConvGeometry(batch, ci, hw, hw, co, k, k, (s, s), (p, p), transposed=tr)
                ho, wo = g.out_hw()
                std = 0.02 if key == "pix2pix" else float(np.sqrt(2.0 / (ci * k * k)))
                xs, ys = g.act_shape("in", self.layout), g.act_shape("out", self.layout)
                l = {"g": g, "name": f"{'convT' if tr else 'conv'} {k}x{k} s{s} {ci}->{co} @{hw}",
                     "xd": torch.randn(*xs, device=dev).to(dt), "dyd": torch.randn(*ys, device=dev).to(dt),
                     "wd": (torch.randn(*g.weight_shape(), device=dev) * std).to(dt),
                     "bd": (torch.randn(co, device=dev) * 0.1).to(dt) if nchw else None,
                     "y": torch.empty(*ys, dtype=dt, device=dev), "dx": torch.empty(*xs, dtype=dt, device=dev)}
                self.layers.append(l)
                fl = conv_flops(batch, ci, hw, co, k, s, p, tr) / 3
                by = pass_bytes(batch * hw * hw * ci, ci * co * k * k, batch * ho * wo * co, self.es)
                for i, ps in enumerate(("fwd", "dgrad", "wgrad")):
                    self.launches.append({"layer": l["name"], "pass": ps, "flops": fl, "bytes": by[i]})
            shapes = []
            for l in self.layers:
                shapes += [l["g"].weight_shape(), (l["g"].c_out,)]
        # Weight and bias gradients land directly in flat fp32 buckets (dw / db are caller-owned pointers of the
        # C ABI), so that one all-reduce per bucket moves them.  Layers are taken in execution order; a bucket is
        # closed once it holds at least `bucket_ratio` times what is still to come (and 8 MB), so the early
        # buckets are large and overlap the remaining layers while the last, exposed one is small.
        ratio = float(os.environ.get("NML_BENCH_BUCKET_RATIO", "0.5"))
        numel = [int(np.prod(shapes[2 * i])) + int(np.prod(shapes[2 * i + 1])) for i in range(len(self.layers))]
        groups = bucket_groups(numel, ratio)
        self.buckets, self.last_of_bucket = [], {}
        for b, grp in enumerate(groups):
            bucket = GradientBucket([sh for i in grp for sh in (shapes[2 * i], shapes[2 * i + 1])], dev)
            self.buckets.append(bucket)
            for j, i in enumerate(grp):
                self.layers[i]["dw"], self.layers[i]["db"] = bucket.view(2 * j), bucket.view(2 * j + 1)
            self.last_of_bucket[grp[-1]] = b
        # SMs left to NCCL while an all-reduce may be in flight (see nml_set_sm_limit); 0 = none
        self.sm_reserve = int(os.environ.get("NML_BENCH_SM_RESERVE", "16")) if world > 1 else 0
        self.sms = torch.cuda.get_device_properties(dev).multi_processor_count
        if world > 1:  # launch order of the data-parallel step: every weight gradient, then forward + dgrad per layer
            self.launches = [x for x in self.launches if x["pass"] == "wgrad"] + [x for x in self.launches if x["pass"] != "wgrad"]
        self.step_flops = sum(x["flops"] for x in self.launches)
        self.bytes_resident = sum(t.numel() * t.element_size() for l in self.layers for t in
                                  (l["xd"], l["dyd"], l["wd"], l["y"], l["dx"], l["dw"]))

    def forward_and_dgrad(self, l):
        ops = self.ops
        if self.key == "linear":
            ops.linear_forward(l["xd"], l["wd"], l["bd"], out=l["y"])
            ops.linear_backward_data(l["dyd"], l["wd"], out=l["dx"])
        else:
            ops.conv_forward(l["g"], l["xd"], l["wd"], l["bd"], layout=self.layout, math=self.math, out=l["y"])
            ops.conv_backward_data(l["g"], l["dyd"], l["wd"], layout=self.layout, math=self.math, out=l["dx"])

    def wgrad(self, l):
        ops = self.ops
        if self.key == "linear":
            ops.linear_backward_weight(l["xd"], l["dyd"], dw=l["dw"], db=l["db"])
        else:
            ops.conv_backward_weight(l["g"], l["xd"], l["dyd"], layout=self.layout, math=self.math, dw=l["dw"], db=l["db"])

    def layer_passes(self, l):
        self.forward_and_dgrad(l)
        self.wgrad(l)

    def step(self, communicate=True):
        if self.world == 1:
            for l in self.layers:
                self.layer_passes(l)
            return
        # Data parallel: the weight gradients are the only thing exchanged, so they are computed first (largest
        # first) and each bucket's all-reduce is issued as soon as its layers are done; the forward and
        # input-gradient passes of all layers then run while the exchange is in flight, on the SMs NCCL leaves.
        pending = []
        for i, l in enumerate(self.layers):
            self.wgrad(l)
            if communicate and i in self.last_of_bucket:
                pending.append(self.buckets[self.last_of_bucket[i]].all_reduce(async_op=True))
                if self.sm_reserve:  # the kernels that follow share the GPU with this exchange
                    self.ops.set_sm_limit(self.sms - self.sm_reserve)
        for l in self.layers:
            self.forward_and_dgrad(l)
        if self.sm_reserve:
            self.ops.set_sm_limit(0)
        for p in pending:
            if p is not None:
                p.wait()

    def capture(self, communicate=True):
        """The launches of one step as CUDA graphs: the C ABI neither allocates nor synchronises, so its calls
        record as they are (tensor maps travel as kernel parameters).  Returns (replay function, launches recorded).
        The all-reduces stay OUTSIDE the graphs: the data-parallel step is cut into one graph per gradient bucket
        (the weight gradients that fill it) and one for the forward and input-gradient passes, and each bucket's
        all-reduce is issued between two replays, exactly where the eager step issues it."""
        torch, ops = self.torch, self.ops
        from nectarml_b200.train import capture_into

        def record(fn):
            g = torch.cuda.CUDAGraph()
            with capture_into(g):  # (garbage collector held off, capture errors checked per thread)
                fn()
            return g

        n0 = ops.launch_count()
        if self.world == 1 or not communicate:
            g = record(lambda: self.step(False))
            return g.replay, ops.launch_count() - n0
        segments, first = [], 0
        for i in range(len(self.layers)):
            if i in self.last_of_bucket:
                span = range(first, i + 1)
                segments.append((record(lambda: [self.wgrad(self.layers[j]) for j in span]), self.last_of_bucket[i]))
                first = i + 1
                if self.sm_reserve:  # planned into every kernel recorded from here on
                    ops.set_sm_limit(self.sms - self.sm_reserve)
        tail = list(range(first, len(self.layers)))
        segments.append((record(lambda: [self.wgrad(self.layers[j]) for j in tail] +
                                        [self.forward_and_dgrad(l) for l in self.layers]), None))
        if self.sm_reserve:
            ops.set_sm_limit(0)

        def replay():
            pending = []
            for g, bucket in segments:
                g.replay()
                if bucket is not None:
                    pending.append(self.buckets[bucket].all_reduce(async_op=True))
            for p in pending:
                if p is not None:
                    p.wait()
        return replay, ops.launch_count() - n0


def time_steps(torch, dist, world, dev, fn, steps):
    """Times `steps` calls on the device between barriers; returns max-over-ranks milliseconds."""
    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
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


def graph_wanted(world):
    """Whether the timed step of the kernel sweeps is replayed from a CUDA graph (NML_BENCH_GRAPH=0: eager)."""
    return os.environ.get("NML_BENCH_GRAPH", "1") != "0"


def measure(wl, args, peaks, sampler, torch, dist, steps, per_layer):
    """Warm-up, the timed region, and per-launch CUDA-event durations of the contraction launches of one workload."""
    ops, world, dev = wl.ops, wl.world, wl.dev
    for _ in range(max(args.warmup, 3)):
        wl.step()
    ops.device_status()

    def settle():
        # Every leg below is a burst of a few tens of milliseconds that starts from an idle GPU, so that they see
        # the same clocks (a 1 kW part power-caps within ~0.1 s of dense tensor work; the sustained leg of the
        # headline workload reports that regime).
        torch.cuda.synchronize()
        time.sleep(args.idle_s)
        if world > 1:
            dist.barrier()

    # per-launch durations of the contraction kernel (with its second-stage reduction where it has one),
    # CUDA events on the launching stream
    n1 = len(wl.launches)
    n_rec = n1 * steps
    settle()
    t0 = time.time()
    ops.profile_begin(n_rec)
    for _ in range(steps):
        wl.step()
    per_launch_ms = ops.profile_end(n_rec)
    clocks_launches = sampler.window(t0, time.time()) if sampler else None

    # The timed step: the launches of one step recorded once into a CUDA graph and replayed (one host call per
    # step instead of one per kernel; the kernels, their order and their arguments are those of the eager step).
    step, step_nocomm, per_step_launches = wl.step, (lambda: wl.step(communicate=False)), None
    graphed = graph_wanted(world)
    if graphed:
        step, per_step_launches = wl.capture(True)
        if world > 1:
            step_nocomm, _ = wl.capture(False)
        for _ in range(2):
            step()
    wl.timed_step, wl.graphed = step, graphed
    settle()
    launches0 = ops.launch_count()
    t0 = time.time()
    ms_total = time_steps(torch, dist, world, dev, step, steps)
    t1 = time.time()
    launches = per_step_launches * steps if graphed else ops.launch_count() - launches0
    clocks = sampler.window(t0, t1) if sampler else None
    ops.device_status()
    comm_ms_exposed = None
    if world > 1:  # the same step without its all-reduces: the difference is what the exchange costs the step
        settle()
        ms_nocomm = time_steps(torch, dist, world, dev, step_nocomm, steps)
        comm_ms_exposed = (ms_total - ms_nocomm) / steps
    reps = len(per_launch_ms) // n1 if n1 else 0
    mean = [sum(per_launch_ms[i:reps * n1:n1]) / reps for i in range(n1)] if reps else []
    kern_ms = sum(mean)
    tensor_peak = (NOMINAL_TF32_TFLOPS / 3) if wl.key == "config1" else peaks["tflops"]
    ridge = tensor_peak * 1e12 / (peaks["hbm_gbs"] * 1e9)  # FLOP per byte above which the tensor pipe is the bound
    table, t_tensor, f_tensor, t_hbm, b_hbm = [], 0.0, 0.0, 0.0, 0.0
    for i, x in enumerate(wl.launches):
        if not mean:
            break
        sec = mean[i] * 1e-3
        hbm = (x["flops"] / x["bytes"]) < ridge
        if hbm:
            t_hbm += sec
            b_hbm += x["bytes"]
        else:
            t_tensor += sec
            f_tensor += x["flops"]
        row = {"layer": x["layer"], "pass": x["pass"], "us": round(mean[i] * 1e3, 1),
               "tflops": round(x["flops"] / sec / 1e12, 1), "gbs": round(x["bytes"] / sec / 1e9, 0),
               "bound": "hbm" if hbm else "tensor",
               "frac": round((x["bytes"] / sec / 1e9 / peaks["hbm_gbs"]) if hbm else (x["flops"] / sec / 1e12 / tensor_peak), 3)}
        table.append(row)
    achieved = wl.step_flops / (kern_ms * 1e-3) / 1e12 if kern_ms > 0 else None
    src = f"{peaks['source']} burst bf16 (MEASURED_PEAKS.json)" if peaks["source"] == "measured" else "fallback"
    if wl.key == "config1":
        src = "NVIDIA nominal dense tf32 (1100 TFLOP/s) / 3, three tensor-core products per fp32 product"
    nominal = (NOMINAL_TF32_TFLOPS / 3) if wl.key == "config1" else NOMINAL_F16_TFLOPS
    roof = {"bound": "tensor", "achieved": achieved, "peak": tensor_peak, "unit": "TFLOP/s",
            "frac": (achieved / tensor_peak) if achieved else None, "peak_source": src,
            "frac_nominal": (achieved / nominal) if achieved else None,
            "nominal_peak": nominal, "nominal_source": "NVIDIA B200 datasheet, dense (half of the 2:4-sparsity figure)",
            "kernel": "umma_conv_kernel", "launches_timed": len(per_launch_ms),
            "clocks": clocks_launches, "traffic": profiled_traffic(wl.key),
            "algorithmic_bytes_per_launch": sum(x["bytes"] for x in wl.launches) / max(n1, 1)}
    if peaks.get("tflops_sustained") and wl.key != "config1":
        roof["frac_of_sustained_peak"] = (achieved / peaks["tflops_sustained"]) if achieved else None
    if t_hbm > 0:  # the layers below the ridge, judged on bandwidth
        roof["hbm_bound_launches"] = {"achieved": b_hbm / t_hbm / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                      "frac": b_hbm / t_hbm / 1e9 / peaks["hbm_gbs"],
                                      "launches": sum(1 for r in table if r["bound"] == "hbm")}
    if t_tensor > 0:
        roof["tensor_bound_launches"] = {"achieved": f_tensor / t_tensor / 1e12, "peak": tensor_peak, "unit": "TFLOP/s",
                                         "frac": f_tensor / t_tensor / 1e12 / tensor_peak,
                                         "launches": sum(1 for r in table if r["bound"] == "tensor")}
    out = {"value": wl.step_flops * world * steps / (ms_total * 1e-3) / 1e12, "unit": "TFLOP/s",
           "ms_per_step": ms_total / steps, "steps": steps, "gpu_launches": int(launches), "clocks": clocks,
           "roofline": roof, "workload": WORKLOAD_NAMES[wl.key], "buckets": len(wl.buckets), "sm_reserve": wl.sm_reserve,
           "launch": ("CUDA graph replay of the step's kernels" + (", all-reduces issued between the graphs of the buckets" if world > 1 else ""))
           if graphed else "one host call per kernel"}
    if comm_ms_exposed is not None:
        out["comm_ms_exposed"] = comm_ms_exposed
        out["roofline"]["achieved_scope"] = "rank 0's GPU, all-reduces in flight"
    if per_layer:
        out["per_layer"] = table
    return out


TRAIN_NAMES = {
    "resnet50_step": ("ResNet-50 training step (bottleneck blocks [3,4,6,3], BatchNorm, ReLU, 1000-way Linear head), fp16 AMP with "
                      "fp32 master weights, synthetic 224x224x3 images ~N(0,1), uniform labels, global batch 2048 sharded over the "
                      "GPUs in micro-batches of at most 256, all-reduce of the flat weight-gradient buffer, fused SGD-momentum update"),
    "pix2pix_step": ("Pix2Pix U-Net generator training step (8 Conv2d + 8 ConvTranspose2d 4x4 s2 p1, skip concatenation, BatchNorm + "
                     "LeakyReLU(0.2) / ReLU, tanh), fp16 AMP, synthetic 256x256x3 inputs U[-1,1], L1 loss against a synthetic target, "
                     "global batch 64 sharded over the GPUs, all-reduce of the flat weight-gradient buffer, fused SGD-momentum update"),
}


def measure_train(kind, args, peaks, sampler, torch, dist, dev, rank, world):
    """img/s of one of the two conv-net training steps at a FIXED global batch (strong scaling)."""
    from nectarml_b200 import ops, train
    torch.manual_seed(4321 + rank)
    # NML_BENCH_SHARD_OF=N times one GPU's share of an N-GPU run (no exchange): the per-GPU shapes of a larger run
    # can be checked and timed on a single GPU
    shard_of = max(world, int(os.environ.get("NML_BENCH_SHARD_OF", "1"))) if world == 1 else world
    if kind == "resnet50_step":
        net, global_batch, hw, loss = train.ResNet50(dev), 2048, 224, "cross_entropy"
        per_gpu = global_batch // shard_of
        micro = min(per_gpu, int(os.environ.get("NML_BENCH_MICRO_BATCH", "256")))
    else:
        net, global_batch, hw, loss = train.Pix2PixGenerator(dev), 64, 256, "l1"
        per_gpu = global_batch // shard_of
        micro = per_gpu
    net.init(seed=11)
    net.store.sm_reserve = int(os.environ.get("NML_BENCH_SM_RESERVE", "16"))
    n_micro = per_gpu // micro
    step = train.TrainStep(net, loss, lr=0.01 if kind == "resnet50_step" else 2e-4, momentum=0.9, weight_decay=1e-4)
    x = (torch.randn(micro, hw, hw, 3, device=dev) if loss == "cross_entropy" else torch.rand(micro, hw, hw, 3, device=dev) * 2 - 1).half()
    target = torch.randint(0, 1000, (micro,), device=dev) if loss == "cross_entropy" else (torch.rand(micro, hw, hw, 3, device=dev) * 2 - 1).half()
    count = global_batch if loss == "cross_entropy" else global_batch * hw * hw * 3
    use_graphs = os.environ.get("NML_BENCH_GRAPHS", "1") != "0"
    net.store.flops = 0.0
    launches_before = ops.launch_count()
    step.micro_batch(x, target, count, first=True, last=False)   # eager once: counts the algorithmic FLOPs, sizes the workspaces
    flops_micro = net.store.flops
    launches_micro = ops.launch_count() - launches_before        # this library's kernels in one micro-batch
    ops.device_status()
    split = None
    if use_graphs and n_micro == 1 and net.split_backward and world > 1 and os.environ.get("NML_BENCH_SPLIT", "1") != "0":
        split = step.capture_split(x, target, count)   # decoder's gradients leave while the encoder's backward runs
    graphs = step.capture(x, target, count, accumulate_variants=(False, True) if n_micro > 1 else (False,)) if use_graphs and not split else None

    def one_step():
        # (synthetic data: every micro-batch reuses the same resident tensors, as the static inputs of a graph do)
        if split:
            step.replay_split(split)
        elif graphs:
            for i in range(n_micro):
                graphs[i > 0][0].replay()
            step.exchange_all()
        else:
            for i in range(n_micro):
                step.micro_batch(x, target, count, first=(i == 0), last=(i == n_micro - 1))
            net.store.wait_exchange()
        step.optimizer_step()

    for _ in range(2):
        one_step()
    ops.device_status()
    steps = max(2, min(args.steps, 4 if kind == "resnet50_step" else 10))
    torch.cuda.synchronize()
    time.sleep(args.idle_s)
    launches0 = ops.launch_count()
    t0 = time.time()
    ms = time_steps(torch, dist, world, dev, one_step, steps)
    t1 = time.time()
    # (a replayed graph does not pass through the library's counter: its launches are those of the captured micro-batch)
    launches = (ops.launch_count() - launches0) + (launches_micro * n_micro * steps if (graphs or split) else 0)
    ops.device_status()
    clocks = sampler.window(t0, t1) if sampler else None
    step_flops = flops_micro * n_micro * world
    achieved = step_flops * steps / (ms * 1e-3) / 1e12
    if shard_of != world:
        global_batch = per_gpu  # a single GPU's share was timed
    return {"value": global_batch * steps / (ms * 1e-3), "unit": "img/s", "img_s": global_batch * steps / (ms * 1e-3),
            "ms_per_step": ms / steps, "steps": steps, "global_batch": global_batch, "per_gpu_batch": per_gpu,
            "micro_batch": micro, "scaling": "strong", "cuda_graphs": bool(graphs or split), "split_backward": bool(split),
            "contraction_tflops": achieved, "contraction_gflop_per_image": step_flops / global_batch / 1e9,
            "frac_of_measured_tensor_peak": achieved / world / peaks["tflops"], "gpu_launches": launches, "clocks": clocks,
            "found_inf": int(net.store.found_inf), "workload": TRAIN_NAMES[kind],
            "note": "whole step: forward, backward, gradient exchange, finiteness check, SGD-momentum update; contraction_tflops "
                    "counts only the Conv2d / ConvTranspose2d / Linear passes' algorithmic FLOPs over the whole step time"}


def pin_to_gpu_numa_node(index: int):
    """Binds this process to the CPUs NVML lists as local to GPU `index` (a read-only NVML query), so that the
    pinned host buffers of the end-to-end leg are allocated on, and driven from, the GPU's own NUMA node.
    Returns the number of CPUs bound to, or None when NVML has nothing to say."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        cpus = {64 * w + b for w, m in enumerate(words) for b in range(64) if (m >> b) & 1}
        cpus &= set(os.sched_getaffinity(0))
        if cpus:
            os.sched_setaffinity(0, cpus)
            return len(cpus)
    except Exception:
        pass
    return None


def run_gpu(args):
    import torch
    import torch.distributed as dist
    from nectarml_b200 import build, ops

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    numa = pin_to_gpu_numa_node(local) if world > 1 else None
    if world > 1:
        # a fixed, small CTA budget for NCCL: the contraction kernels are persistent, one CTA per SM, so every SM
        # NCCL takes is one of theirs (NVSwitch keeps the all-reduce fast at a few CTAs)
        os.environ.setdefault("NCCL_MAX_CTAS", os.environ.get("NML_BENCH_NCCL_CTAS", "16"))
        dist.init_process_group("nccl", device_id=dev)
        if local == 0:  # one rank (re)builds a stale library, the others wait for it
            build.build()
        dist.barrier()
    else:
        build.build()
    peaks = measured_peaks()
    sampler = ClockSampler(local, str(getattr(torch.cuda.get_device_properties(dev), "uuid", "") or "")) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.25)

    if args.workload in TRAIN_NAMES:  # one of the training steps on its own: img/s at the fixed global batch
        r = measure_train(args.workload, args, peaks, sampler, torch, dist, dev, rank, world)
        if sampler:
            sampler.stop()
        if rank == 0:
            print(json.dumps({"metric": "conv-net train img/s", "value": r["value"], "unit": "img/s", "n_gpus": world,
                              "steps": r["steps"], "warmup": 2, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
                              "scaling": "strong", "vs_baseline": None, "dtype": "f16 (fp32 accumulate, fp32 master weights)",
                              "data": "synthetic", "impl": "nectarml_b200",
                              "config": {"workload": TRAIN_NAMES[args.workload], "global_batch": r["global_batch"],
                                         "parallelism": f"dp{world}" if world > 1 else "1 GPU"},
                              "e2e": None, "gpu_launches": r["gpu_launches"], "clocks": r["clocks"], "detail": r}), flush=True)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return r

    wl = Workload(args.workload, dev, rank, world, args.only)
    head = measure(wl, args, peaks, sampler, torch, dist, args.steps, per_layer=True)

    # sustained leg: the same step back to back for >= 3 s, with the clocks seen (time x MHz compares rounds
    # measured at different clocks)
    sustained = None
    if args.sustain_s > 0:
        est_ms = max(head["ms_per_step"], 1e-3)
        n = max(10, int(args.sustain_s * 1e3 / est_ms))
        t0 = time.time()
        ms = time_steps(torch, dist, world, dev, wl.timed_step, n)
        t1 = time.time()
        ck = sampler.window(t0 + 0.5, t1) if sampler else None
        sustained = {"value": wl.step_flops * world * n / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "seconds": ms * 1e-3,
                     "steps": n, "ms_per_step": ms / n, "clocks": ck,
                     "ms_per_step_x_sm_mhz": (ms / n) * ck["sm_mhz"] if ck and ck.get("sm_mhz") else None,
                     "frac_of_sustained_peak": (wl.step_flops * n / (ms * 1e-3) / 1e12 / peaks["tflops_sustained"])
                     if peaks.get("tflops_sustained") and wl.key != "config1" else None}
        ops.device_status()

    # End to end through the public API with host buffers (pinned), copies inside the timed region: every
    # layer's x and dy come from the host and its results go back to it -- the gradients dw, db (`e2e`: what a
    # data-parallel caller takes off the device; y and dx stay there, as the reference's host ops leave every
    # result on the device) or all four results (`e2e_all_results`).  Copies run on their own streams, ordered
    # against the compute stream by events, so a layer's transfers overlap the other layers' kernels; every step
    # ends with the compute stream waiting for that step's last device-to-host copy.
    e2e, e2e_legs = None, {}
    if args.workload == "linear":
        layers = wl.layers
        for l in layers:
            for k_ in ("y", "dx", "dw", "db"):
                l[k_ + "_host"] = torch.empty(l[k_].shape, dtype=l[k_].dtype).pin_memory()
        s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        ev_in = [torch.cuda.Event() for _ in layers]
        ev_done = [torch.cuda.Event() for _ in layers]
        ev_out = [torch.cuda.Event() for _ in layers]

        returned = ["dw", "db"]

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
                cur.wait_event(ev_out[i])  # the previous step's copies of this layer's results have left the device
                wl.layer_passes(l)
                if world > 1:
                    dist.all_reduce(l["dw"])
                    dist.all_reduce(l["db"])
                ev_done[i].record(cur)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_done[i])
                    for k_ in returned:
                        l[k_ + "_host"].copy_(l[k_], non_blocking=True)
                    ev_out[i].record(s_out)
            cur.wait_event(ev_out[-1])

        e2e_legs = {}
        for name, keys in (("e2e_all_results", ["y", "dx", "dw", "db"]), ("e2e", ["dw", "db"])):
            returned[:] = keys
            for _ in range(2):
                step_e2e()
            e2e_steps = max(2, min(args.steps, 5))
            torch.cuda.synchronize()
            time.sleep(args.idle_s)
            e2e_ms = time_steps(torch, dist, world, dev, step_e2e, e2e_steps)
            for l in layers:  # what reached the host is what is on the device
                if not torch.equal(l["db_host"], l["db"].cpu()) or not torch.equal(l["y_host"][:64], l["y"][:64].cpu()):
                    raise SystemExit("bench.py: end-to-end leg returned stale results")
            h2d = sum(l["x"].numel() * 2 + l["dy"].numel() * 2 for l in layers)
            d2h = sum(l[k_].numel() * l[k_].element_size() for l in layers for k_ in keys)
            e2e_legs[name] = {"value": wl.step_flops * world * e2e_steps / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                              "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                              "returns": ", ".join(keys) + " of every layer" + ("" if len(keys) == 4 else
                                                                                " (y and dx stay on the device, where the reference's host ops leave every result)")}
        e2e = e2e_legs["e2e"]

    # the other workloads of the path, each with its own roofline block (device-resident inputs)
    others = {}
    if args.workload == "linear" and not args.only and not args.headline_only:
        wl.timed_step = None   # (its graphs go with it now, not at some later garbage collection)
        del wl
        gc.collect()
        torch.cuda.empty_cache()
        for key, label in (("resnet", "resnet_conv"), ("pix2pix", "pix2pix_conv"), ("config1", "config1_fp32_3xtf32")):
            w2 = Workload(key, dev, rank, world)
            others[label] = measure(w2, args, peaks, sampler, torch, dist, max(3, min(args.steps, 20)), per_layer=True)
            if rank == 0 and world == 1 and not args.no_cpu_baseline:
                others[label]["cpu_baseline"] = cpu_baseline(key, budget_s=4.0)
            w2.timed_step = None
            del w2
            gc.collect()
            torch.cuda.empty_cache()
        for kind in ("resnet50_step", "pix2pix_step"):
            others[kind] = measure_train(kind, args, peaks, sampler, torch, dist, dev, rank, world)
            torch.cuda.empty_cache()
    if sampler:
        sampler.stop()

    out = None
    if rank == 0:
        out = {
            "metric": "conv/linear fwd+bwd TFLOP/s", "value": head["value"], "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": head["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32 via 3xTF32 (fp32 accumulate)" if args.workload == "config1" else "f16 (fp32 accumulate)",
            "data": "synthetic", "impl": "nectarml_b200",
            "config": {"workload": WORKLOAD_NAMES[args.workload], "layers": len(head.get("per_layer", [])) // 3,
                       "parallelism": (f"dp{world} (rows / batch sharded, NCCL all-reduce of {head['buckets']} flat dW/db buckets, "
                                       f"NCCL_MAX_CTAS={os.environ.get('NCCL_MAX_CTAS')}, {head['sm_reserve']} SMs left to it while in flight)")
                       if world > 1 else "1 GPU",
                       "host_cpus_bound": numa, "launch": head["launch"],
                       "l2": "inputs and outputs of one step exceed the 126 MB L2 several times over; every step cycles through it",
                       "timing": f"every timed region is a burst of `steps` steps from an idle GPU ({args.idle_s} s pause); `sustained` is the same step for >= {args.sustain_s} s"},
            "e2e": e2e, "e2e_all_results": e2e_legs.get("e2e_all_results") if e2e else None, "gpu_launches": head["gpu_launches"], "clocks": head["clocks"], "roofline": head["roofline"],
            "per_layer": head.get("per_layer"),
        }
        if "comm_ms_exposed" in head:
            out["comm_ms_exposed"] = head["comm_ms_exposed"]
        if sustained:
            out["sustained"] = sustained
        if others:
            out["workloads"] = others
        if world == 1 and not args.no_cpu_baseline:
            out["cpu_baseline"] = cpu_baseline(args.workload, budget_s=12.0)
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return out


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


def cpu_conv_sample(workload: str, budget_s: float):
    """One layer of the conv workload at batch 1 through the C port of the reference's NumPy loops."""
    from oracle import nectar_oracle as orc
    rng = np.random.default_rng(1237)
    if workload == "pix2pix":
        ci, hw, co, k, s, p, tr = PIX2PIX_SWEEP[2]  # 4x4 s2 128->256 @64
    else:
        ci, hw, co, k, s, p, tr = RESNET_SWEEP[1]  # 3x3 64->64 @56 (also configuration 1's layer)
    ho = conv_out_hw(hw, k, s, p, tr)
    x = rng.standard_normal((1, ci, hw, hw), dtype=np.float32)
    w = rng.standard_normal((co, ci, k, k), dtype=np.float32)
    dy = rng.standard_normal((1, co, ho, ho), dtype=np.float32)
    t0 = time.perf_counter()
    n = 0
    while time.perf_counter() - t0 < budget_s / 3 or n == 0:
        orc.conv2d(x, w, None, (s, s), (p, p))
        orc.conv2d_backward_input(dy, w, x.shape, (s, s), (p, p))
        orc.conv2d_backward_weight(dy, x, w.shape, (s, s), (p, p))
        n += 1
    return n * conv_flops(1, ci, hw, co, k, s, p), time.perf_counter() - t0, \
        f"conv {k}x{k} s{s} {ci}->{co} @{hw} at batch 1 (measured at reduced batch), C port of the reference's NumPy loops, 1 thread"


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
        flops, secs, what = cpu_conv_sample(workload, budget_s)
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
    print(json.dumps({
        "metric": "conv/linear fwd+bwd TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": warm, "ms_per_step": secs / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32 (CPU)", "data": "synthetic", "impl": "reference",
        "config": {"workload": WORKLOAD_NAMES[args.workload], "parallelism": "host cores of rank 0",
                   "note": "the reference's CPU arithmetic (NumPy, fp32) on a bounded sample of the workload per step"},
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="nectarml_b200", choices=["nectarml_b200", "reference"])
    ap.add_argument("--workload", default="linear",
                    choices=["linear", "resnet", "pix2pix", "config1", "resnet50_step", "pix2pix_step"])
    ap.add_argument("--headline-only", action="store_true", help="skip the extra workloads of the default run")
    ap.add_argument("--sustain-s", type=float, default=3.0, help="seconds of the sustained leg (0: skip)")
    ap.add_argument("--idle-s", type=float, default=0.5, help="pause before each timed burst")
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
