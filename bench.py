#!/usr/bin/env python
"""Benchmark of the convolution hot path inside a ResNet-50 training step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload resnet50|vgg16bn|alexnet]

Prints ONE JSON line (rank 0).  ``value`` = images/s of the whole job with the batch already
resident in HBM, timed on the device with CUDA events (max over ranks); ``e2e`` = the same through
the public ``Model.train_batch`` call with pinned host buffers, host->device copy and loss read-back
inside the timed region.  ``roofline`` describes the convolution kernels (the dominant kernels): the
same K steps are run once more with a CUDA event pair around every Conv2D pass (kept out of the loop
that gives ``value``: an event between two kernels keeps the second from starting while the first
drains); ``cpu_baseline`` is the CPU path (the reference's compiled Cython kernels + NumPy where
``oracle/_ref`` holds them, else the restatement) on a bounded sample of the same workload.

``--impl reference`` times that CPU path alone, on the host cores, as the reference arm.
``--conv n,h,w,ci,co,k,stride,pad --conv-pass ...`` times one convolution pass through the C ABI (the
fixed small cases of the kernel profiles).

Synthetic data: x ~ N(0,1) float32 (64, 224, 224, 3) per GPU, labels uniform in [0, 1000), seeded;
weights he-uniform from seed 0 (identical replicas).  A step touches several GB of activations, so
inputs are larger than L2 and no flush is needed between steps.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

METRIC = "resnet50_train_images_per_s"
UNIT = "img/s"
PER_GPU_BATCH = 64

# The default workload is the configuration the headline metric is quoted on (ResNet-50 training); the other two
# benchmark configurations that run whole networks are selectable with --workload.
WORKLOADS = {
    "resnet50": dict(metric=METRIC, name="resnet50_imagenet_train", batch=64, layout="NHWC", hw=224, train=True,
                     build="create_resnet50_imagenet", model_kw=dict(enable_fused_bn_relu=True),
                     input="3x224x224 f32 N(0,1)"),
    "vgg16bn": dict(metric="vgg16bn_train_images_per_s", name="vgg16_bn_imagenet_train", batch=32, layout="NHWC", hw=224,
                    train=True, build="create_vgg16bn_imagenet", model_kw=dict(enable_fused_bn_relu=True),
                    input="3x224x224 f32 N(0,1)"),
    "alexnet": dict(metric="alexnet_inference_images_per_s", name="alexnet_imagenet_inference", batch=64, layout="NCHW",
                    hw=227, train=False, build="create_alexnet_imagenet", model_kw=dict(enable_fused_conv_relu=True),
                    input="3x227x227 uint8 uniform /255 -> f32"),
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm_gbs=d["hbm_gbs"], bf16=d["bf16_tflops"], bf16_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index=0):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu_index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------
# CPU path (reference arm and cpu_baseline)
# ---------------------------------------------------------------------------------------------

def _cpu_threads():
    n = os.cpu_count() or 1
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        pass
    return n


CPU_GLUE = ("layer classes of oracle/cpu_model.py (this repository's restatement of the reference's CPU layers) "
            "driving the reference's own compiled Cython kernels (im2row/im2col, pooling, bias add) and NumPy GEMM")


def _cpu_net(workload, batch):
    from oracle import cpu_model as cm
    wl = WORKLOADS[workload]
    spec = {"resnet50": cm.resnet50_spec, "vgg16bn": lambda: cm.vgg16_spec(batch_norm=True), "alexnet": cm.alexnet_spec}[workload]()
    hw = wl["hw"]
    return cm.CpuNet(spec, (hw, hw, 3), batch, np.float32, wl["layout"], seed=0)


def cpu_images_per_s(workload, batch, steps, warmup, budget_s=None):
    """Steps of one of the whole-network workloads on the host cores with the oracle's CPU model (training step, or
    forward only for the inference workload).  Returns (img/s, kind, seconds per step list)."""
    from oracle import conv_oracle as co
    kind = "reference" if co.default_backend() == "ref" else "port"
    wl = WORKLOADS[workload]
    rng = np.random.Generator(np.random.PCG64(0))
    net = _cpu_net(workload, batch)
    hw = wl["hw"]
    if wl["layout"] == "NCHW":
        x = (rng.integers(0, 256, (batch, 3, hw, hw)).astype(np.float32) / 255.0).astype(np.float32)
    else:
        x = rng.standard_normal((batch, hw, hw, 3)).astype(np.float32)
    labels = rng.integers(0, 1000, batch)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        if wl["train"]:
            net.train_step(x, labels, lr=0.01, momentum=0.9, global_batch=batch)
        else:
            net.forward(x, train=False)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
        if budget_s is not None and i >= warmup and sum(times) > budget_s:
            break
    return batch * len(times) / sum(times), kind, times


def cpu_resnet50_images_per_s(batch, steps, warmup, budget_s=None):
    return cpu_images_per_s("resnet50", batch, steps, warmup, budget_s)


def cpu_conv_pass(n, h, w, ci, co, k, stride, pad, pass_name, layout="NHWC", dtype=np.float32, sample_n=None, reps=3):
    """One Conv2D pass on the host cores through the reference's lowering + GEMM path
    (pydtnn/backends/cpu/layers/conv_2d_cpu.py:183-209, 363-397): im2row/im2col by the compiled Cython kernels where
    oracle/_ref holds them, NumPy ``@`` for the GEMM.  Timed on ``sample_n`` images of the batch (the path is a loop
    over images, so TFLOP/s does not depend on the batch).  Returns (TFLOP/s, kind, seconds, sample_n)."""
    from oracle import conv_oracle as cvo
    kind = "reference" if cvo.default_backend() == "ref" else "port"
    if sample_n is None:
        per_image = 2.0 * ((h + 2 * pad - k) // stride + 1) ** 2 * co * ci * k * k
        sample_n = int(max(1, min(n, 2e10 // per_image)))          # about 20 GFLOP of work per repetition
    g = cvo.Geom(sample_n, h, w, ci, co, k, k, pad, pad, stride, stride, 1, 1)
    rng = np.random.Generator(np.random.PCG64(0))
    nhwc = layout == "NHWC"
    x = rng.standard_normal((sample_n, h, w, ci) if nhwc else (sample_n, ci, h, w)).astype(dtype)
    wt = (rng.standard_normal((ci, k, k, co) if nhwc else (co, ci, k, k)) * np.sqrt(2.0 / (ci * k * k))).astype(dtype)
    dy = rng.standard_normal((sample_n, g.ho, g.wo, co) if nhwc else (sample_n, co, g.ho, g.wo)).astype(dtype)
    keep = {}
    cvo.conv2d_forward(x, wt, None, g, layout, keep=keep)
    best = None
    for _ in range(reps):
        t0 = time.perf_counter()
        if pass_name == "fprop":
            cvo.conv2d_forward(x, wt, None, g, layout)
        elif pass_name == "wgrad":
            cvo.conv2d_backward(x, dy, wt, g, layout, need_dx=False, use_bias=False, keep=dict(keep))
        else:
            # the reference computes both gradients in one call; the input gradient alone = whole call - weight gradient
            cvo.conv2d_backward(x, dy, wt, g, layout, need_dx=True, use_bias=False, keep=dict(keep))
        dt = time.perf_counter() - t0
        best = dt if best is None or dt < best else best
    flops = g.flops * (2 if pass_name == "dgrad" else 1)
    return flops / best / 1e12, kind, best, sample_n


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = _cpu_threads()
    wl = WORKLOADS[args.workload]
    batch = 4
    # size the sample so K+W steps end within a few minutes: probe one step at batch 2
    t0 = time.perf_counter()
    cpu_images_per_s(args.workload, 2, 1, 0)
    probe = time.perf_counter() - t0
    if probe * 2 * (args.steps + args.warmup) > 240:
        batch = 2
    if probe * (args.steps + args.warmup) > 240:
        batch = 1
    ips, kind, times = cpu_images_per_s(args.workload, batch, args.steps, args.warmup)
    ms = 1000.0 * sum(times) / len(times)
    what = "train step" if wl["train"] else "forward pass"
    sample = (f"{wl['name']}: {what} at batch {batch} per step (bounded sample of the {wl['batch']}-image step; the path "
              f"loops over images, so img/s is per image), {len(times)} steps; {CPU_GLUE if kind == 'reference' else 'CPU restatement'}")
    line = {
        "impl": "reference", "metric": wl["metric"], "value": ips, "unit": UNIT, "n_gpus": args.gpus, "steps": len(times),
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl["name"], "per_gpu_batch": wl["batch"], "tensor_format": wl["layout"],
                   "device": "host cores", "sample_batch": batch},
        "cpu_baseline": {"value": ips, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": ips, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------

def run_ours(args):
    import torch
    import torch.distributed as dist
    from pydtnn_b200 import _lib, nets
    from pydtnn_b200.comm import init_process_group_from_env
    from pydtnn_b200.model import Model
    from pydtnn_b200.optimizers import SGD

    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    rank, world = init_process_group_from_env()
    dev = torch.device("cuda", local_rank)
    L = _lib.lib()

    wl = WORKLOADS[args.workload]
    batch, hw, train = wl["batch"], wl["hw"], wl["train"]
    dp_rec = None
    if world > 1 and train:
        # correctness of the data-parallel step before anything is timed: P ranks on shards == 1 rank on the whole
        # batch, replicas bitwise identical (a small batch-norm-free network, a few steps; see pydtnn_b200/dp_check.py)
        from pydtnn_b200 import dp_check
        dp_rec = dp_check.run(world, rank)
    np.random.seed(0)                       # identical replicas
    model = Model(batch_size=batch, tensor_format=wl["layout"], dtype=np.float32, comm=True if world > 1 else None,
                  non_blocking_mpi=True, device=dev, **wl["model_kw"])
    getattr(nets, wl["build"])(model)
    opt = SGD(learning_rate=0.01 * world, momentum=0.9)
    model._ensure_loss()

    rng = np.random.Generator(np.random.PCG64(1000 + rank))
    if args.workload == "alexnet":
        xs = (rng.integers(0, 256, (batch, 3, hw, hw)).astype(np.float32) / 255.0).astype(np.float32)
    else:
        xs = rng.standard_normal((batch, hw, hw, 3)).astype(np.float32)
    x_host = torch.from_numpy(xs).pin_memory()
    y_host = torch.from_numpy(rng.integers(0, 1000, batch).astype(np.int32)).pin_memory()
    model._upload(x_host, y_host)
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if train:
        def device_step():
            model.forward_backward()
            model.apply_update(opt)

        def e2e_step():
            # the next step's batch (here the same pinned tensors) is uploaded under this step's kernels
            loss = model.train_batch(x_host, y_host, opt, next_batch=(x_host, y_host))
            return loss.loss()                 # device -> host read of the per-row losses
    else:
        out_host = torch.empty((batch, 1000), dtype=torch.float32).pin_memory()

        def device_step():
            model.evaluate_batch(None)

        def e2e_step():
            y = model.evaluate_batch(x_host, next_batch=x_host)    # the next call's input uploads under this call's kernels
            out_host.copy_(y.ary.t.view(batch, 1000), non_blocking=True)       # device -> host read of the class scores
            torch.cuda.current_stream().synchronize()
            return float(out_host[0, 0])

    def timed(step_fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step_fn()
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        barrier()
        return float(ms.item())

    for _ in range(max(args.warmup, 3)):
        device_step()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = L.b2c_launch_count()
    ms_total = timed(device_step, args.steps)
    launches = L.b2c_launch_count() - launches0
    # The same steps once more with a CUDA event pair around every Conv2D pass (the roofline figures). They are
    # kept out of the loop timed above: an event between two kernels stops the second from starting while the
    # first drains, which the unprofiled step is free to do.
    model.conv_profile = []
    ms_profiled = timed(device_step, args.steps)
    prof, model.conv_profile = model.conv_profile, None
    clocks = sampler.stop() if rank == 0 else None      # sampled over both loops: the same steps, the same load

    for _ in range(max(args.warmup, 3)):
        e2e_step()
    ms_e2e = timed(e2e_step, args.steps)
    final_loss = e2e_step()

    # ---- roofline of the convolution kernels from the per-launch events --------------------------
    torch.cuda.synchronize()
    per_pass = {}
    per_layer = {}
    for name, layer, e0, e1 in prof:
        ms = e0.elapsed_time(e1)
        d = per_pass.setdefault(name, [0.0, 0.0, 0])
        d[0] += ms; d[1] += layer.flops_per_pass; d[2] += 1
        key = (f"{layer.hi}x{layer.wi}x{layer.ci}->{layer.co} k{layer.kh} s{layer.vstride}", name)
        lbytes = 4.0 * model.batch_size * (layer.hi * layer.wi * layer.ci + layer.ho * layer.wo * layer.co) + \
            4.0 * layer.kh * layer.kw * layer.ci * layer.co
        q = per_layer.setdefault(key, [0.0, 0.0, 0, layer.flops_per_pass / lbytes])
        q[0] += ms; q[1] += layer.flops_per_pass; q[2] += 1
    conv_min_bytes = 0.0
    for name, layer, e0, e1 in prof:
        conv_min_bytes += 4.0 * model.batch_size * (layer.hi * layer.wi * layer.ci + layer.ho * layer.wo * layer.co) + \
            4.0 * layer.kh * layer.kw * layer.ci * layer.co
    conv_ms = sum(v[0] for v in per_pass.values())
    conv_flops = sum(v[1] for v in per_pass.values())
    conv_launches = sum(v[2] for v in per_pass.values())
    peaks = measured_peaks()
    peak_3xtf32 = peaks["bf16_sustained"] / 2.0 / 3.0
    achieved = conv_flops / (conv_ms * 1e-3) / 1e12 if conv_ms > 0 else 0.0
    engines = {}
    for layer in model.get_all_layers():
        if type(layer).__name__ in ("Conv2DGPU", "Conv2DReluGPU", "Conv2DBatchNormalizationGPU", "Conv2DBatchNormalizationReluGPU"):
            import ctypes
            for p, pname in enumerate(("fprop", "dgrad", "wgrad")):
                e = L.b2c_conv_engine_for(ctypes.byref(layer.desc), p)
                engines[pname + ("_tensor" if e == _lib.ENGINE_TENSOR else "_fma")] = engines.get(pname + ("_tensor" if e == _lib.ENGINE_TENSOR else "_fma"), 0) + 1
    # DRAM traffic of the convolution launches: every pass is put in a kernel class, and the class's measured /
    # algorithmic ratio (small ncu captures of one layer per class, profiles/traffic.json) is applied to the pass's
    # own algorithmic bytes; the sum over the passes, per launch, is the line's `traffic`.
    traffic, traffic_note = None, None
    tpath = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(tpath) and conv_launches:
        with open(tpath) as f:
            tj = json.load(f)["classes"]

        def klass(layer, name):
            if layer.ci % 32:
                return "stem_wgrad" if name == "wgrad" else "stem_fprop"
            small = layer.hi <= 14
            if name == "wgrad":
                return "wgrad_small" if small else ("wgrad_1x1_large" if layer.kh == 1 else "wgrad_large")
            if name == "dgrad" and layer.vstride > 1 and layer.kh > 1:
                return "strided_dgrad"
            if small:
                return "l2_resident_fprop_dgrad"
            k = layer.ci if name == "fprop" else layer.co
            if layer.kh == 1 and k <= 256 and layer.hi >= 56:
                return "short_k_fprop_with_bn_sums" if name == "fprop" and getattr(layer, "stats_for_bn", None) is not None \
                    else "short_k_fprop_dgrad"
            return "long_fprop_dgrad"
        total, shares = 0.0, {}
        for name, layer, e0, e1 in prof:
            lb = 4.0 * model.batch_size * (layer.hi * layer.wi * layer.ci + layer.ho * layer.wo * layer.co) + \
                4.0 * layer.kh * layer.kw * layer.ci * layer.co
            c = klass(layer, name)
            total += lb * tj[c]["measured_over_algorithmic"]
            shares[c] = shares.get(c, 0.0) + lb
        traffic = total / conv_launches
        traffic_note = {"basis": "per-class measured/algorithmic DRAM ratios of profiles/traffic.json weighted by each class's "
                                 "algorithmic bytes in this step",
                        "share_of_algorithmic_bytes": {c: round(v / conv_min_bytes, 3) for c, v in sorted(shares.items())},
                        "ratios": {c: tj[c]["measured_over_algorithmic"] for c in sorted(shares)},
                        "classes_over_1.2x": [c for c in sorted(shares) if tj[c]["measured_over_algorithmic"] > 1.2]}
    roofline = {
        "bound": "tensor", "achieved": achieved, "peak": peak_3xtf32, "unit": "TFLOP/s",
        "frac": achieved / peak_3xtf32, "traffic": traffic, "traffic_basis": traffic_note,
        "algorithmic_bytes_per_launch_avg": conv_min_bytes / max(conv_launches, 1),
        "kernel": "Conv2D fprop+dgrad+wgrad launches of the step (implicit GEMM)",
        "peak_basis": f"{peaks['source']} bf16 sustained {peaks['bf16_sustained']:.1f} TFLOP/s / 2 (tf32) / 3 (3xTF32)",
        "launches_timed": conv_launches, "avg_launch_ms": conv_ms / max(conv_launches, 1),
        "flops_per_launch_avg": conv_flops / max(conv_launches, 1),
        "share_of_step": conv_ms / ms_profiled if ms_profiled else None,
        "ms_per_step_with_events": ms_profiled / args.steps,
        "per_pass_tflops": {k: v[1] / (v[0] * 1e-3) / 1e12 for k, v in per_pass.items()},
        "engines": engines,
    }

    if rank != 0:
        return
    imgs = batch * world * args.steps
    value = imgs / (ms_total * 1e-3)
    e2e_value = imgs / (ms_e2e * 1e-3)
    line = {
        "metric": wl["metric"], "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl["name"], "per_gpu_batch": batch,
                   "global_batch": batch * world, "tensor_format": wl["layout"], "input": wl["input"],
                   "optimizer": "SGD momentum 0.9" if train else "none (forward only, Conv+ReLU fused)",
                   "parallelism": f"dp{world}",
                   "grad_exchange": "bucketed NCCL all-reduce overlapped with backward" if world > 1 and train else "none",
                   "l2": "per-step activations (several GB) exceed the 126 MB L2; no flush needed"},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": ms_e2e / args.steps,
                "h2d_bytes_per_step": int(x_host.numel() * 4 + (y_host.numel() * 4 if train else 0)) * world,
                # training reads the two doubles (mean loss, accuracy) the loss kernel leaves on the device
                "d2h_bytes_per_step": int(16 if train else batch * 1000 * 4) * world},
        "gpu_launches": int(launches),
        "roofline": roofline,
        "final_loss": final_loss,
    }
    if dp_rec is not None:
        line["dp_check"] = dp_rec
    if world == 1 and not args.no_cpu_baseline:
        threads = _cpu_threads()
        cpu_batch = {"resnet50": 8, "vgg16bn": 2, "alexnet": 16}[args.workload]
        ips, kind, times = cpu_images_per_s(args.workload, cpu_batch, 1, 0)
        what = "train step" if train else "forward pass"
        line["cpu_baseline"] = {"value": ips, "unit": UNIT, "cores": threads, "kind": kind,
                                "sample": f"one {wl['name']} {what} at batch {cpu_batch} ({times[0]:.1f} s), {wl['layout']} f32; "
                                          + (CPU_GLUE if kind == "reference" else "CPU restatement (oracle/)")}
    if not args.no_layers:
        # per-layer convolution table: time, TFLOP/s, and the fraction of the layer's own bound
        # min(3xTF32 sustained peak, arithmetic intensity x measured HBM bandwidth)
        table = {}
        for k, v in sorted(per_layer.items()):
            tf = v[1] / (v[0] * 1e-3) / 1e12
            bound = min(peak_3xtf32, v[3] * peaks["hbm_gbs"] / 1e3)
            table[f"{k[0]} {k[1]}"] = {"ms": round(v[0] / v[2], 5), "tflops": round(tf, 1), "bound_tflops": round(bound, 1),
                                       "frac": round(tf / bound, 3), "bound": "tensor" if bound >= peak_3xtf32 else "hbm"}
        line["per_layer"] = table
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def measure_fma_peak(L, f64):
    """FMA rate the device sustains on register-resident chains (b2c_probe_fma, CUDA events, best of 3), in
    TFLOP/s: the roofline denominator of the FMA engine."""
    import ctypes
    import torch
    from pydtnn_b200 import _lib
    blocks, iters = 148 * 8, 20000
    sink = torch.empty(blocks * 256, dtype=torch.float64 if f64 else torch.float32, device="cuda")
    flops = ctypes.c_double(0.0)
    st = torch.cuda.current_stream().cuda_stream
    dt = _lib.F64 if f64 else _lib.F32
    _lib.check(L.b2c_probe_fma(dt, blocks, iters, sink.data_ptr(), ctypes.byref(flops), st))
    best = None
    for _ in range(3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        _lib.check(L.b2c_probe_fma(dt, blocks, iters, sink.data_ptr(), ctypes.byref(flops), st))
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        best = ms if best is None or ms < best else best
    return flops.value / (best * 1e-3) / 1e12


def run_single_conv(args):
    """One Conv2D pass through the C ABI on device-resident synthetic tensors: the small, fixed case
    used for kernel profiles. Buffers rotate over more than the L2 size between launches."""
    import ctypes
    import torch
    from pydtnn_b200 import _lib
    n, h, w, ci, co, k, stride, pad = [int(v) for v in args.conv.split(",")]
    L = _lib.lib()
    torch.cuda.set_device(0)
    ho, wo = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
    f64, nchw = args.conv_dtype == "f64", args.conv_layout == "NCHW"
    tdt, esz = (torch.float64, 8) if f64 else (torch.float32, 4)
    eng = {"auto": _lib.ENGINE_AUTO, "fma": _lib.ENGINE_FMA, "tensor": _lib.ENGINE_TENSOR}[args.conv_engine]
    desc = _lib.ConvDesc(_lib.LAYOUT_NCHW if nchw else _lib.LAYOUT_NHWC, _lib.F64 if f64 else _lib.F32,
                         _lib.W_KCRS if nchw else _lib.W_KRSC, eng, n, h, w, ci, co, k, k, pad, pad, stride, stride, 1, 1)
    pidx = {"fprop": 0, "dgrad": 1, "wgrad": 2}[args.conv_pass]
    engine = L.b2c_conv_engine_for(ctypes.byref(desc), pidx)
    nb = max(L.b2c_conv_workspace_bytes(ctypes.byref(desc), p) for p in range(3))
    ws = torch.empty(max(int(nb), 256), dtype=torch.uint8, device="cuda")
    bytes_x, bytes_y = n * h * w * ci * esz, n * ho * wo * co * esz
    nbuf = max(2, int(256e6 // max(bytes_x + bytes_y, 1)) + 1)          # rotate through > 2x L2
    gen = torch.Generator(device="cuda").manual_seed(0)
    xshape, yshape = ((n, ci, h, w), (n, co, ho, wo)) if nchw else ((n, h, w, ci), (n, ho, wo, co))
    xs = [torch.randn(xshape, device="cuda", generator=gen, dtype=tdt) for _ in range(nbuf)]
    ys = [torch.randn(yshape, device="cuda", generator=gen, dtype=tdt) for _ in range(nbuf)]
    wt = torch.randn((co, ci, k, k) if nchw else (co, k, k, ci), device="cuda", generator=gen, dtype=tdt) * (2.0 / (ci * k * k)) ** 0.5
    dw = torch.empty_like(wt)
    st = torch.cuda.current_stream().cuda_stream

    stats = None
    if args.conv_bn_stats:
        sb = L.b2c_conv_stats_bytes(ctypes.byref(desc))
        if pidx != 0 or not sb:
            raise SystemExit("--conv-bn-stats needs a forward pass on the float32 NHWC tensor-core path")
        stats = torch.empty(sb, dtype=torch.uint8, device="cuda")

    def call(i):
        x, y = xs[i % nbuf], ys[i % nbuf]
        if pidx == 0 and stats is not None:
            rc = L.b2c_conv_fprop_stats(ctypes.byref(desc), x.data_ptr(), wt.data_ptr(), None, y.data_ptr(), stats.data_ptr(),
                                        stats.numel(), ws.data_ptr(), ws.numel(), st)
        elif pidx == 0:
            rc = L.b2c_conv_fprop(ctypes.byref(desc), x.data_ptr(), wt.data_ptr(), None, None, 0, y.data_ptr(),
                                  ws.data_ptr(), ws.numel(), st)
        elif pidx == 1:
            rc = L.b2c_conv_dgrad(ctypes.byref(desc), y.data_ptr(), wt.data_ptr(), x.data_ptr(), ws.data_ptr(),
                                  ws.numel(), st)
        else:
            rc = L.b2c_conv_wgrad(ctypes.byref(desc), x.data_ptr(), y.data_ptr(), dw.data_ptr(), None, ws.data_ptr(),
                                  ws.numel(), st)
        _lib.check(rc)

    for i in range(max(args.warmup, 3)):
        call(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        call(i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    flops = 2.0 * n * ho * wo * co * ci * k * k
    min_bytes = float(esz) * (n * h * w * ci + k * k * ci * co + n * ho * wo * co)
    peaks = measured_peaks()
    on_tc = engine == _lib.ENGINE_TENSOR
    # tensor-core engine: measured bf16 / 2 / 3.  FMA engine: the FMA rate measured in this run by the register-resident
    # probe kernel (nominal: 148 SMs x 128 lanes x 2 flops x 1.965 GHz = 74.4 TFLOP/s float32, half of that float64).
    fma_peak = None if on_tc else measure_fma_peak(L, f64)
    peak = peaks["bf16"] / 6.0 if on_tc else fma_peak
    tflops = flops / (ms * 1e-3) / 1e12
    cpu = None
    if not args.no_cpu_baseline:
        ctf, kind, secs, sn = cpu_conv_pass(n, h, w, ci, co, k, stride, pad, args.conv_pass, args.conv_layout,
                                            np.float64 if f64 else np.float32)
        cpu = {"value": ctf, "unit": "TFLOP/s", "cores": _cpu_threads(), "kind": kind,
               "sample": f"the same pass on {sn} of the {n} images ({secs:.2f} s, best of 3): reference lowering "
                         f"(Cython im2row/im2col) + NumPy GEMM" + ("" if kind == "reference" else " restated in oracle/")}
    print(json.dumps({
        "metric": "conv_pass_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "dtype": args.conv_dtype, "data": "synthetic",
        "config": {"workload": f"conv2d_{args.conv_pass}" + ("+bn_stats" if stats is not None else ""), "shape": args.conv, "tensor_format": args.conv_layout,
                   "engine": "tensor" if on_tc else "fma", "l2": f"{nbuf} rotating buffer sets"},
        "roofline": {"bound": "tensor" if on_tc else "fma", "achieved": tflops, "peak": peak, "unit": "TFLOP/s", "frac": tflops / peak,
                     "peak_basis": (f"{peaks['source']} bf16 burst {peaks['bf16']:.1f} / 2 / 3 (kernel timed alone)" if on_tc
                                    else "FMA rate measured in this run by the register-resident probe kernel"),
                     "min_bytes": min_bytes, "hbm_gbs_at_min_bytes": min_bytes / (ms * 1e-3) / 1e9,
                     "arithmetic_intensity": flops / min_bytes},
        "cpu_baseline": cpu}), flush=True)


SWEEP_AXES = ((7, 14, 28, 56, 112), (64, 128, 256, 512), (64, 128, 256, 512), (1, 3, 5, 7), (1, 2))


def sweep_points():
    """The shape sweep: batch 32, H=W x Ci x Co x kernel x stride, 'same' padding, dilation 1 (640 geometries)."""
    import itertools
    return [(32, hw, hw, ci, co, k, s, (k - 1) // 2) for hw, ci, co, k, s in itertools.product(*SWEEP_AXES)]


def run_sweep(args):
    """Every geometry of the shape sweep x {float32, float64} x {NHWC, NCHW} x {fprop, dgrad, wgrad} through the
    C ABI on device-resident synthetic tensors.  Each point: 2 warm-up calls, then `--sweep-iters` calls between one
    CUDA-event pair, operands rotating through more than 2x the L2 size (one set when a tensor alone is larger).
    Writes one CSV row per point to `--out` and prints one JSON line with the distribution of the roofline
    fractions.  The bound of a point is min(compute peak, arithmetic intensity x measured HBM bandwidth); the
    compute peak is measured bf16 burst / 2 / 3 for float32 and the nominal FMA figure for float64."""
    import ctypes
    import statistics
    import torch
    from pydtnn_b200 import _lib
    L = _lib.lib()
    torch.cuda.set_device(0)
    peaks = measured_peaks()
    st = torch.cuda.current_stream().cuda_stream
    pts = sweep_points()
    if args.sweep_limit:
        pts = pts[:: max(1, len(pts) // args.sweep_limit)][: args.sweep_limit]
    combos = [(d, l) for d in args.sweep_dtypes.split(",") for l in args.sweep_layouts.split(",")]
    gen = torch.Generator(device="cuda").manual_seed(0)
    rows, launches0 = [], L.b2c_launch_count()
    fma64_peak = None
    for dname, layout in combos:
        f64, nchw = dname == "f64", layout == "NCHW"
        tdt, esz = (torch.float64, 8) if f64 else (torch.float32, 4)
        biggest = max(max(n * h * w * ci, n * ((h + 2 * p - k) // s + 1) ** 2 * co) for n, h, w, ci, co, k, s, p in pts)
        pool_el = max(biggest, int(320e6) // esz)
        # inputs come from two pools that no call writes, results go to a third: values never feed back
        xin = torch.randn(pool_el, device="cuda", generator=gen, dtype=tdt)
        yin = torch.randn(pool_el, device="cuda", generator=gen, dtype=tdt)
        out = torch.empty(pool_el, device="cuda", dtype=tdt)
        if f64 and fma64_peak is None:
            fma64_peak = measure_fma_peak(L, True)
        peak = fma64_peak if f64 else peaks["bf16"] / 6.0
        for n, h, w, ci, co, k, s, p in pts:
            ho = wo = (h + 2 * p - k) // s + 1
            desc = _lib.ConvDesc(_lib.LAYOUT_NCHW if nchw else _lib.LAYOUT_NHWC, _lib.F64 if f64 else _lib.F32,
                                 _lib.W_KCRS if nchw else _lib.W_KRSC, _lib.ENGINE_AUTO, n, h, w, ci, co, k, k, p, p, s, s, 1, 1)
            nb = max(L.b2c_conv_workspace_bytes(ctypes.byref(desc), q) for q in range(3))
            ws = torch.empty(max(int(nb), 256), dtype=torch.uint8, device="cuda")
            xel, yel, wel = n * h * w * ci, n * ho * wo * co, co * k * k * ci
            nbuf = max(1, min(pool_el // max(xel, yel), int(256e6 // ((xel + yel) * esz)) + 1))
            wt = torch.randn(wel, device="cuda", generator=gen, dtype=tdt) * (2.0 / (ci * k * k)) ** 0.5
            dw = torch.empty_like(wt)
            flops = 2.0 * n * ho * wo * co * ci * k * k
            min_bytes = float(esz) * (xel + wel + yel)
            bound = min(peak, flops / min_bytes * peaks["hbm_gbs"] / 1e3)
            for pidx, pname in enumerate(("fprop", "dgrad", "wgrad")):
                engine = L.b2c_conv_engine_for(ctypes.byref(desc), pidx)

                def call(i):
                    j = i % nbuf
                    xa, ya = xin.data_ptr() + j * xel * esz, yin.data_ptr() + j * yel * esz
                    if pidx == 0:
                        rc = L.b2c_conv_fprop(ctypes.byref(desc), xa, wt.data_ptr(), None, None, 0,
                                              out.data_ptr() + j * yel * esz, ws.data_ptr(), ws.numel(), st)
                    elif pidx == 1:
                        rc = L.b2c_conv_dgrad(ctypes.byref(desc), ya, wt.data_ptr(), out.data_ptr() + j * xel * esz,
                                              ws.data_ptr(), ws.numel(), st)
                    else:
                        rc = L.b2c_conv_wgrad(ctypes.byref(desc), xa, ya, dw.data_ptr(), None, ws.data_ptr(), ws.numel(), st)
                    _lib.check(rc)

                for i in range(2):
                    call(i)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for i in range(args.sweep_iters):
                    call(2 + i)
                e1.record()
                e1.synchronize()
                ms = e0.elapsed_time(e1) / args.sweep_iters
                tf = flops / (ms * 1e-3) / 1e12
                rows.append((dname, layout, pname, h, ci, co, k, s, "tensor" if engine == _lib.ENGINE_TENSOR else "fma",
                             ms, tf, flops / min_bytes, bound, tf / bound))
        torch.cuda.synchronize()
        _lib.check(L.b2c_check_device_status(ctypes.byref(ctypes.c_int(0))))
        del xin, yin, out
        torch.cuda.empty_cache()
    if args.out:
        with open(args.out, "w") as f:
            f.write("dtype,layout,pass,hw,ci,co,k,stride,engine,ms,tflops,flop_per_byte,bound_tflops,frac_of_bound\n")
            for r in rows:
                f.write("%s,%s,%s,%d,%d,%d,%d,%d,%s,%.5f,%.3f,%.2f,%.2f,%.4f\n" % r)
    summary = {}
    for dname, layout in combos:
        for pname in ("fprop", "dgrad", "wgrad"):
            sel = [r for r in rows if r[0] == dname and r[1] == layout and r[2] == pname]
            fr = sorted(r[13] for r in sel)
            summary[f"{dname} {layout} {pname}"] = {
                "points": len(sel), "median_tflops": statistics.median(r[10] for r in sel),
                "max_tflops": max(r[10] for r in sel), "median_frac": statistics.median(fr),
                "p10_frac": fr[len(fr) // 10], "min_frac": fr[0], "share_at_or_above_0.6": sum(v >= 0.6 for v in fr) / len(fr),
                "on_tensor_engine": sum(r[8] == "tensor" for r in sel)}
    cpu = None
    if not args.no_cpu_baseline:
        # the reference's CPU path on a stated subset: 16 evenly spaced geometries, float32 NHWC, three passes each,
        # about 2 GFLOP of work per pass (a few images of the batch)
        sub = sweep_points()[20::40][:16]
        crow, t0 = [], time.perf_counter()
        for n, h, w, ci, co, k, sstr, p in sub:
            per_image = 2.0 * ((h + 2 * p - k) // sstr + 1) ** 2 * co * ci * k * k
            sn = int(max(1, min(n, 2e9 // per_image)))
            for pname in ("fprop", "dgrad", "wgrad"):
                ctf, kind, _, _ = cpu_conv_pass(n, h, w, ci, co, k, sstr, p, pname, "NHWC", np.float32, sample_n=sn, reps=1)
                gpu = [r for r in rows if r[0] == "f32" and r[1] == "NHWC" and r[2] == pname and r[3:8] == (h, ci, co, k, sstr)]
                crow.append((pname, h, ci, co, k, sstr, ctf, gpu[0][10] if gpu else None))
        cpu = {"value": statistics.median(r[6] for r in crow), "unit": "TFLOP/s (median over the subset)", "cores": _cpu_threads(),
               "kind": kind, "sample": f"{len(sub)} geometries x 3 passes, float32 NHWC, a few images each ({time.perf_counter() - t0:.0f} s)",
               "points": [{"pass": r[0], "hw": r[1], "ci": r[2], "co": r[3], "k": r[4], "stride": r[5], "cpu_tflops": round(r[6], 4),
                           "gpu_tflops": None if r[7] is None else round(r[7], 1)} for r in crow]}
    print(json.dumps({
        "cpu_baseline": cpu,
        "metric": "conv_sweep_roofline_frac", "unit": "fraction of min(compute peak, intensity x HBM)", "n_gpus": 1,
        "data": "synthetic", "higher_is_better": True, "points": len(rows), "iters_per_point": args.sweep_iters,
        "gpu_launches": L.b2c_launch_count() - launches0,
        "peaks": {"f32_tflops": peaks["bf16"] / 6.0, "f64_tflops": fma64_peak, "f64_basis": "measured FMA probe", "hbm_gbs": peaks["hbm_gbs"], "source": peaks["source"]},
        "config": {"workload": "conv2d shape sweep, batch 32", "l2": "operands rotate through > 2x L2"},
        "summary": summary}), flush=True)


def run_single_fc(args):
    """One fully connected layer (batch, in, out) through the C ABI on device-resident synthetic tensors: forward,
    weight + bias gradient, input gradient, each timed alone with operands rotating through more than 2x L2."""
    import ctypes
    import torch
    from pydtnn_b200 import _lib
    b, fin, fout = [int(v) for v in args.fc.split(",")]
    L = _lib.lib()
    torch.cuda.set_device(0)
    f64 = args.conv_dtype == "f64"
    tdt, esz, dt = (torch.float64, 8, _lib.F64) if f64 else (torch.float32, 4, _lib.F32)
    eng = {"auto": _lib.ENGINE_AUTO, "fma": _lib.ENGINE_FMA, "tensor": _lib.ENGINE_TENSOR}[args.conv_engine]
    ws = torch.empty(max(int(L.b2c_fc_workspace_bytes(dt, b, fin, fout, eng)), 256), dtype=torch.uint8, device="cuda")
    nbuf = max(2, int(256e6 // (fin * fout * esz)) + 1)
    gen = torch.Generator(device="cuda").manual_seed(0)
    ws_ = [torch.randn(fin, fout, device="cuda", generator=gen, dtype=tdt) * (1.0 / fin) ** 0.5 for _ in range(nbuf)]
    dws = [torch.empty_like(w) for w in ws_]
    x = torch.randn(b, fin, device="cuda", generator=gen, dtype=tdt)
    dy = torch.randn(b, fout, device="cuda", generator=gen, dtype=tdt)
    bias = torch.randn(fout, device="cuda", generator=gen, dtype=tdt)
    y, dx, db = torch.empty_like(dy), torch.empty_like(x), torch.empty_like(bias)
    st = torch.cuda.current_stream().cuda_stream

    def fwd(i):
        _lib.check(L.b2c_fc_forward(dt, eng, b, fin, fout, x.data_ptr(), ws_[i % nbuf].data_ptr(), bias.data_ptr(), y.data_ptr(),
                                    ws.data_ptr(), ws.numel(), st))

    def wgrad(i):
        _lib.check(L.b2c_fc_backward(dt, eng, b, fin, fout, x.data_ptr(), dy.data_ptr(), ws_[i % nbuf].data_ptr(),
                                     dws[i % nbuf].data_ptr(), db.data_ptr(), None, ws.data_ptr(), ws.numel(), st))

    def dgrad(i):
        _lib.check(L.b2c_fc_backward(dt, eng, b, fin, fout, x.data_ptr(), dy.data_ptr(), ws_[i % nbuf].data_ptr(), None, None,
                                     dx.data_ptr(), ws.data_ptr(), ws.numel(), st))

    res = {}
    for name, fn in (("forward", fwd), ("wgrad", wgrad), ("dgrad", dgrad)):
        for i in range(max(args.warmup, 3)):
            fn(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.steps):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        res[name] = e0.elapsed_time(e1) / args.steps
    peaks = measured_peaks()
    flops, wbytes = 2.0 * b * fin * fout, float(esz) * fin * fout
    print(json.dumps({
        "metric": "fc_pass_ms", "unit": "ms", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
        "higher_is_better": False, "dtype": args.conv_dtype, "data": "synthetic",
        "config": {"workload": "fc layer", "shape": args.fc, "l2": f"{nbuf} rotating weight matrices"},
        "passes": {k: {"ms": v, "tflops": flops / (v * 1e-3) / 1e12, "weight_gbs": wbytes / (v * 1e-3) / 1e9,
                       "frac_of_hbm": wbytes / (v * 1e-3) / 1e9 / peaks["hbm_gbs"]} for k, v in res.items()},
        "roofline_note": "each pass reads or writes the weight matrix once: bound = weight bytes / measured HBM bandwidth"}), flush=True)


def run_single_bn(args):
    """Training-mode batch norm (+ fused ReLU) forward and backward on one (n, h, w, c) float32 NHWC tensor through
    the C ABI, tensors rotating through more than 2x L2: the small, fixed case for profiles of the HBM-bound kernels.
    Algorithmic bytes: forward reads x twice and writes y (3 passes), backward reads x and dy twice and writes dx
    (5 passes); the second read of each pair can come from L2 when the tensor fits."""
    import torch
    from pydtnn_b200 import _lib
    n, h, w, c = [int(v) for v in args.bn.split(",")]
    L = _lib.lib()
    torch.cuda.set_device(0)
    numel = n * h * w * c
    nbuf = max(2, int(256e6 // (numel * 4)) + 1)
    gen = torch.Generator(device="cuda").manual_seed(0)
    xs = [torch.randn(n, h, w, c, device="cuda", generator=gen) for _ in range(nbuf)]
    dys = [torch.randn(n, h, w, c, device="cuda", generator=gen) for _ in range(nbuf)]
    ys = [torch.empty_like(x) for x in xs]
    gamma, beta = torch.randn(c, device="cuda", generator=gen), torch.randn(c, device="cuda", generator=gen)
    rm, rv = torch.zeros(c, device="cuda"), torch.ones(c, device="cuda")
    mean, inv_std, dg, db = (torch.empty(c, device="cuda") for _ in range(4))
    scratch = torch.empty(1200 * c, dtype=torch.float64, device="cuda")
    st = torch.cuda.current_stream().cuda_stream

    def fwd(i):
        _lib.check(L.b2c_bn_train_forward(_lib.F32, _lib.LAYOUT_NHWC, n, c, h * w, xs[i % nbuf].data_ptr(), gamma.data_ptr(),
                                          beta.data_ptr(), rm.data_ptr(), rv.data_ptr(), 0.9, 1e-5, 1, ys[i % nbuf].data_ptr(),
                                          mean.data_ptr(), inv_std.data_ptr(), scratch.data_ptr(), scratch.numel() * 8, st))

    def bwd(i):
        _lib.check(L.b2c_bn_train_backward(_lib.F32, _lib.LAYOUT_NHWC, n, c, h * w, xs[i % nbuf].data_ptr(), dys[i % nbuf].data_ptr(),
                                           None, beta.data_ptr(), gamma.data_ptr(), mean.data_ptr(), inv_std.data_ptr(),
                                           dg.data_ptr(), db.data_ptr(), ys[i % nbuf].data_ptr(), scratch.data_ptr(),
                                           scratch.numel() * 8, st))

    res = {}
    for name, fn, passes in (("forward", fwd, 3), ("backward", bwd, 5)):
        for i in range(max(args.warmup, 3)):
            fn(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.steps):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        res[name] = {"ms": ms, "passes": passes, "gbs": passes * numel * 4 / (ms * 1e-3) / 1e9}
    peaks = measured_peaks()
    for v in res.values():
        v["frac_of_hbm"] = v["gbs"] / peaks["hbm_gbs"]
    print(json.dumps({"metric": "bn_train_gbs", "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3),
                      "higher_is_better": True, "dtype": "f32", "data": "synthetic",
                      "config": {"workload": "batch norm + ReLU, training", "shape": args.bn, "l2": f"{nbuf} rotating tensor sets"},
                      "passes": res, "roofline": {"bound": "hbm", "peak": peaks["hbm_gbs"], "unit": "GB/s", "source": peaks["source"]}}),
          flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="resnet50",
                    help="whole-network configuration to time (default: the one the headline metric is quoted on)")
    ap.add_argument("--layers", action="store_true", help="(default now) per-layer convolution timings are in the JSON line")
    ap.add_argument("--no-layers", action="store_true", help="leave the per-layer convolution table out of the JSON line")
    ap.add_argument("--conv", default=None, help="n,h,w,ci,co,k,stride,pad: time one Conv2D pass instead of the model")
    ap.add_argument("--fc", default=None, help="batch,in,out: time one fully connected layer instead of the model")
    ap.add_argument("--bn", default=None, help="n,h,w,c: time training-mode batch norm + ReLU forward and backward on one tensor")
    ap.add_argument("--conv-pass", default="fprop", choices=["fprop", "dgrad", "wgrad"])
    ap.add_argument("--conv-dtype", default="f32", choices=["f32", "f64"])
    ap.add_argument("--conv-layout", default="NHWC", choices=["NHWC", "NCHW"])
    ap.add_argument("--conv-engine", default="auto", choices=["auto", "fma", "tensor"])
    ap.add_argument("--conv-bn-stats", action="store_true",
                    help="with --conv (forward pass): also take the per-channel batch sums of the output (b2c_conv_fprop_stats)")
    ap.add_argument("--sweep", action="store_true", help="time the whole Conv2D shape sweep instead of the model")
    ap.add_argument("--sweep-dtypes", default="f32,f64")
    ap.add_argument("--sweep-layouts", default="NHWC,NCHW")
    ap.add_argument("--sweep-iters", type=int, default=3)
    ap.add_argument("--sweep-limit", type=int, default=0, help="time only about this many evenly spaced geometries")
    ap.add_argument("--out", default=None, help="CSV file for the per-point rows of --sweep")
    args = ap.parse_args()
    if args.sweep:
        run_sweep(args)
        return
    if args.fc:
        run_single_fc(args)
        return
    if args.bn:
        run_single_bn(args)
        return
    if args.conv:
        run_single_conv(args)
        return
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)
        if int(os.environ.get("WORLD_SIZE", "1")) > 1:
            import torch.distributed as dist
            if dist.is_initialized():
                dist.destroy_process_group()


if __name__ == "__main__":
    main()
