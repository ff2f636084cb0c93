#!/usr/bin/env python
"""Benchmark of the AET-CNN training hot path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload small_cnn|alexnet|sweep]

Workload (default, N=1): the CIFAR-shaped small CNN of aet-cnn_b200/cfg/cifar_small.cfg, batch 128 per GPU,
FP32 storage, TF32 tensor-core math, SGD lr 0.1 / momentum 0.9 / decay 5e-4, synthetic seeded inputs
(uniform [0,1) images, uniform labels) standing in for CIFAR-10.  One "step" = forward + backward +
gradient all-reduce (N>1) + update of one batch.  Prints ONE JSON line (rank 0).

  value     images/s over all ranks, inputs resident in HBM, CUDA-graph replay, device-timed: the loop of
            --steps steps is timed `repeats` times (barrier + synchronize on both sides of each, max over
            ranks) and the median repeat is reported
  e2e       the same metric through the public pipelined call (aet_network_train_step_async) with HOST
            buffers: every step's host->device copy from page-locked memory and the read-back of a step's
            loss are inside the timed region (the copy of step s+1 overlaps step s on a copy stream)
  roofline  dominant kernel of the step, timed with CUDA events around each launch in a separate
            instrumented pass (graph replay off), against peaks measured in this run / by the driver
  cpu_baseline  the CPU oracle (reference flags, 1 thread) on a bounded sample, rank 0, N=1 only; the same
            leg checks the device's first-step loss against the oracle's at the full batch

--workload alexnet: the AlexNet-style network (227x227x3, 1000 classes, batch 128) in the same form.
--workload sweep: the reference's per-shape convolution list at batch 256, each pass timed alone.
--impl reference times the CPU restatement of the reference's own path (the reference cannot be
built here) on all host threads, on the same network and batch.
"""
import argparse
import importlib.util
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
SEED = 20241
WORKLOADS = {
    "small_cnn": dict(cfg="cifar_small.cfg", classes=10, batch=128,
                      text="small CNN (cifar_small.cfg: 3x[conv3x3+BN+leaky, maxpool2/2], conv1x1->10, avgpool, softmax-CE) "
                           "full training step, SGD lr 0.1 momentum 0.9 decay 5e-4"),
    "alexnet": dict(cfg="alexnet_style.cfg", classes=1000, batch=128,
                    text="AlexNet-style network (alexnet_style.cfg: conv11x11/4, conv5x5, 3x conv3x3, 3 maxpool3/2, FC4096 x2 "
                         "with dropout, FC1000, softmax-CE; 227x227x3) full training step"),
}
SWEEP_SHAPES = [(3, 32, 32, 64, 3, 1, 1), (64, 16, 16, 128, 3, 1, 1), (128, 8, 8, 256, 3, 1, 1), (256, 8, 8, 256, 3, 1, 1),
                (256, 4, 4, 10, 1, 1, 0)]


def load_package():
    if "aet_cnn_b200" in sys.modules:
        return sys.modules["aet_cnn_b200"]
    pkg_dir = os.path.join(ROOT, "aet-cnn_b200")
    spec = importlib.util.spec_from_file_location("aet_cnn_b200", os.path.join(pkg_dir, "__init__.py"),
                                                  submodule_search_locations=[pkg_dir])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["aet_cnn_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


# dram__bytes_read.sum + dram__bytes_write.sum per launch from the committed ncu captures of the same workload
# (profiles/), keyed by the kernel's full label "kernel.variant#layer" of the small CNN at batch 128.  A kernel
# whose code path changed since its capture has another label and reports null.
NCU_TRAFFIC_BYTES = {}
_traffic_file = os.path.join(ROOT, "profiles", "dram_traffic_small_cnn_batch128.json")
if os.path.exists(_traffic_file):
    with open(_traffic_file) as _f:
        NCU_TRAFFIC_BYTES = json.load(_f)["bytes_per_launch"]


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"], source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


def measure_tf32_peak(torch):
    """Dense TF32 peak of this GPU: a cuBLAS TF32 8192^3 matmul through torch, used only as a peak probe and
    outside every timed region.  Returns (best of 10 single launches, 40 launches back to back) in TFLOP/s."""
    n = 8192
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        a = torch.randn(n, n, device="cuda", dtype=torch.float32)
        b = torch.randn(n, n, device="cuda", dtype=torch.float32)
        c = torch.empty(n, n, device="cuda", dtype=torch.float32)
        for _ in range(3):
            torch.matmul(a, b, out=c)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        best = 1e30
        for _ in range(10):
            e0.record()
            torch.matmul(a, b, out=c)
            e1.record()
            e1.synchronize()
            best = min(best, e0.elapsed_time(e1))
        e0.record()
        for _ in range(40):
            torch.matmul(a, b, out=c)
        e1.record()
        e1.synchronize()
        loop = e0.elapsed_time(e1) / 40.0
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    del a, b, c
    torch.cuda.empty_cache()
    flops = 2.0 * n ** 3
    return flops / (best * 1e-3) / 1e12, flops / (loop * 1e-3) / 1e12


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc, self.first = index, [], None, 0

    def start(self):
        """Starts the poller and waits for its first sample: nvidia-smi's start-up (NVML initialisation over
        every GPU of the box) must not fall into the timed region, where it stalls kernel launches."""
        if os.environ.get("BENCH_NO_CLOCK_SAMPLER"):
            return
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "20"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            t0 = time.time()
            while not self.rows and time.time() - t0 < 15.0 and self.proc.poll() is None:
                time.sleep(0.02)
        except OSError:
            self.proc = None

    def mark(self):
        """Samples taken from now on (and the one just before) count: call when the timed region starts."""
        self.first = max(0, len(self.rows) - 1)

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([v.strip() for v in line.split(",")])

    def stop(self):
        if not self.proc:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.1)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows[self.first:]:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except ValueError:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


def conv_layers(aet, net, cin):
    """(layer index, filters, input channels, filter size) of every convolution, read back through the C ABI."""
    out = []
    for i in range(net.layer_count):
        layer = net.layer(i)
        if layer.kind == aet.CONVOLUTIONAL:
            k = layer.out_shape[0]
            size = int(round((layer.param_count(aet.P_WEIGHTS) / (k * cin)) ** 0.5))
            out.append((i, k, cin, size))
        cin = layer.out_shape[0]
    return out


def init_weights(aet, synth, net, cin):
    """He-normal weights N(0, sqrt(2 / (size^2 * C))) from the shared seeded generator, keyed by layer index."""
    convs = conv_layers(aet, net, cin)
    for i, k, c, size in convs:
        net.layer(i).write(aet.P_WEIGHTS, synth.normal((k, c, size, size), SEED, 1000 + i, 0.0, float(np.sqrt(2.0 / (size * size * c)))))
    return convs


def oracle_net(variant, text, batch, threads, synth, mtcs=False):
    """CPU oracle of the same network with the same initial weights (CPU-baseline and reference legs only).
    The timed legs run the reference's CPU formulation; the first-step check runs its GPU formulation (`mtcs`),
    which is the one the device library follows by default."""
    from oracle import binding as ob
    from oracle import cfgfile
    ob.build("fast" if variant == "fast" else "parity")
    opts, specs = cfgfile.network_spec(text, batch)
    net = ob.Oracle(variant).net(specs, batch, opts["c"], opts["h"], opts["w"], mode=ob.MODE_MTCS if mtcs else ob.MODE_CPU,
                                 threads=threads)
    cin = opts["c"]
    for i, s in enumerate(specs):
        if s["type"] == cfgfile.CONV:
            k, size = s["filters"], s["size"]
            net.set_param(i, ob.P_WEIGHTS, synth.normal((k, cin, size, size), SEED, 1000 + i, 0.0,
                                                        float(np.sqrt(2.0 / (size * size * cin)))))
            cin = k
        elif s["type"] == cfgfile.DROPOUT:
            # the timed baseline needs some mask: fixed uniforms (the reference draws rand() per element, dnn/DropoutLayer.c:55-70)
            n = net.param(i, ob.P_RAND)
            if n is not None:
                net.set_param(i, ob.P_RAND, synth.uniform((n.size,), SEED, 5000 + i))
    return net, opts


def cpu_baseline(wl, text, synth, gpu_first_loss, budget_s=12.0):
    """Single-thread oracle (the reference's CPU path is effectively one thread) on a bounded sample, plus the
    checker: the oracle's first-step loss on the device's own first batch at the full batch size."""
    sample = 16 if wl["classes"] == 10 else 2
    net, opts = oracle_net("fast", text, sample, 1, synth)
    shape = (sample, opts["c"], opts["h"], opts["w"])
    x = synth.uniform(shape, SEED, 0)
    _, truth = synth.labels(sample, wl["classes"], SEED, 1)
    net.train_step(x, truth, opts["learning_rate"], opts["momentum"], opts["decay"])
    t0, steps = time.perf_counter(), 0
    while steps < 8 and (steps == 0 or time.perf_counter() - t0 < budget_s):
        net.train_step(x, truth, opts["learning_rate"], opts["momentum"], opts["decay"])
        steps += 1
    dt = time.perf_counter() - t0
    out = dict(value=sample * steps / dt, unit="images/s", cores=1, kind="port",
               sample="%d full train steps (fwd+bwd+update) of the same network at batch %d, reference flags "
                      "-O3 -ffast-math -march=native, 1 thread" % (steps, sample))
    if gpu_first_loss is not None and wl["classes"] == 10:
        batch = wl["batch"]
        full, opts = oracle_net("fast", text, batch, os.cpu_count() or 1, synth, mtcs=True)
        x = synth.uniform((batch, opts["c"], opts["h"], opts["w"]), SEED, 0)
        _, truth = synth.labels(batch, wl["classes"], SEED, 1)
        ref = full.train_step(x, truth, opts["learning_rate"], opts["momentum"], opts["decay"])
        out["first_step_loss"] = dict(device=gpu_first_loss, oracle=ref, rel_diff=abs(gpu_first_loss - ref) / abs(ref))
    return out


def run_reference(args, rank):
    if rank != 0:
        return
    pkg = load_package()
    import aet_cnn_b200.synth as synth
    wl = WORKLOADS[args.workload if args.workload in WORKLOADS else "small_cnn"]
    text = open(os.path.join(pkg.CFG_DIR, wl["cfg"])).read()
    threads = os.cpu_count() or 1
    # choose the per-step sample so that warmup+steps stay within ~2.5 minutes
    probe_b = 16 if wl["classes"] == 10 else 2
    net, opts = oracle_net("fast", text, probe_b, min(threads, probe_b), synth)
    shape = (opts["c"], opts["h"], opts["w"])
    x = synth.uniform((probe_b,) + shape, SEED, 0)
    _, truth = synth.labels(probe_b, wl["classes"], SEED, 1)
    t0 = time.perf_counter()
    net.train_step(x, truth, opts["learning_rate"], opts["momentum"], opts["decay"])
    per_img = (time.perf_counter() - t0) / probe_b
    total = args.steps + args.warmup
    batch = wl["batch"]
    while batch > probe_b and per_img * batch * total > 150.0:
        batch //= 2
    del net
    use_threads = min(threads, batch)
    net, opts = oracle_net("fast", text, batch, use_threads, synth)
    batches = [(synth.uniform((batch,) + shape, SEED, 2 * s), synth.labels(batch, wl["classes"], SEED, 2 * s + 1)[1]) for s in range(2)]
    for s in range(args.warmup):
        net.train_step(*batches[s % 2], opts["learning_rate"], opts["momentum"], opts["decay"])
    t0 = time.perf_counter()
    for s in range(args.steps):
        net.train_step(*batches[s % 2], opts["learning_rate"], opts["momentum"], opts["decay"])
    dt = time.perf_counter() - t0
    value = batch * args.steps / dt
    sample = ("each step = one full train step of the same network on %d images (of the %d-image batch), "
              "CPU restatement of the reference's path, conv loops batch-parallel on %d threads" % (batch, wl["batch"], use_threads))
    line = {"impl": "reference", "metric": "train images/sec", "value": value, "unit": "images/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * dt / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(wl, wl["batch"], max(1, args.gpus)), "sample_batch": batch,
            "cpu_baseline": {"value": value, "unit": "images/s", "cores": use_threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def workload_config(wl, batch, world):
    """The `config` object of the JSON line, the same for both arms: it names the workload, nothing about how an arm ran it."""
    return {"workload": wl["text"], "batch_per_gpu": batch, "global_batch": batch * world,
            "parallelism": "dp%d" % world if world > 1 else "single",
            "l2": "per-step working set (activations + deltas, ~250 MB at batch 128) exceeds the 126 MB L2; no explicit flush"}


def roofline_of(table, peaks, tf32_burst, tf32_loop):
    """The dominant working kernel of the instrumented pass against the peak that bounds it."""
    table = sorted(table, key=lambda r: -r["total_ms"])
    total_kernel_ms = sum(r["total_ms"] for r in table) or 1.0
    working = [r for r in table if r["algo_flops"] > 0 or r["algo_bytes"] > 0]
    top = working[0] if working else table[0]
    avg_s = top["total_ms"] / top["launches"] / 1000.0
    if top["algo_flops"] > 0:
        roof = dict(bound="tensor", achieved=top["algo_flops"] / avg_s / 1e12, peak=tf32_burst, unit="TFLOP/s",
                    peak_source="measured in this run: cuBLAS TF32 8192^3 matmul, best of 10 launches (a kernel timed alone)",
                    peak_loop40=tf32_loop, algo_per_launch=top["algo_flops"])
        roof["frac_vs_bf16_half"] = roof["achieved"] / (peaks["bf16_tflops"] / 2.0)
    else:
        roof = dict(bound="hbm", achieved=top["algo_bytes"] / avg_s / 1e9, peak=peaks["hbm_gbs"], unit="GB/s",
                    peak_source=peaks["source"] + " copy bandwidth (MEASURED_PEAKS.json)", algo_per_launch=top["algo_bytes"])
    roof.update(frac=roof["achieved"] / roof["peak"], traffic=NCU_TRAFFIC_BYTES.get(top["name"]), kernel=top["name"],
                share_of_step=top["total_ms"] / total_kernel_ms, avg_us=avg_s * 1e6)
    if top.get("span_ms", 0) > 0 and top["algo_flops"] > 0:
        # the same launches on the device's own clock: last CTA exit - first CTA entry, without the launch latency and
        # the event bracket that `avg_us` (and `achieved`, `frac`) include
        span_s = top["span_ms"] / top["launches"] / 1000.0
        roof["device_span_us"] = span_s * 1e6
        roof["frac_device_span"] = top["algo_flops"] / span_s / 1e12 / roof["peak"]
    kernels = [dict(name=r["name"], launches=r["launches"], avg_us=1000.0 * r["total_ms"] / r["launches"],
                    span_us=(1000.0 * r["span_ms"] / r["launches"]) if r.get("span_ms", 0) > 0 else None,
                    share=r["total_ms"] / total_kernel_ms,
                    gbs=(r["algo_bytes"] / (r["total_ms"] / r["launches"] / 1000.0) / 1e9) if r["algo_bytes"] else None,
                    tflops=(r["algo_flops"] / (r["total_ms"] / r["launches"] / 1000.0) / 1e12) if r["algo_flops"] else None)
               for r in table[:14]]
    conv = [r for r in table if r["algo_flops"] > 0 and r["name"].startswith("conv_")]
    conv_ms = sum(r["total_ms"] / r["launches"] for r in conv)
    conv_flops = sum(r["algo_flops"] for r in conv)
    conv_all = dict(tflops=conv_flops / (conv_ms * 1e-3) / 1e12 if conv_ms else None, us_per_step=1000.0 * conv_ms,
                    gflop_per_step=conv_flops / 1e9, frac=(conv_flops / (conv_ms * 1e-3) / 1e12 / tf32_burst) if conv_ms else None)
    return roof, kernels, conv_all


def run_sweep(args, aet, ctx, tf32_burst, tf32_loop):
    """Per-shape timing of the three convolution passes at batch 256 (the reference's kernel list)."""
    import aet_cnn_b200.synth as synth
    N = args.batch if args.batch_given else 256
    shapes = []
    for (C, H, W, K, size, stride, pad) in SWEEP_SHAPES:
        oh, ow = (H + 2 * pad - size) // stride + 1, (W + 2 * pad - size) // stride + 1
        layer = aet.ConvolutionalLayer(ctx, N, H, W, C, K, size, stride, stride, pad, aet.LINEAR, 0, 1)
        layer.write(aet.P_WEIGHTS, synth.normal((K, C, size, size), 3, 1, 0.0, 0.05))
        xin, dx = aet.Tensor(ctx, N, C, H, W), aet.Tensor(ctx, N, C, H, W)
        xin.write(synth.uniform((N, C, H, W), 3, 2))
        layer.write(aet.P_DELTA, synth.normal((N, K, oh, ow), 3, 3))
        st = aet.make_state(input=xin, delta=dx, train=1)
        flops = 2.0 * N * K * C * size * size * oh * ow
        for _ in range(max(args.warmup, 20)):
            layer.forward(st); layer.backward(st)
        ctx.profile(1)
        for _ in range(max(args.steps, 100)):
            layer.forward(st); layer.backward(st)
        table = ctx.profile_read()
        ctx.profile(0)
        res = {"shape": dict(N=N, C=C, H=H, W=W, K=K, size=size, stride=stride, pad=pad), "gflop_per_pass": flops / 1e9, "passes": {}}
        for r in table:
            if r["algo_flops"] > 0:
                us = 1000.0 * r["total_ms"] / r["launches"]
                res["passes"][r["name"]] = dict(us=round(us, 2), tflops=round(flops / us / 1e6, 1), frac=round(flops / us / 1e6 / tf32_burst, 3))
        shapes.append(res)
        layer.close(); xin.close(); dx.close()
    best = max((p["tflops"], name) for s in shapes for name, p in s["passes"].items())
    line = {"metric": "conv TFLOP/s per pass", "value": best[0], "unit": "TFLOP/s", "n_gpus": 1, "steps": max(args.steps, 100),
            "warmup": max(args.warmup, 20), "ms_per_step": None, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "tf32 (fp32 storage and accumulation)", "data": "synthetic",
            "config": {"workload": "convolution sweep, batch %d: fprop + dgrad + wgrad of each shape timed alone with CUDA events "
                                   "around every launch; value = the fastest pass (%s)" % (N, best[1])},
            "roofline": {"bound": "tensor", "peak": tf32_burst, "peak_loop40": tf32_loop, "unit": "TFLOP/s",
                         "peak_source": "measured in this run: cuBLAS TF32 8192^3 matmul, best of 10 launches"},
            "shapes": shapes}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="small_cnn", choices=["small_cnn", "alexnet", "sweep"])
    ap.add_argument("--batch", type=int, default=0, help="per-GPU batch (default: the workload's)")
    ap.add_argument("--repeats", type=int, default=0, help="timed repeats of the --steps loop (default 31, 5 for alexnet)")
    ap.add_argument("--verify-steps", type=int, default=200, help="N>1: steps of the per-step cross-rank weight hash check")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    args.batch_given = args.batch > 0

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local_rank))

    tf32_burst, tf32_loop = measure_tf32_peak(torch)
    aet = load_package()
    import aet_cnn_b200.synth as synth
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    ctx = aet.Context(local_rank, parity=aet.PARITY_MTCS, math=aet.MATH_TF32, stream=stream.cuda_stream)
    if args.workload == "sweep":
        if rank == 0:
            run_sweep(args, aet, ctx, tf32_burst, tf32_loop)
        ctx.close()
        return
    wl = WORKLOADS[args.workload]
    batch = args.batch if args.batch_given else wl["batch"]
    classes = wl["classes"]
    repeats = args.repeats or (31 if args.workload == "small_cnn" else 5)
    text = open(os.path.join(aet.CFG_DIR, wl["cfg"])).read()
    net = aet.NNetwork(ctx, cfg_text=text, train=1, batch=batch)
    _, cin, ih, iw = net.input_shape
    init_weights(aet, synth, net, cin)
    import aet_cnn_b200.parallel as par
    if world > 1:
        net.comm_init(par.exchange_unique_id(aet.comm_unique_id), rank, world)
        exchange = "nccl"
        if world <= 8 and not os.environ.get("AET_NO_PEER_EXCHANGE"):
            # One box, at most 8 ranks: the gradients are summed through peer-mapped buffers inside the update kernel
            # (a gradient arena of up to 4 MB whole, otherwise its last bucket) instead of by the last collective; at 8
            # GPUs this step is 12 us shorter than with NCCL alone.  Every rank must take the same path, so the ranks
            # agree on whether the attach worked everywhere and fall back to NCCL together if it did not.
            ok = 1
            try:
                net.comm_exchange_attach(par.all_gather_bytes(net.comm_exchange_export()))
            except aet.AetError as e:
                ok = 0
                sys.stderr.write("rank %d: peer exchange not attached (%s)\n" % (rank, e))
            flag = torch.tensor([ok], dtype=torch.int32, device="cuda")
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if int(flag.item()) == 1:
                exchange = "peer"
                # a rank still loading its kernels in the first eager step must not look like a dead peer to the others:
                # the benchmark waits up to 10 s for a peer's slice (the library's default of 1 s suits a training loop
                # that wants to notice a lost rank quickly)
                ctx.set_wait_limit(10_000_000_000)
            else:
                net.comm_exchange_detach()

    host_batches, pinned_keep = [], []

    def pin(a):
        """Page-locked copy of a host array (the library copies by DMA straight from such buffers)."""
        t = torch.from_numpy(np.ascontiguousarray(a, np.float32)).pin_memory()
        pinned_keep.append(t)
        return t.numpy()

    for s in range(4):
        tid = par.shard_tensor_id(s, rank, world)
        host_batches.append((pin(synth.uniform((batch, cin, ih, iw), SEED, 2 * tid)), pin(synth.labels(batch, classes, SEED, 2 * tid + 1)[1])))

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    max_over_ranks = par.max_over_ranks
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(step_fn, after_fn=None):
        """`repeats` timings of the loop of --steps steps, each bracketed by barrier + synchronize; max over ranks."""
        out = []
        for _ in range(repeats):
            barrier()
            e0.record(stream)
            for s in range(args.steps):
                step_fn(s)
            if after_fn:
                after_fn()
            e1.record(stream)
            barrier()
            out.append(max_over_ranks(e0.elapsed_time(e1)))
        return out

    # ---- device-resident throughput (graph replay)
    net.input.write(host_batches[0][0]); net.truth.write(host_batches[0][1])
    net.use_graph(True)
    first_loss = net.train_device(want_loss=True)     # step 1 on synthetic tensor 0: checked against the oracle below
    sampler = ClockSampler(local_rank)
    sampler.start()          # polls from here on; its start-up cost stays outside the timed region
    for _ in range(args.warmup):
        net.train_device(want_loss=False)
    ctx.check()
    barrier()
    sampler.mark()
    times = timed(lambda s: net.train_device(want_loss=False))
    clocks = sampler.stop()
    ms_total = statistics.median(times)
    final_loss = net.last_loss()
    weights_identical = par.hashes_identical(net.param_hash())
    launches = net.launches_per_step() * args.steps
    ctx.check()
    value = batch * world * args.steps / (ms_total / 1000.0)

    # ---- end to end through the public pipelined call with host buffers
    for s in range(max(3, args.warmup // 4)):
        net.train_async(*host_batches[s % 4])
    net.last_loss()
    e2e_times = timed(lambda s: net.train_async(*host_batches[s % 4]), after_fn=net.last_loss)
    e2e_ms = statistics.median(e2e_times)
    e2e_value = batch * world * args.steps / (e2e_ms / 1000.0)
    h2d = (batch * cin * ih * iw + batch * classes) * 4
    d2h = 12               # cost, mean loss and the status word of every step
    weights_identical = weights_identical and par.hashes_identical(net.param_hash())

    # ---- N > 1: weights must stay bitwise identical across ranks after EVERY step
    hash_steps_checked = 0
    if world > 1:
        hashes = []
        for s in range(args.verify_steps):
            net.train_device(want_loss=False)
            hashes.append(net.param_hash())
        t = torch.tensor([[h & 0xFFFFFFFF, (h >> 32) & 0xFFFFFFFF] for h in hashes], dtype=torch.int64, device="cuda")
        parts = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(parts, t)
        weights_identical = weights_identical and all(bool(torch.equal(p, parts[0])) for p in parts)
        hash_steps_checked = len(hashes)

    # ---- N > 1: how long the main stream waits for the gradient collectives (device clock around the wait, graph replay)
    comm = None
    if world > 1:
        ctx.set_option("comm_stamps", 1)
        net.use_graph(False); net.use_graph(True)       # the stamps are part of the captured step
        for _ in range(4):
            net.train_device(want_loss=False)
        net.comm_exposed()                              # reset after the eager + capture steps
        barrier()
        for _ in range(min(args.steps, 100)):
            net.train_device(want_loss=False)
        exposed_us, counted = net.comm_exposed()
        ctx.set_option("comm_stamps", 0)
        net.use_graph(False); net.use_graph(True)
        comm = {"exposed_us_per_step": max_over_ranks(exposed_us), "steps": counted, "gradient_exchange": exchange,
                "method": "two one-thread kernels read %globaltimer before and after the main stream's waits for the "
                          "all-reduces and for the peers' gradient slices; mean over the steps, max over ranks"}

    # ---- per-kernel pass for the roofline (eager launches, events around each)
    # The weight-gradient kernels stay on the main stream here, so that no kernel's time includes a
    # concurrent neighbour's.  The dominant kernel is the largest one that does algorithmic work.
    prof_steps = min(args.steps, 20)
    net.use_graph(False)
    ctx.set_option("overlap_wgrad", 0)
    try:
        net.train_device(want_loss=False)
        net.profile(True)
        for _ in range(prof_steps):
            net.train_device(want_loss=False)
        table = net.profile_read()
        net.profile(False)
    finally:
        ctx.set_option("overlap_wgrad", 1)
    peaks = measured_peaks()
    roof, kernels, conv_all = roofline_of(table, peaks, tf32_burst, tf32_loop)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline(wl, text, synth, first_loss if batch == wl["batch"] else None)

    failed = []
    if not weights_identical:
        failed.append("weights differ between ranks")
    if cpu and "first_step_loss" in cpu and cpu["first_step_loss"]["rel_diff"] > 1e-2:
        failed.append("first-step loss differs from the oracle's by more than 1e-2")
    if rank == 0:
        line = {"metric": "train images/sec", "value": value, "unit": "images/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "tf32 (fp32 storage and accumulation)", "data": "synthetic",
                "config": workload_config(wl, batch, world),
                "method": {"execution": "CUDA graph replay of forward+backward+allreduce+update",
                           "timing": "median of %d repeats of the %d-step loop, each bracketed by barrier+synchronize, max over ranks"
                                     % (repeats, args.steps)},
                "repeats": repeats, "ms_per_step_min": min(times) / args.steps, "ms_per_step_max": max(times) / args.steps,
                "e2e": {"value": e2e_value, "unit": "images/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "ms_per_step": e2e_ms / args.steps,
                        "call": "aet_network_train_step_async: host->device copy of step s+1 on a copy stream during step s, "
                                "loss of step s read back during step s+1"},
                "gpu_launches": launches, "clocks": clocks, "roofline": roof, "conv_layers": conv_all, "cpu_baseline": cpu,
                "comm": comm, "final_loss": final_loss, "weights_identical_across_ranks": weights_identical,
                "hash_checked_every_step_for": hash_steps_checked, "kernels": kernels}
        if failed:
            line["failed"] = failed
        print(json.dumps(line), flush=True)
    net.close()
    ctx.close()
    if world > 1:
        dist.destroy_process_group()
    if failed:
        raise SystemExit("bench.py: " + "; ".join(failed))


if __name__ == "__main__":
    main()
