#!/usr/bin/env python
"""Benchmark of the AET-CNN training hot path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N=1): the CIFAR-shaped small CNN of aet-cnn_b200/cfg/cifar_small.cfg, batch 128 per GPU,
FP32 storage, TF32 tensor-core math, SGD lr 0.1 / momentum 0.9 / decay 5e-4, synthetic seeded inputs
(uniform [0,1) images, uniform labels) standing in for CIFAR-10.  One "step" = forward + backward +
gradient all-reduce (N>1) + update of one batch.  Prints ONE JSON line (rank 0).

  value     images/s over all ranks, inputs resident in HBM, CUDA-graph replay, device-timed
  e2e       the same metric through aet_network_train_step with HOST buffers: pinned staging,
            host->device copies and the loss read-back inside the timed region
  roofline  dominant kernel of the step, timed with CUDA events around each launch in a separate
            instrumented pass (graph replay off), against the measured peaks
  cpu_baseline  the CPU oracle (reference flags, 1 thread) on a bounded sample, rank 0, N=1 only

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
CLASSES = 10
CFG = "cifar_small.cfg"


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


# Dense TF32 peak of this pool's B200, measured with a one-off cuBLAS TF32 8192^3 matmul probe
# (692.3 TFLOP/s best of 10, 624.4 over a 40-launch loop); the driver-written MEASURED_PEAKS.json
# records HBM and BF16 only.
TF32_PEAK_TFLOPS = 692.3
# dram__bytes_read.sum + dram__bytes_write.sum per launch from the committed ncu capture of the same
# workload (profiles/), keyed by kernel label; null when the dominant kernel has no capture yet.
NCU_TRAFFIC_BYTES = {   # "kernel label#layer index" of the small CNN at batch 128
    "conv_fprop_thin#0": 2.17e6, "conv_wgrad_thin#0": 35.68e6,
    "conv_fprop_tma_rows#2": 8.75e6, "conv_dgrad_tma_rows#2": 17.11e6, "conv_wgrad_tma_rows#2": 25.19e6,
    "conv_fprop_tma_rows#4": 5.44e6, "conv_dgrad_tma_rows#4": 9.60e6, "conv_wgrad_tma_rows#4": 12.61e6,
    "bn_act_maxpool_fwd#0": 33.58e6, "bn_bwd_reduce_poolwin#0": 50.37e6, "bn_bwd_apply_poolwin#0": 53.28e6,
    "bn_bwd_reduce_poolwin#2": 25.18e6, "bn_bwd_apply_poolwin#2": 25.18e6, "bn_bwd_apply_poolwin#4": 12.60e6,
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"], source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


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
                                          "--format=csv,noheader,nounits", "-lms", "50"], stdout=subprocess.PIPE,
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
        time.sleep(0.15)
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


def init_weights(aet, synth, cfgfile, net, specs, cin):
    for i, s in enumerate(specs):
        if s["type"] != cfgfile.CONV:
            continue
        k, size = s["filters"], s["size"]
        w = synth.normal((k, cin, size, size), SEED, 1000 + i, 0.0, float(np.sqrt(2.0 / (size * size * cin))))
        net.layer(i).write(aet.P_WEIGHTS, w)
        cin = k


def oracle_net(variant, specs, opts, batch, threads, synth, cfgfile):
    from oracle import binding as ob
    ob.build("fast" if variant == "fast" else "parity")
    o = ob.Oracle(variant)
    net = o.net(specs, batch, opts["c"], opts["h"], opts["w"], mode=ob.MODE_CPU, threads=threads)
    cin = opts["c"]
    for i, s in enumerate(specs):
        if s["type"] != cfgfile.CONV:
            continue
        k, size = s["filters"], s["size"]
        net.set_param(i, ob.P_WEIGHTS, synth.normal((k, cin, size, size), SEED, 1000 + i, 0.0,
                                                    float(np.sqrt(2.0 / (size * size * cin)))))
        cin = k
    return net


def cpu_baseline(specs, opts, synth, cfgfile, budget_s=12.0):
    """Single-thread oracle (the reference's CPU path is effectively one thread) on a batch-16 sample."""
    sample = 16
    net = oracle_net("fast", specs, opts, sample, 1, synth, cfgfile)
    x = synth.uniform((sample, opts["c"], opts["h"], opts["w"]), SEED, 0)
    _, truth = synth.labels(sample, CLASSES, SEED, 1)
    net.train_step(x, truth, opts["learning_rate"], opts["momentum"], opts["decay"])
    t0, steps = time.perf_counter(), 0
    while steps < 8 and (steps == 0 or time.perf_counter() - t0 < budget_s):
        net.train_step(x, truth, opts["learning_rate"], opts["momentum"], opts["decay"])
        steps += 1
    dt = time.perf_counter() - t0
    return dict(value=sample * steps / dt, unit="images/s", cores=1, kind="port",
                sample="%d full train steps (fwd+bwd+update) of the same network at batch %d, reference flags "
                       "-O3 -ffast-math -march=native, 1 thread" % (steps, sample))


def run_reference(args, rank):
    if rank != 0:
        return
    pkg = load_package()
    import aet_cnn_b200.cfgfile as cfgfile
    import aet_cnn_b200.synth as synth
    text = open(os.path.join(pkg.CFG_DIR, CFG)).read()
    threads = os.cpu_count() or 1
    # choose the per-step sample so that warmup+steps stay within ~2.5 minutes
    probe_b = 16
    opts, specs = cfgfile.network_spec(text, probe_b)
    net = oracle_net("fast", specs, opts, probe_b, min(threads, probe_b), synth, cfgfile)
    x = synth.uniform((probe_b, 3, 32, 32), SEED, 0)
    _, truth = synth.labels(probe_b, CLASSES, SEED, 1)
    t0 = time.perf_counter()
    net.train_step(x, truth, opts["learning_rate"], opts["momentum"], opts["decay"])
    per_img = (time.perf_counter() - t0) / probe_b
    total = args.steps + args.warmup
    batch = 128
    while batch > 16 and per_img * batch * total > 150.0:
        batch //= 2
    del net
    opts, specs = cfgfile.network_spec(text, batch)
    use_threads = min(threads, batch)
    net = oracle_net("fast", specs, opts, batch, use_threads, synth, cfgfile)
    batches = [(synth.uniform((batch, 3, 32, 32), SEED, 2 * s), synth.labels(batch, CLASSES, SEED, 2 * s + 1)[1]) for s in range(2)]
    for s in range(args.warmup):
        net.train_step(*batches[s % 2], opts["learning_rate"], opts["momentum"], opts["decay"])
    t0 = time.perf_counter()
    for s in range(args.steps):
        net.train_step(*batches[s % 2], opts["learning_rate"], opts["momentum"], opts["decay"])
    dt = time.perf_counter() - t0
    value = batch * args.steps / dt
    sample = ("each step = one full train step of the same network on %d images (of the 128-image batch), "
              "CPU restatement of the reference's path, conv loops batch-parallel on %d threads" % (batch, use_threads))
    line = {"impl": "reference", "metric": "train images/sec", "value": value, "unit": "images/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * dt / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "small CNN (cifar_small.cfg) full training step, batch 128 per GPU", "sample_batch": batch},
            "cpu_baseline": {"value": value, "unit": "images/s", "cores": use_threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=128, help="per-GPU batch")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3

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

    aet = load_package()
    import aet_cnn_b200.cfgfile as cfgfile
    import aet_cnn_b200.synth as synth
    text = open(os.path.join(aet.CFG_DIR, CFG)).read()
    opts, specs = cfgfile.network_spec(text, args.batch)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    ctx = aet.Context(local_rank, parity=aet.PARITY_MTCS, math=aet.MATH_TF32, stream=stream.cuda_stream)
    net = aet.NNetwork(ctx, cfg_text=text, train=1, batch=args.batch)
    init_weights(aet, synth, cfgfile, net, specs, opts["c"])
    import aet_cnn_b200.parallel as par
    if world > 1:
        net.comm_init(par.exchange_unique_id(aet.comm_unique_id), rank, world)
        if world <= 8 and os.environ.get("AET_PEER_EXCHANGE"):
            # opt-in: gradients summed through peer-mapped buffers inside the update kernel instead of by NCCL
            # (measured at 8 GPUs: 0.301 ms per step against 0.294 with NCCL alone, so NCCL stays the default)
            net.comm_exchange_attach(par.all_gather_bytes(net.comm_exchange_export()))

    batch = args.batch
    host_batches, pinned_keep = [], []

    def pin(a):
        """Page-locked copy of a host array (the library copies by DMA straight from such buffers)."""
        t = torch.from_numpy(np.ascontiguousarray(a, np.float32)).pin_memory()
        pinned_keep.append(t)
        return t.numpy()

    for s in range(4):
        tid = par.shard_tensor_id(s, rank, world)
        host_batches.append((pin(synth.uniform((batch, 3, 32, 32), SEED, 2 * tid)), pin(synth.labels(batch, CLASSES, SEED, 2 * tid + 1)[1])))

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    max_over_ranks = par.max_over_ranks

    # ---- device-resident throughput (graph replay)
    net.input.write(host_batches[0][0]); net.truth.write(host_batches[0][1])
    net.use_graph(True)
    sampler = ClockSampler(local_rank)
    sampler.start()          # polls from here on; its start-up cost stays outside the timed region
    for _ in range(args.warmup):
        net.train_device(want_loss=False)
    ctx.check()
    barrier()
    sampler.mark()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        net.train_device(want_loss=False)
    e1.record(stream)
    barrier()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    clocks = sampler.stop()
    final_loss = net.last_loss()
    weights_identical = par.hashes_identical(net.param_hash())
    launches = net.launches_per_step() * args.steps
    ctx.check()
    value = batch * world * args.steps / (ms_total / 1000.0)

    # ---- end to end through the public call with host buffers
    for s in range(3):
        net.train(*host_batches[s % 4])
    barrier()
    e0.record(stream)
    for s in range(args.steps):
        net.train(*host_batches[s % 4])
    e1.record(stream)
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1))
    e2e_value = batch * world * args.steps / (e2e_ms / 1000.0)
    h2d = (batch * 3 * 32 * 32 + batch * CLASSES) * 4
    d2h = 8

    # ---- per-kernel pass for the roofline (eager launches, events around each)
    # The weight-gradient kernels stay on the main stream here, so that no kernel's time includes a
    # concurrent neighbour's.  The dominant kernel is the largest one that does algorithmic work (the
    # finalize launches move a few KB; their event-bracketed time is mostly the bracket).
    prof_steps = min(args.steps, 20)
    net.use_graph(False)
    os.environ["AET_NO_OVERLAP"] = "1"
    try:
        net.train_device(want_loss=False)
        net.profile(True)
        for _ in range(prof_steps):
            net.train_device(want_loss=False)
        table = net.profile_read()
        net.profile(False)
    finally:
        os.environ.pop("AET_NO_OVERLAP", None)
    peaks = measured_peaks()
    table.sort(key=lambda r: -r["total_ms"])
    total_kernel_ms = sum(r["total_ms"] for r in table) or 1.0
    working = [r for r in table if r["algo_flops"] > 0 or r["algo_bytes"] > 0]
    top = working[0] if working else table[0]
    avg_s = top["total_ms"] / top["launches"] / 1000.0
    if top["algo_flops"] > 0:
        roof = dict(bound="tensor", achieved=top["algo_flops"] / avg_s / 1e12, peak=TF32_PEAK_TFLOPS, unit="TFLOP/s",
                    peak_source="measured cuBLAS TF32 8192^3 burst on this pool (bf16 burst in MEASURED_PEAKS.json: %.0f)"
                                % peaks["bf16_tflops"])
    else:
        roof = dict(bound="hbm", achieved=top["algo_bytes"] / avg_s / 1e9, peak=peaks["hbm_gbs"], unit="GB/s",
                    peak_source=peaks["source"] + " copy bandwidth")
    roof.update(frac=roof["achieved"] / roof["peak"], traffic=NCU_TRAFFIC_BYTES.get(top["name"]), kernel=top["name"],
                share_of_step=top["total_ms"] / total_kernel_ms, avg_us=avg_s * 1e6)
    kernels = [dict(name=r["name"], launches=r["launches"], avg_us=1000.0 * r["total_ms"] / r["launches"],
                    share=r["total_ms"] / total_kernel_ms,
                    gbs=(r["algo_bytes"] / (r["total_ms"] / r["launches"] / 1000.0) / 1e9) if r["algo_bytes"] else None,
                    tflops=(r["algo_flops"] / (r["total_ms"] / r["launches"] / 1000.0) / 1e12) if r["algo_flops"] else None)
               for r in table[:12]]

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline(specs, opts, synth, cfgfile)

    if rank == 0:
        line = {"metric": "train images/sec", "value": value, "unit": "images/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "tf32 (fp32 storage and accumulation)", "data": "synthetic",
                "config": {"workload": "small CNN (cifar_small.cfg: 3x[conv3x3+BN+leaky, maxpool2/2], conv1x1->10, avgpool, "
                                       "softmax-CE) full training step, SGD lr 0.1 momentum 0.9 decay 5e-4",
                           "batch_per_gpu": batch, "global_batch": batch * world,
                           "parallelism": "dp%d" % world if world > 1 else "single",
                           "l2": "per-step working set (activations + deltas, ~250 MB) exceeds the 126 MB L2; no explicit flush",
                           "execution": "CUDA graph replay of forward+backward+allreduce+update"},
                "e2e": {"value": e2e_value, "unit": "images/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "ms_per_step": e2e_ms / args.steps},
                "gpu_launches": launches, "clocks": clocks, "roofline": roof, "cpu_baseline": cpu,
                "final_loss": final_loss, "weights_identical_across_ranks": weights_identical, "kernels": kernels}
        print(json.dumps(line), flush=True)
    net.close()
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
