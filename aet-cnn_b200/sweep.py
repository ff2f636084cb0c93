"""Times the three convolution passes (forward, backward-data, backward-weight) of single layers
through the C ABI with CUDA events and prints one JSON line per shape: time, TFLOP/s, and the
kernels that ran.  Default shapes: the benchmark's kernel sweep at batch 256
(C,H,W,K,size,stride,pad) = (3,32,32,64,3,1,1) (64,16,16,128,3,1,1) (128,8,8,256,3,1,1)
(256,8,8,256,3,1,1) (256,4,4,10,1,1,0), weights N(0,0.05), inputs uniform [0,1).

  python aet-cnn_b200/sweep.py [--batch 256] [--iters 100] [--warmup 20]
"""
import argparse
import importlib.util
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
SHAPES = [(3, 32, 32, 64, 3, 1, 1), (64, 16, 16, 128, 3, 1, 1), (128, 8, 8, 256, 3, 1, 1), (256, 8, 8, 256, 3, 1, 1),
          (256, 4, 4, 10, 1, 1, 0)]


def load():
    if "aet_cnn_b200" in sys.modules:
        return sys.modules["aet_cnn_b200"]
    spec = importlib.util.spec_from_file_location("aet_cnn_b200", os.path.join(HERE, "__init__.py"),
                                                  submodule_search_locations=[HERE])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["aet_cnn_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=20)
    args = ap.parse_args()
    import torch
    aet = load()
    import aet_cnn_b200.synth as synth
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    ctx = aet.Context(0, stream=stream.cuda_stream)
    N = args.batch
    for (C, H, W, K, size, stride, pad) in SHAPES:
        oh, ow = (H + 2 * pad - size) // stride + 1, (W + 2 * pad - size) // stride + 1
        layer = aet.ConvolutionalLayer(ctx, N, H, W, C, K, size, stride, stride, pad, aet.LINEAR, 0, 1)
        layer.write(aet.P_WEIGHTS, synth.normal((K, C, size, size), 3, 1, 0.0, 0.05))
        xin, dx = aet.Tensor(ctx, N, C, H, W), aet.Tensor(ctx, N, C, H, W)
        xin.write(synth.uniform((N, C, H, W), 3, 2))
        layer.write(aet.P_DELTA, synth.normal((N, K, oh, ow), 3, 3))
        st = aet.make_state(input=xin, delta=dx, train=1)
        flops = 2.0 * N * K * C * size * size * oh * ow
        for _ in range(args.warmup):
            layer.forward(st); layer.backward(st)
        ctx.profile(1)
        for _ in range(args.iters):
            layer.forward(st); layer.backward(st)
        table = ctx.profile_read()
        ctx.profile(0)
        res = {"shape": dict(N=N, C=C, H=H, W=W, K=K, size=size, stride=stride, pad=pad), "gflop_per_pass": flops / 1e9}
        for r in table:
            if r["algo_flops"] > 0:
                us = 1000.0 * r["total_ms"] / r["launches"]
                res[r["name"]] = dict(us=round(us, 2), tflops=round(flops / us / 1e6, 1))
        print(json.dumps(res), flush=True)
        layer.close(); xin.close(); dx.close()
    ctx.close()


if __name__ == "__main__":
    main()
