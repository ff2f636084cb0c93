"""Helpers shared by the GPU parity tests: run one layer through the C ABI and through the oracle."""
import os
from concurrent.futures import ThreadPoolExecutor

import numpy as np

from oracle import binding as ob

TOL_TF32 = 1e-2      # relative L2, TF32 inputs with FP32 accumulation
TOL_3X = 1e-5        # relative L2, 3xTF32 split


def _chunks(n, parts):
    step = max(1, (n + parts - 1) // parts)
    return [(i, min(n, i + step)) for i in range(0, n, step)]


def oracle_conv_forward_mt(oracle, x, w, stride, pad):
    """The oracle's per-image convolution loop run over slices of the batch on host threads (images are
    independent in the forward pass, so the result is the single-thread one bit for bit)."""
    parts = _chunks(x.shape[0], os.cpu_count() or 1)
    with ThreadPoolExecutor(len(parts)) as ex:
        ys = list(ex.map(lambda r: oracle.conv_forward(x[r[0]:r[1]], w, stride, stride, pad), parts))
    return np.concatenate(ys, 0)


def oracle_conv_backward_mt(oracle, x, w, d, stride, pad, need_dx=True):
    """Backward over slices of the batch on host threads: dX is per image (exact); dW is the sum of the
    slices' weight gradients in slice order (FP32 grouping differs from the one-thread loop by rounding only)."""
    parts = _chunks(x.shape[0], os.cpu_count() or 1)
    with ThreadPoolExecutor(len(parts)) as ex:
        rs = list(ex.map(lambda r: oracle.conv_backward(x[r[0]:r[1]], w, d[r[0]:r[1]], stride, stride, pad, need_dx=need_dx), parts))
    dw = rs[0][0].astype(np.float64)
    for r in rs[1:]:
        dw += r[0]
    return dw.astype(np.float32), (np.concatenate([r[1] for r in rs], 0) if need_dx else None)


def conv_case(aet, ctx, oracle, N, C, H, W, K, size, stride, pad, act, seed, bias=True, want_dx=True, threads=False, groups=1,
              dilation=1):
    """Forward + backward of one convolution (no BN) on the GPU and in the oracle; returns both result dicts.
    threads=True runs the oracle's per-image loops over batch slices on all host cores (full-size cases).
    `stride` may be a pair (stride_x, stride_y) (dnn/ConvolutionalLayer.c:703-715)."""
    import aet_cnn_b200.synth as synth
    sx, sy = stride if isinstance(stride, tuple) else (stride, stride)
    oh, ow = (H + 2 * pad - size) // sy + 1, (W + 2 * pad - size) // sx + 1
    x = synth.uniform((N, C, H, W), seed, 1)
    w = synth.normal((K, C // groups, size, size), seed, 2, 0.0, float(np.sqrt(2.0 / (size * size * C // groups))))
    b = synth.normal((K,), seed, 3, 0.0, 0.1) if bias else np.zeros(K, np.float32)
    dy = synth.normal((N, K, oh, ow), seed, 4)

    layer = aet.ConvolutionalLayer(ctx, N, H, W, C, K, size, sx, sy, pad, act, 0, 1, groups=groups, dilation=dilation)
    layer.write(aet.P_WEIGHTS, w)
    layer.write(aet.P_BIASES, b)
    xin = aet.Tensor(ctx, N, C, H, W)
    xin.write(x)
    dxt = aet.Tensor(ctx, N, C, H, W) if want_dx else None
    st = aet.make_state(input=xin, delta=dxt, train=1)
    layer.forward(st)
    got = dict(y=layer.read(aet.P_OUTPUT).reshape(N, K, oh, ow))
    layer.write(aet.P_DELTA, dy)
    layer.backward(st)
    ctx.check()
    got["dw"] = layer.read(aet.P_WEIGHT_UPDATES).reshape(w.shape)
    got["db"] = layer.read(aet.P_BIAS_UPDATES)
    got["dx"] = dxt.read() if want_dx else None
    layer.close(); xin.close()
    if dxt is not None:
        dxt.close()

    mode = ob.MODE_MTCS
    if threads:
        conv = oracle_conv_forward_mt(oracle, x, w, stride, pad)
    else:
        conv = oracle.conv_forward(x, w, sx, sy, pad, groups=groups, dilation=dilation)
    y = oracle.activate(oracle.add_bias(conv, b), act, mode)
    # The activation gradient is a step function of the layer's stored output.  Backward parity is
    # taken on identical inputs, so the mask comes from the output the device stored: a TF32-rounded
    # value next to a kink may sit on the other side of it, which changes that element's gradient
    # tenfold and says nothing about the backward kernels.
    d = oracle.gradient(got["y"], act, dy)
    if threads:
        dw, dx = oracle_conv_backward_mt(oracle, x, w, d, stride, pad, need_dx=want_dx)
    else:
        dw, dx = oracle.conv_backward(x, w, d, sx, sy, pad, need_dx=want_dx, groups=groups, dilation=dilation)
    ref = dict(y=y, dw=dw, dx=dx, db=oracle.backward_bias(d))
    return got, ref


def kernels_used(ctx):
    """Kernel labels of the profiled launches without their ".variant" suffix."""
    return {r["name"].split(".")[0] for r in ctx.profile_read()}


def variants_used(ctx):
    """Full labels ("kernel.variant") of the profiled launches: which code path each launcher picked."""
    return {r["name"] for r in ctx.profile_read()}
