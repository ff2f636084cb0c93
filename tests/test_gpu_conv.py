"""GPU parity of the implicit-GEMM convolution kernels against the CPU oracle, through the C ABI.
Tolerances: TF32 <= 1e-2, 3xTF32 <= 1e-5 (relative L2 per tensor)."""
import os

import numpy as np
import pytest

from conftest import rel_l2
from gpu_util import TOL_3X, TOL_TF32, conv_case, kernels_used, variants_used

pytestmark = pytest.mark.gpu

# (N, C, H, W, K, size, stride, pad, activation)
GATHER_SHAPES = [
    (2, 3, 8, 8, 5, 3, 1, 1, 2),          # tiny, ragged everything
    (4, 3, 32, 32, 32, 3, 1, 1, 2),       # single conv layer of the reference's CPU-runnable case, small batch
    (3, 4, 9, 7, 6, 3, 2, 1, 1),          # stride 2, odd sizes
    (2, 2, 11, 11, 3, 5, 2, 2, 0),        # 5x5 stride 2
    (2, 3, 35, 35, 16, 11, 4, 0, 1),      # AlexNet-style first layer, reduced
    (5, 20, 6, 6, 40, 6, 1, 0, 1),        # "FC as convolution": filter covers the whole map
    (7, 40, 1, 1, 24, 1, 1, 0, 0),        # 1x1 on a 1x1 map (FC after FC)
    (16, 256, 4, 4, 10, 1, 1, 0, 0),      # classifier conv of the small CNN
    (2, 12, 13, 13, 300, 3, 1, 1, 1),     # more filters than one N tile
]
TMA_SHAPES = [
    (2, 32, 32, 32, 32, 3, 1, 1, 2),
    (4, 64, 16, 16, 128, 3, 1, 1, 2),     # conv2 of the small CNN
    (8, 128, 8, 8, 256, 3, 1, 1, 2),      # conv3 of the small CNN
    (6, 256, 8, 8, 256, 3, 1, 1, 0),      # 256 -> 256 sweep shape, batch not a multiple of the tile
    (32, 64, 4, 4, 64, 1, 1, 0, 1),       # 1x1, eight images per 128-pixel tile
    (2, 32, 64, 64, 64, 3, 1, 1, 0),      # image rows wider than a K slab
    (16, 256, 4, 4, 10, 1, 1, 0, 0),      # classifier conv: fewer filters than one 32-channel row
    (8, 64, 8, 8, 20, 3, 1, 1, 1),        # 20 filters, 3x3
]


def check(got, ref, tol):
    for k in ("y", "dw", "db", "dx"):
        if ref[k] is None:
            continue
        assert got[k].shape == ref[k].shape or got[k].size == ref[k].size, k
        err = rel_l2(got[k].ravel(), ref[k].ravel())
        assert err <= tol, "%s: relative L2 error %.3e > %.1e" % (k, err, tol)
        assert np.isfinite(got[k]).all(), k


@pytest.fixture(scope="module")
def ctx_gather(aet):
    c = aet.Context(0)
    c.set_option("gather_only", 1)
    yield c
    c.close()


@pytest.mark.parametrize("shape", GATHER_SHAPES)
def test_conv_gather_tf32(aet, ctx_gather, oracle, shape):
    ctx_gather.set_math(aet.MATH_TF32)
    got, ref = conv_case(aet, ctx_gather, oracle, *shape, seed=100 + shape[1])
    check(got, ref, TOL_TF32)


@pytest.mark.parametrize("shape", GATHER_SHAPES[:4] + TMA_SHAPES[:2])
def test_conv_gather_3xtf32(aet, ctx_gather, oracle64, shape):
    ctx_gather.set_math(aet.MATH_3XTF32)
    try:
        got, ref = conv_case(aet, ctx_gather, oracle64, *shape, seed=200 + shape[1])
    finally:
        ctx_gather.set_math(aet.MATH_TF32)
    check(got, ref, TOL_3X)


@pytest.mark.parametrize("shape", TMA_SHAPES)
def test_conv_gather_on_tma_shapes(aet, ctx_gather, oracle, shape):
    got, ref = conv_case(aet, ctx_gather, oracle, *shape, seed=300 + shape[1])
    check(got, ref, TOL_TF32)


@pytest.mark.parametrize("shape", TMA_SHAPES)
def test_conv_tma_tf32(aet, ctx, oracle, shape):
    ctx.set_math(aet.MATH_TF32)
    ctx.profile(1)
    try:
        got, ref = conv_case(aet, ctx, oracle, *shape, seed=300 + shape[1])
        used = kernels_used(ctx)
    finally:
        ctx.profile(0)
    assert ({"conv_fprop_tma", "conv_fprop_tma_rows"} & used) and ({"conv_dgrad_tma", "conv_dgrad_tma_rows"} & used) and \
        ({"conv_wgrad_tma", "conv_wgrad_tma_rows"} & used), used
    check(got, ref, TOL_TF32)


# few input channels: the whole K extent fits one stage of the persistent first-layer kernels
THIN_SHAPES = [
    (2, 3, 8, 8, 5, 3, 1, 1, 2),          # one ragged tile
    (4, 3, 32, 32, 32, 3, 1, 1, 2),       # first layer of the reference's CPU-runnable case
    (128, 3, 32, 32, 64, 3, 1, 1, 0),     # first layer of the benchmark network, full batch: several tiles per CTA
    (3, 4, 9, 7, 6, 3, 2, 1, 1),          # stride 2, odd sizes
    (2, 2, 11, 11, 3, 5, 2, 2, 0),        # 5x5 stride 2: K = 100
    (3, 1, 28, 28, 20, 5, 1, 0, 1),       # one input channel, no padding
    (5, 8, 6, 6, 100, 2, 1, 0, 1),        # two cells per tap, 100 filters
]


@pytest.mark.parametrize("shape", THIN_SHAPES)
def test_conv_thin_tf32(aet, ctx, oracle, shape):
    ctx.set_math(aet.MATH_TF32)
    ctx.profile(1)
    try:
        got, ref = conv_case(aet, ctx, oracle, *shape, seed=400 + shape[1])
        used = kernels_used(ctx)
    finally:
        ctx.profile(0)
    assert "conv_fprop_thin" in used, used
    kp = (shape[4] + 3) // 4 * 4
    if kp % 32 == 0 or kp < 32:
        assert "conv_wgrad_thin" in used, used
    check(got, ref, TOL_TF32)


# The benchmark network's second and third convolution at the benchmark's batch (128 images per GPU): above
# ~111 images the row-sharing launcher switches to other code paths than at small batches (two pixel tiles per
# CTA with a second epilogue warp group, column taps merged into the MMA's N for the narrow data gradient, K
# split over a two-CTA cluster, two filter tiles), so these shapes are checked at that size and the path each
# launch took is asserted by its label.  N = 112 is the smallest batch above the two-tile threshold.
BENCH_SHAPES = [
    # shape, {kernel: variant} expected on a 148-SM part
    ((128, 64, 16, 16, 128, 3, 1, 1, 2), {"conv_fprop_tma_rows": "mt2e_n128x1", "conv_dgrad_tma_rows": "sm_mt2_n192x1",
                                          "conv_wgrad_tma_rows": "n64_sp49"}),
    ((128, 128, 8, 8, 256, 3, 1, 1, 2), {"conv_fprop_tma_rows": "mt1_n128x2", "conv_dgrad_tma_rows": "mt1_n128x1_ks2",
                                         "conv_wgrad_tma_rows": "n128_sp24"}),
    ((112, 64, 16, 16, 128, 3, 1, 1, 0), {"conv_fprop_tma_rows": "mt2e_n128x1", "conv_dgrad_tma_rows": "sm_mt2_n192x1"}),
]


@pytest.mark.parametrize("shape,variants", BENCH_SHAPES)
def test_conv_benchmark_shapes_at_benchmark_batch(aet, ctx, oracle, shape, variants):
    ctx.set_math(aet.MATH_TF32)
    ctx.profile(1)
    try:
        got, ref = conv_case(aet, ctx, oracle, *shape, seed=500 + shape[0], threads=True)
        used = variants_used(ctx)
    finally:
        ctx.profile(0)
    for kernel, variant in variants.items():
        assert kernel + "." + variant in used, (kernel, variant, sorted(used))
    check(got, ref, TOL_TF32)


# The per-shape sweep of the reference's benchmark list at its batch of 256 (fprop + dgrad + wgrad each).
SWEEP_SHAPES = [
    (256, 3, 32, 32, 64, 3, 1, 1, 0),
    (256, 64, 16, 16, 128, 3, 1, 1, 0),
    (256, 128, 8, 8, 256, 3, 1, 1, 0),
    (256, 256, 8, 8, 256, 3, 1, 1, 0),
    (256, 256, 4, 4, 10, 1, 1, 0, 0),
]


@pytest.mark.parametrize("shape", SWEEP_SHAPES)
def test_conv_sweep_shapes_at_batch_256(aet, ctx, oracle, shape):
    ctx.set_math(aet.MATH_TF32)
    ctx.profile(1)
    try:
        got, ref = conv_case(aet, ctx, oracle, *shape, seed=600 + shape[1], threads=True)
        used = kernels_used(ctx)
        print("sweep shape", shape, "->", sorted(variants_used(ctx)))
    finally:
        ctx.profile(0)
    # every sweep shape is on a TMA or first-layer kernel; only the 3-channel layer's data gradient (which a
    # network never asks for: nothing precedes its first layer) goes through the gather producer
    allowed = {"conv_dgrad_gather"} if shape[1] < 32 else set()
    assert not any("gather" in k for k in used - allowed), used
    check(got, ref, TOL_TF32)


def test_tma_and_gather_agree_closely(aet, ctx, ctx_gather, oracle):
    """Both producers feed the same MMA with the same TF32 inputs: results differ only by summation order."""
    shape = TMA_SHAPES[1]
    a, _ = conv_case(aet, ctx, oracle, *shape, seed=77)
    b, _ = conv_case(aet, ctx_gather, oracle, *shape, seed=77)
    for k in ("y", "dw", "dx"):
        assert rel_l2(a[k], b[k]) < 1e-5, k


def test_first_layer_skips_dgrad_and_wgrad_accumulates(aet, ctx, oracle):
    got, ref = conv_case(aet, ctx, oracle, 2, 3, 8, 8, 8, 3, 1, 1, 2, seed=5, want_dx=False)
    check(got, ref, TOL_TF32)
    import aet_cnn_b200.synth as synth
    layer = aet.ConvolutionalLayer(ctx, 2, 8, 8, 3, 8, 3, 1, 1, 1, aet.LINEAR, 0, 1)
    x = aet.Tensor(ctx, 2, 3, 8, 8)
    x.write(synth.uniform((2, 3, 8, 8), 9, 1))
    st = aet.make_state(input=x, train=1)
    layer.forward(st)
    dy = synth.normal((2, 8, 8, 8), 9, 2)
    layer.write(aet.P_DELTA, dy)
    layer.backward(st)
    g1 = layer.read(aet.P_WEIGHT_UPDATES)
    layer.write(aet.P_DELTA, dy)
    layer.backward(st)
    g2 = layer.read(aet.P_WEIGHT_UPDATES)
    assert np.allclose(g2, 2 * g1, rtol=1e-5, atol=1e-6)        # weight_updates accumulate until update()
    layer.close(); x.close()


def test_reference_single_conv_case_full_size(aet, ctx, oracle):
    """N=128, 3->32, 32x32, 3x3 pad 1, leaky: output, dX, dW, db against the oracle."""
    got, ref = conv_case(aet, ctx, oracle, 128, 3, 32, 32, 32, 3, 1, 1, 2, seed=20240, bias=False)
    check(got, ref, TOL_TF32)


def test_bad_arguments_are_rejected(aet, ctx):
    with pytest.raises(aet.AetError):
        aet.ConvolutionalLayer(ctx, 1, 8, 8, 3, 4, 3, groups=2)
    with pytest.raises(aet.AetError):
        aet.ConvolutionalLayer(ctx, 1, 2, 2, 3, 4, 5)                   # empty output
    layer = aet.ConvolutionalLayer(ctx, 1, 8, 8, 3, 4, 3, 1, 1, 1)
    wrong = aet.Tensor(ctx, 1, 3, 7, 8)
    with pytest.raises(aet.AetError):
        layer.forward(aet.make_state(input=wrong))
    layer.close(); wrong.close()
