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


# Maps whose rows do not divide the 128-pixel tile / 32-pixel slab (the 27x27 and 13x13 maps of an AlexNet-style
# network): the TMA kernels tile them as whole rows of one image and leave the rest of the tile unused.
RAGGED_SHAPES = [
    (4, 96, 27, 27, 256, 5, 1, 2, 1),      # AlexNet-style conv 2: 5x5, 4 rows per tile, 7 tiles per image (the last one 3 rows)
    (4, 256, 13, 13, 384, 3, 1, 1, 1),     # conv 3: 9 rows per tile, 2 tiles per image; 384 filters = three 128-filter tiles
    (5, 384, 13, 13, 256, 3, 1, 1, 2),     # conv 5
    (3, 64, 13, 13, 64, 3, 1, 1, 2),       # one N tile, odd batch
    (2, 32, 7, 20, 32, 3, 1, 1, 0),        # non-square: 6 + 1 rows
    (2, 64, 9, 100, 32, 1, 1, 0, 1),       # one row per tile (w > 64), 1x1
    (2, 32, 12, 40, 64, 3, 1, 1, 2),       # rows wider than a weight-gradient K slab: two 32-column slabs per row
    (1, 64, 56, 56, 64, 3, 1, 1, 1),       # a 56x56 map (ResNet-style): two rows per forward tile, 32 + 24 columns per slab pair
]


@pytest.mark.parametrize("shape", RAGGED_SHAPES)
def test_conv_tma_ragged_maps(aet, ctx, oracle, shape):
    ctx.set_math(aet.MATH_TF32)
    ctx.profile(1)
    try:
        got, ref = conv_case(aet, ctx, oracle, *shape, seed=700 + shape[1], threads=shape[1] >= 96)
        used = variants_used(ctx)
    finally:
        ctx.profile(0)
    names = {u.split("#")[0] for u in used}
    want = {"conv_fprop_tma.ragged", "conv_dgrad_tma.ragged"}
    # a weight-gradient K slab is 32 pixels: narrower maps are tiled as whole rows, wider ones as 32-column pieces of a row
    want.add("conv_wgrad_tma.ragged" if shape[3] <= 32 else "conv_wgrad_tma.wide")
    assert want <= names, sorted(names)
    check(got, ref, TOL_TF32)
    # and the same shapes with the option off go to the gather kernel and agree with it closely
    ctx.set_option("ragged", 0)
    ctx.profile(1)
    try:
        alt, _ = conv_case(aet, ctx, oracle, *shape, seed=700 + shape[1], threads=shape[1] >= 96)
        used = kernels_used(ctx)
    finally:
        ctx.profile(0)
        ctx.set_option("ragged", 1)
    assert "conv_fprop_gather" in used, used
    for key in ("y", "dw", "dx", "db"):
        assert rel_l2(got[key], alt[key]) < 2e-3, key


@pytest.mark.parametrize("shape", [
    (8, 256, 1, 1, 1000, 1, 1, 0, 0),      # a 1000-class fully connected layer as a 1x1 convolution
    (3, 64, 8, 8, 100, 3, 1, 1, 2),        # 100 filters, 3x3
    (4, 96, 13, 13, 50, 3, 1, 1, 1),       # 50 filters (two K slabs, the second 18 wide) on a ragged map
])
def test_conv_tma_forward_takes_any_filter_count(aet, ctx, oracle, shape):
    """The forward TMA kernel reads the filters as rows of its second operand and the data-gradient kernel as its K
    dimension, so their count need not be a multiple of 32 (what lies past the last filter is zero-filled by the copy);
    the weight gradient of such a layer uses the other kernels."""
    ctx.set_math(aet.MATH_TF32)
    ctx.profile(1)
    try:
        got, ref = conv_case(aet, ctx, oracle, *shape, seed=750 + shape[4])
        used = kernels_used(ctx)
    finally:
        ctx.profile(0)
    assert {"conv_fprop_tma", "conv_fprop_tma_rows"} & used, used
    assert {"conv_dgrad_tma", "conv_dgrad_tma_rows"} & used and "conv_dgrad_gather" not in used, used
    check(got, ref, TOL_TF32)


@pytest.mark.parametrize("shape,split", [
    # a fully connected layer as a whole-map filter: one 128-row tile, K = 9216 (its data gradient has 16 K slabs: not split)
    ((128, 256, 6, 6, 512, 6, 1, 0, 1), {"conv_fprop_tma.ks"}),
    # FC after FC, 500 outputs (the last filter tile and the last K slab are partial)
    ((96, 1024, 1, 1, 500, 1, 1, 0, 0), {"conv_fprop_tma.ks"}),
    # 4096 outputs: the data gradient's K range (128 slabs) is split, the forward pass (16 slabs, 32 tiles) is not
    ((128, 512, 1, 1, 4096, 1, 1, 0, 1), {"conv_dgrad_tma.ks"}),
    # a small batch of a wide 3x3 layer: three pixel tiles, 72 K slabs (its data gradient runs on the row-sharing kernel)
    ((6, 256, 8, 8, 256, 3, 1, 1, 2), {"conv_fprop_tma.ks"}),
    # ... and a 1x1 layer of the same kind, whose data gradient is the plain kernel's: 64 K slabs
    ((6, 256, 8, 8, 2048, 1, 1, 0, 1), {"conv_dgrad_tma.ks"}),
])
def test_conv_few_tiles_split_the_k_range(aet, ctx, oracle, shape, split):
    """Forward pass and data gradient of a layer with few output tiles and a long K loop split their K range over
    blockIdx.z and sum the partial tiles in a second kernel (with bias and activation for the forward pass)."""
    ctx.set_math(aet.MATH_TF32)
    ctx.profile(1)
    try:
        got, ref = conv_case(aet, ctx, oracle, *shape, seed=760 + shape[4], threads=True)
        used = variants_used(ctx)
    finally:
        ctx.profile(0)
    names = {u.split("#")[0] for u in used}
    assert split <= names, sorted(names)
    assert ("fprop_reduce" in names) == ("conv_fprop_tma.ks" in split), sorted(names)
    check(got, ref, TOL_TF32)
    ctx.set_option("fd_split", 0)
    try:
        plain, _ = conv_case(aet, ctx, oracle, *shape, seed=760 + shape[4], threads=True)
    finally:
        ctx.set_option("fd_split", 1)
    for key in ("y", "dx"):
        assert rel_l2(got[key].ravel(), plain[key].ravel()) < 2e-3, key


# few input channels: the whole K extent fits one stage of the persistent first-layer kernels
THIN_SHAPES = [
    (2, 3, 8, 8, 5, 3, 1, 1, 2),          # one ragged tile
    (4, 3, 32, 32, 32, 3, 1, 1, 2),       # first layer of the reference's CPU-runnable case
    (128, 3, 32, 32, 64, 3, 1, 1, 0),     # first layer of the benchmark network, full batch: several tiles per CTA
    (3, 4, 9, 7, 6, 3, 2, 1, 1),          # stride 2, odd sizes
    (2, 2, 11, 11, 3, 5, 2, 2, 0),        # 5x5 stride 2: K = 100
    (3, 1, 28, 28, 20, 5, 1, 0, 1),       # one input channel, no padding
    (5, 8, 6, 6, 100, 2, 1, 0, 1),        # two cells per tap, 100 filters
    (2, 3, 12, 16, 8, 5, 1, 2, 0),        # 5x5 with padding: the narrow data-gradient kernel's second instantiation
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
    # shape, context options, {kernel: variant} expected on a 148-SM part ("" = the kernel has no variants)
    # defaults: forward on the plain TMA kernel, data and weight gradient on the row-sharing kernels
    ((128, 64, 16, 16, 128, 3, 1, 1, 2), {}, {"conv_fprop_tma": "", "conv_dgrad_tma_rows": "sm_mt2_n192x1", "conv_wgrad_tma_rows": "n64_sp49"}),
    ((128, 128, 8, 8, 256, 3, 1, 1, 2), {}, {"conv_fprop_tma": "", "conv_dgrad_tma_rows": "mt1_n128x1_ks2", "conv_wgrad_tma_rows": "n128_sp24"}),
    # the row-sharing forward kernel (option rows_fprop)
    ((128, 64, 16, 16, 128, 3, 1, 1, 2), {"rows_fprop": 1}, {"conv_fprop_tma_rows": "mt2e_n128x1", "conv_dgrad_tma_rows": "sm_mt2_n192x1",
                                                             "conv_wgrad_tma_rows": "n64_sp49"}),
    ((128, 128, 8, 8, 256, 3, 1, 1, 2), {"rows_fprop": 1}, {"conv_fprop_tma_rows": "mt1_n128x2", "conv_dgrad_tma_rows": "mt1_n128x1_ks2",
                                                            "conv_wgrad_tma_rows": "n128_sp24"}),
    ((112, 64, 16, 16, 128, 3, 1, 1, 0), {"rows_fprop": 1}, {"conv_fprop_tma_rows": "mt2e_n128x1", "conv_dgrad_tma_rows": "sm_mt2_n192x1"}),
    # CTA pairs (cta_group::2 MMAs, each CTA loading half of the filter tile), off by default
    ((128, 64, 16, 16, 128, 3, 1, 1, 2), {"pair": 1, "rows_fprop": 1}, {"conv_fprop_tma_rows": "mt2e_n128x1_p2", "conv_dgrad_tma_rows": "sm_mt2_n192x1_p2"}),
    ((128, 128, 8, 8, 256, 3, 1, 1, 2), {"pair": 1, "rows_fprop": 1}, {"conv_fprop_tma_rows": "mt1_n128x2_p2", "conv_dgrad_tma_rows": "mt1_n128x1_ks2_p2"}),
    ((16, 64, 16, 16, 128, 3, 1, 1, 1), {"pair": 1, "rows_fprop": 1}, {"conv_fprop_tma_rows": "*_p2", "conv_dgrad_tma_rows": "*_p2"}),
    # two accumulators per tile (alternate filter rows), off by default; also without the rotated K order
    ((128, 128, 8, 8, 256, 3, 1, 1, 2), {"dual_acc": 1, "rows_fprop": 1}, {"conv_fprop_tma_rows": "mt1d_n128x2", "conv_dgrad_tma_rows": "mt1d_n128x1_ks2"}),
    ((128, 128, 8, 8, 256, 3, 1, 1, 2), {"dual_acc": 1, "pair": 1, "rotate": 0, "rows_fprop": 1},
     {"conv_fprop_tma_rows": "mt1d_n128x2_p2", "conv_dgrad_tma_rows": "mt1d_n128x1_ks2_p2"}),
]


@pytest.mark.parametrize("shape,options,variants", BENCH_SHAPES)
def test_conv_benchmark_shapes_at_benchmark_batch(aet, ctx, oracle, shape, options, variants):
    ctx.set_math(aet.MATH_TF32)
    saved = {name: ctx.get_option(name) for name in options}
    for name, value in options.items():
        ctx.set_option(name, value)
    ctx.profile(1)
    try:
        got, ref = conv_case(aet, ctx, oracle, *shape, seed=500 + shape[0], threads=True)
        used = variants_used(ctx)
    finally:
        ctx.profile(0)
        for name, value in saved.items():
            ctx.set_option(name, value)
    for kernel, variant in variants.items():
        if variant == "":
            assert kernel in used, (kernel, sorted(used))
        elif variant.startswith("*"):
            assert any(u.startswith(kernel + ".") and u.endswith(variant[1:]) for u in used), (kernel, variant, sorted(used))
        else:
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


# Large strided filters on an image (the thin-K kernels stop at K = 128): regrouped into s x s pixel blocks they are
# stride-1 convolutions over s*s*4 channels, which the TMA kernels run (conv_s2d.cuh).
S2D_SHAPES = [
    (4, 3, 47, 47, 16, 11, 4, 0, 1),      # AlexNet-style first layer, reduced: 3x3 block taps on a 12x12 regrouped map, 64 channels
    (3, 3, 59, 59, 96, 11, 4, 0, 1),      # ... with its 96 filters (a whole number of 32-filter blocks: TMA weight gradient)
    (2, 3, 23, 27, 32, 7, 2, 3, 2),       # 7x7 stride 2 with padding (ResNet-style stem): 4x4 block taps, 16 -> 32 channels
    (2, 1, 38, 38, 8, 6, 3, 1, 0),        # one input channel, stride 3 (36 -> 64 channels), even filter
    (5, 4, 30, 30, 40, 8, 2, 0, 1),       # filter size a multiple of the stride
    (4, 3, 22, 22, 64, 8, 2, 0, 2),       # 8x8 output map: the weight gradient is regrouped too
    (2, 3, 71, 71, 32, 11, 4, 0, 1),      # 16x16 output map, 11x11 / 4
]
S2D_WGRAD = S2D_SHAPES[-2:]


@pytest.mark.parametrize("shape", S2D_SHAPES)
def test_conv_regrouped_strided_first_layer(aet, ctx, oracle, shape):
    ctx.set_math(aet.MATH_TF32)
    ctx.profile(1)
    try:
        got, ref = conv_case(aet, ctx, oracle, *shape, seed=900 + shape[5])
        used = kernels_used(ctx)
    finally:
        ctx.profile(0)
    assert {"conv_s2d_input", "conv_s2d_weights"} <= used, used
    assert {"conv_fprop_tma", "conv_fprop_tma_rows"} & used and "conv_fprop_gather" not in used, used
    # the weight gradient is regrouped only where its 32-pixel K slabs tile the output map
    print("regrouped shape", shape, "->", sorted(used))
    if shape in S2D_WGRAD:
        assert "conv_s2d_fold" in used and {"conv_wgrad_tma", "conv_wgrad_tma_rows"} & used and "conv_wgrad_gather" not in used, used
    check(got, ref, TOL_TF32)
    # with the option off the same layer runs on the gather kernel and agrees closely
    ctx.set_option("s2d", 0)
    ctx.profile(1)
    try:
        plain, _ = conv_case(aet, ctx, oracle, *shape, seed=900 + shape[5])
        used = kernels_used(ctx)
    finally:
        ctx.profile(0)
        ctx.set_option("s2d", 1)
    assert "conv_fprop_gather" in used and "conv_s2d_input" not in used, used
    for k in ("y", "dw"):
        assert rel_l2(got[k].ravel(), plain[k].ravel()) <= 2e-3, k


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
    # every sweep shape is on a TMA or first-layer kernel; the 3-channel layer's data gradient (which a network never
    # asks for: nothing precedes its first layer) has a CUDA-core kernel of its own
    assert not any("gather" in k for k in used), used
    if shape[1] < 32:
        assert "conv_dgrad_narrow" in used, used
    check(got, ref, TOL_TF32)


# every activation whose gradient is a function of its output (dnn/Activation.h:41-113), numbered as in the C ABI
ACTIVATIONS = list(range(3, 14))


@pytest.mark.parametrize("act", ACTIVATIONS)
def test_conv_activation_family(aet, ctx, oracle, act):
    """Forward value and the gradient through the activation (evaluated on the stored output) for the activations
    beyond linear / relu / leaky, in a convolution's epilogue and backward kernels, TMA and gather producers."""
    for shape in [(4, 32, 8, 8, 32, 3, 1, 1), (2, 3, 9, 7, 6, 3, 2, 1)]:
        got, ref = conv_case(aet, ctx, oracle, *shape, act, seed=700 + act)
        check(got, ref, TOL_TF32)


@pytest.mark.parametrize("act1,act2", [("logistic", "elu"), ("swish", "mish"), ("mish", "swish")])
def test_conv_bn_with_other_activations_matches_oracle_network(aet, ctx, oracle64, act1, act2):
    """BN layers recompute the activation and its gradient from the saved convolution result: a two-layer network with
    output-gradient activations (logistic, elu) and with the two whose gradient needs the value before the activation
    (swish, mish: dnn/IOData.c:75-105, dnn/Activation.c:303-330) against the oracle, 3xTF32 math.  The first layer's
    2x2 pool is fused, so both the window-major and the plain BN backward kernels see these activations."""
    import aet_cnn_b200.synth as synth
    from oracle import binding as ob
    from oracle import cfgfile
    text = ("[net]\nbatch=4\nheight=8\nwidth=8\nchannels=3\nlearning_rate=0.01\nmomentum=0.9\ndecay=0.0005\n"
            "[convolutional]\nfilters=8\nsize=3\nstride=1\npad=1\nbatch_normalize=1\nactivation=%s\n"
            "[maxpool]\nsize=2\nstride=2\n"
            "[convolutional]\nfilters=12\nsize=3\nstride=1\npad=1\nbatch_normalize=1\nactivation=%s\n"
            "[convolutional]\nfilters=5\nsize=1\nstride=1\npad=0\nactivation=tanh\n[avgpool]\n[softmax]\n") % (act1, act2)
    opts, specs = cfgfile.network_spec(text)
    ctx.set_math(aet.MATH_3XTF32)
    try:
        net = aet.NNetwork(ctx, cfg_text=text, train=1)
        onet = oracle64.net(specs, 4, 3, 8, 8, mode=ob.MODE_MTCS)
        cin = 3
        for i, s in enumerate(specs):
            if s["type"] == cfgfile.CONV:
                w = synth.normal((s["filters"], cin, s["size"], s["size"]), 13, 50 + i, 0.0, 0.3)
                net.layer(i).write(aet.P_WEIGHTS, w); onet.set_param(i, ob.P_WEIGHTS, w)
                cin = s["filters"]
        for step in range(3):
            x = synth.uniform((4, 3, 8, 8), 13, 2 * step)
            _, t = synth.labels(4, 5, 13, 2 * step + 1)
            loss = net.train(x, t)
            oloss = onet.train_step(x, t, opts["learning_rate"], opts["momentum"], opts["decay"])
            assert abs(loss - oloss) <= 1e-4 * abs(oloss), (step, loss, oloss)
        for i, s in enumerate(specs):
            if s["type"] == cfgfile.CONV:
                assert rel_l2(net.layer(i).read(aet.P_WEIGHTS), onet.param(i, ob.P_WEIGHTS)) < 1e-4, i
        ctx.check()
        net.close()
    finally:
        ctx.set_math(aet.MATH_TF32)


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


# (N, C, H, W, K, size, stride, pad, act, groups, dilation)
GROUP_DILATION_SHAPES = [
    None,
    (2, 16, 8, 8, 16, 3, 1, 1, 1, 4, 1),       # four groups of 4 channels -> 4 filters
    (2, 64, 8, 8, 64, 3, 1, 1, 2, 2, 1),       # two groups of 32 -> 32
    (2, 16, 6, 6, 32, 1, 1, 0, 0, 2, 1),       # grouped 1x1
    (2, 8, 8, 8, 8, 3, 2, 1, 1, 2, 1),         # grouped, stride 2
    (2, 4, 12, 12, 8, 3, 1, 1, 2, 1, 2),       # dilation 2
    (2, 32, 10, 10, 32, 3, 1, 1, 0, 1, 3),     # dilation 3 on a TMA-eligible channel count (runs on the gather producer)
    (2, 16, 11, 9, 16, 5, 1, 2, 1, 2, 2),      # groups and dilation together, 5x5
]


@pytest.mark.parametrize("shape", GROUP_DILATION_SHAPES[1:])
def test_conv_groups_and_dilation(aet, ctx, oracle, shape):
    """Channel groups (dnn/ConvolutionalLayer.c:716-722) and dilated taps (dnn/Im2Col.c:65-103): output, dX, dW, db."""
    *base, groups, dilation = shape
    got, ref = conv_case(aet, ctx, oracle, *base, seed=800 + base[1] + groups, groups=groups, dilation=dilation)
    check(got, ref, TOL_TF32)


@pytest.mark.parametrize("shape", [
    (3, 8, 12, 12, 16, 3, (2, 1), 1, 1),     # stride_x = 2, stride_y = 1
    (3, 8, 12, 12, 16, 3, (1, 2), 1, 2),     # stride_x = 1, stride_y = 2
    (2, 32, 9, 14, 32, 5, (3, 2), 2, 1),     # 5x5, both strides different, ragged map
])
def test_conv_unequal_strides(aet, ctx, oracle, shape):
    """stride_x != stride_y (dnn/ConvolutionalLayer.c:703-715, the cfg keys stride_x / stride_y): output, dX, dW, db."""
    got, ref = conv_case(aet, ctx, oracle, *shape, seed=900 + shape[1])
    check(got, ref, TOL_TF32)


def test_bad_arguments_are_rejected(aet, ctx):
    with pytest.raises(aet.AetError):
        aet.ConvolutionalLayer(ctx, 1, 8, 8, 3, 4, 3, groups=2)                # 3 channels do not split in two
    with pytest.raises(aet.AetError):
        aet.ConvolutionalLayer(ctx, 1, 8, 8, 8, 12, 3, groups=2)               # 6 filters per group: not a multiple of 4
    with pytest.raises(aet.AetError):
        aet.ConvolutionalLayer(ctx, 1, 8, 8, 8, 8, 4, 1, 1, 1, dilation=2)     # dilation needs an odd filter padded by size/2
    with pytest.raises(aet.AetError):
        aet.ConvolutionalLayer(ctx, 1, 2, 2, 3, 4, 5)                   # empty output
    layer = aet.ConvolutionalLayer(ctx, 1, 8, 8, 3, 4, 3, 1, 1, 1)
    wrong = aet.Tensor(ctx, 1, 3, 7, 8)
    with pytest.raises(aet.AetError):
        layer.forward(aet.make_state(input=wrong))
    layer.close(); wrong.close()
