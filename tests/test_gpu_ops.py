"""GPU parity of the bandwidth-bound kernels against the CPU oracle, through the C ABI: batch norm
fused with the activation (both parity modes), pooling (bit-exact argmax indices), softmax +
cross-entropy, dropout (shared mask) and the SGD-momentum update."""
import numpy as np
import pytest

from conftest import rel_l2
from oracle import binding as ob

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", [ob.MODE_MTCS, ob.MODE_CPU])
@pytest.mark.parametrize("shape,act", [((4, 6, 5, 5), 2), ((8, 64, 16, 16), 2), ((3, 10, 7, 3), 1), ((2, 300, 4, 4), 0)])
def test_conv_bn_layer_forward_backward(aet, ctx, oracle64, mode, shape, act):
    """1x1 identity-free check: conv(1x1) + BN + activation; the conv is exact enough in 3xTF32 that
    the comparison isolates the BN kernels."""
    import aet_cnn_b200.synth as synth
    N, K, H, W = shape
    C = 8
    ctx.set_parity(mode)
    ctx.set_math(aet.MATH_3XTF32)
    try:
        x = synth.normal((N, C, H, W), 31, 1, 0.3, 1.0)
        w = synth.normal((K, C, 1, 1), 31, 2, 0, 0.5)
        gamma = synth.uniform((K,), 31, 3) + 0.5
        beta = synth.normal((K,), 31, 4, 0, 0.2)
        dy = synth.normal((N, K, H, W), 31, 5)
        rm0, rv0 = synth.normal((K,), 31, 6), synth.uniform((K,), 31, 7) + 0.5
        layer = aet.ConvolutionalLayer(ctx, N, H, W, C, K, 1, 1, 1, 0, act, 1, 1)
        layer.write(aet.P_WEIGHTS, w); layer.write(aet.P_SCALES, gamma); layer.write(aet.P_BIASES, beta)
        layer.write(aet.P_ROLLING_MEAN, rm0); layer.write(aet.P_ROLLING_VARIANCE, rv0)
        xin, dxt = aet.Tensor(ctx, N, C, H, W), aet.Tensor(ctx, N, C, H, W)
        xin.write(x)
        st = aet.make_state(input=xin, delta=dxt, train=1)
        layer.forward(st)
        y = layer.read(aet.P_OUTPUT).reshape(shape)
        mean, var = layer.read(aet.P_MEAN), layer.read(aet.P_VARIANCE)
        rm, rv = layer.read(aet.P_ROLLING_MEAN), layer.read(aet.P_ROLLING_VARIANCE)
        xs, xn = layer.read(aet.P_X).reshape(shape), layer.read(aet.P_X_NORM).reshape(shape)
        layer.write(aet.P_DELTA, dy)
        layer.backward(st)
        ctx.check()
        dgam, dbeta = layer.read(aet.P_SCALE_UPDATES), layer.read(aet.P_BIAS_UPDATES)
        dx = dxt.read()
        # inference branch with the rolling statistics
        layer.forward(aet.make_state(input=xin, train=0))
        y_eval = layer.read(aet.P_OUTPUT).reshape(shape)
        layer.close(); xin.close(); dxt.close()
    finally:
        ctx.set_parity(ob.MODE_MTCS)
        ctx.set_math(aet.MATH_TF32)

    conv = oracle64.conv_forward(x, w)
    f = oracle64.bn_forward(mode, True, conv, gamma, beta, rm0, rv0)
    yo = oracle64.activate(f["y"], act, mode)
    assert rel_l2(xs, conv) < 1e-5
    assert rel_l2(mean, f["mean"]) < 1e-5 and rel_l2(var, f["variance"]) < 1e-4
    assert rel_l2(rm, f["rolling_mean"]) < 1e-5 and rel_l2(rv, f["rolling_variance"]) < 1e-5
    assert rel_l2(xn, f["x_norm"]) < 1e-4
    assert rel_l2(y, yo) < 1e-4
    d = oracle64.gradient(yo, act, dy)
    b = oracle64.bn_backward(mode, d, f["x"], f["x_norm"], f["mean"], f["variance"], gamma)
    assert rel_l2(dgam, b["scale_updates"]) < 1e-4
    if mode == ob.MODE_MTCS:
        assert rel_l2(dbeta, b["bias_updates"]) < 1e-4
    else:
        assert np.array_equal(dbeta, np.zeros_like(dbeta))     # the reference's CPU path never updates the BN shift
    _, dxo = oracle64.conv_backward(x, w, b["delta"])
    assert rel_l2(dx, dxo) < 2e-4
    e = oracle64.bn_forward(mode, False, conv, gamma, beta, f["rolling_mean"], f["rolling_variance"])
    assert rel_l2(y_eval, oracle64.activate(e["y"], act, mode)) < 1e-4


@pytest.mark.parametrize("mode", [ob.MODE_MTCS, ob.MODE_CPU])
@pytest.mark.parametrize("geom", [(4, 6, 8, 8, 2, 2, 1), (2, 3, 9, 9, 3, 2, 0), (2, 5, 7, 6, 3, 2, 2), (3, 64, 16, 16, 2, 2, 1),
                                  (2, 4, 5, 5, 2, 1, 1), (1, 2, 6, 6, 3, 3, 2)])
def test_maxpool_values_and_indices_bit_exact(aet, ctx, oracle, mode, geom):
    import aet_cnn_b200.synth as synth
    N, C, H, W, size, stride, padding = geom
    ctx.set_parity(mode)
    try:
        x = synth.normal((N, C, H, W), 41, size)
        x[0, 0, :2, :2] = 1.5                                  # a tie inside the first window
        layer = aet.MaxPoolLayer(ctx, N, H, W, C, size, stride, stride, padding, 1)
        xin, pd = aet.Tensor(ctx, N, C, H, W), aet.Tensor(ctx, N, C, H, W)
        xin.write(x)
        st = aet.make_state(input=xin, delta=pd, train=1)
        layer.forward(st)
        oc, oh, ow = layer.out_shape
        y = layer.read(aet.P_OUTPUT).reshape(N, oc, oh, ow)
        idx = layer.read(aet.P_INDEXES).reshape(N, oc, oh, ow)
        dy = synth.normal((N, oc, oh, ow), 41, 99)
        layer.write(aet.P_DELTA, dy)
        prev0 = synth.normal((N, C, H, W), 41, 98)
        pd.write(prev0)
        layer.backward(st)                                      # adds into the previous delta
        got_pd = pd.read()
        layer.close(); xin.close(); pd.close()
    finally:
        ctx.set_parity(ob.MODE_MTCS)
    yo, io = oracle.maxpool_forward(mode, x, size, stride, stride, padding)
    assert y.shape == yo.shape
    assert np.array_equal(idx, io), "argmax indices must be bit-exact"
    assert np.array_equal(y, yo)
    assert np.allclose(got_pd, oracle.maxpool_backward(dy, io, prev0), rtol=1e-6, atol=1e-6)


def test_avgpool_forward_backward(aet, ctx, oracle):
    import aet_cnn_b200.synth as synth
    N, C, H, W = 5, 10, 4, 4
    x = synth.normal((N, C, H, W), 51, 1)
    layer = aet.AvgPoolLayer(ctx, N, W, H, C)
    xin, pd = aet.Tensor(ctx, N, C, H, W), aet.Tensor(ctx, N, C, H, W)
    xin.write(x)
    st = aet.make_state(input=xin, delta=pd, train=1)
    layer.forward(st)
    y = layer.read(aet.P_OUTPUT).reshape(N, C)
    dy = synth.normal((N, C), 51, 2)
    layer.write(aet.P_DELTA, dy)
    prev0 = synth.normal((N, C, H, W), 51, 3)
    pd.write(prev0)
    layer.backward(st)
    got = pd.read()
    layer.close(); xin.close(); pd.close()
    assert rel_l2(y, oracle.avgpool_forward(x)) < 1e-6
    assert rel_l2(got, oracle.avgpool_backward(dy, prev0)) < 1e-6


@pytest.mark.parametrize("mode", [ob.MODE_MTCS, ob.MODE_CPU])
@pytest.mark.parametrize("N,classes,groups", [(128, 10, 1), (7, 1000, 1), (4, 12, 3)])
def test_softmax_cross_entropy(aet, ctx, oracle, mode, N, classes, groups):
    import aet_cnn_b200.synth as synth
    ctx.set_parity(mode)
    try:
        x = synth.normal((N, classes), 61, 1, 0, 3.0)
        _, truth = synth.labels(N, classes, 61, 2)
        layer = aet.SoftMaxLayer(ctx, N, classes, groups, 1.0)
        xin, tr, pd = aet.Tensor(ctx, N, classes), aet.Tensor(ctx, N, classes), aet.Tensor(ctx, N, classes)
        xin.write(x); tr.write(truth)
        st = aet.make_state(input=xin, delta=pd, truth=tr, train=1)
        layer.forward(st)
        p = layer.read(aet.P_OUTPUT).reshape(N, classes)
        delta = layer.read(aet.P_DELTA).reshape(N, classes)
        loss = layer.read(aet.P_LOSS).reshape(N, classes)
        cost = layer.cost()
        prev0 = synth.normal((N, classes), 61, 3)
        pd.write(prev0)
        layer.backward(st)
        got_pd = pd.read().reshape(N, classes)
        layer.close(); xin.close(); tr.close(); pd.close()
    finally:
        ctx.set_parity(ob.MODE_MTCS)
    r = oracle.softmax_forward(mode, x, truth, groups)
    assert rel_l2(p, r["p"]) < 2e-6
    assert rel_l2(delta, r["delta"]) < 2e-6
    assert np.array_equal(loss != 0, r["loss"] != 0)            # labels are integers: the support must match exactly
    assert rel_l2(loss, r["loss"]) < 2e-6
    assert abs(cost - r["cost"]) <= 2e-6 * abs(r["cost"]) + 1e-6
    assert rel_l2(got_pd, prev0 + r["delta"]) < 2e-6


def test_dropout_mask_and_scale(aet, ctx, oracle):
    import aet_cnn_b200.synth as synth
    N, C = 6, 40
    prev = aet.ConvolutionalLayer(ctx, N, 1, 1, 8, C, 1, 1, 1, 0, aet.LINEAR, 0, 1)
    drop = aet.DropoutLayer(ctx, N, C, 0.5, prev)
    vals = synth.normal((N, C, 1, 1), 71, 1)
    prev.write(aet.P_OUTPUT, vals)
    st = aet.make_state(input=prev.output, delta=prev.delta, train=1)
    drop.forward(st)
    r = drop.read(aet.P_RAND)
    out = prev.read(aet.P_OUTPUT)
    assert 0.0 <= r.min() and r.max() < 1.0 and 0.3 < (r < 0.5).mean() < 0.7
    assert np.array_equal(out, oracle.dropout_forward(vals.ravel(), r, 0.5))   # same mask => bit-identical
    d = synth.normal((N, C, 1, 1), 71, 2)
    prev.write(aet.P_DELTA, d)
    drop.backward(st)
    assert np.array_equal(prev.read(aet.P_DELTA), oracle.dropout_forward(d.ravel(), r, 0.5))
    drop.forward(st)
    assert not np.array_equal(drop.read(aet.P_RAND), r)          # a new mask every step
    prev.write(aet.P_OUTPUT, vals)
    drop.forward(aet.make_state(input=prev.output, train=0))     # identity at inference
    assert np.array_equal(prev.read(aet.P_OUTPUT), vals.ravel())
    drop.close(); prev.close()


def test_sgd_momentum_three_steps(aet, ctx, oracle):
    import aet_cnn_b200.synth as synth
    N, C, K = 4, 6, 5
    layer = aet.ConvolutionalLayer(ctx, N, 5, 5, C, K, 3, 1, 1, 1, aet.LINEAR, 1, 1)
    w = synth.normal((K, C, 3, 3), 81, 1, 0, 0.2)
    b = synth.normal((K,), 81, 2)
    s = synth.uniform((K,), 81, 3) + 0.5
    layer.write(aet.P_WEIGHTS, w); layer.write(aet.P_BIASES, b); layer.write(aet.P_SCALES, s)
    uw, ub, us = np.zeros_like(w), np.zeros_like(b), np.zeros_like(s)
    for step in range(3):
        gw = synth.normal(w.shape, 81, 10 + step)
        gb, gs = synth.normal((K,), 81, 20 + step), synth.normal((K,), 81, 30 + step)
        # pending gradients enter through the same accumulator the backward pass uses
        layer.write(aet.P_WEIGHT_UPDATES, uw + gw); layer.write(aet.P_BIAS_UPDATES, ub + gb)
        layer.write(aet.P_SCALE_UPDATES, us + gs)
        layer.update(N, 0.1, 0.9, 5e-4, 1.0)
        w, uw = oracle.sgd_weights(w, uw + gw, N, 0.1, 0.9, 5e-4)
        b, ub = oracle.sgd_plain(b, ub + gb, N, 0.1, 0.9)
        s, us = oracle.sgd_plain(s, us + gs, N, 0.1, 0.9)
        uw = uw.reshape(w.shape)
        assert rel_l2(layer.read(aet.P_WEIGHTS), w) < 1e-6
        assert rel_l2(layer.read(aet.P_WEIGHT_UPDATES), uw) < 1e-6
        assert rel_l2(layer.read(aet.P_BIASES), b) < 1e-6 and rel_l2(layer.read(aet.P_SCALES), s) < 1e-6
    layer.close()


def test_tensor_roundtrip_and_padding(aet, ctx):
    import aet_cnn_b200.synth as synth
    for shape in [(2, 3, 5, 7), (1, 10, 1, 1), (3, 64, 4, 4)]:
        t = aet.Tensor(ctx, *shape)
        assert t.shape == shape and np.array_equal(t.read(), np.zeros(shape, np.float32))
        x = synth.normal(shape, 91, 1)
        t.write(x)
        assert np.array_equal(t.read(), x)
        t.zero()
        assert not t.read().any()
        t.close()


# (N, C, H, W, K): first-layer kernel; row-sharing TMA kernel with one pixel tile per CTA; the same at the benchmark
# batch, where it runs two pixel tiles per CTA and a second epilogue warp group writes its own partial row; tiles
# spanning several images with the K range split over a CTA pair (batch 32) and with two filter tiles (batch 128);
# general gather kernel with ragged filter counts
EPILOGUE_STAT_SHAPES = [(128, 3, 32, 32, 64), (16, 64, 16, 16, 128), (128, 64, 16, 16, 128), (32, 128, 8, 8, 256),
                        (128, 128, 8, 8, 256), (5, 12, 9, 7, 20), (5, 12, 9, 7, 16), (3, 8, 6, 6, 44), (2, 3, 8, 8, 5)]


@pytest.mark.parametrize("shape", EPILOGUE_STAT_SHAPES)
def test_bn_statistics_from_conv_epilogue_match_the_separate_pass(aet, ctx, shape):
    """Training-mode batch statistics gathered inside the convolution's epilogue against the
    stand-alone reduction over the stored output (same shift, same finalize): float summation order only."""
    import os
    import aet_cnn_b200.synth as synth
    N, C, H, W, K = shape
    res = {}
    # (without statistics to gather, a forward pass with few tiles would split its K range and sum in another order:
    # both runs keep one CTA per tile, so that only the statistics path differs)
    ctx.set_option("fd_split", 0)
    try:
        for tag in ("epilogue", "separate"):
            ctx.set_option("epilogue_stats", tag == "epilogue")
            try:
                layer = aet.ConvolutionalLayer(ctx, N, H, W, C, K, 3, 1, 1, 1, aet.LEAKY, 1, 1)
                layer.write(aet.P_WEIGHTS, synth.normal((K, C, 3, 3), 31, 1, 0.0, 0.2))
                x = aet.Tensor(ctx, N, C, H, W)
                x.write(synth.uniform((N, C, H, W), 31, 2))
                st = aet.make_state(input=x, train=1)
                ctx.profile(1)
                layer.forward(st)
                layer.forward(st)      # second pass: the shift is the first pass's batch mean
                used = {r["name"].split(".")[0] for r in ctx.profile_read()}
                ctx.profile(0)
                assert ("bn_stats" in used) == (tag == "separate"), used
                res[tag] = (layer.read(aet.P_MEAN), layer.read(aet.P_VARIANCE), layer.read(aet.P_ROLLING_MEAN),
                            layer.read(aet.P_OUTPUT))
                layer.close(); x.close()
            finally:
                ctx.set_option("epilogue_stats", 1)
    finally:
        ctx.set_option("fd_split", 1)
    for a, b in zip(res["epilogue"], res["separate"]):
        assert np.isfinite(a).all()
        assert rel_l2(a.ravel(), b.ravel()) < 2e-6
