"""Pins the CPU oracle: hand-computable cases, fixtures from an independent float64 implementation
(tests/golden/ops_f64.npz), the im2col/col2im adjoint identity, finite differences, and the
documented differences between the reference's CPU and MTCS formulas."""
import ctypes as C
import os

import numpy as np
import pytest

from conftest import ROOT, rel_l2
from oracle import binding as ob

G = np.load(os.path.join(ROOT, "tests", "golden", "ops_f64.npz"))


def test_rng_matches_numpy_generator(oracle, aet):
    import aet_cnn_b200.synth as synth
    for seed, tid in [(20241, 0), (7, 12345)]:
        assert np.array_equal(oracle.uniform((1000,), seed, tid), synth.uniform((1000,), seed, tid))
        a, b = oracle.normal((501,), seed, tid, 0.5, 2.0), synth.normal((501,), seed, tid, 0.5, 2.0)
        assert np.allclose(a, b, rtol=2e-6, atol=2e-6)   # libm vs numpy transcendental rounding
    u = synth.uniform((100000,), 1, 2)
    assert 0.0 <= u.min() and u.max() < 1.0 and abs(u.mean() - 0.5) < 0.01


def test_gemm_all_transposes(oracle):
    rng = np.random.default_rng(0)
    M, N, K = 5, 7, 6
    for TA in (0, 1):
        for TB in (0, 1):
            A = rng.standard_normal((K, M) if TA else (M, K)).astype(np.float32)
            B = rng.standard_normal((N, K) if TB else (K, N)).astype(np.float32)
            Cm = rng.standard_normal((M, N)).astype(np.float32)
            ref = 0.5 * Cm + 2.0 * ((A.T if TA else A).astype(np.float64) @ (B.T if TB else B))
            out = Cm.copy()
            f = C.POINTER(C.c_float)
            oracle.lib.aeto_gemm(TA, TB, M, N, K, 2.0, A.ctypes.data_as(f), A.shape[1], B.ctypes.data_as(f), B.shape[1],
                                 0.5, out.ctypes.data_as(f), N)
            assert np.allclose(out, ref, rtol=1e-5, atol=1e-5)


def test_conv_hand_case(oracle):
    # 1 image, 1 channel, 3x3 ramp, one 3x3 all-ones filter, pad 1: every output is a window sum
    x = np.arange(9, dtype=np.float32).reshape(1, 1, 3, 3)
    w = np.ones((1, 1, 3, 3), np.float32)
    y = oracle.conv_forward(x, w, 1, 1, 1)
    assert np.array_equal(y.ravel(), np.array([8, 15, 12, 21, 36, 27, 20, 33, 24], np.float32))
    # 2 channels, 1x1 filter = per-pixel dot product
    x2 = np.stack([np.full((2, 2), 2.0), np.full((2, 2), 3.0)])[None].astype(np.float32)
    w2 = np.array([1.0, -1.0], np.float32).reshape(1, 2, 1, 1)
    assert np.array_equal(oracle.conv_forward(x2, w2).ravel(), np.full(4, -1.0, np.float32))


@pytest.mark.parametrize("name", ["conv_a", "conv_b", "conv_c", "conv_d"])
def test_conv_against_float64_fixture(oracle, name):
    stride, pad = (int(v) for v in G[name + "_geom"])
    x, w, dy = G[name + "_x"], G[name + "_w"], G[name + "_dy"]
    y = oracle.conv_forward(x, w, stride, stride, pad)
    dw, dx = oracle.conv_backward(x, w, dy, stride, stride, pad)
    assert rel_l2(y, G[name + "_y"]) < 2e-6
    assert rel_l2(dw, G[name + "_dw"]) < 2e-6
    assert rel_l2(dx, G[name + "_dx"]) < 2e-6


def test_conv_wgrad_accumulates_and_dgrad_overwrites(oracle):
    x, w, dy = G["conv_a_x"], G["conv_a_w"], G["conv_a_dy"]
    dw1, _ = oracle.conv_backward(x, w, dy, 1, 1, 1)
    dw2, _ = oracle.conv_backward(x, w, dy, 1, 1, 1, dw=dw1)
    assert np.allclose(dw2, 2 * dw1, rtol=1e-5, atol=1e-6)


def test_im2col_col2im_adjoint(oracle):
    rng = np.random.default_rng(1)
    c, h, w, k, pad, stride = 3, 7, 6, 3, 1, 2
    oh, ow = oracle.conv_out(h, k, stride, pad), oracle.conv_out(w, k, stride, pad)
    x = rng.standard_normal((c, h, w)).astype(np.float32)
    ycol = rng.standard_normal((c * k * k, oh * ow)).astype(np.float32)
    col = np.zeros_like(ycol)
    im = np.zeros_like(x)
    f = C.POINTER(C.c_float)
    oracle.lib.aeto_im2col(x.ctypes.data_as(f), c, h, w, k, k, pad, pad, stride, stride, col.ctypes.data_as(f))
    oracle.lib.aeto_col2im(ycol.ctypes.data_as(f), c, h, w, k, k, pad, pad, stride, stride, im.ctypes.data_as(f))
    assert abs(float((col.astype(np.float64) * ycol).sum()) - float((x.astype(np.float64) * im).sum())) < 1e-3


def test_bias_and_activation(oracle):
    y = np.array([-2.0, -0.5, 0.0, 0.5, 3.0], np.float32).reshape(1, 1, 1, 5)
    assert np.allclose(oracle.activate(y, ob.LEAKY, ob.MODE_MTCS).ravel(), [-0.2, -0.05, 0, 0.5, 3])
    assert np.allclose(oracle.activate(y, ob.RELU).ravel(), [0, 0, 0, 0.5, 3])
    assert np.array_equal(oracle.activate(y, ob.LINEAR), y)
    d = np.ones_like(y)
    assert np.allclose(oracle.gradient(y, ob.LEAKY, d).ravel(), [0.1, 0.1, 0.1, 1, 1])   # gradient at y == 0 is the slope
    assert np.allclose(oracle.gradient(y, ob.RELU, d).ravel(), [0, 0, 0, 1, 1])
    t = np.zeros((2, 3, 2, 2), np.float32)
    assert np.array_equal(oracle.add_bias(t, [1, 2, 3])[1, :, 0, 0], [1, 2, 3])
    assert np.array_equal(oracle.backward_bias(np.ones((2, 3, 2, 2), np.float32)), [8, 8, 8])


def test_bn_mtcs_against_float64_fixture(oracle):
    r = oracle.bn_forward(ob.MODE_MTCS, True, G["bn_x"], G["bn_g"], G["bn_b"], np.zeros(3), np.zeros(3))
    assert rel_l2(r["y"], G["bn_y"]) < 2e-6
    assert rel_l2(r["mean"], G["bn_mean"]) < 1e-6 and rel_l2(r["variance"], G["bn_var"]) < 1e-5
    assert np.allclose(r["rolling_mean"], 0.01 * G["bn_mean"], rtol=1e-5)
    b = oracle.bn_backward(ob.MODE_MTCS, G["bn_dy"], r["x"], r["x_norm"], r["mean"], r["variance"], G["bn_g"])
    assert rel_l2(b["scale_updates"], G["bn_dg"]) < 1e-5
    assert rel_l2(b["bias_updates"], G["bn_db"]) < 1e-5
    # the MTCS kernels mix eps placements (1e-5 forward, 1e-6 in two backward terms, eps outside the
    # sqrt in the third), so dx matches the exact derivative only to ~eps/var
    assert rel_l2(b["delta"], G["bn_dx"]) < 2e-3


def test_bn_cpu_mode_documented_differences(oracle):
    x = G["bn_x"]
    m = x.shape[0] * x.shape[2] * x.shape[3]
    r = oracle.bn_forward(ob.MODE_CPU, True, x, G["bn_g"], G["bn_b"], np.zeros(3), np.zeros(3))
    assert rel_l2(r["variance"], G["bn_var"] * m / (m - 1)) < 1e-4          # divisor m-1
    assert np.allclose(r["rolling_mean"], 0.1 * r["mean"], rtol=1e-5)        # .9 / .1
    b = oracle.bn_backward(ob.MODE_CPU, G["bn_dy"], r["x"], r["x_norm"], r["mean"], r["variance"], G["bn_g"])
    assert np.array_equal(b["bias_updates"], np.zeros(3, np.float32))       # the CPU path never forms the shift gradient
    e = oracle.bn_forward(ob.MODE_CPU, False, x, G["bn_g"], G["bn_b"], r["mean"], r["variance"])
    assert rel_l2(e["y"], r["y"]) < 1e-5                                    # eval with the batch statistics reproduces train


@pytest.mark.parametrize("name,size,stride", [("mp2", 2, 2), ("mp3", 3, 2)])
def test_maxpool_against_fixture(oracle, name, size, stride):
    x = G[name + "_x"]
    for mode in (ob.MODE_CPU, ob.MODE_MTCS):
        y, idx = oracle.maxpool_forward(mode, x, size, stride, stride, 0)
        assert np.array_equal(y, G[name + "_y"].astype(np.float32))
        n, c, h, w = x.shape
        plane = (np.arange(n)[:, None] * c + np.arange(c)[None, :]) * h * w      # reference indices span the whole tensor
        assert np.array_equal(idx - plane[:, :, None, None], G[name + "_idx"])
        dx = oracle.maxpool_backward(G[name + "_dy"], idx, np.zeros_like(x))
        assert rel_l2(dx, G[name + "_dx"]) < 1e-6


def test_maxpool_default_padding_ties_and_all_padding(oracle):
    # Darknet default padding = size-1: 2/2 on 4x4 -> 2x2 with offset 0
    x = np.zeros((1, 1, 4, 4), np.float32)
    y, idx = oracle.maxpool_forward(ob.MODE_CPU, x, 2, 2, 2, 1)
    assert y.shape == (1, 1, 2, 2)
    assert np.array_equal(idx.ravel(), [0, 2, 8, 10])            # ties keep the FIRST element in row/col scan order
    # size 3 stride 2 with default padding 2: 5 -> 3 outputs, window offset -1
    x = np.arange(25, dtype=np.float32).reshape(1, 1, 5, 5)
    y, idx = oracle.maxpool_forward(ob.MODE_MTCS, x, 3, 2, 2, 2)
    assert y.shape == (1, 1, 3, 3) and y[0, 0, 0, 0] == 6 and y[0, 0, 2, 2] == 24
    # a window that only sees -inf inputs keeps index -1 (MTCS pad value -inf, strict '>')
    x = np.full((1, 1, 2, 2), -np.inf, np.float32)
    y, idx = oracle.maxpool_forward(ob.MODE_MTCS, x, 2, 2, 2, 1)
    assert idx[0, 0, 0, 0] == -1 and np.isneginf(y[0, 0, 0, 0])
    y, idx = oracle.maxpool_forward(ob.MODE_CPU, x, 2, 2, 2, 1)
    assert idx[0, 0, 0, 0] == -1 and y[0, 0, 0, 0] == -np.finfo(np.float32).max


def test_avgpool(oracle):
    x = np.arange(2 * 3 * 4, dtype=np.float32).reshape(2, 3, 2, 2)
    y = oracle.avgpool_forward(x)
    assert np.allclose(y, x.reshape(2, 3, 4).mean(-1))
    pd = oracle.avgpool_backward(np.ones((2, 3), np.float32), np.ones_like(x))
    assert np.allclose(pd, 1.25)                                   # adds delta / (H*W)


def test_softmax_xent_against_fixture(oracle):
    for mode in (ob.MODE_CPU, ob.MODE_MTCS):
        r = oracle.softmax_forward(mode, G["sm_x"], G["sm_truth"])
        assert rel_l2(r["p"], G["sm_p"]) < 2e-6
        assert abs(r["cost"] - float(G["sm_cost"])) < 1e-4 * abs(float(G["sm_cost"]))
        assert rel_l2(r["delta"], -G["sm_dx"]) < 2e-6             # the reference stores the NEGATIVE gradient t - p
        assert np.count_nonzero(r["loss"]) == 6
    g2 = oracle.softmax_forward(ob.MODE_CPU, G["sm_x"], None, groups=2)
    assert np.allclose(g2["p"].reshape(6, 2, 5).sum(-1), 1.0, atol=1e-6)


def test_dropout_shares_mask(oracle):
    x = np.ones(8, np.float32)
    r = np.array([0.1, 0.49, 0.5, 0.9, 0.0, 0.51, 0.3, 0.7], np.float32)
    assert np.array_equal(oracle.dropout_forward(x, r, 0.5), [0, 0, 2, 2, 0, 2, 0, 2])


def test_sgd_three_steps_closed_form(oracle):
    lr, mom, decay, B = (float(v) for v in G["sgd_h"])
    w, u = G["sgd_w0"].astype(np.float32), np.zeros(50, np.float32)
    for g in G["sgd_g"]:
        u = u + g.astype(np.float32)
        w, u = oracle.sgd_weights(w, u, int(B), lr, mom, decay)
    assert rel_l2(w, G["sgd_w"]) < 1e-6 and rel_l2(u, G["sgd_u"]) < 1e-6
    p, up = oracle.sgd_plain(np.ones(4), np.full(4, 2.0), 2, 0.5, 0.9)
    assert np.allclose(p, 1.5) and np.allclose(up, 1.8)


def _tiny_net_specs():
    return [dict(type=ob.CONV, filters=4, size=3, stride_x=1, stride_y=1, pad=1, batch_normalize=1, activation=ob.LEAKY),
            dict(type=ob.MAXPOOL, size=2, stride_x=2, stride_y=2, pad=1),
            dict(type=ob.CONV, filters=3, size=1, stride_x=1, stride_y=1, pad=0, batch_normalize=0, activation=ob.LINEAR),
            dict(type=ob.AVGPOOL), dict(type=ob.SOFTMAX, groups=1, temperature=1.0)]


def test_network_gradient_by_finite_differences(oracle64, aet):
    """dLoss/dW of the whole oracle network (MTCS formulas) against central differences."""
    import aet_cnn_b200.synth as synth
    net = oracle64.net(_tiny_net_specs(), 3, 2, 6, 6, mode=ob.MODE_MTCS)
    x = synth.uniform((3, 2, 6, 6), 5, 1)
    _, truth = synth.labels(3, 3, 5, 2)
    w0 = synth.normal((4 * 2 * 9,), 5, 3, 0, 0.4)
    w2 = synth.normal((3 * 4,), 5, 4, 0, 0.4)
    net.set_param(0, ob.P_WEIGHTS, w0)
    net.set_param(2, ob.P_WEIGHTS, w2)
    net.forward(x, truth)
    net.backward(x)
    g0 = net.param(0, ob.P_WEIGHT_UPDATES).copy()    # holds sum(t - p)-driven NEGATIVE gradient
    g2 = net.param(2, ob.P_WEIGHT_UPDATES).copy()

    def loss_at(layer, w):
        net.set_param(layer, ob.P_WEIGHTS, w)
        net.forward(x, truth)
        return float(net.cost())

    eps = 2e-3
    for layer, w, g in ((0, w0, g0), (2, w2, g2)):
        for i in range(0, w.size, 7):
            wp, wm = w.copy(), w.copy()
            wp[i] += eps
            wm[i] -= eps
            fd = (loss_at(layer, wp) - loss_at(layer, wm)) / (2 * eps)
            assert abs(-g[i] - fd) < 2e-2 * max(1.0, abs(fd)), (layer, i, g[i], fd)
        net.set_param(layer, ob.P_WEIGHTS, w)


def test_network_train_step_lowers_loss_and_threads_agree(oracle, aet):
    import aet_cnn_b200.synth as synth
    losses = {}
    for threads in (1, 3):
        net = oracle.net(_tiny_net_specs(), 6, 2, 6, 6, mode=ob.MODE_MTCS, threads=threads)
        net.set_param(0, ob.P_WEIGHTS, synth.normal((72,), 5, 3, 0, 0.4))
        net.set_param(2, ob.P_WEIGHTS, synth.normal((12,), 5, 4, 0, 0.4))
        x = synth.uniform((6, 2, 6, 6), 5, 1)
        _, truth = synth.labels(6, 3, 5, 2)
        losses[threads] = [net.train_step(x, truth, 0.05, 0.9, 5e-4) for _ in range(8)]
    assert losses[1][-1] < losses[1][0]
    assert np.allclose(losses[1], losses[3], rtol=1e-4)


def test_learning_rate_schedule_known_values(oracle):
    """NNetwork.getCurrentRate (dnn/NNetwork.c:215-246) on hand-computed points."""
    lr = 0.1
    assert oracle.current_rate(7, 0, lr) == pytest.approx(0.1)
    assert oracle.current_rate(2, 0, lr, burn_in=4, power=2.0) == pytest.approx(0.1 * (2 / 4) ** 2)
    assert oracle.current_rate(7, 1, lr, step=3, scale=0.5) == pytest.approx(0.1 * 0.5 ** 2)          # 7 / 3 = 2
    assert oracle.current_rate(5, 2, lr, steps=(2, 5, 7), scales=(0.5, 0.1, 2.0)) == pytest.approx(0.1 * 0.5 * 0.1)
    assert oracle.current_rate(1, 2, lr, steps=(2, 5, 7), scales=(0.5, 0.1, 2.0)) == pytest.approx(0.1)
    assert oracle.current_rate(3, 3, lr, gamma=0.9) == pytest.approx(0.1 * 0.9 ** 3)
    assert oracle.current_rate(5, 4, lr, max_batches=20, power=3.0) == pytest.approx(0.1 * (1 - 5 / 20) ** 3)
    assert oracle.current_rate(6, 5, lr, gamma=0.7, step=4) == pytest.approx(0.1 / (1 + np.exp(0.7 * 2)))
    # batch_num - step is unsigned in the reference: below `step` it wraps, exp overflows and the rate is 0
    assert oracle.current_rate(2, 5, lr, gamma=0.7, step=4) == 0.0


def test_non_finite_scrub_known_values(oracle):
    v = np.array([1.0, np.nan, -np.inf, 2.0], np.float32)
    assert np.array_equal(oracle.reset_nan_and_inf(v), np.array([1.0, 0.0, 0.0, 2.0], np.float32))
    assert np.array_equal(oracle.fix_nan_and_inf(v), np.array([1.0, 0.5, 1.0 / 3.0, 2.0], np.float32))


def test_inference_helpers_known_values(oracle):
    """fuseConvBatchnorm, topK and transposeMatrix on hand-computed cases."""
    b, w = oracle.fuse_conv_batchnorm([1.0, -2.0], [2.0, 0.5], [0.5, 1.0], [3.99999, 0.24999], np.array([[1.0, 2.0], [4.0, -8.0]], np.float32))
    assert np.allclose(b, [1.0 - 2.0 * 0.5 / 2.0, -2.0 - 0.5 * 1.0 / 0.5], rtol=1e-6)
    assert np.allclose(w, [[1.0, 2.0], [4.0, -8.0]], rtol=1e-6)              # scale / sqrt(var + 1e-5) = 1 for both filters
    assert list(oracle.top_k(np.array([0.1, 0.7, 0.05, 0.15], np.float32), 2)) == [1, 3]
    assert list(oracle.top_k(np.array([0.2, 0.2, 0.6], np.float32), 3)) == [2, 1, 0]      # a displaced entry falls behind its equals
    assert list(oracle.transpose_matrix([1, 2, 3, 4, 5, 6], 2, 3)) == [1, 4, 2, 5, 3, 6]


def test_shortcut_known_values(oracle):
    """ShortcutLayer without weights (dnn/ShortcutLayer.c:272-353, :132-230): sources are added over the flat per-sample
    index range they have, so a narrower source reaches only the first channels; backward adds the delta to the
    previous delta and to every source's delta over the same range."""
    x = np.arange(12, dtype=np.float32).reshape(2, 6)
    wide = 10 * np.ones((2, 8), np.float32)
    narrow = np.array([[1, 2, 3], [4, 5, 6]], np.float32)
    out = oracle.shortcut_forward(x, [wide, narrow])
    want = x + 10
    want[:, :3] += narrow
    assert np.array_equal(out, want)
    delta = np.arange(12, dtype=np.float32).reshape(2, 6) + 1
    pd = np.ones((2, 6), np.float32)
    dw, dn = np.zeros((2, 8), np.float32), np.full((2, 3), 2, np.float32)
    oracle.shortcut_backward(delta, pd, [dw, dn])
    assert np.array_equal(pd, delta + 1)
    assert np.array_equal(dw[:, :6], delta) and np.all(dw[:, 6:] == 0)
    assert np.array_equal(dn, delta[:, :3] + 2)


def test_residual_network_gradient_by_finite_differences(oracle64):
    """A residual block (conv, conv, shortcut from the first conv) through the whole-network oracle: the shortcut's
    output is activation(conv 2 + conv 1), and the weight gradient of the convolution behind the block agrees with
    central differences of the cost (the block's forward is what the differences exercise)."""
    from oracle import cfgfile
    text = """[net]
batch=2
height=4
width=4
channels=2
[convolutional]
filters=4
size=3
stride=1
pad=1
activation=leaky
[convolutional]
filters=4
size=3
stride=1
pad=1
activation=leaky
[shortcut]
from=-2
activation=leaky
[convolutional]
filters=3
size=1
stride=1
pad=0
activation=linear
[avgpool]
[softmax]
"""
    opts, specs = cfgfile.network_spec(text, 2)
    assert specs[2]["type"] == cfgfile.SHORTCUT and specs[2]["from"] == [0]
    net = oracle64.net(specs, 2, 2, 4, 4)
    rng = np.random.default_rng(5)
    for i in (0, 1, 3):
        w = net.param(i, ob.P_WEIGHTS)
        net.set_param(i, ob.P_WEIGHTS, rng.normal(0, .5, w.shape).astype(np.float32))
    x = rng.uniform(0, 1, (2, 2, 4, 4)).astype(np.float32)
    truth = np.zeros((2, 3), np.float32); truth[0, 1] = truth[1, 2] = 1
    net.forward(x, truth); net.backward(x)
    # forward: the shortcut's output is leaky(conv2 + conv1)
    o0, o1, o2 = (net.param(i, ob.P_OUTPUT).astype(np.float64) for i in (0, 1, 2))
    pre = o0 + o1
    assert np.allclose(o2, np.where(pre > 0, pre, .1 * pre), atol=1e-6)
    # backward on the unaffected last convolution: central differences of the cost
    g = net.param(3, ob.P_WEIGHT_UPDATES).copy()
    w3 = net.param(3, ob.P_WEIGHTS).copy()
    eps = 1e-3
    for k in range(0, w3.size, 5):
        wp, wm = w3.copy(), w3.copy()
        wp.flat[k] += eps; wm.flat[k] -= eps
        net.set_param(3, ob.P_WEIGHTS, wp); net.forward(x, truth); cp = net.cost()
        net.set_param(3, ob.P_WEIGHTS, wm); net.forward(x, truth); cm = net.cost()
        num = (cp - cm) / (2 * eps)
        # weight_updates accumulate the NEGATIVE gradient of the cost (the update adds them)
        assert abs(-g.flat[k] - num) < 2e-3 * max(1.0, abs(num)), (k, g.flat[k], num)
    net.set_param(3, ob.P_WEIGHTS, w3)


def test_swish_and_mish_known_values(oracle):
    """swish = v * sigmoid(v), mish = v * tanh(softplus(v)) (dnn/IOData.c:75-105) and their gradients
    (dnn/Activation.c:303-330) against float64 closed forms and central differences."""
    v = np.linspace(-6, 6, 49).astype(np.float32)
    v64 = v.astype(np.float64)
    sig = 1 / (1 + np.exp(-v64))
    sp = np.log1p(np.exp(v64))
    want = {ob.SWISH: v64 * sig, ob.MISH: v64 * np.tanh(sp)}
    for act in (ob.SWISH, ob.MISH):
        for mode in (ob.MODE_MTCS, ob.MODE_CPU):
            y = oracle.activate(v.copy(), act, mode)
            assert np.allclose(y, want[act], rtol=2e-6, atol=2e-6), act
        eps = 1e-4
        f = (lambda t: t / (1 + np.exp(-t))) if act == ob.SWISH else (lambda t: t * np.tanh(np.log1p(np.exp(t))))
        num = (f(v64 + eps) - f(v64 - eps)) / (2 * eps)
        g = oracle.gradient_input(oracle.activate(v.copy(), act, ob.MODE_MTCS), v, act, np.ones_like(v))
        assert np.allclose(g, num, rtol=1e-4, atol=1e-5), act
    # the thresholds of softplus (dnn/Activation.h:108-113): above 20 the input passes through, below -20 it is exp(v),
    # whose tanh the reference's float formula 2 / (1 + expf(-2x)) - 1 rounds to zero
    big = oracle.activate(np.array([25.0, -25.0], np.float32), ob.MISH, ob.MODE_MTCS)
    assert big[0] == 25.0 and abs(big[1]) < 1e-9


def test_stopbackward_freezes_the_front_and_dont_update_holds_a_layer(oracle):
    """dnn/NetworkFactory.c:883-896,979-991 and dnn/NNetwork.c:648-651,667-709: layers in front of the last stopbackward
    layer never change; that layer sees no gradient but is still updated, so each step multiplies in the momentum-fed
    decay: after one step W' = W * (1 - lr * decay); dont_update = 1 holds a trained layer for the first iteration of
    the GPU update loop and releases the accumulated gradient on the second; the CPU loop does not know the key."""
    from oracle import cfgfile
    text = ("[net]\nbatch=4\nheight=6\nwidth=6\nchannels=2\nlearning_rate=0.1\nmomentum=0.9\ndecay=0.01\n"
            "[convolutional]\nfilters=3\nsize=3\nstride=1\npad=1\nactivation=leaky\n"
            "[convolutional]\nfilters=3\nsize=3\nstride=1\npad=1\nactivation=leaky\nstopbackward=1\n"
            "[convolutional]\nfilters=4\nsize=3\nstride=1\npad=1\nactivation=leaky\ndont_update=1\n"
            "[convolutional]\nfilters=3\nsize=1\nstride=1\npad=0\nactivation=linear\n[avgpool]\n[softmax]\n")
    opts, specs = cfgfile.network_spec(text)
    rng = np.random.default_rng(3)
    for mode in (ob.MODE_MTCS, ob.MODE_CPU):
        net = oracle.net(specs, 4, 2, 6, 6, mode=mode)
        start, cin = {}, 2
        for i, s in enumerate(specs):
            if s["type"] == cfgfile.CONV:
                start[i] = rng.normal(0, 0.4, (s["filters"], cin, s["size"], s["size"])).astype(np.float32)
                net.set_param(i, ob.P_WEIGHTS, start[i])
                start[i] = start[i].ravel()
                cin = s["filters"]
        x = rng.uniform(-1, 1, (4, 2, 6, 6)).astype(np.float32)
        t = np.eye(3, dtype=np.float32)[[0, 1, 2, 1]]
        net.train_step(x, t, 0.1, 0.9, 0.01)
        assert np.array_equal(net.param(0, ob.P_WEIGHTS), start[0])
        np.testing.assert_allclose(net.param(1, ob.P_WEIGHTS), start[1] * np.float32(1 - 0.1 * 0.01), rtol=1e-6)
        assert np.array_equal(net.param(2, ob.P_WEIGHTS), start[2]) == (mode == ob.MODE_MTCS)
        assert not np.array_equal(net.param(3, ob.P_WEIGHTS), start[3])
        pending = net.param(2, ob.P_WEIGHT_UPDATES).copy()
        if mode == ob.MODE_MTCS:
            assert np.any(pending)                     # the gradient of the held step waits in weight_updates
        net.train_step(x, t, 0.1, 0.9, 0.01)
        assert not np.array_equal(net.param(2, ob.P_WEIGHTS), start[2])
        assert np.array_equal(net.param(0, ob.P_WEIGHTS), start[0]) and not np.any(net.param(0, ob.P_WEIGHT_UPDATES))


@pytest.mark.parametrize("shape", [(2, 3, 23, 23, 5, 11, 4, 0), (2, 3, 17, 21, 4, 7, 2, 3), (1, 1, 20, 20, 3, 6, 3, 1)])
def test_strided_convolution_equals_its_regrouped_stride_one_form(oracle, shape):
    """The algebra behind the device library's treatment of large strided first-layer filters, on the oracle alone:
    with the (zero-padded) input regrouped into s x s pixel blocks and the filter likewise, a stride-s convolution is
    a ceil(R/s) x ceil(R/s) stride-1 convolution without padding over s*s*C channels - the same products plus zeros -
    and the real weight gradient is a gather from the regrouped layer's, every tap exactly once."""
    n, c, h, w, k, size, s, pad = shape
    rng = np.random.default_rng(size)
    x = rng.uniform(-1, 1, (n, c, h, w)).astype(np.float32)
    wt = rng.normal(0, 0.3, (k, c, size, size)).astype(np.float32)
    y = oracle.conv_forward(x, wt, s, s, pad)
    oh, ow = y.shape[2:]
    rb = (size + s - 1) // s
    hb, wb = oh + rb - 1, ow + rb - 1
    xp = np.zeros((n, c, hb * s, wb * s), np.float32)        # padded on every side, cut to whole blocks
    hh, ww = min(h, hb * s - pad), min(w, wb * s - pad)
    xp[:, :, pad:pad + hh, pad:pad + ww] = x[:, :, :hh, :ww]
    # xb[n][(dy*s + dx)*C + ch][by][bx] = xp[n][ch][by*s + dy][bx*s + dx]
    xb = xp.reshape(n, c, hb, s, wb, s).transpose(0, 3, 5, 1, 2, 4).reshape(n, s * s * c, hb, wb)
    wp = np.zeros((k, c, rb * s, rb * s), np.float32)
    wp[:, :, :size, :size] = wt
    wbk = wp.reshape(k, c, rb, s, rb, s).transpose(0, 3, 5, 1, 2, 4).reshape(k, s * s * c, rb, rb)
    yb = oracle.conv_forward(np.ascontiguousarray(xb), np.ascontiguousarray(wbk), 1, 1, 0)
    assert yb.shape == y.shape
    np.testing.assert_allclose(yb, y, rtol=1e-5, atol=1e-5)
    d = rng.normal(0, 1, y.shape).astype(np.float32)
    dw, _ = oracle.conv_backward(x, wt, d, s, s, pad, need_dx=False)
    dwb, _ = oracle.conv_backward(np.ascontiguousarray(xb), np.ascontiguousarray(wbk), d, 1, 1, 0, need_dx=False)
    fold = dwb.reshape(k, s, s, c, rb, rb).transpose(0, 3, 4, 1, 5, 2).reshape(k, c, rb * s, rb * s)[:, :, :size, :size]
    np.testing.assert_allclose(fold, dw, rtol=1e-4, atol=1e-4)
