"""Whole-network parity on the GPU: the CIFAR-shaped small CNN trained for several SGD steps through
the C ABI against the CPU oracle (loss curve and every parameter), CUDA-graph replay against eager
execution (bitwise), the Darknet .weights container, and the reduced AlexNet-style step."""
import os
import tempfile

import numpy as np
import pytest

from conftest import rel_l2
from oracle import binding as ob

pytestmark = pytest.mark.gpu

PARAMS = ["P_WEIGHTS", "P_BIASES", "P_SCALES", "P_ROLLING_MEAN", "P_ROLLING_VARIANCE", "P_WEIGHT_UPDATES"]


def build_pair(aet, ctx, oracle, cfg_name, batch, mode=ob.MODE_MTCS, seed=20241, threads=1):
    from oracle import cfgfile
    import aet_cnn_b200.synth as synth
    text = open(os.path.join(aet.CFG_DIR, cfg_name)).read()
    ctx.set_parity(mode)
    net = aet.NNetwork(ctx, cfg_text=text, train=1, batch=batch)
    opts, specs = cfgfile.network_spec(text, batch)
    onet = oracle.net(specs, batch, opts["c"], opts["h"], opts["w"], mode=mode, threads=threads)
    cin = opts["c"]
    for i, s in enumerate(specs):
        if s["type"] != cfgfile.CONV:
            continue
        k, size = s["filters"], s["size"]
        w = synth.normal((k, cin, size, size), seed, 1000 + i, 0.0, float(np.sqrt(2.0 / (size * size * cin))))
        net.layer(i).write(aet.P_WEIGHTS, w)
        onet.set_param(i, ob.P_WEIGHTS, w)
        cin = k
    return net, onet, opts, specs


def batch_for(opts, classes, batch, seed, step):
    import aet_cnn_b200.synth as synth
    x = synth.uniform((batch, opts["c"], opts["h"], opts["w"]), seed, 2 * step)
    _, truth = synth.labels(batch, classes, seed, 2 * step + 1)
    return x, truth


@pytest.mark.parametrize("mode", [ob.MODE_MTCS, ob.MODE_CPU])
def test_small_cnn_training_matches_oracle(aet, ctx, oracle64, mode):
    """3xTF32 math, six SGD steps.  The first forward pass (continuous functions only) must agree to
    1e-5.  After that the network is a chaotic map of piecewise functions (leaky kinks, max-pool
    argmax): a value that lands on the other side of a kink changes one gradient element tenfold, so
    whole-network gradients are compared at 5e-2 and the loss curve at 2e-3; op-level parity on
    identical inputs (test_gpu_conv.py, test_gpu_ops.py and the layerwise test below) is the tight one."""
    batch, steps = 16, 6
    ctx.set_math(aet.MATH_3XTF32)
    try:
        net, onet, opts, specs = build_pair(aet, ctx, oracle64, "cifar_small.cfg", batch, mode)
        x, truth = batch_for(opts, 10, batch, 20241, 0)
        net.input.write(x); net.truth.write(truth)
        net.forward(aet.make_state(input=net.input, truth=net.truth, train=1))
        onet.forward(x, truth)
        for i in range(net.layer_count):
            err = rel_l2(net.layer(i).read(aet.P_OUTPUT), onet.param(i, ob.P_OUTPUT))
            assert err < 1e-5, ("forward", i, err)
        assert abs(net.cost() - onet.cost()) < 1e-5 * abs(onet.cost())
        # rebuild both so that the rolling statistics start from zero again
        net.close()
        net, onet, opts, specs = build_pair(aet, ctx, oracle64, "cifar_small.cfg", batch, mode)
        worst = {}
        for step in range(steps):
            x, truth = batch_for(opts, 10, batch, 20241, step)
            loss = net.train(x, truth)
            oloss = onet.train_step(x, truth, opts["learning_rate"], opts["momentum"], opts["decay"])
            assert abs(loss - oloss) <= 2e-3 * abs(oloss), (step, loss, oloss)
            if step in (0, steps - 1):
                for i, s in enumerate(specs):
                    for pname in PARAMS:
                        ref = onet.param(i, getattr(ob, pname))
                        if ref is None or not np.any(ref):
                            continue
                        err = rel_l2(net.layer(i).read(getattr(aet, pname)), ref)
                        worst[pname] = max(worst.get(pname, 0.0), err)
                        # momentum buffers and the BN shifts (which start at zero) are small differences of
                        # large sums: looser than the weights themselves
                        tol = 1e-1 if pname.endswith("UPDATES") or pname == "P_BIASES" else 1e-2
                        assert err < tol, (step, i, pname, err)
        print("worst relative L2 after %d steps:" % steps, worst)
        ctx.check()
        net.close()
    finally:
        ctx.set_math(aet.MATH_TF32)
        ctx.set_parity(ob.MODE_MTCS)


# code path of every TMA convolution launch of the small CNN at the benchmark batch on a 148-SM part
BENCH_VARIANTS = {"conv_fprop_tma#2", "conv_dgrad_tma_rows.sm_mt2_n192x1#2", "conv_wgrad_tma_rows.n64_sp49#2",
                  "conv_fprop_tma#4", "conv_dgrad_tma_rows.mt1_n128x1_ks2#4", "conv_wgrad_tma_rows.n128_sp24#4"}


@pytest.mark.parametrize("batch", [16, 128])
def test_small_cnn_tf32_first_step_layerwise(aet, ctx, oracle, batch):
    """Default TF32 math on the whole network: activations and batch statistics within 1e-2 of the FP32
    oracle, and every convolution's backward kernels within 1e-2 when the oracle is given the SAME inputs
    the device kernels consumed (the layer's input activations and its post-BN-backward delta).  Batch 128
    is the benchmark's: the launchers pick other code paths there than at 16, asserted by their labels."""
    from oracle import cfgfile
    from gpu_util import oracle_conv_backward_mt
    net, onet, opts, specs = build_pair(aet, ctx, oracle, "cifar_small.cfg", batch, threads=os.cpu_count() or 1)
    x, truth = batch_for(opts, 10, batch, 7, 0)
    net.input.write(x); net.truth.write(truth)
    ctx.profile(1)
    net.forward(aet.make_state(input=net.input, truth=net.truth, train=1))
    net.backward(aet.make_state(input=net.input, truth=net.truth, train=1))
    labels = {r["name"] for r in ctx.profile_read()}
    ctx.profile(0)
    if batch == 128:
        assert BENCH_VARIANTS <= labels, sorted(labels)
    onet.forward(x, truth)
    onet.backward(x)
    ctx.check()
    for i in range(net.layer_count):
        got = net.layer(i).read(aet.P_OUTPUT)
        assert rel_l2(got, onet.param(i, ob.P_OUTPUT)) < 1e-2, i
        if specs[i]["type"] == cfgfile.CONV and specs[i]["batch_normalize"]:
            # statistics gathered by the convolution's epilogue (two partial rows per CTA at batch 128)
            assert rel_l2(net.layer(i).read(aet.P_MEAN), onet.param(i, ob.P_MEAN)) < 1e-2, i
            assert rel_l2(net.layer(i).read(aet.P_VARIANCE), onet.param(i, ob.P_VARIANCE)) < 1e-2, i
    assert abs(net.cost() - onet.cost()) < 1e-2 * abs(onet.cost())
    # the softmax delta's support (the labels) is integer data: exact
    assert np.array_equal(net.layer(8).read(aet.P_LOSS) != 0, onet.param(8, ob.P_LOSS) != 0)
    cin, hin, win = opts["c"], opts["h"], opts["w"]
    shapes = []
    for i, s in enumerate(specs):
        oc, oh, ow = net.layer(i).out_shape
        shapes.append((cin, hin, win, oc, oh, ow))
        cin, hin, win = oc, oh, ow
    for i, s in enumerate(specs):
        if s["type"] != cfgfile.CONV:
            continue
        c, h, w, oc, oh, ow = shapes[i]
        xin = x if i == 0 else net.layer(i - 1).read(aet.P_OUTPUT).reshape(batch, c, h, w)
        delta = net.layer(i).read(aet.P_DELTA).reshape(batch, oc, oh, ow)      # as consumed by wgrad / dgrad
        wts = net.layer(i).read(aet.P_WEIGHTS).reshape(oc, c, s["size"], s["size"])
        dw, dx = oracle_conv_backward_mt(oracle, xin, wts, delta, s["stride_x"], s["pad"], need_dx=i > 0)
        assert rel_l2(net.layer(i).read(aet.P_WEIGHT_UPDATES), dw) < 1e-2, ("wgrad", i)
        if i > 0:
            assert rel_l2(net.layer(i - 1).read(aet.P_DELTA), dx) < 1e-2, ("dgrad", i)
        # coarse whole-network agreement (kink / argmax flips upstream change ~sqrt(flip fraction) of it)
        assert rel_l2(net.layer(i).read(aet.P_WEIGHT_UPDATES), onet.param(i, ob.P_WEIGHT_UPDATES)) < 0.2, i
    net.close()


def test_small_cnn_100_steps_at_batch_128_track_the_oracle(aet, ctx):
    """The reference's small-CNN training case at its stated size: batch 128, 100 SGD steps (lr 0.1, momentum 0.9,
    decay 5e-4), a fresh synthetic batch every step, default TF32 math with CUDA-graph replay, against the CPU
    oracle (its timing build on all host cores: same formulas, summation order as the compiler leaves it).
    After the first step (before the piecewise network has had time to amplify rounding) every parameter agrees
    within 1e-2.  Over the run the two trajectories are separate samples of a chaotic map (leaky kinks, argmax
    flips), so the loss curves are compared as curves: every step within 2 % of the oracle's loss, the mean
    relative difference over the 100 steps within 0.2 % (measured: 0.24 % at the worst step, 0.02 % mean)."""
    from oracle import cfgfile
    batch, steps = 128, 100
    fast = ob.Oracle("fast")
    net, onet, opts, specs = build_pair(aet, ctx, fast, "cifar_small.cfg", batch, threads=os.cpu_count() or 1)
    net.use_graph(True)
    gl, ol = [], []
    for step in range(steps):
        x, truth = batch_for(opts, 10, batch, 20241, step)
        gl.append(net.train(x, truth))
        ol.append(onet.train_step(x, truth, opts["learning_rate"], opts["momentum"], opts["decay"]))
        if step == 0:
            for i, s in enumerate(specs):
                if s["type"] != cfgfile.CONV:
                    continue
                for pname in ("P_WEIGHTS", "P_SCALES", "P_ROLLING_MEAN", "P_ROLLING_VARIANCE"):
                    ref = onet.param(i, getattr(ob, pname))
                    if ref is None or not np.any(ref):
                        continue
                    err = rel_l2(net.layer(i).read(getattr(aet, pname)), ref)
                    assert err < 1e-2, (i, pname, err)
    ctx.check()
    gl, ol = np.array(gl), np.array(ol)
    rel = np.abs(gl - ol) / np.abs(ol)
    print("100-step loss curve: first %.4f/%.4f last %.4f/%.4f, max rel diff %.3e at step %d, mean rel diff %.3e"
          % (gl[0], ol[0], gl[-1], ol[-1], rel.max(), int(rel.argmax()), rel.mean()))
    assert np.isfinite(gl).all()
    assert rel[0] < 1e-3
    assert rel.max() < 0.02 and rel.mean() < 0.002
    net.close()


def test_graph_replay_is_bitwise_identical_to_eager(aet, ctx, oracle):
    batch, steps = 8, 5
    hashes = []
    for use_graph in (False, True):
        net, _, opts, _ = build_pair(aet, ctx, oracle, "cifar_small.cfg", batch)
        net.use_graph(use_graph)
        losses = []
        for step in range(steps):
            x, truth = batch_for(opts, 10, batch, 3, step)
            losses.append(net.train(x, truth))
        hashes.append((net.param_hash(), tuple(losses)))
        assert net.launches_per_step() > 20
        ctx.check()
        net.close()
    assert hashes[0] == hashes[1]


def _run_variant(aet, ctx, oracle, options):
    """One forward + backward + two more training steps of the small CNN (batch 8) with the context `options`
    (name -> value) in force while the network is built."""
    batch, steps = 8, 3
    saved = {k: ctx.get_option(k) for k in options}
    for k, v in options.items():
        ctx.set_option(k, v)
    try:
        net, _, opts, specs = build_pair(aet, ctx, oracle, "cifar_small.cfg", batch)
    finally:
        for k, v in saved.items():
            ctx.set_option(k, v)
    x, truth = batch_for(opts, 10, batch, 3, 0)
    net.input.write(x); net.truth.write(truth)
    net.forward(aet.make_state(input=net.input, truth=net.truth, train=1))
    net.backward(aet.make_state(input=net.input, truth=net.truth, train=1))
    outs = [net.layer(i).read(aet.P_OUTPUT) for i in range(net.layer_count)]   # conv outputs are formed lazily
    idx = [net.layer(i).read(aet.P_INDEXES) for i in (1, 3, 5)]
    grads = [net.layer(i).read(aet.P_WEIGHT_UPDATES) for i in (0, 2, 4, 6)]
    bgrads = [net.layer(6).read(aet.P_BIAS_UPDATES)]
    sgrads = [net.layer(i).read(aet.P_SCALE_UPDATES) for i in (0, 2, 4)]
    deltas = [net.layer(i).read(aet.P_DELTA) for i in (0, 2, 4, 5, 6, 7)]
    net.update()
    losses = [net.train(*batch_for(opts, 10, batch, 3, step)) for step in range(1, steps)]
    res = dict(outs=outs, idx=idx, grads=grads, bgrads=bgrads, sgrads=sgrads, deltas=deltas, losses=losses,
               launches=net.launches_per_step())
    net.close()
    return res


def test_fused_bn_pool_path_matches_layer_by_layer(aet, ctx, oracle):
    """Inside a network a BN convolution produces the following max-pool's output itself and folds the
    pool's backward into its BN backward kernels; the context option "fuse" = 0 runs every layer's own kernels instead.
    Forward results are bit-identical; gradients differ only by summation order.  (The linear classifier
    head and the first layer's pool-sized backward are switched off in both runs: they change the arithmetic and
    have their own tests below.)"""
    f = _run_variant(aet, ctx, oracle, {"linear_head": 0, "stem": 0})
    u = _run_variant(aet, ctx, oracle, {"fuse": 0})
    for a, b in zip(f["outs"], u["outs"]):
        assert np.array_equal(a, b)
    for a, b in zip(f["idx"], u["idx"]):
        assert np.array_equal(a, b)
    for key in ("grads", "bgrads", "sgrads", "deltas"):
        for a, b in zip(f[key], u[key]):
            assert rel_l2(a, b) < 2e-4, (key, rel_l2(a, b))   # FP32 partial sums grouped differently
    assert np.allclose(f["losses"], u["losses"], rtol=1e-4)
    assert f["launches"] < u["launches"]          # fewer launches when fused


STEM_CFG = """[net]
batch={batch}
width={w}
height={h}
channels={c}
learning_rate=0.1
momentum=0.9
decay=0.0005
policy=constant
max_batches=1000

[convolutional]
filters={k}
size=3
stride=1
pad=1
batch_normalize=1
activation={act}

[maxpool]
size=2
stride=2

[convolutional]
filters=10
size=1
stride=1
pad=0
activation=linear

[avgpool]

[softmax]
groups=1
"""


@pytest.mark.parametrize("batch,c,h,w,k,act,mode", [
    (128, 3, 32, 32, 64, "leaky", ob.MODE_MTCS),     # the benchmark network's first layer
    (5, 3, 24, 40, 64, "relu", ob.MODE_MTCS),        # ragged: rows not a multiple of the Gram strip, non-square
    (7, 1, 16, 16, 64, "leaky", ob.MODE_CPU),        # one input channel, the CPU classes' formulas
    (3, 2, 10, 6, 128, "logistic", ob.MODE_MTCS),    # 512 threads per block, a slow-path activation
    (2, 3, 8, 80, 64, "leaky", ob.MODE_MTCS),        # three chunks of windows per pool row, the last one partial
    (4, 3, 12, 12, 64, "mish", ob.MODE_MTCS),        # gradient from the value before the activation
])
def test_first_layer_pool_sized_backward(aet, ctx, oracle64, batch, c, h, w, k, act, mode):
    """The first convolution (BN, fused 2x2 max-pool) takes its scale / shift / weight gradients from the pool-sized
    tensors and the Gram matrix of the input patches instead of forming the full-resolution delta.  Against the FP64
    oracle and against the general path (option "stem" = 0), 3xTF32 math: the same gradients to 2e-5 of their norm;
    the delta a host tap reads afterwards is the general path's."""
    from oracle import cfgfile
    import aet_cnn_b200.synth as synth
    text = STEM_CFG.format(batch=batch, c=c, h=h, w=w, k=k, act=act)
    ctx.set_math(aet.MATH_3XTF32)
    ctx.set_parity(mode)
    x = synth.uniform((batch, c, h, w), 77, 0)
    _, truth = synth.labels(batch, 10, 77, 1)
    w0 = synth.normal((k, c, 3, 3), 77, 2, 0.0, float(np.sqrt(2.0 / (9 * c))))
    w1 = synth.normal((10, k, 1, 1), 77, 3, 0.0, float(np.sqrt(2.0 / k)))
    res = {}
    try:
        for stem in (1, 0):
            ctx.set_option("stem", stem)
            net = aet.NNetwork(ctx, cfg_text=text, train=1, batch=batch)
            ctx.set_option("stem", 1)
            net.layer(0).write(aet.P_WEIGHTS, w0)
            net.layer(2).write(aet.P_WEIGHTS, w1)
            net.input.write(x); net.truth.write(truth)
            ctx.profile(1)
            net.forward(aet.make_state(input=net.input, truth=net.truth, train=1))
            net.backward(aet.make_state(input=net.input, truth=net.truth, train=1))
            records = ctx.profile_read()
            ctx.profile(0)
            names = {r["name"].split(".")[0].split("#")[0] for r in records}
            full = [r["name"] for r in records]
            assert ("stem_bwd_sparse" in names) == bool(stem), sorted(names)
            assert any(n.startswith("conv_wgrad") and n.endswith("#0") for n in full) != bool(stem), sorted(full)
            res[stem] = {p: net.layer(0).read(getattr(aet, p)) for p in ("P_WEIGHT_UPDATES", "P_SCALE_UPDATES", "P_BIAS_UPDATES", "P_DELTA")}
            ctx.check()
            # a second pass accumulates on top of the first (the gradient arena is only cleared by the update)
            net.forward(aet.make_state(input=net.input, truth=net.truth, train=1))
            net.backward(aet.make_state(input=net.input, truth=net.truth, train=1))
            twice = net.layer(0).read(aet.P_WEIGHT_UPDATES)
            assert rel_l2(twice, 2 * res[stem]["P_WEIGHT_UPDATES"]) < 1e-5
            net.close()
    finally:
        ctx.set_option("stem", 1)
        ctx.set_math(aet.MATH_TF32)
        ctx.set_parity(ob.MODE_MTCS)
    opts, specs = cfgfile.network_spec(text, batch)
    onet = oracle64.net(specs, batch, c, h, w, mode=mode, threads=os.cpu_count() or 1)
    onet.set_param(0, ob.P_WEIGHTS, w0)
    onet.set_param(2, ob.P_WEIGHTS, w1)
    onet.forward(x, truth)
    onet.backward(x)
    for p in ("P_WEIGHT_UPDATES", "P_SCALE_UPDATES"):
        ref = onet.param(0, getattr(ob, p))
        assert rel_l2(res[1][p], ref) < 2e-5, (p, rel_l2(res[1][p], ref), rel_l2(res[0][p], ref))
        assert rel_l2(res[1][p], res[0][p]) < 2e-4, (p, rel_l2(res[1][p], res[0][p]))   # the general path's 3xTF32 GEMM is the looser one
    if mode == ob.MODE_MTCS:
        assert rel_l2(res[1]["P_BIAS_UPDATES"], res[0]["P_BIAS_UPDATES"]) < 2e-5
    assert rel_l2(res[1]["P_DELTA"], res[0]["P_DELTA"]) < 1e-5


RESNET_CFG = """[net]
batch={batch}
width=16
height=16
channels=3
learning_rate=0.05
momentum=0.9
decay=0.0005
policy=constant
max_batches=1000

[convolutional]
filters=32
size=3
stride=1
pad=1
batch_normalize=1
activation=leaky

[maxpool]
size=2
stride=2

[convolutional]
filters=32
size=3
stride=1
pad=1
batch_normalize=1
activation=leaky

[convolutional]
filters=32
size=3
stride=1
pad=1
batch_normalize=1
activation=linear

[shortcut]
from=-3
activation=leaky

[convolutional]
filters=64
size=3
stride=1
pad=1
batch_normalize=1
activation=leaky

[maxpool]
size=2
stride=2

[convolutional]
filters=20
size=1
stride=1
pad=0
activation=linear

[convolutional]
filters=24
size=1
stride=1
pad=0
activation=leaky

[shortcut]
from=6,-2
activation={act2}

[convolutional]
filters=10
size=1
stride=1
pad=0
activation=linear

[avgpool]

[softmax]
groups=1
"""


@pytest.mark.parametrize("act2", ["linear", "relu"])
def test_residual_network_matches_oracle(aet, ctx, oracle64, act2):
    """ResNet-style cfg: a shortcut over a two-convolution block (source = a max-pool layer), and a second shortcut with
    two sources, one with more channels than the layer (64 against 24: its first 24 are added) and one with fewer (20:
    it reaches the first 20 channels) (dnn/ShortcutLayer.c, dnn/NetworkFactory.c:175-246).  3xTF32 math against the FP64 oracle: every layer's output, the
    deltas the shortcuts write into their sources, every weight gradient, and four SGD steps of losses."""
    from oracle import cfgfile
    import aet_cnn_b200.synth as synth
    batch = 6
    text = RESNET_CFG.format(batch=batch, act2=act2)
    ctx.set_math(aet.MATH_3XTF32)
    try:
        net = aet.NNetwork(ctx, cfg_text=text, train=1, batch=batch)
        opts, specs = cfgfile.network_spec(text, batch)
        assert specs[4]["from"] == [1] and specs[9]["from"] == [6, 7]
        onet = oracle64.net(specs, batch, 3, 16, 16, threads=os.cpu_count() or 1)
        cin = 3
        for i, s in enumerate(specs):
            if s["type"] == cfgfile.CONV:
                w = synth.normal((s["filters"], cin, s["size"], s["size"]), 31, i, 0.0, float(np.sqrt(2.0 / (s["size"] ** 2 * cin))))
                net.layer(i).write(aet.P_WEIGHTS, w)
                onet.set_param(i, ob.P_WEIGHTS, w)
                cin = s["filters"]
        x = synth.uniform((batch, 3, 16, 16), 31, 100)
        _, truth = synth.labels(batch, 10, 31, 101)
        net.input.write(x); net.truth.write(truth)
        ctx.profile(1)
        net.forward(aet.make_state(input=net.input, truth=net.truth, train=1))
        net.backward(aet.make_state(input=net.input, truth=net.truth, train=1))
        names = {r["name"].split("#")[0] for r in ctx.profile_read()}
        ctx.profile(0)
        assert "shortcut_fwd" in names and "shortcut_bwd" in names, sorted(names)
        onet.forward(x, truth); onet.backward(x)
        ctx.check()
        for i in range(net.layer_count):
            assert rel_l2(net.layer(i).read(aet.P_OUTPUT), onet.param(i, ob.P_OUTPUT)) < 2e-5, ("output", i)
        for i in (1, 3, 4, 6, 7, 8, 9):   # the sources' deltas and the shortcuts' own
            assert rel_l2(net.layer(i).read(aet.P_DELTA), onet.param(i, ob.P_DELTA)) < 2e-4, ("delta", i)
        for i, s in enumerate(specs):
            if s["type"] == cfgfile.CONV:
                assert rel_l2(net.layer(i).read(aet.P_WEIGHT_UPDATES), onet.param(i, ob.P_WEIGHT_UPDATES)) < 2e-4, ("wgrad", i)
        net.update()
        onet.update(batch, opts["learning_rate"], opts["momentum"], opts["decay"])
        net.use_graph(True)
        for step in range(1, 5):
            xs = synth.uniform((batch, 3, 16, 16), 31, 100 + 2 * step)
            _, ts = synth.labels(batch, 10, 31, 101 + 2 * step)
            got = net.train(xs, ts)
            want = onet.train_step(xs, ts, opts["learning_rate"], opts["momentum"], opts["decay"])
            assert abs(got - want) < 2e-3 * abs(want), (step, got, want)
        ctx.check()
        net.close()
    finally:
        ctx.set_math(aet.MATH_TF32)


RAGGED_BN_CFG = """[net]
batch=6
width=13
height=13
channels=32
learning_rate=0.05
momentum=0.9
decay=0.0005

[convolutional]
filters=64
size=3
stride=1
pad=1
batch_normalize=1
activation=leaky

[convolutional]
filters=32
size=3
stride=1
pad=1
batch_normalize=1
activation=leaky

[convolutional]
filters=10
size=1
stride=1
pad=0
activation=linear

[avgpool]

[softmax]
groups=1
"""


def test_batchnorm_statistics_from_ragged_tiles(aet, ctx, oracle):
    """BN convolutions on 13x13 maps: the TMA forward kernel tiles each image as 9 + 4 rows and its epilogue's batch
    statistics must count exactly the pixels that exist.  Default TF32 math against the oracle: means, variances,
    outputs, weight gradients."""
    from oracle import cfgfile
    import aet_cnn_b200.synth as synth
    batch = 6
    net = aet.NNetwork(ctx, cfg_text=RAGGED_BN_CFG, train=1, batch=batch)
    opts, specs = cfgfile.network_spec(RAGGED_BN_CFG, batch)
    onet = oracle.net(specs, batch, 32, 13, 13, threads=os.cpu_count() or 1)
    cin = 32
    for i, s in enumerate(specs):
        if s["type"] == cfgfile.CONV:
            w = synth.normal((s["filters"], cin, s["size"], s["size"]), 41, i, 0.0, float(np.sqrt(2.0 / (s["size"] ** 2 * cin))))
            net.layer(i).write(aet.P_WEIGHTS, w)
            onet.set_param(i, ob.P_WEIGHTS, w)
            cin = s["filters"]
    x = synth.uniform((batch, 32, 13, 13), 41, 100)
    _, truth = synth.labels(batch, 10, 41, 101)
    net.input.write(x); net.truth.write(truth)
    ctx.profile(1)
    net.forward(aet.make_state(input=net.input, truth=net.truth, train=1))
    net.backward(aet.make_state(input=net.input, truth=net.truth, train=1))
    names = {r["name"].split("#")[0] for r in ctx.profile_read()}
    ctx.profile(0)
    assert {"conv_fprop_tma.ragged", "conv_dgrad_tma.ragged", "conv_wgrad_tma.ragged"} <= names, sorted(names)
    assert "bn_stats" not in names, sorted(names)      # the statistics came out of the convolution's epilogue
    onet.forward(x, truth); onet.backward(x)
    ctx.check()
    for i in (0, 1):
        assert rel_l2(net.layer(i).read(aet.P_MEAN), onet.param(i, ob.P_MEAN)) < 1e-2, i
        assert rel_l2(net.layer(i).read(aet.P_VARIANCE), onet.param(i, ob.P_VARIANCE)) < 1e-2, i
        assert rel_l2(net.layer(i).read(aet.P_OUTPUT), onet.param(i, ob.P_OUTPUT)) < 1e-2, i
    for i in (0, 1, 2):
        assert rel_l2(net.layer(i).read(aet.P_WEIGHT_UPDATES), onet.param(i, ob.P_WEIGHT_UPDATES)) < 5e-2, i
    net.close()


def test_linear_head_matches_the_separate_layers(aet, ctx, oracle):
    """In a network's training pass the 1x1 classifier convolution, the global average pool and the softmax
    run on the pooled vectors (exact FP32) instead of as a TF32 convolution over the feature map: everything
    up to the classifier's input is bit-identical, the head's results agree within the TF32 tolerance, and
    the convolution's own output and delta are still there when a host tap reads them."""
    f = _run_variant(aet, ctx, oracle, {})
    u = _run_variant(aet, ctx, oracle, {"linear_head": 0})
    for i, (a, b) in enumerate(zip(f["outs"], u["outs"])):
        if i <= 6:
            assert np.array_equal(a, b), i          # layer 6 = the convolution's lazily formed output
        else:
            assert rel_l2(a, b) < 1e-2, (i, rel_l2(a, b))
    for key in ("grads", "bgrads", "sgrads", "deltas"):
        for a, b in zip(f[key], u[key]):
            assert np.isfinite(a).all()
            assert rel_l2(a, b) < 1e-2, (key, rel_l2(a, b))
    assert np.allclose(f["losses"], u["losses"], rtol=2e-2)
    assert f["launches"] < u["launches"]


def test_weights_file_roundtrip_and_layout(aet, ctx, oracle):
    batch = 4
    net, _, opts, specs = build_pair(aet, ctx, oracle, "cifar_small.cfg", batch)
    x, truth = batch_for(opts, 10, batch, 3, 0)
    net.train(x, truth)
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "small.weights")
        net.save_weights(path)
        raw = np.fromfile(path, np.uint8)
        header = raw[:12].view(np.int32)
        assert tuple(header) == (0, 2, 5)                       # major, minor, revision
        assert raw[12:20].view(np.uint64)[0] == batch           # seen = iterations * batch
        body = raw[20:].view(np.float32)
        # first record: biases[64], scales[64], rolling_mean[64], rolling_variance[64], weights[64*3*3*3]
        l0 = net.layer(0)
        assert np.array_equal(body[:64], l0.read(aet.P_BIASES))
        assert np.array_equal(body[64:128], l0.read(aet.P_SCALES))
        assert np.array_equal(body[128:192], l0.read(aet.P_ROLLING_MEAN))
        assert np.array_equal(body[256:256 + 1728], l0.read(aet.P_WEIGHTS))
        expect = sum((4 if s["batch_normalize"] else 1) * s["filters"] for s in specs if s["type"] == 0)
        expect += 64 * 27 + 128 * 64 * 9 + 256 * 128 * 9 + 10 * 256
        assert body.size == expect
        net2 = aet.NNetwork(ctx, cfg_text=net.cfg_text, train=1, batch=batch)
        net2.load_weights(path)
        for i, s in enumerate(specs):
            if s["type"] == 0:
                assert np.array_equal(net2.layer(i).read(aet.P_WEIGHTS), net.layer(i).read(aet.P_WEIGHTS))
        p1, p2 = net.predict(x), net2.predict(x)
        assert np.array_equal(p1, p2) and np.allclose(p1.sum(1), 1.0, atol=1e-5)
        with open(path, "r+b") as f:
            f.truncate(200)
        with pytest.raises(aet.AetError):
            net2.load_weights(path)                              # a short file is an error, not a crash
        net2.close()
    net.close()


def test_resume_from_weights_and_momentum_files_is_bit_exact(aet, ctx, oracle):
    """A run stopped after three steps and resumed in a fresh network from the .weights file plus the momentum side file
    continues exactly like the uninterrupted run (same parameter hash after three more steps); from the .weights file
    alone it does not (the reference's container has no momentum buffers, dnn/NNetwork.c:112-147)."""
    batch = 8

    def steps(net, opts, first, last):
        for s in range(first, last):
            net.train(*batch_for(opts, 10, batch, 11, s))

    net, _, opts, _ = build_pair(aet, ctx, oracle, "cifar_small.cfg", batch)
    steps(net, opts, 0, 3)
    with tempfile.TemporaryDirectory() as d:
        wpath, mpath = os.path.join(d, "a.weights"), os.path.join(d, "a.momentum")
        net.save_weights(wpath)
        net.save_momentum(mpath)
        steps(net, opts, 3, 6)
        want = net.param_hash()
        net.close()
        hashes = {}
        for with_momentum in (True, False):
            fresh, _, _, _ = build_pair(aet, ctx, oracle, "cifar_small.cfg", batch)
            fresh.load_weights(wpath)
            if with_momentum:
                fresh.load_momentum(mpath)
            steps(fresh, opts, 3, 6)
            hashes[with_momentum] = fresh.param_hash()
            fresh.close()
        with open(mpath, "rb") as f:
            assert f.read(4) == b"AETM"
        with pytest.raises(aet.AetError):
            net2, _, _, _ = build_pair(aet, ctx, oracle, "cifar_small.cfg", batch)
            try:
                net2.load_momentum(wpath)       # not a momentum file
            finally:
                net2.close()
    assert hashes[True] == want
    assert hashes[False] != want


def test_bad_cfg_is_rejected(aet, ctx):
    for text in ["[convolutional]\nfilters=2\n",
                 "[net]\nbatch=2\nheight=8\nwidth=8\nchannels=3\n[convolutional]\nfilters=4\nsize=3\nactivation=gelu\n",
                 # swish / mish only on batch-normalised convolutions
                 "[net]\nbatch=2\nheight=8\nwidth=8\nchannels=3\n[convolutional]\nfilters=4\nsize=3\nactivation=mish\n",
                 "[net]\nbatch=2\nheight=8\nwidth=8\nchannels=3\n[yolo]\n",
                 "[net]\nbatch=2\nheight=8\nwidth=8\nchannels=3\n[convolutional]\nfilters=4\nactivation=leaky\nxnor=1\n",
                 # per-layer keys that would change the training loop and are not restated
                 "[net]\nbatch=2\nheight=8\nwidth=8\nchannels=3\n[convolutional]\nfilters=4\nactivation=leaky\nonlyforward=1\n",
                 "[net]\nbatch=2\nheight=8\nwidth=8\nchannels=3\n[convolutional]\nfilters=4\nactivation=leaky\ntrain_only_bn=1\n",
                 "[net]\nbatch=2\nheight=8\nwidth=8\nchannels=3\n[softmax]\n"]:
        with pytest.raises(aet.AetError):
            aet.NNetwork(ctx, cfg_text=text)


def test_alexnet_style_reduced_step(aet, ctx, oracle):
    """The AlexNet-style network (11x11/4, 5x5, FC as convolution, dropout) at batch 4, one step,
    the dropout masks shared with the oracle."""
    from oracle import cfgfile
    batch = 4
    net, onet, opts, specs = build_pair(aet, ctx, oracle, "alexnet_style.cfg", batch)
    x, truth = batch_for(opts, 1000, batch, 11, 0)
    net.input.write(x); net.truth.write(truth)
    st = aet.make_state(input=net.input, truth=net.truth, train=1)
    net.forward(st)
    for i, s in enumerate(specs):
        if s["type"] == cfgfile.DROPOUT:
            onet.set_param(i, ob.P_RAND, net.layer(i).read(aet.P_RAND))
    onet.forward(x, truth)
    net.backward(aet.make_state(input=net.input, truth=net.truth, train=1))
    onet.backward(x)
    ctx.check()
    assert [net.layer(i).out_shape for i in (0, 1, 3, 7, 8, 12)] == [(96, 55, 55), (96, 27, 27), (256, 13, 13), (256, 6, 6),
                                                                   (4096, 1, 1), (1000, 1, 1)]
    for i in range(net.layer_count):
        assert rel_l2(net.layer(i).read(aet.P_OUTPUT), onet.param(i, ob.P_OUTPUT)) < 2e-2, i
    assert abs(net.cost() - onet.cost()) < 1e-2 * abs(onet.cost())
    for i in (0, 2, 8, 12):     # coarse: relu kinks and argmax ties upstream flip under TF32 rounding
        assert rel_l2(net.layer(i).read(aet.P_WEIGHT_UPDATES), onet.param(i, ob.P_WEIGHT_UPDATES)) < 0.2, i
    net.close()


def test_train_step_from_pinned_and_pageable_buffers_is_the_same(aet, ctx, oracle):
    """aet_network_train_step copies by DMA straight from page-locked caller buffers and through the
    context's pinned mirror otherwise: same losses, same weights, bit for bit."""
    import torch
    batch = 8
    hashes, losses = [], []
    for pinned in (False, True):
        net, _, opts, specs = build_pair(aet, ctx, oracle, "cifar_small.cfg", batch)
        keep, ls = [], []
        for step in range(4):
            x, t = batch_for(opts, 10, batch, 11, step)
            if pinned:
                xt, tt = torch.from_numpy(x).pin_memory(), torch.from_numpy(t).pin_memory()
                keep += [xt, tt]
                x, t = xt.numpy(), tt.numpy()
            ls.append(net.train(x, t))
        ctx.check()
        hashes.append(net.param_hash()); losses.append(ls)
        net.close()
    assert losses[0] == losses[1]
    assert hashes[0] == hashes[1]


FREEZE_CFG = """[net]
batch={batch}
height=16
width=16
channels=3
learning_rate=0.05
momentum=0.9
decay=0.01
[convolutional]
filters=64
size=3
stride=1
pad=1
batch_normalize=1
activation=leaky
[maxpool]
size=2
stride=2
[convolutional]
filters=32
size=3
stride=1
pad=1
batch_normalize=1
activation=leaky
{stop}
[convolutional]
filters=32
size=3
stride=1
pad=1
activation=relu
{hold}
[convolutional]
filters=5
size=1
stride=1
pad=0
activation=linear
{head}
[avgpool]
[softmax]
"""


@pytest.mark.parametrize("mode", [ob.MODE_MTCS, ob.MODE_CPU])
@pytest.mark.parametrize("where", ["middle", "head"])
def test_stopbackward_and_dont_update_match_oracle(aet, ctx, oracle64, mode, where):
    """Fine-tuning keys (dnn/NetworkFactory.c:883-896,926-934,979-991; dnn/NNetwork.c:648-651,667-709): the backward walk
    ends before the last stopbackward layer, the layers in front of it only run forward and keep their weights bit for
    bit, that layer itself is still updated (weight decay on a gradient nothing writes), and dont_update = 2 holds a
    layer's weights for two iterations in the GPU parity mode while its gradients keep accumulating (the CPU update
    loop ignores the key).  With the key on the classifier convolution the fused head is taken apart.  Five steps, so the
    steps after the second run as CUDA-graph replays and the held layer is released inside the replayed graph."""
    from oracle import cfgfile
    import aet_cnn_b200.synth as synth
    batch = 6
    text = FREEZE_CFG.format(batch=batch, stop="stopbackward=1" if where == "middle" else "",
                             hold="dont_update=2", head="stopbackward=1" if where == "head" else "")
    ctx.set_math(aet.MATH_3XTF32)
    ctx.set_parity(mode)
    try:
        net = aet.NNetwork(ctx, cfg_text=text, train=1, batch=batch)
        opts, specs = cfgfile.network_spec(text, batch)
        stop = 2 if where == "middle" else 4
        assert specs[stop]["stopbackward"] == 1 and specs[3]["dont_update"] == 2
        onet = oracle64.net(specs, batch, 3, 16, 16, mode=mode)
        cin, start = 3, {}
        for i, s in enumerate(specs):
            if s["type"] == cfgfile.CONV:
                w = synth.normal((s["filters"], cin, s["size"], s["size"]), 77, i, 0.0, float(np.sqrt(2.0 / (s["size"] ** 2 * cin))))
                net.layer(i).write(aet.P_WEIGHTS, w)
                onet.set_param(i, ob.P_WEIGHTS, w)
                start[i] = w.ravel().copy()
                cin = s["filters"]
        held = []
        for step in range(5):
            x = synth.uniform((batch, 3, 16, 16), 77, 100 + 2 * step)
            _, t = synth.labels(batch, 5, 77, 101 + 2 * step)
            loss = net.train(x, t)
            oloss = onet.train_step(x, t, opts["learning_rate"], opts["momentum"], opts["decay"])
            assert abs(loss - oloss) <= 1e-4 * abs(oloss), (step, loss, oloss)
            held.append(np.array_equal(net.layer(3).read(aet.P_WEIGHTS), start[3]))
        for i in start:
            got, want = net.layer(i).read(aet.P_WEIGHTS), onet.param(i, ob.P_WEIGHTS)
            assert rel_l2(got, want) < 1e-4, (i, rel_l2(got, want))
            if i < stop:
                assert np.array_equal(got, start[i]), i              # frozen: not one bit moved
                assert not np.any(net.layer(i).read(aet.P_WEIGHT_UPDATES)), i
            elif i == stop:
                # updated without a gradient: five steps of momentum-accumulated weight decay, nothing else
                assert not np.array_equal(got, start[i])
                assert np.array_equal(net.layer(i).read(aet.P_BIASES), np.zeros(specs[i]["filters"], np.float32))
        if where == "middle":
            # layer 3 sits behind the stop layer, so it trains: held for two iterations in the GPU mode only
            assert held == ([True, True, False, False, False] if mode == ob.MODE_MTCS else [False] * 5), held
        else:
            assert all(held)                                         # in front of the stop layer: never updated
        ctx.check()
        net.close()
    finally:
        ctx.set_math(aet.MATH_TF32)
        ctx.set_parity(ob.MODE_MTCS)


def test_weights_file_partial_loads(aet, ctx, oracle):
    """loadWeights(filename, cutoff) with the per-layer keys dontload and dontloadscales (dnn/NNetwork.c:64-110,
    dnn/ConvolutionalLayer.c:455-486): a cutoff reads only the first layers, a dontload layer is passed over without
    consuming its record, dontloadscales reads biases and weights with no batch-norm block between them, and a file that
    ends at a record boundary (a backbone saved with fewer layers) leaves the remaining layers as they were."""
    import aet_cnn_b200.synth as synth
    cfg = ("[net]\nbatch=2\nheight=8\nwidth=8\nchannels=4\n"
           "[convolutional]\nfilters=4\nsize=3\nstride=1\npad=1\nbatch_normalize=1\nactivation=leaky\n{k0}\n"
           "[convolutional]\nfilters=4\nsize=3\nstride=1\npad=1\nbatch_normalize=1\nactivation=leaky\n{k1}\n"
           "[convolutional]\nfilters=3\nsize=1\nstride=1\npad=0\nactivation=linear\n[avgpool]\n[softmax]\n")
    src = aet.NNetwork(ctx, cfg_text=cfg.format(k0="", k1=""), train=1)
    for i, n in ((0, 4), (1, 4), (2, 3)):
        src.layer(i).write(aet.P_WEIGHTS, synth.normal(src.layer(i).read(aet.P_WEIGHTS).shape, 5, i, 0.0, 0.5))
        src.layer(i).write(aet.P_BIASES, synth.uniform((n,), 5, 10 + i))
        if i < 2:
            src.layer(i).write(aet.P_SCALES, 1 + synth.uniform((n,), 5, 20 + i))
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "src.weights")
        src.save_weights(path)

        def fresh(k0="", k1=""):
            net = aet.NNetwork(ctx, cfg_text=cfg.format(k0=k0, k1=k1), train=1)
            return net, [net.layer(i).read(aet.P_WEIGHTS) for i in range(3)]

        def same(a, b, i, what):
            return np.array_equal(a.layer(i).read(what), b.layer(i).read(what))

        net, init = fresh()
        net.load_weights(path, cutoff=1)                             # layer 0 only
        assert same(net, src, 0, aet.P_WEIGHTS) and same(net, src, 0, aet.P_SCALES)
        assert np.array_equal(net.layer(1).read(aet.P_WEIGHTS), init[1]) and np.array_equal(net.layer(2).read(aet.P_WEIGHTS), init[2])
        net.close()

        net, init = fresh(k0="dontload=1")                           # record 0 lands in layer 1 (same shape)
        net.load_weights(path, cutoff=2)
        assert np.array_equal(net.layer(0).read(aet.P_WEIGHTS), init[0])
        assert np.array_equal(net.layer(1).read(aet.P_WEIGHTS), src.layer(0).read(aet.P_WEIGHTS))
        assert np.array_equal(net.layer(1).read(aet.P_SCALES), src.layer(0).read(aet.P_SCALES))
        net.close()

        # a file whose only record has no batch-norm block, and which ends there
        short = os.path.join(d, "short.weights")
        bias = synth.uniform((4,), 6, 0)
        wts = synth.normal((4, 4, 3, 3), 6, 1, 0.0, 0.5)
        with open(short, "wb") as f:
            np.array([0, 2, 5], np.int32).tofile(f)
            np.array([128], np.uint64).tofile(f)
            bias.tofile(f)
            wts.tofile(f)
        net, init = fresh(k0="dontloadscales=1")
        net.load_weights(short)
        assert np.array_equal(net.layer(0).read(aet.P_BIASES), bias) and np.array_equal(net.layer(0).read(aet.P_WEIGHTS), wts.ravel())
        assert np.array_equal(net.layer(0).read(aet.P_SCALES), np.ones(4, np.float32))
        assert np.array_equal(net.layer(1).read(aet.P_WEIGHTS), init[1]) and np.array_equal(net.layer(2).read(aet.P_WEIGHTS), init[2])
        net.close()
    src.close()
