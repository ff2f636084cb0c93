"""Runtime behaviour of the network entry points on the GPU, through the C ABI: the bounded-wait status path,
the learning-rate schedule against the oracle's restatement of NNetwork.getCurrentRate, gradient accumulation
over `subdivisions`, the non-finite scrub of the update, the pipelined train step, and the option switches."""
import numpy as np
import pytest

from conftest import rel_l2
from oracle import binding as ob
from oracle import cfgfile

pytestmark = pytest.mark.gpu

TINY = """[net]
batch=%(batch)d
subdivisions=%(sub)d
width=8
height=8
channels=3
learning_rate=0.05
momentum=0.9
decay=0.0005
%(extra)s
[convolutional]
filters=8
size=3
stride=1
pad=1
batch_normalize=%(bn)d
activation=leaky
[maxpool]
size=2
stride=2
[convolutional]
filters=5
size=1
stride=1
pad=0
activation=linear
[avgpool]
[softmax]
groups=1
"""


def tiny_cfg(batch=4, sub=1, bn=1, extra="policy=constant"):
    return TINY % dict(batch=batch, sub=sub, bn=bn, extra=extra)


def test_a_wait_nobody_satisfies_runs_out_and_reports_through_the_status_word(aet, ctx):
    """Every device-side wait is bounded.  With the limit lowered to 1 ms a warp that waits on a barrier nothing
    arrives at gives up, the kernel returns normally, aet_context_check reports AET_E_TIMEOUT, and the context
    keeps working (a convolution afterwards is correct)."""
    import aet_cnn_b200.synth as synth
    ctx.set_wait_limit(1_000_000)
    try:
        ctx.wait_probe()
        with pytest.raises(aet.AetError) as e:
            ctx.check()
        assert "aet error -5" in str(e.value)                      # AET_E_TIMEOUT
        ctx.check()                                                # the status word was cleared by the read
    finally:
        ctx.set_wait_limit(1_000_000_000)
    layer = aet.ConvolutionalLayer(ctx, 2, 8, 8, 32, 32, 3, 1, 1, 1, aet.LINEAR, 0, 1)
    w = synth.normal((32, 32, 3, 3), 3, 1, 0.0, 0.1)
    layer.write(aet.P_WEIGHTS, w)
    x = aet.Tensor(ctx, 2, 32, 8, 8)
    xv = synth.uniform((2, 32, 8, 8), 3, 2)
    x.write(xv)
    layer.forward(aet.make_state(input=x, train=1))
    ctx.check()
    import torch
    ref = torch.nn.functional.conv2d(torch.from_numpy(xv).double(), torch.from_numpy(w).double(), padding=1).numpy()
    assert rel_l2(layer.read(aet.P_OUTPUT), ref) < 1e-2
    layer.close(); x.close()


POLICIES = [
    ("policy=constant", dict(policy=0)),
    ("policy=constant\nburn_in=4\npower=2", dict(policy=0, burn_in=4, power=2.0)),
    ("policy=step\nstep=3\nscale=0.5", dict(policy=1, step=3, scale=0.5)),
    ("policy=steps\nsteps=2,5,7\nscales=0.5,0.1,2", dict(policy=2, steps=(2, 5, 7), scales=(0.5, 0.1, 2.0))),
    ("policy=exp\ngamma=0.9", dict(policy=3, gamma=0.9)),
    ("policy=poly\nmax_batches=20\npower=3", dict(policy=4, max_batches=20, power=3.0)),
    ("policy=sig\ngamma=0.7\nstep=4", dict(policy=5, gamma=0.7, step=4)),
    ("policy=sig\ngamma=-0.7\nstep=4\nburn_in=2", dict(policy=5, gamma=-0.7, step=4, burn_in=2)),
]


@pytest.mark.parametrize("extra,kw", POLICIES)
def test_learning_rate_schedule_matches_the_reference_formulas(aet, ctx, oracle, extra, kw):
    """aet_network_learning_rate after every training step against the oracle's NNetwork.getCurrentRate
    (dnn/NNetwork.c:215-246), including the unsigned `batch_num - step` of the sig policy."""
    import aet_cnn_b200.synth as synth
    batch = 2
    net = aet.NNetwork(ctx, cfg_text=tiny_cfg(batch=batch, extra=extra), train=1)
    x = synth.uniform((batch, 3, 8, 8), 5, 1)
    _, t = synth.labels(batch, 5, 5, 2)
    for step in range(10):
        want = oracle.current_rate(step, learning_rate=0.05, **kw)
        got = net.learning_rate()
        assert got == pytest.approx(want, rel=1e-6, abs=1e-12), (step, got, want)
        net.train(x, t)
    net.close()


@pytest.mark.parametrize("sub", [2, 3])
def test_subdivisions_accumulate_gradients_and_update_once(aet, ctx, oracle64, sub):
    """[net] subdivisions = S: S calls accumulate the weight gradients, the S-th updates with
    update_batch = batch * S (dnn/NNetwork.c:762-774, 667-680).  Against the oracle driven the same way
    (S forward/backward passes, one update), 3xTF32 math, two groups, eager and graph replay."""
    import aet_cnn_b200.synth as synth
    per_call = 4
    text = tiny_cfg(batch=per_call * sub, sub=sub)
    opts, specs = cfgfile.network_spec(text)
    assert opts["batch"] == per_call and opts["subdivisions"] == sub
    ctx.set_math(aet.MATH_3XTF32)
    try:
        results = []
        for use_graph in (False, True):
            net = aet.NNetwork(ctx, cfg_text=text, train=1)
            assert net.batch == per_call
            net.use_graph(use_graph)
            onet = oracle64.net(specs, per_call, 3, 8, 8, mode=ob.MODE_MTCS)
            w0 = synth.normal((8, 3, 3, 3), 9, 1, 0.0, 0.3)
            w2 = synth.normal((5, 8, 1, 1), 9, 2, 0.0, 0.3)
            net.layer(0).write(aet.P_WEIGHTS, w0); net.layer(2).write(aet.P_WEIGHTS, w2)
            onet.set_param(0, ob.P_WEIGHTS, w0); onet.set_param(2, ob.P_WEIGHTS, w2)
            call = 0
            for group in range(4):
                for s in range(sub):
                    x = synth.uniform((per_call, 3, 8, 8), 9, 10 + 2 * call)
                    _, t = synth.labels(per_call, 5, 9, 11 + 2 * call)
                    loss = net.train(x, t)
                    onet.forward(x, t)
                    onet.backward(x)
                    assert loss == pytest.approx(onet.cost() / per_call, rel=2e-4)
                    if s < sub - 1:      # no update yet: the weights are still the group's
                        assert rel_l2(net.layer(0).read(aet.P_WEIGHTS), onet.param(0, ob.P_WEIGHTS)) < 1e-5
                    call += 1
                onet.update(per_call * sub, opts["learning_rate"], opts["momentum"], opts["decay"])
                for i in (0, 2):
                    assert rel_l2(net.layer(i).read(aet.P_WEIGHTS), onet.param(i, ob.P_WEIGHTS)) < 1e-4, (group, i)
            ctx.check()
            results.append(net.param_hash())
            net.close()
        assert results[0] == results[1]          # graph replay (two graphs: accumulate-only and final) is bitwise the eager result
    finally:
        ctx.set_math(aet.MATH_TF32)


def test_adam_update_matches_the_reference_routine(aet, ctx, oracle64):
    """[net] adam=1: adam_update_gpu (mtcs/MtcsConvLayer.c:494-524) applied to weights, biases and scales, against the
    oracle's gradients (3xTF32 math) pushed through the restated routine, four steps."""
    import aet_cnn_b200.synth as synth
    batch = 4
    text = tiny_cfg(batch=batch, extra="policy=constant\nadam=1\nB1=0.9\nB2=0.999\neps=0.000001")
    opts, specs = cfgfile.network_spec(text)
    ctx.set_math(aet.MATH_3XTF32)
    try:
        net = aet.NNetwork(ctx, cfg_text=text, train=1)
        onet = oracle64.net(specs, batch, 3, 8, 8, mode=ob.MODE_MTCS)
        w0 = synth.normal((8, 3, 3, 3), 19, 1, 0.0, 0.3)
        w2 = synth.normal((5, 8, 1, 1), 19, 2, 0.0, 0.3)
        net.layer(0).write(aet.P_WEIGHTS, w0); net.layer(2).write(aet.P_WEIGHTS, w2)
        onet.set_param(0, ob.P_WEIGHTS, w0); onet.set_param(2, ob.P_WEIGHTS, w2)
        pairs = [(0, ob.P_WEIGHTS, ob.P_WEIGHT_UPDATES), (0, ob.P_BIASES, ob.P_BIAS_UPDATES), (0, ob.P_SCALES, ob.P_SCALE_UPDATES),
                 (2, ob.P_WEIGHTS, ob.P_WEIGHT_UPDATES), (2, ob.P_BIASES, ob.P_BIAS_UPDATES)]
        mom = {k: (np.zeros(onet.param(k[0], k[1]).size, np.float32), np.zeros(onet.param(k[0], k[1]).size, np.float32)) for k in pairs}
        for step in range(4):
            x = synth.uniform((batch, 3, 8, 8), 19, 10 + 2 * step)
            _, t = synth.labels(batch, 5, 19, 11 + 2 * step)
            loss = net.train(x, t)
            onet.forward(x, t)
            onet.backward(x)
            assert loss == pytest.approx(onet.cost() / batch, rel=2e-4)
            for k in pairs:
                oracle64.adam_update(onet.param(k[0], k[1]), onet.param(k[0], k[2]), mom[k][0], mom[k][1], 0.9, 0.999, 1e-6,
                                     opts["decay"], opts["learning_rate"], batch, step + 1)
            for layer, wsel, _ in pairs:
                got = net.layer(layer).read({ob.P_WEIGHTS: aet.P_WEIGHTS, ob.P_BIASES: aet.P_BIASES, ob.P_SCALES: aet.P_SCALES}[wsel])
                assert rel_l2(got, onet.param(layer, wsel)) < 2e-4, (step, layer, wsel)
        ctx.check()
        net.close()
    finally:
        ctx.set_math(aet.MATH_TF32)


def test_update_scrubs_non_finite_values_like_the_reference_gpu_update(aet, ctx, oracle):
    """mtcs/MtcsConvLayer.c:586-587: before the update, NaN/Inf pending weight updates become 0 and NaN/Inf weights
    become 1/(index+1); the status word then reports AET_E_NAN (informational).  The CPU formulation does not scrub."""
    K, C = 8, 4
    for mode in (ob.MODE_MTCS, ob.MODE_CPU):
        ctx.set_parity(mode)
        try:
            layer = aet.ConvolutionalLayer(ctx, 1, 4, 4, C, K, 1, 1, 1, 0, aet.LINEAR, 0, 1)
            w = np.linspace(-1, 1, K * C).astype(np.float32)
            u = np.linspace(0.5, -0.5, K * C).astype(np.float32)
            w[3], w[17] = np.nan, np.inf
            u[5], u[17] = -np.inf, np.nan
            layer.write(aet.P_WEIGHTS, w); layer.write(aet.P_WEIGHT_UPDATES, u)
            layer.update(2, 0.1, 0.9, 0.0, 1.0)
            gw, gu = layer.read(aet.P_WEIGHTS), layer.read(aet.P_WEIGHT_UPDATES)
            layer.close()
            if mode == ob.MODE_MTCS:
                uu = oracle.reset_nan_and_inf(u)
                ww = oracle.fix_nan_and_inf(w)
                ww2, uu2 = oracle.sgd_weights(ww, uu, 2, 0.1, 0.9, 0.0)
                # 1x1 filters over 4 channels: the device layout [filter][tap][channel] equals the host's, so do the indices
                assert np.isfinite(gw).all() and np.isfinite(gu).all()
                assert rel_l2(gw, ww2) < 1e-6 and rel_l2(gu, uu2) < 1e-6
                with pytest.raises(aet.AetError) as e:
                    ctx.check()
                assert "aet error -7" in str(e.value)              # AET_E_NAN
            else:
                assert not np.isfinite(gw[[3, 17]]).any()
                ctx.check()
        finally:
            ctx.set_parity(ob.MODE_MTCS)


def test_pipelined_train_step_is_the_synchronous_step_with_the_loss_one_call_late(aet, ctx):
    """aet_network_train_step_async double-buffers the upload and returns the previous call's loss: same losses,
    same weights, bit for bit, from pageable and from page-locked buffers."""
    import torch
    import aet_cnn_b200.synth as synth
    batch, steps = 8, 7
    text = open(aet.CFG_DIR + "/cifar_small.cfg").read()
    batches = [(synth.uniform((batch, 3, 32, 32), 21, 2 * s), synth.labels(batch, 10, 21, 2 * s + 1)[1]) for s in range(steps)]

    def fresh():
        net = aet.NNetwork(ctx, cfg_text=text, train=1, batch=batch)
        net.layer(0).write(aet.P_WEIGHTS, synth.normal((64, 3, 3, 3), 21, 100, 0.0, 0.27))
        net.layer(2).write(aet.P_WEIGHTS, synth.normal((128, 64, 3, 3), 21, 101, 0.0, 0.06))
        net.layer(4).write(aet.P_WEIGHTS, synth.normal((256, 128, 3, 3), 21, 102, 0.0, 0.04))
        net.layer(6).write(aet.P_WEIGHTS, synth.normal((10, 256, 1, 1), 21, 103, 0.0, 0.09))
        net.use_graph(True)
        return net

    net = fresh()
    sync_losses = [net.train(x, t) for x, t in batches]
    sync_hash = net.param_hash()
    net.close()
    for pinned in (False, True):
        net = fresh()
        keep, losses = [], []
        for x, t in batches:
            if pinned:
                xt, tt = torch.from_numpy(x).pin_memory(), torch.from_numpy(t).pin_memory()
                keep += [xt, tt]
                x, t = xt.numpy(), tt.numpy()
            losses.append(net.train_async(x, t))
        losses.append(net.last_loss())
        assert np.isnan(losses[0])
        assert losses[1:] == sync_losses, pinned
        assert net.param_hash() == sync_hash, pinned
        ctx.check()
        net.close()


@pytest.mark.parametrize("channels", [3, 1])
def test_device_augmentation_matches_the_reference_chain(aet, ctx, oracle, channels):
    """rotate/scale/shift crop with bilinear sampling, left-right flip and HSV distortion (dnn/NImage.c) fused in one
    kernel that writes the network input, against the oracle's restatement image by image.  The draws are inputs on
    both sides.  Values are in [0,1]; float arithmetic in the same order, so the bound is a few ulps of 1."""
    import aet_cnn_b200.synth as synth
    batch, size, sh, sw = 6, 8, 19, 23
    text = tiny_cfg(batch=batch).replace("channels=3", "channels=%d" % channels)
    net = aet.NNetwork(ctx, cfg_text=text, train=1)
    src = synth.uniform((batch, channels, sh, sw), 77, 1)
    rng = np.random.default_rng(5)
    params = []
    for b in range(batch):
        params.append(dict(rad=float(rng.uniform(-0.4, 0.4)) if b else 0.0, scale=float(rng.uniform(0.4, 1.3)),
                           dx=float(rng.uniform(-3, 3)), dy=float(rng.uniform(-3, 3)), aspect=float(rng.uniform(0.8, 1.25)),
                           flip=int(b % 2), dhue=float(rng.uniform(-0.1, 0.1)), dsat=float(rng.uniform(0.7, 1.5)),
                           dexp=float(rng.uniform(0.7, 1.5))))
    net.augment_input(src, params)
    got = net.input.read()
    for b in range(batch):
        want = oracle.augment_image(src[b], size, **params[b])
        assert np.abs(got[b] - want).max() < 2e-6, (b, np.abs(got[b] - want).max())
    assert got.min() >= 0.0 and (channels != 3 or got.max() <= 1.0)
    # the augmented batch trains like any other input
    _, t = synth.labels(batch, 5, 77, 2)
    net.truth.write(t)
    loss = net.train_device()
    assert np.isfinite(loss)
    net.close()


def test_option_switches(aet, ctx):
    assert ctx.get_option("rows") == 1
    ctx.set_option("rows", 0)
    assert ctx.get_option("rows") == 0
    ctx.set_option("rows", 1)
    with pytest.raises(aet.AetError):
        ctx.set_option("no_such_switch", 1)
