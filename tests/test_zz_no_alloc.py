"""The allocation-free bias-gradient entry point against the column sums themselves and the layer entry point.

Some callers cannot allocate device memory while they run (a process whose device pool is fixed and handed out
at start-up, a service inside a phase where cudaMalloc is off limits).  aet_backward_bias_static keeps its partial
sums in a fixed array inside the library; here it must reproduce sum over pixels of delta -- what
aet_layer_backward accumulates into bias_updates -- on two calls in a row (the array is shared and reused).
This file sorts last on purpose: a run that stops at the first failure has already run the rest."""
import numpy as np
import pytest

from conftest import rel_l2

pytestmark = pytest.mark.gpu


def test_static_scratch_bias_gradient_matches_layer_backward(aet, ctx):
    import torch
    import aet_cnn_b200.synth as synth
    N, C, H, W, K = 8, 8, 12, 12, 64            # K multiple of 4: device rows are K floats, no padding
    layer = aet.ConvolutionalLayer(ctx, N, H, W, C, K, 1, 1, 1, 0, aet.LINEAR, 0, 1)
    xin = aet.Tensor(ctx, N, C, H, W)
    xin.write(synth.uniform((N, C, H, W), 123, 1))
    st = aet.make_state(input=xin, train=1)
    layer.forward(st)
    out = torch.zeros(K, dtype=torch.float32, device="cuda")
    expect_acc = np.zeros(K, np.float64)
    for call in range(2):
        dy = synth.normal((N, K, H, W), 123, 10 + call)
        # existing entry point: layer backward accumulates sum(delta) into bias_updates
        layer.write(aet.P_BIAS_UPDATES, np.zeros(K, np.float32))
        layer.write(aet.P_DELTA, dy)
        layer.backward(st)
        ref = layer.read(aet.P_BIAS_UPDATES)
        # new entry point on raw device pointers: [pixels][channels] rows, accumulating across calls
        d = torch.from_numpy(np.ascontiguousarray(dy.transpose(0, 2, 3, 1)).reshape(N * H * W, K)).cuda()
        torch.cuda.synchronize()
        aet.backward_bias_static(d.data_ptr(), out.data_ptr(), N * H * W, K)
        torch.cuda.synchronize()
        sums = dy.astype(np.float64).sum(axis=(0, 2, 3))          # the definition, in double
        assert rel_l2(ref, sums) < 1e-6                           # the layer entry point against the definition
        expect_acc = expect_acc + sums
        got = out.cpu().numpy()
        assert rel_l2(got, expect_acc) < 1e-6, (call, rel_l2(got, expect_acc))
    layer.close(); xin.close()


@pytest.mark.parametrize("pixels,channels", [(300, 12), (1000, 100), (96, 1280), (40, 2052), (100000, 64)])
def test_static_scratch_channel_layouts_against_the_column_sums(aet, ctx, pixels, channels):
    """Channel counts that exercise every thread-to-channel map of the reduction: fewer channels than a warp covers
    (12), a ragged last block of the finalize kernel (100), more than 1024 channels (two channel slabs in the grid),
    and a long pixel axis (many blocks).  Launched on a stream of the caller's, twice in a row, against dy.sum(0)."""
    import torch
    rng = np.random.default_rng(pixels + channels)
    stream = torch.cuda.Stream()
    out = torch.zeros(channels, dtype=torch.float32, device="cuda")
    expect = np.zeros(channels, np.float64)
    for call in range(2):
        dy = rng.standard_normal((pixels, channels)).astype(np.float32)
        d = torch.from_numpy(dy).cuda()
        torch.cuda.synchronize()
        aet.backward_bias_static(d.data_ptr(), out.data_ptr(), pixels, channels, stream=stream.cuda_stream)
        stream.synchronize()
        expect += dy.astype(np.float64).sum(0)
        got = out.cpu().numpy()
        err = np.abs(got - expect).max() / max(1.0, np.abs(expect).max())
        assert err < 2e-6, (call, err)


def test_static_scratch_rejects_oversized_and_bad_arguments(aet, ctx):
    import torch
    d = torch.zeros(4096 * 1024, dtype=torch.float32, device="cuda")
    o = torch.zeros(1024, dtype=torch.float32, device="cuda")
    with pytest.raises(aet.AetError) as e:
        aet.backward_bias_static(d.data_ptr(), o.data_ptr(), 4096, 1024)     # needs more than the fixed array
    assert "static array" in str(e.value)
    with pytest.raises(aet.AetError):
        aet.backward_bias_static(d.data_ptr(), o.data_ptr(), 16, 6)          # channels not a multiple of 4
    with pytest.raises(aet.AetError):
        aet.backward_bias_static(0, o.data_ptr(), 16, 8)
