"""Two-GPU data parallel through the C ABI (skipped on a box with one GPU): NCCL all-reduce against the peer
exchange fused into the update kernel, the data-parallel weights against the CPU oracle's emulation of the ranks, and
a peer that never publishes its gradients (bounded wait, whole update skipped, AET_E_TIMEOUT)."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu


def test_two_ranks_nccl_and_peer_exchange_agree():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29633", os.path.join(here, "multi_gpu_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1]
    out = json.loads(line[len("RESULT "):])
    for mode in ("nccl", "peer"):
        assert out[mode]["identical_across_ranks"], mode          # weights bitwise identical on both ranks
    assert out["nccl"]["hash"] == out["peer"]["hash"]             # two ranks: the same sum either way (and the stamps change nothing)
    us, counted = out["nccl"]["comm_exposed"]
    assert counted == 5 and 0.0 <= us < 1e5, out["nccl"]["comm_exposed"]    # one wait per step, a plausible duration
    # peer exchange: the wait for the peers' slices is bracketed the same way (four steps), then one step after the detach
    us, counted = out["peer"]["comm_exposed"]
    assert counted == 5 and 0.0 <= us < 1e5, out["peer"]["comm_exposed"]
    assert out["nccl"]["losses"] == out["peer"]["losses"]
    # the data-parallel result itself against the CPU oracle's emulation of the two ranks (3xTF32 math, two steps)
    assert out["oracle"], out
    for layer, e in out["oracle"].items():
        assert e["weights"] < 1e-4 and e["change"] < 5e-2, (layer, e)
    # a rank that sits out a step: the other rank's update is skipped as a whole and the step reports the timeout
    assert "aet error -5" in out["absent_peer"]["message"], out["absent_peer"]
    assert out["absent_peer"]["unchanged"], out["absent_peer"]


def test_two_contexts_on_two_devices_in_one_process(aet):
    """One process, one context per GPU (the ABI allows it): kernels that need the large dynamic shared-memory opt-in
    must get it on BOTH devices (function attributes are per device), and the same training steps give the same
    parameters on either GPU."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import aet_cnn_b200.synth as synth
    text = open(os.path.join(aet.CFG_DIR, "cifar_small.cfg")).read()
    batch = 128          # the benchmark's batch: the row-sharing and thin kernels with > 48 KB of shared memory run
    x = [synth.uniform((batch, 3, 32, 32), 5, 2 * s) for s in range(2)]
    t = [synth.labels(batch, 10, 5, 2 * s + 1)[1] for s in range(2)]
    hashes, losses = [], []
    for dev in (0, 1):
        ctx = aet.Context(dev)
        net = aet.NNetwork(ctx, cfg_text=text, train=1, batch=batch)
        import bench
        bench.init_weights(aet, synth, net, 3)
        losses.append([net.train(x[s], t[s]) for s in range(2)])
        ctx.check()
        hashes.append(net.param_hash())
        net.close(); ctx.close()
    assert hashes[0] == hashes[1]
    assert losses[0] == losses[1]
