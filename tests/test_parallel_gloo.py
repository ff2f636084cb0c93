"""World-size-2 CPU (gloo) tests of the data-parallel host logic: id exchange, sharding, max-over-ranks
timing, hash agreement, and the gradient-exchange rule itself -- the per-step gradient is summed across
ranks, NOT the momentum buffer it is accumulated into -- emulated with the CPU oracle."""
import os
import socket
import sys

import numpy as np
import torch.multiprocessing as mp

from conftest import ROOT, load_package


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _specs(ob):
    return [dict(type=ob.CONV, filters=4, size=3, stride_x=1, stride_y=1, pad=1, batch_normalize=1, activation=ob.LEAKY),
            dict(type=ob.MAXPOOL, size=2, stride_x=2, stride_y=2, pad=1),
            dict(type=ob.CONV, filters=3, size=1, stride_x=1, stride_y=1, pad=0, batch_normalize=0, activation=ob.LINEAR),
            dict(type=ob.AVGPOOL), dict(type=ob.SOFTMAX, groups=1, temperature=1.0)]


def _make_net(ob, oracle, synth, batch):
    net = oracle.net(_specs(ob), batch, 2, 6, 6, mode=ob.MODE_MTCS)
    net.set_param(0, ob.P_WEIGHTS, synth.normal((72,), 5, 3, 0, 0.4))
    net.set_param(2, ob.P_WEIGHTS, synth.normal((12,), 5, 4, 0, 0.4))
    return net


GRADS = [(0, "P_WEIGHT_UPDATES"), (0, "P_BIAS_UPDATES"), (0, "P_SCALE_UPDATES"), (2, "P_WEIGHT_UPDATES"), (2, "P_BIAS_UPDATES")]


def _dp_step(ob, nets, batches, world, reduce_fn):
    from dp_oracle import dp_step
    dp_step(ob, nets, batches, world, reduce_fn, GRADS)


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    aet = load_package()
    import aet_cnn_b200.parallel as par
    import aet_cnn_b200.synth as synth
    from oracle import binding as ob
    out = {}
    uid = par.exchange_unique_id(lambda: bytes(range(128)))
    out["uid"] = uid
    out["max"] = par.max_over_ranks(10.0 + rank)
    out["same_hash"] = par.hashes_identical(0xDEADBEEF12345678)
    out["diff_hash"] = par.hashes_identical(0xDEADBEEF12345678 + rank)
    out["ids"] = [par.shard_tensor_id(s, rank, world) for s in range(3)]
    oracle = ob.Oracle("parity")
    net = _make_net(ob, oracle, synth, 4)
    for step in range(3):
        tid = par.shard_tensor_id(step, rank, world)
        x = synth.uniform((4, 2, 6, 6), 9, 2 * tid)
        t = synth.labels(4, 3, 9, 2 * tid + 1)[1]
        _dp_step(ob, [net], [(x, t)], world, lambda arrs: par.allreduce_sum_(arrs[0]))
    out["w0"] = net.param(0, ob.P_WEIGHTS).copy()
    out["w2"] = net.param(2, ob.P_WEIGHTS).copy()
    out["u0"] = net.param(0, ob.P_WEIGHT_UPDATES).copy()
    q.put((rank, out))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gloo_data_parallel_logic():
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=180) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res[0]["uid"] == res[1]["uid"] == bytes(range(128))
    assert res[0]["max"] == res[1]["max"] == 11.0
    assert res[0]["same_hash"] and res[1]["same_hash"]
    assert not res[0]["diff_hash"] and not res[1]["diff_hash"]
    assert sorted(res[0]["ids"] + res[1]["ids"]) == list(range(6))          # disjoint and complete
    for k in ("w0", "w2", "u0"):
        assert np.array_equal(res[0][k], res[1][k]), k                      # ranks stay bitwise identical

    # serial emulation of the same two ranks in one process
    load_package()
    import aet_cnn_b200.synth as synth
    from oracle import binding as ob
    oracle = ob.Oracle("parity")
    nets = [_make_net(ob, oracle, synth, 4) for _ in range(world)]

    def reduce_fn(arrs):
        total = arrs[0] + arrs[1]
        for a in arrs:
            a[:] = total

    for step in range(3):
        batches = []
        for r in range(world):
            tid = step * world + r
            batches.append((synth.uniform((4, 2, 6, 6), 9, 2 * tid), synth.labels(4, 3, 9, 2 * tid + 1)[1]))
        _dp_step(ob, nets, batches, world, reduce_fn)
    assert np.array_equal(nets[0].param(0, ob.P_WEIGHTS), res[0]["w0"])
    assert np.array_equal(nets[0].param(2, ob.P_WEIGHTS), res[0]["w2"])

    # the trap: summing the momentum-carrying buffer instead of the step gradient gives other weights
    wrong = [_make_net(ob, oracle, synth, 4) for _ in range(world)]
    for step in range(3):
        for r, net in enumerate(wrong):
            tid = step * world + r
            x, t = synth.uniform((4, 2, 6, 6), 9, 2 * tid), synth.labels(4, 3, 9, 2 * tid + 1)[1]
            net.forward(x, t)
            net.backward(x)
        for k in GRADS:
            reduce_fn([net.param(k[0], getattr(ob, k[1])) for net in wrong])
        for net in wrong:
            net.update(4 * world, 0.05, 0.9, 5e-4)
    assert not np.allclose(wrong[0].param(0, ob.P_WEIGHTS), res[0]["w0"], rtol=1e-4, atol=1e-6)
