"""Worker of tests/test_gpu_multi.py: one rank of a two-GPU data-parallel run.  Trains the small CNN for a few
steps once with the NCCL all-reduce and once with the peer exchange fused into the update kernel, and
prints one JSON line with the parameter hashes (they must agree across ranks, and, with two ranks, across
the two modes: a + b is the same sum in either order)."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import bench  # noqa: E402

aet = bench.load_package()
from oracle import cfgfile  # noqa: E402
import aet_cnn_b200.parallel as par  # noqa: E402
import aet_cnn_b200.synth as synth  # noqa: E402


def run(mode, rank, world, local_rank, steps=4, batch=16):
    text = open(os.path.join(aet.CFG_DIR, "cifar_small.cfg")).read()
    opts, specs = cfgfile.network_spec(text, batch)
    ctx = aet.Context(local_rank)
    ctx.set_option("comm_stamps", 1)          # time the main stream's waits for the exchange (two extra tiny kernels each)
    net = aet.NNetwork(ctx, cfg_text=text, train=1, batch=batch)
    bench.init_weights(aet, synth, net, 3)
    net.comm_init(par.exchange_unique_id(aet.comm_unique_id), rank, world)
    if mode == "peer":
        net.comm_exchange_attach(par.all_gather_bytes(net.comm_exchange_export()))
    net.use_graph(True)
    losses = []
    for s in range(steps + 1):
        if mode == "peer" and s == steps:
            net.comm_exchange_detach()        # the last step goes through the collectives again
        tid = par.shard_tensor_id(s, rank, world)
        losses.append(net.train(synth.uniform((batch, 3, 32, 32), 7, 2 * tid), synth.labels(batch, 10, 7, 2 * tid + 1)[1]))
    ctx.check()
    h = net.param_hash()
    same = par.hashes_identical(h)
    exposed = net.comm_exposed()
    net.close(); ctx.close()
    return dict(hash=h, identical_across_ranks=same, losses=losses, comm_exposed=exposed)


def oracle_check(rank, world, local_rank, steps=2, batch=8):
    """Two data-parallel steps on the GPUs (3xTF32 math, NCCL exchange) against the same two steps emulated with the
    CPU oracle: one oracle network per rank, gradients summed over the ranks, update with the global batch.
    Returns the relative L2 error of every convolution's weights and of the weight CHANGE since initialisation
    (the part the exchange is responsible for)."""
    import numpy as np
    from oracle import binding as ob
    from dp_oracle import dp_step, grad_keys, sum_in_place
    text = open(os.path.join(aet.CFG_DIR, "cifar_small.cfg")).read()
    opts, specs = cfgfile.network_spec(text, batch)
    ctx = aet.Context(local_rank, math=aet.MATH_3XTF32)
    net = aet.NNetwork(ctx, cfg_text=text, train=1, batch=batch)
    bench.init_weights(aet, synth, net, 3)
    convs = [i for i, s in enumerate(specs) if s["type"] == cfgfile.CONV]
    w0 = {i: net.layer(i).read(aet.P_WEIGHTS) for i in convs}
    net.comm_init(par.exchange_unique_id(aet.comm_unique_id), rank, world)
    for s in range(steps):
        tid = par.shard_tensor_id(s, rank, world)
        net.train(synth.uniform((batch, 3, 32, 32), 7, 2 * tid), synth.labels(batch, 10, 7, 2 * tid + 1)[1])
    ctx.check()
    got = {i: net.layer(i).read(aet.P_WEIGHTS) for i in convs}
    net.close(); ctx.close()
    errs = {}
    if rank == 0:
        oracle = ob.Oracle("acc64")
        nets = []
        for r in range(world):
            o = oracle.net(specs, batch, 3, 32, 32, mode=ob.MODE_MTCS)
            for i in convs:
                o.set_param(i, ob.P_WEIGHTS, w0[i])
            nets.append(o)
        keys = grad_keys(ob, specs)
        for s in range(steps):
            batches = []
            for r in range(world):
                tid = par.shard_tensor_id(s, r, world)
                batches.append((synth.uniform((batch, 3, 32, 32), 7, 2 * tid), synth.labels(batch, 10, 7, 2 * tid + 1)[1]))
            dp_step(ob, nets, batches, world, sum_in_place, keys, opts["learning_rate"], opts["momentum"], opts["decay"])
        for i in convs:
            ref = nets[0].param(i, ob.P_WEIGHTS).astype(np.float64)
            g, z = got[i].ravel().astype(np.float64), w0[i].ravel().astype(np.float64)
            errs[str(i)] = dict(weights=float(np.linalg.norm(g - ref) / np.linalg.norm(ref)),
                                change=float(np.linalg.norm((g - z) - (ref - z)) / np.linalg.norm(ref - z)))
    return errs


def absent_peer(rank, world, local_rank, batch=16):
    """A rank that sits out a step, seen from the other rank (peer exchange attached, 50 ms wait limit): the update's
    gate kernel waits for a slice that is never published, gives up, and the whole update is skipped - the step
    reports AET_E_TIMEOUT and the parameters are bit for bit those of the last complete step.  The absent rank leaves
    between steps with nothing in flight; the ranks meet again on the host."""
    text = open(os.path.join(aet.CFG_DIR, "cifar_small.cfg")).read()
    ctx = aet.Context(local_rank)
    net = aet.NNetwork(ctx, cfg_text=text, train=1, batch=batch)
    bench.init_weights(aet, synth, net, 3)
    net.comm_init(par.exchange_unique_id(aet.comm_unique_id), rank, world)
    net.comm_exchange_attach(par.all_gather_bytes(net.comm_exchange_export()))
    ctx.set_wait_limit(50 * 1000 * 1000)
    x, truth = synth.uniform((batch, 3, 32, 32), 9, rank), synth.labels(batch, 10, 9, 100 + rank)[1]
    for _ in range(2):
        net.train(x, truth)
    ctx.check()
    before = net.param_hash()
    torch.cuda.synchronize()
    dist.barrier()
    res = {}
    if rank == 0:
        message = ""
        try:
            net.train(x, truth)
        except Exception as e:   # noqa: BLE001 - the binding raises its own error type with the status code in the text
            message = str(e)
        res = dict(message=message, unchanged=net.param_hash() == before)
    torch.cuda.synchronize()
    dist.barrier()
    net.close(); ctx.close()
    return res


def main():
    rank, world, local_rank = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    out = {m: run(m, rank, world, local_rank) for m in ("nccl", "peer")}
    out["oracle"] = oracle_check(rank, world, local_rank)
    out["absent_peer"] = absent_peer(rank, world, local_rank)
    if rank == 0:
        print("RESULT " + json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
