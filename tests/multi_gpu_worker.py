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
import bench  # noqa: E402

aet = bench.load_package()
import aet_cnn_b200.cfgfile as cfgfile  # noqa: E402
import aet_cnn_b200.parallel as par  # noqa: E402
import aet_cnn_b200.synth as synth  # noqa: E402


def run(mode, rank, world, local_rank, steps=4, batch=16):
    text = open(os.path.join(aet.CFG_DIR, "cifar_small.cfg")).read()
    opts, specs = cfgfile.network_spec(text, batch)
    ctx = aet.Context(local_rank)
    net = aet.NNetwork(ctx, cfg_text=text, train=1, batch=batch)
    bench.init_weights(aet, synth, cfgfile, net, specs, 3)
    net.comm_init(par.exchange_unique_id(aet.comm_unique_id), rank, world)
    if mode == "peer":
        net.comm_exchange_attach(par.all_gather_bytes(net.comm_exchange_export()))
    net.use_graph(True)
    losses = []
    for s in range(steps):
        tid = par.shard_tensor_id(s, rank, world)
        losses.append(net.train(synth.uniform((batch, 3, 32, 32), 7, 2 * tid), synth.labels(batch, 10, 7, 2 * tid + 1)[1]))
    ctx.check()
    h = net.param_hash()
    same = par.hashes_identical(h)
    net.close(); ctx.close()
    return dict(hash=h, identical_across_ranks=same, losses=losses)


def main():
    rank, world, local_rank = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    out = {m: run(m, rank, world, local_rank) for m in ("nccl", "peer")}
    if rank == 0:
        print("RESULT " + json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
