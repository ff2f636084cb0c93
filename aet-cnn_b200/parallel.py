"""Host-side plumbing of batch data-parallel training (one process per GPU).

The device side (NCCL all-reduce of the gradient arena, issued per bucket during backward) lives in
csrc/network.cu; these helpers only move small host values between ranks through torch.distributed
(any backend: NCCL on GPUs, gloo in the CPU tests)."""
import numpy as np
import torch
import torch.distributed as dist


def is_dist():
    return dist.is_available() and dist.is_initialized()


def _dev():
    return torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else torch.device("cpu")


def exchange_unique_id(make_id, nbytes=128):
    """Rank 0 creates the communicator id (bytes), every rank returns the same bytes."""
    if not is_dist() or dist.get_world_size() == 1:
        return bytes(make_id())
    buf = torch.zeros(nbytes, dtype=torch.uint8, device=_dev())
    if dist.get_rank() == 0:
        raw = bytes(make_id())
        if len(raw) != nbytes:
            raise ValueError("unique id must be %d bytes" % nbytes)
        buf.copy_(torch.frombuffer(bytearray(raw), dtype=torch.uint8))
    dist.broadcast(buf, 0)
    return bytes(buf.cpu().numpy().tobytes())


def all_gather_bytes(raw):
    """Every rank's byte string (all of one length), in rank order."""
    if not is_dist() or dist.get_world_size() == 1:
        return [bytes(raw)]
    mine = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(_dev())
    parts = [torch.zeros_like(mine) for _ in range(dist.get_world_size())]
    dist.all_gather(parts, mine)
    return [bytes(p.cpu().numpy().tobytes()) for p in parts]


def max_over_ranks(value):
    """The slowest rank's time: multi-GPU numbers are the max over ranks, never a wall clock."""
    if not is_dist() or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=_dev())
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def hashes_identical(h):
    """True on every rank iff all ranks hold the same 64-bit parameter hash."""
    if not is_dist() or dist.get_world_size() == 1:
        return True
    parts = torch.tensor([h & 0xFFFFFFFF, (h >> 32) & 0xFFFFFFFF], dtype=torch.int64, device=_dev())
    gathered = [torch.zeros_like(parts) for _ in range(dist.get_world_size())]
    dist.all_gather(gathered, parts)
    return all(bool(torch.equal(g, gathered[0])) for g in gathered)


def shard_tensor_id(step, rank, world):
    """Rank r of `world` draws synthetic tensor step*world + r: disjoint shards of one global batch."""
    return step * world + rank


def update_batch(per_gpu_batch, subdivisions, world):
    """The divisor of the SGD step (`update_batch`, dnn/NNetwork.c:669) for the global batch."""
    return per_gpu_batch * subdivisions * world


def allreduce_sum_(array):
    """In-place sum of a float32 numpy array over ranks (CPU emulation of the gradient exchange)."""
    if not is_dist() or dist.get_world_size() == 1:
        return array
    t = torch.from_numpy(array)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return array
