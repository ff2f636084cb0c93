"""Seeded synthetic tensors (numpy) for parity runs and benchmarks.

Stream definition (identical to the C generator the CPU oracle uses; a test keeps them equal):
  state_i = (seed ^ tensor_id) + (i + 1) * 0x9E3779B97F4A7C15  (mod 2^64)
  u_i     = (splitmix64_finaliser(state_i) >> 40) * 2^-24       in [0, 1)
  normal  = sqrtf(-2 logf(max(u_2j, 2^-24))) * cosf(2 pi u_2j+1), float32 arithmetic.
The reference trains on CIFAR images; these tensors only take their shapes and value ranges.
"""
import numpy as np

_GOLD = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


def _mix(z):
    z = (z ^ (z >> np.uint64(30))) * _M1
    z = (z ^ (z >> np.uint64(27))) * _M2
    return z ^ (z >> np.uint64(31))


def uniform(shape, seed, tensor_id):
    n = int(np.prod(shape))
    with np.errstate(over="ignore"):
        base = np.uint64(seed) ^ np.uint64(tensor_id)
        s = base + (np.arange(1, n + 1, dtype=np.uint64)) * _GOLD
        z = _mix(s)
    return ((z >> np.uint64(40)).astype(np.float32) * np.float32(1.0 / 16777216.0)).reshape(shape)


def normal(shape, seed, tensor_id, mean=0.0, std=1.0):
    n = int(np.prod(shape))
    u = uniform((2 * n,), seed, tensor_id)
    u1 = np.maximum(u[0::2], np.float32(1.0 / 16777216.0))
    u2 = u[1::2]
    g = np.sqrt(np.float32(-2.0) * np.log(u1)).astype(np.float32) * np.cos(np.float32(6.28318530717958647692) * u2).astype(np.float32)
    return (np.float32(mean) + np.float32(std) * g).astype(np.float32).reshape(shape)


def labels(batch, classes, seed, tensor_id):
    """Uniform integer labels floor(u * classes) and their one-hot float encoding (dnn/TruthData.c:13-21)."""
    u = uniform((batch,), seed, tensor_id)
    y = np.minimum((u * classes).astype(np.int64), classes - 1)
    onehot = np.zeros((batch, classes), np.float32)
    onehot[np.arange(batch), y] = 1.0
    return y, onehot


def shard_tensor_id(step, rank, world):
    """Disjoint per-rank batches of one global batch: rank r of `world` draws tensor step*world + r."""
    return step * world + rank
