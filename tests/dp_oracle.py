"""Data-parallel training step emulated with the CPU oracle (test infrastructure): every emulated rank runs
forward + backward on its shard, the per-step gradients -- NOT the momentum buffers they are accumulated into --
are summed over the ranks, and every rank applies the same update with the global batch as divisor.  Shared by
the gloo test of the host logic and by the two-GPU worker, which checks the device result against it."""


def grad_keys(ob, specs):
    """(layer, parameter) pairs that carry gradients: weights, biases (the BN shift in MTCS mode), BN scales."""
    keys = []
    for i, s in enumerate(specs):
        if s["type"] != ob.CONV:
            continue
        keys += [(i, "P_WEIGHT_UPDATES"), (i, "P_BIAS_UPDATES")]
        if s.get("batch_normalize"):
            keys.append((i, "P_SCALE_UPDATES"))
    return keys


def dp_step(ob, nets, batches, world, reduce_fn, keys, lr=0.05, mom=0.9, decay=5e-4):
    """One data-parallel step over `nets` (one per emulated rank held by this process)."""
    carries = []
    for net, (x, t) in zip(nets, batches):
        carry = {k: net.param(k[0], getattr(ob, k[1])).copy() for k in keys}
        for k in keys:
            net.param(k[0], getattr(ob, k[1]))[:] = 0          # this step's gradient only
        net.forward(x, t)
        net.backward(x)
        carries.append(carry)
    for k in keys:
        reduce_fn([net.param(k[0], getattr(ob, k[1])) for net in nets])
    for net, carry in zip(nets, carries):
        for k in keys:
            net.param(k[0], getattr(ob, k[1]))[:] += carry[k]  # momentum history is per rank and identical
        net.update(nets[0].batch * world, lr, mom, decay)


def sum_in_place(arrs):
    total = arrs[0].copy()
    for a in arrs[1:]:
        total += a
    for a in arrs:
        a[:] = total
