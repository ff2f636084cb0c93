"""Generates tests/golden/ops_f64.npz: known-answer vectors for the operators on the hot path,
computed by an INDEPENDENT implementation (PyTorch CPU, float64 autograd) on seeded inputs.
They pin the CPU oracle (oracle/aet_oracle.c), which in turn checks the CUDA library.

Run from the repository root:  python tests/golden/make_golden.py
The reference project itself ships no golden vectors and cannot be built in this environment.
"""
import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.join(ROOT, "aet-cnn_b200"))
import synth  # noqa: E402

torch.set_default_dtype(torch.float64)
out = {}


def t(a, grad=False):
    x = torch.tensor(np.asarray(a, np.float64))
    x.requires_grad_(grad)
    return x


# ---- convolution cases: (name, N, C, H, W, K, size, stride, pad)
for name, N, C, H, W, K, size, stride, pad in [
    ("conv_a", 2, 3, 8, 8, 5, 3, 1, 1),
    ("conv_b", 2, 4, 9, 7, 6, 3, 2, 1),
    ("conv_c", 1, 6, 5, 5, 4, 1, 1, 0),
    ("conv_d", 2, 2, 11, 11, 3, 5, 2, 2),
]:
    x = synth.uniform((N, C, H, W), 11, sum(map(ord, name)))
    w = synth.normal((K, C, size, size), 11, sum(map(ord, name)) + 1, 0, 0.3)
    xt, wt = t(x, True), t(w, True)
    y = F.conv2d(xt, wt, None, stride, pad)
    dy = synth.normal(tuple(y.shape), 11, sum(map(ord, name)) + 2)
    y.backward(t(dy))
    out[name + "_x"], out[name + "_w"], out[name + "_dy"] = x, w, dy
    out[name + "_y"] = y.detach().numpy()
    out[name + "_dx"], out[name + "_dw"] = xt.grad.numpy(), wt.grad.numpy()
    out[name + "_geom"] = np.array([stride, pad])


# ---- batch norm, training mode, biased variance + eps inside the sqrt (the MTCS form)
x = synth.normal((4, 3, 5, 5), 12, 1, 0.5, 2.0)
g = synth.uniform((3,), 12, 2) + 0.5
b = synth.normal((3,), 12, 3)
dy = synth.normal((4, 3, 5, 5), 12, 4)
xt, gt, bt = t(x, True), t(g, True), t(b, True)
mean = xt.mean(dim=(0, 2, 3), keepdim=True)
var = ((xt - mean) ** 2).mean(dim=(0, 2, 3), keepdim=True)
y = (xt - mean) / torch.sqrt(var + 1e-5) * gt.view(1, 3, 1, 1) + bt.view(1, 3, 1, 1)
y.backward(t(dy))
out.update(bn_x=x, bn_g=g, bn_b=b, bn_dy=dy, bn_y=y.detach().numpy(), bn_mean=mean.detach().numpy().ravel(),
           bn_var=var.detach().numpy().ravel(), bn_dx=xt.grad.numpy(), bn_dg=gt.grad.numpy(), bn_db=bt.grad.numpy())

# ---- max pool 2/2 and 3/2 (no padding) with argmax
for name, size, stride in [("mp2", 2, 2), ("mp3", 3, 2)]:
    x = synth.normal((2, 3, 9, 9), 13, size)
    xt = t(x, True)
    y, idx = F.max_pool2d(xt, size, stride, return_indices=True)
    dy = synth.normal(tuple(y.shape), 13, size + 10)
    y.backward(t(dy))
    out[name + "_x"], out[name + "_y"], out[name + "_idx"] = x, y.detach().numpy(), idx.numpy()
    out[name + "_dy"], out[name + "_dx"] = dy, xt.grad.numpy()

# ---- softmax + cross entropy (sum over the batch), gradient wrt logits
x = synth.normal((6, 10), 14, 1, 0, 3.0)
_, onehot = synth.labels(6, 10, 14, 2)
xt = t(x, True)
logp = F.log_softmax(xt, dim=1)
loss = -(t(onehot) * logp).sum()
loss.backward()
out.update(sm_x=x, sm_truth=onehot, sm_p=torch.softmax(t(x), 1).numpy(), sm_cost=np.array(loss.item()),
           sm_dx=xt.grad.numpy())

# ---- SGD with momentum, three steps, closed form in float64
w0 = synth.normal((50,), 15, 1)
grads = [synth.normal((50,), 15, 2 + i) for i in range(3)]
w, u = w0.astype(np.float64), np.zeros(50)
lr, mom, decay, B = 0.1, 0.9, 5e-4, 8
for gi in grads:
    u = u + gi            # backward accumulates into the momentum buffer
    u = u - decay * B * w
    w = w + lr / B * u
    u = u * mom
out.update(sgd_w0=w0, sgd_g=np.stack(grads), sgd_w=w, sgd_u=u, sgd_h=np.array([lr, mom, decay, B]))

np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "ops_f64.npz"), **out)
print("wrote", len(out), "arrays")
