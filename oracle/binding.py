"""TEST INFRASTRUCTURE ONLY -- ctypes binding of the CPU oracle (oracle/aet_oracle.c).

Imported by tests/, by ``__graft_entry__.smoke()`` and by the CPU-baseline legs of
``bench.py``; the product package never imports it.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LINEAR, RELU, LEAKY, LOGISTIC, RELU6, RELIE, RAMP, TANH, PLSE, ELU, LOGGY, HARDTAN, LHTAN, SELU, SWISH, MISH = range(16)
MODE_CPU, MODE_MTCS = 0, 1
CONV, MAXPOOL, AVGPOOL, SOFTMAX, DROPOUT, SHORTCUT = 0, 1, 2, 3, 4, 5
(P_WEIGHTS, P_WEIGHT_UPDATES, P_BIASES, P_BIAS_UPDATES, P_SCALES, P_SCALE_UPDATES, P_ROLLING_MEAN,
 P_ROLLING_VARIANCE, P_MEAN, P_VARIANCE, P_OUTPUT, P_DELTA, P_X, P_X_NORM, P_INDEXES, P_LOSS, P_RAND) = range(17)

_f = C.POINTER(C.c_float)
_i = C.POINTER(C.c_int)


class LayerSpec(C.Structure):
    _fields_ = [("type", C.c_int), ("filters", C.c_int), ("size", C.c_int), ("stride_x", C.c_int),
                ("stride_y", C.c_int), ("pad", C.c_int), ("batch_normalize", C.c_int), ("activation", C.c_int),
                ("probability", C.c_float), ("temperature", C.c_float), ("groups", C.c_int),
                ("learning_rate_scale", C.c_float), ("n_from", C.c_int), ("from_", C.c_int * 4),
                ("stopbackward", C.c_int), ("dont_update", C.c_int)]


def build(variant="parity"):
    """Compile the oracle with its Makefile; 'fast' uses the reference's flags for timing."""
    target = "fast" if variant == "fast" else "all"
    subprocess.run(["make", "-s", "-C", HERE, target], check=True)


def _fp(a):
    return a.ctypes.data_as(_f)


def _arr(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class Oracle:
    """One loaded build of the oracle: 'parity' (default), 'acc64' or 'fast'."""

    def __init__(self, variant="parity"):
        name = {"parity": "libaet_oracle.so", "acc64": "libaet_oracle_acc64.so", "fast": "libaet_oracle_fast.so"}[variant]
        path = os.path.join(HERE, "_build", name)
        build("fast" if variant == "fast" else "parity")   # make rebuilds only what is older than its sources
        L = self.lib = C.CDLL(path)
        L.aeto_gemm.argtypes = [C.c_int] * 5 + [C.c_float, _f, C.c_int, _f, C.c_int, C.c_float, _f, C.c_int]
        L.aeto_im2col.argtypes = [_f] + [C.c_int] * 9 + [_f]
        L.aeto_col2im.argtypes = [_f] + [C.c_int] * 9 + [_f]
        L.aeto_conv_out.argtypes = [C.c_int] * 4
        L.aeto_conv_workspace.argtypes = [C.c_int] * 7
        L.aeto_conv_workspace.restype = C.c_size_t
        L.aeto_conv_forward.argtypes = [_f, _f, _f, _f] + [C.c_int] * 9
        L.aeto_conv_backward.argtypes = [_f, _f, _f, _f, _f, _f] + [C.c_int] * 9
        L.aeto_conv_forward_ex.argtypes = [_f, _f, _f, _f] + [C.c_int] * 11
        L.aeto_conv_backward_ex.argtypes = [_f, _f, _f, _f, _f, _f] + [C.c_int] * 11
        L.aeto_add_bias.argtypes = [_f, _f, C.c_int, C.c_int, C.c_int]
        L.aeto_backward_bias.argtypes = [_f, _f, C.c_int, C.c_int, C.c_int]
        L.aeto_activate.argtypes = [_f, C.c_size_t, C.c_int, C.c_int]
        L.aeto_gradient.argtypes = [_f, C.c_size_t, C.c_int, _f]
        L.aeto_bn_forward.argtypes = [C.c_int, C.c_int, _f, C.c_int, C.c_int, C.c_int] + [_f] * 8
        L.aeto_bn_backward.argtypes = [C.c_int] + [_f] * 10 + [C.c_int] * 3
        L.aeto_maxpool_out.argtypes = [C.c_int] * 4
        L.aeto_maxpool_forward.argtypes = [C.c_int, _f, _f, _i] + [C.c_int] * 8
        L.aeto_maxpool_backward.argtypes = [_f, _i, _f, C.c_size_t]
        L.aeto_avgpool_forward.argtypes = [_f, _f, C.c_int, C.c_int, C.c_int]
        L.aeto_avgpool_backward.argtypes = [_f, _f, C.c_int, C.c_int, C.c_int]
        L.aeto_softmax_forward.argtypes = [C.c_int, _f, _f, _f, _f, _f, C.c_int, C.c_int, C.c_int, C.c_float]
        L.aeto_softmax_forward.restype = C.c_float
        L.aeto_softmax_backward.argtypes = [_f, _f, C.c_size_t, C.c_float]
        L.aeto_dropout_forward.argtypes = [_f, _f, C.c_size_t, C.c_float]
        L.aeto_dropout_backward.argtypes = [_f, _f, C.c_size_t, C.c_float]
        L.aeto_gradient_input.argtypes = [_f, _f, C.c_size_t, C.c_int, _f]
        L.aeto_shortcut_forward.argtypes = [_f, _f, C.c_int, C.c_size_t, C.c_int, C.POINTER(_f), C.POINTER(C.c_size_t)]
        L.aeto_shortcut_backward.argtypes = [_f, _f, C.c_int, C.c_size_t, C.c_int, C.POINTER(_f), C.POINTER(C.c_size_t)]
        L.aeto_sgd_weights.argtypes = [_f, _f, C.c_size_t, C.c_int, C.c_float, C.c_float, C.c_float]
        L.aeto_sgd_plain.argtypes = [_f, _f, C.c_size_t, C.c_int, C.c_float, C.c_float]
        L.aeto_net_create.argtypes = [C.POINTER(LayerSpec)] + [C.c_int] * 7
        L.aeto_net_create.restype = C.c_void_p
        L.aeto_net_free.argtypes = [C.c_void_p]
        L.aeto_net_param.argtypes = [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_size_t)]
        L.aeto_net_param.restype = C.c_void_p
        L.aeto_net_out_shape.argtypes = [C.c_void_p, C.c_int, _i, _i, _i]
        L.aeto_net_forward.argtypes = [C.c_void_p, _f, _f, C.c_int]
        L.aeto_net_backward.argtypes = [C.c_void_p, _f, _f]
        L.aeto_net_update.argtypes = [C.c_void_p, C.c_int, C.c_float, C.c_float, C.c_float]
        L.aeto_net_cost.argtypes = [C.c_void_p]
        L.aeto_net_cost.restype = C.c_float
        L.aeto_net_train_step.argtypes = [C.c_void_p, _f, _f, C.c_float, C.c_float, C.c_float]
        L.aeto_net_train_step.restype = C.c_float
        L.aeto_current_rate.argtypes = [C.c_size_t, C.c_int, C.c_float, C.c_int, C.c_float, C.c_int, C.c_float, _i, _f, C.c_int,
                                        C.c_float, C.c_int]
        L.aeto_current_rate.restype = C.c_float
        L.aeto_fix_nan_and_inf.argtypes = [_f, C.c_size_t]
        L.aeto_reset_nan_and_inf.argtypes = [_f, C.c_size_t]
        L.aeto_fuse_conv_batchnorm.argtypes = [_f, _f, _f, _f, _f, C.c_int, C.c_size_t]
        L.aeto_top_k.argtypes = [_f, C.c_int, C.c_int, _i]
        L.aeto_transpose_matrix.argtypes = [_f, C.c_int, C.c_int]
        L.aeto_augment_image.argtypes = [_f, C.c_int, C.c_int, C.c_int, _f, C.c_int] + [C.c_float] * 5 + [C.c_int] + [C.c_float] * 3
        L.aeto_adam_update.argtypes = [_f, _f, _f, _f, C.c_float, C.c_float, C.c_float, C.c_float, C.c_float, C.c_size_t, C.c_int, C.c_int]
        L.aeto_fill_uniform.argtypes = [_f, C.c_size_t, C.c_uint64, C.c_uint64]
        L.aeto_fill_normal.argtypes = [_f, C.c_size_t, C.c_uint64, C.c_uint64, C.c_float, C.c_float]

    # ---- synthetic tensors ----
    def uniform(self, shape, seed, tensor_id):
        a = np.empty(shape, np.float32)
        self.lib.aeto_fill_uniform(_fp(a), a.size, seed, tensor_id)
        return a

    def normal(self, shape, seed, tensor_id, mean=0.0, std=1.0):
        a = np.empty(shape, np.float32)
        self.lib.aeto_fill_normal(_fp(a), a.size, seed, tensor_id, mean, std)
        return a

    # ---- single operators (NCHW numpy in, numpy out) ----
    def conv_out(self, n, size, stride, pad):
        return self.lib.aeto_conv_out(n, size, stride, pad)

    def conv_forward(self, x, w, stride_x=1, stride_y=None, pad=0, groups=1, dilation=1):
        stride_y = stride_x if stride_y is None else stride_y
        x, w = _arr(x), _arr(w)
        b, c, h, wd = x.shape
        n, _, size, _ = w.shape
        oh, ow = self.conv_out(h, size, stride_y, pad), self.conv_out(wd, size, stride_x, pad)
        y = np.zeros((b, n, oh, ow), np.float32)
        ws = np.zeros(max(1, self.lib.aeto_conv_workspace(c, h, wd, size, stride_x, stride_y, pad)), np.float32)
        if groups == 1 and dilation == 1:
            self.lib.aeto_conv_forward(_fp(x), _fp(w), _fp(y), _fp(ws), b, c, h, wd, n, size, stride_x, stride_y, pad)
        else:
            self.lib.aeto_conv_forward_ex(_fp(x), _fp(w), _fp(y), _fp(ws), b, c, h, wd, n, size, stride_x, stride_y, pad, groups, dilation)
        return y

    def conv_backward(self, x, w, delta, stride_x=1, stride_y=None, pad=0, dw=None, need_dx=True, groups=1, dilation=1):
        stride_y = stride_x if stride_y is None else stride_y
        x, w, delta = _arr(x), _arr(w), _arr(delta)
        b, c, h, wd = x.shape
        n, _, size, _ = w.shape
        dw = np.zeros_like(w) if dw is None else _arr(dw).copy()
        dx = np.zeros_like(x) if need_dx else None
        ws = np.zeros(max(1, self.lib.aeto_conv_workspace(c, h, wd, size, stride_x, stride_y, pad)), np.float32)
        if groups == 1 and dilation == 1:
            self.lib.aeto_conv_backward(_fp(x), _fp(w), _fp(delta), _fp(dw), _fp(dx) if need_dx else None, _fp(ws),
                                        b, c, h, wd, n, size, stride_x, stride_y, pad)
        else:
            self.lib.aeto_conv_backward_ex(_fp(x), _fp(w), _fp(delta), _fp(dw), _fp(dx) if need_dx else None, _fp(ws),
                                           b, c, h, wd, n, size, stride_x, stride_y, pad, groups, dilation)
        return dw, dx

    def add_bias(self, y, b):
        y = _arr(y).copy()
        n, c = y.shape[:2]
        self.lib.aeto_add_bias(_fp(y), _fp(_arr(b)), n, c, y[0, 0].size)
        return y

    def backward_bias(self, delta, db=None):
        delta = _arr(delta)
        n, c = delta.shape[:2]
        db = np.zeros(c, np.float32) if db is None else _arr(db).copy()
        self.lib.aeto_backward_bias(_fp(db), _fp(delta), n, c, delta[0, 0].size)
        return db

    def activate(self, y, activation, mode=MODE_CPU):
        y = _arr(y).copy()
        self.lib.aeto_activate(_fp(y), y.size, activation, mode)
        return y

    def gradient(self, y, activation, delta):
        d = _arr(delta).copy()
        self.lib.aeto_gradient(_fp(_arr(y)), d.size, activation, _fp(d))
        return d

    def gradient_input(self, y, v, activation, delta):
        """swish / mish: delta * f'(v) from the output y and the value before the activation v."""
        d = _arr(delta).copy()
        self.lib.aeto_gradient_input(_fp(_arr(y)), _fp(_arr(v)), d.size, activation, _fp(d))
        return d

    def bn_forward(self, mode, train, x, scales, biases, rolling_mean, rolling_variance):
        y = _arr(x).copy()
        b, c = y.shape[:2]
        sp = y[0, 0].size
        mean, var = np.zeros(c, np.float32), np.zeros(c, np.float32)
        rm, rv = _arr(rolling_mean).copy(), _arr(rolling_variance).copy()
        xs, xn = np.zeros_like(y), np.zeros_like(y)
        self.lib.aeto_bn_forward(mode, int(train), _fp(y), b, c, sp, _fp(_arr(scales)), _fp(_arr(biases)), _fp(mean),
                                 _fp(var), _fp(rm), _fp(rv), _fp(xs), _fp(xn))
        return dict(y=y, mean=mean, variance=var, rolling_mean=rm, rolling_variance=rv, x=xs, x_norm=xn)

    def bn_backward(self, mode, delta, x, x_norm, mean, variance, scales, scale_updates=None, bias_updates=None):
        d = _arr(delta).copy()
        b, c = d.shape[:2]
        sp = d[0, 0].size
        ds = np.zeros(c, np.float32) if scale_updates is None else _arr(scale_updates).copy()
        db = np.zeros(c, np.float32) if bias_updates is None else _arr(bias_updates).copy()
        md, vd = np.zeros(c, np.float32), np.zeros(c, np.float32)
        self.lib.aeto_bn_backward(mode, _fp(d), _fp(_arr(x)), _fp(_arr(x_norm)), _fp(_arr(mean)), _fp(_arr(variance)),
                                  _fp(_arr(scales)), _fp(ds), _fp(db), _fp(md), _fp(vd), b, c, sp)
        return dict(delta=d, scale_updates=ds, bias_updates=db, mean_delta=md, variance_delta=vd)

    def maxpool_forward(self, mode, x, size, stride_x, stride_y, padding):
        x = _arr(x)
        b, c, h, w = x.shape
        oh = self.lib.aeto_maxpool_out(h, size, stride_y, padding)
        ow = self.lib.aeto_maxpool_out(w, size, stride_x, padding)
        y = np.zeros((b, c, oh, ow), np.float32)
        idx = np.zeros((b, c, oh, ow), np.int32)
        self.lib.aeto_maxpool_forward(mode, _fp(x), _fp(y), idx.ctypes.data_as(_i), b, c, h, w, size, stride_x,
                                      stride_y, padding)
        return y, idx

    def maxpool_backward(self, delta, idx, prev_delta):
        pd = _arr(prev_delta).copy()
        idx = np.ascontiguousarray(idx, np.int32)
        self.lib.aeto_maxpool_backward(_fp(_arr(delta)), idx.ctypes.data_as(_i), _fp(pd), idx.size)
        return pd

    def avgpool_forward(self, x):
        x = _arr(x)
        b, c = x.shape[:2]
        y = np.zeros((b, c), np.float32)
        self.lib.aeto_avgpool_forward(_fp(x), _fp(y), b, c, x[0, 0].size)
        return y

    def avgpool_backward(self, delta, prev_delta):
        pd = _arr(prev_delta).copy()
        b, c = pd.shape[:2]
        self.lib.aeto_avgpool_backward(_fp(_arr(delta)), _fp(pd), b, c, pd[0, 0].size)
        return pd

    def softmax_forward(self, mode, x, truth, groups=1, temperature=1.0):
        x = _arr(x).reshape(x.shape[0], -1)
        b, n = x.shape
        p, d, loss = np.zeros_like(x), np.zeros_like(x), np.zeros_like(x)
        cost = self.lib.aeto_softmax_forward(mode, _fp(x), _fp(p), _fp(_arr(truth)) if truth is not None else None,
                                             _fp(d), _fp(loss), b, n, groups, temperature)
        return dict(p=p, delta=d, loss=loss, cost=cost)

    def sgd_weights(self, w, u, batch, lr, momentum, decay):
        w, u = _arr(w).copy(), _arr(u).copy()
        self.lib.aeto_sgd_weights(_fp(w), _fp(u), w.size, batch, lr, momentum, decay)
        return w, u

    def sgd_plain(self, p, u, batch, lr, momentum):
        p, u = _arr(p).copy(), _arr(u).copy()
        self.lib.aeto_sgd_plain(_fp(p), _fp(u), p.size, batch, lr, momentum)
        return p, u

    def current_rate(self, batch_num, policy, learning_rate, burn_in=0, power=4.0, step=1, scale=1.0, steps=(), scales=(),
                     gamma=1.0, max_batches=0):
        """NNetwork.getCurrentRate; policy 0 constant, 1 step, 2 steps, 3 exp, 4 poly, 5 sig."""
        st = np.ascontiguousarray(steps, np.int32)
        sc = np.ascontiguousarray(scales, np.float32)
        n = min(st.size, sc.size)
        return self.lib.aeto_current_rate(batch_num, policy, learning_rate, burn_in, power, step, scale,
                                          st.ctypes.data_as(_i) if n else None, _fp(sc) if n else None, n, gamma, max_batches)

    def fix_nan_and_inf(self, v):
        v = _arr(v).copy().reshape(-1)
        self.lib.aeto_fix_nan_and_inf(_fp(v), v.size)
        return v

    def reset_nan_and_inf(self, v):
        v = _arr(v).copy().reshape(-1)
        self.lib.aeto_reset_nan_and_inf(_fp(v), v.size)
        return v

    def fuse_conv_batchnorm(self, biases, scales, rolling_mean, rolling_variance, weights):
        """Returns (biases, weights) after ConvolutionalLayer.fuseConvBatchnorm; weights [filters][...]."""
        b, w = _arr(biases).copy(), _arr(weights).copy()
        self.lib.aeto_fuse_conv_batchnorm(_fp(b), _fp(_arr(scales)), _fp(_arr(rolling_mean)), _fp(_arr(rolling_variance)),
                                          _fp(w), b.size, w.size // b.size)
        return b, w

    def top_k(self, a, k):
        a = _arr(a).reshape(-1)
        idx = np.zeros(k, np.int32)
        self.lib.aeto_top_k(_fp(a), a.size, k, idx.ctypes.data_as(_i))
        return idx

    def transpose_matrix(self, a, rows, cols):
        a = _arr(a).copy().reshape(-1)
        self.lib.aeto_transpose_matrix(_fp(a), rows, cols)
        return a

    def augment_image(self, src, size, rad, scale, dx, dy, aspect, flip, dhue, dsat, dexp):
        """rotateCrop + flip + distort of one image [c][sh][sw] into [c][size][size] (dnn/NImage.c)."""
        src = _arr(src)
        c, sh, sw = src.shape
        dst = np.zeros((c, size, size), np.float32)
        self.lib.aeto_augment_image(_fp(src), c, sh, sw, _fp(dst), size, rad, scale, dx, dy, aspect, int(flip), dhue, dsat, dexp)
        return dst

    def adam_update(self, w, d, m, v, B1, B2, eps, decay, rate, batch, t):
        """In place on float32 numpy arrays (views of the oracle network's storage are fine)."""
        self.lib.aeto_adam_update(_fp(w), _fp(d), _fp(m), _fp(v), B1, B2, eps, decay, rate, w.size, batch, t)

    def dropout_forward(self, x, r, probability):
        x = _arr(x).copy()
        self.lib.aeto_dropout_forward(_fp(x), _fp(_arr(r)), x.size, probability)
        return x

    def shortcut_forward(self, x, adds):
        """x: [batch, outputs]; adds: list of [batch, outputs_i].  Returns input + sources, before the activation."""
        x = _arr(x)
        adds = [_arr(a) for a in adds]
        out = np.empty_like(x)
        ptrs = (_f * len(adds))(*[_fp(a) for a in adds])
        sizes = (C.c_size_t * len(adds))(*[a.shape[1] for a in adds])
        self.lib.aeto_shortcut_forward(_fp(x), _fp(out), x.shape[0], x.shape[1], len(adds), ptrs, sizes)
        return out

    def shortcut_backward(self, delta, delta_out, layer_deltas):
        """Adds delta [batch, outputs] into delta_out (or None) and into every layer_deltas[i] [batch, outputs_i], in place."""
        delta = _arr(delta)
        ptrs = (_f * len(layer_deltas))(*[_fp(a) for a in layer_deltas])
        sizes = (C.c_size_t * len(layer_deltas))(*[a.shape[1] for a in layer_deltas])
        self.lib.aeto_shortcut_backward(_fp(delta), _fp(delta_out) if delta_out is not None else None, delta.shape[0],
                                        delta.shape[1], len(layer_deltas), ptrs, sizes)

    def net(self, specs, batch, c, h, w, mode=MODE_MTCS, threads=1):
        return OracleNet(self, specs, batch, c, h, w, mode, threads)


class OracleNet:
    """Whole-network oracle; ``specs`` is a list of dicts with the LayerSpec field names."""

    def __init__(self, oracle, specs, batch, c, h, w, mode, threads):
        self.o, self.lib = oracle, oracle.lib
        arr = (LayerSpec * len(specs))()
        for s, d in zip(arr, specs):
            for k, v in d.items():
                if k == "from":
                    s.n_from = len(v)
                    for q, idx in enumerate(v):
                        s.from_[q] = idx
                else:
                    setattr(s, k, v)
            if not s.stride_y:
                s.stride_y = s.stride_x
        self.n, self.batch = len(specs), batch
        self.in_shape = (batch, c, h, w)
        self.h = self.lib.aeto_net_create(arr, len(specs), batch, c, h, w, mode, threads)

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.aeto_net_free(self.h)
            self.h = None

    def out_shape(self, layer):
        c, h, w = C.c_int(), C.c_int(), C.c_int()
        self.lib.aeto_net_out_shape(self.h, layer, C.byref(c), C.byref(h), C.byref(w))
        return (self.batch, c.value, h.value, w.value)

    def param(self, layer, which):
        """A live numpy view (float32, or int32 for indexes) of the oracle's storage."""
        cnt = C.c_size_t()
        p = self.lib.aeto_net_param(self.h, layer, which, C.byref(cnt))
        if not p or cnt.value == 0:
            return None
        ctype = C.c_int if which == P_INDEXES else C.c_float
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(ctype)), shape=(cnt.value,))

    def set_param(self, layer, which, value):
        v = self.param(layer, which)
        v[:] = np.asarray(value).reshape(-1)

    def forward(self, x, truth, train=True):
        self.lib.aeto_net_forward(self.h, _fp(_arr(x)), _fp(_arr(truth)) if truth is not None else None, int(train))

    def backward(self, x, input_delta=None):
        self.lib.aeto_net_backward(self.h, _fp(_arr(x)), _fp(input_delta) if input_delta is not None else None)

    def update(self, update_batch, lr, momentum, decay):
        self.lib.aeto_net_update(self.h, update_batch, lr, momentum, decay)

    def cost(self):
        return self.lib.aeto_net_cost(self.h)

    def train_step(self, x, truth, lr, momentum, decay):
        return self.lib.aeto_net_train_step(self.h, _fp(_arr(x)), _fp(_arr(truth)), lr, momentum, decay)
