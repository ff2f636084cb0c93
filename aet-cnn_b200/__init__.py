"""Host-side mirror of the AET-CNN layer / network interface over libaet_b200.so.

The compute lives entirely in the CUDA library behind the C ABI declared in
``include/aet_b200.h``; this module only binds it with ctypes and keeps the reference's
names (``ConvolutionalLayer.forward(state)``, ``NNetwork.train`` ...).  There is no CPU
path: if the library is missing, or no sm_100 device is present, construction raises.

The directory name contains a hyphen, so load it with importlib under the module name
``aet_cnn_b200`` (see ``load()`` in tests/conftest.py, bench.py and __graft_entry__.py).
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libaet_b200.so")
CFG_DIR = os.path.join(HERE, "cfg")

LINEAR, RELU, LEAKY, LOGISTIC, RELU6, RELIE, RAMP, TANH, PLSE, ELU, LOGGY, HARDTAN, LHTAN, SELU, SWISH, MISH = range(16)
CONVOLUTIONAL, MAXPOOL, AVGPOOL, SOFTMAX, DROPOUT, SHORTCUT = 0, 1, 2, 3, 4, 5
PARITY_CPU, PARITY_MTCS = 0, 1
MATH_TF32, MATH_3XTF32 = 0, 1
(P_WEIGHTS, P_WEIGHT_UPDATES, P_BIASES, P_BIAS_UPDATES, P_SCALES, P_SCALE_UPDATES, P_ROLLING_MEAN,
 P_ROLLING_VARIANCE, P_MEAN, P_VARIANCE, P_OUTPUT, P_DELTA, P_X, P_X_NORM, P_INDEXES, P_LOSS, P_RAND) = range(17)

# every symbol include/aet_b200.h declares
EXPORTS = """aet_last_error aet_version aet_context_create aet_context_destroy aet_context_set_stream
aet_context_stream aet_context_set_parity aet_context_set_math aet_context_synchronize aet_context_check
aet_context_profile aet_context_profile_read aet_context_launch_count aet_context_set_option aet_context_get_option aet_context_set_wait_limit aet_context_wait_probe
aet_tensor_create aet_tensor_destroy aet_tensor_shape aet_tensor_write aet_tensor_read aet_tensor_zero
aet_tensor_count aet_convolutional_layer_create aet_maxpool_layer_create aet_avgpool_layer_create
aet_softmax_layer_create aet_dropout_layer_create aet_shortcut_layer_create aet_layer_destroy aet_layer_forward aet_layer_backward
aet_layer_update aet_layer_init_delta aet_layer_output aet_layer_delta aet_layer_kind aet_layer_out_shape
aet_layer_cost aet_layer_param_count aet_layer_read aet_layer_write aet_layer_load_weights
aet_layer_save_weights aet_network_create aet_network_create_from_string aet_network_create_ex
aet_network_destroy aet_network_layer_count aet_network_layer aet_network_batch aet_network_input_shape
aet_network_outputs aet_network_input aet_network_truth aet_network_learning_rate aet_network_set_hyper
aet_network_seen aet_network_forward aet_network_backward aet_network_update aet_network_cost
aet_network_augment_input aet_network_fuse_conv_batchnorm aet_network_predict_topk aet_network_validate aet_network_train_step aet_network_train_step_async aet_network_train_step_device aet_network_last_loss aet_network_predict
aet_network_use_graph aet_network_load_weights aet_network_load_weights_upto aet_network_save_weights aet_network_load_momentum aet_network_save_momentum aet_network_comm_exposed aet_network_param_hash
aet_network_profile aet_network_profile_read aet_network_launches_per_step aet_comm_unique_id
aet_network_comm_init aet_network_comm_destroy aet_network_grad_arena aet_backward_bias_static
aet_network_comm_exchange_export aet_network_comm_exchange_attach aet_network_comm_exchange_detach""".split()


class AetError(RuntimeError):
    pass


class State(C.Structure):
    """dnn/NLayer.h:21-29 NetworkState."""
    _fields_ = [("truth", C.c_void_p), ("input", C.c_void_p), ("delta", C.c_void_p), ("workspace", C.c_void_p),
                ("train", C.c_int), ("index", C.c_int)]


class Augment(C.Structure):
    """aet_augment: the per-image draws of the reference's augmentation chain."""
    _fields_ = [("rad", C.c_float), ("scale", C.c_float), ("dx", C.c_float), ("dy", C.c_float), ("aspect", C.c_float),
                ("flip", C.c_int), ("dhue", C.c_float), ("dsat", C.c_float), ("dexp", C.c_float)]


class KernelTime(C.Structure):
    _fields_ = [("name", C.c_char * 48), ("launches", C.c_int), ("total_ms", C.c_double), ("algo_bytes", C.c_double),
                ("algo_flops", C.c_double), ("span_ms", C.c_double)]


_lib = None


def lib():
    """Loads the C-ABI library once; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise AetError("libaet_b200.so is missing: build it with `python aet-cnn_b200/build.py` "
                       "(there is no fallback implementation)")
    L = C.CDLL(LIB_PATH)
    vp, i, f = C.c_void_p, C.c_int, C.c_float
    sig = {
        "aet_last_error": (C.c_char_p, []), "aet_version": (C.c_char_p, []),
        "aet_context_create": (vp, [i]), "aet_context_destroy": (None, [vp]),
        "aet_context_set_stream": (i, [vp, vp]), "aet_context_stream": (vp, [vp]),
        "aet_context_set_parity": (i, [vp, i]), "aet_context_set_math": (i, [vp, i]),
        "aet_context_synchronize": (i, [vp]), "aet_context_check": (i, [vp]),
        "aet_context_profile": (i, [vp, i]),
        "aet_context_profile_read": (i, [vp, C.POINTER(KernelTime), i, C.POINTER(i)]),
        "aet_context_launch_count": (C.c_long, [vp]),
        "aet_context_set_option": (i, [vp, C.c_char_p, i]),
        "aet_context_get_option": (i, [vp, C.c_char_p, C.POINTER(i)]),
        "aet_context_set_wait_limit": (i, [vp, C.c_ulonglong]), "aet_context_wait_probe": (i, [vp]),
        "aet_tensor_create": (vp, [vp, i, i, i, i]), "aet_tensor_destroy": (None, [vp]),
        "aet_tensor_shape": (i, [vp] + [C.POINTER(i)] * 4), "aet_tensor_write": (i, [vp, vp]),
        "aet_tensor_read": (i, [vp, vp]), "aet_tensor_zero": (i, [vp]), "aet_tensor_count": (C.c_size_t, [vp]),
        "aet_convolutional_layer_create": (vp, [vp] + [i] * 14),
        "aet_maxpool_layer_create": (vp, [vp] + [i] * 9),
        "aet_avgpool_layer_create": (vp, [vp, i, i, i, i]),
        "aet_softmax_layer_create": (vp, [vp, i, i, i, f]),
        "aet_dropout_layer_create": (vp, [vp, i, i, f, vp]),
        "aet_shortcut_layer_create": (vp, [vp, i, i, i, i, i, C.POINTER(vp), i, i]),
        "aet_layer_destroy": (None, [vp]),
        "aet_layer_forward": (i, [vp, State]), "aet_layer_backward": (i, [vp, State]),
        "aet_layer_update": (i, [vp, i, f, f, f, f]), "aet_layer_init_delta": (i, [vp]),
        "aet_layer_output": (vp, [vp]), "aet_layer_delta": (vp, [vp]), "aet_layer_kind": (i, [vp]),
        "aet_layer_out_shape": (i, [vp] + [C.POINTER(i)] * 3), "aet_layer_cost": (f, [vp]),
        "aet_layer_param_count": (C.c_size_t, [vp, i]), "aet_layer_read": (i, [vp, i, vp]),
        "aet_layer_write": (i, [vp, i, vp]), "aet_layer_load_weights": (i, [vp, vp]),
        "aet_layer_save_weights": (i, [vp, vp]),
        "aet_network_create": (vp, [vp, C.c_char_p, i]),
        "aet_network_create_from_string": (vp, [vp, C.c_char_p, i]),
        "aet_network_create_ex": (vp, [vp, C.c_char_p, i, i]),
        "aet_network_destroy": (None, [vp]), "aet_network_layer_count": (i, [vp]),
        "aet_network_layer": (vp, [vp, i]), "aet_network_batch": (i, [vp]),
        "aet_network_input_shape": (i, [vp] + [C.POINTER(i)] * 3), "aet_network_outputs": (i, [vp]),
        "aet_network_input": (vp, [vp]), "aet_network_truth": (vp, [vp]),
        "aet_network_learning_rate": (f, [vp]), "aet_network_set_hyper": (i, [vp, f, f, f]),
        "aet_network_seen": (C.c_int64, [vp]),
        "aet_network_forward": (i, [vp, State]), "aet_network_backward": (i, [vp, State]),
        "aet_network_update": (i, [vp]), "aet_network_cost": (f, [vp]),
        "aet_network_train_step": (i, [vp, vp, vp, C.POINTER(f)]),
        "aet_network_train_step_device": (i, [vp, C.POINTER(f)]),
        "aet_network_train_step_async": (i, [vp, vp, vp, C.POINTER(f)]),
        "aet_network_last_loss": (i, [vp, C.POINTER(f)]),
        "aet_network_predict": (i, [vp, vp, vp]),
        "aet_network_augment_input": (i, [vp, vp, i, i, vp]),
        "aet_network_fuse_conv_batchnorm": (i, [vp]), "aet_network_predict_topk": (i, [vp, vp, i, vp]),
        "aet_network_validate": (i, [vp, vp, vp, i, i, C.POINTER(f), C.POINTER(f)]), "aet_network_use_graph": (i, [vp, i]),
        "aet_network_load_weights": (i, [vp, C.c_char_p]), "aet_network_load_weights_upto": (i, [vp, C.c_char_p, i]), "aet_network_save_weights": (i, [vp, C.c_char_p]),
        "aet_network_load_momentum": (i, [vp, C.c_char_p]), "aet_network_save_momentum": (i, [vp, C.c_char_p]),
        "aet_network_comm_exposed": (i, [vp, C.POINTER(C.c_double), C.POINTER(C.c_longlong)]),
        "aet_network_param_hash": (i, [vp, C.POINTER(C.c_uint64)]),
        "aet_network_profile": (i, [vp, i]),
        "aet_network_profile_read": (i, [vp, C.POINTER(KernelTime), i, C.POINTER(i)]),
        "aet_network_launches_per_step": (i, [vp]),
        "aet_comm_unique_id": (i, [vp]), "aet_network_comm_init": (i, [vp, vp, i, i]),
        "aet_network_comm_exchange_export": (i, [vp, vp]), "aet_network_comm_exchange_attach": (i, [vp, vp]), "aet_network_comm_exchange_detach": (i, [vp]),
        "aet_network_comm_destroy": (i, [vp]),
        "aet_network_grad_arena": (i, [vp, C.POINTER(vp), C.POINTER(C.c_size_t)]),
        "aet_backward_bias_static": (i, [vp, vp, C.c_longlong, i, vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)      # AttributeError here = the library does not export a declared symbol
        fn.restype, fn.argtypes = res, args
    _lib = L
    return L


def _check(code):
    if code != 0:
        raise AetError("aet error %d: %s" % (code, lib().aet_last_error().decode()))


def _need(handle):
    if not handle:
        raise AetError(lib().aet_last_error().decode() or "null handle")
    return handle


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class Context:
    """One device + stream (replaces the reference's MtcsTool / MtcsStream singletons)."""

    def __init__(self, device=0, parity=PARITY_MTCS, math=MATH_TF32, stream=None):
        self.L = lib()
        self.h = _need(self.L.aet_context_create(device))
        _check(self.L.aet_context_set_parity(self.h, parity))
        _check(self.L.aet_context_set_math(self.h, math))
        if stream is not None:
            _check(self.L.aet_context_set_stream(self.h, C.c_void_p(stream)))

    def set_parity(self, parity):
        _check(self.L.aet_context_set_parity(self.h, parity))

    def set_math(self, math):
        _check(self.L.aet_context_set_math(self.h, math))

    def set_option(self, name, value):
        """Behaviour switch by name (kernel choice, fusions, stream overlap); see include/aet_b200.h."""
        _check(self.L.aet_context_set_option(self.h, name.encode(), int(value)))

    def get_option(self, name):
        v = C.c_int()
        _check(self.L.aet_context_get_option(self.h, name.encode(), C.byref(v)))
        return v.value

    def set_wait_limit(self, nanoseconds):
        _check(self.L.aet_context_set_wait_limit(self.h, int(nanoseconds)))

    def wait_probe(self):
        _check(self.L.aet_context_wait_probe(self.h))

    def synchronize(self):
        _check(self.L.aet_context_synchronize(self.h))

    def check(self):
        _check(self.L.aet_context_check(self.h))

    def profile(self, enable):
        _check(self.L.aet_context_profile(self.h, int(enable)))

    def profile_read(self, capacity=128):
        tab = (KernelTime * capacity)()
        n = C.c_int()
        _check(self.L.aet_context_profile_read(self.h, tab, capacity, C.byref(n)))
        return [dict(name=t.name.decode(), launches=t.launches, total_ms=t.total_ms, span_ms=t.span_ms, algo_bytes=t.algo_bytes,
                     algo_flops=t.algo_flops) for t in tab[:n.value]]

    def launch_count(self):
        return self.L.aet_context_launch_count(self.h)

    def close(self):
        if self.h:
            self.L.aet_context_destroy(self.h)
            self.h = None


class Tensor:
    """NData / IOData / DeltaData / TruthData: FP32, host view NCHW."""

    def __init__(self, ctx, batch=None, c=None, h=1, w=1, handle=None):
        self.ctx, self.L = ctx, ctx.L
        self.owned = handle is None
        self.h = handle if handle is not None else _need(self.L.aet_tensor_create(ctx.h, batch, c, h, w))

    @property
    def shape(self):
        v = [C.c_int() for _ in range(4)]
        _check(self.L.aet_tensor_shape(self.h, *[C.byref(x) for x in v]))
        return tuple(x.value for x in v)

    def write(self, host):
        a = _f32(host)
        if a.size != self.L.aet_tensor_count(self.h):
            raise AetError("tensor write: size mismatch")
        _check(self.L.aet_tensor_write(self.h, a.ctypes.data_as(C.c_void_p)))

    def read(self):
        a = np.empty(self.shape, np.float32)
        _check(self.L.aet_tensor_read(self.h, a.ctypes.data_as(C.c_void_p)))
        return a

    def zero(self):
        _check(self.L.aet_tensor_zero(self.h))

    def close(self):
        if self.owned and self.h:
            self.L.aet_tensor_destroy(self.h)
        self.h = None


def make_state(input=None, delta=None, truth=None, train=1, index=0):
    s = State()
    s.input = input.h if input is not None else None
    s.delta = delta.h if delta is not None else None
    s.truth = truth.h if truth is not None else None
    s.workspace = None
    s.train, s.index = train, index
    return s


class Layer:
    """NLayer: forward / backward / update plus parameter taps."""

    def __init__(self, ctx, handle, owned=True):
        self.ctx, self.L, self.h, self.owned = ctx, ctx.L, _need(handle), owned

    def forward(self, state):
        _check(self.L.aet_layer_forward(self.h, state))

    def backward(self, state):
        _check(self.L.aet_layer_backward(self.h, state))

    def update(self, batch, learning_rate, momentum, decay, loss_scale=1.0):
        _check(self.L.aet_layer_update(self.h, batch, learning_rate, momentum, decay, loss_scale))

    def init_delta(self):
        _check(self.L.aet_layer_init_delta(self.h))

    @property
    def output(self):
        return Tensor(self.ctx, handle=self.L.aet_layer_output(self.h))

    @property
    def delta(self):
        return Tensor(self.ctx, handle=self.L.aet_layer_delta(self.h))

    @property
    def kind(self):
        return self.L.aet_layer_kind(self.h)

    @property
    def out_shape(self):
        v = [C.c_int() for _ in range(3)]
        _check(self.L.aet_layer_out_shape(self.h, *[C.byref(x) for x in v]))
        return tuple(x.value for x in v)

    def cost(self):
        return self.L.aet_layer_cost(self.h)

    def param_count(self, which):
        return self.L.aet_layer_param_count(self.h, which)

    def read(self, which):
        n = self.param_count(which)
        if n == 0:
            return None
        a = np.empty(n, np.int32 if which == P_INDEXES else np.float32)
        _check(self.L.aet_layer_read(self.h, which, a.ctypes.data_as(C.c_void_p)))
        return a

    def write(self, which, host):
        a = _f32(host).reshape(-1)
        if a.size != self.param_count(which):
            raise AetError("layer write: expected %d values, got %d" % (self.param_count(which), a.size))
        _check(self.L.aet_layer_write(self.h, which, a.ctypes.data_as(C.c_void_p)))

    def close(self):
        if self.owned and self.h:
            self.L.aet_layer_destroy(self.h)
        self.h = None


class ConvolutionalLayer(Layer):
    """dnn/ConvolutionalLayer.h:87-91 (FP32; channel groups, dilation and unequal strides included)."""

    def __init__(self, ctx, batch, h, w, c, n, size, stride_x=1, stride_y=None, padding=0, activation=LINEAR,
                 batch_normalize=0, train=1, groups=1, dilation=1):
        stride_y = stride_x if stride_y is None else stride_y
        super().__init__(ctx, ctx.L.aet_convolutional_layer_create(ctx.h, batch, h, w, c, n, groups, size, stride_x,
                                                                  stride_y, dilation, padding, activation,
                                                                  batch_normalize, train))


class MaxPoolLayer(Layer):
    """dnn/MaxPoolLayer.h:29-30."""

    def __init__(self, ctx, batch, h, w, c, size, stride_x, stride_y=None, padding=None, train=1):
        stride_y = stride_x if stride_y is None else stride_y
        padding = size - 1 if padding is None else padding
        super().__init__(ctx, ctx.L.aet_maxpool_layer_create(ctx.h, batch, h, w, c, size, stride_x, stride_y, padding, train))


class AvgPoolLayer(Layer):
    def __init__(self, ctx, batch, w, h, c):
        super().__init__(ctx, ctx.L.aet_avgpool_layer_create(ctx.h, batch, w, h, c))


class SoftMaxLayer(Layer):
    def __init__(self, ctx, batch, inputs, groups=1, temperature=1.0):
        super().__init__(ctx, ctx.L.aet_softmax_layer_create(ctx.h, batch, inputs, groups, temperature))


class DropoutLayer(Layer):
    def __init__(self, ctx, batch, inputs, probability, prev):
        super().__init__(ctx, ctx.L.aet_dropout_layer_create(ctx.h, batch, inputs, probability, prev.h))


class ShortcutLayer(Layer):
    """ShortcutLayer without weights (dnn/ShortcutLayer.c): activation(input + outputs of `sources`)."""

    def __init__(self, ctx, batch, h, w, c, sources, activation=LINEAR, train=1):
        arr = (C.c_void_p * len(sources))(*[s.h for s in sources])
        super().__init__(ctx, ctx.L.aet_shortcut_layer_create(ctx.h, batch, h, w, c, len(sources), arr, activation, train))
        self.sources = list(sources)


class NNetwork:
    """dnn/NNetwork.h:141-195 built by NetworkFactory.createNetwork from a Darknet-style cfg."""

    def __init__(self, ctx, cfg_path=None, cfg_text=None, train=1, batch=0):
        self.ctx, self.L = ctx, ctx.L
        if cfg_text is None:
            with open(cfg_path) as f:
                cfg_text = f.read()
        self.cfg_text = cfg_text
        self.h = _need(self.L.aet_network_create_ex(ctx.h, cfg_text.encode(), train, batch))
        self._loss = C.c_float()

    @property
    def batch(self):
        return self.L.aet_network_batch(self.h)

    @property
    def input_shape(self):
        v = [C.c_int() for _ in range(3)]
        _check(self.L.aet_network_input_shape(self.h, *[C.byref(x) for x in v]))
        return (self.batch,) + tuple(x.value for x in v)

    @property
    def outputs(self):
        return self.L.aet_network_outputs(self.h)

    @property
    def layer_count(self):
        return self.L.aet_network_layer_count(self.h)

    def layer(self, i):
        return Layer(self.ctx, self.L.aet_network_layer(self.h, i), owned=False)

    @property
    def input(self):
        return Tensor(self.ctx, handle=self.L.aet_network_input(self.h))

    @property
    def truth(self):
        return Tensor(self.ctx, handle=self.L.aet_network_truth(self.h))

    def set_hyper(self, learning_rate, momentum, decay):
        _check(self.L.aet_network_set_hyper(self.h, learning_rate, momentum, decay))

    def learning_rate(self):
        return self.L.aet_network_learning_rate(self.h)

    def forward(self, state):
        _check(self.L.aet_network_forward(self.h, state))

    def backward(self, state):
        _check(self.L.aet_network_backward(self.h, state))

    def update(self):
        _check(self.L.aet_network_update(self.h))

    def cost(self):
        return self.L.aet_network_cost(self.h)

    def train(self, x, truth):
        """NNetwork.train(InputData*, TruthData*) + update(): host batch in, mean loss out."""
        x, truth = _f32(x), _f32(truth)
        _check(self.L.aet_network_train_step(self.h, x.ctypes.data_as(C.c_void_p), truth.ctypes.data_as(C.c_void_p),
                                             C.byref(self._loss)))
        return self._loss.value

    def train_async(self, x, truth):
        """Pipelined train step: queues this batch (its upload overlaps the previous step) and returns the
        PREVIOUS call's mean loss (NaN on the first call).  `x` and `truth` must be float32 C-contiguous arrays;
        page-locked ones must stay unchanged until the next call returns."""
        if x.dtype != np.float32 or truth.dtype != np.float32 or not x.flags.c_contiguous or not truth.flags.c_contiguous:
            raise AetError("train_async: float32 C-contiguous arrays required (the copy is asynchronous)")
        _check(self.L.aet_network_train_step_async(self.h, x.ctypes.data_as(C.c_void_p), truth.ctypes.data_as(C.c_void_p),
                                                   C.byref(self._loss)))
        return self._loss.value

    def train_device(self, want_loss=True):
        _check(self.L.aet_network_train_step_device(self.h, C.byref(self._loss) if want_loss else None))
        return self._loss.value if want_loss else None

    def last_loss(self):
        _check(self.L.aet_network_last_loss(self.h, C.byref(self._loss)))
        return self._loss.value

    def predict(self, x):
        x = _f32(x)
        out = np.empty((self.batch, self.outputs), np.float32)
        _check(self.L.aet_network_predict(self.h, x.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p)))
        return out

    def augment_input(self, src, params):
        """Device-side rotate/crop + flip + HSV distortion of `src` [batch][c][sh][sw] into the network's input tensor;
        `params` is a list of dicts with the aet_augment fields (one per image)."""
        src = _f32(src)
        arr = (Augment * len(params))()
        for a, p in zip(arr, params):
            for k, v in p.items():
                setattr(a, k, v)
        _check(self.L.aet_network_augment_input(self.h, src.ctypes.data_as(C.c_void_p), src.shape[2], src.shape[3], arr))

    def fuse_conv_batchnorm(self):
        """NNetwork.fuseConvBatchnorm: fold BN into the convolutions (inference only afterwards)."""
        _check(self.L.aet_network_fuse_conv_batchnorm(self.h))

    def predict_topk(self, x, k):
        x = _f32(x)
        out = np.empty((self.batch, min(k, self.outputs)), np.int32)
        _check(self.L.aet_network_predict_topk(self.h, x.ctypes.data_as(C.c_void_p), k, out.ctypes.data_as(C.c_void_p)))
        return out

    def validate(self, images, class_ids, k):
        """Top-1 and top-k accuracy over `images` [count][c][h][w] (Classifier.validateSingle's loop)."""
        images = _f32(images)
        ids = np.ascontiguousarray(class_ids, np.int32)
        t1, tk = C.c_float(), C.c_float()
        _check(self.L.aet_network_validate(self.h, images.ctypes.data_as(C.c_void_p), ids.ctypes.data_as(C.c_void_p),
                                           len(ids), k, C.byref(t1), C.byref(tk)))
        return t1.value, tk.value

    def use_graph(self, enable=True):
        _check(self.L.aet_network_use_graph(self.h, int(enable)))

    def load_weights(self, path, cutoff=-1):
        """NNetwork.loadWeights(filename, cutoff): only the layers in front of index `cutoff` (-1: all)."""
        _check(self.L.aet_network_load_weights_upto(self.h, path.encode(), int(cutoff)))

    def save_weights(self, path):
        _check(self.L.aet_network_save_weights(self.h, path.encode()))

    def load_momentum(self, path):
        _check(self.L.aet_network_load_momentum(self.h, path.encode()))

    def save_momentum(self, path):
        """Side file with the momentum buffers the .weights container leaves out (bit-exact resume)."""
        _check(self.L.aet_network_save_momentum(self.h, path.encode()))

    def param_hash(self):
        v = C.c_uint64()
        _check(self.L.aet_network_param_hash(self.h, C.byref(v)))
        return v.value

    def profile(self, enable):
        _check(self.L.aet_network_profile(self.h, int(enable)))

    def profile_read(self, capacity=128):
        tab = (KernelTime * capacity)()
        n = C.c_int()
        _check(self.L.aet_network_profile_read(self.h, tab, capacity, C.byref(n)))
        return [dict(name=t.name.decode(), launches=t.launches, total_ms=t.total_ms, span_ms=t.span_ms, algo_bytes=t.algo_bytes,
                     algo_flops=t.algo_flops) for t in tab[:n.value]]

    def launches_per_step(self):
        return self.L.aet_network_launches_per_step(self.h)

    def comm_init(self, unique_id, rank, world):
        buf = C.create_string_buffer(bytes(unique_id), 128)
        _check(self.L.aet_network_comm_init(self.h, buf, rank, world))

    def comm_exposed(self):
        """(mean microseconds per step the main stream waited for the gradient collectives, steps counted); needs the
        context option "comm_stamps"."""
        us, n = C.c_double(), C.c_longlong()
        _check(self.L.aet_network_comm_exposed(self.h, C.byref(us), C.byref(n)))
        return us.value, n.value

    def comm_exchange_export(self):
        """This rank's 80-byte blob for the peer exchange of the last gradient bucket."""
        buf = C.create_string_buffer(80)
        _check(self.L.aet_network_comm_exchange_export(self.h, buf))
        return buf.raw

    def comm_exchange_attach(self, blobs):
        """`blobs`: every rank's export, in rank order."""
        raw = b"".join(bytes(b) for b in blobs)
        _check(self.L.aet_network_comm_exchange_attach(self.h, C.create_string_buffer(raw, len(raw))))

    def comm_exchange_detach(self):
        """Back to the collectives alone (all ranks together)."""
        _check(self.L.aet_network_comm_exchange_detach(self.h))

    def grad_arena(self):
        p, n = C.c_void_p(), C.c_size_t()
        _check(self.L.aet_network_grad_arena(self.h, C.byref(p), C.byref(n)))
        return p.value, n.value

    def close(self):
        if self.h:
            self.L.aet_network_destroy(self.h)
            self.h = None


def backward_bias_static(delta_ptr, bias_updates_ptr, pixels, channels, stream=None):
    """bias_updates[c] += sum_p delta[p][c] on raw device pointers, with the partial sums in the
    library's fixed device array: for callers that may not allocate device memory while running."""
    _check(lib().aet_backward_bias_static(C.c_void_p(delta_ptr), C.c_void_p(bias_updates_ptr), pixels, channels,
                                          C.c_void_p(stream) if stream else None))


def comm_unique_id():
    buf = C.create_string_buffer(128)
    _check(lib().aet_comm_unique_id(buf))
    return buf.raw
