"""ctypes view of the autograd engine C API (``<prefix>_*`` functions).

The same wrapper drives the CUDA library (prefix ``rth``) and, in tests, the CPU
oracle (prefix ``orc``), so a test builds one graph on both and compares, which
is the scheme of the reference's differential tests
(tests/ops_cuda_backward_tests.rs:74-144).  Names follow the reference's public
API: ``ops.add``, ``Tensor.backward``, ``Tensor.grad``, ``Adam.step`` ...
"""
import ctypes as C

import numpy as np

_i64p = C.POINTER(C.c_int64)
_f32p = C.POINTER(C.c_float)
_f64p = C.POINTER(C.c_double)

ERROR_KINDS = {
    1: "ShapeMismatch", 2: "IncompatibleShapes", 3: "InvalidIndex", 4: "InvalidOperation",
    5: "InternalLogicError", 6: "DimensionMismatch", 7: "CudaError", 8: "OutOfMemory",
    9: "Unimplemented", 10: "EmptyTensor", 11: "ShapeError", 12: "NoGradientError",
    13: "GradientCheckError", 14: "Timeout", 15: "Nccl", 16: "InitializationError",
}


class EngineError(RuntimeError):
    """Mirror of the reference's ``Error`` enum (src/error.rs:8-98): ``kind`` is the variant name."""

    def __init__(self, code, message):
        super().__init__(f"{ERROR_KINDS.get(code, code)}: {message}")
        self.code = code
        self.kind = ERROR_KINDS.get(code, str(code))


def _i64(values):
    arr = (C.c_int64 * max(len(values), 1))(*[int(v) for v in values])
    return arr


def _f64(values):
    arr = (C.c_double * max(len(values), 1))(*[float(v) for v in values])
    return arr


class Tensor:
    def __init__(self, engine, handle):
        self.engine = engine
        self.handle = handle

    def __del__(self):
        try:
            self.engine._call("tensor_free", C.c_int64(self.handle))
        except Exception:
            pass

    @property
    def shape(self):
        nd = C.c_int(0)
        self.engine._call("tensor_ndim", C.c_int64(self.handle), C.byref(nd))
        buf = (C.c_int64 * max(nd.value, 1))()
        self.engine._call("tensor_shape", C.c_int64(self.handle), buf)
        return tuple(int(buf[i]) for i in range(nd.value))

    @property
    def requires_grad(self):
        v = C.c_int(0)
        self.engine._call("tensor_requires_grad", C.c_int64(self.handle), C.byref(v))
        return bool(v.value)

    def numpy(self):
        shape = self.shape
        out = np.empty(shape, dtype=np.float32)
        n = int(np.prod(shape, dtype=np.int64)) if len(shape) else 1
        self.engine._call("tensor_to_host", C.c_int64(self.handle), out.ctypes.data_as(_f32p), C.c_int64(n))
        return out

    def update_from_host(self, data):
        a = np.require(data, dtype=np.float32, requirements='C')
        self.engine._call("tensor_update_from_host", C.c_int64(self.handle), a.ctypes.data_as(_f32p), C.c_int64(a.size))

    @property
    def grad(self):
        has = C.c_int(0)
        self.engine._call("tensor_has_grad", C.c_int64(self.handle), C.byref(has))
        if not has.value:
            return None
        out = C.c_int64(0)
        self.engine._call("tensor_grad", C.c_int64(self.handle), C.byref(out))
        return Tensor(self.engine, out.value)

    def set_grad(self, grad):
        self.engine._call("tensor_set_grad", C.c_int64(self.handle), C.c_int64(grad.handle))

    def zero_grad(self):
        self.engine._call("tensor_zero_grad", C.c_int64(self.handle))

    def backward(self):
        self.engine._call("backward", C.c_int64(self.handle))

    def view(self, shape):
        return self.engine.ops.view(self, shape)

    def broadcast_to(self, shape):
        return self.engine.ops.broadcast_to(self, shape)


class _Ops:
    """``ops::*`` of the reference (src/ops/mod.rs), same names and argument order."""

    def __init__(self, engine):
        self._e = engine

    def _run(self, name, inputs, ip=(), fp=()):
        return self._e.op(name, inputs, ip, fp)


def _axis(a):
    return -1 if a is None else int(a)


_RED = {"none": 0, "sum": 1, "mean": 2}

for _n in ("matmul", "mul", "add", "sub", "div", "powf", "maximum", "minimum"):
    setattr(_Ops, _n, (lambda n: lambda self, a, b: self._run(n, [a, b]))(_n))
for _n in ("equal", "not_equal", "greater", "greater_equal", "less", "less_equal"):  # src/ops/mod.rs:1273-1331: not differentiable
    setattr(_Ops, _n, (lambda n: lambda self, a, b: self._run(n, [a, b]))(_n))
# Backend::cos / tan and their backward (src/backend/mod.rs:486-507); the reference's ops:: front-end does not expose them
_Ops.backend_cos = lambda self, x: self._run("backend_cos", [x])
_Ops.backend_tan = lambda self, x: self._run("backend_tan", [x])
_Ops.backend_cos_backward = lambda self, x, g: self._run("backend_cos_backward", [x, g])
_Ops.backend_tan_backward = lambda self, x, g: self._run("backend_tan_backward", [x, g])
for _n in ("relu", "sigmoid", "abs", "exp", "ln", "sqrt", "tanh", "softplus", "square", "sin", "transpose"):
    setattr(_Ops, _n, (lambda n: lambda self, x: self._run(n, [x]))(_n))
for _n in ("mean", "sum", "max", "min", "prod", "logsumexp"):
    setattr(_Ops, _n, (lambda n: lambda self, x, axis=None: self._run(n, [x], [_axis(axis)]))(_n))
for _n in ("log_softmax", "argmax", "argmin", "expand_dims"):
    setattr(_Ops, _n, (lambda n: lambda self, x, axis: self._run(n, [x], [int(axis)]))(_n))
for _n in ("elu", "mul_scalar", "div_scalar", "powf_scalar"):
    setattr(_Ops, _n, (lambda n: lambda self, x, s: self._run(n, [x], (), [s]))(_n))
_Ops.clip = lambda self, x, lo, hi: self._run("clip", [x], (), [lo, hi])
_Ops.squeeze = lambda self, x, axis=None: self._run("squeeze", [x], [_axis(axis)])
_Ops.concat = lambda self, tensors, axis: self._run("concat", list(tensors), [int(axis)])
_Ops.view = lambda self, x, shape: self._run("view", [x], list(shape))
_Ops.broadcast_to = lambda self, x, shape: self._run("broadcast_to", [x], list(shape))
_Ops.slice = lambda self, x, ranges: self._run("slice", [x], [v for r in ranges for v in r])
_Ops.conv2d = lambda self, x, w, bias=None, stride=(1, 1), padding=(0, 0): self._run(
    "conv2d", [x, w] + ([bias] if bias is not None else []), list(stride) + list(padding))
_Ops.conv2d_transpose = lambda self, x, w, bias=None, stride=(1, 1), padding=(0, 0): self._run(
    "conv2d_transpose", [x, w] + ([bias] if bias is not None else []), list(stride) + list(padding))
_Ops.max_pool2d = lambda self, x, kernel_size, stride, padding: self._run(
    "max_pool2d", [x], list(kernel_size) + list(stride) + list(padding))
_Ops.mse_loss = lambda self, p, t, reduction="mean": self._run("mse_loss", [p, t], [_RED[reduction]])
_Ops.binary_cross_entropy_with_logits = lambda self, l, t, reduction="mean": self._run(
    "binary_cross_entropy_with_logits", [l, t], [_RED[reduction]])
_Ops.softmax_cross_entropy = lambda self, l, t, axis, reduction="mean": self._run(
    "softmax_cross_entropy", [l, t], [int(axis), _RED[reduction]])


class Optimizer:
    def __init__(self, engine, kind, params, hyper):
        self.engine = engine
        self.parameters = list(params)
        out = C.c_int64(0)
        engine._call("optim_create", C.c_int(kind), _i64([p.handle for p in params]), C.c_int(len(params)),
                     _f64(hyper), C.c_int(len(hyper)), C.byref(out))
        self.handle = out.value

    def __del__(self):
        try:
            self.engine._call("optim_free", C.c_int64(self.handle))
        except Exception:
            pass

    def step(self):
        self.engine._call("optim_step", C.c_int64(self.handle))

    def zero_grad(self):
        self.engine._call("optim_zero_grad", C.c_int64(self.handle))

    def state(self, which, idx):
        out = C.c_int64(0)
        self.engine._call("optim_state", C.c_int64(self.handle), C.c_int(which), C.c_int(idx), C.byref(out))
        return Tensor(self.engine, out.value)


class Trainer:
    """One of the five benchmark workloads with the reference's per-tensor optimizer API."""

    def __init__(self, engine, config, dims):
        self.engine = engine
        out = C.c_int64(0)
        engine._call("trainer_create", C.c_int(config), _i64(dims), C.c_int(len(dims)), C.byref(out))
        self.handle = out.value
        n = C.c_int(0)
        engine._call("trainer_num_params", C.c_int64(self.handle), C.byref(n))
        self.params = []
        for i in range(n.value):
            h = C.c_int64(0)
            engine._call("trainer_param", C.c_int64(self.handle), C.c_int(i), C.byref(h))
            self.params.append(Tensor(engine, h.value))

    def __del__(self):
        try:
            self.engine._call("trainer_free", C.c_int64(self.handle))
        except Exception:
            pass

    def set_hyper(self, *hp):
        self.engine._call("trainer_set_hyper", C.c_int64(self.handle), _f64(hp), C.c_int(len(hp)))

    def _run(self, inputs, mode):
        out = C.c_int64(0)
        self.engine._call("trainer_run", C.c_int64(self.handle), _i64([t.handle for t in inputs]),
                          C.c_int(len(inputs)), C.c_int(mode), C.byref(out))
        return Tensor(self.engine, out.value)

    def forward(self, inputs):
        return self._run(inputs, 0)

    def forward_backward(self, inputs):
        return self._run(inputs, 1)

    def step(self, inputs):
        return self._run(inputs, 2)

    def optimizer_step(self):
        self.engine._call("trainer_optimizer_step", C.c_int64(self.handle))

    def optim_state(self, which, idx):
        out = C.c_int64(0)
        self.engine._call("trainer_optim_state", C.c_int64(self.handle), C.c_int(which), C.c_int(idx), C.byref(out))
        return Tensor(self.engine, out.value)


class Engine:
    def __init__(self, lib, prefix):
        self.lib = lib
        self.prefix = prefix
        self.ops = _Ops(self)
        getattr(lib, f"{prefix}_last_error").restype = C.c_char_p

    def _call(self, name, *args):
        fn = getattr(self.lib, f"{self.prefix}_{name}")
        fn.restype = C.c_int
        rc = fn(*args)
        if rc != 0:
            msg = getattr(self.lib, f"{self.prefix}_last_error")()
            raise EngineError(rc, msg.decode() if msg else "")

    def tensor(self, data, shape=None, requires_grad=False):
        """``Tensor::from_vec(data, shape, requires_grad)`` (src/tensor.rs:948-950)."""
        a = np.require(data, dtype=np.float32, requirements='C')
        if shape is None:
            shape = a.shape
        shape = tuple(int(s) for s in shape)
        n = int(np.prod(shape, dtype=np.int64)) if len(shape) else 1
        if a.size != n:
            raise EngineError(1, f"Shape mismatch: expected {list(shape)}, got [{a.size}]")
        out = C.c_int64(0)
        self._call("tensor_from_host", a.ctypes.data_as(_f32p), _i64(shape), C.c_int(len(shape)),
                   C.c_int(1 if requires_grad else 0), C.byref(out))
        return Tensor(self, out.value)

    # ---- random factories (Backend::random_uniform / random_normal / bernoulli / kaiming_uniform, src/backend/mod.rs:57-69) ----
    def manual_seed(self, seed):
        """Seeds the backend's generator (the reference draws from rand's unseedable thread-local generator)."""
        self.op("manual_seed", [], [int(seed)])

    def random_uniform(self, shape, low, high):
        return self.op("random_uniform", [], list(shape), [low, high])

    def random_normal(self, shape, mean, std_dev):
        return self.op("random_normal", [], list(shape), [mean, std_dev])

    def bernoulli(self, shape, p):
        return self.op("bernoulli", [], list(shape), [p])

    def kaiming_uniform(self, fan_in, shape, requires_grad=False):
        """``Tensor::kaiming_uniform(fan_in, shape, requires_grad)`` (src/tensor.rs:953-960)."""
        return self.op("kaiming_uniform", [], [int(fan_in)] + list(shape), [1.0 if requires_grad else 0.0])

    # ---- data::get_random_batch (src/data.rs:125-209) ----
    def get_batch(self, x, y, indices):
        """Rows ``indices`` of x and y as two new tensors (gathered by the backend: on the device for CUDA)."""
        ox, oy = C.c_int64(0), C.c_int64(0)
        self._call("get_batch", C.c_int64(x.handle), C.c_int64(y.handle), _i64(indices), C.c_int(len(indices)), C.c_int64(0),
                   C.c_uint64(0), C.byref(ox), C.byref(oy))
        return Tensor(self, ox.value), Tensor(self, oy.value)

    def get_random_batch(self, x, y, batch_size, seed=0):
        """``batch_size`` distinct random rows of x and y (sampling without replacement, seeded)."""
        ox, oy = C.c_int64(0), C.c_int64(0)
        self._call("get_batch", C.c_int64(x.handle), C.c_int64(y.handle), _i64([]), C.c_int(0), C.c_int64(int(batch_size)),
                   C.c_uint64(int(seed)), C.byref(ox), C.byref(oy))
        return Tensor(self, ox.value), Tensor(self, oy.value)

    def op(self, name, inputs, ip=(), fp=()):
        out = C.c_int64(0)
        self._call("op", name.encode(), _i64([t.handle for t in inputs]), C.c_int(len(inputs)),
                   _i64(ip), C.c_int(len(ip)), _f64(fp), C.c_int(len(fp)), C.byref(out))
        return Tensor(self, out.value)

    def op_backward(self, output, grad):
        """Calls the backward closure of the op that produced ``output`` with ``grad`` directly."""
        outs = (C.c_int64 * 16)()
        n = C.c_int(0)
        self._call("op_backward", C.c_int64(output.handle), C.c_int64(grad.handle), outs, C.c_int(16), C.byref(n))
        return [Tensor(self, outs[i]) for i in range(n.value)]

    def Sgd(self, params, lr):
        return Optimizer(self, 0, params, [lr])

    def Adam(self, params, lr, beta1=0.9, beta2=0.999, epsilon=1e-8):
        return Optimizer(self, 1, params, [lr, beta1, beta2, epsilon])

    def MomentumSGD(self, params, lr, momentum=0.9):
        return Optimizer(self, 2, params, [lr, momentum])

    def AdaGrad(self, params, lr, epsilon=1e-8):
        return Optimizer(self, 3, params, [lr, epsilon])

    def trainer(self, config, dims):
        return Trainer(self, config, dims)
