"""Raw ctypes declarations of the C ABI in include/rt_b200.h (one Python attribute per
exported function) plus a few helpers to move numpy arrays to and from device buffers.
The parity tests call the kernels through this module."""
import ctypes as C
import re
import os

import numpy as np

_f32p = C.POINTER(C.c_float)
_i64p = C.POINTER(C.c_int64)

RT_OK = 0
# enum values of include/rt_b200.h
UNARY = dict(relu=0, elu=1, exp=2, ln=3, sin=4, tanh=5, sigmoid=6, softplus=7, square=8, sqrt=9, abs=10, clip=11,
             mul_scalar=12, div_scalar=13, cos=14, tan=15)
BINARY = dict(add=0, sub=1, mul=2, div=3, powf=4, maximum=5, minimum=6, equal=7, not_equal=8, greater=9,
              greater_equal=10, less=11, less_equal=12)
REDUCE = dict(sum=0, mean=1, max=2, min=3, prod=4, logsumexp=5, argmax=6, argmin=7)


def header_path():
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "include", "rt_b200.h")


def declared_symbols():
    """Names of every function declared in include/rt_b200.h."""
    text = open(header_path()).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rt_[a-z0-9_]+)\s*\(", text)))


class RtError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"rt status {code}: {msg}")
        self.code = code


class DeviceArray:
    """A device buffer with a shape, owned by a CApi context."""

    def __init__(self, api, ptr, shape):
        self.api, self.ptr, self.shape = api, ptr, tuple(int(s) for s in shape)

    @property
    def size(self):
        return int(np.prod(self.shape, dtype=np.int64)) if len(self.shape) else 1

    def numpy(self):
        out = np.empty(self.shape, dtype=np.float32)
        self.api.check(self.api.lib.rt_memcpy_d2h(self.api.ctx, out.ctypes.data_as(C.c_void_p), self.ptr,
                                                  C.c_size_t(out.nbytes)))
        return out

    def __del__(self):
        try:
            if self.ptr and self.api.ctx:
                self.api.lib.rt_free(self.api.ctx, self.ptr)
        except Exception:
            pass


class CApi:
    """One ``rt_ctx`` plus typed access to every ``rt_*`` entry point."""

    def __init__(self, device=0, ctx=None):
        from . import load_library

        self.lib = load_library()
        self.lib.rt_last_error.restype = C.c_char_p
        self.lib.rt_stream.restype = C.c_void_p
        self._owns = ctx is None
        if ctx is None:
            h = C.c_void_p()
            rc = self.lib.rt_ctx_create(C.c_int(device), C.byref(h))
            if rc != RT_OK:
                raise RtError(rc, "rt_ctx_create failed: no usable CUDA device (this library has no CPU fallback)")
            ctx = h
        self.ctx = ctx

    def close(self):
        if self._owns and self.ctx:
            self.lib.rt_ctx_destroy(self.ctx)
        self.ctx = None

    def check(self, rc):
        if rc != RT_OK:
            raise RtError(rc, self.lib.rt_last_error(self.ctx).decode())

    def empty(self, shape):
        shape = tuple(int(s) for s in shape)
        n = int(np.prod(shape, dtype=np.int64)) if len(shape) else 1
        p = C.c_void_p()
        self.check(self.lib.rt_malloc(self.ctx, C.c_size_t(4 * max(n, 1)), C.byref(p)))
        return DeviceArray(self, p, shape)

    def to_device(self, array):
        a = np.require(array, dtype=np.float32, requirements='C')
        d = self.empty(a.shape)
        self.check(self.lib.rt_memcpy_h2d(self.ctx, d.ptr, a.ctypes.data_as(C.c_void_p), C.c_size_t(a.nbytes)))
        return d

    def sync(self):
        self.check(self.lib.rt_sync(self.ctx))

    @staticmethod
    def i64(values):
        return (C.c_int64 * max(len(values), 1))(*[int(v) for v in values])

    def launches(self):
        n = C.c_int64(0)
        self.check(self.lib.rt_kernel_launch_count(self.ctx, C.byref(n)))
        return n.value

    def call(self, name, *args):
        """Calls ``rt_<name>(ctx, *args)`` and raises on a non-zero status."""
        self.check(getattr(self.lib, "rt_" + name)(self.ctx, *args))
