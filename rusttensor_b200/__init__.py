"""rusttensor_b200 -- a B200 (sm_100a) CUDA backend for the backward pass and optimizer
step of a RustTensor-style autograd library.

Layers (bottom up):
  librt_b200.so       hand-written CUDA kernels behind the C ABI of include/rt_b200.h
  librt_b200_host.so  C++ host: the generic autograd engine instantiated for the CUDA
                      backend (`rth_*`) and the data-parallel training step
  this package        ctypes bindings: `capi` (raw C ABI), `engine()` (Tensor / ops /
                      optimizers, the reference's public API), `DataParallelTrainer`

There is no CPU fallback: using the package without the built libraries or without a
CUDA device raises.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "librt_b200.so")
HOST_LIB_PATH = os.path.join(_HERE, "librt_b200_host.so")

_lib = None
_host = None
_engine = None


class BackendUnavailable(RuntimeError):
    pass


def load_library():
    """The C-ABI CUDA library (loads without a GPU; calls fail without one)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise BackendUnavailable(
                f"{LIB_PATH} is missing: build it with `python -m rusttensor_b200._build` "
                "(or __graft_entry__.build()); there is no CPU fallback")
        _lib = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
    return _lib


def load_host_library():
    global _host
    if _host is None:
        load_library()
        if not os.path.exists(HOST_LIB_PATH):
            raise BackendUnavailable(f"{HOST_LIB_PATH} is missing: run `python -m rusttensor_b200._build`")
        _host = ctypes.CDLL(HOST_LIB_PATH)
    return _host


def init(device=None):
    """Creates the process-wide device context (idempotent).  ``device`` defaults to LOCAL_RANK or 0."""
    host = load_host_library()
    if device is None:
        device = int(os.environ.get("LOCAL_RANK", "0"))
    rc = host.rth_init(ctypes.c_int(device))
    if rc != 0:
        host.rth_last_error.restype = ctypes.c_char_p
        raise BackendUnavailable(
            f"rth_init({device}) failed with code {rc}: {host.rth_last_error().decode()} -- "
            "this backend needs a CUDA device (sm_100a); there is no CPU fallback")
    return host


def engine(device=None):
    """The autograd engine on the CUDA backend: ``engine().tensor(...)``, ``engine().ops.add(...)`` ..."""
    global _engine
    if _engine is None:
        from .frontend import Engine

        _engine = Engine(init(device), "rth")
    return _engine


def context_handle():
    """The ``rt_ctx*`` of the engine's context, for calling the raw C ABI on engine tensors."""
    host = init()
    host.rth_ctx.restype = ctypes.c_void_p
    return ctypes.c_void_p(host.rth_ctx())


from .capi import CApi  # noqa: E402
from .trainer import DataParallelTrainer  # noqa: E402
