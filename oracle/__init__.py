"""ORACLE -- test infrastructure, not product code.

Loads ``oracle/liboracle.so`` (the CPU restatement of the reference's CPU
backend, see cpu_backend.hpp) and exposes it through the same ``Engine`` wrapper
the CUDA library uses.  Only tests, ``__graft_entry__.smoke()`` and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` may import this
package.
"""
import ctypes
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_lib = None


def build(force=False):
    """Compile liboracle.so with oracle/Makefile (g++ only, no GPU needed)."""
    if force and os.path.exists(_LIB_PATH):
        os.remove(_LIB_PATH)
    subprocess.run(["make", "-C", _HERE], check=True, stdout=subprocess.DEVNULL)
    return _LIB_PATH


def load():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        try:
            _lib = ctypes.CDLL(_LIB_PATH)
        except OSError:
            build(force=True)
            _lib = ctypes.CDLL(_LIB_PATH)
    return _lib


def engine():
    """An ``Engine`` whose tensors live in host memory and whose math is the oracle's."""
    from rusttensor_b200.frontend import Engine

    return Engine(load(), "orc")


def set_conv_dx_faithful(on):
    """True (default): conv2d_backward reproduces the reference's input-gradient defect
    (src/ops/cpu_ops.rs:266,271).  False: mathematically correct col2im."""
    load().orc_set_conv_dx_faithful(1 if on else 0)
