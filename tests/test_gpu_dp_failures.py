"""Failure handling of the communicator layer of librt_b200.so, with the failing call faked on the host.

A scripted stand-in for NCCL (tests/fakes/fake_nccl.c) is loaded through RT_B200_NCCL_LIBRARY, so no rank, kernel or
collective has to fail for real: the library under test sees "in progress" answers that never settle, an asynchronous
error, and a slow start, and must turn them into RT_ERR_TIMEOUT / RT_ERR_NCCL with the communicator aborted and the
context still usable.  One case uses the real NCCL: rank 0 of a two-rank job whose second rank never starts (nothing is
launched on the GPU before the deadline ends the call).  Each case runs in a child process because the library resolves
NCCL once per process."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_CHILD = r"""
import ctypes as C, os, sys, time
import numpy as np
sys.path.insert(0, os.environ["RT_ROOT"])
import rusttensor_b200 as rt
from rusttensor_b200.capi import RtError
case = os.environ["CASE"]
capi = rt.CApi(device=0)
fake = C.CDLL(os.environ["RT_B200_NCCL_LIBRARY"]) if os.environ.get("RT_B200_NCCL_LIBRARY") else None
def counts():
    out = (C.c_int * 4)()
    fake.fake_nccl_counts(out)
    return list(out)                      # abort, destroy, all-reduce, poll
def still_usable():
    a = capi.to_device(np.arange(1000, dtype=np.float32))
    capi.call("unary", C.c_int(0), a.ptr, a.ptr, C.c_int64(1000), C.c_float(0), C.c_float(0))
    capi.sync()
ident = (C.c_uint8 * 128)()
assert capi.lib.rt_dp_unique_id(ident) == 0
def init(timeout_ms):
    capi.call("dp_init_deadline", C.c_int(0), C.c_int(2), ident, C.c_int64(timeout_ms))
buf = capi.to_device(np.ones(4096, np.float32))

if case in ("init_never", "real_never_joins"):
    t0 = time.time()
    try:
        init(1500)
        print("UNEXPECTED: joined"); sys.exit(1)
    except RtError as e:
        assert e.code == 14, e            # RT_ERR_TIMEOUT
        assert "aborted" in str(e)
    assert 1.0 < time.time() - t0 < 60
    if fake:
        assert counts()[0] == 1           # the half-built communicator was aborted, once
    still_usable()
    try:
        capi.call("dp_allreduce_sum", buf.ptr, C.c_int64(4096))
        print("UNEXPECTED: all-reduce without a communicator"); sys.exit(1)
    except RtError as e:
        assert e.code == 15 and "no communicator" in str(e)
elif case == "init_slow":
    init(5000)
    assert counts()[3] >= 6               # polled until it settled
    capi.call("dp_allreduce_sum", buf.ptr, C.c_int64(4096))
    capi.sync()
    assert counts()[:3] == [0, 0, 1]
elif case == "allreduce_progress":
    init(5000)
    before = counts()[3]
    capi.call("dp_allreduce_sum", buf.ptr, C.c_int64(4096))
    assert counts()[3] - before == 4      # three "in progress" answers, then success
    capi.sync()
elif case == "async_error":
    init(5000)
    code = C.c_int(0)
    for _ in range(2):                    # polls 2 and 3 (the first was spent by init): healthy
        capi.call("dp_async_error", C.byref(code))
        assert code.value == 0
    try:
        capi.call("dp_async_error", C.byref(code))
        print("UNEXPECTED: no error reported"); sys.exit(1)
    except RtError as e:
        assert e.code == 15 and "remote process exited" in str(e) and code.value == 6
    assert counts()[0] == 1
    still_usable()
elif case == "watchdog":
    # the step's event is still pending when the communicator reports the error: the wait ends at once with the error
    init(5000)
    big = capi.empty((64 * 1024 * 1024,))
    ev = C.c_void_p()
    capi.call("event_create", C.byref(ev))
    for _ in range(200):                  # some milliseconds of queued work
        capi.call("fill", big.ptr, C.c_float(1.0), C.c_int64(big.size))
    capi.call("event_record", ev)
    t0 = time.time()
    try:
        capi.call("dp_wait_event", ev)
        print("UNEXPECTED: the wait saw no error"); sys.exit(1)
    except RtError as e:
        assert e.code == 15, e
    assert counts()[0] == 1
    capi.sync()                           # the queued fills finish normally
    capi.call("dp_wait_event", ev)        # no communicator any more: a plain wait
    capi.call("event_destroy", ev)
    still_usable()
capi.close()
print("CASE_OK", case)
"""


@pytest.fixture(scope="module")
def fake_nccl(tmp_path_factory):
    out = tmp_path_factory.mktemp("fake_nccl") / "libfake_nccl.so"
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-o", str(out), os.path.join(ROOT, "tests", "fakes", "fake_nccl.c")], check=True)
    return str(out)


def _run(tmp_path, case, mode, library):
    script = tmp_path / "child.py"
    script.write_text(_CHILD)
    env = dict(os.environ, RT_ROOT=ROOT, CASE=case, FAKE_NCCL_MODE=mode, NCCL_NVLS_ENABLE="0")
    env.pop("RT_B200_NCCL_BLOCKING", None)
    if library:
        env["RT_B200_NCCL_LIBRARY"] = library
    else:
        env.pop("RT_B200_NCCL_LIBRARY", None)
    p = subprocess.run([sys.executable, str(script)], env=env, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0 and f"CASE_OK {case}" in p.stdout, (p.returncode, p.stdout[-3000:], p.stderr[-3000:])


@pytest.mark.parametrize("case,mode", [("init_never", "init_never"), ("init_slow", "init_slow"), ("allreduce_progress", "allreduce_progress"),
                                       ("async_error", "async_error"), ("watchdog", "async_error")])
def test_communicator_failures_faked_on_the_host(tmp_path, fake_nccl, case, mode):
    _run(tmp_path, case, mode, fake_nccl)


def test_real_nccl_rank_that_never_joins_times_out_and_the_context_survives(tmp_path):
    """Rank 0 of a two-rank communicator whose peer never starts: the non-blocking initialisation is polled until the
    deadline, aborted, and reported as RT_ERR_TIMEOUT.  No kernel or collective is launched before that."""
    _run(tmp_path, "real_never_joins", "ok", None)
