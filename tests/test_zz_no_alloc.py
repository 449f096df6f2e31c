"""rt_reduce_sum_static_scratch (include/rt_b200.h): the axis sum whose split partial sums live in a fixed
device array.  Checked through the C ABI against rt_reduce(RT_RED_SUM), on repeated calls, with other shapes in
between (the array keeps old contents), and for its documented refusals.  The file name sorts last so that the
test also runs after every other GPU test has used the device."""
import ctypes as C

import numpy as np
import pytest

from helpers import assert_close
from rusttensor_b200.capi import REDUCE, RtError

pytestmark = pytest.mark.gpu

SHAPES = (
    (1, 1 << 22, 1),      # one long row: chunked, partial sums in the fixed array
    (3, 70000, 1),        # a few long rows
    (1000, 17, 1),        # short rows: single pass
    (40, 600, 1),         # one warp per row
    (1, 4096, 4096),      # column sums, split along the reduced axis, 128-bit loads
    (5, 300, 7),          # odd inner extent: scalar loads
    (2, 9000, 4),
    (1, 100000, 3),
    (0, 5, 3),            # nothing to do
    (4, 0, 6),            # empty reduction: zeros
)


def _mem(capi):
    res, used, n = C.c_int64(0), C.c_int64(0), C.c_int64(0)
    capi.call("mem_stats", C.byref(res), C.byref(used), C.byref(n))
    return res.value, used.value, n.value


def _static_sum(capi, dx, shape, out):
    outer, ln, inner = shape
    capi.call("reduce_sum_static_scratch", dx.ptr if dx is not None else None, C.c_int64(outer), C.c_int64(ln), C.c_int64(inner),
              out.ptr if out is not None else None)


def test_matches_rt_reduce_and_repeats_exactly(capi):
    _static_sum(capi, None, (0, 1, 1), None)  # set-up call: looks up the array's address
    first = {}
    for rep in range(2):          # the second sweep finds the array full of the other shapes' partial sums
        for shape in SHAPES:
            outer, ln, inner = shape
            x = np.random.default_rng(hash(shape) % (1 << 31)).standard_normal(shape).astype(np.float32)
            dx = capi.to_device(x) if x.size else None
            n_out = outer * inner
            ref = capi.empty((outer, inner)) if n_out else None
            out = capi.empty((outer, inner)) if n_out else None
            if n_out:
                capi.call("reduce", C.c_int(REDUCE["sum"]), dx.ptr if dx is not None else None, C.c_int64(outer), C.c_int64(ln),
                          C.c_int64(inner), ref.ptr)
            before = _mem(capi)
            _static_sum(capi, dx, shape, out)
            _static_sum(capi, dx, shape, out)   # two calls in a row
            assert _mem(capi) == before, f"the call changed the allocator's state for {shape}"
            if not n_out:
                continue
            got = out.numpy()
            assert_close(got, ref.numpy(), 1e-5, f"static-scratch sum {shape} vs rt_reduce", abs_floor=1e-3)
            assert_close(got, x.astype(np.float64).sum(axis=1), 1e-4, f"static-scratch sum {shape} vs float64", abs_floor=1e-2)
            if rep == 0:
                first[shape] = got.copy()
            else:
                assert np.array_equal(got, first[shape]), f"{shape}: result depends on what the array held before"


def test_refuses_what_it_cannot_hold(capi):
    x = capi.to_device(np.ones((70000, 3, 2), np.float32))
    out = capi.empty((70000, 2))
    with pytest.raises(RtError) as ei:
        _static_sum(capi, x, (70000, 3, 2), out)
    assert "65535" in str(ei.value)
    with pytest.raises(RtError):
        _static_sum(capi, x, (-1, 3, 2), out)
    # the same shape is fine for the allocating entry point
    capi.call("reduce", C.c_int(REDUCE["sum"]), x.ptr, C.c_int64(70000), C.c_int64(3), C.c_int64(2), out.ptr)
    assert np.array_equal(out.numpy(), np.full((70000, 2), 3.0, np.float32))
