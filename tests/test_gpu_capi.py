"""Calls through the raw C ABI (include/rt_b200.h) with device pointers, against numpy / the oracle."""
import ctypes as C

import numpy as np
import pytest

from helpers import assert_close, rng
from rusttensor_b200.capi import BINARY, REDUCE, UNARY, RtError

pytestmark = pytest.mark.gpu


def test_unary_backward_vectorised_and_tail(capi):
    r = rng(61)
    for n in (1, 3, 4, 5, 1023, 1 << 20, (1 << 20) + 3):
        x = r.standard_normal(n).astype(np.float32)
        g = r.standard_normal(n).astype(np.float32)
        dx, dg, dd = capi.to_device(x), capi.to_device(g), capi.empty((n,))
        capi.call("unary_backward", C.c_int(UNARY["tanh"]), dx.ptr, dg.ptr, dd.ptr, C.c_int64(n), C.c_float(0), C.c_float(0))
        assert_close(dd.numpy(), g * (1 - np.tanh(x.astype(np.float64)) ** 2), 1e-4, f"tanh_backward n={n}")
        capi.call("unary_backward", C.c_int(UNARY["relu"]), dx.ptr, dg.ptr, dd.ptr, C.c_int64(n), C.c_float(0), C.c_float(0))
        assert np.array_equal(dd.numpy(), g * (x > 0))


def test_unaligned_pointers_take_the_scalar_path(capi):
    r = rng(62)
    n = 1000
    x = r.standard_normal(n + 1).astype(np.float32)
    dx, dy = capi.to_device(x), capi.empty((n + 1,))
    off = lambda d: C.c_void_p(d.ptr.value + 4)
    capi.call("unary", C.c_int(UNARY["exp"]), off(dx), off(dy), C.c_int64(n), C.c_float(0), C.c_float(0))
    assert_close(dy.numpy()[1:], np.exp(x[1:].astype(np.float64)), 1e-5, "exp on an unaligned pointer")


def test_binary_backward_rowvec_fused_column_sum(capi):
    r = rng(63)
    for rows, cols in ((4096, 512), (1000, 132), (37, 4), (3, 260)):
        a = r.standard_normal((rows, cols)).astype(np.float32)
        b = r.standard_normal(cols).astype(np.float32)
        g = r.standard_normal((rows, cols)).astype(np.float32)
        da_, db_, dg_ = capi.to_device(a), capi.to_device(b), capi.to_device(g)
        oa, ob = capi.empty((rows, cols)), capi.empty((cols,))
        capi.call("binary_backward", C.c_int(BINARY["mul"]), da_.ptr, capi.i64([rows, cols]), C.c_int(2), db_.ptr,
                  capi.i64([cols]), C.c_int(1), dg_.ptr, oa.ptr, ob.ptr)
        assert_close(oa.numpy(), g.astype(np.float64) * b, 1e-5, "dA")
        assert_close(ob.numpy(), (g.astype(np.float64) * a).sum(0), 1e-4, f"db {rows}x{cols}")
        # run-to-run determinism of the two-pass reduction
        ob2 = capi.empty((cols,))
        capi.call("binary_backward", C.c_int(BINARY["mul"]), da_.ptr, capi.i64([rows, cols]), C.c_int(2), db_.ptr,
                  capi.i64([cols]), C.c_int(1), dg_.ptr, None, ob2.ptr)
        assert np.array_equal(ob.numpy(), ob2.numpy())


def test_unbroadcast_patterns(capi):
    r = rng(64)
    cases = [((6, 5), (5,)), ((6, 5), (6, 1)), ((6, 5), ()), ((2, 3, 4), (3, 1)), ((2, 3, 4), (1, 3, 1)), ((4, 3, 5, 6), (3, 1, 1)),
             ((300, 70), (70,)), ((2, 1, 4), (4,)), ((5,), (5,))]
    for gs, ts in cases:
        g = r.standard_normal(gs).astype(np.float32)
        out = capi.empty(ts)
        capi.call("unbroadcast", capi.to_device(g).ptr, capi.i64(gs), C.c_int(len(gs)), capi.i64(ts), C.c_int(len(ts)), out.ptr)
        ref = g.astype(np.float64)
        lead = len(gs) - len(ts)
        if lead:
            ref = ref.sum(axis=tuple(range(lead)))
        for i, t in enumerate(ts):
            if t == 1 and ref.shape[i] != 1:
                ref = ref.sum(axis=i, keepdims=True)
        assert_close(out.numpy(), ref.reshape(ts), 1e-4, f"unbroadcast {gs}->{ts}")
    with pytest.raises(RtError) as ei:
        capi.call("unbroadcast", capi.to_device(np.zeros((4, 3))).ptr, capi.i64([4, 3]), C.c_int(2), capi.i64([2]), C.c_int(1), capi.empty((2,)).ptr)
    assert ei.value.code == 2


def test_reduce_shapes(capi):
    r = rng(65)
    for outer, ln, inner in ((1, 1 << 22, 1), (3, 70000, 1), (1000, 17, 1), (1, 4096, 4096), (5, 300, 7), (2, 9000, 4), (70000, 3, 2)):
        x = r.standard_normal((outer, ln, inner)).astype(np.float32)
        dx = capi.to_device(x)
        for kind, f in (("sum", np.sum), ("max", np.max), ("min", np.min)):
            out = capi.empty((outer, inner))
            capi.call("reduce", C.c_int(REDUCE[kind]), dx.ptr, C.c_int64(outer), C.c_int64(ln), C.c_int64(inner), out.ptr)
            assert_close(out.numpy(), f(x.astype(np.float64), axis=1), 1e-4, f"{kind} [{outer},{ln},{inner}]")
    host = C.c_float(0)
    x = r.standard_normal(100001).astype(np.float32)
    capi.call("sum_all_host", capi.to_device(x).ptr, C.c_int64(x.size), C.byref(host))
    assert abs(host.value - x.astype(np.float64).sum()) < 1e-2


def test_gemm_transposes_ld_and_accumulate(capi):
    r = rng(66)
    m, n, k = 70, 50, 90
    for ta in (0, 1):
        for tb in (0, 1):
            a = r.standard_normal((k, m) if ta else (m, k)).astype(np.float32)
            b = r.standard_normal((n, k) if tb else (k, n)).astype(np.float32)
            c0 = r.standard_normal((m, n)).astype(np.float32)
            dc = capi.to_device(c0)
            capi.call("gemm", C.c_int(ta), C.c_int(tb), C.c_int64(m), C.c_int64(n), C.c_int64(k), capi.to_device(a).ptr,
                      C.c_int64(a.shape[1]), capi.to_device(b).ptr, C.c_int64(b.shape[1]), dc.ptr, C.c_int64(n), C.c_int(1))
            A = a.T if ta else a
            B = b.T if tb else b
            assert_close(dc.numpy(), c0 + A.astype(np.float64) @ B.astype(np.float64), 1e-4, f"gemm ta={ta} tb={tb} accumulate")
    # split-K path: tiny output, long reduction
    a = r.standard_normal((20000, 24)).astype(np.float32)
    g = r.standard_normal((20000, 40)).astype(np.float32)
    out = capi.empty((24, 40))
    capi.call("gemm", C.c_int(1), C.c_int(0), C.c_int64(24), C.c_int64(40), C.c_int64(20000), capi.to_device(a).ptr, C.c_int64(24),
              capi.to_device(g).ptr, C.c_int64(40), out.ptr, C.c_int64(40), C.c_int(0))
    assert_close(out.numpy(), a.astype(np.float64).T @ g.astype(np.float64), 1e-4, "split-K gemm")


def test_gemm_narrow_products(capi):
    """Classifier-head shapes (N <= 16) and their input gradients (K <= 16) take dedicated kernels: every storage
    order, padded leading dimensions, accumulate, ragged extents around the 32-row / 128-k tiles."""
    r = rng(74)
    shapes = [(256, 10, 128), (128, 10, 256), (256, 128, 10), (1, 1, 1), (33, 16, 129), (31, 3, 4097), (5000, 7, 40),
              (65, 200, 16), (3, 2, 5)]
    for (m, n, k) in shapes:
        for ta in (0, 1):
            for tb in (0, 1):
                for acc in (0, 1):
                    pad_a, pad_b, pad_c = 3, 2, 5
                    a = r.standard_normal((k, m + pad_a) if ta else (m, k + pad_a)).astype(np.float32)
                    b = r.standard_normal((n, k + pad_b) if tb else (k, n + pad_b)).astype(np.float32)
                    c0 = r.standard_normal((m, n + pad_c)).astype(np.float32)
                    dc = capi.to_device(c0)
                    capi.call("gemm", C.c_int(ta), C.c_int(tb), C.c_int64(m), C.c_int64(n), C.c_int64(k), capi.to_device(a).ptr,
                              C.c_int64(a.shape[1]), capi.to_device(b).ptr, C.c_int64(b.shape[1]), dc.ptr, C.c_int64(n + pad_c),
                              C.c_int(acc))
                    A = (a[:, :m].T if ta else a[:, :k]).astype(np.float64)
                    B = (b[:, :k].T if tb else b[:, :n]).astype(np.float64)
                    want = c0.astype(np.float64)
                    want[:, :n] = (want[:, :n] if acc else 0.0) + A @ B
                    assert_close(dc.numpy(), want, 1e-4, f"narrow gemm {m}x{n}x{k} ta={ta} tb={tb} acc={acc}")
                    assert np.array_equal(dc.numpy()[:, n:], c0[:, n:]), "padding columns of C were written"


def test_optimizer_multi_matches_per_tensor(capi):
    r = rng(67)
    sizes = [1, 7, 4096, 5000, 33]
    ps = [r.standard_normal(s).astype(np.float32) for s in sizes]
    gs = [r.standard_normal(s).astype(np.float32) * 10 for s in sizes]
    single, multi = [], []
    for p, g in zip(ps, gs):
        dp, dg, dm, dv = capi.to_device(p), capi.to_device(np.clip(g, -5, 5) * 0.5), capi.to_device(np.zeros_like(p)), capi.to_device(np.zeros_like(p))
        capi.call("adam_step", dp.ptr, dg.ptr, dm.ptr, dv.ptr, C.c_int64(p.size), C.c_float(1e-3), C.c_float(0.9), C.c_float(0.999),
                  C.c_float(1e-8), C.c_int64(3))
        single.append((dp.numpy(), dm.numpy(), dv.numpy()))
    dps = [capi.to_device(p) for p in ps]
    dgs = [capi.to_device(g) for g in gs]
    dms = [capi.to_device(np.zeros_like(p)) for p in ps]
    dvs = [capi.to_device(np.zeros_like(p)) for p in ps]
    arr = lambda ds: (C.c_void_p * len(ds))(*[d.ptr for d in ds])
    capi.call("optimizer_step_multi", C.c_int(1), C.c_int(len(ps)), arr(dps), arr(dgs), arr(dms), arr(dvs), capi.i64(sizes),
              C.c_float(1e-3), C.c_float(0.9), C.c_float(0.999), C.c_float(1e-8), C.c_float(0), C.c_int64(3), C.c_float(0.5),
              C.c_int(1), C.c_float(-5), C.c_float(5))
    for i in range(len(ps)):
        assert_close(dps[i].numpy(), single[i][0], 1e-6, "multi-tensor Adam params")
        assert_close(dms[i].numpy(), single[i][1], 1e-6, "m")
        assert_close(dvs[i].numpy(), single[i][2], 1e-6, "v")


def test_argument_validation(capi):
    with pytest.raises(RtError) as ei:
        capi.call("unary", C.c_int(99), None, None, C.c_int64(4), C.c_float(0), C.c_float(0))
    assert ei.value.code == 4
    with pytest.raises(RtError) as ei:
        capi.call("unary", C.c_int(UNARY["div_scalar"]), capi.empty((4,)).ptr, capi.empty((4,)).ptr, C.c_int64(4), C.c_float(0), C.c_float(0))
    assert ei.value.code == 4
    with pytest.raises(RtError):
        capi.call("adam_step", capi.empty((4,)).ptr, capi.empty((4,)).ptr, capi.empty((4,)).ptr, capi.empty((4,)).ptr, C.c_int64(4),
                  C.c_float(1e-3), C.c_float(0.9), C.c_float(0.999), C.c_float(1e-8), C.c_int64(0))
    # empty tensors are no-ops
    capi.call("unary", C.c_int(0), None, None, C.c_int64(0), C.c_float(0), C.c_float(0))
    capi.call("reduce", C.c_int(0), None, C.c_int64(0), C.c_int64(5), C.c_int64(3), None)


def test_upload_pipeline_and_events(capi):
    """rt_upload_*: two pinned / staging buffer pairs alternate; data arrives in submit order; rt_event_* waits."""
    n = 1 << 16
    up = C.c_void_p()
    capi.call("upload_create", C.c_size_t(4 * n), C.byref(up))
    ev = C.c_void_p()
    capi.call("event_create", C.byref(ev))
    dst = capi.empty((n,))
    acc = capi.to_device(np.zeros(n, np.float32))
    sh = capi.i64([n])
    seen = []
    for step in range(5):
        p = C.c_void_p()
        capi.call("upload_host_buffer", up, C.byref(p))
        seen.append(p.value)
        host = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_float)), shape=(n,))
        host[...] = np.arange(n, dtype=np.float32) + 1000.0 * step
        capi.call("upload_submit", up, dst.ptr)
        # consume on the context's stream: acc += dst
        capi.call("binary", C.c_int(BINARY["add"]), acc.ptr, sh, C.c_int(1), dst.ptr, sh, C.c_int(1), acc.ptr)
        capi.call("event_record", ev)
    capi.call("event_synchronize", ev)
    assert seen[0] != seen[1] and seen[0] == seen[2] == seen[4] and seen[1] == seen[3]
    want = 5 * np.arange(n, dtype=np.float64) + 1000.0 * (0 + 1 + 2 + 3 + 4)
    assert np.array_equal(acc.numpy(), want.astype(np.float32))
    capi.call("event_destroy", ev)
    capi.call("upload_destroy", up)


def test_upload_submit_all_and_publish_to_host(capi):
    """rt_upload_submit_all: several uploads, one staging -> destination kernel (sizes that are and are not multiples of 16
    bytes, a destination that is not 16-byte aligned); rt_publish_to_host: values land in pinned memory once an event recorded
    after the call has completed, and a destination that is not pinned host memory is refused."""
    sizes = [1 << 16, 2560, 7, 1]
    ups = []
    for n in sizes:
        up = C.c_void_p()
        capi.call("upload_create", C.c_size_t(4 * n), C.byref(up))
        ups.append(up)
    big = capi.empty((sizes[0] + 1,))
    dsts = [capi.empty((n,)) for n in sizes[1:]]
    ptrs = [C.c_void_p(big.ptr.value + 4)] + [d.ptr for d in dsts]  # the first destination starts 4 bytes into its buffer
    ev = C.c_void_p()
    capi.call("event_create", C.byref(ev))
    up_arr = (C.c_void_p * len(ups))(*[u.value for u in ups])
    dst_arr = (C.c_void_p * len(ups))(*[q.value for q in ptrs])
    total = capi.to_device(np.zeros(1, np.float32))
    out = C.c_void_p()
    capi.call("host_alloc", C.c_size_t(4), C.byref(out))
    host_out = np.ctypeslib.as_array(C.cast(out, C.POINTER(C.c_float)), shape=(1,))
    for step in range(3):
        want = []
        for up, n in zip(ups, sizes):
            p = C.c_void_p()
            capi.call("upload_host_buffer", up, C.byref(p))
            host = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_float)), shape=(n,))
            host[...] = np.arange(n, dtype=np.float32) * (step + 1) + n
            want.append(host.copy())
        capi.call("upload_submit_all", up_arr, dst_arr, C.c_int(len(ups)))
        capi.call("reduce", C.c_int(REDUCE["sum"]), dsts[0].ptr, C.c_int64(1), C.c_int64(sizes[1]), C.c_int64(1), total.ptr)
        capi.call("publish_to_host", out, total.ptr, C.c_int64(1))
        capi.call("event_record", ev)
        capi.call("event_synchronize", ev)
        assert_close(host_out.copy(), np.array([want[1].astype(np.float64).sum()]), 1e-5, "published sum")
        got = [big.numpy()[1:]] + [d.numpy() for d in dsts]
        for g, w in zip(got, want):
            assert np.array_equal(g, w)
    twice = (C.c_void_p * 2)(ups[0].value, ups[0].value)
    pageable = np.zeros(4, np.float32)
    for name, args in (("upload_submit_all", (up_arr, dst_arr, C.c_int(0))), ("upload_submit_all", (twice, dst_arr, C.c_int(2))),
                       ("publish_to_host", (pageable.ctypes.data_as(C.c_void_p), total.ptr, C.c_int64(1))),
                       ("publish_to_host", (total.ptr, total.ptr, C.c_int64(1)))):
        with pytest.raises(RtError) as ei:
            capi.call(name, *args)
        assert ei.value.code == 4
    capi.call("host_free", out)
    capi.call("event_destroy", ev)
    for up in ups:
        capi.call("upload_destroy", up)


def test_side_stream_sections(capi):
    """Work issued between rt_side_stream_begin and _end runs after what was queued before and is waited for by _join;
    nesting, joining inside a section and allocating inside a section are refused."""
    n = 1 << 20
    a = capi.to_device(np.full(n, 2.0, np.float32))
    b, c = capi.empty((n,)), capi.empty((n,))
    capi.call("unary", C.c_int(UNARY["square"]), a.ptr, b.ptr, C.c_int64(n), C.c_float(0), C.c_float(0))   # main: b = 4
    capi.call("side_stream_begin")
    capi.call("unary", C.c_int(UNARY["exp"]), b.ptr, c.ptr, C.c_int64(n), C.c_float(0), C.c_float(0))      # side: c = e^4
    with pytest.raises(RtError):
        capi.call("side_stream_begin")
    with pytest.raises(RtError):
        capi.call("side_stream_join")
    with pytest.raises(RtError):
        capi.empty((16,))
    capi.call("side_stream_end")
    capi.call("unary", C.c_int(UNARY["square"]), b.ptr, a.ptr, C.c_int64(n), C.c_float(0), C.c_float(0))   # main: a = 16
    capi.call("side_stream_join")
    capi.call("binary", C.c_int(BINARY["add"]), a.ptr, capi.i64([n]), C.c_int(1), c.ptr, capi.i64([n]), C.c_int(1), b.ptr)
    assert_close(b.numpy(), np.full(n, 16.0 + np.exp(4.0)), 1e-6, "side stream result joined into the main stream")
    capi.call("side_stream_join")  # nothing pending: a no-op
    with pytest.raises(RtError):
        capi.call("side_stream_end")


def test_fused_relu_max_pool_is_bit_identical_to_the_two_ops(capi):
    r = rng(71)
    i64, i32 = C.c_int64, C.c_int
    for (n, c, h, w, k, st, pd) in ((3, 5, 8, 12, 2, 2, 0), (2, 3, 9, 7, 3, 2, 1), (2, 2, 6, 6, 2, 1, 0), (4, 32, 28, 28, 2, 2, 0)):
        x = r.standard_normal((n, c, h, w)).astype(np.float32)
        x[r.random(x.shape) < 0.1] = 0.0   # exact zeros and all-negative windows exercise the first-maximum rule
        ho, wo = (h + 2 * pd - k) // st + 1, (w + 2 * pd - k) // st + 1
        g = r.standard_normal((n, c, ho, wo)).astype(np.float32)
        dx_, dg = capi.to_device(x), capi.to_device(g)
        args = (i64(n), i64(c), i64(h), i64(w), i32(k), i32(k), i32(st), i32(st), i32(pd), i32(pd))
        # two ops
        rl, y0, i0 = capi.empty(x.shape), capi.empty(g.shape), capi.empty(g.shape)
        capi.call("unary", i32(UNARY["relu"]), dx_.ptr, rl.ptr, i64(x.size), C.c_float(0), C.c_float(0))
        capi.call("max_pool2d", rl.ptr, *args, y0.ptr, i0.ptr)
        dp, d0 = capi.empty(x.shape), capi.empty(x.shape)
        capi.call("max_pool2d_backward", dg.ptr, i0.ptr, *args, dp.ptr)
        capi.call("unary_backward", i32(UNARY["relu"]), dx_.ptr, dp.ptr, d0.ptr, i64(x.size), C.c_float(0), C.c_float(0))
        # fused
        y1, i1, d1 = capi.empty(g.shape), capi.empty(g.shape), capi.empty(x.shape)
        capi.call("relu_max_pool2d", dx_.ptr, *args, y1.ptr, i1.ptr)
        capi.call("relu_max_pool2d_backward", dx_.ptr, dg.ptr, i1.ptr, *args, d1.ptr)
        assert np.array_equal(y1.numpy(), y0.numpy()) and np.array_equal(i1.numpy(), i0.numpy())
        assert np.array_equal(d1.numpy(), d0.numpy())


@pytest.mark.parametrize("shape", [(4, 1, 28, 28, 32, 1), (3, 1, 12, 8, 20, 1), (2, 1, 10, 10, 5, 0), (2, 3, 8, 12, 6, 1), (2, 32, 14, 14, 64, 1)],
                         ids=str)
def test_fused_conv_relu_pool_is_bit_identical_to_the_three_ops(capi, shape):
    """rt_conv2d_relu_max_pool2x2 against rt_conv2d -> relu -> rt_max_pool2d(2x2, stride 2): pooled values, indices and the
    gradient of the convolution output (from the pooled output, without the un-pooled tensor) must be equal bit for bit - for the
    single-channel 3x3 layers that run as one kernel (16 and 4 channels in the last group, no padding) and for the shapes that
    run as convolution + fused pooling."""
    n, cin, h, w, cout, pad = shape
    r = rng(77)
    i64, i32 = C.c_int64, C.c_int
    x = r.standard_normal((n, cin, h, w)).astype(np.float32)
    wt = (r.standard_normal((cout, cin, 3, 3)) / 3.0).astype(np.float32)
    b = r.standard_normal(cout).astype(np.float32)
    b[::3] = -5.0                                           # whole windows below zero: relu ties, first position wins
    ho, wo = h + 2 * pad - 2, w + 2 * pad - 2
    assert ho % 2 == 0 and wo % 2 == 0
    dx_, dw_, db_ = capi.to_device(x), capi.to_device(wt), capi.to_device(b)
    conv_args = (i64(n), i64(cin), i64(h), i64(w), i64(cout), i32(3), i32(3), i32(1), i32(1), i32(pad), i32(pad))
    pool_args = (i64(n), i64(cout), i64(ho), i64(wo), i32(2), i32(2), i32(2), i32(2), i32(0), i32(0))
    conv, rl = capi.empty((n, cout, ho, wo)), capi.empty((n, cout, ho, wo))
    y0, i0 = capi.empty((n, cout, ho // 2, wo // 2)), capi.empty((n, cout, ho // 2, wo // 2))
    capi.call("conv2d", dx_.ptr, dw_.ptr, db_.ptr, *conv_args, conv.ptr)
    capi.call("unary", i32(UNARY["relu"]), conv.ptr, rl.ptr, i64(conv.size), C.c_float(0), C.c_float(0))
    capi.call("max_pool2d", rl.ptr, *pool_args, y0.ptr, i0.ptr)
    g = capi.to_device(r.standard_normal(y0.shape).astype(np.float32))
    dp, d0 = capi.empty(conv.shape), capi.empty(conv.shape)
    capi.call("max_pool2d_backward", g.ptr, i0.ptr, *pool_args, dp.ptr)
    capi.call("unary_backward", i32(UNARY["relu"]), conv.ptr, dp.ptr, d0.ptr, i64(conv.size), C.c_float(0), C.c_float(0))
    y1, i1, d1 = capi.empty(y0.shape), capi.empty(y0.shape), capi.empty(conv.shape)
    capi.call("conv2d_relu_max_pool2x2", dx_.ptr, dw_.ptr, db_.ptr, *conv_args, y1.ptr, i1.ptr)
    capi.call("relu_max_pool2x2_backward_from_output", y1.ptr, g.ptr, i1.ptr, i64(n), i64(cout), i64(ho), i64(wo), d1.ptr)
    assert np.array_equal(y1.numpy(), y0.numpy())
    assert np.array_equal(i1.numpy(), i0.numpy())
    assert np.array_equal(d1.numpy(), d0.numpy())
    assert (y0.numpy() == 0).any() and (y0.numpy() > 0).any()


def test_fused_conv_relu_pool_rejects_odd_outputs(capi):
    from rusttensor_b200.capi import RtError

    x, wt = capi.to_device(np.zeros((1, 1, 7, 7), np.float32)), capi.to_device(np.zeros((2, 1, 3, 3), np.float32))
    y, idx = capi.empty((1, 2, 3, 3)), capi.empty((1, 2, 3, 3))
    with pytest.raises(RtError) as ei:
        capi.call("conv2d_relu_max_pool2x2", x.ptr, wt.ptr, None, C.c_int64(1), C.c_int64(1), C.c_int64(7), C.c_int64(7), C.c_int64(2), C.c_int(3),
                  C.c_int(3), C.c_int(1), C.c_int(1), C.c_int(1), C.c_int(1), y.ptr, idx.ptr)
    assert ei.value.code == 4


def test_gradient_accumulation_inside_the_producing_kernels(capi):
    """rt_matmul_backward_accumulate adds a^T g to a gradient that already exists (and still returns dA), rt_sum_rows_accumulate
    adds the column sums of g to an existing bias gradient: what add_grad does with a separate addition for a weight used at
    every timestep.  Widths that are and are not multiples of four (the epilogue's 128-bit path and its scalar path)."""
    r = rng(81)
    i64 = C.c_int64
    for (m, k, n) in ((64, 577, 2048), (64, 512, 65), (33, 70, 36), (128, 256, 128)):
        a = r.standard_normal((m, k)).astype(np.float32)
        b = r.standard_normal((k, n)).astype(np.float32)
        g = r.standard_normal((m, n)).astype(np.float32)
        old = r.standard_normal((k, n)).astype(np.float32)
        da, acc = capi.empty((m, k)), capi.to_device(old)
        a_d, b_d, g_d = capi.to_device(a), capi.to_device(b), capi.to_device(g)  # kept alive: a released block is handed out again
        capi.call("matmul_backward_accumulate", a_d.ptr, b_d.ptr, g_d.ptr, i64(m), i64(k), i64(n), da.ptr, acc.ptr)
        assert_close(da.numpy(), (g.astype(np.float64) @ b.astype(np.float64).T), 1e-4, f"dA {m}x{k}x{n}")
        assert_close(acc.numpy(), old.astype(np.float64) + a.astype(np.float64).T @ g.astype(np.float64), 1e-4, f"accumulated dB {m}x{k}x{n}")
        # without dA (the first operand takes no gradient)
        acc2 = capi.to_device(old)
        capi.call("matmul_backward_accumulate", a_d.ptr, b_d.ptr, g_d.ptr, i64(m), i64(k), i64(n), None, acc2.ptr)
        assert np.array_equal(acc2.numpy(), acc.numpy())
    for (rows, cols) in ((64, 2048), (1, 5), (7, 300), (0, 9)):
        g = r.standard_normal((rows, cols)).astype(np.float32)
        old = r.standard_normal(cols).astype(np.float32)
        acc = capi.to_device(old)
        g_d = capi.to_device(g) if rows else None
        capi.call("sum_rows_accumulate", g_d.ptr if rows else None, i64(rows), i64(cols), acc.ptr)
        assert_close(acc.numpy(), old.astype(np.float64) + g.astype(np.float64).sum(axis=0), 1e-5, f"bias accumulation {rows}x{cols}")


def test_blocking_copies_are_refused_during_capture(capi):
    """A copy that synchronises the stream cannot be recorded in a graph; it is refused with a clear error instead of breaking
    the capture, which can still be ended and replayed."""
    a = capi.to_device(np.arange(8, dtype=np.float32))
    host = np.zeros(8, np.float32)
    graph = C.c_void_p()
    capi.call("graph_begin")
    try:
        with pytest.raises(RtError) as ei:
            capi.check(capi.lib.rt_memcpy_d2h(capi.ctx, host.ctypes.data_as(C.c_void_p), a.ptr, C.c_size_t(32)))
        assert ei.value.code == 4 and "graph" in str(ei.value)
        with pytest.raises(RtError):
            capi.check(capi.lib.rt_memcpy_h2d(capi.ctx, a.ptr, host.ctypes.data_as(C.c_void_p), C.c_size_t(32)))
        capi.call("unary", C.c_int(UNARY["exp"]), a.ptr, a.ptr, C.c_int64(8), C.c_float(0), C.c_float(0))
    finally:
        capi.call("graph_end", C.byref(graph))
    capi.call("graph_launch", graph)
    capi.sync()
    assert_close(a.numpy(), np.exp(np.arange(8, dtype=np.float32)), 1e-6, "captured kernel replayed")
    capi.call("graph_destroy", graph)


def test_max_pool_backward_with_overlapping_windows_is_reproducible(capi):
    """stride < kernel: several windows can route their gradient to one input element.  The sum is formed in the order
    of the reference's sequential scatter (ascending output index), so it equals a float32 replay of that loop bit for
    bit and does not change from run to run."""
    r = rng(75)
    i64, i32 = C.c_int64, C.c_int
    for (n, c, h, w, k, st, pd) in ((2, 3, 9, 7, 3, 2, 1), (2, 2, 6, 6, 2, 1, 0), (1, 1, 5, 5, 3, 1, 1), (3, 4, 12, 12, 4, 2, 0)):
        x = r.integers(-2, 3, (n, c, h, w)).astype(np.float32)   # many ties: shared maxima between neighbouring windows
        ho, wo = (h + 2 * pd - k) // st + 1, (w + 2 * pd - k) // st + 1
        g = r.standard_normal((n, c, ho, wo)).astype(np.float32)
        dx_, dg = capi.to_device(x), capi.to_device(g)
        args = (i64(n), i64(c), i64(h), i64(w), i32(k), i32(k), i32(st), i32(st), i32(pd), i32(pd))
        y, idx = capi.empty(g.shape), capi.empty(g.shape)
        capi.call("max_pool2d", dx_.ptr, *args, y.ptr, idx.ptr)
        runs = []
        for _ in range(4):
            d = capi.empty(x.shape)
            capi.call("max_pool2d_backward", dg.ptr, idx.ptr, *args, d.ptr)
            runs.append(d.numpy())
        want = np.zeros_like(x)
        flat = np.rint(idx.numpy()).astype(np.int64)
        for b in range(n):
            for ch in range(c):
                for yo in range(ho):
                    for xo in range(wo):
                        ky, kx = divmod(int(flat[b, ch, yo, xo]), k)
                        iy, ix = yo * st + ky - pd, xo * st + kx - pd
                        if 0 <= iy < h and 0 <= ix < w:
                            want[b, ch, iy, ix] = np.float32(want[b, ch, iy, ix] + g[b, ch, yo, xo])
        for d in runs:
            assert np.array_equal(d, want)


def test_two_stream_backward_is_bit_identical_to_serial(capi):
    """matmul / conv / conv-transpose backward issue their independent halves on two streams (scratch allocated on the
    side stream, frees parked until the join).  Alternating shapes back to back, so that scratch blocks get recycled
    between the streams, every gradient must equal the single-stream result bit for bit."""
    r = rng(76)
    i64, i32 = C.c_int64, C.c_int

    def run_all():
        outs = []
        for rep in range(3):
            for (m, k, n) in ((256, 3136, 128), (64, 577, 2048), (256, 128, 10), (70, 90, 50)):
                rr = rng(1000 + m + k + n)
                a = capi.to_device(rr.standard_normal((m, k)).astype(np.float32))
                b = capi.to_device(rr.standard_normal((k, n)).astype(np.float32))
                g = capi.to_device(rr.standard_normal((m, n)).astype(np.float32))
                da, db = capi.empty((m, k)), capi.empty((k, n))
                capi.call("matmul_backward", a.ptr, b.ptr, g.ptr, i64(m), i64(k), i64(n), da.ptr, db.ptr)
                outs += [da.numpy(), db.numpy()]
            for (nb, cin, hw, cout, ks, st, pd) in ((16, 32, 14, 64, 3, 1, 1), (4, 3, 9, 5, 3, 2, 1), (8, 1, 28, 32, 3, 1, 1)):
                rr = rng(2000 + nb + cin + hw)
                ho = (hw + 2 * pd - ks) // st + 1
                x = capi.to_device(rr.standard_normal((nb, cin, hw, hw)).astype(np.float32))
                w = capi.to_device(rr.standard_normal((cout, cin, ks, ks)).astype(np.float32))
                g = capi.to_device(rr.standard_normal((nb, cout, ho, ho)).astype(np.float32))
                dx, dw, db = capi.empty((nb, cin, hw, hw)), capi.empty((cout, cin, ks, ks)), capi.empty((cout,))
                capi.call("conv2d_backward", x.ptr, w.ptr, g.ptr, i64(nb), i64(cin), i64(hw), i64(hw), i64(cout), i32(ks), i32(ks),
                          i32(st), i32(st), i32(pd), i32(pd), dx.ptr, dw.ptr, db.ptr)
                outs += [dx.numpy(), dw.numpy(), db.numpy()]
                # transposed: x [nb, cout, ho, ho] -> y [nb, cin, hw', hw'], weights [cout, cin, ks, ks]
                ot = (ho - 1) * st + ks - 2 * pd
                xt = capi.to_device(rr.standard_normal((nb, cout, ho, ho)).astype(np.float32))
                gt = capi.to_device(rr.standard_normal((nb, cin, ot, ot)).astype(np.float32))
                dxt, dwt, dbt = capi.empty((nb, cout, ho, ho)), capi.empty((cout, cin, ks, ks)), capi.empty((cin,))
                capi.call("conv2d_transpose_backward", xt.ptr, w.ptr, gt.ptr, i64(nb), i64(cout), i64(ho), i64(ho), i64(cin), i32(ks),
                          i32(ks), i32(st), i32(st), i32(pd), i32(pd), dxt.ptr, dwt.ptr, dbt.ptr)
                outs += [dxt.numpy(), dwt.numpy(), dbt.numpy()]
        return outs

    try:
        capi.call("set_concurrent_backward", i32(0))
        serial = run_all()
        capi.call("set_concurrent_backward", i32(1))
        forked = run_all()
    finally:
        capi.call("set_concurrent_backward", i32(1))
    assert len(serial) == len(forked)
    for i, (a, b) in enumerate(zip(serial, forked)):
        assert np.array_equal(a, b), f"output {i} differs between the two-stream and the single-stream backward"


def test_fused_softmax_cross_entropy(capi):
    r = rng(72)
    for rows, classes in ((1, 1), (7, 10), (256, 10), (64, 65), (1000, 33)):
        x = (3 * r.standard_normal((rows, classes))).astype(np.float32)
        t = np.eye(classes, dtype=np.float32)[r.integers(0, classes, rows)]
        t[0] = r.random(classes).astype(np.float32)   # a soft target row
        gup = np.array([1.7], np.float32)
        dx_, dt, dgu = capi.to_device(x), capi.to_device(t), capi.to_device(gup)
        loss, dl, dtt = capi.empty((1,)), capi.empty(x.shape), capi.empty(x.shape)
        capi.call("softmax_cross_entropy", dx_.ptr, dt.ptr, C.c_int64(rows), C.c_int64(classes), loss.ptr)
        capi.call("softmax_cross_entropy_backward", dx_.ptr, dt.ptr, dgu.ptr, C.c_int64(rows), C.c_int64(classes), dl.ptr, dtt.ptr)
        x64, t64 = x.astype(np.float64), t.astype(np.float64)
        ls = x64 - x64.max(1, keepdims=True)
        ls = ls - np.log(np.exp(ls).sum(1, keepdims=True))
        assert_close(loss.numpy(), np.array([-(ls * t64).sum() / rows]), 1e-5, f"loss [{rows},{classes}]")
        sc = -1.7 / rows
        assert_close(dl.numpy(), sc * (t64 - np.exp(ls) * t64.sum(1, keepdims=True)), 1e-4, "dlogits", abs_floor=1e-7)
        assert_close(dtt.numpy(), sc * ls, 1e-5, "dtargets")
        capi.call("softmax_cross_entropy_backward", dx_.ptr, dt.ptr, dgu.ptr, C.c_int64(rows), C.c_int64(classes), dl.ptr, None)
    with pytest.raises(RtError):
        capi.call("softmax_cross_entropy", dx_.ptr, dt.ptr, C.c_int64(0), C.c_int64(5), loss.ptr)


def test_fused_lstm_cell(capi):
    r = rng(73)
    sig = lambda v: 1.0 / (1.0 + np.exp(-v))
    for batch, hidden in ((1, 1), (3, 5), (64, 128), (7, 33)):
        gates = (2 * r.standard_normal((batch, 4 * hidden))).astype(np.float32)
        cp = r.standard_normal((batch, hidden)).astype(np.float32)
        up = r.standard_normal((batch, hidden)).astype(np.float32)
        dg_, dcp, dup = capi.to_device(gates), capi.to_device(cp), capi.to_device(up)
        dims = (C.c_int64(batch), C.c_int64(hidden))
        g64 = gates.astype(np.float64)
        i, f, g, o = (g64[:, k * hidden:(k + 1) * hidden] for k in range(4))
        si, sf, tg, so = sig(i), sig(f), np.tanh(g), sig(o)
        # c = sigmoid(f) * c_prev + sigmoid(i) * tanh(g)
        c, dgates, dprev = capi.empty(cp.shape), capi.empty(gates.shape), capi.empty(cp.shape)
        capi.call("lstm_cell_c", dg_.ptr, dcp.ptr, *dims, c.ptr)
        capi.call("lstm_cell_c_backward", dg_.ptr, dcp.ptr, dup.ptr, *dims, dgates.ptr, dprev.ptr)
        c64 = sf * cp + si * tg
        assert_close(c.numpy(), c64, 1e-5, f"c [{batch},{hidden}]", abs_floor=1e-6)
        want = np.concatenate([up * tg * si * (1 - si), up * cp * sf * (1 - sf), up * si * (1 - tg * tg), np.zeros_like(c64)], axis=1)
        assert_close(dgates.numpy(), want, 1e-4, "c: dgates", abs_floor=1e-6)
        assert_close(dprev.numpy(), up * sf, 1e-5, "c: dc_prev", abs_floor=1e-6)
        capi.call("lstm_cell_c_backward", dg_.ptr, dcp.ptr, dup.ptr, *dims, None, dprev.ptr)
        capi.call("lstm_cell_c_backward", dg_.ptr, dcp.ptr, dup.ptr, *dims, dgates.ptr, None)
        # h = sigmoid(o) * tanh(c)
        h, dgates2, dc = capi.empty(cp.shape), capi.empty(gates.shape), capi.empty(cp.shape)
        capi.call("lstm_cell_h", dg_.ptr, c.ptr, *dims, h.ptr)
        capi.call("lstm_cell_h_backward", dg_.ptr, c.ptr, dup.ptr, *dims, dgates2.ptr, dc.ptr)
        tc = np.tanh(c.numpy().astype(np.float64))
        assert_close(h.numpy(), so * tc, 1e-5, "h", abs_floor=1e-6)
        want = np.concatenate([np.zeros((batch, 3 * hidden)), up * tc * so * (1 - so)], axis=1)
        assert_close(dgates2.numpy(), want, 1e-4, "h: dgates", abs_floor=1e-6)
        assert_close(dc.numpy(), up * so * (1 - tc * tc), 1e-4, "h: dc", abs_floor=1e-6)
    capi.call("lstm_cell_c", dg_.ptr, dcp.ptr, C.c_int64(0), C.c_int64(4), c.ptr)   # empty batch: nothing to do
    with pytest.raises(RtError):
        capi.call("lstm_cell_h", dg_.ptr, dcp.ptr, C.c_int64(-1), C.c_int64(4), h.ptr)


def test_peer_wait_runs_out_and_the_update_is_skipped_everywhere(capi):
    """The exchange over peer memory, emulated on one GPU (both "ranks" are local buffers; nothing here waits on another
    launch).  First the flag of rank 1 is never written: rt_dp_wait_peers gives up after its poll limit, the optimizer
    kernel that follows changes nothing - parameters, first and second moments stay bit-identical - and the next
    synchronising call reports RT_ERR_TIMEOUT.  Then the flag is set from the host and the same sequence applies one
    Adam step on the sum of both ranks' gradients."""
    from rusttensor_b200.capi import RtError

    r = np.random.default_rng(5)
    n1, n2 = 70001, 333
    sizes = capi.i64([n1, n2])
    pad1 = (n1 + 3) // 4 * 4
    flat_len = pad1 + (n2 + 3) // 4 * 4
    p_host = [r.standard_normal(n).astype(np.float32) for n in (n1, n2)]
    g0, g1 = r.standard_normal(flat_len).astype(np.float32), r.standard_normal(flat_len).astype(np.float32)
    params = [capi.to_device(a) for a in p_host]
    m = [capi.to_device(np.zeros(n, np.float32)) for n in (n1, n2)]
    v = [capi.to_device(np.zeros(n, np.float32)) for n in (n1, n2)]
    flat0 = [capi.to_device(g0), capi.to_device(g1)]      # even steps: rank 0's and rank 1's packed gradients
    flat1 = [capi.to_device(g1), capi.to_device(g0)]      # odd steps (the other way round, to tell the buffers apart)
    state = capi.to_device(np.zeros(4, np.float32))       # RT_STEP_STATE_WORDS ints, all zero
    flags = capi.to_device(np.zeros(8, np.float32))       # this rank's flag array
    ptrs = lambda arrs: (C.c_void_p * len(arrs))(*[a.ptr for a in arrs])
    grads = (C.c_void_p * 2)(flat0[0].ptr.value, flat0[0].ptr.value + 4 * pad1)

    def step(spin_limit):
        capi.call("dp_step_begin", state.ptr)
        capi.call("dp_wait_peers", flags.ptr, C.c_int(0), C.c_int(2), state.ptr, C.c_uint32(spin_limit))
        capi.call("optimizer_step_multi_peers", C.c_int(1), C.c_int(2), ptrs(params), grads, ptrs(m), ptrs(v), sizes, C.c_float(1e-3),
                  C.c_float(0.9), C.c_float(0.999), C.c_float(1e-8), C.c_float(0.0), C.c_float(0.5), ptrs(flat0), ptrs(flat1), C.c_int(0),
                  C.c_int(2), state.ptr)

    step(spin_limit=2000)                                  # rank 1 never signals step 1
    with pytest.raises(RtError) as ei:
        capi.sync()
    assert ei.value.code == 14                             # RT_ERR_TIMEOUT
    for a, b in zip(params, p_host):
        assert np.array_equal(a.numpy(), b)
    assert all(not x.numpy().any() for x in m + v)
    words = state.numpy().view(np.int32)
    assert words[0] == 1 and words[1] == -1 and words[2] == 1
    # rank 1 "signals" step 2; step 2 reads buffer 0 (2 & 1 == 0): gradient = (g0 + g1) / 2
    fl = np.zeros(8, np.int32)
    fl[1] = 2
    capi.check(capi.lib.rt_memcpy_h2d(capi.ctx, flags.ptr, fl.ctypes.data_as(C.c_void_p), C.c_size_t(fl.nbytes)))
    step(spin_limit=0)
    capi.sync()
    words = state.numpy().view(np.int32)
    assert words[0] == 2 and words[1] == 2 and words[2] == 2
    g = (g0 + g1) * np.float32(0.5)
    t = 2                                                   # the optimizer step count advanced with the failed step too
    for i, (n, off) in enumerate(((n1, 0), (n2, pad1))):
        gi = g[off:off + n].astype(np.float32)
        mi = np.float32(0.1) * gi
        vi = np.float32(0.001) * (gi * gi)
        bc1, bc2 = np.float32(1) - np.float32(0.9) ** t, np.float32(1) - np.float32(0.999) * np.float32(0.999)
        want = p_host[i] - np.float32(1e-3) * (mi / bc1) / (np.sqrt(vi / bc2) + np.float32(1e-8))
        assert_close(params[i].numpy(), want, 1e-5, f"peer Adam step, tensor {i}")
        assert_close(m[i].numpy(), mi, 1e-6, "first moment")
