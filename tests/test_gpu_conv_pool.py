"""conv2d / conv2d_transpose / max_pool2d / matmul on the CUDA backend vs the CPU oracle.
Pooling indices must be bit-exact; conv input gradients are compared with the oracle's
mathematically correct mode (the reference CPU code reuses column 0, src/ops/cpu_ops.rs:266),
everything else with the faithful mode."""
import numpy as np
import pytest

import oracle
import ref_f64
from helpers import assert_close, rng

pytestmark = pytest.mark.gpu
TOL = 1e-4

CONV = [
    (2, 3, 8, 8, 4, 3, (1, 1), (1, 1)), (1, 1, 7, 5, 2, 3, (1, 1), (0, 0)), (2, 2, 9, 9, 3, 3, (2, 2), (1, 1)),
    (1, 4, 6, 6, 5, 5, (1, 1), (2, 2)), (4, 1, 28, 28, 32, 3, (1, 1), (1, 1)), (3, 32, 14, 14, 64, 3, (1, 1), (1, 1)),
    (2, 5, 11, 13, 7, 3, (2, 1), (0, 1)), (1, 64, 12, 12, 128, 3, (1, 1), (1, 1)), (16, 32, 14, 14, 64, 3, (1, 1), (1, 1)),
    (8, 1, 28, 28, 32, 3, (1, 1), (1, 1)), (2, 64, 20, 20, 128, 3, (1, 1), (1, 1)), (3, 8, 10, 9, 16, 5, (1, 1), (2, 2)),
    # single-channel 3x3 inputs (the whole-image weight/bias gradient kernel): more images than SMs, more than 32 output
    # channels (two channel groups), a channel count that is no multiple of four, no padding, one image
    (301, 1, 12, 10, 5, 3, (1, 1), (1, 1)), (5, 1, 9, 11, 70, 3, (1, 1), (0, 0)), (1, 1, 28, 28, 33, 3, (1, 1), (1, 1)),
    (6, 1, 10, 16, 7, 3, (1, 1), (1, 1)), (3, 1, 10, 14, 9, 3, (1, 1), (0, 0)),  # output rows of 16 and 12 pixels: four pixels per lane
]


@pytest.mark.parametrize("n,cin,h,w,cout,k,stride,pad", CONV, ids=str)
def test_conv2d_forward_backward(oracle_engine, gpu_engine, contraction_path, n, cin, h, w, cout, k, stride, pad):
    r = rng(41)
    x = r.standard_normal((n, cin, h, w)).astype(np.float32)
    wt = (r.standard_normal((cout, cin, k, k)) / np.sqrt(cin * k * k)).astype(np.float32)
    b = r.standard_normal(cout).astype(np.float32)
    res = {}
    for name, e in (("cpu", oracle_engine), ("gpu", gpu_engine)):
        xt, wtt, bt = e.tensor(x, requires_grad=True), e.tensor(wt, requires_grad=True), e.tensor(b, requires_grad=True)
        y = e.ops.conv2d(xt, wtt, bt, stride, pad)
        if name == "cpu":
            g = rng(42).standard_normal(y.shape).astype(np.float32)
        y.set_grad(e.tensor(g))
        if name == "cpu":
            oracle.set_conv_dx_faithful(False)
        try:
            y.backward()
        finally:
            oracle.set_conv_dx_faithful(True)
        res[name] = (y.numpy(), xt.grad.numpy(), wtt.grad.numpy(), bt.grad.numpy())
    for i, what in enumerate(("forward", "dX", "dW", "db")):
        assert_close(res["gpu"][i], res["cpu"][i], TOL, f"conv2d {what}")
    dx64, dw64, db64 = ref_f64.conv2d_backward(x, wt, g, stride, pad)
    assert_close(res["gpu"][1], dx64, TOL, "conv2d dX vs float64")
    assert_close(res["gpu"][2], dw64, TOL, "conv2d dW vs float64")


@pytest.mark.parametrize("cin", [3, 1])
def test_conv2d_without_bias_and_frozen_input(oracle_engine, gpu_engine, contraction_path, cin):
    r = rng(43)
    x = r.standard_normal((2, cin, 6, 6)).astype(np.float32)
    w = r.standard_normal((4, cin, 3, 3)).astype(np.float32)
    res = []
    for e in (oracle_engine, gpu_engine):
        xt, wt = e.tensor(x, requires_grad=False), e.tensor(w, requires_grad=True)
        y = e.ops.conv2d(xt, wt, None, (1, 1), (1, 1))
        e.ops.sum(e.ops.square(y), None).backward()
        assert xt.grad is None
        res.append(wt.grad.numpy())
    assert_close(res[1], res[0], TOL, "dW without bias")


CONVT = [(2, 3, 4, 4, 2, 4, (2, 2), (1, 1)), (1, 2, 5, 3, 3, 3, (1, 1), (0, 0)), (1, 2, 3, 3, 2, 3, (2, 2), (0, 0)),
         (2, 1, 4, 4, 1, 2, (2, 2), (0, 0)), (2, 16, 7, 7, 8, 4, (2, 2), (1, 1)), (1, 128, 6, 6, 64, 4, (2, 2), (1, 1)),
         (4, 128, 14, 14, 64, 4, (2, 2), (1, 1)), (2, 6, 5, 7, 4, 3, (1, 2), (1, 0))]


@pytest.mark.parametrize("n,cin,h,w,cout,k,stride,pad", CONVT, ids=str)
def test_conv2d_transpose_forward_backward(oracle_engine, gpu_engine, contraction_path, n, cin, h, w, cout, k, stride, pad):
    r = rng(44)
    x = r.standard_normal((n, cin, h, w)).astype(np.float32)
    wt = (r.standard_normal((cin, cout, k, k)) / np.sqrt(cin * k * k)).astype(np.float32)
    b = r.standard_normal(cout).astype(np.float32)
    res = {}
    for name, e in (("cpu", oracle_engine), ("gpu", gpu_engine)):
        xt, wtt, bt = e.tensor(x, requires_grad=True), e.tensor(wt, requires_grad=True), e.tensor(b, requires_grad=True)
        y = e.ops.conv2d_transpose(xt, wtt, bt, stride, pad)
        if name == "cpu":
            g = rng(45).standard_normal(y.shape).astype(np.float32)
        y.set_grad(e.tensor(g))
        y.backward()
        res[name] = (y.numpy(), xt.grad.numpy(), wtt.grad.numpy(), bt.grad.numpy())
    for i, what in enumerate(("forward", "dX", "dW", "db")):
        assert_close(res["gpu"][i], res["cpu"][i], TOL, f"conv2d_transpose {what}")


POOL = [((2, 3, 8, 8), (2, 2), (2, 2), (0, 0)), ((4, 32, 28, 28), (2, 2), (2, 2), (0, 0)), ((4, 64, 14, 14), (2, 2), (2, 2), (0, 0)),
        ((1, 2, 7, 9), (3, 3), (2, 2), (1, 1)), ((1, 1, 5, 5), (3, 2), (1, 1), (0, 1)), ((2, 2, 9, 7), (2, 2), (2, 2), (0, 0)),
        ((1, 3, 6, 6), (2, 2), (3, 3), (0, 0)), ((2, 2, 8, 8), (3, 3), (1, 1), (1, 1))]


@pytest.mark.parametrize("shape,k,s,p", POOL, ids=str)
def test_max_pool2d_indices_bit_exact_and_backward(oracle_engine, gpu_engine, capi, shape, k, s, p):
    import ctypes as C

    r = rng(46)
    x = np.maximum(r.standard_normal(shape), 0).astype(np.float32)  # post-ReLU ties: whole windows of zeros
    res = []
    for e in (oracle_engine, gpu_engine):
        xt = e.tensor(x, requires_grad=True)
        y = e.ops.max_pool2d(xt, k, s, p)
        g = rng(47).standard_normal(y.shape).astype(np.float32)
        y.set_grad(e.tensor(g))
        y.backward()
        res.append((y.numpy(), xt.grad.numpy()))
    assert np.array_equal(res[0][0], res[1][0]), "pooled values must be identical"
    assert_close(res[1][1], res[0][1], 1e-6, "max_pool2d backward")
    # the index tensor itself, through the C ABI, against the float64-free numpy definition
    _, idx_ref = ref_f64.max_pool2d(x, k, s, p)
    dx = capi.to_device(x)
    dy, di = capi.empty(idx_ref.shape), capi.empty(idx_ref.shape)
    capi.call("max_pool2d", dx.ptr, C.c_int64(shape[0]), C.c_int64(shape[1]), C.c_int64(shape[2]), C.c_int64(shape[3]),
              C.c_int(k[0]), C.c_int(k[1]), C.c_int(s[0]), C.c_int(s[1]), C.c_int(p[0]), C.c_int(p[1]), dy.ptr, di.ptr)
    assert np.array_equal(di.numpy(), idx_ref), "argmax indices must be bit-exact"


MATMUL = [(2, 2, 2), (64, 784, 128), (64, 128, 10), (256, 3136, 128), (64, 577, 2048), (1, 7, 1), (130, 70, 33), (5, 1, 9), (257, 129, 65)]


@pytest.mark.parametrize("m,k,n", MATMUL, ids=str)
def test_matmul_forward_backward(oracle_engine, gpu_engine, contraction_path, m, k, n):
    r = rng(48)
    a = r.standard_normal((m, k)).astype(np.float32)
    b = (r.standard_normal((k, n)) / np.sqrt(k)).astype(np.float32)
    g = r.standard_normal((m, n)).astype(np.float32)
    res = []
    for e in (oracle_engine, gpu_engine):
        at, bt = e.tensor(a, requires_grad=True), e.tensor(b, requires_grad=True)
        c = e.ops.matmul(at, bt)
        c.set_grad(e.tensor(g))
        c.backward()
        res.append((c.numpy(), at.grad.numpy(), bt.grad.numpy()))
    ref = (a.astype(np.float64) @ b.astype(np.float64), g.astype(np.float64) @ b.astype(np.float64).T,
           a.astype(np.float64).T @ g.astype(np.float64))
    for i, what in enumerate(("C", "dA", "dB")):
        assert_close(res[1][i], res[0][i], TOL, f"matmul {what} vs oracle")
        assert_close(res[1][i], ref[i], TOL, f"matmul {what} vs float64")


def test_matmul_shape_errors(gpu_engine):
    from rusttensor_b200.frontend import EngineError

    a, b = gpu_engine.tensor(np.zeros((2, 3))), gpu_engine.tensor(np.zeros((4, 2)))
    with pytest.raises(EngineError) as ei:
        gpu_engine.ops.matmul(a, b)
    assert ei.value.kind == "IncompatibleShapes"
    with pytest.raises(EngineError) as ei:
        gpu_engine.ops.matmul(gpu_engine.tensor(np.zeros((2,))), b)
    assert ei.value.kind == "DimensionMismatch"
