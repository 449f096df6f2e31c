"""conv2d / conv2d_transpose / max_pool2d have no CPU test in the reference ("parity unpinned").
These tests bound the oracle's restatement of the reference source against independent float64
definitions and document the reference's conv2d input-gradient defect."""
import numpy as np
import pytest

import oracle
import ref_f64
from helpers import assert_close, rng

CONV_CASES = [
    # n, cin, h, w, cout, k, stride, pad
    (2, 3, 8, 8, 4, 3, (1, 1), (1, 1)),
    (1, 1, 7, 5, 2, 3, (1, 1), (0, 0)),
    (2, 2, 9, 9, 3, 3, (2, 2), (1, 1)),
    (1, 4, 6, 6, 5, 5, (1, 1), (2, 2)),
]


@pytest.mark.parametrize("n,cin,h,w,cout,k,stride,pad", CONV_CASES)
def test_conv2d_forward_and_weight_bias_grads(oracle_engine, n, cin, h, w, cout, k, stride, pad):
    e, ops = oracle_engine, oracle_engine.ops
    r = rng(1)
    x = r.standard_normal((n, cin, h, w)).astype(np.float32)
    wt = r.standard_normal((cout, cin, k, k)).astype(np.float32)
    b = r.standard_normal(cout).astype(np.float32)
    xt, wtt, bt = e.tensor(x, requires_grad=True), e.tensor(wt, requires_grad=True), e.tensor(b, requires_grad=True)
    y = ops.conv2d(xt, wtt, bt, stride, pad)
    yref = ref_f64.conv2d(x, wt, b, stride, pad)
    assert y.shape == yref.shape
    assert_close(y.numpy(), yref, 1e-4, "conv2d forward")
    g = r.standard_normal(yref.shape).astype(np.float32)
    y.set_grad(e.tensor(g))
    oracle.set_conv_dx_faithful(False)
    try:
        y.backward()
    finally:
        oracle.set_conv_dx_faithful(True)
    dx, dw, db = ref_f64.conv2d_backward(x, wt, g, stride, pad)
    assert_close(wtt.grad.numpy(), dw, 1e-4, "dW")
    assert_close(bt.grad.numpy(), db, 1e-4, "db")
    assert_close(xt.grad.numpy(), dx, 1e-4, "dX (corrected mode)")


def test_conv2d_input_gradient_defect_of_the_reference(oracle_engine):
    """In faithful mode the oracle reproduces src/ops/cpu_ops.rs:266,271: every output pixel
    scatters column 0 of grad_cols, so dX equals the contribution of output pixel (0,0) applied at
    every window position; dW and db are unaffected."""
    e, ops = oracle_engine, oracle_engine.ops
    r = rng(2)
    x = r.standard_normal((1, 2, 5, 5)).astype(np.float32)
    w = r.standard_normal((3, 2, 3, 3)).astype(np.float32)
    g = r.standard_normal((1, 3, 5, 5)).astype(np.float32)
    xt, wt = e.tensor(x, requires_grad=True), e.tensor(w, requires_grad=True)
    y = ops.conv2d(xt, wt, None, (1, 1), (1, 1))
    y.set_grad(e.tensor(g))
    y.backward()
    faithful = xt.grad.numpy()
    # restate the defect independently: column 0 = gradient of output pixel (0,0) only
    col0 = np.einsum("ockl,o->ckl", w.astype(np.float64), g[0, :, 0, 0].astype(np.float64))
    exp = np.zeros((2, 7, 7))
    for yo in range(5):
        for xo in range(5):
            exp[:, yo:yo + 3, xo:xo + 3] += col0
    assert_close(faithful[0], exp[:, 1:6, 1:6], 1e-4, "faithful dX")
    dx, dw, _ = ref_f64.conv2d_backward(x, w, g, (1, 1), (1, 1))
    assert_close(wt.grad.numpy(), dw, 1e-4, "dW is unaffected by the defect")
    assert np.max(np.abs(faithful - dx)) > 1e-2, "the defect is visible"


CONVT_CASES = [
    (2, 3, 4, 4, 2, 4, (2, 2), (1, 1)),
    (1, 2, 5, 3, 3, 3, (1, 1), (0, 0)),
    (1, 2, 3, 3, 2, 3, (2, 2), (0, 0)),
    (2, 1, 4, 4, 1, 2, (2, 2), (0, 0)),
]


@pytest.mark.parametrize("n,cin,h,w,cout,k,stride,pad", CONVT_CASES)
def test_conv2d_transpose_forward_backward(oracle_engine, n, cin, h, w, cout, k, stride, pad):
    e, ops = oracle_engine, oracle_engine.ops
    r = rng(3)
    x = r.standard_normal((n, cin, h, w)).astype(np.float32)
    wt = r.standard_normal((cin, cout, k, k)).astype(np.float32)
    b = r.standard_normal(cout).astype(np.float32)
    xt, wtt, bt = e.tensor(x, requires_grad=True), e.tensor(wt, requires_grad=True), e.tensor(b, requires_grad=True)
    y = ops.conv2d_transpose(xt, wtt, bt, stride, pad)
    yref = ref_f64.conv2d_transpose(x, wt, b, stride, pad)
    assert y.shape == yref.shape
    assert_close(y.numpy(), yref, 1e-4, "conv2d_transpose forward")
    g = r.standard_normal(yref.shape).astype(np.float32)
    y.set_grad(e.tensor(g))
    y.backward()
    dx, dw, db = ref_f64.conv2d_transpose_backward(x, wt, g, stride, pad)
    assert_close(xt.grad.numpy(), dx, 1e-4, "dX")
    assert_close(wtt.grad.numpy(), dw, 1e-4, "dW")
    assert_close(bt.grad.numpy(), db, 1e-4, "db")


@pytest.mark.parametrize("shape,k,s,p", [((2, 3, 8, 8), (2, 2), (2, 2), (0, 0)), ((1, 2, 7, 9), (3, 3), (2, 2), (1, 1)),
                                          ((1, 1, 5, 5), (3, 2), (1, 1), (0, 1))])
def test_max_pool2d_indices_and_backward(oracle_engine, shape, k, s, p):
    e, ops = oracle_engine, oracle_engine.ops
    r = rng(4)
    x = np.maximum(r.standard_normal(shape), 0).astype(np.float32)  # post-ReLU: many exact ties at 0
    xt = e.tensor(x, requires_grad=True)
    y = ops.max_pool2d(xt, k, s, p)
    yref, idx = ref_f64.max_pool2d(x, k, s, p)
    assert np.array_equal(y.numpy(), yref)
    g = r.standard_normal(yref.shape).astype(np.float32)
    y.set_grad(e.tensor(g))
    y.backward()
    exp = np.zeros(shape, dtype=np.float64)
    for yo in range(yref.shape[2]):
        for xo in range(yref.shape[3]):
            ky, kx = (idx[:, :, yo, xo] // k[1]).astype(int), (idx[:, :, yo, xo] % k[1]).astype(int)
            for n in range(shape[0]):
                for c in range(shape[1]):
                    iy, ix = yo * s[0] + ky[n, c] - p[0], xo * s[1] + kx[n, c] - p[1]
                    if 0 <= iy < shape[2] and 0 <= ix < shape[3]:
                        exp[n, c, iy, ix] += g[n, c, yo, xo]
    assert_close(xt.grad.numpy(), exp, 1e-6, "max_pool2d backward")
