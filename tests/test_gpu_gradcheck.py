"""The reference's finite-difference acceptance list for a CUDA backend
(tests/test_gradient_checker_cuda.rs:25-718): same inputs, same epsilon, same tolerance,
same comparator (src/test_utils.rs:17-265), run on the new backend."""
import numpy as np
import pytest

from helpers import max_abs_rel

pytestmark = pytest.mark.gpu

EPS, TOL = 1e-4, 2e-2


def check_gradient(engine, func, arrays, requires, idx, epsilon, tolerance):
    """src/test_utils.rs:17-61: analytical gradient through backward() vs central differences."""
    tensors = [engine.tensor(a, requires_grad=r) for a, r in zip(arrays, requires)]
    loss = func(engine.ops, tensors)
    assert int(np.prod(loss.shape, dtype=np.int64)) == 1
    loss.backward()
    g = tensors[idx].grad
    analytical = np.zeros(max(arrays[idx].size, 1), np.float32) if g is None else g.numpy().ravel()
    numerical = np.zeros_like(analytical)
    base = np.asarray(arrays[idx], dtype=np.float32)
    for i in range(analytical.size):
        vals = []
        for sign in (+1, -1):
            d = base.copy().ravel()
            d[i] = np.float32(d[i] + np.float32(sign * epsilon))
            ts = [engine.tensor(d.reshape(base.shape) if j == idx else a, requires_grad=r) for j, (a, r) in enumerate(zip(arrays, requires))]
            vals.append(np.float32(func(engine.ops, ts).numpy().ravel()[0]))
        numerical[i] = np.float32(vals[0] - vals[1]) / np.float32(2.0 * epsilon)
    err = max_abs_rel(analytical, numerical)
    assert err <= tolerance, f"analytical {analytical} vs numerical {numerical}: max rel err {err:.3e} > {tolerance}"


A = lambda v, s=None: np.array(v, dtype=np.float32).reshape(s if s is not None else (len(v),))
mean = lambda ops, t: ops.mean(t, None)
pool_in = A([(x % 10) / 10.0 for x in range(1, 37)], (1, 1, 6, 6))

# name, cite, func, arrays, requires_grad, indices to check, epsilon, tolerance
CASES = [
    ("mse_loss", ":25", lambda o, t: o.mse_loss(t[0], t[1], "mean"), [A([1, 2, 3]), A([1.5, 2.5, 3.5])], [True, False], [0], EPS, TOL),
    ("abs", ":43", lambda o, t: mean(o, o.abs(t[0])), [A([-3.0, -0.001, 0.001, 2.0, 4.0])], [True], [0], EPS, TOL),
    ("mul", ":62", lambda o, t: mean(o, o.mul(t[0], t[1])), [A([1, -2]), A([3, 4])], [True, True], [0, 1], EPS, TOL),
    ("exp", ":84", lambda o, t: mean(o, o.exp(t[0])), [A([-1.0, 0.0, 1.0, 1.5])], [True], [0], EPS, 3e-2),
    ("ln", ":102", lambda o, t: mean(o, o.ln(t[0])), [A([0.1, 0.5, 1.0, 2.0, 10.0])], [True], [0], EPS, 3e-2),
    ("add", ":122", lambda o, t: mean(o, o.add(t[0], t[1])), [A([1, 2, -3]), A([4, -5, 6])], [True, True], [0, 1], EPS, TOL),
    ("matmul", ":148", lambda o, t: mean(o, o.matmul(t[0], t[1])), [A([1, 2, 3, 4], (2, 2)), A([5, 6, 7, 8], (2, 2))], [True, True], [0, 1], EPS, 2e-2),
    ("relu", ":182", lambda o, t: mean(o, o.relu(t[0])), [A([-2.0, -0.001, 0.001, 3.0])], [True], [0], EPS, TOL),
    ("sigmoid", ":201", lambda o, t: mean(o, o.sigmoid(t[0])), [A([-2.0, 0.0, 1.5, 3.0])], [True], [0], EPS, 3e-2),
    ("mean_global", ":220", lambda o, t: o.mean(t[0], None), [A([1, 2, 3, 4, 5, 6], (2, 3))], [True], [0], EPS, 3e-2),
    ("mean_axis", ":236", lambda o, t: mean(o, o.mean(t[0], 0)), [A([1, 2, 3, 4, 5, 6], (2, 3))], [True], [0], EPS, TOL),
    ("mean_axis1", ":236", lambda o, t: mean(o, o.mean(t[0], 1)), [A([1, 2, 3, 4, 5, 6], (2, 3))], [True], [0], EPS, TOL),
    ("sum_global", ":255", lambda o, t: o.sum(t[0], None), [A([1, -2, 3, -4], (2, 2))], [True], [0], EPS, TOL),
    ("sum_axis", ":271", lambda o, t: mean(o, o.sum(t[0], 1)), [A([1, 2, 3, 4, 5, 6], (2, 3))], [True], [0], EPS, 3e-2),
    ("log_softmax", ":290", lambda o, t: mean(o, o.log_softmax(t[0], 1)), [A([1.0, 2.0, 1.5, 0.5], (2, 2))], [True], [0], EPS, 2e-2),
    ("max_global", ":314", lambda o, t: o.max(t[0], None), [A([1.0, 5.0, 2.0, 4.99, 3.0, 0.0], (2, 3))], [True], [0], EPS, 3e-2),
    ("max_axis", ":338", lambda o, t: mean(o, o.max(t[0], 1)), [A([1.0, 5.0, 2.0, 5.01, 3.0, 6.0], (2, 3))], [True], [0], EPS, 3e-2),
    ("min_global", ":364", lambda o, t: mean(o, o.min(t[0], None)), [A([1, 2, 3, 4], (2, 2))], [True], [0], 1e-3, 1e-3),
    ("min_axis", ":378", lambda o, t: mean(o, o.min(t[0], 0)), [A([1, 2, 3, 4], (2, 2))], [True], [0], 1e-3, 1e-3),
    ("prod_global", ":392", lambda o, t: mean(o, o.prod(t[0], None)), [A([2.0, 3.0, 2.5, 3.5], (2, 2))], [True], [0], 1e-3, 5e-2),
    ("prod_axis", ":408", lambda o, t: mean(o, o.prod(t[0], 0)), [A([2.0, 3.0, 2.5, 3.5], (2, 2))], [True], [0], 1e-3, 5e-2),
    ("logsumexp_global", ":422", lambda o, t: mean(o, o.logsumexp(t[0], None)), [A([1, 2, 3, 4], (2, 2))], [True], [0], 1e-3, 5e-2),
    ("logsumexp_axis", ":445", lambda o, t: mean(o, o.logsumexp(t[0], 0)), [A([1, 2, 3, 4], (2, 2))], [True], [0], 1e-3, 5e-2),
    ("div", ":464", lambda o, t: mean(o, o.div(t[0], t[1])), [A([1, 4, 9]), A([2, 2, 3])], [True, True], [0, 1], EPS, 3e-2),
    ("sub", ":488", lambda o, t: mean(o, o.sub(t[0], t[1])), [A([5, 4]), A([1, 2])], [True, True], [0, 1], EPS, TOL),
    ("tanh", ":510", lambda o, t: mean(o, o.tanh(t[0])), [A([-1.0, 0.0, 1.0])], [True], [0], 1e-4, 1e-3),
    ("softplus", ":526", lambda o, t: mean(o, o.softplus(t[0])), [A([-2.0, 0.0, 1.0, 3.0])], [True], [0], EPS, 3e-2),
    ("bce_with_logits", ":543", lambda o, t: o.binary_cross_entropy_with_logits(t[0], t[1], "mean"), [A([-1.0, 0.5, 2.0]), A([0.0, 1.0, 1.0])], [True, False], [0], EPS, TOL),
    ("powf", ":567", lambda o, t: mean(o, o.powf(t[0], t[1])), [A([1, 2, 3]), A([2, 3, 0.5])], [True, True], [0, 1], EPS, 1e-2),
    ("square", ":595", lambda o, t: mean(o, o.square(t[0])), [A([-2.0, 0.5, 3.0])], [True], [0], EPS, TOL),
    ("maximum", ":615", lambda o, t: mean(o, o.maximum(t[0], t[1])), [A([1, 4, 2]), A([3, 2, 1])], [True, True], [0, 1], EPS, 3e-2),
    ("sqrt", ":638", lambda o, t: mean(o, o.sqrt(t[0])), [A([0.1, 0.5, 1.0, 4.0, 9.0])], [True], [0], EPS, 3e-2),
    ("elu", ":658", lambda o, t: mean(o, o.elu(t[0], 1.0)), [A([-2.0, -0.5, 0.0, 0.5, 2.0])], [True], [0], EPS, 3e-2),
    ("softmax_cross_entropy", ":678", lambda o, t: o.softmax_cross_entropy(t[0], t[1], 1, "mean"),
     [A([0.5, 1.5, -1.0, 2.0, 0.0, -0.5], (2, 3)), A([0.0, 1.0, 0.0, 0.3, 0.7, 0.0], (2, 3))], [True, False], [0], EPS, 3e-2),
    ("max_pool2d", ":699", lambda o, t: mean(o, o.max_pool2d(t[0], (2, 2), (2, 2), (0, 0))), [pool_in], [True], [0], 1e-2, 5e-2),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: c[0])
def test_gradient_checker_case(gpu_engine, case):
    name, cite, func, arrays, requires, indices, eps, tol = case
    for idx in indices:
        check_gradient(gpu_engine, func, arrays, requires, idx, eps, tol)


def test_gradient_checker_cases_pass_on_the_oracle_too(oracle_engine):
    """Same list on the CPU oracle (what tests/test_gradient_checker.rs does for the CPU backend)."""
    for name, cite, func, arrays, requires, indices, eps, tol in CASES:
        for idx in indices:
            check_gradient(oracle_engine, func, arrays, requires, idx, eps, tol)


# extra finite-difference checks for the contractions the reference leaves unpinned
def test_conv_and_conv_transpose_gradients_by_finite_differences(gpu_engine):
    r = np.random.default_rng(7)
    x = r.standard_normal((1, 2, 5, 5)).astype(np.float32)
    w = r.standard_normal((3, 2, 3, 3)).astype(np.float32)
    b = r.standard_normal(3).astype(np.float32)
    f = lambda o, t: o.mean(o.square(o.conv2d(t[0], t[1], t[2], (1, 1), (1, 1))), None)
    for idx in (0, 1, 2):
        check_gradient(gpu_engine, f, [x, w, b], [True, True, True], idx, 1e-2, 5e-2)
    wt = r.standard_normal((2, 3, 4, 4)).astype(np.float32)
    f2 = lambda o, t: o.mean(o.square(o.conv2d_transpose(t[0], t[1], t[2], (2, 2), (1, 1))), None)
    x2 = r.standard_normal((1, 2, 3, 3)).astype(np.float32)
    for idx in (0, 1, 2):
        check_gradient(gpu_engine, f2, [x2, wt, b], [True, True, True], idx, 1e-2, 5e-2)
