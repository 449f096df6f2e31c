"""Shared test utilities: the golden-program interpreter, comparison metrics and seeded inputs."""
import json
import os

import numpy as np

from rusttensor_b200.frontend import EngineError

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_known_answers.json")


def load_cases():
    with open(GOLDEN) as f:
        return json.load(f)["cases"]


def max_abs_rel(a, b):
    """The reference's own comparator (src/test_utils.rs:239-245): per element
    |a-b| / max(|a|,|b|) when both magnitudes exceed 1e-8, else |a-b|; the maximum."""
    a = np.asarray(a, dtype=np.float64).ravel()
    b = np.asarray(b, dtype=np.float64).ravel()
    assert a.shape == b.shape, (a.shape, b.shape)
    if a.size == 0:
        return 0.0
    err = np.abs(a - b)
    both = (np.abs(a) > 1e-8) & (np.abs(b) > 1e-8)
    den = np.maximum(np.abs(a), np.abs(b))
    rel = np.where(both, err / np.where(den == 0, 1, den), err)
    rel = np.where(np.isnan(a) & np.isnan(b), 0.0, rel)
    rel = np.where((a == b), 0.0, rel)  # equal infinities
    return float(np.max(rel))


def assert_close(got, ref, tol=1e-4, what="", abs_floor=0.0):
    """max-abs-rel <= tol, or, for the near-zero outputs of long zero-mean sums whose relative
    error is unbounded for any summation order, |a-b| <= tol*max(|a|,|b|) + 1e-6*max|ref| + abs_floor.

    abs_floor is used only for parameters after an Adam step: Adam divides by sqrt(v)+eps, so for an
    element whose gradient is a near-zero sum (|g| comparable to eps) the rounding noise the gradient
    check itself allows becomes a change of up to noise/|g| of a full step lr; callers pass a few
    1e-4 * lr."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    if got.size == 0:
        return
    m = max_abs_rel(got, ref)
    if m <= tol:
        return
    scale = float(np.max(np.abs(ref[np.isfinite(ref)]))) if np.isfinite(ref).any() else 0.0
    bound = tol * np.maximum(np.abs(got), np.abs(ref)) + 1e-6 * scale + abs_floor
    bad = ~(np.abs(got - ref) <= bound) & ~((got == ref) | (np.isnan(got) & np.isnan(ref)))
    assert not bad.any(), (f"{what}: max-abs-rel {m:.3e} > {tol}; {int(bad.sum())} of {got.size} elements outside the "
                           f"mixed bound, worst |d|={np.max(np.abs(got - ref)[bad]):.3e} (ref scale {scale:.3e})")


def run_case(engine, case):
    """Replays one golden program on `engine`; returns the dict of named tensors / optimizers."""
    env = {}
    for st in case["steps"]:
        kind = st[0]
        if kind == "tensor":
            _, name, data, shape, rg = st
            env[name] = engine.tensor(np.array(data, dtype=np.float32), shape, rg)
        elif kind == "op":
            _, out, op, ins, ip, fp = st
            env[out] = engine.op(op, [env[i] for i in ins], ip, fp)
        elif kind == "set_grad":
            _, name, data, shape = st
            env[name].set_grad(engine.tensor(np.array(data, dtype=np.float32), shape))
        elif kind == "backward":
            env[st[1]].backward()
        elif kind == "op_backward":
            _, outs, of, data, shape = st
            grads = engine.op_backward(env[of], engine.tensor(np.array(data, dtype=np.float32), shape))
            for n, g in zip(outs, grads):
                env[n] = g
        elif kind == "optim":
            _, name, k, params, hyper = st
            ctor = [engine.Sgd, engine.Adam, engine.MomentumSGD, engine.AdaGrad][k]
            env[name] = ctor([env[p] for p in params], *hyper)
        elif kind == "step":
            env[st[1]].step()
        elif kind == "expect":
            _, what, name, values, tol = st
            if what == "value":
                got = env[name].numpy().ravel()
            elif what == "grad":
                g = env[name].grad
                assert g is not None, f"{case['name']}: {name} has no gradient"
                got = g.numpy().ravel()
            elif what == "shape":
                got = np.array(env[name].shape, dtype=np.float64)
            elif what == "grad_shape":
                got = np.array(env[name].grad.shape, dtype=np.float64)
            elif what in ("state0", "state1"):
                got = env[name].state(0 if what == "state0" else 1, 0).numpy().ravel()
            else:
                raise ValueError(what)
            exp = np.array(values, dtype=np.float64)
            assert got.shape == exp.shape, f"{case['name']}: {what} {name}: {got.shape} vs {exp.shape}"
            if got.size:
                assert np.max(np.abs(got - exp)) <= tol + 1e-12, f"{case['name']} ({case['cite']}): {what} {name}: got {got}, expected {exp}"
        elif kind == "expect_prefix":
            _, what, name, values, tol = st
            got = env[name].grad.numpy().ravel()[: len(values)]
            assert np.max(np.abs(got - np.array(values))) <= tol, f"{case['name']}: {name}: {got} vs {values}"
        elif kind == "expect_finite":
            assert np.all(np.isfinite(env[st[2]].grad.numpy())), case["name"]
        elif kind == "expect_sum_abs_lt":
            assert abs(float(env[st[2]].grad.numpy().sum())) < st[3], case["name"]
        elif kind == "expect_posinf":
            g = env[st[2]].grad.numpy().ravel()
            assert np.all(np.isposinf(g)), f"{case['name']}: {g}"
        elif kind == "expect_error":
            _, _, op, ins, ip, fp, err = st
            try:
                engine.op(op, [env[i] for i in ins], ip, fp)
            except EngineError as e:
                assert e.kind == err, f"{case['name']}: error kind {e.kind}, expected {err}"
            else:
                raise AssertionError(f"{case['name']}: {op} should fail with {err}")
        else:
            raise ValueError(kind)
    return env


from rusttensor_b200.workloads import kaiming_uniform, one_hot, rng, setup_trainer, workload_data  # noqa: E402,F401
