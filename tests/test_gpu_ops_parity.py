"""Differential tests: the same graph on the CPU oracle and on the CUDA backend from the same
host data, compared with the reference's tolerance (TOLERANCE = 1e-4,
tests/ops_cuda_backward_tests.rs:41-70), on odd shapes, broadcast shapes, 0-D and empty tensors."""
import numpy as np
import pytest

from helpers import assert_close, rng
from rusttensor_b200.frontend import EngineError

pytestmark = pytest.mark.gpu

TOL = 1e-4
SHAPES = [(), (1,), (7,), (5, 3), (4, 128), (33, 257), (2, 3, 5, 7), (0,), (3, 0, 2), (1031,), (256, 1024)]


def both(oracle_engine, gpu_engine, build, arrays, requires_grad=None, seed_grad=None):
    """Runs build(engine, tensors) on both engines; returns [(values, grads...)] per engine."""
    outs = []
    for e in (oracle_engine, gpu_engine):
        ts = [e.tensor(a, requires_grad=(True if requires_grad is None else requires_grad[i])) for i, a in enumerate(arrays)]
        y = build(e, ts)
        res = {"y": y.numpy(), "shape": y.shape}
        if y.requires_grad:
            if seed_grad is not None:
                y.set_grad(e.tensor(seed_grad(y.shape)))
            elif len(y.shape) != 0:  # only a 0-D root is seeded implicitly (src/tensor.rs:1157-1170)
                g = rng(77).standard_normal(y.shape).astype(np.float32)
                y.set_grad(e.tensor(g, y.shape))
            y.backward()
            res["grads"] = [None if t.grad is None else (t.grad.numpy(), t.grad.shape) for t in ts]
        outs.append(res)
    return outs


def compare(outs, what, tol=TOL):
    o, g = outs
    assert o["shape"] == g["shape"], f"{what}: shape {g['shape']} vs oracle {o['shape']}"
    assert_close(g["y"], o["y"], tol, f"{what} forward")
    if "grads" in o:
        for i, (a, b) in enumerate(zip(o["grads"], g["grads"])):
            assert (a is None) == (b is None), f"{what}: grad {i} presence"
            if a is not None:
                assert a[1] == b[1], f"{what}: grad {i} shape {b[1]} vs {a[1]}"
                assert_close(b[0], a[0], tol, f"{what} grad {i}")


UNARY = {
    "relu": (lambda r, s: r.standard_normal(s), ()),
    "sigmoid": (lambda r, s: r.standard_normal(s) * 3, ()),
    "abs": (lambda r, s: r.standard_normal(s), ()),
    "exp": (lambda r, s: r.standard_normal(s), ()),
    "ln": (lambda r, s: r.uniform(0.1, 4, s), ()),
    "sqrt": (lambda r, s: r.uniform(0.1, 4, s), ()),
    "tanh": (lambda r, s: r.standard_normal(s) * 2, ()),
    "softplus": (lambda r, s: r.standard_normal(s) * 3, ()),
    "square": (lambda r, s: r.standard_normal(s), ()),
    "sin": (lambda r, s: r.standard_normal(s) * 3, ()),
}


@pytest.mark.parametrize("shape", SHAPES, ids=str)
@pytest.mark.parametrize("op", sorted(UNARY))
def test_unary_forward_backward(oracle_engine, gpu_engine, op, shape):
    x = UNARY[op][0](rng(hash(op) % 1000), shape).astype(np.float32)
    if op == "relu" and x.size:
        x.flat[0] = 0.0  # the mask is strict: x > 0
    compare(both(oracle_engine, gpu_engine, lambda e, t: getattr(e.ops, op)(t[0]), [x]), f"{op}{shape}")


@pytest.mark.parametrize("shape", [(7,), (33, 257), (0,)], ids=str)
def test_parametrised_unary(oracle_engine, gpu_engine, shape):
    x = rng(5).standard_normal(shape).astype(np.float32) * 2
    compare(both(oracle_engine, gpu_engine, lambda e, t: e.ops.elu(t[0], 0.7), [x]), "elu")
    compare(both(oracle_engine, gpu_engine, lambda e, t: e.ops.clip(t[0], -0.5, 1.0), [x]), "clip")
    compare(both(oracle_engine, gpu_engine, lambda e, t: e.ops.mul_scalar(t[0], -1.5), [x]), "mul_scalar")
    compare(both(oracle_engine, gpu_engine, lambda e, t: e.ops.div_scalar(t[0], 3.0), [x], requires_grad=[False]), "div_scalar")
    if x.size:  # a [1]-shaped exponent cannot broadcast against an empty base (see the next test)
        compare(both(oracle_engine, gpu_engine, lambda e, t: e.ops.powf_scalar(e.ops.abs(t[0]), 2.5), [x + 3.0]), "powf_scalar")


def test_extent_zero_against_extent_one(oracle_engine, gpu_engine):
    """add/mul/powf: an extent 0 cannot pair with an extent 1 (the reference takes max(0,1)=1 and then
    fails to stretch the empty operand); sub/div go through ndarray's operators, where it can."""
    for e in (oracle_engine, gpu_engine):
        a, b = e.tensor(np.zeros((0,), np.float32)), e.tensor(np.ones((1,), np.float32))
        for op in ("add", "mul", "powf", "maximum"):
            with pytest.raises(EngineError) as ei:
                getattr(e.ops, op)(a, b)
            assert ei.value.kind == "IncompatibleShapes"
        assert e.ops.sub(a, b).shape == (0,)
        assert e.ops.div(a, b).shape == (0,)


BROADCAST_PAIRS = [((5, 3), (5, 3)), ((4, 128), (128,)), ((33, 257), (257,)), ((128,), (4, 128)), ((6, 5), ()), ((), (6, 5)),
                   ((3, 1), (1, 4)), ((2, 3, 4), (3, 1)), ((2, 1, 4), (5, 1)), ((7,), (1,)), ((4, 4, 8), (4, 1, 8)),
                   ((512, 256), (256,)), ((0, 3), (1, 3)), ((2, 3, 4, 5), (4, 5))]


@pytest.mark.parametrize("sa,sb", BROADCAST_PAIRS, ids=str)
@pytest.mark.parametrize("op", ["add", "sub", "mul", "div", "maximum", "minimum", "powf"])
def test_binary_broadcast_forward_backward(oracle_engine, gpu_engine, op, sa, sb):
    r = rng(11)
    a = r.standard_normal(sa).astype(np.float32)
    b = r.standard_normal(sb).astype(np.float32)
    if op == "div":
        b = (np.sign(b) * (np.abs(b) + 0.5)).astype(np.float32)
    if op == "powf":
        a = (np.abs(a) + 0.5).astype(np.float32)
    if 0 in sa + sb and op != "sub":
        # outside sub/div an extent 0 cannot meet an extent 1 (test_extent_zero_against_extent_one);
        # div's backward multiplies through `mul`, so it fails the same way in the reference.
        pytest.skip("extent 0 against extent 1 is only defined for sub")
    compare(both(oracle_engine, gpu_engine, lambda e, t: getattr(e.ops, op)(t[0], t[1]), [a, b]), f"{op}{sa}{sb}")


def test_binary_incompatible_shapes_error(gpu_engine):
    a, b = gpu_engine.tensor(np.zeros((2, 3))), gpu_engine.tensor(np.zeros((4,)))
    for op in ("add", "mul", "powf", "maximum"):
        with pytest.raises(EngineError) as ei:
            getattr(gpu_engine.ops, op)(a, b)
        assert ei.value.kind == "IncompatibleShapes"


def test_comparisons_and_ties(oracle_engine, gpu_engine):
    a = np.array([[1, 2, 3], [4, 5, 6]], np.float32)
    b = np.array([1, 5, 3], np.float32)
    # maximum / minimum route a tie to the first operand (src/backend/cpu.rs:1921-1927, 2049-2056)
    compare(both(oracle_engine, gpu_engine, lambda e, t: e.ops.maximum(t[0], t[1]), [a, b]), "maximum ties")
    compare(both(oracle_engine, gpu_engine, lambda e, t: e.ops.minimum(t[0], t[1]), [a, b]), "minimum ties")


COMPARISONS = ["equal", "not_equal", "greater", "greater_equal", "less", "less_equal"]


@pytest.mark.parametrize("sa,sb", [((5, 3), (5, 3)), ((33, 257), (257,)), ((6, 5), ()), ((3, 1), (1, 4)), ((2, 3, 4, 5), (4, 5)),
                                   ((1031,), (1031,)), ((256, 1024), (1024,)), ((0, 3), (0, 3))], ids=str)
@pytest.mark.parametrize("op", COMPARISONS)
def test_comparisons_forward(oracle_engine, gpu_engine, op, sa, sb):
    """1.0 / 0.0 outputs, bit-exact against the oracle (src/backend/cpu.rs:684-898): equal / not_equal use |a-b| < 1e-9,
    the ordered comparisons are exact.  Inputs are rounded so that many elements tie; the results carry no gradient."""
    r = rng(41)
    a = np.round(r.standard_normal(sa) * 2).astype(np.float32)
    b = np.round(r.standard_normal(sb) * 2).astype(np.float32)
    if a.size:
        a.flat[0] = np.float32(b.flat[0] if b.size else 0.0) + np.float32(1e-10)  # inside the 1e-9 band after fp32 rounding
    res = []
    for e in (oracle_engine, gpu_engine):
        y = getattr(e.ops, op)(e.tensor(a, requires_grad=True), e.tensor(b, requires_grad=True))
        assert not y.requires_grad
        res.append((y.shape, y.numpy()))
    assert res[0][0] == res[1][0]
    assert np.array_equal(res[0][1], res[1][1]), op
    want = {"equal": np.abs(a - b) < 1e-9, "not_equal": np.abs(a - b) >= 1e-9, "greater": a > b, "greater_equal": a >= b,
            "less": a < b, "less_equal": a <= b}[op]
    assert np.array_equal(res[1][1], np.broadcast_to(want, res[1][0]).astype(np.float32))


@pytest.mark.parametrize("shape", SHAPES, ids=str)
@pytest.mark.parametrize("op", ["cos", "tan"])
def test_backend_cos_tan_forward_backward(oracle_engine, gpu_engine, op, shape):
    """Backend::cos / tan and cos_backward / tan_backward (src/backend/cpu.rs:2118-2202) against the oracle and against
    float64 numpy; tan's inputs stay away from its poles."""
    r = rng(43)
    x = (r.uniform(-1.3, 1.3, shape) if op == "tan" else r.standard_normal(shape) * 3).astype(np.float32)
    g = r.standard_normal(shape).astype(np.float32)
    out = []
    for e in (oracle_engine, gpu_engine):
        xt, gt = e.tensor(x), e.tensor(g)
        y = getattr(e.ops, f"backend_{op}")(xt)
        dx = getattr(e.ops, f"backend_{op}_backward")(xt, gt)
        assert y.shape == tuple(shape) and dx.shape == tuple(shape)
        out.append((y.numpy(), dx.numpy()))
    assert_close(out[1][0], out[0][0], TOL, f"{op}{shape} forward")
    assert_close(out[1][1], out[0][1], TOL, f"{op}{shape} backward")
    x64 = x.astype(np.float64)
    if op == "cos":
        assert_close(out[1][0], np.cos(x64), TOL, "cos vs float64")
        assert_close(out[1][1], -np.sin(x64) * g, TOL, "cos_backward vs float64")
    else:
        assert_close(out[1][0], np.tan(x64), TOL, "tan vs float64")
        assert_close(out[1][1], g / np.cos(x64) ** 2, TOL, "tan_backward vs float64")


RED_SHAPES = [((5,), 0), ((5, 3), 0), ((5, 3), 1), ((2, 3, 4), 1), ((64, 10), 1), ((256, 65), 1), ((3, 4099), 1), ((4099, 3), 0),
              ((300, 2000), 0), ((2, 5000, 3), 1), ((1, 1), 1), ((7, 1), 0), ((2, 3, 4, 5), 2)]


@pytest.mark.parametrize("shape,axis", RED_SHAPES, ids=str)
@pytest.mark.parametrize("op", ["sum", "mean", "max", "min", "logsumexp", "prod"])
def test_axis_reductions_forward_backward(oracle_engine, gpu_engine, op, shape, axis):
    r = rng(21)
    x = r.standard_normal(shape).astype(np.float32)
    if op == "prod":
        x = (1.0 + 0.05 * x).astype(np.float32)
    compare(both(oracle_engine, gpu_engine, lambda e, t: getattr(e.ops, op)(t[0], axis), [x]), f"{op}{shape}@{axis}", 2e-4 if op == "prod" else TOL)


@pytest.mark.parametrize("shape", [(), (1,), (37,), (5, 3), (1000003,), (129, 1025)], ids=str)
@pytest.mark.parametrize("op", ["sum", "mean", "max", "min", "logsumexp"])
def test_global_reductions_forward_backward(oracle_engine, gpu_engine, op, shape):
    x = rng(22).standard_normal(shape).astype(np.float32)
    compare(both(oracle_engine, gpu_engine, lambda e, t: getattr(e.ops, op)(t[0], None), [x]), f"{op}{shape}")


def test_max_min_ties_split_evenly(oracle_engine, gpu_engine):
    x = np.array([[1, 5, 5], [2, 2, 2], [0, -1, 0]], np.float32)
    for op in ("max", "min"):
        for axis in (None, 0, 1):
            compare(both(oracle_engine, gpu_engine, lambda e, t: getattr(e.ops, op)(t[0], axis), [x]), f"{op} ties axis={axis}")


@pytest.mark.parametrize("shape,axis", [((2,), 0), ((64, 10), 1), ((256, 65), 1), ((3, 5, 4), 1), ((5, 3000), 1), ((16, 4096), 1), ((10, 64), 0)], ids=str)
def test_log_softmax_forward_backward(oracle_engine, gpu_engine, shape, axis):
    x = (rng(23).standard_normal(shape) * 3).astype(np.float32)
    compare(both(oracle_engine, gpu_engine, lambda e, t: e.ops.log_softmax(t[0], axis), [x]), f"log_softmax{shape}@{axis}")


def test_argmax_argmin_bit_exact(oracle_engine, gpu_engine):
    x = np.round(rng(24).standard_normal((17, 33)) * 2).astype(np.float32)  # many ties
    for op in ("argmax", "argmin"):
        for axis in (0, 1):
            o = getattr(oracle_engine.ops, op)(oracle_engine.tensor(x), axis).numpy()
            g = getattr(gpu_engine.ops, op)(gpu_engine.tensor(x), axis).numpy()
            assert np.array_equal(o, g), (op, axis)


def test_layout_ops(oracle_engine, gpu_engine):
    x = rng(25).standard_normal((6, 10)).astype(np.float32)
    compare(both(oracle_engine, gpu_engine, lambda e, t: e.ops.transpose(t[0]), [x]), "transpose")
    compare(both(oracle_engine, gpu_engine, lambda e, t: e.ops.slice(t[0], [(1, 4), (2, 9)]), [x]), "slice")
    compare(both(oracle_engine, gpu_engine, lambda e, t: e.ops.view(t[0], (3, 20)), [x]), "view")
    compare(both(oracle_engine, gpu_engine, lambda e, t: e.ops.expand_dims(t[0], 1), [x]), "expand_dims")
    compare(both(oracle_engine, gpu_engine, lambda e, t: e.ops.squeeze(e.ops.expand_dims(t[0], 0), 0), [x]), "squeeze")
    b = rng(26).standard_normal((10,)).astype(np.float32)
    compare(both(oracle_engine, gpu_engine, lambda e, t: e.ops.broadcast_to(t[0], (6, 10)), [b]), "broadcast_to")
    y = rng(27).standard_normal((6, 3)).astype(np.float32)
    compare(both(oracle_engine, gpu_engine, lambda e, t: e.ops.concat([t[0], t[1]], 1), [x, y]), "concat axis1")
    z = rng(28).standard_normal((2, 10)).astype(np.float32)
    compare(both(oracle_engine, gpu_engine, lambda e, t: e.ops.concat([t[0], t[1]], 0), [x, z]), "concat axis0")


def test_composite_losses(oracle_engine, gpu_engine):
    r = rng(29)
    p, t = r.standard_normal((6, 4)).astype(np.float32), r.standard_normal((6, 4)).astype(np.float32)
    rg = [True, False]
    compare(both(oracle_engine, gpu_engine, lambda e, ts: e.ops.mse_loss(ts[0], ts[1], "mean"), [p, t], rg), "mse_loss")
    y = (r.uniform(0, 1, (6, 4)) > 0.5).astype(np.float32)
    compare(both(oracle_engine, gpu_engine, lambda e, ts: e.ops.binary_cross_entropy_with_logits(ts[0], ts[1], "mean"), [p, y], rg), "bce")
    oh = np.eye(4, dtype=np.float32)[r.integers(0, 4, 6)]
    for red in ("mean", "sum", "none"):
        compare(both(oracle_engine, gpu_engine, lambda e, ts: e.ops.softmax_cross_entropy(ts[0], ts[1], 1, red), [p, oh], rg), f"sce {red}")


def test_grad_accumulation_fan_in(oracle_engine, gpu_engine):
    x = rng(30).standard_normal((9, 5)).astype(np.float32)

    def build(e, t):
        a = e.ops.square(t[0])
        b = e.ops.add(a, e.ops.mul_scalar(a, -0.5))
        c = e.ops.add(e.ops.sin(t[0]), b)
        return e.ops.sum(e.ops.mul(c, t[0]), None)

    compare(both(oracle_engine, gpu_engine, build, [x]), "fan-in accumulation")


def test_optimizers_multi_step(oracle_engine, gpu_engine):
    r = rng(31)
    p0 = r.standard_normal((37, 5)).astype(np.float32)
    grads = [r.standard_normal((37, 5)).astype(np.float32) for _ in range(4)]
    for name, args in (("Sgd", (0.1,)), ("Adam", (1e-2, 0.9, 0.999, 1e-8)), ("MomentumSGD", (1e-2, 0.9)), ("AdaGrad", (0.1, 1e-8))):
        res = []
        for e in (oracle_engine, gpu_engine):
            p = e.tensor(p0, requires_grad=True)
            opt = getattr(e, name)([p], *args)
            for g in grads:
                p.set_grad(e.tensor(g))
                opt.step()
            st = [] if name == "Sgd" else [opt.state(0, 0).numpy()] + ([opt.state(1, 0).numpy()] if name == "Adam" else [])
            res.append((p.numpy(), st))
        assert_close(res[1][0], res[0][0], TOL, f"{name} params after 4 steps")
        for a, b in zip(res[0][1], res[1][1]):
            assert_close(b, a, TOL, f"{name} state")
