"""Writes tests/golden/reference_known_answers.json.

Each case restates one known-answer test of the reference library: the literal inputs
of that test, the sequence of public-API calls it makes, and the values it asserts
(re-derived here from the formula the test states, in float64, and rounded to f32 the
way the test computes them).  The cases are small programs in a tiny step language so
that the same case can be replayed on the CPU oracle and on the CUDA backend:

  ["tensor", name, data, shape, requires_grad]
  ["op", out, opname, [inputs], int_params, float_params]     (see frontend.Engine.op)
  ["set_grad", name, data, shape]
  ["backward", name]
  ["op_backward", [outs], of_tensor, data, shape]             direct call of the op's backward
  ["optim", name, kind, [params], hyper] / ["step", name]
  ["expect", what, name, values, abs_tol]   what: value | grad | shape | grad_shape | state0 | state1
  ["expect_finite", "grad", name] / ["expect_sum_abs_lt", "grad", name, bound] / ["expect_posinf", "grad", name]

Run from the repository root:  python tests/golden/make_golden.py
"""
import json
import math
import os

import numpy as np

f32 = np.float32
cases = []


def case(name, cite, steps):
    cases.append({"name": name, "cite": cite, "steps": steps})


def T(name, data, shape, rg=True):
    return ["tensor", name, [float(v) for v in data], list(shape), bool(rg)]


def OP(out, op, ins, ip=(), fp=()):
    return ["op", out, op, list(ins), [int(v) for v in ip], [float(v) for v in fp]]


def EX(what, name, values, tol):
    return ["expect", what, name, [float(v) for v in np.asarray(values, dtype=np.float64).ravel()], float(tol)]


# --- tests/ops_cpu_tests.rs ----------------------------------------------------------------------
case("add_backward", "tests/ops_cpu_tests.rs:299-331", [
    T("a", [1, 2], [2]), T("b", [3, 4], [2]), OP("c", "add", ["a", "b"]), OP("loss", "mean", ["c"], [-1]),
    ["backward", "loss"], EX("grad", "a", [0.5, 0.5], 1e-6), EX("grad", "b", [0.5, 0.5], 1e-6),
    EX("grad_shape", "a", [2], 0)])
case("mul_backward", "tests/ops_cpu_tests.rs:334-365", [
    T("a", [1, 2], [2]), T("b", [3, 4], [2]), OP("c", "mul", ["a", "b"]), OP("loss", "mean", ["c"], [-1]),
    ["backward", "loss"], EX("grad", "a", [1.5, 2.0], 1e-6), EX("grad", "b", [0.5, 1.0], 1e-6)])
case("matmul_backward", "tests/ops_cpu_tests.rs:368-396", [
    T("a", [1, 2, 3, 4], [2, 2]), T("b", [5, 6, 7, 8], [2, 2]), OP("c", "matmul", ["a", "b"]),
    OP("loss", "mean", ["c"], [-1]), ["backward", "loss"],
    EX("grad", "a", [2.75, 3.75, 2.75, 3.75], 1e-6), EX("grad", "b", [1.0, 1.0, 1.5, 1.5], 1e-6),
    EX("grad_shape", "a", [2, 2], 0)])
case("mean_backward", "tests/ops_cpu_tests.rs:399-417", [
    T("a", [1, 2, 3, 4], [2, 2]), OP("loss", "mean", ["a"], [-1]), ["backward", "loss"],
    EX("grad", "a", [0.25] * 4, 1e-6)])
case("relu_backward", "tests/ops_cpu_tests.rs:420-439", [
    T("a", [-1, 0, 1, 2], [2, 2]), OP("r", "relu", ["a"]), OP("loss", "mean", ["r"], [-1]), ["backward", "loss"],
    EX("grad", "a", [0, 0, 0.25, 0.25], 1e-6)])
case("log_softmax_backward", "tests/ops_cpu_tests.rs:442-460", [
    T("a", [1, 2], [2]), OP("b", "log_softmax", ["a"], [0]), OP("loss", "mean", ["b"], [-1]), ["backward", "loss"],
    EX("grad", "a", [0.231049, -0.231049], 1e-5)])
case("grad_accumulation", "tests/ops_cpu_tests.rs:463-483", [
    T("a", [2.0], []), OP("b", "mul", ["a", "a"]), OP("c", "mul", ["a", "a"]), OP("loss", "add", ["b", "c"]),
    ["backward", "loss"], EX("grad", "a", [8.0], 1e-6), EX("grad", "b", [1.0], 1e-6), EX("grad", "c", [1.0], 1e-6),
    EX("grad_shape", "a", [], 0)])
case("broadcast_add_backward", "tests/ops_cpu_tests.rs:486-536", [
    T("a", [2.0], []), T("b", [1, 2, 3], [3]), OP("c", "add", ["a", "b"]), OP("loss", "mean", ["c"], [-1]),
    ["backward", "loss"], EX("grad", "a", [1.0], 1e-6), EX("grad", "b", [1 / 3] * 3, 1e-6),
    EX("grad_shape", "a", [], 0), EX("grad_shape", "b", [3], 0)])
case("broadcast_mul_backward", "tests/ops_cpu_tests.rs:539-589", [
    T("a", [2.0], []), T("b", [1, 2, 3], [3]), OP("c", "mul", ["a", "b"]), OP("loss", "mean", ["c"], [-1]),
    ["backward", "loss"], EX("grad", "a", [2.0], 1e-6), EX("grad", "b", [2 / 3] * 3, 1e-6),
    EX("grad_shape", "a", [], 0)])
case("reduction_backward_sum_axis0", "tests/ops_cpu_tests.rs:592-625", [
    T("a", [1, 2, 3, 4], [2, 2]), OP("s", "sum", ["a"], [0]), OP("loss", "mean", ["s"], [-1]), ["backward", "loss"],
    EX("grad", "a", [0.5] * 4, 1e-6), EX("grad_shape", "a", [2, 2], 0)])
case("reduction_backward_mean_axis1", "tests/ops_cpu_tests.rs:627-675", [
    T("a", [1, 2, 3, 4, 5, 6], [2, 3]), OP("m", "mean", ["a"], [1]), OP("loss", "mean", ["m"], [-1]),
    ["backward", "loss"], EX("grad", "a", [1 / 6] * 6, 1e-6), EX("grad_shape", "a", [2, 3], 0)])
case("numerical_stability_log_softmax", "tests/ops_cpu_tests.rs:678-697", [
    T("a", [1000.0, 1000.1, 1000.2], [3]), OP("b", "log_softmax", ["a"], [0]), OP("loss", "mean", ["b"], [-1]),
    ["backward", "loss"], ["expect_finite", "grad", "a"], ["expect_sum_abs_lt", "grad", "a", 1e-6],
    EX("grad_shape", "a", [3], 0)])
case("numerical_stability_ln_small", "tests/ops_cpu_tests.rs:699-711", [
    T("s", [1e-30], []), OP("l", "ln", ["s"]), OP("loss", "mean", ["l"], [-1]), ["backward", "loss"],
    ["expect_finite", "grad", "s"]])
case("numerical_stability_exp_large", "tests/ops_cpu_tests.rs:713-731", [
    T("x", [1e30], []), OP("e", "exp", ["x"]), OP("loss", "mean", ["e"], [-1]), ["backward", "loss"],
    ["expect_posinf", "grad", "x"]])
case("powf_gradient", "tests/ops_cpu_tests.rs:992-1093", [
    T("base", [2, 3, 4], [3]), T("exp", [3, 2, 0.5], [3]), OP("r", "powf", ["base", "exp"]),
    OP("loss", "mean", ["r"], [-1]), ["backward", "loss"],
    ["expect_prefix", "grad", "base", [4.0, 2.0], 1e-5],
    ["expect_prefix", "grad", "exp", [float(f32(8.0) * f32(math.log(2.0)) / f32(3.0)),
                                        float(f32(9.0) * f32(math.log(3.0)) / f32(3.0))], 1e-5]])
case("slice_backward_rows", "tests/ops_cpu_tests.rs:1492-1519", [
    T("x", [1, 2, 3, 4], [2, 2]), OP("s", "slice", ["x"], [0, 1, 0, 2]), EX("value", "s", [1, 2], 0),
    EX("shape", "s", [1, 2], 0), ["set_grad", "s", [10, 20], [1, 2]], ["backward", "s"],
    EX("grad", "x", [10, 20, 0, 0], 0), EX("grad_shape", "x", [2, 2], 0)])
case("slice_backward_cols", "tests/ops_cpu_tests.rs:1521-1543", [
    T("x", [1, 2, 3, 4], [2, 2]), OP("s", "slice", ["x"], [0, 2, 0, 1]), EX("value", "s", [1, 3], 0),
    EX("shape", "s", [2, 1], 0), ["set_grad", "s", [30, 40], [2, 1]], ["backward", "s"],
    EX("grad", "x", [30, 0, 40, 0], 0)])
case("clip_forward", "tests/ops_cpu_tests.rs:1549-1567", [
    T("a", [-1, 0.5, 2, 3], [2, 2], False), OP("c1", "clip", ["a"], (), [0.0, 2.0]), EX("value", "c1", [0, 0.5, 2, 2], 0),
    OP("c2", "clip", ["a"], (), [-0.5, 1.0]), EX("value", "c2", [-0.5, 0.5, 1, 1], 0),
    ["expect_error", "op", "clip", ["a"], [], [2.0, 1.0], "InvalidOperation"]])
case("clip_backward", "tests/ops_cpu_tests.rs:1570-1597", [
    T("x", [-1, 0.5, 2, 3], [2, 2]), OP("c", "clip", ["x"], (), [0.0, 2.0]), ["set_grad", "c", [1, 1, 1, 1], [2, 2]],
    ["backward", "c"], EX("grad", "x", [0, 1, 1, 0], 0), EX("grad_shape", "x", [2, 2], 0)])
# --- tests/ops_cpu_backward_tests.rs -----------------------------------------------------------
case("sum_backward_global", "tests/ops_cpu_backward_tests.rs:9-17", [
    T("x", [1, 2, 3, 4], [2, 2]), OP("y", "sum", ["x"], [-1]), ["backward", "y"], EX("grad", "x", [1, 1, 1, 1], 0)])
case("sum_backward_axis0", "tests/ops_cpu_backward_tests.rs:19-27", [
    T("x", [1, 2, 3, 4], [2, 2]), OP("y", "sum", ["x"], [0]), ["set_grad", "y", [1, 1], [2]], ["backward", "y"],
    EX("grad", "x", [1, 1, 1, 1], 0)])
case("sum_backward_axis1", "tests/ops_cpu_backward_tests.rs:29-37", [
    T("x", [1, 2, 3, 4], [2, 2]), OP("y", "sum", ["x"], [1]), ["set_grad", "y", [1, 1], [2]], ["backward", "y"],
    EX("grad", "x", [1, 1, 1, 1], 0)])
case("max_backward_global_with_ties", "tests/ops_cpu_backward_tests.rs:41-70", [
    T("x", [1, 5, 2, 5, 3, 0], [2, 3]), OP("m", "max", ["x"], [-1]), OP("loss", "mean", ["m"], [-1]),
    ["backward", "loss"], EX("grad", "x", [0, 0.5, 0, 0.5, 0, 0], 1e-6)])
case("min_backward_global_with_ties", "tests/ops_cpu_backward_tests.rs:73-113", [
    T("x", [1, 5, 2, 3, 1, 6], [2, 3]), OP("m", "min", ["x"], [-1]), OP("loss", "mean", ["m"], [-1]),
    ["backward", "loss"], EX("grad", "x", [0.5, 0, 0, 0, 0.5, 0], 1e-6)])
case("min_backward_direct_global", "tests/ops_cpu_backward_tests.rs:116-133", [
    T("x", [1, 2, 3, 4, 5, 6], [2, 3]), OP("m", "min", ["x"], [-1]), ["op_backward", ["gx"], "m", [1.0], [1]],
    EX("value", "gx", [1, 0, 0, 0, 0, 0], 0)])
case("min_backward_direct_axis0", "tests/ops_cpu_backward_tests.rs:135-146", [
    T("x", [1, 2, 3, 4, 5, 6], [2, 3]), OP("m", "min", ["x"], [0]), ["op_backward", ["gx"], "m", [1, 1, 1], [3]],
    EX("value", "gx", [1, 1, 1, 0, 0, 0], 0)])
case("prod_backward_direct", "tests/ops_cpu_backward_tests.rs:150-169", [
    T("x", [2, 3, 4], [3]), OP("p", "prod", ["x"], [-1]), ["op_backward", ["gx"], "p", [1.0], [1]],
    EX("value", "gx", [12, 8, 6], 1e-5)])
e = np.exp(np.array([1, 2, 3], dtype=np.float32)).astype(np.float32)
case("logsumexp_backward_direct", "tests/ops_cpu_backward_tests.rs:172-198", [
    T("x", [1, 2, 3], [3]), OP("l", "logsumexp", ["x"], [-1]), ["op_backward", ["gx"], "l", [1.0], [1]],
    EX("value", "gx", (e / e.sum(dtype=np.float32)).astype(np.float32), 1e-5)])
# --- tests/test_concat.rs, tests/test_expand_dims.rs ----------------------------------------
case("concat_backward_axis0", "tests/test_concat.rs:73-102", [
    T("a", [1, 2], [1, 2]), T("b", [3, 4], [1, 2]), OP("r", "concat", ["a", "b"], [0]), EX("shape", "r", [2, 2], 0),
    ["set_grad", "r", [10, 20, 30, 40], [2, 2]], ["backward", "r"], EX("grad", "a", [10, 20], 0),
    EX("grad", "b", [30, 40], 0), EX("grad_shape", "a", [1, 2], 0)])
case("concat_backward_axis1", "tests/test_concat.rs:104-134", [
    T("c", [1, 2], [2, 1]), T("d", [3, 4], [2, 1]), OP("r", "concat", ["c", "d"], [1]), EX("shape", "r", [2, 2], 0),
    EX("value", "r", [1, 3, 2, 4], 0), ["set_grad", "r", [10, 20, 30, 40], [2, 2]], ["backward", "r"],
    EX("grad", "c", [10, 30], 0), EX("grad", "d", [20, 40], 0), EX("grad_shape", "c", [2, 1], 0)])
case("expand_dims_backward_axis0", "tests/test_expand_dims.rs:76-96", [
    T("x", [1, 2, 3], [3]), OP("e", "expand_dims", ["x"], [0]), EX("shape", "e", [1, 3], 0),
    ["set_grad", "e", [10, 20, 30], [1, 3]], ["backward", "e"], EX("grad", "x", [10, 20, 30], 0),
    EX("grad_shape", "x", [3], 0)])
case("expand_dims_backward_middle", "tests/test_expand_dims.rs:119-138", [
    T("x", [1, 2, 3, 4], [2, 2]), OP("e", "expand_dims", ["x"], [1]), EX("shape", "e", [2, 1, 2], 0),
    ["set_grad", "e", [10, 20, 30, 40], [2, 1, 2]], ["backward", "e"], EX("grad", "x", [10, 20, 30, 40], 0),
    EX("grad_shape", "x", [2, 2], 0)])
# --- optimizers: tests/optim_tests.rs, src/optim.rs ------------------------------------------
p0 = np.array([1.0, 2.0], dtype=f32)
g = np.array([0.1, -0.2], dtype=f32)
lr, mu, b1, b2, eps = f32(0.1), f32(0.9), f32(0.9), f32(0.999), f32(1e-8)
vel = (mu * f32(0) + g).astype(f32)
case("momentum_sgd_one_step", "tests/optim_tests.rs:11-50; src/optim.rs:383-411", [
    T("p", p0, [2]), ["set_grad", "p", g, [2]], ["optim", "o", 2, ["p"], [float(lr), float(mu)]], ["step", "o"],
    EX("value", "p", (p0 - lr * vel).astype(f32), 1e-6), EX("state0", "o", vel, 1e-6)])
m = ((f32(1) - b1) * g).astype(f32)
v = ((f32(1) - b2) * (g * g)).astype(f32)
mh = (m / (f32(1) - b1)).astype(f32)
vh = (v / (f32(1) - b2)).astype(f32)
case("adam_one_step", "tests/optim_tests.rs:53-134", [
    T("p", p0, [2]), ["set_grad", "p", g, [2]], ["optim", "o", 1, ["p"], [float(lr), float(b1), float(b2), float(eps)]],
    ["step", "o"], EX("value", "p", (p0 - lr * mh / (np.sqrt(vh) + eps)).astype(f32), 1e-5), EX("state0", "o", m, 1e-5),
    EX("state1", "o", v, 1e-5)])
acc = (g * g).astype(f32)
case("adagrad_one_step", "tests/optim_tests.rs:321-366", [
    T("p", p0, [2]), ["set_grad", "p", g, [2]], ["optim", "o", 3, ["p"], [float(lr), float(eps)]], ["step", "o"],
    EX("value", "p", (p0 - lr * g / (np.sqrt(acc) + eps)).astype(f32), 1e-5), EX("state0", "o", acc, 1e-5)])
case("sgd_step", "src/optim.rs:452-480", [
    T("p", [1, 2, 3], [3]), ["set_grad", "p", [0.1, 0.2, 0.3], [3]], ["optim", "o", 0, ["p"], [0.1]], ["step", "o"],
    EX("value", "p", [1 - 0.1 * 0.1, 2 - 0.1 * 0.2, 3 - 0.1 * 0.3], 1e-6)])

def _plain(o):
    if isinstance(o, np.ndarray):
        return [float(v) for v in o.ravel()]
    if isinstance(o, (np.floating, np.integer)):
        return float(o)
    if isinstance(o, (list, tuple)):
        return [_plain(v) for v in o]
    if isinstance(o, dict):
        return {k: _plain(v) for k, v in o.items()}
    return o


cases = _plain(cases)
out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_known_answers.json")
with open(out, "w") as f:
    json.dump({"source": "known-answer tests of the reference library (file:line in each case)", "cases": cases}, f, indent=1)
print(f"wrote {len(cases)} cases to {out}")
