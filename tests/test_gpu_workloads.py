"""The five benchmark workloads: CUDA backend vs CPU oracle on the same seeded inputs.
Gradients, updated parameters and optimizer state within 1e-4 (max-abs-rel with the documented
floor for near-zero sums)."""
import numpy as np
import pytest

import oracle
import rusttensor_b200
from helpers import assert_close, setup_trainer, workload_data

pytestmark = pytest.mark.gpu
TOL = 1e-4

SMALL = {
    1: [8, 20, 16, 5],
    2: [64, 48],
    3: [4, 8, 4, 6, 16, 5],
    4: [2, 3, 8, 5],
    5: [11, 8, 4, 3],
}
FULL = {1: [64, 784, 128, 10], 2: [4096, 4096], 3: [256, 28, 32, 64, 128, 10], 4: [8, 64, 56, 128], 5: [65, 512, 128, 64]}


def run_reference_step(engine, config, dims, params, inputs, steps=1, conv_dx_correct=False, variant=0):
    # variant 100: the same network built from the fused forward ops (ops::fused_*)
    tr = setup_trainer(engine, config + variant, dims, params)
    ins = [engine.tensor(a, requires_grad=(config == 4 and i == 0)) for i, a in enumerate(inputs)]
    losses = []
    if conv_dx_correct:
        oracle.set_conv_dx_faithful(False)
    try:
        for _ in range(steps):
            loss = tr.step(ins) if config != 2 else tr.forward_backward(ins)
            losses.append(float(loss.numpy()))
    finally:
        oracle.set_conv_dx_faithful(True)
    grads = [p.grad.numpy() for p in tr.params]
    vals = [p.numpy() for p in tr.params]
    extra = [ins[0].grad.numpy()] if config == 4 else []
    states = []
    if config in (1, 3, 5):
        states = [tr.optim_state(0, i).numpy() for i in range(len(tr.params))] + [tr.optim_state(1, i).numpy() for i in range(len(tr.params))]
    elif config == 4:
        states = [tr.optim_state(0, i).numpy() for i in range(len(tr.params))]
    return dict(loss=losses, grads=grads, params=vals, extra=extra, states=states)


LR = {1: 1e-3, 3: 1e-3, 4: 1e-2, 5: 1e-3, 2: 0.0}


def compare_runs(cpu, gpu, what, tol=TOL, lr=0.0):
    assert_close(np.array(gpu["loss"]), np.array(cpu["loss"]), tol, f"{what} loss")
    for k in ("grads", "params", "extra", "states"):
        assert len(cpu[k]) == len(gpu[k])
        for i, (a, b) in enumerate(zip(cpu[k], gpu[k])):
            # updated parameters: an extra 5e-4 of one step for elements whose gradient is a
            # near-zero sum (see helpers.assert_close)
            assert_close(b, a, tol, f"{what} {k}[{i}]", abs_floor=5e-4 * lr if k == "params" else 0.0)


@pytest.mark.parametrize("config", [1, 2, 3, 4, 5])
def test_small_workload_matches_oracle(oracle_engine, gpu_engine, contraction_path, config):
    dims = SMALL[config]
    params, inputs = workload_data(config, dims, seed=0)
    # conv input gradients: the CUDA kernels are mathematically correct, so configs whose
    # parameter gradients sit downstream of a conv dX (3: conv1 behind conv2's dX; 4: dX itself)
    # are compared with the oracle's corrected mode.
    correct = config in (3, 4)
    cpu = run_reference_step(oracle_engine, config, dims, params, inputs, steps=2, conv_dx_correct=correct)
    gpu = run_reference_step(gpu_engine, config, dims, params, inputs, steps=2)
    compare_runs(cpu, gpu, f"C{config} small", lr=LR[config])


def test_c3_reference_defect_is_confined(oracle_engine, gpu_engine):
    """With the reference's conv dX defect reproduced (faithful mode) everything NOT downstream of
    a conv input gradient still matches the CUDA path: conv2 / fc gradients of C3."""
    dims = SMALL[3]
    params, inputs = workload_data(3, dims, seed=1)
    cpu = run_reference_step(oracle_engine, 3, dims, params, inputs, steps=1, conv_dx_correct=False)
    gpu = run_reference_step(gpu_engine, 3, dims, params, inputs, steps=1)
    for i in range(2, 8):  # conv2_w, conv2_b, fc1_w, fc1_b, fc2_w, fc2_b
        assert_close(gpu["grads"][i], cpu["grads"][i], TOL, f"C3 faithful grads[{i}]")
    gap = np.max(np.abs(gpu["grads"][0] - cpu["grads"][0]))
    print(f"conv1_w gradient gap caused by the reference defect: {gap:.3e}")


def adam_first_step_bound(p_ref, g_ref, lr=1e-3, eps=1e-8, tol=TOL):
    """Tolerance for a parameter after the FIRST Adam step, obtained by pushing the gradient tolerance
    through the update.  At t=1, m_hat = g and v_hat = g^2, so p' = p - lr*g/(|g|+eps); its derivative
    w.r.t. g is lr*eps/(|g|+eps)^2.  A gradient may differ by dg = tol*|g| + 1e-6*max|g| (the bound the
    gradient comparison itself uses), hence |dp'| <= tol*|p'| + lr*eps*dg/(|g|+eps)^2.  The second term
    only matters for elements whose gradient is a near-zero sum (|g| ~ eps), where Adam's normalisation
    turns rounding noise into a visible fraction of one step."""
    g = np.abs(np.asarray(g_ref, dtype=np.float64))
    dg = tol * g + 1e-6 * float(g.max() if g.size else 0.0)
    return tol * np.abs(np.asarray(p_ref, dtype=np.float64)) + lr * eps * dg / (g + eps) ** 2 + 1e-9


_FULL_ORACLE = {}


def full_size_oracle(oracle_engine, config):
    """One oracle pass per configuration and test session (C2 takes ~5 s, C5 ~8 s, C4 at batch 8 ~5 s on one host thread)."""
    if config not in _FULL_ORACLE:
        dims = FULL[config]
        params, inputs = workload_data(config, dims, seed=2)
        _FULL_ORACLE[config] = (params, inputs, run_reference_step(oracle_engine, config, dims, params, inputs, steps=1,
                                                                   conv_dx_correct=config in (3, 4)))
    return _FULL_ORACLE[config]


@pytest.mark.parametrize("config", [1, 2, 3, 4, 5])
def test_full_size_workload_matches_oracle(oracle_engine, gpu_engine, contraction_path, config):
    """The benchmark configurations at the sizes they are quoted on, on both contraction paths.  C4 keeps its full channel
    counts and 56x56 images (the shapes that select the large-channel kernels: 128-column tiles, the four stride phases of
    the transposed convolution, the 2048-step split-K chains) but runs at batch 8 instead of 128: the oracle's
    transposed convolution is the reference's 7-deep scalar loop nest and takes minutes at batch 128."""
    dims = FULL[config]
    params, inputs, cpu = full_size_oracle(oracle_engine, config)
    gpu = run_reference_step(gpu_engine, config, dims, params, inputs, steps=1)
    assert_close(np.array(gpu["loss"]), np.array(cpu["loss"]), TOL, "loss")
    for k in ("grads", "states", "extra"):
        assert len(cpu[k]) == len(gpu[k])
        for i, (a, b) in enumerate(zip(cpu[k], gpu[k])):
            assert_close(b, a, TOL, f"C{config} full {k}[{i}]")
    for i, (a, b) in enumerate(zip(cpu["params"], gpu["params"])):
        if config in (1, 3, 5):  # Adam
            bound = adam_first_step_bound(a, cpu["grads"][i])
            bad = np.abs(b.astype(np.float64) - a) > bound
            assert not bad.any(), f"C{config} full params[{i}]: {int(bad.sum())} elements outside the propagated Adam bound, worst {np.max(np.abs(b - a)[bad]):.3e}"
        else:  # momentum SGD is linear in the gradient (C4); C2 has no optimizer
            assert_close(b, a, TOL, f"C{config} full params[{i}]", abs_floor=5e-4 * LR[config])


@pytest.mark.parametrize("config", [1, 3, 4, 5])
def test_fused_trainer_eager_and_graph_match_per_tensor_path(gpu_engine, config):
    """DataParallelTrainer (fused multi-tensor optimizer, CUDA-graph replay) == the per-tensor API."""
    dims = SMALL[config]
    params, inputs = workload_data(config, dims, seed=3)
    ref = run_reference_step(gpu_engine, config, dims, params, inputs, steps=3)
    for mode in ("eager", "graph"):
        tr = rusttensor_b200.DataParallelTrainer(config, dims)
        for t, p in zip(tr.params, params):
            t.update_from_host(p)
        losses = []
        for _ in range(3):
            if mode == "eager":
                losses.append(tr.step_eager(inputs))
            else:
                tr.step(inputs)
                losses.append(tr.last_loss())
        if mode == "graph":
            assert tr.graph_nodes() > 0
        assert_close(np.array(losses), np.array(ref["loss"]), 1e-5, f"C{config} {mode} losses")
        for i, p in enumerate(tr.params):
            assert_close(p.numpy(), ref["params"][i], 1e-5, f"C{config} {mode} params[{i}]")
        n = len(tr.params)
        for i in range(n):
            assert_close(tr.state(0, i).numpy(), ref["states"][i], 1e-5, f"C{config} {mode} state0[{i}]")


def test_graph_replay_is_deterministic_and_uses_fresh_inputs(gpu_engine):
    dims = SMALL[3]
    params, in_a = workload_data(3, dims, seed=4)
    _, in_b = workload_data(3, dims, seed=5)
    runs = []
    for _ in range(2):
        tr = rusttensor_b200.DataParallelTrainer(3, dims)
        for t, p in zip(tr.params, params):
            t.update_from_host(p)
        out = []
        for ins in (in_a, in_b, in_a):
            tr.step(ins)
            out.append(tr.last_loss())
        runs.append((out, [p.numpy() for p in tr.params]))
    assert runs[0][0] == runs[1][0]
    assert runs[0][0][0] != runs[0][0][1]
    for a, b in zip(runs[0][1], runs[1][1]):
        assert np.array_equal(a, b)


def test_pipelined_steps_equal_plain_steps(gpu_engine):
    """step_pipelined (double-buffered upload on a copy stream, loss read one step late) computes exactly what
    step() + last_loss() computes, also when the host runs several steps ahead of the device."""
    dims = SMALL[3]
    params, in_a = workload_data(3, dims, seed=6)
    _, in_b = workload_data(3, dims, seed=7)
    _, in_c = workload_data(3, dims, seed=8)
    sequence = [in_a, in_b, in_c, in_a, in_b]

    def fresh():
        tr = rusttensor_b200.DataParallelTrainer(3, dims)
        for t, p in zip(tr.params, params):
            t.update_from_host(p)
        return tr

    plain = fresh()
    ref = []
    for ins in sequence:
        plain.step(ins)
        ref.append(plain.last_loss())
    piped = fresh()
    got = []
    for ins in sequence:
        for i, a in enumerate(ins):
            piped.pipeline_buffer(i)[...] = a
        prev = piped.step_pipelined()
        if prev is not None:
            got.append(prev)
    got.append(piped.pipeline_flush())
    assert got == ref
    for a, b in zip(plain.params, piped.params):
        assert np.array_equal(a.numpy(), b.numpy())


@pytest.mark.parametrize("config", [1, 3, 4, 5])
def test_fused_forward_ops_match_the_reference_chain(oracle_engine, gpu_engine, config):
    """Configuration 100 + c builds network c from the fused forward ops (relu + max_pool2d in one kernel, the
    classification loss in one kernel).  It must match the oracle running the reference's own chain of ops, to the
    same tolerance as the unfused CUDA path, and max-pool routing must stay identical."""
    dims = SMALL[config]
    params, inputs = workload_data(config, dims, seed=9)
    cpu = run_reference_step(oracle_engine, config, dims, params, inputs, steps=2, conv_dx_correct=config in (3, 4))
    gpu = run_reference_step(gpu_engine, config, dims, params, inputs, steps=2, variant=100)
    compare_runs(cpu, gpu, f"C{config} fused forward", lr=LR[config])


def test_fused_forward_full_size_cnn(oracle_engine, gpu_engine):
    dims = FULL[3]
    params, inputs = workload_data(3, dims, seed=2)
    cpu = run_reference_step(oracle_engine, 3, dims, params, inputs, steps=1, conv_dx_correct=True)
    gpu = run_reference_step(gpu_engine, 3, dims, params, inputs, steps=1, variant=100)
    assert_close(np.array(gpu["loss"]), np.array(cpu["loss"]), TOL, "loss")
    for k in ("grads", "states"):
        for i, (a, b) in enumerate(zip(cpu[k], gpu[k])):
            assert_close(b, a, TOL, f"C3 fused full {k}[{i}]")
