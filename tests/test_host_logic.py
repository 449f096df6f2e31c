"""CPU-only checks of the host side: the C-ABI library loads and exports every declared symbol,
the product refuses to run without a GPU (no fallback), host-side validation in the engine, and
the data-parallel gradient exchange semantics on two gloo ranks."""
import ctypes
import os
import subprocess
import sys

import numpy as np
import pytest

import rusttensor_b200
from rusttensor_b200.capi import declared_symbols

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    lib = rusttensor_b200.load_library()
    syms = declared_symbols()
    assert len(syms) >= 50
    missing = [s for s in syms if not hasattr(lib, s)]
    assert not missing, missing


def test_rust_binding_is_generated_from_the_current_header(tmp_path):
    """include/b200_backend.rs is what include/gen_rust_shim.py makes of include/rt_b200.h today: a changed header without a
    regenerated binding fails here."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("gen_rust_shim", os.path.join(ROOT, "include", "gen_rust_shim.py"))
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    fresh = gen.TEMPLATE.replace("@ENUMS@", gen.enum_consts()).replace("@FFI@", gen.ffi_block()).replace("@IMPL@", gen.impl_block())
    assert fresh == open(os.path.join(ROOT, "include", "b200_backend.rs")).read()
    names = [n for n, _, _ in gen.parse_header()]
    assert len(names) == len(set(names)) >= 99


def test_host_library_exports_engine_api():
    host = rusttensor_b200.load_host_library()
    for name in ("rth_init", "rth_op", "rth_backward", "rth_tensor_from_host", "rth_optim_step", "rth_trainer_run",
                 "rth_dp_create", "rth_dp_step_graph", "rth_dp_capture"):
        assert hasattr(host, name), name


def test_product_does_not_link_or_import_the_oracle():
    """The shipped libraries and package must not depend on oracle/ in any way."""
    for lib in (rusttensor_b200.LIB_PATH, rusttensor_b200.HOST_LIB_PATH):
        out = subprocess.run(["ldd", lib], capture_output=True, text=True).stdout
        assert "oracle" not in out
    pkg = os.path.join(ROOT, "rusttensor_b200")
    for dirpath, _, files in os.walk(pkg):
        if "build" in dirpath:
            continue
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".hpp", ".cpp", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "import oracle" not in text and "oracle/" not in text and "cpu_backend.hpp" not in text, f


@pytest.mark.skipif(rusttensor_b200.load_library().rt_device_count() > 0, reason="a GPU is present")
def test_fails_loudly_without_a_gpu():
    code = ("import rusttensor_b200\n"
            "try:\n    rusttensor_b200.engine()\nexcept rusttensor_b200.BackendUnavailable as e:\n    print('UNAVAILABLE', e)\n")
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=ROOT)
    assert "UNAVAILABLE" in out.stdout and "no CPU fallback" in out.stdout, out.stdout + out.stderr
    lib = rusttensor_b200.load_library()
    ctx = ctypes.c_void_p()
    assert lib.rt_ctx_create(0, ctypes.byref(ctx)) == 7  # RT_ERR_CUDA
    assert not ctx.value


def test_engine_host_side_validation(oracle_engine):
    """Shape bookkeeping and error kinds of the generic engine (shared by both backends)."""
    from rusttensor_b200.frontend import EngineError

    e, ops = oracle_engine, oracle_engine.ops
    a = e.tensor(np.zeros((2, 3)), requires_grad=True)
    with pytest.raises(EngineError) as ei:
        ops.matmul(a, e.tensor(np.zeros((2, 3))))
    assert ei.value.kind == "IncompatibleShapes"
    with pytest.raises(EngineError) as ei:
        ops.view(a, (4, 2))
    assert ei.value.kind == "IncompatibleShapes"
    with pytest.raises(EngineError) as ei:
        ops.slice(a, [(0, 3), (0, 3)])
    assert ei.value.kind == "InvalidIndex"
    with pytest.raises(EngineError) as ei:
        ops.div_scalar(a, 2.0)  # backward not implemented in the reference (src/ops/mod.rs:786-790)
    assert ei.value.kind == "InvalidOperation"
    with pytest.raises(EngineError) as ei:
        ops.sum(a, 0).backward()  # non-scalar root without a seed gradient (src/tensor.rs:1163-1170)
    assert ei.value.kind == "InvalidOperation"
    with pytest.raises(EngineError) as ei:
        a.set_grad(e.tensor(np.zeros((3, 2))))  # the reference panics here (src/tensor.rs:1029-1036)
    assert ei.value.kind == "ShapeMismatch"
    s = ops.sum(a, None)
    assert s.shape == ()
    assert ops.argmax(e.tensor([1.0, 3.0, 2.0]), 0).shape == ()


def test_optimizers_skip_parameters_without_gradient(oracle_engine):
    e = oracle_engine
    p, q = e.tensor([1.0, 2.0], requires_grad=True), e.tensor([3.0], requires_grad=True)
    p.set_grad(e.tensor([1.0, 1.0]))
    opt = e.Sgd([p, q], 0.5)
    opt.step()
    assert np.allclose(p.numpy(), [0.5, 1.5]) and np.allclose(q.numpy(), [3.0])
    opt.zero_grad()
    assert p.grad is None


_WORKER = r"""
import os, sys, json
import numpy as np
import torch, torch.distributed as dist
sys.path.insert(0, os.environ["RT_ROOT"]); sys.path.insert(0, os.path.join(os.environ["RT_ROOT"], "tests"))
import oracle
from helpers import setup_trainer, workload_data
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:" + os.environ["RT_PORT"], rank=rank, world_size=world)
e = oracle.engine()
dims = [6, 12, 8, 4]
params, inputs = workload_data(1, dims, seed=0, rank=rank)
tr = setup_trainer(e, 1, dims, params)
tr.forward_backward([e.tensor(a) for a in inputs])
flat = torch.from_numpy(np.concatenate([p.grad.numpy().ravel() for p in tr.params]))
dist.all_reduce(flat)                      # one all-reduce over the flat gradient buffer
flat /= world                              # the 1/world the fused optimizer folds in
gathered = [torch.zeros_like(torch.from_numpy(a)) for _ in range(world) for a in [inputs[0]]]
xs = [torch.zeros(inputs[0].shape) for _ in range(world)]; ys = [torch.zeros(inputs[1].shape) for _ in range(world)]
dist.all_gather(xs, torch.from_numpy(inputs[0])); dist.all_gather(ys, torch.from_numpy(inputs[1]))
if rank == 0:
    big = [world * dims[0]] + dims[1:]
    tr2 = setup_trainer(e, 1, big, params)
    tr2.forward_backward([e.tensor(torch.cat(xs).numpy()), e.tensor(torch.cat(ys).numpy())])
    ref = np.concatenate([p.grad.numpy().ravel() for p in tr2.params])
    err = float(np.max(np.abs(ref - flat.numpy())))
    print("RESULT", json.dumps({"err": err, "scale": float(np.max(np.abs(ref)))}))
dist.barrier(); dist.destroy_process_group()
"""


def test_data_parallel_gradient_mean_equals_global_batch_on_two_gloo_ranks(tmp_path):
    """Averaging per-rank gradients of per-rank mean losses == the gradient of the mean loss over the
    global batch: the contract of the data-parallel step (world_size 2, gloo, CPU oracle)."""
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    port = str(29500 + os.getpid() % 2000)
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", RT_ROOT=ROOT, RT_PORT=port, MASTER_ADDR="127.0.0.1")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = [p.communicate(timeout=240) for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    line = [l for l in outs[0][0].splitlines() if l.startswith("RESULT")][0]
    import json

    res = json.loads(line.split(" ", 1)[1])
    assert res["err"] <= 1e-5 * max(res["scale"], 1.0), res
