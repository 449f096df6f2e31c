"""Checkpoint files: the reference's serde_json tensor layout (src/tensor.rs:38-47, 130-165, 444-502) written and read bit
for bit; CPU-only tests run against the oracle engine, the resume-parity test on the CUDA trainer."""
import json

import numpy as np
import pytest

import rusttensor_b200
from helpers import workload_data
from rusttensor_b200 import checkpoint


def bits(a):
    return np.asarray(a, dtype=np.float32).view(np.uint32)


def test_tensor_record_has_the_reference_layout_and_round_trips_bitwise():
    r = np.random.default_rng(0)
    a = (r.standard_normal((3, 5, 7)) * 10.0 ** r.integers(-30, 30, (3, 5, 7))).astype(np.float32)
    a.flat[:6] = [0.0, -0.0, np.finfo(np.float32).max, np.finfo(np.float32).tiny, 1e-45, -1.17549435e-38]
    g = r.standard_normal((3, 5, 7)).astype(np.float32)
    rec = checkpoint.tensor_record(a, g, True, device=0)
    assert list(rec) == ["data", "shape", "grad", "requires_grad", "device"]          # field order of SerializableTensor
    assert rec["shape"] == [3, 5, 7] and rec["requires_grad"] is True and rec["device"] == {"Cuda": 0}
    assert checkpoint.tensor_record(a)["device"] == "Cpu" and checkpoint.tensor_record(a)["grad"] is None
    data, grad, rg = checkpoint.record_arrays(json.loads(json.dumps(rec)))
    assert np.array_equal(bits(data), bits(a)) and np.array_equal(bits(grad), bits(g)) and rg


def test_reads_a_file_as_serde_json_writes_it():
    """Shortest-form floats, `null` gradient, unit-variant device: what serde_json emits for SerializableTensor."""
    text = '{"data":[1.0,-2.5,0.1,3e-7,16777216.0,1e10],"shape":[2,3],"grad":null,"requires_grad":true,"device":"Cpu"}'
    data, grad, rg = checkpoint.record_arrays(json.loads(text))
    assert data.shape == (2, 3) and grad is None and rg
    assert np.array_equal(data, np.array([[1.0, -2.5, 0.1], [3e-7, 16777216.0, 1e10]], np.float32))
    with pytest.raises(ValueError):
        checkpoint.record_arrays(json.loads('{"data":[1.0,2.0],"shape":[3],"grad":null,"requires_grad":false,"device":"Cpu"}'))


def test_non_finite_values_become_null():
    rec = checkpoint.tensor_record(np.array([1.0, np.nan, np.inf, -np.inf], np.float32))
    assert rec["data"] == [1.0, None, None, None]
    json.dumps(rec, allow_nan=False)  # valid JSON
    assert np.isnan(checkpoint.record_arrays(rec)[0][1:]).all()


def test_save_and_load_tensor_on_the_oracle_engine(oracle_engine, tmp_path):
    e = oracle_engine
    x = e.tensor(np.arange(6, dtype=np.float32).reshape(2, 3) / 7, requires_grad=True)
    e.ops.sum(e.ops.square(x), None).backward()
    path = tmp_path / "tensor.json"
    checkpoint.save_tensor(x, path, device=None)
    doc = json.loads(path.read_text())
    assert doc["device"] == "Cpu" and doc["shape"] == [2, 3] and len(doc["grad"]) == 6
    y = checkpoint.load_tensor(e, path)
    assert y.shape == (2, 3) and y.requires_grad
    assert np.array_equal(bits(y.numpy()), bits(x.numpy())) and np.array_equal(bits(y.grad.numpy()), bits(x.grad.numpy()))


@pytest.mark.gpu
@pytest.mark.parametrize("config", [3, 4])
def test_resume_is_bit_identical(gpu_engine, tmp_path, config):
    """k steps in one run == j steps, save, load into a fresh trainer, k - j steps (parameters, optimizer state, step counter)."""
    dims = {3: [4, 8, 4, 6, 16, 5], 4: [2, 3, 8, 5]}[config]
    params, _ = workload_data(config, dims, seed=0)
    batches = [workload_data(config, dims, seed=10 + s)[1] for s in range(5)]

    def fresh():
        tr = rusttensor_b200.DataParallelTrainer(config, dims)
        for t, p in zip(tr.params, params):
            t.update_from_host(p)
        return tr

    def run(tr, steps):
        out = []
        for b in steps:
            tr.step(b)
            out.append(tr.last_loss())
        return out

    whole = fresh()
    ref_losses = run(whole, batches)
    first = fresh()
    losses = run(first, batches[:2])
    path = tmp_path / "ckpt.json"
    checkpoint.save_checkpoint(first, path)
    doc = json.loads(path.read_text())
    assert doc["t"] == 2 and doc["format"] == checkpoint.FORMAT and len(doc["params"]) == len(first.params)
    assert doc["params"][0]["device"] == {"Cuda": 0} and doc["params"][0]["shape"] == list(first.params[0].shape)
    second = fresh()
    checkpoint.load_checkpoint(second, path)
    assert second.step_count == 2
    losses += run(second, batches[2:])
    assert losses == ref_losses
    n = len(whole.params)
    for i in range(n):
        assert np.array_equal(bits(second.params[i].numpy()), bits(whole.params[i].numpy())), f"parameter {i}"
        assert np.array_equal(bits(second.state(0, i).numpy()), bits(whole.state(0, i).numpy())), f"state {i}"
        if whole.optimizer_kind == 1:
            assert np.array_equal(bits(second.state(1, i).numpy()), bits(whole.state(1, i).numpy())), f"second moment {i}"


@pytest.mark.gpu
def test_checkpoint_of_another_workload_is_refused(gpu_engine, tmp_path):
    a = rusttensor_b200.DataParallelTrainer(3, [4, 8, 4, 6, 16, 5])
    b = rusttensor_b200.DataParallelTrainer(1, [8, 20, 16, 5])
    c = rusttensor_b200.DataParallelTrainer(4, [2, 3, 8, 5])
    path = tmp_path / "ckpt.json"
    checkpoint.save_checkpoint(a, path)
    with pytest.raises(ValueError):
        checkpoint.load_checkpoint(b, path)   # other tensors
    with pytest.raises(ValueError):
        checkpoint.load_checkpoint(c, path)   # other optimizer


@pytest.mark.gpu
def test_graph_is_recaptured_when_a_view_moves_an_input(gpu_engine):
    """A view of an input shares its buffer; the next upload then gives the input a buffer of its own (copy on write).  The
    captured graph would keep reading the old one: the trainer notices the moved pointer and captures again."""
    dims = [4, 8, 4, 6, 16, 5]
    params, in_a = workload_data(3, dims, seed=0)
    _, in_b = workload_data(3, dims, seed=1)

    def fresh():
        tr = rusttensor_b200.DataParallelTrainer(3, dims)
        for t, p in zip(tr.params, params):
            t.update_from_host(p)
        return tr

    plain = fresh()
    ref = []
    for ins in (in_a, in_b, in_a):
        plain.step(ins)
        ref.append(plain.last_loss())
    tr = fresh()
    tr.step(in_a)
    got = [tr.last_loss()]
    alias = gpu_engine.ops.view(tr.inputs[0], (dims[0], dims[1] * dims[1]))  # keeps the input's buffer shared
    for ins in (in_b, in_a):
        tr.step(ins)
        got.append(tr.last_loss())
    assert got == ref
    assert alias.shape == (dims[0], dims[1] * dims[1])
    for a, b in zip(plain.params, tr.params):
        assert np.array_equal(a.numpy(), b.numpy())
