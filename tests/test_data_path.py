"""src/data.rs: load_csv (CPU tests, on the oracle engine) and get_random_batch (oracle on CPU, device gather on the GPU)."""
import numpy as np
import pytest

from rusttensor_b200 import data
from rusttensor_b200.frontend import EngineError


def write(tmp_path, text):
    p = tmp_path / "d.csv"
    p.write_text(text)
    return str(p)


def test_load_csv_normalises_and_one_hot_encodes(oracle_engine, tmp_path):
    x, y = data.load_csv(oracle_engine, write(tmp_path, "3,0,255,51\n0,102,0,255\n9,1,2,3\n"))
    assert x.shape == (3, 3) and y.shape == (3, 10) and not x.requires_grad and not y.requires_grad
    assert np.array_equal(x.numpy(), (np.array([[0, 255, 51], [102, 0, 255], [1, 2, 3]], np.float32) / np.float32(255)))
    want = np.zeros((3, 10), np.float32)
    want[[0, 1, 2], [3, 0, 9]] = 1
    assert np.array_equal(y.numpy(), want)


def test_load_csv_empty_file(oracle_engine, tmp_path):
    x, y = data.load_csv(oracle_engine, write(tmp_path, ""))
    assert x.shape == (0, 0) and y.shape == (0, 10)


@pytest.mark.parametrize("text,fragment", [
    ("x,1,2\n", "Invalid label format at row 0"),
    ("10,1,2\n", "Invalid label value at row 0"),
    ("-1,1,2\n", "Invalid label value"),
    ("2.5,1,2\n", "Invalid label value"),
    ("1,1,abc\n", "Invalid feature format at row 0, column 2"),
    ("1\n", "Row with label but no features"),
    ("1,2,3\n2,4\n", "Inconsistent number of features at row 1. Expected 2, found 1"),
])
def test_load_csv_errors(oracle_engine, tmp_path, text, fragment):
    with pytest.raises(EngineError) as ei:
        data.load_csv(oracle_engine, write(tmp_path, text))
    assert ei.value.kind == "InvalidOperation" and fragment in str(ei.value)


def test_load_csv_missing_file(oracle_engine, tmp_path):
    with pytest.raises(EngineError) as ei:
        data.load_csv(oracle_engine, str(tmp_path / "nope.csv"))
    assert ei.value.kind == "CsvError"


def _dataset(n=37, f=12, c=10, seed=0):
    r = np.random.default_rng(seed)
    x = r.standard_normal((n, f)).astype(np.float32)
    y = np.eye(c, dtype=np.float32)[r.integers(0, c, n)]
    return x, y


def check_batches(e):
    x, y = _dataset()
    xt, yt = e.tensor(x), e.tensor(y)
    bx, by = e.get_batch(xt, yt, [5, 0, 36, 5])
    assert bx.shape == (4, 12) and by.shape == (4, 10) and not bx.requires_grad
    assert np.array_equal(bx.numpy(), x[[5, 0, 36, 5]]) and np.array_equal(by.numpy(), y[[5, 0, 36, 5]])
    rx, ry = e.get_random_batch(xt, yt, 16, seed=3)
    assert rx.shape == (16, 12) and ry.shape == (16, 10)
    # every sampled row is a row of the data set, rows are distinct (sampling without replacement), x and y stay paired
    rows = [int(np.flatnonzero((x == r).all(axis=1))[0]) for r in rx.numpy()]
    assert len(set(rows)) == 16 and np.array_equal(ry.numpy(), y[rows])
    rx2, _ = e.get_random_batch(xt, yt, 16, seed=3)
    assert np.array_equal(rx.numpy(), rx2.numpy())                       # seeded
    full, _ = e.get_random_batch(xt, yt, 37, seed=1)
    assert sorted(map(tuple, full.numpy())) == sorted(map(tuple, x))     # a permutation of the whole set
    # 1-D tensors: one feature per row (src/data.rs:162-163)
    v = e.tensor(np.arange(37, dtype=np.float32))
    b1, _ = e.get_batch(v, yt, [3, 4])
    assert b1.shape == (2, 1) and np.array_equal(b1.numpy().ravel(), [3, 4])
    # the reference's checks, in its order (src/data.rs:133-157)
    for call, kind in ((lambda: e.get_random_batch(e.tensor(np.zeros((0, 3), np.float32)), yt, 1), "EmptyTensor"),
                       (lambda: e.get_random_batch(xt, e.tensor(np.zeros((36, 10), np.float32)), 4), "ShapeMismatch"),
                       (lambda: e.get_random_batch(xt, yt, 38), "DimensionMismatch"),
                       (lambda: e.get_batch(xt, yt, [37]), None)):
        with pytest.raises(EngineError) as ei:
            call()
        if kind:
            assert ei.value.kind == kind


def test_random_batches_on_the_oracle(oracle_engine):
    check_batches(oracle_engine)


@pytest.mark.gpu
def test_random_batches_gathered_on_the_device(gpu_engine):
    check_batches(gpu_engine)


@pytest.mark.gpu
def test_gather_rows_through_the_c_abi(capi):
    import ctypes as C

    r = np.random.default_rng(1)
    for rows, row_len in ((100, 784), (33, 7), (5, 1), (64, 12)):
        src = r.standard_normal((rows, row_len)).astype(np.float32)
        idx = r.integers(0, rows, 41).astype(np.int32)
        d_src = capi.to_device(src)
        d_idx = capi.to_device(idx.view(np.float32))  # 4-byte integers through the float upload helper
        out = capi.empty((41, row_len))
        capi.call("gather_rows", d_src.ptr, C.c_int64(rows), C.c_int64(row_len), d_idx.ptr, C.c_int64(41), out.ptr)
        assert np.array_equal(out.numpy(), src[idx])


@pytest.mark.gpu
def test_steps_from_a_device_resident_data_set_equal_host_batches(gpu_engine):
    """step_dataset(indices) == step(host batch of the same rows): same losses, same parameters, bit for bit."""
    import rusttensor_b200
    from helpers import workload_data

    dims = [4, 8, 4, 6, 16, 5]
    params, _ = workload_data(3, dims, seed=0)
    r = np.random.default_rng(2)
    X = r.uniform(0, 1, (50, 1, 8, 8)).astype(np.float32)
    Y = np.eye(5, dtype=np.float32)[r.integers(0, 5, 50)]
    batches = [r.choice(50, 4, replace=False) for _ in range(5)]

    def fresh():
        tr = rusttensor_b200.DataParallelTrainer(3, dims)
        for t, p in zip(tr.params, params):
            t.update_from_host(p)
        return tr

    host = fresh()
    ref = []
    for b in batches:
        host.step([X[b], Y[b]])
        ref.append(host.last_loss())
    dev = fresh()
    dev.attach_dataset([X, Y])
    got = [l for l in (dev.step_dataset(b) for b in batches) if l is not None]
    got.append(dev.pipeline_flush())
    assert got == ref
    for a, b in zip(host.params, dev.params):
        assert np.array_equal(a.numpy(), b.numpy())
    with pytest.raises(EngineError):
        dev.step_dataset([0, 1, 2, 50])
