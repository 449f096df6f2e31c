"""Random tensor factories on the device (Backend::random_uniform / random_normal / bernoulli / kaiming_uniform,
src/backend/mod.rs:57-69).  The reference draws from rand's thread-local generator, which cannot be seeded, so its own
tests (tests/ops_cpu_tests.rs random_* cases, src/init.rs:54-110) check ranges, moments and shapes; so do these, plus the
properties the counter-based generator adds: a seed reproduces the values, and consecutive calls continue one stream."""
import ctypes as C

import numpy as np
import pytest

from rusttensor_b200.frontend import EngineError

pytestmark = pytest.mark.gpu
N = 1 << 20


def test_uniform_range_and_moments(gpu_engine):
    gpu_engine.manual_seed(7)
    x = gpu_engine.random_uniform((N,), -2.0, 3.0).numpy()
    assert x.shape == (N,) and x.dtype == np.float32
    assert x.min() >= -2.0 and x.max() < 3.0
    assert abs(x.mean() - 0.5) < 0.01 and abs(x.var() - 25.0 / 12.0) < 0.02
    hist, _ = np.histogram(x, bins=50, range=(-2.0, 3.0))
    assert np.all(np.abs(hist - N / 50) < 6 * np.sqrt(N / 50))  # flat within six standard deviations per bin


def test_normal_moments(gpu_engine):
    gpu_engine.manual_seed(8)
    x = gpu_engine.random_normal((N,), 1.5, 0.5).numpy().astype(np.float64)
    z = (x - 1.5) / 0.5
    assert abs(z.mean()) < 0.005 and abs(z.std() - 1.0) < 0.005
    assert abs((z ** 3).mean()) < 0.02 and abs((z ** 4).mean() - 3.0) < 0.05
    assert np.all(np.isfinite(x)) and np.abs(z).max() > 4.0  # tails are populated, no infinities from log(0)


def test_bernoulli_frequency(gpu_engine):
    gpu_engine.manual_seed(9)
    for p in (0.0, 0.25, 0.9, 1.0):
        x = gpu_engine.bernoulli((N,), p).numpy()
        assert set(np.unique(x)) <= {0.0, 1.0}
        assert abs(x.mean() - p) <= 4 * np.sqrt(max(p * (1 - p), 1e-12) / N) + 1e-12


def test_seed_reproduces_and_calls_continue_the_stream(gpu_engine):
    gpu_engine.manual_seed(123)
    a = gpu_engine.random_uniform((1000,), 0.0, 1.0).numpy()
    b = gpu_engine.random_normal((37, 5), 0.0, 1.0).numpy()
    gpu_engine.manual_seed(123)
    a2 = gpu_engine.random_uniform((1000,), 0.0, 1.0).numpy()
    b2 = gpu_engine.random_normal((37, 5), 0.0, 1.0).numpy()
    assert np.array_equal(a, a2) and np.array_equal(b, b2)
    gpu_engine.manual_seed(124)
    assert not np.array_equal(a, gpu_engine.random_uniform((1000,), 0.0, 1.0).numpy())
    # two calls of 512 elements = one call of 1024 (a call of n elements consumes (n + 3) / 4 counter values)
    gpu_engine.manual_seed(5)
    parts = np.concatenate([gpu_engine.random_uniform((512,), 0.0, 1.0).numpy() for _ in range(2)])
    gpu_engine.manual_seed(5)
    assert np.array_equal(parts, gpu_engine.random_uniform((1024,), 0.0, 1.0).numpy())


def test_values_do_not_depend_on_size_or_launch_geometry(capi):
    """Element i is a function of (seed, offset + i / 4) only: a prefix of a long call equals a short call."""
    big, small = capi.empty((1 << 18,)), capi.empty((1003,))
    seed, off = C.c_uint64(99), C.c_uint64(17)
    capi.call("random_normal", big.ptr, C.c_int64(big.size), C.c_float(0), C.c_float(1), seed, off)
    capi.call("random_normal", small.ptr, C.c_int64(small.size), C.c_float(0), C.c_float(1), seed, off)
    assert np.array_equal(big.numpy()[:1003], small.numpy())
    shifted = capi.empty((1000,))
    capi.call("random_normal", shifted.ptr, C.c_int64(1000), C.c_float(0), C.c_float(1), seed, C.c_uint64(17 + 25))
    assert np.array_equal(big.numpy()[100:1100], shifted.numpy())  # offset + 25 counters = 100 elements further on


def test_kaiming_uniform_bound_and_shape(gpu_engine):
    gpu_engine.manual_seed(11)
    w = gpu_engine.kaiming_uniform(784, (784, 128), requires_grad=True)
    assert w.shape == (784, 128) and w.requires_grad
    x = w.numpy()
    bound = np.sqrt(6.0 / 784)
    assert np.abs(x).max() <= bound and np.abs(x).max() > 0.99 * bound
    assert abs(x.mean()) < 1e-3 and abs(x.std() - bound / np.sqrt(3)) < 1e-3


def test_empty_shapes_and_parameter_errors(oracle_engine, gpu_engine):
    """Same shortcuts and failures on both backends (src/backend/cpu.rs:133-181, src/init.rs:7-30)."""
    for e in (oracle_engine, gpu_engine):
        assert e.random_uniform((0, 3), 0.0, 1.0).shape == (0, 3)
        assert e.random_normal((2, 0), 0.0, 1.0).numpy().size == 0
        assert e.bernoulli((0,), 0.5).shape == (0,)
        assert e.kaiming_uniform(10, (4, 0)).shape == (4, 0)
        assert e.random_uniform((), 2.0, 3.0).shape == ()
        for call, kind in ((lambda: e.random_uniform((4,), 1.0, 1.0), "InitializationError"),
                           (lambda: e.random_uniform((4,), 2.0, 1.0), "InitializationError"),
                           (lambda: e.random_uniform((4,), 0.0, float("inf")), "InitializationError"),
                           (lambda: e.random_normal((4,), 0.0, float("nan")), "InitializationError"),
                           (lambda: e.bernoulli((4,), 1.5), "InitializationError"),
                           (lambda: e.bernoulli((4,), -0.1), "InitializationError"),
                           (lambda: e.kaiming_uniform(0, (3, 3)), "InvalidOperation"),
                           (lambda: e.kaiming_uniform(9, ()), "InvalidOperation")):
            with pytest.raises(EngineError) as ei:
                call()
            assert ei.value.kind == kind
