"""Seeded synthetic parameters and inputs of the five benchmark workloads (stand-ins for MNIST images, labels and a
character corpus: neither dataset ships with the reference) and the helper that loads them into a trainer.  Used by
``bench.py``, the smoke test and the parity tests, so that all of them run the same data."""
import numpy as np


def rng(seed):
    return np.random.default_rng(seed)


def kaiming_uniform(r, fan_in, shape):
    """U(-sqrt(6/fan_in), +sqrt(6/fan_in)) (src/init.rs:26-32), seeded."""
    lim = np.sqrt(6.0 / fan_in)
    return r.uniform(-lim, lim, size=shape).astype(np.float32)


def one_hot(r, n, classes):
    y = np.zeros((n, classes), dtype=np.float32)
    y[np.arange(n), r.integers(0, classes, size=n)] = 1.0
    return y


def workload_data(config, dims, seed, rank=0):
    """Seeded synthetic parameters and inputs with the shapes / distributions of the benchmark
    configurations (stand-ins for MNIST images, labels and a character corpus)."""
    r = rng(1234 + 1000 * config + seed)
    rd = rng(99 + 1000 * config + seed * 17 + rank)  # per-rank data, identical parameters
    d = dims
    if config == 1:
        params = [kaiming_uniform(r, d[1], (d[1], d[2])), np.zeros(d[2], np.float32),
                  kaiming_uniform(r, d[2], (d[2], d[3])), np.zeros(d[3], np.float32)]
        inputs = [rd.uniform(0, 1, (d[0], d[1])).astype(np.float32), one_hot(rd, d[0], d[3])]
    elif config == 2:
        params = [r.standard_normal((d[0], d[1])).astype(np.float32), r.standard_normal(d[1]).astype(np.float32)]
        inputs = []
    elif config == 3:
        hw, p2 = d[1], d[1] // 4
        params = [kaiming_uniform(r, 9, (d[2], 1, 3, 3)), np.zeros(d[2], np.float32),
                  kaiming_uniform(r, d[2] * 9, (d[3], d[2], 3, 3)), np.zeros(d[3], np.float32),
                  kaiming_uniform(r, d[3] * p2 * p2, (d[3] * p2 * p2, d[4])), np.zeros(d[4], np.float32),
                  kaiming_uniform(r, d[4], (d[4], d[5])), np.zeros(d[5], np.float32)]
        inputs = [rd.uniform(0, 1, (d[0], 1, hw, hw)).astype(np.float32), one_hot(rd, d[0], d[5])]
    elif config == 4:
        params = [kaiming_uniform(r, d[1] * 9, (d[3], d[1], 3, 3)), (0.01 * r.standard_normal(d[3])).astype(np.float32),
                  kaiming_uniform(r, d[3] * 16, (d[3], d[1], 4, 4)), (0.01 * r.standard_normal(d[1])).astype(np.float32)]
        inputs = [rd.standard_normal((d[0], d[1], d[2], d[2])).astype(np.float32),
                  rd.standard_normal((d[0], d[1], d[2], d[2])).astype(np.float32)]
    elif config == 5:
        V, H, T, B = d
        params = [kaiming_uniform(r, V + H, (V + H, 4 * H)), np.zeros(4 * H, np.float32),
                  kaiming_uniform(r, H, (H, V)), np.zeros(V, np.float32)]
        inputs = [one_hot(rd, T * B, V), one_hot(rd, T * B, V)]
    else:
        raise ValueError(config)
    return params, inputs


def setup_trainer(engine, config, dims, params, hyper=None):
    tr = engine.trainer(config, dims)
    for t, p in zip(tr.params, params):
        t.update_from_host(p)
    if hyper:
        tr.set_hyper(*hyper)
    return tr
