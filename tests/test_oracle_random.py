"""The CPU oracle's random factories follow the contract of src/backend/cpu.rs:133-194 and src/init.rs:7-52 (ranges,
moments, empty-shape shortcuts, parameter checks); the generator itself (rand's thread_rng) is not part of the reference
tree, so no sequence of values exists to compare."""
import numpy as np
import pytest

from rusttensor_b200.frontend import EngineError


def test_oracle_factories_have_the_same_moments(oracle_engine):
    """The CPU restatement follows the same contract (different generator): ranges and first moments."""
    oracle_engine.manual_seed(3)
    u = oracle_engine.random_uniform((200000,), -1.0, 2.0).numpy()
    assert u.min() >= -1.0 and u.max() < 2.0 and abs(u.mean() - 0.5) < 0.01
    n = oracle_engine.random_normal((200000,), -1.0, 2.0).numpy()
    assert abs(n.mean() + 1.0) < 0.02 and abs(n.std() - 2.0) < 0.02
    assert abs(oracle_engine.bernoulli((200000,), 0.3).numpy().mean() - 0.3) < 0.01


def test_oracle_factory_errors(oracle_engine):
    assert oracle_engine.random_uniform((0, 3), 0.0, 1.0).shape == (0, 3)
    assert oracle_engine.kaiming_uniform(10, (4, 0)).shape == (4, 0)
    for call, kind in ((lambda: oracle_engine.random_uniform((4,), 1.0, 1.0), "InitializationError"),
                       (lambda: oracle_engine.bernoulli((4,), 1.5), "InitializationError"),
                       (lambda: oracle_engine.kaiming_uniform(0, (3, 3)), "InvalidOperation"),
                       (lambda: oracle_engine.kaiming_uniform(9, ()), "InvalidOperation")):
        with pytest.raises(EngineError) as ei:
            call()
        assert ei.value.kind == kind
