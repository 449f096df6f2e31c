"""CUDA backend vs the reference's known-answer tests (same fixture that pins the oracle)."""
import pytest

from helpers import load_cases, run_case

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case", load_cases(), ids=lambda c: c["name"])
def test_cuda_reproduces_reference_known_answers(gpu_engine, case):
    run_case(gpu_engine, case)
