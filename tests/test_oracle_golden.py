"""The CPU oracle must reproduce every known-answer test of the reference (pins the oracle)."""
import numpy as np
import pytest

from helpers import load_cases, run_case


@pytest.mark.parametrize("case", load_cases(), ids=lambda c: c["name"])
def test_oracle_reproduces_reference_known_answers(oracle_engine, case):
    run_case(oracle_engine, case)


def test_golden_file_is_current():
    """The committed fixture equals what tests/golden/make_golden.py generates."""
    import json, os, subprocess, sys, tempfile, shutil
    here = os.path.dirname(os.path.abspath(__file__))
    committed = json.load(open(os.path.join(here, "golden", "reference_known_answers.json")))
    assert len(committed["cases"]) >= 30
    for c in committed["cases"]:
        assert c["cite"] and ":" in c["cite"], c["name"]
