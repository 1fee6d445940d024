"""The CPU restatement (oracle/torpor_oracle.cpp) against the golden tables recorded
from the reference's own headers (tests/golden/make_golden.py), and -- where the
reference checker is built -- the reference against those tables too, which pins
the recordings themselves."""
import json
import os

import pytest

import evictor_cases
import scenarios


@pytest.mark.parametrize("name", list(scenarios.SCENARIOS))
def test_oracle_reproduces_reference_tables(oracle_backend, name):
    scenarios.assert_same(scenarios.run(oracle_backend, name), scenarios.load_golden(name), f"oracle/{name}")


@pytest.mark.parametrize("name", ["mixed5", "workspace", "two_gpu"])
def test_reference_still_matches_its_recordings(ref_backend, name):
    scenarios.assert_same(scenarios.run(ref_backend, name), scenarios.load_golden(name), f"reference/{name}")


@pytest.mark.parametrize("kind", ["LRU", "IA"])
def test_oracle_evictor_matches_reference_victims(oracle_backend, kind):
    with open(os.path.join(scenarios.GOLDEN_DIR, f"evictor_{kind}.json")) as f:
        cases = json.load(f)
    assert len(cases) >= 10
    for i, case in enumerate(cases):
        ev = oracle_backend.lib.evictor(kind, evictor_cases.GPU_COUNT, evictor_cases.BUDGET)
        got = evictor_cases.replay(ev, case["ops"])
        ev.close()
        assert got == case["victims"], f"{kind} sequence {i}"
