"""Eviction policy of the shipped library against the victims the reference chose
(golden) and against the CPU restatement on fresh seeded sequences."""
import json
import os

import pytest

import evictor_cases
import scenarios
from torpor_b200 import _cabi
from torpor_b200.memory_manager import Evictor, SwapError


@pytest.mark.parametrize("kind", ["LRU", "IA"])
def test_victims_match_reference_golden(built, kind):
    with open(os.path.join(scenarios.GOLDEN_DIR, f"evictor_{kind}.json")) as f:
        cases = json.load(f)
    for i, case in enumerate(cases):
        ev = Evictor(kind, evictor_cases.GPU_COUNT, evictor_cases.BUDGET)
        got = evictor_cases.replay(ev, case["ops"])
        ev.close()
        assert got == case["victims"], f"{kind} sequence {i}"


@pytest.mark.parametrize("kind", ["LRU", "IA"])
def test_victims_match_oracle_on_longer_sequences(oracle_backend, kind):
    cases = evictor_cases.record(oracle_backend.lib, kind)
    total = 0
    for case in cases:
        ev = Evictor(kind, evictor_cases.GPU_COUNT, evictor_cases.BUDGET)
        assert evictor_cases.replay(ev, case["ops"]) == case["victims"]
        ev.close()
        total += sum(len(v) for v in case["victims"])
    assert total > 50  # the sequences do evict


@pytest.mark.parametrize("kind", ["LRU", "IA"])
def test_live_differential_against_the_reference_evictor(built, ref_backend, kind):
    """Beyond the recordings: forty more seeded sequences, the reference's own evictor run now."""
    total = 0
    for i, ops in enumerate(evictor_cases.sequences(kind, n_seq=40, n_ops=200, first=100)):
        # The library first.  The generator's guard against unsatisfiable requests does not know which
        # models were evicted as victims; where the library refuses a request the reference would spin
        # for ever (evictor.hpp:84-95,211-224), so the sequence is compared up to that point.
        ev = Evictor(kind, evictor_cases.GPU_COUNT, evictor_cases.BUDGET)
        got = []
        for k, op in enumerate(ops):
            try:
                got += evictor_cases.replay(ev, [op])
            except SwapError:
                ops = ops[:k]
                break
        ev.close()
        ref = ref_backend.lib.evictor(kind, evictor_cases.GPU_COUNT, evictor_cases.BUDGET)
        want = evictor_cases.replay(ref, ops)
        ref.close()
        assert got == want, f"{kind} sequence {100 + i}"
        total += sum(len(v) for v in want)
    assert total > 500


@pytest.mark.parametrize("kind", ["LRU", "IA"])
def test_unsatisfiable_request_is_an_error_not_a_spin(built, kind):
    ev = Evictor(kind, 1, 1000)
    assert ev.check_and_add(0, "a", 600, 1) == []
    ev.lock(0, "a")
    with pytest.raises(SwapError) as e:
        ev.check_and_add(0, "b", 600, 1)      # the reference loops forever here (evictor.hpp:84-95,211-224)
    assert e.value.code == _cabi.ERR_STATE
    with pytest.raises(SwapError):
        ev.check_and_add(0, "huge", 1000, 1)  # `>=`: a model of exactly the budget never fits
    ev.unlock(0, "a")
    assert ev.check_and_add(0, "b", 600, 1) == ["a"]
    ev.close()
