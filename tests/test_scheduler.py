"""Swap scheduler (include/server/controller.hpp:296-389): the shipped library and the CPU
restatement against decisions recorded from the reference's own Controller object
(controller.hpp compiled where it lies with its socket and executor headers shadowed;
tests/golden/scheduler_*.json) on the reference's 4-GPU tables, and against each other on an
8-GPU NVSwitch layout the reference's hard-coded tables cannot express."""
import json
import os

import pytest

import scenarios
import scheduler_cases as SC
from scheduler_cases import nvswitch
from torpor_b200.memory_manager import ModelRepo, Scheduler, repo_reset


def golden(policy):
    with open(os.path.join(scenarios.GOLDEN_DIR, f"scheduler_{policy}.json")) as f:
        return json.load(f)


def engine_stream(n, policy, pairs, nv, seed):
    repo_reset()
    SC.reseed_libc()
    s = Scheduler(n, policy, pairs, nv)
    got = SC.drive(s, lambda m, g, full: (ModelRepo.add_model_info if full else ModelRepo.remove_model_info)(m, g), n, seed)
    s.close()
    repo_reset()
    return got


@pytest.mark.parametrize("policy", ["IA", "RAND"])
def test_engine_decisions_match_the_reference_controller(built, policy):
    want = golden(policy)
    assert len(want) == len(SC.SEEDS)
    for seed, w in zip(SC.SEEDS, want):
        got = engine_stream(4, policy, SC.REF_PAIRS, SC.REF_NVLINK, seed)
        assert got == w, f"{policy} seed {seed}"
        kinds = {d[3] for d in got}
        assert {-1, 0} <= kinds and (policy == "RAND" or 1 in kinds)   # queued, in place, and replica swaps all occur


@pytest.mark.parametrize("policy", ["IA", "RAND"])
def test_restatement_decisions_match_the_reference_controller(oracle_backend, policy):
    assert SC.record(oracle_backend, policy) == golden(policy)


@pytest.mark.parametrize("policy", ["IA", "RAND"])
def test_reference_controller_still_matches_its_recordings(ref_backend, policy):
    assert SC.record(ref_backend, policy) == golden(policy)


@pytest.mark.parametrize("policy", ["IA", "RAND"])
def test_live_differential_against_the_reference_controller(built, ref_backend, policy):
    """Beyond the recordings: twenty more seeded streams, decided by the reference's Controller now."""
    seeds = range(50, 70)
    want = SC.record(ref_backend, policy, seeds)
    for seed, w in zip(seeds, want):
        assert engine_stream(4, policy, SC.REF_PAIRS, SC.REF_NVLINK, seed) == w, f"{policy} seed {seed}"


@pytest.mark.parametrize("policy", ["IA", "RAND"])
def test_eight_gpu_layout_matches_the_restatement(built, oracle_backend, policy):
    pairs, nv = SC.nvswitch(8)
    for seed in range(4):
        oracle_backend.reset()
        SC.reseed_libc()
        o = oracle_backend.lib.scheduler(8, policy, pairs, nv)
        want = SC.drive(o, lambda m, g, full: oracle_backend.lib.set_model_status(m, g, full), 8, seed)
        o.close()
        assert engine_stream(8, policy, pairs, nv, seed) == want, f"{policy} seed {seed}"
    oracle_backend.reset()


def test_defaults_describe_an_nvswitch_box(built):
    repo_reset()
    s = Scheduler(8)
    s.set_level("f", 2)
    assert s.decide("f") == (0, -1, 4)                 # nothing resident: host swap, heavy model
    s.set_status(0, 4); s.set_status(1, 0)
    assert s.decide("f")[0] == 2                        # GPU 1's sibling (0) is busier than GPU 2's (3)
    ModelRepo.add_model_info("f", 0)
    g, src, st = s.decide("f")
    assert src == 0 and st == 1 and g == 7              # replica swap over NVLink; the scan keeps the last idle GPU
    s.set_status(0, -1)
    assert s.decide("f") == (0, -1, 0)                  # resident and idle: run in place
    for g in range(8):
        s.set_status(g, 3)
    assert s.decide("f") == (-1, -1, -1)                # nothing available: the caller queues
    s.close(); repo_reset()


def test_link_lending_reads_the_same_occupancy_signal(built):
    """Helpers for a swap-in over several PCIe links: available GPUs whose uplink is not shared with
    the target, with a loading GPU or with another helper."""
    repo_reset()
    s = Scheduler(8)                                     # default table: GPU i shares its uplink with i^1
    assert s.helpers(0) == [2, 4, 6]                     # 1 shares the target's uplink; 3, 5, 7 share a helper's
    s.set_status(3, 3)                                   # GPU 3 loads over PCIe: its sibling 2 would add nothing
    assert s.helpers(0) == [4, 6]
    s.set_status(4, 0)                                   # GPU 4 runs in place: busy, but its link is idle
    assert s.helpers(0) == [5, 6] and s.helpers(0, include_running=True) == [4, 6]
    s.close()
    own = list(range(8))                                 # every GPU has its uplink alone
    s = Scheduler(8, "IA", own, nvswitch(8)[1])
    assert s.helpers(2) == [0, 1, 3, 4, 5, 6, 7]
    s.set_status(5, 4); s.set_status(6, 1)
    assert s.helpers(2) == [0, 1, 3, 4, 7] and s.helpers(2, include_running=True) == [0, 1, 3, 4, 6, 7]
    s.close(); repo_reset()
