"""Request handling of the controller (include/server/controller.hpp:130-262, 392-453): the
shipped library and the CPU restatement against traces recorded from the reference's own
``Controller::start`` loop (controller.hpp compiled where it lies, its socket stand-in feeding one
scripted event per turn; tests/golden/controller_*.json) on the reference's 4-GPU tables, and
against each other on an 8-GPU NVSwitch layout."""
import json
import os

import pytest

import controller_cases as CC
import scenarios
from scheduler_cases import nvswitch, reseed_libc
from torpor_b200.memory_manager import (Controller, MemoryManager, ModelRepo, SwapError, repo_reset,
                                        REQ_EXECUTE, REQ_EXECUTE_AFTER_LOAD, SIGNAL_EXECUTE, SIGNAL_LOAD,
                                        SIGNAL_STARTUP, STATUS_AVAIL)

MiB = 1 << 20


def golden(sp, ep):
    with open(os.path.join(scenarios.GOLDEN_DIR, f"controller_{sp}_{ep}.json")) as f:
        return json.load(f)


class Mirror:
    """The shipped controller behind the checker libraries' method names."""

    def __init__(self, c):
        self.c = c

    def request(self, kind, func, payload=""):
        return CC.as_lines(self.c.request(kind, func, payload))

    def complete(self, executor):
        return CC.as_lines(self.c.complete(executor))


def engine_run(n, sp, ep, pairs, nv, seed):
    repo_reset()
    reseed_libc()
    m = MemoryManager(0, device=-1, server_id=0, gpu_count=n)
    CC.register_sizes(m, CC.model_blocks(seed))
    c = Controller(n, CC.limit_of(seed), sp, ep, pairs, nv)
    got = CC.drive(Mirror(c), seed, n_gpu=n)
    c.close(); m.close()
    repo_reset()
    return got


def kinds(run):
    return {(ln.split(" ")[0], int(ln.split(" ")[2])) for ev in run for ln in ev[1:] if ln.startswith("S")}


@pytest.mark.parametrize("sp,ep", CC.COMBOS)
def test_engine_traces_match_the_reference_controller_loop(built, sp, ep):
    want = golden(sp, ep)
    assert len(want) == len(CC.SEEDS)
    for seed, w in zip(CC.SEEDS, want):
        got = engine_run(4, sp, ep, CC.REF_PAIRS, CC.REF_NVLINK, seed)
        assert got == w, f"{sp}/{ep} seed {seed}"
    seen = set().union(*[kinds(w) for w in want])
    # cold starts, notifications, executions, unloads and loads from the host store all occur, and (the random
    # policy never picks a source GPU, controller.hpp:316-318) loads from a replica
    assert {("S", 0), ("S", 1), ("S", 2), ("S", 3), ("S", 4)} <= seen and (sp == "RAND" or any(k[1] > 4 for k in seen))
    evicted = sum(1 for w in want for ev in w if not ev[0].startswith("R3") for ln in ev[1:] if ln.split(" ")[:1] == ["S"] and ln.split(" ")[2] == "3")
    queued = sum(1 for w in want for ev in w if ev[0].startswith("R1") and len(ev) == 1)
    assert evicted > 10 and queued > 50          # the eviction policy and the request queue are exercised


@pytest.mark.parametrize("sp,ep", CC.COMBOS)
def test_restatement_traces_match_the_reference_controller_loop(oracle_backend, sp, ep):
    assert CC.record(oracle_backend, sp, ep) == golden(sp, ep)


@pytest.mark.parametrize("sp,ep", CC.COMBOS[:2])
def test_reference_controller_loop_still_matches_its_recordings(ref_backend, sp, ep):
    assert CC.record(ref_backend, sp, ep) == golden(sp, ep)


@pytest.mark.parametrize("sp,ep", CC.COMBOS)
def test_live_differential_against_the_reference_controller_loop(built, ref_backend, sp, ep):
    """Beyond the recordings: twelve more seeded streams per policy pair, the reference's loop run now."""
    seeds = range(100, 112)
    want = CC.record(ref_backend, sp, ep, seeds)
    for seed, w in zip(seeds, want):
        assert engine_run(4, sp, ep, CC.REF_PAIRS, CC.REF_NVLINK, seed) == w, f"{sp}/{ep} seed {seed}"


@pytest.mark.parametrize("sp,ep", CC.COMBOS)
def test_eight_gpu_layout_matches_the_restatement(built, oracle_backend, sp, ep):
    pairs, nv = nvswitch(8)
    for seed in range(3):
        oracle_backend.reset()
        reseed_libc()
        CC.register_sizes(oracle_backend.manager(server_id=0, budget=0, gpu_count=8), CC.model_blocks(seed))
        o = oracle_backend.lib.controller(8, CC.limit_of(seed), sp, ep, pairs, nv)
        want = CC.drive(o, seed, n_gpu=8)
        o.close()
        assert engine_run(8, sp, ep, pairs, nv, seed) == want, f"{sp}/{ep} seed {seed}"
    oracle_backend.reset()


def test_request_that_cannot_be_made_room_for_is_refused_not_spun_on(built):
    """The reference loops forever here (evictor.hpp:211-224); the library answers with an error,
    sends nothing and leaves the GPU available."""
    repo_reset()
    m = MemoryManager(0, device=-1, server_id=0, gpu_count=2)
    for f, size in (("a", 64 * MiB), ("b", 128 * MiB)):
        m.track_begin(f); m.malloc(f, size, True); m.track_end(f)
    c = Controller(2, 100 * MiB, "IA", "LRU")
    assert [e for e in c.request(REQ_EXECUTE_AFTER_LOAD, "a", "1") if e[0] == "S" and e[2] == SIGNAL_STARTUP] == [("S", 0, SIGNAL_STARTUP, "a")]
    assert c.complete(0) == []
    assert ModelRepo.active_devices("a") == [0]
    with pytest.raises(SwapError):
        c.request(REQ_EXECUTE, "b", "1")                 # 128 MiB can never fit a 100 MiB limit
    assert c.executor_status(1) == (STATUS_AVAIL, "") and c.queue_depth() == 0
    ev = c.request(REQ_EXECUTE, "a")                     # the controller still works: resident and idle, runs in place
    assert ev == [("S", 0, SIGNAL_LOAD, "a"), ("S", 0, SIGNAL_EXECUTE, "a"), ("A", 0, 0)]
    assert c.executor_status(0) == (0, "a")
    c.close(); m.close(); repo_reset()


def test_requests_queue_when_every_gpu_is_busy_and_take_the_next_completion(built):
    repo_reset()
    m = MemoryManager(0, device=-1, server_id=0, gpu_count=2)
    for f in ("a", "b", "c"):
        m.track_begin(f); m.malloc(f, 16 * MiB, True); m.track_end(f)
    c = Controller(2, 1 << 30, "IA", "IA")
    c.request(REQ_EXECUTE_AFTER_LOAD, "a", "0"); c.request(REQ_EXECUTE_AFTER_LOAD, "b", "2")
    assert c.request(REQ_EXECUTE_AFTER_LOAD, "c", "") == [] and c.queue_depth() == 1     # no acknowledgement yet
    assert c.request(REQ_EXECUTE, "a") == [] and c.queue_depth() == 2
    ev = c.complete(1)                                   # the queued cold start takes GPU 1
    assert ev == [("S", 0, 0, "c"), ("S", 1, SIGNAL_STARTUP, "c"), ("A", 0, 1)]
    ev = c.complete(0)                                   # "a" is resident on GPU 0, which just became free
    assert ev == [("S", 0, SIGNAL_LOAD, "a"), ("S", 0, SIGNAL_EXECUTE, "a"), ("A", 0, 0)]
    assert c.queue_depth() == 0
    c.close(); m.close(); repo_reset()


def test_pinned_replicas_in_the_way_queue_the_request_until_a_completion(built):
    """Where the reference would spin on a GPU whose residents are all pinned as swap sources, the
    request waits like one that found every GPU busy and is served by the next completion."""
    repo_reset()
    m = MemoryManager(0, device=-1, server_id=0, gpu_count=2)
    for f in ("a", "b", "c"):
        m.track_begin(f); m.malloc(f, 64 * MiB, True); m.track_end(f)
    c = Controller(2, 100 * MiB, "IA", "LRU")
    c.request(REQ_EXECUTE_AFTER_LOAD, "a", "1"); c.complete(0)
    c.request(REQ_EXECUTE_AFTER_LOAD, "b", "1"); c.complete(1)
    assert c.request(REQ_EXECUTE, "a") == [("S", 0, SIGNAL_LOAD, "a"), ("S", 0, SIGNAL_EXECUTE, "a"), ("A", 0, 0)]
    # a second request for "a": GPU 1 copies it from GPU 0 (signal 4 + 1 + 0), "b" makes room; "a" on GPU 0 is now pinned
    assert c.request(REQ_EXECUTE, "a") == [("S", 1, 3, "b"), ("S", 1, SIGNAL_LOAD + 1, "a"), ("S", 1, SIGNAL_EXECUTE, "a"), ("A", 0, 1)]
    assert c.complete(0) == []
    # "b" would go to the idle GPU 0, whose only resident is pinned: queued, nothing sent, GPU 0 stays available
    assert c.request(REQ_EXECUTE, "b") == [] and c.queue_depth() == 1 and c.executor_status(0)[0] == STATUS_AVAIL
    # GPU 1 finishes its copy: the pin goes, and the queued request takes GPU 1 (its replica of "a" makes room)
    assert c.complete(1) == [("S", 1, 3, "a"), ("S", 1, SIGNAL_LOAD, "b"), ("S", 1, SIGNAL_EXECUTE, "b"), ("A", 0, 1)]
    assert c.queue_depth() == 0 and ModelRepo.active_devices("a") == [0]

    # a cold start that has finished is entered even when pins keep its GPU over the limit
    c.complete(1)                                                        # "b" now resident on GPU 1
    c.request(REQ_EXECUTE, "b"); c.request(REQ_EXECUTE, "b")             # GPU 1 runs it; GPU 0 copies from GPU 1 ("a" evicted, "b" on 1 pinned)
    assert c.executor_status(0) == (1, "b") and c.executor_status(1) == (0, "b")
    assert c.request(REQ_EXECUTE_AFTER_LOAD, "c", "1") == []             # both busy: the cold start waits
    assert [e for e in c.complete(1) if e[0] == "S" and e[2] == SIGNAL_STARTUP] == [("S", 1, SIGNAL_STARTUP, "c")]
    assert c.complete(1) == []                                           # "b" on GPU 1 is still pinned by GPU 0: nothing to unload, no error
    assert sorted(ModelRepo.active_devices("c")) == [1] and sorted(ModelRepo.active_devices("b")) == [1]
    c.complete(0)                                                        # the copy ends, the pin goes
    assert sorted(ModelRepo.active_devices("b")) == [0, 1]
    # GPU 1 holds "b" and "c" (128 MiB against a 100 MiB limit); with the pin gone the policy works as before
    assert c.request(REQ_EXECUTE, "a") == [("S", 0, 3, "b"), ("S", 0, SIGNAL_LOAD, "a"), ("S", 0, SIGNAL_EXECUTE, "a"), ("A", 0, 0)]
    c.close(); m.close(); repo_reset()
