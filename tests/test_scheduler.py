"""Swap scheduler of the shipped library against the CPU restatement of the controller's
decision functions (include/server/controller.hpp:296-389) on seeded request streams, with
the reference's own 4-GPU tables and with an 8-GPU NVSwitch layout.  (The controller itself
cannot be compiled without zmq/protobuf, so this row is checked against the restatement
only.)"""
import ctypes

import numpy as np
import pytest

from torpor_b200.memory_manager import ModelRepo, Scheduler, repo_reset

REF_PAIRS = [1, 0, 3, 2]                                               # controller.hpp:117
REF_NVLINK = [[0, 1, 1, 2], [1, 0, 2, 1], [1, 2, 0, 2], [2, 1, 2, 0]]  # controller.hpp:118


def nvswitch(n):
    return [i ^ 1 for i in range(n)], [[0 if i == j else 2 for j in range(n)] for i in range(n)]


def drive(sched, set_replica, n_gpu, seed, n_ops=600):
    """A request stream: decisions are applied the way the controller applies them
    (GPU busy until completion, replica registered on completion, random unloads)."""
    rng = np.random.default_rng(seed)
    models = [f"m{i}" for i in range(10)]
    for m in models:
        sched.set_level(m, int(rng.integers(0, 4)) - 0)
    busy = {}
    homes = {m: set() for m in models}
    out = []
    for _ in range(n_ops):
        r = rng.random()
        if r < 0.55:
            m = models[int(rng.integers(0, len(models)))]
            g, src, st = sched.decide(m)
            out.append((m, g, src, st))
            if g >= 0:
                sched.set_status(g, st)
                busy[g] = m
        elif r < 0.9 and busy:
            g = sorted(busy)[int(rng.integers(0, len(busy)))]
            m = busy.pop(g)
            sched.set_status(g, -1)
            set_replica(m, g, True)
            homes[m].add(g)
        else:
            m = models[int(rng.integers(0, len(models)))]
            for g in sorted(homes[m]):
                if g not in busy:
                    set_replica(m, g, False)
                    homes[m].discard(g)
                    break
    return out


@pytest.mark.parametrize("policy", ["IA", "RAND"])
@pytest.mark.parametrize("layout", ["reference_4gpu", "nvswitch_8gpu"])
def test_decisions_match_the_restatement(built, oracle_backend, policy, layout):
    n, pairs, nv = (4, REF_PAIRS, REF_NVLINK) if layout == "reference_4gpu" else (8, *nvswitch(8))
    libc = ctypes.CDLL("libc.so.6")
    for seed in range(4):
        oracle_backend.reset()
        libc.srand(1)
        o = oracle_backend.lib.scheduler(n, policy, pairs, nv)
        want = drive(o, lambda m, g, full: oracle_backend.lib.set_model_status(m, g, full), n, seed)
        o.close()
        repo_reset()
        libc.srand(1)
        s = Scheduler(n, policy, pairs, nv)
        got = drive(s, lambda m, g, full: (ModelRepo.add_model_info if full else ModelRepo.remove_model_info)(m, g), n, seed)
        s.close()
        assert got == want, f"{policy}/{layout} seed {seed}"
        kinds = {d[3] for d in got}
        assert {-1, 0} <= kinds and (policy == "RAND" or 1 in kinds)   # queued, local, and replica swaps all occur
    repo_reset(); oracle_backend.reset()


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
