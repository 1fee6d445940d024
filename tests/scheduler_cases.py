"""Seeded request streams for the swap scheduler (include/server/controller.hpp:296-389).

``drive`` applies every decision the way the controller does (the chosen GPU is busy until a
completion, which registers the new replica; replicas are unloaded at random), so the stream
that follows depends on the decisions: equal decision lists mean equal behaviour throughout."""
import ctypes

import numpy as np

REF_PAIRS = [1, 0, 3, 2]                                               # controller.hpp:117
REF_NVLINK = [[0, 1, 1, 2], [1, 0, 2, 1], [1, 2, 0, 2], [2, 1, 2, 0]]  # controller.hpp:118
SEEDS = range(6)


def nvswitch(n):
    return [i ^ 1 for i in range(n)], [[0 if i == j else 2 for j in range(n)] for i in range(n)]


def reseed_libc():
    ctypes.CDLL("libc.so.6").srand(1)     # random_schedule draws from rand() (:317)


def drive(sched, set_replica, n_gpu, seed, n_ops=600):
    rng = np.random.default_rng(seed)
    models = [f"m{i}" for i in range(10)]
    for m in models:
        sched.set_level(m, int(rng.integers(0, 4)))
    busy = {}
    homes = {m: set() for m in models}
    out = []
    for _ in range(n_ops):
        r = rng.random()
        if r < 0.55:
            m = models[int(rng.integers(0, len(models)))]
            g, src, st = sched.decide(m)
            out.append([m, g, src, st])
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


def record(tso_backend, policy, seeds=SEEDS):
    """Decision lists of a checker library on the reference's 4-GPU tables, one per seed."""
    runs = []
    for seed in seeds:
        tso_backend.reset()
        reseed_libc()
        s = tso_backend.lib.scheduler(4, policy, REF_PAIRS, REF_NVLINK)
        runs.append(drive(s, lambda m, g, full: tso_backend.lib.set_model_status(m, g, full), 4, seed))
        s.close()
    tso_backend.reset()
    return runs
