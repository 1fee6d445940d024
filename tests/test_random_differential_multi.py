"""Randomised differential test of the host logic over several GPUs: models cold-started on random
GPUs, then evictions and swap-ins on random GPUs -- from the host store, from a replica on another
GPU, or from a GPU whose replica is not marked healthy (which falls back to the host store,
memory_manager.hpp:213-224) -- with the controller's bookkeeping of healthy replicas in between.
Replayed on the shipped plan-only engines, on the CPU restatement and, where built, on the
reference's own headers; after every step the tables of the GPU that acted must be identical."""
import numpy as np
import pytest

import scenarios
from test_random_differential import BLOCK_SIZES

N_GPU = 3


def random_stream(seed):
    rng = np.random.default_rng([77, seed])
    n_models = int(rng.integers(3, 6))
    ops = []
    home = {}
    for k in range(n_models):
        blocks = []
        for _ in range(int(rng.integers(1, 6))):
            size = int(BLOCK_SIZES[int(rng.integers(0, len(BLOCK_SIZES)))])
            offs = sorted(set(int(o) * 512 for o in rng.integers(0, size // 512 - 8, size=int(rng.integers(1, 5)))))
            pars = []
            for i, o in enumerate(offs):
                room = (offs[i + 1] if i + 1 < len(offs) else size) - o
                pars.append((o, int(rng.integers(1, min(room, 2048) + 1))))
            blocks.append((size, pars))
        g = int(rng.integers(0, N_GPU))
        home[f"m{k}"] = g
        ops.append(("cold", g, f"m{k}", blocks, float(rng.uniform(0.4, 1.0)), int(rng.integers(0, 1 << 30))))
    resident = {(f, g): (home[f] == g) for f in home for g in range(N_GPU)}
    healthy = {(f, g): False for f in home for g in range(N_GPU)}
    for _ in range(int(rng.integers(30, 70))):
        f = f"m{int(rng.integers(0, n_models))}"
        g = int(rng.integers(0, N_GPU))
        r = rng.random()
        if r < 0.25:
            # the controller registers or forgets a replica (model_repo.hpp:82-90); only a resident one is registered
            if healthy[(f, g)]:
                ops.append(("status", f, g, False)); healthy[(f, g)] = False
            elif resident[(f, g)]:
                ops.append(("status", f, g, True)); healthy[(f, g)] = True
        elif resident[(f, g)]:
            if healthy[(f, g)]:
                ops.append(("status", f, g, False)); healthy[(f, g)] = False     # unloaded replicas are forgotten first
            ops.append(("evict", g, f)); resident[(f, g)] = False
        else:
            others = [h for h in range(N_GPU) if h != g]
            src = -1 if rng.random() < 0.4 else int(others[int(rng.integers(0, len(others)))])
            ops.append(("swap_in", g, f, src)); resident[(f, g)] = True
    return ops


def replay(backend, ops):
    backend.reset()
    rec = scenarios.Recorder(backend)
    try:
        ms = [backend.manager(server_id=g, budget=0, gpu_count=N_GPU) for g in range(N_GPU)]
        for op in ops:
            if op[0] == "cold":
                _, g, f, blocks, access, seed = op
                rng = np.random.default_rng(seed)
                m = ms[g]
                m.track_begin(f)
                params = []
                for size, pars in blocks:
                    b = m.malloc(f, size, True)
                    for off, n in pars:
                        assert m.memcpy_h2d_model(f, b + off, np.zeros(n, dtype=np.uint8)) == 0
                        params.append(b + off)
                m.sync_done(f)
                m.malloc(f, 2 << 20, False)
                for p in params:
                    if rng.random() < access:
                        m.mark_access(p)
                m.track_end(f)
                rec.snap(m, f, "cold")
            elif op[0] == "status":
                backend.set_status(op[1], op[2], op[3])
            elif op[0] == "evict":
                ms[op[1]].evict(op[2]); rec.snap(ms[op[1]], op[2], "evict")
            elif op[0] == "swap_in":
                m = ms[op[1]]
                m.swap_in(op[2], op[3]); m.wait_ready(op[2]); rec.snap(m, op[2], "in")
                rec.scalar("alloc", int(m.check_alloc(op[2])))
    finally:
        backend.reset()
    return rec.out


@pytest.mark.parametrize("seed", range(10))
def test_multi_gpu_streams_agree_with_the_restatement(built, oracle_backend, seed):
    ops = random_stream(seed)
    want = replay(oracle_backend, ops)
    got = replay(scenarios.EngineBackend(device=-1), ops)
    scenarios.assert_same(got, want, f"seed {seed}")
    assert len(want) > 30 and any(op[0] == "swap_in" and op[3] >= 0 for op in ops)


@pytest.mark.parametrize("seed", range(6))
def test_restatement_agrees_with_the_reference_on_multi_gpu_streams(built, oracle_backend, ref_backend, seed):
    ops = random_stream(seed)
    scenarios.assert_same(replay(oracle_backend, ops), replay(ref_backend, ops), f"oracle vs reference, seed {seed}")
