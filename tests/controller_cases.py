"""Seeded event streams for the controller's request handling (include/server/controller.hpp:
130-262): router requests of every type and executor completions, closed-loop.

``drive`` watches the signals each event produces to know which executors are busy, so the
stream that follows depends on what the controller under test did: equal traces mean equal
behaviour throughout (placement, scheduling, queueing, eviction, source pins, acknowledgements).

Sizes keep the reference out of its endless loop (evictor.hpp:84-95,211-224): a model is at most
a quarter of the smallest limit and a GPU holds at most three pins (one per other GPU), so an
eviction scan always finds enough unpinned bytes."""
import numpy as np

from scheduler_cases import REF_NVLINK, REF_PAIRS, reseed_libc

GiB = 1 << 30
MiB = 1 << 20
REQ_EXECUTE_AFTER_LOAD, REQ_EXECUTE, REQ_LOAD, REQ_UNLOAD = 0, 1, 2, 3
COMBOS = [("IA", "IA"), ("IA", "LRU"), ("RAND", "LRU"), ("RAND", "IA")]   # (SCHEDULE_POLICY, EVICT_POLICY)
SEEDS = range(4)
N_MODELS = 16


def limit_of(seed):
    return 2 * GiB if seed == 3 else GiB


def model_blocks(seed):
    """Per model, the blocks its cold start allocates: [(bytes, is_model)]; total_size_ sums them all
    (model_repo.hpp:140), so the non-model workspace block counts toward the eviction budget."""
    rng = np.random.default_rng(1000 + seed)
    out = {}
    for i in range(N_MODELS):
        big = int(rng.integers(1, 8)) * 16 * MiB                  # one irregular block, 16..112 MiB
        mids = int(rng.integers(0, 6))                            # 20 MiB blocks
        blocks = [(big, True)] + [(20 * MiB, True)] * mids + [(2 * MiB, True), (2 * MiB, False)]
        out[f"m{i}"] = blocks                                     # at most 112 + 100 + 4 = 216 MiB
    return out


def register_sizes(manager, blocks):
    """Cold-start allocations of every model on one manager, so that the repository knows the sizes."""
    for f, bl in blocks.items():
        manager.track_begin(f)
        for size, is_model in bl:
            manager.malloc(f, size, is_model)
        manager.track_end(f)


def as_lines(events):
    """Trace lines of the shipped mirror's event tuples."""
    return [f"S {e[1]} {e[2]} {e[3]}" if e[0] == "S" else f"A {e[1]} {e[2]}" for e in events]


def drive(ctrl, seed, n_gpu=4, n_ops=400):
    """Returns [[event description, trace lines...], ...]."""
    rng = np.random.default_rng(seed)
    models = [f"m{i}" for i in range(N_MODELS)]
    started = []                       # cold start requested
    busy = set()
    out = []

    def apply(desc, lines):
        for ln in lines:
            p = ln.split(" ")
            if p[0] == "S" and int(p[2]) in (1, 2):      # Startup or Execute: that executor now runs
                busy.add(int(p[1]))
        out.append([desc] + list(lines))

    for _ in range(n_ops):
        r = rng.random()
        if (r < 0.12 or not started) and len(started) < len(models):
            f = models[len(started)]
            started.append(f)
            payload = ["0", "1", "2", "", "7"][int(rng.integers(0, 5))]
            apply(f"R0 {f} {payload}", ctrl.request(REQ_EXECUTE_AFTER_LOAD, f, payload))
        elif r < 0.55:
            f = started[min(int(rng.zipf(1.3)) - 1, len(started) - 1)]
            apply(f"R1 {f}", ctrl.request(REQ_EXECUTE, f, ""))
        elif r < 0.90:
            if not busy:
                continue
            g = sorted(busy)[int(rng.integers(0, len(busy)))]
            busy.discard(g)
            apply(f"C {g}", ctrl.complete(g))
        elif r < 0.94:
            f = started[int(rng.integers(0, len(started)))]
            payload = "" if rng.random() < 0.5 else str(int(rng.integers(0, n_gpu)))
            apply(f"R3 {f} {payload}", ctrl.request(REQ_UNLOAD, f, payload))
        elif r < 0.98:
            idle = [g for g in range(n_gpu) if g not in busy]
            if not idle:
                continue
            f = started[int(rng.integers(0, len(started)))]
            g = idle[int(rng.integers(0, len(idle)))]
            apply(f"R1 {f} {g}", ctrl.request(REQ_EXECUTE, f, str(g)))
        else:
            f = started[int(rng.integers(0, len(started)))]
            apply(f"R2 {f}", ctrl.request(REQ_LOAD, f, ""))
    while busy:                        # drain: completions start what is still queued
        g = sorted(busy)[0]
        busy.discard(g)
        apply(f"C {g}", ctrl.complete(g))
    return out


def record(tso_backend, sched_policy, evict_policy, seeds=SEEDS):
    """Traces of a checker library on the reference's 4-GPU tables, one per seed."""
    runs = []
    for seed in seeds:
        tso_backend.reset()
        reseed_libc()
        register_sizes(tso_backend.manager(server_id=0, budget=0, gpu_count=4), model_blocks(seed))
        c = tso_backend.lib.controller(4, limit_of(seed), sched_policy, evict_policy, REF_PAIRS, REF_NVLINK)
        runs.append(drive(c, seed))
        c.close()
    tso_backend.reset()
    return runs
