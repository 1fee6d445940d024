"""Seeded operation sequences for the eviction policies (include/server/evictor.hpp).

``sequences(kind)`` yields op lists; ``replay(evictor, ops)`` runs one and returns what
each check_and_add evicted.  Sequences never ask for an eviction that cannot be
satisfied -- the reference spins forever there (evictor.hpp:84-95,211-224) -- which
``safe`` guarantees by tracking the unlocked bytes per GPU.
"""
from __future__ import annotations

from typing import Dict, List

import numpy as np

GPU_COUNT = 4
BUDGET = 1000


def sequences(kind: str, n_seq: int = 12, n_ops: int = 160, first: int = 0) -> List[List[list]]:
    out = []
    for s in range(first, first + n_seq):
        rng = np.random.default_rng([31, s, 0 if kind == "LRU" else 1])
        n_models = int(rng.integers(6, 20))
        sizes = {f"m{i}": int(rng.integers(40, 420)) for i in range(n_models)}
        levels = {f"m{i}": int(rng.integers(0, 3)) for i in range(n_models)}
        resident: List[Dict[str, int]] = [dict() for _ in range(GPU_COUNT)]
        locked: List[set] = [set() for _ in range(GPU_COUNT)]
        ops = []
        for _ in range(n_ops):
            g = int(rng.integers(0, GPU_COUNT))
            m = f"m{int(rng.integers(0, n_models))}"
            r = rng.random()
            if r < 0.70:
                if m not in resident[g]:
                    # only ask when the unlocked residents can make room
                    locked_bytes = sum(sz for k, sz in resident[g].items() if k in locked[g])
                    if locked_bytes + sizes[m] >= BUDGET:
                        continue
                ops.append(["add", g, m, sizes[m], levels[m]])
            elif r < 0.80:
                ops.append(["force", g, m])
            elif r < 0.92:
                if kind == "LRU" and m not in resident[g]:
                    continue
                ops.append(["lock", g, m])
                locked[g].add(m)
            else:
                ops.append(["unlock", g, m])
                locked[g].discard(m)
            # mirror residency with the policy-independent facts only: who is present
            if ops[-1][0] == "add":
                resident[g][m] = sizes[m]
            elif ops[-1][0] == "force":
                resident[g].pop(m, None)
        out.append(ops)
    return out


def replay(ev, ops, on_victims=None) -> List[List[str]]:
    results = []
    for op in ops:
        if op[0] == "add":
            v = ev.check_and_add(op[1], op[2], op[3], op[4])
            results.append(v)
            if on_victims:
                on_victims(op[1], v)
        elif op[0] == "force":
            ev.force_evict(op[1], op[2])
        elif op[0] == "lock":
            ev.lock(op[1], op[2])
        elif op[0] == "unlock":
            ev.unlock(op[1], op[2])
    return results


def record(tso_lib, kind: str):
    """[{ops, victims}] with the victims the given checker library produces."""
    cases = []
    for ops in sequences(kind):
        ev = tso_lib.evictor(kind, GPU_COUNT, BUDGET)
        kept = []
        victims = []
        resident = [dict() for _ in range(GPU_COUNT)]
        locked = [set() for _ in range(GPU_COUNT)]
        for op in ops:
            if op[0] == "add":
                g, m, sz = op[1], op[2], op[3]
                if m not in resident[g]:
                    # exact guard, using the true residency of this run
                    evictable = sum(s for k, s in resident[g].items() if k not in locked[g])
                    cur = sum(resident[g].values())
                    if cur - evictable + sz >= BUDGET:
                        continue
                v = ev.check_and_add(g, m, sz, op[4])
                for x in v:
                    resident[g].pop(x, None)
                resident[g][m] = sz
                victims.append(v)
            elif op[0] == "force":
                ev.force_evict(op[1], op[2])
                resident[op[1]].pop(op[2], None)
            elif op[0] == "lock":
                if kind == "LRU" and op[2] not in resident[op[1]]:
                    continue
                ev.lock(op[1], op[2])
                locked[op[1]].add(op[2])
            elif op[0] == "unlock":
                ev.unlock(op[1], op[2])
                locked[op[1]].discard(op[2])
            kept.append(op)
        ev.close()
        cases.append({"ops": kept, "victims": victims})
    return cases
