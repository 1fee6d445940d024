"""Randomised differential test of the host logic: seeded random executor call streams
(models of random block shapes, workspace blocks of every size class, frees, evictions and
swap-ins in random order, partial access orders, both pool policies) replayed on the shipped
plan-only engine and on the CPU restatement (itself pinned to the reference's golden tables);
after every step the canonical tables must be identical."""
import numpy as np
import pytest

import scenarios

MiB = 1 << 20
# request sizes of every pool class: regular 2 / 20 MiB, irregular (rounded to 16..128 MiB), beyond a chunk
BLOCK_SIZES = [2 * MiB, 2 * MiB, 2 * MiB, 20 * MiB, 20 * MiB, 12 * MiB, 16 * MiB, 24 * MiB, 32 * MiB, 48 * MiB,
               86 * MiB, 128 * MiB, 130 * MiB, 250 * MiB]


def random_stream(seed, block_manager):
    rng = np.random.default_rng([99, seed])
    n_models = int(rng.integers(3, 7))
    ops = [("manager", block_manager)]
    for k in range(n_models):
        blocks = []
        for _ in range(int(rng.integers(1, 9))):
            size = int(BLOCK_SIZES[int(rng.integers(0, len(BLOCK_SIZES)))])
            n_par = int(rng.integers(1, 6))
            offs = sorted(set(int(o) * 512 for o in rng.integers(0, size // 512 - 8, size=n_par)))
            pars = []
            for i, o in enumerate(offs):
                room = (offs[i + 1] if i + 1 < len(offs) else size) - o
                pars.append((o, int(rng.integers(0, min(room, 4096) + 1))))
            blocks.append((size, pars))
        ws = [int(BLOCK_SIZES[int(rng.integers(0, len(BLOCK_SIZES)))]) for _ in range(int(rng.integers(0, 4)))]
        access = float(rng.uniform(0.3, 1.0))
        ops.append(("cold", f"m{k}", blocks, ws, access, int(rng.integers(0, 1 << 30))))
    resident = {f"m{k}": True for k in range(n_models)}
    freed = set()
    for _ in range(int(rng.integers(25, 60))):
        f = f"m{int(rng.integers(0, n_models))}"
        r = rng.random()
        if r < 0.08:
            ops.append(("free_ws", f))
        elif r < 0.14:
            # a later request's workspace: half of them arrive outside any tracking (an ordinary request through
            # the executor), so the pool's active-chunk lists are not closed after them (block_manager.hpp:275-286)
            ops.append(("malloc_ws", f, int(BLOCK_SIZES[int(rng.integers(0, len(BLOCK_SIZES)))]), bool(rng.random() < 0.5)))
        elif resident[f]:
            ops.append(("evict", f)); resident[f] = False
        else:
            ops.append(("swap_in", f)); resident[f] = True
    return ops


def replay(backend, ops):
    backend.reset()
    rec = scenarios.Recorder(backend)
    m = None
    ws_ptrs = {}
    try:
        for op in ops:
            if op[0] == "manager":
                m = backend.manager(budget=0, block_manager=op[1])
            elif op[0] == "cold":
                _, f, blocks, ws, access, seed = op
                rng = np.random.default_rng(seed)
                m.track_begin(f)
                params = []
                for size, pars in blocks:
                    b = m.malloc(f, size, True)
                    for off, n in pars:
                        assert m.memcpy_h2d_model(f, b + off, np.zeros(n, dtype=np.uint8)) == 0
                        params.append(b + off)
                m.sync_done(f)
                ws_ptrs[f] = [m.malloc(f, s, False) for s in ws]
                for p in params:
                    if rng.random() < access:
                        m.mark_access(p)
                m.track_end(f)
                rec.snap(m, f, "cold")
            elif op[0] == "free_ws":
                if ws_ptrs[op[1]]:
                    m.free(op[1], ws_ptrs[op[1]].pop(0))
                rec.snap(m, op[1], "free")
            elif op[0] == "malloc_ws":
                if op[3]:
                    m.track_begin(op[1])  # during the function's first run
                    ws_ptrs[op[1]].append(m.malloc(op[1], op[2], False))
                    m.track_end(op[1])
                else:
                    ws_ptrs[op[1]].append(m.malloc(op[1], op[2], False))
                rec.snap(m, op[1], "malloc")
            elif op[0] == "evict":
                m.evict(op[1]); rec.snap(m, op[1], "evict")
            elif op[0] == "swap_in":
                m.swap_in(op[1]); m.wait_ready(op[1]); rec.snap(m, op[1], "in")
                rec.scalar("alloc_" + op[1], int(m.check_alloc(op[1])))
    finally:
        backend.reset()
    return rec.out


def reuses_a_block_name(ops):
    """True if somewhere in the stream a new block of a function is granted an address that already
    names another live block of that function (its first address, free again since an eviction).  The
    reference then overwrites the old block's entry and goes on with corrupted tables -- with real
    bytes behind them it may crash -- so such streams are compared on the plan-only engine and the
    restatement only.  Found by replaying on the plan-only engine, whose placement is the reference's."""
    from torpor_b200.memory_manager import MemoryManager, repo_reset
    repo_reset()
    m, ws_ptrs, found = None, {}, False
    try:
        for op in ops:
            if op[0] == "manager":
                m = MemoryManager(0, device=-1, block_manager=op[1])
            elif op[0] == "cold":
                _, f, blocks, ws, access, seed = op
                m.track_begin(f)
                for size, pars in blocks:
                    b = m.malloc(f, size, True)
                    for off, n in pars:
                        m.memcpy_h2d_model(f, b + off, np.zeros(n, dtype=np.uint8))
                m.sync_done(f)
                ws_ptrs[f] = [m.malloc(f, s, False) for s in ws]
                m.track_end(f)
            elif op[0] == "free_ws":
                if ws_ptrs[op[1]]:
                    m.free(op[1], ws_ptrs[op[1]].pop(0))
            elif op[0] == "malloc_ws":
                names = {int(r[0]) for r in m.dump_blocks(op[1])}
                p = m.malloc(op[1], op[2], False)
                found = found or p in names
                ws_ptrs[op[1]].append(p)
            elif op[0] == "evict":
                m.evict(op[1])
            elif op[0] == "swap_in":
                m.swap_in(op[1])
    finally:
        if m:
            m.close()
        repo_reset()
    return found


@pytest.mark.parametrize("block_manager", ["Buddy", "Fixed"])
@pytest.mark.parametrize("seed", range(12))
def test_random_streams_agree_with_the_restatement(built, oracle_backend, seed, block_manager):
    ops = random_stream(seed, block_manager)
    want = replay(oracle_backend, ops)
    got = replay(scenarios.EngineBackend(device=-1), ops)
    scenarios.assert_same(got, want, f"seed {seed} / {block_manager}")
    assert len(want) > 30


@pytest.mark.parametrize("block_manager", ["Buddy", "Fixed"])
@pytest.mark.parametrize("seed", range(10))
def test_restatement_agrees_with_the_reference_on_random_streams(built, oracle_backend, ref_backend, seed, block_manager):
    """Where the reference's own headers are built: the restatement follows them on the random
    streams too, not only on the recorded scenarios."""
    ops = random_stream(seed, block_manager)
    if reuses_a_block_name(ops):
        pytest.skip("a block's name is granted again in this stream: the reference corrupts its own tables there")
    scenarios.assert_same(replay(oracle_backend, ops), replay(ref_backend, ops), f"oracle vs reference, seed {seed} / {block_manager}")
