"""Host logic of the shipped engine -- pool placement, table rebind, translation,
eviction order -- against the golden tables of the reference and against the CPU
restatement, on plan-only engines (no GPU, no byte moves)."""
import numpy as np
import pytest

import scenarios
from torpor_b200 import _cabi
from torpor_b200 import workloads as W
from torpor_b200.memory_manager import MemoryManager, SwapError, repo_reset


@pytest.fixture(scope="module")
def plan_backend(built):
    return scenarios.EngineBackend(device=-1)


@pytest.mark.parametrize("name", list(scenarios.SCENARIOS))
def test_engine_tables_match_reference_golden(plan_backend, name):
    scenarios.assert_same(scenarios.run(plan_backend, name), scenarios.load_golden(name), f"engine/{name}")


@pytest.mark.parametrize("name", ["churn_buddy", "workspace"])
def test_engine_tables_match_oracle_live(plan_backend, oracle_backend, name):
    scenarios.assert_same(scenarios.run(plan_backend, name), scenarios.run(oracle_backend, name), f"engine-vs-oracle/{name}")


def test_pool_geometry(built):
    repo_reset()
    for budget, chunks in ((0, 40), (25 << 30, 240), (40 << 30, 360), (40 * 10**9, 338)):
        m = MemoryManager(budget, device=-1)
        base, n, canon = m.pool_info()
        assert n == chunks and base == canon == 0x600000000000
        m.close()


def test_plan_only_engine_moves_no_bytes(built):
    repo_reset()
    m = MemoryManager(0, device=-1)
    ws = W.weight_set("bert_tiny")
    W.cold_start(m, "f", ws)
    p = m.dump_params("f")
    with pytest.raises(SwapError) as e:
        m.read_phys(int(p[0, 3]), 16)
    assert e.value.code == _cabi.ERR_NO_DEVICE
    with pytest.raises(SwapError):
        m.checksum_resident("f")
    # the host store is still the authoritative copy
    for i in (0, 7, len(ws.tensors) - 1):
        assert np.array_equal(m.read_host_store("f", int(p[i, 0]), int(p[i, 1])), W.tensor_bytes(ws, i))
    m.close()
    repo_reset()


def test_pool_exhaustion_is_an_error_not_an_exit(built):
    repo_reset()
    m = MemoryManager(0, device=-1)  # 40 chunks = 5 GiB
    ws = W.weight_set("llama_tiny")
    zeros = lambda i: np.zeros(ws.tensors[i].nbytes, dtype=np.uint8)
    with pytest.raises(SwapError) as e:
        for k in range(200):
            W.cold_start(m, f"f{k}", ws, tensor_data=zeros, workspace_blocks=(100 << 20,))
    assert e.value.code == _cabi.ERR_POOL_EXHAUSTED
    m.close()
    repo_reset()


def test_failed_swap_in_rolls_back(built):
    """A swap-in that does not fit leaves pool and tables as they were."""
    repo_reset()
    m = MemoryManager(0, device=-1)
    ws = W.weight_set("llama_tiny")
    zeros = lambda i: np.zeros(ws.tensors[i].nbytes, dtype=np.uint8)
    big = (100 << 20,) * 4
    n = 0
    W.cold_start(m, "victim", ws, tensor_data=zeros, workspace_blocks=big)
    m.evict("victim")
    try:
        while True:
            W.cold_start(m, f"f{n}", ws, tensor_data=zeros, workspace_blocks=big)
            n += 1
    except SwapError:
        pass
    before = m.dump_blocks("victim")
    with pytest.raises(SwapError) as e:
        m.swap_in("victim")
    assert e.value.code == _cabi.ERR_POOL_EXHAUSTED
    assert np.array_equal(before[:, 3], m.dump_blocks("victim")[:, 3])
    m.evict(f"f{n - 1}")
    m.evict(f"f{n - 2}")
    m.swap_in("victim")
    assert m.check_alloc("victim")
    m.close()
    repo_reset()


def test_small_irregular_request_takes_a_whole_slot(built):
    """Requests of 8 MiB or less that are not 2 MiB: the reference hands the chunk base out
    twice (block_manager.hpp:75-104 with a zero step); the engine gives each its own slot."""
    repo_reset()
    m = MemoryManager(0, device=-1)
    m.track_begin("f")
    a = m.malloc("f", 4 << 20, False)
    b = m.malloc("f", 6 << 20, False)
    c = m.malloc("f", 1 << 20, False)
    m.track_end("f")
    assert len({a, b, c}) == 3 and abs(a - b) >= (16 << 20) and abs(b - c) >= (16 << 20)
    m.close()
    repo_reset()


def test_unknown_model_and_bad_arguments(built):
    repo_reset()
    m = MemoryManager(0, device=-1)
    with pytest.raises(SwapError) as e:
        m.swap_in("nope")
    assert e.value.code == _cabi.ERR_UNKNOWN_MODEL
    with pytest.raises(SwapError) as e:
        m.evict("nope")
    assert e.value.code == _cabi.ERR_UNKNOWN_MODEL
    assert m.get_cuda_addr("nope", 0x1234) == 0x1234          # memory_manager.hpp:270
    m.track_begin("f")
    blk = m.malloc("f", 2 << 20, True)
    assert m.memcpy_h2d_model("f", blk + (4 << 20), np.zeros(16, np.uint8)) == _cabi.ERR_NOT_FOUND
    assert m.memcpy_h2d_model("f", blk + (2 << 20) - 8, np.zeros(16, np.uint8)) == _cabi.ERR_INVALID
    assert m.memcpy_h2d_model("f", blk, np.zeros(0, np.uint8)) == 0   # empty upload is a parameter of size 0
    assert m.mark_access(blk) == 1 and m.mark_access(blk + 64) == 0
    m.track_end("f")
    m.evict("f") if False else None
    m.close()
    repo_reset()


def test_swap_in_that_does_not_fit_leaves_nothing_behind():
    """Where the reference exits (block_manager.hpp:343-352) the engine refuses the swap-in: blocks it
    had taken go back to the pool, the model's table is what it was, and the pool serves the next
    swap-in as if the attempt had never been made."""
    from torpor_b200.memory_manager import MemoryManager, SwapError, repo_reset
    MiB = 1 << 20
    repo_reset()
    m = MemoryManager(0, device=-1, server_id=0, gpu_count=1)          # 40 chunks of 128 MiB

    def cold(f, n, size):
        m.track_begin(f)
        ptrs = [m.malloc(f, size, True) for _ in range(n)]
        for p in ptrs:
            m.memcpy_h2d_model(f, p, np.zeros(16, dtype=np.uint8))
        m.sync_done(f)
        for p in ptrs:
            m.mark_access(p)
        m.track_end(f)

    def spans(f):
        return {(int(r[4]), int(r[4] + r[1])) for r in m.dump_blocks(f, canonical=True) if r[3]}

    cold("A", 16, 128 * MiB); cold("B", 10, 128 * MiB); cold("S", 6, 2 * MiB)
    m.evict("A"); m.evict("B")
    cold("C", 16, 128 * MiB)
    m.swap_in("A")                                                      # 16 + 16 + 1 chunks in use, 7 free
    before_b, before_s = m.dump_blocks("B", canonical=True).copy(), spans("S")
    with pytest.raises(SwapError) as err:
        m.swap_in("B")                                                  # needs 10
    assert "POOL_EXHAUSTED" in str(err.value)
    assert np.array_equal(m.dump_blocks("B", canonical=True), before_b) and not m.check_alloc("B")
    m.evict("C")
    m.swap_in("B")                                                      # fits now
    assert m.check_alloc("B") and len(spans("B")) == 10
    live = [spans(f) for f in ("A", "B", "S")]
    assert spans("S") == before_s
    flat = sorted(x for s in live for x in s)
    assert all(flat[i][1] <= flat[i + 1][0] for i in range(len(flat) - 1)), "two live blocks overlap"
    with pytest.raises(SwapError):
        m.swap_in("C")                                                  # A 16 + B 10 + S 1 = 27 in use; C's 16 do not fit
    assert [spans(f) for f in ("A", "B", "S")] == live and not m.check_alloc("C")
    m.evict("A")
    m.swap_in("C")
    assert m.check_alloc("C") and len(spans("C")) == 16
    m.close(); repo_reset()


def test_guard_against_granting_a_blocks_name_again(monkeypatch):
    """A block is named by the first address it was given.  After an eviction that address is free, and
    the pool's LIFO order hands it straight to the function's next malloc: the reference then replaces
    the old block's entry with the new block (model_repo.hpp:133-141) and the model has lost a block.
    The engine does the same by default (the reference's decisions, one for one) and keeps both
    blocks with TORPOR_SWAP_GUARD_NAMES=1."""
    from torpor_b200.memory_manager import MemoryManager, repo_reset
    MiB = 1 << 20

    def run():
        repo_reset()
        m = MemoryManager(0, device=-1)
        m.track_begin("f")
        blocks = [m.malloc("f", 32 * MiB, True), m.malloc("f", 48 * MiB, True)]
        for b in blocks:
            m.memcpy_h2d_model("f", b + 4096, np.zeros(64, dtype=np.uint8))
        m.sync_done("f")
        for b in blocks:
            m.mark_access(b + 4096)
        m.track_end("f")
        m.evict("f")
        extra = m.malloc("f", 32 * MiB, False)          # a later request's workspace
        m.swap_in("f")
        table = m.dump_blocks("f")
        moved = [m.translate("f", b + 4096) for b in blocks]
        m.close(); repo_reset()
        return blocks, extra, table, moved

    monkeypatch.delenv("TORPOR_SWAP_GUARD_NAMES", raising=False)
    blocks, extra, table, moved = run()
    assert extra in blocks and len(table) == 2           # as the reference: the new block took a model block's place

    monkeypatch.setenv("TORPOR_SWAP_GUARD_NAMES", "1")
    blocks, extra, table, moved = run()
    assert extra not in blocks and len(table) == 3
    assert sorted(int(r[0]) for r in table) == sorted(blocks + [extra])
    spans = sorted((int(r[4]), int(r[4] + r[1])) for r in table if r[3])
    assert len(spans) == 3 and all(spans[i][1] <= spans[i + 1][0] for i in range(2))     # three live, disjoint blocks
    assert all(a != 0 for a in moved)


def test_full_size_llama_tables_equal_the_restatement(built, monkeypatch):
    """The 13.5 GB Llama-2-7B-shaped set at full size, tables only: the plan-only engine and the CPU
    restatement, both given sizes without bytes, agree word for word on the block and pointer
    tables of four swap-ins with evictions between (the placement changes from one to the next)."""
    import numpy as np
    from oracle import tso
    from torpor_b200 import workloads as W
    from torpor_b200.memory_manager import MemoryManager, SizeOnly, repo_reset
    monkeypatch.setenv("TORPOR_ORACLE_TABLES_ONLY", "1")
    ws = W.weight_set("llama2_7b")
    budget = W.pool_budget_for(ws)
    repo_reset()
    lib = tso.load("oracle")
    lib.reset_world()
    eng = MemoryManager(budget, device=-1)
    orc = lib.manager(budget=budget)
    sizes = lambda i: SizeOnly(ws.tensors[i].nbytes)
    W.cold_start(eng, "llama", ws, tensor_data=sizes)
    W.cold_start(orc, "llama", ws, tensor_data=sizes)
    seen = []
    for it in range(4):
        eng.evict("llama"); orc.evict("llama")
        eng.swap_in("llama"); orc.swap_in("llama")
        tab = eng.dump_params("llama", canonical=True)
        assert np.array_equal(tab, orc.dump_params("llama")), it
        assert np.array_equal(eng.dump_blocks("llama", canonical=True), orc.dump_blocks("llama")), it
        seen.append(tab)
    assert len(tab) == 291 and not np.array_equal(seen[0], seen[1])
    # and the helper the benchmark uses gives the same tables
    eng.close(); orc.close(); lib.reset_world(); repo_reset()
    replay = W.plan_tables(ws, "llama", budget=budget, swaps=4)
    for it in range(4):
        assert np.array_equal(replay[it][1], seen[it])
    repo_reset()
