"""Parity tests proper: the CUDA engine, through the C ABI, against the CPU checker and
the golden tables of the reference -- resident bytes, rebound pointer table, host bytes
after swap-out -- on the benchmark's weight sets."""
import ctypes
from concurrent.futures import ThreadPoolExecutor

import numpy as np
import pytest

import scenarios
from torpor_b200 import _cabi
from torpor_b200 import workloads as W
from torpor_b200.memory_manager import MemoryManager, ModelRepo, SwapError, checksum_host, repo_reset

pytestmark = pytest.mark.gpu

MiB = 1 << 20


@pytest.fixture(scope="module")
def gpu_backend(built):
    import torch
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    assert "libtorpor_swap.so" in _cabi.lib()._name
    return scenarios.EngineBackend(device=0)


@pytest.fixture()
def fresh(built):
    repo_reset()
    yield
    repo_reset()


# ---------------------------------------------------------------- tables

@pytest.mark.parametrize("name", list(scenarios.SCENARIOS))
def test_pointer_tables_match_reference_golden(gpu_backend, name):
    """Same scenarios as on the plan-only engine, now with real placement and the kernel
    publishing readiness: canonical tables equal the reference's word for word."""
    scenarios.assert_same(scenarios.run(gpu_backend, name), scenarios.load_golden(name), f"gpu/{name}")


# ---------------------------------------------------------------- bytes

def load_both(eng, orc, func, ws, **kw):
    """Cold start on the engine and on the checker; returns both address books."""
    return W.cold_start(eng, func, ws, **kw), W.cold_start(orc, func, ws, **kw)


def assert_resident_equal(eng, orc, func, ws, full=True):
    """Pointer table equal to the checker's, bytes at every translated address equal to the
    bytes the checker holds at the corresponding address."""
    tab = eng.dump_params(func, canonical=True)
    want = orc.dump_params(func)
    assert np.array_equal(tab, want)
    assert np.array_equal(eng.dump_blocks(func, canonical=True), orc.dump_blocks(func))
    phys = eng.dump_params(func)
    if full:
        for i in range(len(phys)):
            n = int(phys[i, 1])
            have = eng.read_phys(eng.get_cuda_addr(func, int(phys[i, 0])), n)
            assert np.array_equal(have, orc.read_phys(int(want[i, 3]), n)), f"tensor {i}"
    sums = eng.checksum_resident(func)
    for i in range(len(phys)):
        ref = checksum_host(orc.read_phys(int(want[i, 3]), int(want[i, 1])))
        assert np.array_equal(sums[i], ref), f"checksum of tensor {i}"


def test_config1_resnet50_swap_in(fresh, oracle_backend):
    """ResNet-50 fp32 set (161 tensors, 102,228,128 B): host store -> 2 MiB-block pool with rebind."""
    oracle_backend.reset()
    ws = W.weight_set("resnet50")
    eng, orc = MemoryManager(0, device=0), oracle_backend.manager(budget=0)
    load_both(eng, orc, "r50", ws)
    assert_resident_equal(eng, orc, "r50", ws)           # after cold start
    for _ in range(2):
        eng.evict("r50"); orc.evict("r50")
        eng.swap_in("r50"); eng.wait_ready("r50"); orc.swap_in("r50")
        assert_resident_equal(eng, orc, "r50", ws)
    st = eng.stats()
    assert st["kernel_launches"] >= 2 and st["bytes_moved"] >= 2 * ws.nbytes
    eng.close()
    oracle_backend.reset()


def test_config2_bert_base_round_trip(fresh, oracle_backend):
    """BERT-base fp32 set: swap-in, then swap-out with write-back; bit-exact both ways.  The
    reference's swap-out moves nothing, so host bytes after it are the uploaded bytes."""
    oracle_backend.reset()
    ws = W.weight_set("bert_base")
    eng, orc = MemoryManager(0, device=0), oracle_backend.manager(budget=0)
    lm, lm_orc = load_both(eng, orc, "bert", ws)
    eng.evict("bert"); orc.evict("bert")
    eng.swap_in("bert"); eng.wait_ready("bert"); orc.swap_in("bert")
    assert_resident_equal(eng, orc, "bert", ws)
    eng.evict("bert", writeback=True); orc.evict("bert")
    assert np.array_equal(eng.dump_params("bert", canonical=True), orc.dump_params("bert"))
    for i, (v, v_orc) in enumerate(zip(lm.tensor_vaddr, lm_orc.tensor_vaddr)):
        n = ws.tensors[i].nbytes
        assert np.array_equal(eng.read_host_store("bert", v, n), orc.read_host_store("bert", v_orc, n)), f"tensor {i}"
    eng.swap_in("bert"); eng.wait_ready("bert"); orc.swap_in("bert")
    assert_resident_equal(eng, orc, "bert", ws, full=False)
    eng.close()
    oracle_backend.reset()


def test_writeback_carries_device_side_changes(fresh):
    """The write-back kernel really moves resident bytes: change a tensor on the device,
    evict with write-back, and the host store (and the next swap-in) shows the change."""
    ws = W.weight_set("bert_tiny")
    eng = MemoryManager(0, device=0)
    lm = W.cold_start(eng, "f", ws)
    k = 9
    new = (np.arange(ws.tensors[k].nbytes) % 251).astype(np.uint8)
    assert eng.cudaMemcpyAsyncBackendHtoD(lm.tensor_vaddr[k], new, 0, False, "f") == 0
    eng.evict("f", writeback=False)                       # the reference's swap-out: change is lost
    assert np.array_equal(eng.read_host_store("f", lm.tensor_vaddr[k], new.size), W.tensor_bytes(ws, k))
    eng.swap_in("f"); eng.wait_ready("f")
    assert eng.cudaMemcpyAsyncBackendHtoD(lm.tensor_vaddr[k], new, 0, False, "f") == 0
    eng.evict("f", writeback=True)
    assert np.array_equal(eng.read_host_store("f", lm.tensor_vaddr[k], new.size), new)
    assert np.array_equal(eng.read_host_store("f", lm.tensor_vaddr[k + 1], 64), W.tensor_bytes(ws, k + 1)[:64])
    eng.swap_in("f"); eng.wait_ready("f")
    assert np.array_equal(eng.read_phys(eng.get_cuda_addr("f", lm.tensor_vaddr[k]), new.size), new)
    eng.close()


def test_config3_bert_large_fp16(fresh, oracle_backend):
    oracle_backend.reset()
    ws = W.weight_set("bert_large")
    eng, orc = MemoryManager(0, device=0), oracle_backend.manager(budget=0)
    load_both(eng, orc, "bl", ws)
    eng.evict("bl"); orc.evict("bl")
    eng.swap_in("bl"); eng.wait_ready("bl"); orc.swap_in("bl")
    assert_resident_equal(eng, orc, "bl", ws, full=False)
    eng.close()
    oracle_backend.reset()


def test_replica_swap_on_device(fresh, oracle_backend):
    """Swap-in from a resident replica held by a second engine (the reference's GPU-to-GPU
    path, memory_manager.hpp:394-396); both engines sit on cuda:0 here."""
    oracle_backend.reset()
    ws = W.weight_set("llama_tiny")
    a, b = MemoryManager(0, device=0, server_id=0, gpu_count=2), MemoryManager(0, device=0, server_id=1, gpu_count=2)
    oa, ob = oracle_backend.manager(server_id=0, budget=0, gpu_count=2), oracle_backend.manager(server_id=1, budget=0, gpu_count=2)
    W.cold_start(b, "m", ws); W.cold_start(ob, "m", ws)
    ModelRepo.add_model_info("m", 1); oracle_backend.set_status("m", 1, True)
    a.swap_in("m", 1); a.wait_ready("m"); oa.swap_in("m", 1)
    assert_resident_equal(a, oa, "m", ws)
    assert ModelRepo.active_devices("m") == [1]
    a.close(); b.close()
    oracle_backend.reset()


def test_unaccessed_parameters_are_not_moved(fresh):
    """Only parameters the first run touched travel (memory_manager.hpp:356,378); the others
    translate to their rebound address, which holds whatever the pool block held."""
    ws = W.weight_set("bert_tiny")
    eng = MemoryManager(0, device=0)
    data = lambda i: np.full(ws.tensors[i].nbytes, 1 + i % 200, dtype=np.uint8)
    lm = scenarios.cold_start_partial(eng, "f", ws, data, (2 * MiB,), lambda i: i % 2 == 0)
    eng.evict("f")
    other = W.cold_start(eng, "g", W.weight_set("bert_tiny"), tensor_data=lambda i: np.zeros(ws.tensors[i].nbytes, np.uint8))
    eng.evict("g")
    eng.swap_in("f"); eng.wait_ready("f")
    tab = eng.dump_params("f")
    moved = 0
    for row in tab:
        i = lm.tensor_vaddr.index(int(row[0]))
        got = eng.read_phys(eng.get_cuda_addr("f", int(row[0])), int(row[1]))
        if i % 2 == 0:
            assert row[4] == _cabi.READY_CUDA and np.array_equal(got, data(i))
            moved += int(row[1])
        else:
            assert row[4] == _cabi.READY_HOST and row[6] == 0
    assert moved == sum(t.nbytes for i, t in enumerate(ws.tensors) if i % 2 == 0)
    eng.close()


def test_llama_shaped_blocks_beyond_a_chunk(fresh, oracle_backend):
    """Llama-shaped set with tensors larger than a 128 MiB chunk (embedding / lm_head, 250 MiB):
    the reference leaves the pool for them (block_manager.hpp:295-300); tables still agree,
    bytes are checked by checksum, and repeated cycles reuse instead of leaking."""
    oracle_backend.reset()
    ws = W.weight_set("llama_mid")
    eng, orc = MemoryManager(0, device=0), oracle_backend.manager(budget=0)
    pool = ThreadPoolExecutor(8)
    data = list(pool.map(lambda i: W.tensor_bytes(ws, i), range(len(ws.tensors))))
    W.cold_start(eng, "l", ws, tensor_data=lambda i: data[i])
    W.cold_start(orc, "l", ws, tensor_data=lambda i: data[i])
    host_sums = np.array([checksum_host(d) for d in data])
    import torch
    free0 = None
    for it in range(3):
        eng.evict("l", writeback=(it == 1)); orc.evict("l")
        eng.swap_in("l"); eng.wait_ready("l"); orc.swap_in("l")
        assert np.array_equal(eng.dump_params("l", canonical=True), orc.dump_params("l"))
        assert np.array_equal(eng.dump_blocks("l", canonical=True), orc.dump_blocks("l"))
        assert np.array_equal(eng.checksum_resident("l"), host_sums)
        free = torch.cuda.mem_get_info()[0]
        if free0 is None:
            free0 = free
        assert free >= free0 - 64 * MiB, "device memory keeps shrinking across swap cycles"
    eng.close()
    oracle_backend.reset()


# ---------------------------------------------------------------- the mover alone

def test_placement_kernel_alignments_and_ragged_sizes(fresh):
    """Every head/tail/width path of the kernel: all 16 relative alignments of source and
    destination, sizes from 0 to a few tiles, with guard bytes on both sides."""
    import torch
    eng = MemoryManager(0, device=0)
    rng = np.random.default_rng(5)
    sizes = [0, 1, 2, 3, 15, 16, 17, 31, 255, 4096, 4097, 65535, 65536, 65537, 200001]
    span = 256 * 1024
    n = len(sizes) * 16
    src_host = torch.from_numpy(rng.integers(0, 256, size=n * span, dtype=np.uint8))
    src = src_host.cuda()
    dst = torch.full((n * span,), 0xEE, dtype=torch.uint8, device="cuda")
    s_list, d_list, b_list = [], [], []
    k = 0
    for size in sizes:
        for rel in range(16):
            so = k * span + 64 + (rel * 7) % 16
            do = k * span + 64 + (rel * 11 + 5) % 16
            s_list.append(src.data_ptr() + so); d_list.append(dst.data_ptr() + do); b_list.append(size)
            k += 1
    eng.place_segments(s_list, d_list, b_list, tile_bytes=65536)
    out = dst.cpu().numpy()
    inp = src_host.numpy()
    want = np.full(n * span, 0xEE, dtype=np.uint8)
    for s, d, b in zip(s_list, d_list, b_list):
        so, do = s - src.data_ptr(), d - dst.data_ptr()
        want[do:do + b] = inp[so:so + b]
    assert np.array_equal(out, want)
    eng.close()


def test_tiles_dealt_to_several_launches_publish_once(fresh):
    """Sharding primitive: the same segment list run as 3 strided launches covers every byte
    exactly once, and each row of the pointer table is published by whoever finishes last."""
    import torch
    eng = MemoryManager(0, device=0)
    rng = np.random.default_rng(6)
    sizes = [5, 70000, 1 << 20, 333333, 16, (3 << 20) + 48]
    offs = np.cumsum([0] + [((s + 511) // 512) * 512 for s in sizes])
    total = int(offs[-1])
    src = torch.from_numpy(rng.integers(0, 256, size=total, dtype=np.uint8)).cuda()
    dst = torch.zeros(total, dtype=torch.uint8, device="cuda")
    done = torch.zeros(len(sizes), dtype=torch.int32, device="cuda")
    t_phys = torch.zeros(len(sizes), dtype=torch.int64, device="cuda")
    t_flag = torch.zeros(len(sizes), dtype=torch.int32, device="cuda")
    pub = _cabi.Publish(done.data_ptr(), t_phys.data_ptr(), t_flag.data_ptr(), 0, 0, _cabi.READY_CUDA, 0)
    s_list = [src.data_ptr() + int(o) for o in offs[:-1]]
    d_list = [dst.data_ptr() + int(o) for o in offs[:-1]]
    for r in range(3):
        eng.place_segments(s_list, d_list, sizes, tile_bytes=65536, tile_first=r, tile_stride=3, publish=pub)
        if r < 2:
            assert int(t_flag[2].item()) == 0          # the 1 MiB segment has tiles in every share
    for o, s in zip(offs[:-1], sizes):
        assert torch.equal(dst[int(o):int(o) + s], src[int(o):int(o) + s])
    assert t_flag.tolist() == [_cabi.READY_CUDA] * len(sizes)
    assert t_phys.tolist() == d_list
    assert done.tolist() == [0] * len(sizes)           # counters re-arm themselves
    eng.close()


@pytest.mark.parametrize("name,static", [("resnet50", False), ("llama_tiny", True)])
def test_sharded_swap_with_the_helper_engines_on_this_gpu(fresh, oracle_backend, name, static):
    """The sharded swap-in of the multi-GPU tests on a box with one GPU: the target and three helper
    engines (server ids 0-3) all sit on device 0, so the whole mechanism runs -- four launches
    of the placement kernel on four streams, tiles drawn from the counter on the target (or dealt
    t mod 4), system-scope tile counters, each row published once by whichever launch finishes
    it -- only the links are not separate.  No launch waits for another, so they may run in any
    order or one after the other.  Result: the single-GPU table of the checker, and the bytes."""
    n = 4
    oracle_backend.reset()
    ws = W.weight_set(name)
    engines = [MemoryManager(0, device=0, server_id=d, gpu_count=n, shard_static=static,
                             host_arena_bytes=(W.host_store_bytes(ws) if d == 0 else 0))
               for d in range(n)]
    orc = oracle_backend.manager(budget=0, gpu_count=n)
    W.cold_start(engines[0], "m", ws); W.cold_start(orc, "m", ws)
    sums = np.array([checksum_host(W.tensor_bytes(ws, i)) for i in range(len(ws.tensors))])
    for cycle in range(3):
        engines[0].evict("m"); orc.evict("m")
        engines[0].swap_in_sharded("m", engines[1:]); engines[0].wait_ready("m"); orc.swap_in("m")
        assert np.array_equal(engines[0].dump_params("m", canonical=True), orc.dump_params("m"))
        assert np.array_equal(engines[0].dump_blocks("m", canonical=True), orc.dump_blocks("m"))
        assert np.array_equal(engines[0].checksum_resident("m"), sums)
    for d in range(1, n):
        assert engines[d].stats()["kernel_launches"] == 3       # every helper took part in every cycle, one launch each
    # and a plain swap-in on the target afterwards starts from clean tile counters
    engines[0].evict("m"); orc.evict("m")
    engines[0].swap_in("m"); engines[0].wait_ready("m"); orc.swap_in("m")
    assert np.array_equal(engines[0].dump_params("m", canonical=True), orc.dump_params("m"))
    assert np.array_equal(engines[0].checksum_resident("m"), sums)
    for e in engines:
        e.close()
    oracle_backend.reset()


def test_more_segments_than_the_launch_scratch_holds_at_first(fresh):
    """A raw segment list longer than the engine's initial launch scratch (4096 entries) makes the
    scratch grow; the host store and the rest of the engine must come through that untouched."""
    import torch
    ws = W.weight_set("bert_tiny")
    eng = MemoryManager(0, device=0)
    lm = W.cold_start(eng, "m", ws)
    n, piece = 6000, 1040                                  # 16-byte multiples, not a power of two
    rng = np.random.default_rng(8)
    src = torch.from_numpy(rng.integers(0, 256, size=n * piece, dtype=np.uint8)).cuda()
    dst = torch.zeros(n * piece, dtype=torch.uint8, device="cuda")
    order = rng.permutation(n)
    s_list = [src.data_ptr() + int(i) * piece for i in order]
    d_list = [dst.data_ptr() + int(k) * piece for k in range(n)]
    eng.place_segments(s_list, d_list, [piece] * n, tile_bytes=4096)
    want = src.cpu().numpy().reshape(n, piece)[order].reshape(-1)
    assert np.array_equal(dst.cpu().numpy(), want)
    eng.place_segments(s_list[:10], d_list[:10], [piece] * 10, tile_bytes=4096)      # and the grown scratch is reused
    # the model the engine holds still swaps in bit-exact afterwards
    eng.evict("m"); eng.swap_in("m"); eng.wait_ready("m")
    sums = np.array([checksum_host(W.tensor_bytes(ws, i)) for i in range(len(ws.tensors))])
    assert np.array_equal(eng.checksum_resident("m"), sums)
    eng.close()


# ---------------------------------------------------------------- bounded waits, errors

def test_waits_are_bounded(fresh):
    ws = W.weight_set("bert_tiny")
    eng = MemoryManager(0, device=0)
    W.cold_start(eng, "f", ws)
    eng.evict("f")
    with pytest.raises(SwapError) as e:
        eng.wait_ready("f", timeout_ns=20_000_000)      # nothing was asked to swap in
    assert e.value.code == _cabi.ERR_TIMEOUT
    eng.swap_in("f"); eng.wait_ready("f")                # engine still usable
    assert eng.check_alloc("f")
    eng.close()


def test_full_size_llama2_7b_properties(fresh):
    """The 13.5 GB Llama-2-7B-shaped set at full size: per-tensor checksums of the resident
    bytes equal the host-side checksums after swap-in, every parameter is rebound into the
    placed blocks, write-back leaves the host store unchanged, and a second cycle lands on
    the same tables (idempotence)."""
    ws = W.weight_set("llama2_7b")
    eng = MemoryManager(12 << 30, device=0, host_arena_bytes=14 << 30)
    sums = {}

    def data(i):
        b = W.tensor_bytes(ws, i)
        sums[i] = checksum_host(b)
        return b

    with ThreadPoolExecutor(12) as pool:
        cache = {}
        futs = {i: pool.submit(data, i) for i in range(len(ws.tensors))}
        lm = W.cold_start(eng, "llama", ws, tensor_data=lambda i: futs.pop(i).result())
    host_sums = np.array([sums[i] for i in range(len(ws.tensors))])
    assert np.array_equal(eng.checksum_resident("llama"), host_sums)
    tables = []
    for it in range(2):
        eng.evict("llama", writeback=(it == 0))
        eng.swap_in("llama"); eng.wait_ready("llama")
        tab = eng.dump_params("llama", canonical=True)
        blk = eng.dump_blocks("llama", canonical=True)
        assert (tab[:, 4] == _cabi.READY_CUDA).all() and (tab[:, 3] == tab[:, 5]).all()
        starts = {int(b[0]): (int(b[4]), int(b[1])) for b in blk}
        for row in tab:                                   # rebind: same offset inside the new block
            cuda, size = starts[int(row[2])]
            assert int(row[3]) - cuda == int(row[0]) - int(row[2]) and int(row[3]) + int(row[1]) <= cuda + size
        assert np.array_equal(eng.checksum_resident("llama"), host_sums)
        tables.append((tab, blk))
    assert eng.stats()["bytes_moved"] >= 3 * ws.nbytes
    # ... and the tables of both swap-ins equal the CPU checker's, word for word, at full size: the
    # checker replays the same calls holding tables only (no parameter byte is stored or moved)
    import os
    from oracle import tso
    from torpor_b200.memory_manager import SizeOnly
    os.environ["TORPOR_ORACLE_TABLES_ONLY"] = "1"
    try:
        orc_lib = tso.load("oracle")
        orc_lib.reset_world()
        orc = orc_lib.manager(budget=12 << 30)
        W.cold_start(orc, "llama", ws, tensor_data=lambda i: SizeOnly(ws.tensors[i].nbytes))
        for it in range(2):
            orc.evict("llama")
            orc.swap_in("llama")
            assert np.array_equal(tables[it][0], orc.dump_params("llama")), f"pointer table of swap-in {it}"
            assert np.array_equal(tables[it][1], orc.dump_blocks("llama")), f"block table of swap-in {it}"
        orc.close()
        orc_lib.reset_world()
    finally:
        del os.environ["TORPOR_ORACLE_TABLES_ONLY"]
    # host store untouched by the write-back of unmodified weights
    for i in (0, 1, 150, 290):
        v, n = lm.tensor_vaddr[i], min(ws.tensors[i].nbytes, 1 << 20)
        assert np.array_equal(eng.read_host_store("llama", v, n), W.tensor_bytes(ws, i)[:n])
    eng.close()


def test_mixed_request_stream_with_eviction(fresh):
    """A short serverless stream (Zipf popularity, Poisson arrivals) over two engines with a
    memory cap small enough to force LRU evictions: every request completes, swaps come both
    from the host store and from replicas, and evicted models come back bit-exact."""
    from torpor_b200 import serving
    out = serving.run_stream(n_gpus=2, n_models=10, rate=300.0, duration_s=2.0, cap_bytes=300 << 20, seed=4,
                             archs=("bert_tiny", "llama_tiny", "resnet50"), devices=[0, 0], zero_weights=True)
    assert out["completed"] == out["requests"] > 400
    assert out["swaps"] > 20 and out["evictions_in_service"] > 5
    assert out["swaps_from_host"] > 0 and out["swap_ms_p99"] < 2000
    assert out["sustained_swap_gbs"] > 0.1

    # the same machinery with real weights: after churn the survivor's bytes are still right
    srv = serving.SwapServer(2, 190 << 20, devices=[0, 0])
    for i, a in enumerate(["resnet50", "llama_tiny", "resnet50", "llama_tiny"]):
        srv.cold_start(f"fn{i}", a, 50 + i)
    for f in ["fn0", "fn1", "fn2", "fn3", "fn0", "fn2", "fn1"]:
        srv.submit(f, 0.0)
        while srv.busy():
            srv.poll()
    ws = W.weight_set("llama_tiny", seed=51)
    homes = ModelRepo.active_devices("fn1")
    assert homes, "fn1 should be resident somewhere after its last request"
    eng = srv.engines[homes[0]]
    sums = np.array([checksum_host(W.tensor_bytes(ws, i)) for i in range(len(ws.tensors))])
    assert np.array_equal(eng.checksum_resident("fn1"), sums)
    assert srv.evictions > 0
    srv.close()


def test_stream_ordered_translation(fresh):
    """get_cuda_addr without blocking the host: the address comes back at once, the caller's
    stream waits on the pointer table's generation word, and work enqueued behind it sees the
    parameter's bytes -- not what the pool block held before."""
    import torch
    from torpor_b200.memory_manager import place_segments_static
    ws_a, ws_b = W.weight_set("bert_base", seed=101), W.weight_set("bert_base", seed=202)
    eng = MemoryManager(0, device=0)
    la = W.cold_start(eng, "A", ws_a)
    eng.evict("A")
    lb = W.cold_start(eng, "B", ws_b)
    last = len(ws_a.tensors) - 2                       # pooler weight: near the end of the access order
    n = ws_a.tensors[last].nbytes
    stream = torch.cuda.Stream()
    scratch = torch.zeros(n, dtype=torch.uint8, device="cuda")
    waited_any = False
    for cycle in range(3):
        eng.evict("B")                                  # B's bytes stay behind in the freed blocks
        eng.swap_in("A")                                # asynchronous
        addr, waited = eng.get_cuda_addr_async("A", la.tensor_vaddr[last], stream.cuda_stream)
        waited_any = waited_any or waited
        place_segments_static(0, [addr], [scratch.data_ptr()], [n], stream=stream.cuda_stream)
        stream.synchronize()
        assert np.array_equal(scratch.cpu().numpy(), W.tensor_bytes(ws_a, last)), f"cycle {cycle}"
        assert addr == eng.get_cuda_addr("A", la.tensor_vaddr[last])
        eng.wait_ready("A")
        eng.evict("A")
        eng.swap_in("B"); eng.wait_ready("B")
        addr_b, waited_b = eng.get_cuda_addr_async("B", lb.tensor_vaddr[last], stream.cuda_stream)
        assert not waited_b                             # already resident: no wait is enqueued
    assert waited_any, "the last parameter was never still in flight when asked for"
    eng.evict("B")
    with pytest.raises(SwapError) as e:                 # nothing in flight: a wait could never be satisfied
        eng.get_cuda_addr_async("B", lb.tensor_vaddr[last], stream.cuda_stream)
    assert e.value.code == _cabi.ERR_STATE
    eng.close()


def _drained(stream, seconds):
    """Poll a stream (never block on it) until it has run dry or `seconds` have passed."""
    import time
    deadline = time.perf_counter() + seconds
    while time.perf_counter() < deadline:
        if stream.query():
            return True
        time.sleep(0.002)
    return stream.query()


def test_stream_ordered_wait_is_let_go_when_the_swap_never_completes(fresh):
    """The wait that tsw_translate_async enqueues has a way out.  A swap is planned (blocks placed,
    table rebound, rows handed out) but nobody moves its tiles, so the generation word is never
    written by a kernel.  When the whole-model wait gives up, the host writes the word: the stream
    drains, the work queued behind the wait runs, and translation and polling report the row as
    failed until the model is swapped in for real.  Nothing spins on the device, and whatever an
    assertion says, the teardown lets the stream go before anything blocks on it."""
    import time
    import torch
    ws = W.weight_set("bert_base", seed=77)
    eng = MemoryManager(0, device=0)
    lm = W.cold_start(eng, "A", ws)
    eng.evict("A")
    last = len(ws.tensors) - 2
    vaddr = lm.tensor_vaddr[last]
    stream = torch.cuda.Stream()
    marker = torch.zeros(1, dtype=torch.int32, device="cuda")
    # The kernel that will sit behind the wait is launched once beforehand: the first launch of a
    # kernel loads its module, which synchronises the whole device -- behind a pending wait that
    # would never return.  (True of any stream-ordered wait, whoever enqueues it.)
    with torch.cuda.stream(stream):
        marker.add_(1)
        marker.sub_(1)
    torch.cuda.synchronize()
    assert int(marker.cpu()[0]) == 0
    try:
        segs, tile, pub = eng.swap_plan("A")            # planned; no tile will ever be moved
        assert len(segs) > 0
        addr, waited = eng.get_cuda_addr_async("A", vaddr, stream.cuda_stream)
        assert waited and addr != 0
        with torch.cuda.stream(stream):
            marker.add_(1)                              # queued behind the wait
        time.sleep(0.05)
        assert not stream.query(), "the stream did not wait for the parameter"
        with pytest.raises(SwapError) as e:             # the bound: the whole-model wait runs out ...
            eng.wait_ready("A", timeout_ns=50_000_000)
        assert e.value.code == _cabi.ERR_TIMEOUT
        assert _drained(stream, 5.0), "the waiting stream was not let go"      # ... and takes the waiters with it
        assert int(marker.cpu()[0]) == 1
        with pytest.raises(SwapError) as e:             # the row is known to have failed
            eng.get_cuda_addr("A", vaddr)
        assert e.value.code == _cabi.ERR_KERNEL
        with pytest.raises(SwapError) as e:
            eng.poll_ready("A")
        assert e.value.code == _cabi.ERR_KERNEL
        # a second waiter, let go on request this time
        addr2, waited2 = None, False
        with pytest.raises(SwapError) as e:             # a failed row takes no new waiters
            eng.get_cuda_addr_async("A", vaddr, stream.cuda_stream)
        assert e.value.code == _cabi.ERR_KERNEL
    finally:
        eng.release_waiters("A")                        # unconditionally: no stream stays behind a wait
        eng.swap_in("A")                                # the real swap: generations only grow, so it satisfies any wait
        eng.wait_ready("A")
        assert _drained(stream, 5.0)
    # after the real swap the parameter is there, and translation works again
    got = eng.read_phys(eng.get_cuda_addr("A", vaddr), ws.tensors[last].nbytes)
    assert np.array_equal(got, W.tensor_bytes(ws, last))
    assert eng.poll_ready("A") == 0
    # eviction lets waiters of an abandoned plan go as well
    eng.evict("A")
    eng.swap_plan("A")
    addr, waited = eng.get_cuda_addr_async("A", vaddr, stream.cuda_stream)
    assert waited
    eng.evict("A")
    assert _drained(stream, 5.0), "eviction left a stream waiting"
    eng.close()


def test_bulk_copy_mover_is_bit_exact(fresh):
    """The opt-in bulk-copy mover (cp.async.bulk through shared memory, one thread per CTA)
    moves the same bytes and publishes the same table as the load/store kernel: swap-in from
    the host store, replica swap, write-back, and the sharded dealing by tickets."""
    import torch
    ws = W.weight_set("llama_tiny")
    sums = np.array([checksum_host(W.tensor_bytes(ws, i)) for i in range(len(ws.tensors))])
    tables = []
    for mover in (0, 1):
        repo_reset()
        b = MemoryManager(0, device=0, server_id=1, gpu_count=2, mover=mover)
        a = MemoryManager(0, device=0, server_id=0, gpu_count=2, mover=mover)
        lm = W.cold_start(b, "m", ws)
        ModelRepo.add_model_info("m", 1)
        for src in (-1, 1):
            a.swap_in("m", src); a.wait_ready("m")
            assert np.array_equal(a.checksum_resident("m"), sums), (mover, src)
            tables.append(a.dump_params("m", canonical=True))
            a.evict("m")
        a.swap_in_sharded("m", [b]); a.wait_ready("m")        # two engines draw tiles from one counter
        assert np.array_equal(a.checksum_resident("m"), sums)
        new = (np.arange(ws.tensors[3].nbytes) % 199).astype(np.uint8)
        v = lm.tensor_vaddr[3]
        assert a.cudaMemcpyAsyncBackendHtoD(v, new, 0, False, "m") == 0
        torch.cuda.synchronize()
        a.evict("m", writeback=True)
        assert np.array_equal(a.read_host_store("m", v, new.size), new)
        assert a.stats()["kernel_launches"] >= 5
        a.close(); b.close()
    assert np.array_equal(tables[0], tables[2]) and np.array_equal(tables[1], tables[3])


def test_copy_engine_assisted_mover_is_bit_exact(fresh, oracle_backend):
    """mover = 2: on a swap-in from the host store the parameters of 4 MiB and more are moved by the
    copy engine (a publish kernel behind each), the smaller ones by the placement kernel at the same
    time.  Bytes, tables and readiness equal the checker's, cycle after cycle, and a replica swap or
    a sharded swap on the same engine still goes through the kernel alone."""
    oracle_backend.reset()
    ws = W.weight_set("bert_large")
    sizes = [t.nbytes for t in ws.tensors]
    assert min(sizes) < (4 << 20) <= max(sizes)                 # both movers get work
    eng = MemoryManager(0, device=0, server_id=0, gpu_count=2, mover=2)
    peer = MemoryManager(0, device=0, server_id=1, gpu_count=2, mover=2)
    orc = oracle_backend.manager(budget=0, gpu_count=2)
    lm, _ = load_both(eng, orc, "m", ws)
    for cycle in range(3):
        eng.evict("m"); orc.evict("m")
        eng.swap_in("m"); orc.swap_in("m")
        # the launch path first: every parameter waits for its own row
        for v in lm.tensor_vaddr:
            assert eng.get_cuda_addr("m", v) != 0
        eng.wait_ready("m")
        assert_resident_equal(eng, orc, "m", ws, full=(cycle == 0))
    launches = eng.stats()["kernel_launches"]
    big = sum(1 for n in sizes if n >= (4 << 20))
    assert launches >= 3 * (big + 1)                            # one publish kernel per large parameter + the mover, per swap-in
    # the other sources are untouched by the setting
    ModelRepo.add_model_info("m", 0)
    peer.swap_in("m", 0); peer.wait_ready("m")
    sums = np.array([checksum_host(W.tensor_bytes(ws, i)) for i in range(len(ws.tensors))])
    assert np.array_equal(peer.checksum_resident("m"), sums)
    peer.evict("m")
    eng.evict("m", writeback=True)
    eng.swap_in_sharded("m", [peer]); eng.wait_ready("m")
    assert np.array_equal(eng.checksum_resident("m"), sums)
    eng.close(); peer.close()
    oracle_backend.reset()


def test_pipelined_mover_is_bit_exact(fresh):
    """tsw_place_segments_pipelined: copy engine host -> this GPU's staging area, chunk by chunk, and the
    placement kernel staging -> destination behind it.  Ragged segments, odd alignments, a tile range
    that starts and ends inside segments, chunks smaller than a segment and chunks spanning several:
    the bytes inside the range arrive, nothing outside it is touched, and rows complete when the
    remaining tiles are moved by the ordinary entry point."""
    import torch
    rng = np.random.default_rng(31)
    sizes = [int(x) for x in rng.choice([1, 7, 16, 100, 4096, 65536, 65537, 300000, 1 << 20, 3 << 20], size=60)]
    span = [((s + 15) // 16) * 16 + 64 for s in sizes]
    offs = np.concatenate([[0], np.cumsum(span)]).astype(np.int64)
    total = int(offs[-1]) + 64
    host = torch.from_numpy(rng.integers(0, 256, size=total, dtype=np.uint8)).pin_memory()
    shift = [int(x) for x in rng.integers(0, 16, size=len(sizes))]
    s_off = [int(offs[i]) + 16 + shift[i] for i in range(len(sizes))]
    d_off = [int(offs[i]) + 32 + shift[i] for i in range(len(sizes))]
    tile = 64 * 1024
    n_tiles = sum((s + tile - 1) // tile for s in sizes)
    eng = MemoryManager(0, device=0)
    inp = host.numpy()
    from torpor_b200.memory_manager import make_segments
    for lo, hi, chunk in ((0, 0, 5), (7, n_tiles - 9, 3), (n_tiles // 3, 2 * n_tiles // 3, 64)):
        hi_eff = hi if hi else n_tiles
        dst = torch.full((total,), 0xA5, dtype=torch.uint8, device="cuda")
        done = torch.zeros(len(sizes), dtype=torch.int32, device="cuda")
        t_phys = torch.zeros(len(sizes), dtype=torch.int64, device="cuda")
        t_flag = torch.zeros(len(sizes), dtype=torch.int32, device="cuda")
        pub = _cabi.Publish(done.data_ptr(), t_phys.data_ptr(), t_flag.data_ptr(), 0, 0, _cabi.READY_CUDA, 0)
        segs = make_segments([host.data_ptr() + o for o in s_off], [dst.data_ptr() + o for o in d_off], sizes, list(range(len(sizes))))
        torch.cuda.synchronize()
        eng.place_segment_array_pipelined(segs, tile, lo, hi, pub, chunk_tiles=chunk, sync=True)
        got = dst.cpu().numpy()
        want = np.full(total, 0xA5, dtype=np.uint8)
        t = 0
        for so, do, n in zip(s_off, d_off, sizes):
            for k in range((n + tile - 1) // tile):
                if lo <= t < hi_eff:
                    a, b = k * tile, min(n, (k + 1) * tile)
                    want[do + a:do + b] = inp[so + a:so + b]
                t += 1
        assert np.array_equal(got, want), (lo, hi, chunk)
        # the rest of the tiles through the ordinary entry point: now every row completes and is published
        if lo > 0:
            eng.place_segment_array(segs, tile, 0, 1, lo, pub, sync=True)
        if hi_eff < n_tiles:
            eng.place_segment_array(segs, tile, hi_eff, 1, 0, pub, sync=True)
        full = np.full(total, 0xA5, dtype=np.uint8)
        for so, do, n in zip(s_off, d_off, sizes):
            full[do:do + n] = inp[so:so + n]
        assert np.array_equal(dst.cpu().numpy(), full)
        assert (t_flag.cpu().numpy() == _cabi.READY_CUDA).all() and (done.cpu().numpy() == 0).all()
        assert np.array_equal((t_phys - dst.data_ptr()).cpu().numpy(), np.array(d_off))
    assert eng.stats()["kernel_launches"] > 10
    eng.close()


def test_topology_discovery_on_this_box(fresh):
    """tsw_topology_discover on however many GPUs the box has (one is enough): a PCIe uplink group
    per GPU, a link class per ordered pair, nothing on the diagonal -- and tables the scheduler and
    controller accept in place of the reference's 4-GPU constants (controller.hpp:116-118)."""
    import torch
    from torpor_b200.memory_manager import Scheduler, discover_topology
    n = torch.cuda.device_count()
    pairs, nv = discover_topology(n)
    assert len(pairs) == n and all(0 <= p < n for p in pairs)
    assert len(nv) == n and all(len(r) == n for r in nv)
    assert all(nv[i][i] == 0 for i in range(n))
    assert all(nv[i][j] in (-1, 1, 2) for i in range(n) for j in range(n) if i != j)
    for policy in ("IA", "Random"):
        s = Scheduler(n, policy, pairs, nv)
        gpu, src = s.decide("never_seen")[:2]
        assert 0 <= gpu < n and src == -1                     # a function no GPU holds: a cold start, no source
        s.close()
    # one engine on one GPU opens a context on that GPU only
    eng = MemoryManager(0, device=0, server_id=0, gpu_count=n)
    ws = W.weight_set("bert_tiny")
    W.cold_start(eng, "t", ws)
    eng.evict("t"); eng.swap_in("t"); eng.wait_ready("t")
    sums = np.array([checksum_host(W.tensor_bytes(ws, i)) for i in range(len(ws.tensors))])
    assert np.array_equal(eng.checksum_resident("t"), sums)
    eng.close()
