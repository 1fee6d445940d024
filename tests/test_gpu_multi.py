"""Multi-GPU parity: a swap-in sharded over several GPUs' PCIe links, and a replica swap
across NVLink, must leave exactly what a single-GPU swap-in leaves -- same pointer table as
the CPU checker, same resident bytes.  Needs at least two GPUs (skipped otherwise)."""
import os
import socket
import sys

import numpy as np
import pytest

import scenarios
from torpor_b200 import _cabi
from torpor_b200 import workloads as W
from torpor_b200.memory_manager import MemoryManager, ModelRepo, checksum_host, repo_reset

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def gpu_count():
    import torch
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


needs2 = pytest.mark.skipif(gpu_count() < 2, reason="needs two GPUs")


@needs2
@pytest.mark.parametrize("name,static", [("resnet50", False), ("llama_tiny", True), ("bert_large", False)])
def test_sharded_swap_in_process_equals_single_gpu_swap(built, oracle_backend, name, static):
    """Sharded swap-in (tiles drawn from the shared counter, or dealt t mod N) of the ResNet-50,
    a Llama-shaped and the BERT-large fp16 set over every GPU of the box."""
    n = min(gpu_count(), 8)
    repo_reset(); oracle_backend.reset()
    ws = W.weight_set(name)
    engines = [MemoryManager(0, device=d, server_id=d, gpu_count=n, shard_static=static,
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
        assert engines[d].stats()["kernel_launches"] == 3       # every GPU took part in every cycle, one launch each
    for e in engines:
        e.close()
    repo_reset(); oracle_backend.reset()


@needs2
def test_replica_swap_across_nvlink(built, oracle_backend):
    repo_reset(); oracle_backend.reset()
    ws = W.weight_set("bert_base")
    a = MemoryManager(0, device=0, server_id=0, gpu_count=2)
    b = MemoryManager(0, device=1, server_id=1, gpu_count=2)
    oa, ob = oracle_backend.manager(server_id=0, budget=0, gpu_count=2), oracle_backend.manager(server_id=1, budget=0, gpu_count=2)
    W.cold_start(b, "m", ws); W.cold_start(ob, "m", ws)
    ModelRepo.add_model_info("m", 1); oracle_backend.set_status("m", 1, True)
    a.swap_in("m", 1); a.wait_ready("m"); oa.swap_in("m", 1)
    assert np.array_equal(a.dump_params("m", canonical=True), oa.dump_params("m"))
    sums = np.array([checksum_host(W.tensor_bytes(ws, i)) for i in range(len(ws.tensors))])
    assert np.array_equal(a.checksum_resident("m"), sums)
    a.close(); b.close()
    repo_reset(); oracle_backend.reset()


@needs2
def test_topology_discovery_feeds_the_scheduler(built):
    from torpor_b200.memory_manager import Scheduler, discover_topology
    n = gpu_count()
    pairs, nv = discover_topology(n)
    assert len(pairs) == n and all(0 <= p < n for p in pairs)
    assert all(nv[i][i] == 0 for i in range(n)) and all(nv[i][j] in (-1, 1, 2) for i in range(n) for j in range(n) if i != j)
    assert any(nv[0][j] == 2 for j in range(1, n)), "an NVLink machine has at least one fast peer"
    s = Scheduler(n, "IA", pairs, nv)
    repo_reset()
    assert s.decide("f")[0] == 0
    s.close()


@needs2
def test_mixed_stream_evicts_and_swaps_across_gpus(built):
    """The mixed serverless stream at reduced scale over the real GPUs of the box (up to four), with a
    cap small enough for steady LRU eviction: every request completes, victims are unloaded, swap-ins
    come from the host store over PCIe and from other GPUs' replicas over NVLink, concurrently."""
    from torpor_b200 import serving
    from torpor_b200.memory_manager import discover_topology
    n = min(gpu_count(), 4)
    pairs, nv = discover_topology(n)
    out = serving.run_stream(n_gpus=n, n_models=16, rate=300.0, duration_s=3.0, cap_bytes=300 << 20, seed=4,
                             archs=("bert_tiny", "llama_tiny", "resnet50"), zero_weights=True,
                             pcie_pairs=pairs, nvlink=nv)
    assert out["completed"] == out["requests"] > 600
    assert out["evictions_in_service"] > 5
    assert out["swaps_from_host"] > 0 and out["swaps_from_replica"] > 0
    assert out["swap_ms_p99"] < 2000 and out["sustained_swap_gbs"] > 0.1


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, shm, out_dir, devices=None):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from torpor_b200 import sharded
    dev = devices[rank] if devices else rank        # CUDA ordinal of this rank's engine
    torch.cuda.set_device(dev)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    ws = W.weight_set("llama_tiny")
    repo_reset()
    if rank == 0:
        eng = MemoryManager(0, device=dev, server_id=0, gpu_count=world, host_arena_bytes=W.host_store_bytes(ws), host_arena_shm=shm)
        W.cold_start(eng, "m", ws)
        eng.evict("m")
    else:
        eng = MemoryManager(0, device=dev, server_id=rank, gpu_count=world, block_manager="Fixed")
    dist.barrier()
    sw = sharded.ShardedSwap(eng, rank, world, None, shm_name=shm, max_segments=256)
    sw.attach_arena(); sw.share_regions()
    ok = True
    sums = np.array([checksum_host(W.tensor_bytes(ws, i)) for i in range(len(ws.tensors))]) if rank == 0 else None
    tables = []
    sw.chunk_tiles = 3                      # pipelined mode: several copy-engine chunks even for this small set
    for mode in ("direct", "staged", "pipelined", "direct", "pipelined", "staged"):
        sw.swap_in("m", mode)
        if rank == 0:
            ok = ok and np.array_equal(eng.checksum_resident("m"), sums)
            tab = eng.dump_params("m", canonical=True)
            ok = ok and bool((tab[:, 4] == _cabi.READY_CUDA).all()) and bool((tab[:, 3] == tab[:, 5]).all())
            ok = ok and eng.get_cuda_addr("m", int(eng.dump_params("m")[3, 0])) == int(eng.dump_params("m")[3, 3])
        sw.evict("m")
    launches = eng.stats()["kernel_launches"]
    np.save(os.path.join(out_dir, f"r{rank}.npy"), np.array([int(ok), launches]))
    dist.barrier()
    sw.close()
    eng.close()
    dist.destroy_process_group()


@needs2
@pytest.mark.timeout(600)
def test_sharded_swap_one_process_per_gpu(built, tmp_path):
    """Two processes, one GPU each: pool opened over CUDA IPC, host store in shared memory."""
    import torch.multiprocessing as mp
    world = 2
    shm = f"/torpor_swap_test_{os.getpid()}"
    mp.spawn(_rank_main, args=(world, _free_port(), shm, str(tmp_path)), nprocs=world, join=True)
    res = [np.load(os.path.join(str(tmp_path), f"r{r}.npy")) for r in range(world)]
    assert res[0][0] == 1, "resident bytes or pointer table wrong after a sharded swap"
    assert res[1][1] >= 4, "the helper rank launched no kernels"


needs1 = pytest.mark.skipif(gpu_count() < 1, reason="needs a GPU")


@needs1
@pytest.mark.timeout(600)
def test_sharded_swap_one_process_per_rank_sharing_one_gpu(built, tmp_path):
    """The same two processes on a box with ONE GPU: both engines on device 0, the target's pool
    opened by the helper process over CUDA IPC, the host store in shared memory, tiles drawn from
    the counter in the target's memory.  The links are not separate, everything else is the
    multi-GPU path (all three dealings).  No kernel waits for another kernel, so the two
    processes' launches may run in any order on the shared device."""
    import torch.multiprocessing as mp
    world = 2
    shm = f"/torpor_swap_test1_{os.getpid()}"
    mp.spawn(_rank_main, args=(world, _free_port(), shm, str(tmp_path), [0, 0]), nprocs=world, join=True)
    res = [np.load(os.path.join(str(tmp_path), f"r{r}.npy")) for r in range(world)]
    assert res[0][0] == 1, "resident bytes or pointer table wrong after a sharded swap"
    assert res[1][1] >= 4, "the helper rank launched no kernels"


def _rank_losing_helper(rank, world, port, shm, out_dir, devices=None):
    sys.path.insert(0, ROOT)
    import datetime
    import torch
    import torch.distributed as dist
    from torpor_b200 import sharded
    dev = devices[rank] if devices else rank
    torch.cuda.set_device(dev)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=5))
    ws = W.weight_set("llama_tiny")
    repo_reset()
    if rank == 0:
        eng = MemoryManager(0, device=dev, server_id=0, gpu_count=world, host_arena_bytes=W.host_store_bytes(ws), host_arena_shm=shm)
        W.cold_start(eng, "m", ws)
        eng.evict("m")
    else:
        eng = MemoryManager(0, device=dev, server_id=rank, gpu_count=world, block_manager="Fixed")
    dist.barrier()
    sw = sharded.ShardedSwap(eng, rank, world, None, shm_name=shm, max_segments=256)
    sw.attach_arena(); sw.share_regions()
    sw.swap_in("m", "direct"); sw.evict("m")
    sw.swap_in("m", "staged"); sw.evict("m")
    if rank != 0:
        # leave between two swaps: place_segments ran synchronously, nothing of this rank is in flight
        torch.cuda.synchronize()
        os._exit(0)
    sums = np.array([checksum_host(W.tensor_bytes(ws, i)) for i in range(len(ws.tensors))])
    ok = not sw.alone
    for mode in ("direct", "staged", "direct"):
        sw.swap_in("m", mode)                       # the first of these finds the helper gone
        ok = ok and sw.alone and np.array_equal(eng.checksum_resident("m"), sums)
        tab = eng.dump_params("m", canonical=True)
        ok = ok and bool((tab[:, 4] == _cabi.READY_CUDA).all()) and bool((tab[:, 3] == tab[:, 5]).all())
        sw.evict("m")
    eng.swap_in("m"); eng.wait_ready("m")           # and the engine's ordinary path is intact afterwards
    ok = ok and np.array_equal(eng.checksum_resident("m"), sums)
    np.save(os.path.join(out_dir, "r0.npy"), np.array([int(ok)]))
    sw.close()
    eng.close()
    os._exit(0)


@needs2
@pytest.mark.timeout(600)
def test_target_swaps_alone_after_its_helper_process_is_gone(built, tmp_path):
    """Failure made on the host: the helper process exits between two swaps (no kernel in flight, no
    collective library on the data path).  The target's next control message fails, it stops asking for
    help, and every later swap-in is bit-exact, moved by the target alone."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    shm = f"/torpor_swap_lost_{os.getpid()}"
    port = _free_port()
    procs = [ctx.Process(target=_rank_losing_helper, args=(r, 2, port, shm, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    assert np.load(os.path.join(str(tmp_path), "r0.npy"))[0] == 1


@needs1
@pytest.mark.timeout(600)
def test_target_swaps_alone_after_its_helper_process_is_gone_on_one_gpu(built, tmp_path):
    """The lost-helper case with both processes on device 0 (a box with one GPU): the helper leaves
    between two swaps with nothing in flight; the target notices on its next control message and
    carries on alone, bit-exact."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    shm = f"/torpor_swap_lost1_{os.getpid()}"
    port = _free_port()
    procs = [ctx.Process(target=_rank_losing_helper, args=(r, 2, port, shm, str(tmp_path), [0, 0])) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    assert np.load(os.path.join(str(tmp_path), "r0.npy"))[0] == 1
