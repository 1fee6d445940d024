"""The N > 1 path on CPU: two gloo ranks run the collective sharded swap-in on plan-only
engines.  Nothing moves, but everything around the kernel runs: the target's placement and
rebind, packing and broadcast of the moves, the per-rank tile shares of both dealing schemes,
address rebasing, and the commit -- whose table must equal an ordinary single-GPU swap-in."""
import os
import socket
import sys

import numpy as np
import pytest
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from torpor_b200 import sharded, workloads as W
    from torpor_b200.memory_manager import MemoryManager, repo_reset
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    ws = W.weight_set("resnet50")
    zeros = lambda i: np.zeros(ws.tensors[i].nbytes, dtype=np.uint8)
    eng = None
    if rank == 0:
        repo_reset()
        eng = MemoryManager(0, device=-1)
        W.cold_start(eng, "m", ws, tensor_data=zeros)
        W.cold_start(eng, "other", W.weight_set("bert_tiny"), tensor_data=lambda i: np.zeros(W.weight_set("bert_tiny").tensors[i].nbytes, np.uint8))
        eng.evict("m")
        eng.evict("other")
    sw = sharded.ShardedSwap(eng, rank, world, None, shm_name=None, max_segments=512)
    sw.attach_arena()
    sw.share_regions()
    res = {}
    for mode in ("direct", "staged", "pipelined"):
        r = sw.swap_in("m", mode)
        segs, tile = sw.last_plan
        first = sharded.tiles_of(segs, tile)
        res[mode] = {"tiles": list(sw.my_tiles), "n_tiles": int(first[-1]), "n_segs": len(segs),
                     "rows": segs["row"].tolist(), "row_tiles": segs["row_tiles"].tolist(),
                     "per_seg": np.diff(first).tolist(), "dst": segs["dst"].tolist(), "row_dst": segs["row_dst"].tolist()}
        if rank == 0:
            res[mode]["params"] = eng.dump_params("m", canonical=True).tolist()
            res[mode]["blocks"] = eng.dump_blocks("m", canonical=True).tolist()
            res[mode]["alloc"] = eng.check_alloc("m")
        sw.evict("m")
    if rank == 0:
        # the same cycle done the ordinary way on the same engine must land on the same tables
        eng.swap_in("m"); eng.wait_ready("m")
        res["plain"] = {"params": eng.dump_params("m", canonical=True).tolist()}
        eng.close()
        repo_reset()
    np.save(os.path.join(out_dir, f"r{rank}.npy"), np.array([res], dtype=object), allow_pickle=True)
    dist.barrier()
    sw.close()
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_two_ranks_cover_every_tile_once_and_commit_the_reference_table(built, tmp_path):
    world = 2
    port = _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    res = [np.load(os.path.join(str(tmp_path), f"r{r}.npy"), allow_pickle=True)[0] for r in range(world)]
    for mode in ("direct", "staged", "pipelined"):
        a, b = res[0][mode], res[1][mode]
        assert a["n_segs"] == b["n_segs"] == 161 and a["n_tiles"] == b["n_tiles"] > 161
        assert a["rows"] == b["rows"] and a["dst"] == b["dst"]        # every rank got the same moves
        tiles = sorted(a["tiles"] + b["tiles"])
        assert tiles == list(range(a["n_tiles"]))                       # each tile exactly once
        assert abs(len(a["tiles"]) - len(b["tiles"])) <= 1
        assert a["row_tiles"] == a["per_seg"] and a["row_dst"] == a["dst"]   # one segment per parameter here
        params = np.array(a["params"], dtype=np.uint64)
        assert (params[:, 4] == 2).all() and (params[:, 3] == params[:, 5]).all() and a["alloc"]
    # a sharded swap leaves exactly the table of an ordinary swap-in of the same state
    p_direct = np.array(res[0]["direct"]["params"], dtype=np.uint64)
    p_plain = np.array(res[0]["plain"]["params"], dtype=np.uint64)
    assert np.array_equal(p_direct[:, [0, 1, 2, 4, 6]], p_plain[:, [0, 1, 2, 4, 6]])


def test_shares_and_rebasing():
    sys.path.insert(0, ROOT)
    from torpor_b200 import sharded
    from torpor_b200.memory_manager import SEGMENT_DTYPE
    for total in (0, 1, 7, 64, 1000):
        for world in (1, 2, 3, 8):
            cover = []
            for r in range(world):
                lo, hi = sharded.contiguous_share(total, r, world)
                cover += list(range(lo, hi))
            assert cover == list(range(total))
    segs = np.zeros(3, dtype=SEGMENT_DTYPE)
    segs["bytes"] = [10, 65536 * 2 + 1, 0]
    segs["row"] = [4, 4, 9]
    segs["dst"] = [1000, 2000, 3000]
    out = sharded.fill_rows(segs, 65536)
    assert out["row_tiles"].tolist() == [4, 4, 0] and out["row_dst"].tolist() == [1000, 1000, 3000]
    m = sharded.AddressMap()
    m.set([(0x1000, 0x100, 0x9000), (0x5000, 0x1000, 0x20000)])
    assert m.rebase(np.array([0x1000, 0x10ff, 0x5800], dtype=np.uint64)).tolist() == [0x9000, 0x90ff, 0x20800]
    with pytest.raises(ValueError):
        m.rebase(np.array([0x1100], dtype=np.uint64))
    with pytest.raises(ValueError):
        m.rebase(np.array([0x10], dtype=np.uint64))


def _worker_losing_a_helper(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    import datetime
    import torch.distributed as dist
    from torpor_b200 import sharded, workloads as W
    from torpor_b200.memory_manager import MemoryManager, repo_reset
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=5))
    ws = W.weight_set("resnet50")
    eng = None
    if rank == 0:
        repo_reset()
        eng = MemoryManager(0, device=-1)
        W.cold_start(eng, "m", ws, tensor_data=lambda i: np.zeros(ws.tensors[i].nbytes, dtype=np.uint8))
        eng.evict("m")
    sw = sharded.ShardedSwap(eng, rank, world, None, shm_name=None, max_segments=512)
    sw.attach_arena()
    sw.share_regions()
    sw.swap_in("m", "direct")
    sw.evict("m")
    if rank != 0:
        os._exit(0)                      # the helper goes away between two swaps, without a word
    res = {"alone_before": sw.alone}
    for mode in ("direct", "staged", "direct"):
        sw.swap_in("m", mode)
        res.setdefault("tiles", []).append((len(sw.my_tiles), sw.last["tiles"]))
        res.setdefault("params", []).append(eng.dump_params("m", canonical=True).tolist())
        res.setdefault("alloc", []).append(eng.check_alloc("m"))
        sw.evict("m")
    res["alone_after"], res["reason"] = sw.alone, sw.lost_reason
    eng.swap_in("m"); eng.wait_ready("m")
    res["plain"] = eng.dump_params("m", canonical=True).tolist()
    res["board_said_gone"] = not sw.board.still_at_work(1, sw.seq)      # the helper's process is gone: nothing to wait for
    sw.close()
    eng.close()
    repo_reset()
    np.save(os.path.join(out_dir, "r0.npy"), np.array([res], dtype=object), allow_pickle=True)
    os._exit(0)                          # no orderly shutdown of a group whose other member is gone


@pytest.mark.timeout(300)
def test_target_carries_on_alone_when_its_helper_goes_away(built, tmp_path):
    """Failure made on the host: the helper rank exits between two swaps.  The target's next control
    message fails (at once or at the group's 5 s timeout); it stops asking for help and moves every
    tile itself, and the tables it ends up with are those of an ordinary swap-in."""
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_worker_losing_a_helper, args=(r, 2, port, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    res = np.load(os.path.join(str(tmp_path), "r0.npy"), allow_pickle=True)[0]
    assert res["alone_before"] is False and res["alone_after"] is True and res["reason"]
    assert res["board_said_gone"] is True
    for mine, total in res["tiles"]:
        assert mine == total > 161                                       # the target took every tile
    assert all(res["alloc"])
    plain = np.array(res["plain"], dtype=np.uint64)
    for params in res["params"]:
        p = np.array(params, dtype=np.uint64)
        assert (p[:, 4] == 2).all() and np.array_equal(p[:, [0, 1, 2, 4, 6]], plain[:, [0, 1, 2, 4, 6]])


def test_progress_board_tells_finished_from_gone():
    """The shared-memory board the target reads when a control message failed in mid-swap: a rank is
    'still at work' only while its process lives and it has not finished the swap in question."""
    import subprocess
    from torpor_b200 import sharded
    name = f"torpor_swap_board_test_{os.getpid()}"
    owner = sharded.ProgressBoard(name, 3, 0, create=True)
    peer = sharded.ProgressBoard(name, 3, 1, create=False)          # same process here: its pid is alive
    assert owner.still_at_work(1, 5)
    peer.finished(5)
    assert not owner.still_at_work(1, 5) and owner.still_at_work(1, 6)
    # rank 2: a process that has already exited
    child = subprocess.Popen([sys.executable, "-c", "pass"])
    child.wait()
    owner.words[4], owner.words[5] = child.pid, 0
    assert not owner.still_at_work(2, 1)
    # a rank that never registered
    owner.words[4] = 0
    assert not owner.still_at_work(2, 1)
    peer.close()
    owner.close()
    assert not os.path.exists("/dev/shm/" + name)
