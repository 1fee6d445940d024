"""Sharded swap-in with one process per GPU.

One rank (the *target*, rank 0) owns the pool the model ends up in; every rank lends its
PCIe link.  Per swap the target places blocks and rebinds the pointer table
(``tsw_swap_plan``), broadcasts the moves, and every rank runs the placement kernel on its
own GPU over its share of the tiles: reading the shared page-locked host store across its
own PCIe link and storing straight into the target's pool blocks across NVLink (the pool
is opened through CUDA IPC).  Completion counters and the pointer table sit on the target,
so whichever GPU finishes a parameter publishes it; the target then commits the rows
(``tsw_swap_commit``).  No collective moves data: ``torch.distributed`` (a gloo group)
carries only the few KB of control messages.  (An NCCL send/recv gather was measured beside the peer
stores and is slower; ``bench.py --nccl-gather`` repeats the measurement.)

Three ways of dealing out the tiles:
  direct     every rank's CTAs draw tiles from one counter on the target (or, statically, tile t goes
             to rank t mod N); host store -> target pool in one kernel per rank.
  pipelined  rank r owns the contiguous tile range r; its copy engine brings the range into local HBM
             chunk by chunk while the placement kernel stores the chunks already there into the
             target's pool across NVLink (``tsw_place_segments_pipelined``): for boxes whose links are
             fed evenly, where the copy engine reads host memory a few per cent faster than the SMs.
  staged     rank r owns the contiguous tile range r; its share is first pulled into local HBM
             (``prepare``), and the timed move is local HBM -> target pool across NVLink -- the
             gather stage on its own.

The reference has no counterpart (its swap uses one GPU's link, memory_manager.hpp:331-438);
the result must equal that single-GPU swap-in, which the tests check.
"""
from __future__ import annotations

import os
import time
from typing import Dict, List, Optional, Tuple

import numpy as np

from . import _cabi
from .memory_manager import SEGMENT_DTYPE, MemoryManager

PUB_WORDS = 8          # tsw_publish as words: done, phys, flag, host_phys, host_flag, flag_value, ticket_chunk, ticket
HEADER_WORDS = 8       # n_segments, tile_bytes, regions_epoch, mode, 4 spare


def tiles_of(segs: np.ndarray, tile: int) -> np.ndarray:
    """Tile prefix sums of a segment list: segment k owns tiles [first[k], first[k+1])."""
    n = (segs["bytes"].astype(np.uint64) + np.uint64(tile - 1)) // np.uint64(tile)
    return np.concatenate([[0], np.cumsum(n)]).astype(np.int64)


def fill_rows(segs: np.ndarray, tile: int, force: bool = False) -> np.ndarray:
    """Make ``row_tiles`` / ``row_dst`` explicit so that every rank launches the same table.
    ``force`` recounts rows that already carry a count (made for another tile size)."""
    segs = segs.copy()
    if force:
        segs["row_tiles"] = 0
    first = tiles_of(segs, tile)
    per_seg = np.diff(first).astype(np.uint32)
    rows = segs["row"]
    total: Dict[int, int] = {}
    first_dst: Dict[int, int] = {}
    for i in range(len(segs)):
        r = int(rows[i])
        total[r] = total.get(r, 0) + int(per_seg[i])
        first_dst.setdefault(r, int(segs["dst"][i]))
    for i in range(len(segs)):
        if segs["row_tiles"][i] == 0:
            segs["row_tiles"][i] = total[int(rows[i])]
            segs["row_dst"][i] = first_dst[int(rows[i])]
    return segs


def contiguous_share(total_tiles: int, rank: int, world: int) -> Tuple[int, int]:
    """Tile range [lo, hi) of ``rank`` when ``total_tiles`` are cut into ``world`` equal runs."""
    lo = (total_tiles * rank) // world
    hi = (total_tiles * (rank + 1)) // world
    return lo, hi


class AddressMap:
    """Rebase addresses of the target process into this process: device regions opened over
    IPC and the shared host arena."""

    def __init__(self):
        self.base0 = np.zeros(0, dtype=np.uint64)
        self.size = np.zeros(0, dtype=np.uint64)
        self.local = np.zeros(0, dtype=np.uint64)

    def set(self, entries: List[Tuple[int, int, int]]):
        entries = sorted(entries)
        self.base0 = np.array([e[0] for e in entries], dtype=np.uint64)
        self.size = np.array([e[1] for e in entries], dtype=np.uint64)
        self.local = np.array([e[2] for e in entries], dtype=np.uint64)

    def rebase(self, addr: np.ndarray) -> np.ndarray:
        addr = np.asarray(addr, dtype=np.uint64)
        if addr.size == 0:
            return addr
        idx = np.searchsorted(self.base0, addr, side="right").astype(np.int64) - 1
        if (idx < 0).any():
            raise ValueError("address below every shared region")
        off = addr - self.base0[idx]
        if (off >= self.size[idx]).any():
            bad = int(addr[np.nonzero(off >= self.size[idx])[0][0]])
            raise ValueError(f"address {bad:#x} is in no region shared by the target")
        return self.local[idx] + off

    def rebase_one(self, addr: int) -> int:
        return int(self.rebase(np.array([addr], dtype=np.uint64))[0]) if addr else 0


class ProgressBoard:
    """A few words of POSIX shared memory beside the control plane: every rank's process id and the
    number of the last swap whose share it has finished (its kernel drained).  When a control message
    fails in the middle of a swap, the target reads here whether a helper is gone or is still moving
    tiles into the pool -- instead of guessing by the clock -- before it takes the swap over."""

    def __init__(self, name: str, world: int, rank: int, create: bool):
        import mmap
        self.path = "/dev/shm/" + name.lstrip("/")
        self.world, self.rank = world, rank
        size = 16 * world
        fd = os.open(self.path, os.O_RDWR | (os.O_CREAT if create else 0), 0o600)
        try:
            if create:
                os.ftruncate(fd, size)
            self.mm = mmap.mmap(fd, size)
        finally:
            os.close(fd)
        self.words = np.frombuffer(self.mm, dtype=np.int64)      # [pid_0, done_0, pid_1, done_1, ...]
        self.words[2 * rank] = os.getpid()
        self.words[2 * rank + 1] = 0
        self.owner = create

    def finished(self, seq: int):
        self.words[2 * self.rank + 1] = seq

    def still_at_work(self, rank: int, seq: int) -> bool:
        """True while ``rank`` is a live process that has not finished swap ``seq``."""
        pid, done = int(self.words[2 * rank]), int(self.words[2 * rank + 1])
        if done >= seq or pid <= 0:
            return False
        try:
            with open(f"/proc/{pid}/stat") as f:
                state = f.read().rsplit(")", 1)[1].split()[0]
            return state not in ("Z", "X")                       # exited and not yet reaped counts as gone
        except OSError:
            return False

    def close(self):
        self.words = None
        try:
            self.mm.close()
        except BufferError:
            pass
        if self.owner:
            try:
                os.unlink(self.path)
            except OSError:
                pass


class ShardedSwap:
    """Collective swap-in over the ranks of ``group`` (a gloo process group for control).

    ``engine`` is this rank's engine on its own GPU; on rank 0 it is the target and was
    created with ``host_arena_shm=shm_name``.  All ranks call the same methods in the same
    order.  With ``engine=None`` (tests on CPU) only the planning and rebasing logic runs.
    """

    def __init__(self, engine: Optional[MemoryManager], rank: int, world: int, group=None,
                 shm_name: Optional[str] = None, max_segments: int = 4096):
        import torch.distributed as dist
        self.dist = dist
        self.engine = engine
        self.rank, self.world, self.group = rank, world, group
        self.shm_name = shm_name
        self.max_segments = max_segments
        self.map = AddressMap()
        self.epoch = -1
        self.region_bases: List[int] = []
        self.arena_entry: Optional[Tuple[int, int, int]] = None
        self.staging = {}           # (func, lo, hi, tile) -> torch uint8 buffer
        self.last = {}
        # without a CUDA engine only planning, sharing and rebasing run (CPU tests)
        self.dry = engine is None or engine.device < 0
        self.dynamic = True         # direct mode: draw tiles from a shared counter instead of t mod N
        self.staged_tile = 512 * 1024
        self.chunk_tiles = 128      # pipelined mode: tiles per copy-engine chunk (64 MiB)
        # the target's overrides of the engine's host-side tile size and of the tiles taken per draw
        # from the shared counter, for one swap to the next (measurement sweeps); 0 = the engine's own
        self.tile_override = 0
        self.chunk_override = 0
        # Helpers only lend bandwidth.  When a control message to them fails (a helper process is gone,
        # or the group's timeout ran out) the target stops asking and from then on swaps by itself.
        self.alone = world == 1
        self.lost_reason = ""
        self.settle_s = 10.0        # upper bound on the target's wait for helpers that are alive and still at work
        self.board: Optional[ProgressBoard] = None
        self.seq = 0                # swaps begun; the same on every rank

    # ---- control plane
    def _collective(self, fn, mine):
        """Run one control-plane collective; ``mine`` is the answer when this rank is on its own."""
        if self.alone:
            return mine
        try:
            return fn()
        except RuntimeError as ex:              # gloo reports a lost peer or a timeout this way
            if self.rank != 0:
                raise
            self.alone = True
            self.lost_reason = str(ex).splitlines()[0][:200] if str(ex) else type(ex).__name__
            return mine

    def _bcast_words(self, words: np.ndarray) -> np.ndarray:
        import torch

        def run():
            t = torch.from_numpy(words.view(np.int64))
            self.dist.broadcast(t, src=0, group=self.group)
            return t.numpy().view(np.uint64)
        return self._collective(run, words)

    def _bcast_obj(self, obj):
        def run():
            box = [obj]
            self.dist.broadcast_object_list(box, src=0, group=self.group)
            return box[0]
        return self._collective(run, obj)

    def _max_over_ranks(self, value: float) -> float:
        import torch

        def run():
            t = torch.tensor([value], dtype=torch.float64)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX, group=self.group)
            return float(t[0])
        return self._collective(run, value)

    def attach_arena(self):
        """Map the target's host store into every rank (once)."""
        info = self.engine.arena_info() if (self.rank == 0 and self.engine) else None
        info = self._bcast_obj(info)
        # the progress board: made by the target, opened by everyone
        name = None
        if self.rank == 0:
            name = f"torpor_swap_board_{os.getpid()}_{id(self) & 0xffffff:x}"
            self.board = ProgressBoard(name, self.world, 0, create=True)
        name = self._bcast_obj(name)
        if self.rank != 0 and name:
            self.board = ProgressBoard(name, self.world, self.rank, create=False)
        if self.dry:
            self.arena_entry = None
            return
        if info is None or info["size"] == 0:
            raise RuntimeError("the target engine has no shared host arena")
        if self.rank == 0:
            local = info["dev_base"]
        else:
            local = self.engine.arena_attach(self.shm_name, info["size"])
        self.arena_entry = (info["dev_base"], info["size"], local)

    def share_regions(self):
        """(Re)open the target's device allocations in every rank."""
        regs = self.engine.ipc_regions() if (self.rank == 0 and self.engine and not self.dry) else None
        regs = self._bcast_obj(regs)
        entries = [self.arena_entry] if self.arena_entry else []
        for base, size, handle in regs or []:
            if self.rank == 0:
                entries.append((base, size, base))
            else:
                entries.append((base, size, self.engine.ipc_open(handle)))
        self.map.set(entries)
        self.region_bases = sorted(b for b, _, _ in (regs or []))

    # ---- data plane
    def plan(self, func: str, mode: int):
        """Target: place + rebind and pack the moves; everyone: receive them."""
        buf = np.zeros(HEADER_WORDS + PUB_WORDS + self.max_segments * (SEGMENT_DTYPE.itemsize // 8), dtype=np.uint64)
        if self.rank == 0:
            segs, tile, pub = self.engine.swap_plan(func)
            if len(segs) > self.max_segments:
                raise RuntimeError("raise max_segments")
            bases = [] if self.dry else sorted(b for b, _, _ in self.engine.ipc_regions())
            changed = bases != self.region_bases
            if self.tile_override and mode == 0:
                tile = self.tile_override
            buf[0], buf[1], buf[2], buf[3] = len(segs), tile, 1 if changed else 0, mode
            buf[HEADER_WORDS:HEADER_WORDS + PUB_WORDS] = [pub.done_count, pub.table_phys, pub.table_flag, 0, 0,
                                                          pub.flag_value, self.chunk_override or pub.ticket_chunk, pub.ticket]
            raw = segs.view(np.uint64)
            buf[HEADER_WORDS + PUB_WORDS:HEADER_WORDS + PUB_WORDS + raw.size] = raw
        buf = self._bcast_words(buf)
        n, tile, changed = int(buf[0]), int(buf[1]), int(buf[2])
        if changed:
            self.share_regions()
        pubw = buf[HEADER_WORDS:HEADER_WORDS + PUB_WORDS]
        w = SEGMENT_DTYPE.itemsize // 8
        segs = buf[HEADER_WORDS + PUB_WORDS:HEADER_WORDS + PUB_WORDS + n * w].copy().view(SEGMENT_DTYPE)
        # Tile size of this swap: the target's host tile for moves that cross PCIe; larger tiles
        # for the staged gather, whose source is HBM.  Every rank derives the same numbering.
        if mode == 1:
            tile = self.staged_tile
        return fill_rows(segs, tile, force=True), tile, pubw

    def _local_publish(self, pubw, dynamic: bool) -> _cabi.Publish:
        m = self.map
        return _cabi.Publish(m.rebase_one(int(pubw[0])), m.rebase_one(int(pubw[1])), m.rebase_one(int(pubw[2])),
                             0, 0, int(pubw[5]), int(pubw[6]), m.rebase_one(int(pubw[7])) if dynamic else 0)

    def localize(self, segs: np.ndarray) -> np.ndarray:
        out = segs.copy()
        out["src"] = self.map.rebase(segs["src"])
        out["dst"] = self.map.rebase(segs["dst"])
        out["row_dst"] = segs["row_dst"]          # published value: the TARGET's address, not ours
        return out

    def swap_in(self, func: str, mode: str = "direct") -> dict:
        """Collective swap-in of ``func`` into the target's pool.  Returns timing of this rank's
        kernel and the maximum over ranks (device time, CUDA events)."""
        t0 = time.perf_counter()
        self.seq += 1
        segs, tile, pubw = self.plan(func, 0 if mode == "direct" else 1)
        n_tiles = int(tiles_of(segs, tile)[-1]) if len(segs) else 0
        dev_ns = 0.0
        if mode not in ("direct", "pipelined", "staged"):
            raise ValueError(f"unknown dealing mode {mode!r}")
        if mode == "direct":
            self.my_tiles = range(self.rank, n_tiles, self.world)
        else:
            self.my_tiles = range(*contiguous_share(n_tiles, self.rank, self.world))
        self.last_plan = (segs, tile)
        if self.alone and self.rank == 0:
            self.my_tiles = range(n_tiles)
        if len(segs) and not self.dry:
            local = self.localize(segs)
            pub = self._local_publish(pubw, dynamic=(mode == "direct" and self.dynamic and not self.alone))
            if self.alone:
                # nobody to share with (any more): the target moves every tile itself, from the host store
                self.engine.place_segment_array(local, tile, 0, 1, 0, pub, sync=True)
            elif mode == "direct" and self.dynamic:
                # every rank draws tiles from the counter on the target: faster links move more
                self.engine.place_segment_array(local, tile, 0, 1, 0, pub, sync=True)
            elif mode == "direct":
                self.engine.place_segment_array(local, tile, self.rank, self.world, 0, pub, sync=True)
            elif mode == "pipelined":
                lo, hi = contiguous_share(n_tiles, self.rank, self.world)
                if hi > lo:
                    self.engine.place_segment_array_pipelined(local, tile, lo, hi, pub, self.chunk_tiles, sync=True)
            else:
                lo, hi = contiguous_share(n_tiles, self.rank, self.world)
                buf = self._staging(func, segs, tile, lo, hi)
                first = tiles_of(segs, tile)[:-1]
                local["src"] = (np.uint64(buf.data_ptr()) + ((first - lo) * tile).astype(np.int64).view(np.uint64))
                if hi > lo:
                    self.engine.place_segment_array(local, tile, lo, 1, hi, pub, sync=True)
            dev_ns = float(self.engine.stats()["last_swap_device_ns"])
        if self.board is not None:
            self.board.finished(self.seq)       # this rank's kernel has drained (the launches above are synchronous)
        t_done = time.perf_counter()
        was_alone = self.alone
        dev_max = self._max_over_ranks(dev_ns)          # doubles as the completion barrier
        if self.rank == 0 and self.engine is not None:
            self._commit(func, lost_now=self.alone and not was_alone)
        self.last = {"tiles": n_tiles, "segments": len(segs), "tile_bytes": tile, "device_ns": dev_ns,
                     "device_ns_max": dev_max, "local_wall_s": t_done - t0, "wall_s": time.perf_counter() - t0}
        return self.last

    def _commit(self, func: str, lost_now: bool):
        """Take the published rows over.  If the control plane was lost during this very swap, helpers
        that are still alive may be moving tiles into the pool: the progress board says who has
        finished and who is gone, and the target waits for the rest (at most ``settle_s``) before it
        moves what is missing alone -- nobody may still be storing into blocks that the take-over,
        or a later eviction, hands to someone else."""
        from ._cabi import SwapError
        if lost_now:
            deadline = time.perf_counter() + self.settle_s
            while time.perf_counter() < deadline:
                if self.board is None or not any(self.board.still_at_work(r, self.seq) for r in range(1, self.world)):
                    break
                time.sleep(0.005)
        try:
            self.engine.swap_commit(func)
            return
        except SwapError:
            if not lost_now:
                raise
        self.engine.swap_in(func)           # clears the abandoned tile counters, moves the unfinished parameters
        self.engine.wait_ready(func)

    def _staging(self, func, segs, tile, lo, hi):
        """This rank's contiguous share of the swap, resident in local HBM."""
        import torch
        key = (func, lo, hi, tile)
        if key in self.staging:
            return self.staging[key]
        buf = torch.empty(max(1, (hi - lo) * tile), dtype=torch.uint8, device=f"cuda:{self.engine.device}")
        pull = segs.copy()
        first = tiles_of(segs, tile)[:-1]
        pull["src"] = self.map.rebase(segs["src"])
        pull["dst"] = (np.uint64(buf.data_ptr()) + ((first - lo) * tile).astype(np.int64).view(np.uint64))
        if hi > lo:
            self.engine.place_segment_array(pull, tile, lo, 1, hi, None, sync=True)
        self.staging[key] = buf
        return buf

    def evict(self, func: str):
        if self.rank == 0 and self.engine is not None:
            self.engine.evict(func)

    def close(self):
        if self.board is not None:
            self.board.close()
            self.board = None


# ------------------------------------------------------------------ benchmark driver (torchrun)

class _RawDevice:
    """A run of device memory that no torch allocation owns, as an object torch can wrap."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (int(nbytes),), "typestr": "|u1", "data": (int(ptr), False), "version": 3}


def nccl_gather(sw: "ShardedSwap", func: str, group, reps: int = 5) -> Optional[dict]:
    """The gather stage over NCCL instead of peer stores, for comparison: every helper sends its
    staged share (resident in its HBM) with ncclSend, the target receives (a) each share into one
    contiguous buffer -- NCCL's best case, the scatter into pool blocks would still have to follow --
    and (b) piece by piece straight into the pool blocks of the current placement.  Call right after
    a staged swap-in of ``func`` (the placement and the staged shares are then in place).
    Device time on the target (CUDA events), best of ``reps``."""
    import torch
    import torch.distributed as dist
    segs, tile = sw.last_plan
    first = tiles_of(segs, tile)
    n_tiles = int(first[-1])
    dev = torch.device(f"cuda:{sw.engine.device}")
    shares = [contiguous_share(n_tiles, r, sw.world) for r in range(sw.world)]

    def share_bytes(r):
        lo, hi = shares[r]
        return sum(max(0, min(int(segs["bytes"][k]), (min(hi, int(first[k + 1])) - int(first[k])) * tile)
                          - max(0, (max(lo, int(first[k])) - int(first[k])) * tile)) for k in range(len(segs))
                   if min(hi, int(first[k + 1])) > max(lo, int(first[k])))

    def pieces(r):
        """(offset in rank r's staging buffer, destination address on the target, bytes)"""
        lo, hi = shares[r]
        out = []
        for k in range(len(segs)):
            a, b = max(lo, int(first[k])), min(hi, int(first[k + 1]))
            if b <= a:
                continue
            off0 = (a - int(first[k])) * tile
            off1 = min(int(segs["bytes"][k]), (b - int(first[k])) * tile)
            if off1 > off0:
                out.append(((a - lo) * tile, int(segs["dst"][k]) + off0, off1 - off0))
        return out

    my_lo, my_hi = shares[sw.rank]
    mine = sw.staging.get((func, my_lo, my_hi, tile))
    if mine is None:
        return None
    inbound = sum(share_bytes(r) for r in range(1, sw.world))
    result = {"inbound_bytes": inbound}
    for mode in ("contiguous", "into_pool_blocks"):
        ops, keep = [], []
        if sw.rank == 0:
            for r in range(1, sw.world):
                if mode == "contiguous":
                    buf = torch.empty((shares[r][1] - shares[r][0]) * tile, dtype=torch.uint8, device=dev)
                    keep.append(buf)
                    ops.append(dist.P2POp(dist.irecv, buf, r, group=group))
                else:
                    for _, dst, n in pieces(r):
                        t = torch.as_tensor(_RawDevice(dst, n), device=dev)
                        keep.append(t)
                        ops.append(dist.P2POp(dist.irecv, t, r, group=group))
        else:
            if mode == "contiguous":
                ops.append(dist.P2POp(dist.isend, mine, 0, group=group))
            else:
                for off, _, n in pieces(sw.rank):
                    ops.append(dist.P2POp(dist.isend, mine[off:off + n], 0, group=group))
        best = None
        for _ in range(reps + 1):
            dist.barrier(group=sw.group)
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for w in dist.batch_isend_irecv(ops):
                w.wait()
            b.record()
            torch.cuda.synchronize()
            ms = sw._max_over_ranks(a.elapsed_time(b))
            best = ms if best is None else min(best, ms)
        result[mode] = {"ms": best, "inbound_gbs": inbound / (best / 1e3) / 1e9, "ops_per_helper": len(ops) if sw.rank else None}
        del keep
    return result


def bench_main(args, bench):
    """bench.py at N > 1: one rank per GPU; rank 0's GPU is the target."""
    import statistics
    import torch
    import torch.distributed as dist
    from . import workloads as W
    from .memory_manager import repo_reset

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world == 1:
        raise SystemExit("bench.py --gpus N with N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    # Control messages only: the data plane is the placement kernel's peer stores, no collective.
    dist.init_process_group("gloo")
    ctrl = dist.group.WORLD
    # Which GPU each rank drives.  With as many GPUs as ranks: rank r drives GPU r.  On a box with more
    # GPUs than ranks the links are not equal (GPUs behind a busier or farther root port are fed at half
    # the rate of the others), so the target measures every GPU's host-link rate with all of them
    # copying at once -- in a child process, so that no context stays open on GPUs the job does not use
    # -- and the best-fed N take part, the best of them as the target.
    devices, probe = None, None
    if rank == 0:
        if args.devices:
            devices = [int(d) for d in args.devices.split(",")]
        elif torch.cuda.device_count() > world:
            import json
            import subprocess
            import sys
            r = subprocess.run([sys.executable, os.path.abspath(bench.__file__), "--link-probe"], stdout=subprocess.PIPE,
                               stderr=subprocess.PIPE, text=True, timeout=300)
            for ln in r.stdout.splitlines():
                if ln.startswith("{"):
                    probe = json.loads(ln)["link_probe"]["concurrent_h2d_gbs"]
            if probe:
                devices = sorted(range(len(probe)), key=lambda g: -probe[g])[:world]
    box = [devices, probe]
    dist.broadcast_object_list(box, src=0)
    devices, probe = box
    if not devices or len(devices) != world:
        devices = list(range(world))
    local_rank = devices[rank]
    torch.cuda.set_device(local_rank)
    ncpu = os.cpu_count() or 1
    peaks, peak_kind = bench.measured_peaks()

    ws = W.weight_set(args.workload)
    K, Wm = args.steps, args.warmup
    K_g = min(K, 10)
    B = ws.nbytes

    # the reference on this box's host cores, rank 0 only, before the engines take the GPU's memory
    cpu_baseline = None
    if rank == 0 and not args.no_cpu_baseline:
        cpu_baseline = bench.cpu_baselines(args)
    dist.barrier(group=ctrl)

    shm = f"/torpor_swap_{os.environ.get('MASTER_PORT', '0')}_{os.getppid()}"
    repo_reset()
    tile_host = args.tile_kib * 1024
    budget = W.pool_budget_for(ws)
    sums, tables, vaddrs = {}, [], []
    cold_s = 0.0
    if rank == 0:
        sweep_swaps = 40 if args.sweep else 0
        tables = W.plan_tables(ws, "model", budget=budget, gpu_count=world, swaps=4 + 3 * (Wm + K) + (Wm + K_g) + sweep_swaps + 8)
        repo_reset()
        eng = MemoryManager(budget, device=local_rank, server_id=0, gpu_count=world, host_arena_bytes=W.host_store_bytes(ws),
                            host_arena_shm=shm, tile_bytes_host=tile_host, ticket_chunk=args.ticket_chunk, host_store_mode=args.host_store,
                            grid_ctas=getattr(args, "grid_ctas", 0))
    else:
        eng = MemoryManager(0, device=local_rank, server_id=rank, gpu_count=world, block_manager="Fixed",
                            grid_ctas=getattr(args, "grid_ctas", 0))
    sw = ShardedSwap(eng, rank, world, ctrl, shm_name=shm, max_segments=max(1024, len(ws.tensors) + 16))

    if rank == 0:
        pool, data, sums = bench.generate_tensors(ws, min(ncpu, 16), with_sums=True)
        t0 = time.time()
        loaded = W.cold_start(eng, "model", ws, tensor_data=data)
        vaddrs = loaded.tensor_vaddr
        pool.shutdown()
        torch.cuda.synchronize()
        cold_s = time.time() - t0
        eng.evict("model")
    ver = bench.Verifier(ws, sums, tables)
    dist.barrier(group=ctrl)
    sw.attach_arena()
    sw.share_regions()

    def swap(mode):
        r = sw.swap_in("model", mode)
        ver.swapped()
        return r

    def check(where):
        """The target checks every tensor and both tables; every rank waits.  Returns the seconds it took."""
        t0 = time.perf_counter()
        failure = None
        if rank == 0:
            try:
                ver.check(eng, "model", where)
            except RuntimeError as ex:
                failure = str(ex)
        failure = sw._bcast_obj(failure)
        if failure:
            raise RuntimeError(failure)
        return time.perf_counter() - t0

    def timed(mode, steps, warmup, through_translate=False, where="", verify=True):
        for _ in range(warmup):
            swap(mode); sw.evict("model")
        dev, pause = [], 0.0
        launches0 = eng.stats()["kernel_launches"]
        dist.barrier(group=ctrl)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for k in range(steps):
            r = swap(mode)
            if through_translate and rank == 0:
                for v in vaddrs:                 # the launch path: every parameter, in access order
                    eng.translate("model", v)
            dev.append(r["device_ns_max"])
            if verify and k == steps - 1:        # the last timed swap-in is the one that is checked; clock paused
                l1 = eng.stats()["kernel_launches"]
                pause = check(where)
                launches0 += eng.stats()["kernel_launches"] - l1
            sw.evict("model")
        torch.cuda.synchronize()
        dist.barrier(group=ctrl)
        wall = time.perf_counter() - t0 - pause
        wall = sw._max_over_ranks(wall)
        return wall, dev, eng.stats()["kernel_launches"] - launches0

    # correctness of both ways of dealing before anything is timed (also fills the staged shares)
    swap("direct"); check("before timing, direct"); sw.evict("model")
    swap("staged"); check("before timing, staged"); sw.evict("model")

    sampler = bench.ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    wall_v, dev_v, launches_v = timed("direct", K, Wm, where="after the timed sharded swap-ins")
    wall_e, dev_e, launches_e = timed("direct", K, Wm, through_translate=True, where="after the timed executor-path swap-ins")
    wall_g, dev_g, _ = timed("staged", K_g, Wm, where="after the timed gathers")
    # the executor path once more with the copy engines pulling (contiguous shares, pipelined with the peer stores)
    wall_p, dev_p, launches_p = timed("pipelined", K, Wm, through_translate=True, where="after the timed pipelined swap-ins")
    clocks = sampler.stop() if rank == 0 else None

    sweep = None
    if args.sweep:
        sweep = []
        for tile_kib in (64, 128, 256):
            for chunk in (1, 4, 16):
                sw.tile_override, sw.chunk_override = tile_kib * 1024, chunk
                w_s, d_s, _ = timed("direct", 3, 1, where=f"sweep tile {tile_kib} KiB, {chunk} tiles per draw")
                sweep.append({"tile_kib": tile_kib, "tiles_per_draw": chunk, "gbs_wall": B * 3 / w_s / 1e9,
                              "gbs_device": B / (statistics.mean(d_s) / 1e9) / 1e9})
        sw.tile_override = sw.chunk_override = 0

    nccl = None
    if args.nccl_gather:
        g = dist.new_group(backend="nccl")
        swap("staged")
        nccl = nccl_gather(sw, "model", g)
        check("after the NCCL gather comparison")
        sw.evict("model")

    # what the box's copy engines reach when every participating GPU pulls page-locked host
    # memory at once: the practical ceiling of the links, next to the theoretical one
    x = torch.empty(1 << 30, dtype=torch.uint8).pin_memory()
    y = torch.empty(1 << 30, dtype=torch.uint8, device=f"cuda:{local_rank}")
    dma_best = 0.0
    for _ in range(4):
        torch.cuda.synchronize()
        dist.barrier(group=ctrl)
        t0 = time.perf_counter()
        y.copy_(x, non_blocking=True)
        torch.cuda.synchronize()
        dt = sw._max_over_ranks(time.perf_counter() - t0)
        dma_best = max(dma_best, world * (1 << 30) / dt / 1e9)
    # ... and when each keeps pulling for a fixed time (the sum of the rates, not equal shares)
    dist.barrier(group=ctrl)
    t_end = time.perf_counter() + 1.0
    pulled = 0
    while time.perf_counter() < t_end:
        y.copy_(x, non_blocking=True)
        torch.cuda.synchronize()
        pulled += 1 << 30
    rates = torch.zeros(world, dtype=torch.float64)
    rates[rank] = pulled / 1.0 / 1e9
    dist.all_reduce(rates, group=ctrl)
    del x, y

    total_launches = torch.tensor([launches_v, launches_e, launches_p], dtype=torch.int64)
    dist.all_reduce(total_launches, group=ctrl)

    line = None
    if rank == 0:
        value = B * K / wall_v / 1e9
        e2e = B * K / wall_e / 1e9
        e2e_ms, e2e_dev_ms, e2e_dealing = wall_e / K * 1e3, statistics.mean(dev_e) / 1e6, "direct"
        piped = B * K / wall_p / 1e9
        e2e_by_dealing = {"direct": e2e, "pipelined": piped}
        if piped > e2e:         # what a deployment on this box would configure: the faster of the two, as measured here
            e2e, e2e_ms, e2e_dev_ms, e2e_dealing = piped, wall_p / K * 1e3, statistics.mean(dev_p) / 1e6, "pipelined"
        kern_v = statistics.mean(dev_v) / 1e9
        kern_g = statistics.mean(dev_g) / 1e9
        inbound = B * (world - 1) / world
        peak = bench.PCIE_GEN5_X16_GBS * world
        feed_sum = float(rates.sum())
        line = {
            "metric": "model_swap_in_throughput", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": K, "warmup": Wm, "ms_per_step": wall_v / K * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": bench.workload_config(args, world),
            "value_arm": "sharded swap-in from the shared page-locked host store: every rank's GPU reads tiles over its own PCIe "
                         "link and stores them into the target's pool over NVLink; plan, control messages, commit and evict "
                         "inside the timed region, max over ranks",
            "e2e": {"value": e2e, "unit": "GB/s", "ms_per_model": e2e_ms,
                    "h2d_bytes_per_step": B + 40 * len(ws.tensors) * world, "d2h_bytes_per_step": 12 * len(ws.tensors),
                    "device_ms_per_model": e2e_dev_ms, "dealing": e2e_dealing, "gbs_by_dealing": e2e_by_dealing,
                    "what": "the sharded swap-in followed, on the target, by tsw_translate of every parameter in access "
                            "order (the launch path), then tsw_evict; measured with tiles drawn from the shared counter and "
                            "read by the kernels (direct) and with contiguous shares pulled by each GPU's copy engine and "
                            "stored to the target by the kernel behind it (pipelined), the faster one reported"},
            "roofline": {"bound": "pcie", "achieved": B / kern_v / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": (B / kern_v / 1e9) / peak, "frac_wall": value / peak,
                         "peak_kind": f"theoretical PCIe Gen5 x16 x {world} participating GPUs (no PCIe figure in MEASURED_PEAKS.json)",
                         "kernel": "place_kernel (host store -> target pool: zero-copy reads over PCIe, peer stores over NVLink)",
                         "algorithmic_bytes_per_launch": B, "launch_ms": kern_v * 1e3,
                         "traffic": bench.DRAM_WRITE_PER_ALGO_BYTE_HOST * B,
                         "copy_engines_equal_shares_gbs": dma_best,
                         "copy_engines_continuous_per_gpu_gbs": [round(float(v), 2) for v in rates],
                         "copy_engines_continuous_sum_gbs": feed_sum,
                         "frac_of_measured_feed": value / max(feed_sum, dma_best) if max(feed_sum, dma_best) else None,
                         "dealing": "tiles drawn from a shared counter on the target (faster links move more)"},
            "gather_stage": {"bound": "nvlink", "achieved": inbound / kern_g / 1e9, "peak": 900.0, "unit": "GB/s",
                             "frac": inbound / kern_g / 1e9 / 900.0, "peak_measured": 770.0,
                             "frac_of_measured": inbound / kern_g / 1e9 / 770.0,
                             "peak_kind": "nominal NVLink 5 per direction per GPU; measured peer-copy rate on this pool beside it",
                             "kernel": "place_kernel (each rank's share in its HBM -> target pool over NVLink)",
                             "algorithmic_bytes_per_launch": inbound, "launch_ms": kern_g * 1e3, "steps": K_g,
                             "swap_gbs_wall": B * K_g / wall_g / 1e9, "nccl": nccl,
                             "what": "not the metric: the gather on its own, inputs already in the helpers' HBM"},
            "verified": ver.record(after_timed=True),
            "cpu_baseline": cpu_baseline,
            "gpu_launches": int(total_launches[0]),
            "gpu_launches_e2e": int(total_launches[2] if e2e_dealing == "pipelined" else total_launches[1]),
            "clocks": clocks, "host_cores": ncpu, "cold_start_s": cold_s,
            "settings": {"tile_bytes_host": tile_host or 65536, "tiles_per_draw": args.ticket_chunk or 1, "host_store_mode": args.host_store,
                         "grid_ctas": getattr(args, "grid_ctas", 0) or "6 per SM",
                         "devices": devices, "link_probe_concurrent_h2d_gbs": probe},
        }
        if sweep is not None:
            line["sweep"] = sweep
    dist.barrier(group=ctrl)
    sw.close()
    eng.close()
    repo_reset()
    dist.destroy_process_group()
    return line
