"""Host-side mirror of the reference's ``MemoryManager`` over the C ABI.

``MemoryManager`` carries the public method names of
``server::manager::MemoryManager`` (include/server/memory_manager.hpp:36-298)
with the same argument meaning, so that a scenario written against the
reference reads the same here.  The short aliases (``malloc``, ``swap_in`` ...)
are the names the test scenarios and ``workloads.cold_start`` use for every
implementation of the path.

Nothing in this module moves bytes itself: every call goes into
``libtorpor_swap.so``.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import numpy as np

from . import _cabi
from ._cabi import SwapError, check

DEFAULT_TIMEOUT_NS = 30_000_000_000

# tsw_segment as a numpy record (include/torpor_swap.h)
SEGMENT_DTYPE = np.dtype([("src", "<u8"), ("dst", "<u8"), ("bytes", "<u8"), ("row_dst", "<u8"),
                          ("row", "<u4"), ("row_tiles", "<u4")])


def make_segments(src, dst, nbytes, rows=None, row_dst=None, row_tiles=None) -> np.ndarray:
    n = len(src)
    segs = np.zeros(n, dtype=SEGMENT_DTYPE)
    segs["src"] = np.asarray(src, dtype=np.uint64)
    segs["dst"] = np.asarray(dst, dtype=np.uint64)
    segs["bytes"] = np.asarray(nbytes, dtype=np.uint64)
    segs["row"] = np.arange(n, dtype=np.uint32) if rows is None else np.asarray(rows, dtype=np.uint32)
    if row_dst is not None:
        segs["row_dst"] = np.asarray(row_dst, dtype=np.uint64)
    if row_tiles is not None:
        segs["row_tiles"] = np.asarray(row_tiles, dtype=np.uint32)
    return segs


def repo_reset() -> None:
    check(_cabi.lib().tsw_repo_reset())


class ModelRepo:
    """The process-wide fields the controller reads (include/server/model_repo.hpp:82-90,180-185)."""

    @staticmethod
    def add_model_info(func: str, gpu: int) -> None:
        check(_cabi.lib().tsw_repo_add_model_info(func.encode(), gpu))

    @staticmethod
    def remove_model_info(func: str, gpu: int) -> None:
        check(_cabi.lib().tsw_repo_remove_model_info(func.encode(), gpu))

    @staticmethod
    def status(func: str, gpu: int) -> int:
        return _cabi.lib().tsw_repo_model_status(func.encode(), gpu)

    @staticmethod
    def total_size(func: str) -> int:
        return _cabi.lib().tsw_repo_total_size(func.encode())

    @staticmethod
    def active_devices(func: str) -> List[int]:
        buf = (C.c_int * 64)()
        n = _cabi.lib().tsw_repo_active_devices(func.encode(), buf, 64)
        return sorted(buf[i] for i in range(min(n, 64)))


class SizeOnly:
    """Stands for ``nbytes`` bytes that are not supplied: what a plan-only engine is given as a
    parameter's payload when only placement and tables are wanted."""

    def __init__(self, nbytes: int):
        self.nbytes = int(nbytes)


class MemoryManager:
    """One swap engine (one per GPU).

    ``device=-1`` gives a plan-only engine: it places blocks and rebinds the
    pointer table exactly as a CUDA engine would, makes no CUDA call and moves
    no byte; every data call on it raises ``TSW_ERR_NO_DEVICE``.
    """

    def __init__(self, budget: int = 25 << 30, *, device: int = 0, server_id: int = 0, gpu_count: int = 1,
                 block_manager: str = "Buddy", host_arena_bytes: int = 0, host_arena_shm: Optional[str] = None,
                 grid_ctas: int = 0, tile_bytes_host: int = 0, tile_bytes_device: int = 0, shard_static: bool = False,
                 mover: int = 0, host_store_mode: int = 0, ticket_chunk: int = 0, grid_ctas_host: int = 0):
        self.L = _cabi.lib()
        cfg = _cabi.Config()
        self.L.tsw_config_default(C.byref(cfg))
        cfg.device = device
        cfg.server_id = server_id
        cfg.gpu_count = gpu_count
        cfg.budget_bytes = budget
        cfg.pool_policy = _cabi.POOL_FIXED if block_manager == "Fixed" else _cabi.POOL_BUDDY
        cfg.host_arena_bytes = host_arena_bytes
        self._shm = host_arena_shm.encode() if host_arena_shm else None
        cfg.host_arena_shm = self._shm
        cfg.grid_ctas = grid_ctas
        cfg.tile_bytes_host = tile_bytes_host
        cfg.tile_bytes_device = tile_bytes_device
        cfg.shard_static = 1 if shard_static else 0
        cfg.mover = mover
        cfg.host_store_mode = host_store_mode
        cfg.ticket_chunk = ticket_chunk
        cfg.grid_ctas_host = grid_ctas_host
        h = C.c_void_p()
        check(self.L.tsw_engine_create(C.byref(cfg), C.byref(h)))
        self.h = h
        self.device = device
        self.server_id = server_id

    # ---- life cycle
    def close(self) -> None:
        if self.h:
            self.L.tsw_engine_destroy(self.h)
            self.h = None

    destroy_trans_thread = close

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # ---- reference method names
    def set_track_model_memory(self, func: str) -> None:
        check(self.L.tsw_track_begin(self.h, func.encode()))

    def unset_track_model_memory(self, func: str) -> None:
        check(self.L.tsw_track_end(self.h, func.encode()))

    def cudaMallocBackend(self, size: int, load_model_flag: bool, func: str) -> int:
        out = C.c_uint64()
        check(self.L.tsw_malloc(self.h, func.encode(), size, 1 if load_model_flag else 0, C.byref(out)))
        return out.value

    def cudaFreeBackend(self, ptr: int, func: str) -> None:
        check(self.L.tsw_free(self.h, func.encode(), ptr))

    def cudaMemcpyAsyncBackendHtoD(self, dst: int, payload, stream: int, load_model_flag: bool, func: str) -> int:
        if isinstance(payload, SizeOnly):     # plan-only engines: the parameter's size without its bytes
            return self.L.tsw_memcpy_h2d_model(self.h, func.encode(), dst, None, payload.nbytes, stream)
        data = np.ascontiguousarray(payload).view(np.uint8).reshape(-1)
        fn = self.L.tsw_memcpy_h2d_model if load_model_flag else self.L.tsw_memcpy_h2d
        return fn(self.h, func.encode(), dst, data.ctypes.data, data.nbytes, stream)

    def cudaMemcpyAsyncBackendDtoH(self, src: int, count: int, stream: int, func: str) -> np.ndarray:
        out = np.empty(count, dtype=np.uint8)
        check(self.L.tsw_memcpy_d2h(self.h, func.encode(), out.ctypes.data, src, count, stream))
        return out

    def cudaMemcpyAsyncBackendDtoD(self, dst: int, src: int, count: int, stream: int, func: str) -> None:
        check(self.L.tsw_memcpy_d2d(self.h, func.encode(), dst, src, count, stream))

    def cudaMemsetAsyncBackend(self, ptr: int, value: int, count: int, stream: int, func: str) -> None:
        check(self.L.tsw_memset(self.h, func.encode(), ptr, value, count, stream))

    def init_model_readiness(self, func: str) -> None:
        check(self.L.tsw_sync_done(self.h, func.encode()))

    def try_insert_model_access(self, ptr: int) -> bool:
        return check(self.L.tsw_mark_access(self.h, ptr)) == 1

    def check_model_alloc_status(self, func: str) -> bool:
        return check(self.L.tsw_check_alloc(self.h, func.encode())) == 1

    def sig_trans_thread(self, func: str, src_gpu: int = -1) -> None:
        check(self.L.tsw_swap_in(self.h, func.encode(), src_gpu))

    def evict_model(self, func: str, free_memory: bool = False, writeback: bool = False) -> None:
        check(self.L.tsw_evict(self.h, func.encode(), 1 if writeback else 0))

    def get_cuda_addr(self, func: str, ptr: int, search_amid: bool = True,
                      timeout_ns: int = DEFAULT_TIMEOUT_NS) -> int:
        out = C.c_uint64()
        check(self.L.tsw_translate(self.h, func.encode(), ptr, 1 if search_amid else 0, timeout_ns, C.byref(out)))
        return out.value

    def get_cuda_addr_async(self, func: str, ptr: int, stream: int):
        """Stream-ordered ``get_cuda_addr``: (address, waited).  If the parameter is still on its
        way, ``stream`` is made to wait for it; the host does not block."""
        out, waited = C.c_uint64(), C.c_int()
        check(self.L.tsw_translate_async(self.h, func.encode(), ptr, stream, C.byref(out), C.byref(waited)))
        return out.value, bool(waited.value)

    def release_waiters(self, func: str) -> int:
        """Let go of every stream still waiting for a parameter of ``func`` (tsw_release_waiters)."""
        return check(self.L.tsw_release_waiters(self.h, func.encode()))

    def is_model_address(self, func: str, ptr: int) -> bool:
        return check(self.L.tsw_is_model_address(self.h, func.encode(), ptr)) == 1

    def valid_memory_address(self, func: str, ptr: int) -> bool:
        return check(self.L.tsw_valid_memory_address(self.h, func.encode(), ptr)) == 1

    # ---- scenario aliases shared with the checkers
    def track_begin(self, f): self.set_track_model_memory(f)
    def track_end(self, f): self.unset_track_model_memory(f)
    def malloc(self, f, size, is_model): return self.cudaMallocBackend(size, is_model, f)
    def free(self, f, vptr): self.cudaFreeBackend(vptr, f)
    def memcpy_h2d_model(self, f, dst, data): return self.cudaMemcpyAsyncBackendHtoD(dst, data, 0, True, f)
    def sync_done(self, f): self.init_model_readiness(f)
    def mark_access(self, vptr): return 1 if self.try_insert_model_access(vptr) else 0
    def swap_in(self, f, src_gpu=-1): self.sig_trans_thread(f, src_gpu)
    def evict(self, f, writeback=False): self.evict_model(f, writeback=writeback)
    def translate(self, f, vptr): return self.get_cuda_addr(f, vptr)
    def check_alloc(self, f): return self.check_model_alloc_status(f)

    def swap_in_sharded(self, func: str, helpers: Sequence["MemoryManager"]) -> None:
        arr = (C.c_void_p * max(1, len(helpers)))(*[h.h for h in helpers])
        check(self.L.tsw_swap_in_sharded(self.h, func.encode(), arr, len(helpers)))

    def place_segments(self, src, dst, nbytes, rows=None, tile_bytes: int = 0, tile_first: int = 0,
                       tile_stride: int = 1, tile_end: int = 0, publish: Optional[_cabi.Publish] = None,
                       sync: bool = True, row_dst=None, row_tiles=None) -> None:
        """Run the placement kernel over explicit (src, dst, bytes) segments."""
        segs = make_segments(src, dst, nbytes, rows, row_dst, row_tiles)
        self.place_segment_array(segs, tile_bytes, tile_first, tile_stride, tile_end, publish, sync)

    def place_segment_array(self, segs: np.ndarray, tile_bytes: int = 0, tile_first: int = 0, tile_stride: int = 1,
                            tile_end: int = 0, publish: Optional[_cabi.Publish] = None, sync: bool = True) -> None:
        """Same, with the segments already in the ABI's layout (``SEGMENT_DTYPE``)."""
        segs = np.ascontiguousarray(segs, dtype=SEGMENT_DTYPE)
        check(self.L.tsw_place_segments(self.h, segs.ctypes.data, len(segs), tile_bytes, tile_first, tile_stride,
                                        tile_end, C.byref(publish) if publish is not None else None,
                                        1 if sync else 0))

    def place_segment_array_pipelined(self, segs: np.ndarray, tile_bytes: int, tile_first: int, tile_end: int,
                                      publish: Optional[_cabi.Publish] = None, chunk_tiles: int = 0, sync: bool = True) -> None:
        """Tiles [tile_first, tile_end) of ``segs`` in two pipelined steps: copy engine host -> this GPU,
        placement kernel this GPU -> destination (``tsw_place_segments_pipelined``)."""
        segs = np.ascontiguousarray(segs, dtype=SEGMENT_DTYPE)
        check(self.L.tsw_place_segments_pipelined(self.h, segs.ctypes.data, len(segs), tile_bytes, tile_first, tile_end,
                                                  C.byref(publish) if publish is not None else None, chunk_tiles,
                                                  1 if sync else 0))

    # ---- one process per GPU: plan here, move elsewhere, commit here
    def swap_plan(self, func: str):
        """Place and rebind like ``sig_trans_thread`` but return the moves instead of running
        them: (segments as ``SEGMENT_DTYPE`` array, tile bytes, publish block)."""
        n_max = max(16, self.L.tsw_dump_params(self.h, func.encode(), 0, None, 0))
        segs = np.zeros(n_max, dtype=SEGMENT_DTYPE)
        tile = C.c_uint32()
        pub = _cabi.Publish()
        n = check(self.L.tsw_swap_plan(self.h, func.encode(), segs.ctypes.data, n_max, C.byref(tile), C.byref(pub)))
        return segs[:n], tile.value, pub

    def swap_commit(self, func: str) -> None:
        check(self.L.tsw_swap_commit(self.h, func.encode()))

    def ipc_regions(self):
        """[(base, size, handle bytes)] of every device allocation a peer process must map."""
        n = check(self.L.tsw_ipc_regions(self.h, None, 0))
        arr = (_cabi.IpcRegion * max(n, 1))()
        check(self.L.tsw_ipc_regions(self.h, arr, n))
        return [(arr[i].base, arr[i].size, bytes(arr[i].handle)) for i in range(n)]

    def ipc_open(self, handle: bytes) -> int:
        out = C.c_uint64()
        buf = C.create_string_buffer(handle, 64)
        check(self.L.tsw_ipc_open(self.h, buf, C.byref(out)))
        return out.value

    def pointer_info(self, addr: int):
        t, d, dp, hp = C.c_int(), C.c_int(), C.c_uint64(), C.c_uint64()
        check(self.L.tsw_pointer_info(self.h, addr, C.byref(t), C.byref(d), C.byref(dp), C.byref(hp)))
        return {"type": t.value, "device": d.value, "device_pointer": dp.value, "host_pointer": hp.value}

    def arena_info(self):
        a, b, c, d = C.c_uint64(), C.c_uint64(), C.c_uint64(), C.c_uint64()
        check(self.L.tsw_arena_info(self.h, C.byref(a), C.byref(b), C.byref(c), C.byref(d)))
        return {"host_base": a.value, "dev_base": b.value, "size": c.value, "used": d.value}

    def arena_attach(self, shm_name: str, size: int) -> int:
        out = C.c_uint64()
        check(self.L.tsw_arena_attach(self.h, shm_name.encode(), size, C.byref(out)))
        return out.value

    def poll_ready(self, func: str) -> int:
        """Accessed parameters of ``func`` not on the device yet (0 = swap-in complete)."""
        return check(self.L.tsw_poll_ready(self.h, func.encode()))

    def wait_ready(self, func: str, timeout_ns: int = DEFAULT_TIMEOUT_NS) -> None:
        check(self.L.tsw_wait_ready(self.h, func.encode(), timeout_ns))

    # ---- introspection
    def pool_info(self):
        a, b, c = C.c_uint64(), C.c_uint64(), C.c_uint64()
        check(self.L.tsw_pool_info(self.h, C.byref(a), C.byref(b), C.byref(c)))
        return a.value, b.value, c.value

    def pool_chunks(self) -> np.ndarray:
        base, n, _ = self.pool_info()
        return np.uint64(base) + np.arange(n, dtype=np.uint64) * np.uint64(128 << 20)

    def dump_blocks(self, func: str, canonical: bool = False) -> np.ndarray:
        c = 1 if canonical else 0
        n = self.L.tsw_dump_blocks(self.h, func.encode(), c, None, 0)
        out = np.zeros((max(n, 1), 6), dtype=np.uint64)
        self.L.tsw_dump_blocks(self.h, func.encode(), c, out.ctypes.data, n)
        return out[:n]

    def dump_params(self, func: str, canonical: bool = False) -> np.ndarray:
        c = 1 if canonical else 0
        n = self.L.tsw_dump_params(self.h, func.encode(), c, None, 0)
        out = np.zeros((max(n, 1), 7), dtype=np.uint64)
        self.L.tsw_dump_params(self.h, func.encode(), c, out.ctypes.data, n)
        return out[:n]

    def canonical_address(self, func: str, addr: int) -> int:
        out = C.c_uint64()
        check(self.L.tsw_canonical_address(self.h, func.encode(), addr, C.byref(out)))
        return out.value

    def read_phys(self, addr: int, size: int) -> np.ndarray:
        out = np.empty(size, dtype=np.uint8)
        check(self.L.tsw_read_phys(self.h, addr, out.ctypes.data, size))
        return out

    def read_host_store(self, func: str, vptr: int, size: int) -> np.ndarray:
        out = np.empty(size, dtype=np.uint8)
        check(self.L.tsw_read_host_store(self.h, func.encode(), vptr, out.ctypes.data, size))
        return out

    def checksum_resident(self, func: str) -> np.ndarray:
        n = self.L.tsw_dump_params(self.h, func.encode(), 0, None, 0)
        out = np.zeros((max(n, 1), 2), dtype=np.uint64)
        check(self.L.tsw_checksum_resident(self.h, func.encode(), out.ctypes.data, n))
        return out[:n]

    def stats(self):
        a, b, c = C.c_uint64(), C.c_uint64(), C.c_uint64()
        check(self.L.tsw_stats(self.h, C.byref(a), C.byref(b), C.byref(c)))
        return {"kernel_launches": a.value, "bytes_moved": b.value, "last_swap_device_ns": c.value}


STATIC_MAX_SEGMENTS = 16384


def place_segments_static(device: int, src, dst, nbytes, rows=None, tile_bytes: int = 0, tile_first: int = 0,
                          tile_stride: int = 1, publish: Optional[_cabi.Publish] = None, stream: int = 0) -> None:
    """The placement kernel over explicit segments without any allocation on the way
    (``tsw_place_segments_static``): for callers on a server's steady-state path, where
    cudaMalloc would stall or fail.  At most ``STATIC_MAX_SEGMENTS`` segments per call; the
    call is asynchronous on ``stream``, and calls on one device must not overlap on the GPU."""
    segs = make_segments(src, dst, nbytes, rows)
    check(_cabi.lib().tsw_place_segments_static(device, segs.ctypes.data, len(segs), tile_bytes, tile_first, tile_stride,
                                                C.byref(publish) if publish is not None else None, stream))


def place_segments_static_status(device: int, stream: int = 0, clear: bool = False) -> int:
    """The word in which the allocation-free mover reports a table that did not fit its tile
    numbering (what overlapping calls on one device produce); 0 = nothing reported.  Synchronises
    ``stream``.  (``tsw_place_segments_static_status``)"""
    word = C.c_uint32()
    check(_cabi.lib().tsw_place_segments_static_status(device, stream, C.byref(word), 1 if clear else 0))
    return word.value


class Evictor:
    """LRUEvictor / InterferenceAwareEvictor (include/server/evictor.hpp)."""

    def __init__(self, kind: str, gpu_count: int, budget: int):
        self.L = _cabi.lib()
        h = C.c_void_p()
        check(self.L.tsw_evictor_create(kind.encode(), gpu_count, budget, C.byref(h)))
        self.h = h

    def close(self):
        if self.h:
            self.L.tsw_evictor_destroy(self.h)
            self.h = None

    def check_and_add(self, gpu: int, func: str, size: int, level: int = 1) -> List[str]:
        buf = C.create_string_buffer(1 << 16)
        n = check(self.L.tsw_evictor_check_and_add(self.h, gpu, func.encode(), size, level, buf, len(buf)))
        return buf.value.decode().split("\n") if n else []

    def force_evict(self, gpu, func): check(self.L.tsw_evictor_force_evict(self.h, gpu, func.encode()))
    def lock(self, gpu, func): check(self.L.tsw_evictor_lock(self.h, gpu, func.encode()))
    def unlock(self, gpu, func): check(self.L.tsw_evictor_unlock(self.h, gpu, func.encode()))


# ExecutorStatus_* (include/server/controller.hpp:18-24)
STATUS_AVAIL, STATUS_RUN_LOCAL, STATUS_RUN_NVLINK = -1, 0, 1
STATUS_RUN_PCIE_LIGHT, STATUS_RUN_PCIE_MEDIAN, STATUS_RUN_PCIE_HEAVY, STATUS_RUN_COLD_START = 2, 3, 4, 5


def discover_topology(gpu_count: int):
    """(pcie_pairs, nvlink matrix) of this machine, in the form ``Scheduler`` takes."""
    pairs = (C.c_int * gpu_count)()
    nv = (C.c_int * (gpu_count * gpu_count))()
    check(_cabi.lib().tsw_topology_discover(gpu_count, pairs, nv))
    return list(pairs), [[nv[i * gpu_count + j] for j in range(gpu_count)] for i in range(gpu_count)]


class Scheduler:
    """The controller's swap decision (include/server/controller.hpp:296-389) for N GPUs."""

    def __init__(self, gpu_count: int, policy: str = "IA", pcie_pairs=None, nvlink=None):
        self.L = _cabi.lib()
        h = C.c_void_p()
        pp = (C.c_int * gpu_count)(*pcie_pairs) if pcie_pairs is not None else None
        nv = (C.c_int * (gpu_count * gpu_count))(*[v for row in nvlink for v in row]) if nvlink is not None else None
        check(self.L.tsw_sched_create(gpu_count, policy.encode(), pp, nv, C.byref(h)))
        self.h = h

    def close(self):
        if self.h:
            self.L.tsw_sched_destroy(self.h)
            self.h = None

    def set_status(self, gpu: int, status: int): check(self.L.tsw_sched_set_status(self.h, gpu, status))
    def set_level(self, func: str, level: int): check(self.L.tsw_sched_set_level(self.h, func.encode(), level))

    def helpers(self, dst: int, include_running: bool = False) -> List[int]:
        """GPUs whose PCIe link is free to help a swap-in of ``dst`` from the host store."""
        buf = (C.c_int * 64)()
        n = check(self.L.tsw_sched_helpers(self.h, dst, 1 if include_running else 0, buf, 64))
        return list(buf[:min(n, 64)])

    def decide(self, func: str):
        g, s, st = C.c_int(), C.c_int(), C.c_int()
        check(self.L.tsw_sched_decide(self.h, func.encode(), C.byref(g), C.byref(s), C.byref(st)))
        return g.value, s.value, st.value


# RequestType (proto/signal.proto) and ExecutorSignal_* (common/include/utils.hpp:70-74)
REQ_EXECUTE_AFTER_LOAD, REQ_EXECUTE, REQ_LOAD, REQ_UNLOAD = 0, 1, 2, 3
SIGNAL_NOTIFY, SIGNAL_STARTUP, SIGNAL_EXECUTE, SIGNAL_UNLOAD, SIGNAL_LOAD = 0, 1, 2, 3, 4


class Controller:
    """Request and completion handling of the controller (include/server/controller.hpp:130-262,
    392-453) over the library's scheduler and eviction policy.

    ``request`` and ``complete`` return what the reference would have sent while handling that
    event, in its order: ``("S", gpu, signal, func)`` for a signal to an executor (a load is
    ``SIGNAL_LOAD + 1 + src_gpu``) and ``("A", ack, resp)`` for the acknowledgement to the router.
    """

    def __init__(self, gpu_count: int, mem_limit_bytes: int, schedule_policy: str = "IA", evict_policy: str = "IA",
                 pcie_pairs=None, nvlink=None):
        self.L = _cabi.lib()
        self.n = gpu_count
        self._events: List[tuple] = []
        self._on_signal = _cabi.SIGNAL_FN(lambda user, gpu, sig, func: self._events.append(("S", gpu, sig, func.decode())))
        self._on_ack = _cabi.ACK_FN(lambda user, ack, resp: self._events.append(("A", ack, resp)))
        pp = (C.c_int * gpu_count)(*pcie_pairs) if pcie_pairs is not None else None
        nv = (C.c_int * (gpu_count * gpu_count))(*[v for row in nvlink for v in row]) if nvlink is not None else None
        h = C.c_void_p()
        check(self.L.tsw_ctrl_create(gpu_count, mem_limit_bytes, schedule_policy.encode(), evict_policy.encode(), pp, nv,
                                     self._on_signal, self._on_ack, None, C.byref(h)))
        self.h = h

    def close(self):
        if self.h:
            self.L.tsw_ctrl_destroy(self.h)
            self.h = None

    def _drain(self, rc: int) -> List[tuple]:
        out, self._events = self._events, []
        check(rc)
        return out

    def request(self, kind: int, func: str, payload: str = "") -> List[tuple]:
        return self._drain(self.L.tsw_ctrl_request(self.h, kind, func.encode(), payload.encode()))

    def complete(self, executor: int) -> List[tuple]:
        return self._drain(self.L.tsw_ctrl_complete(self.h, executor))

    def executor_status(self, gpu: int):
        st = C.c_int()
        buf = C.create_string_buffer(512)
        check(self.L.tsw_ctrl_executor_status(self.h, gpu, C.byref(st), buf, 512))
        return st.value, buf.value.decode()

    def queue_depth(self) -> int:
        return check(self.L.tsw_ctrl_queue_depth(self.h))

    def helpers(self, dst: int, include_running: bool = False) -> List[int]:
        """GPUs whose PCIe link is free to help a swap-in of ``dst`` from the host store."""
        buf = (C.c_int * 64)()
        n = check(self.L.tsw_ctrl_helpers(self.h, dst, 1 if include_running else 0, buf, 64))
        return list(buf[:min(n, 64)])


def checksum_host(data: np.ndarray) -> np.ndarray:
    """The checksum of ``tsw_checksum_resident`` computed with numpy on host bytes."""
    b = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
    pad = (-b.size) % 4
    if pad:
        b = np.concatenate([b, np.zeros(pad, dtype=np.uint8)])
    w = b.view(np.uint32).astype(np.uint64)
    s1 = np.uint64(0)
    s2 = np.uint64(0)
    step = 1 << 22
    with np.errstate(over="ignore"):
        for i in range(0, w.size, step):
            c = w[i:i + step]
            s1 = s1 + c.sum(dtype=np.uint64)
            idx = np.arange(i + 1, i + 1 + c.size, dtype=np.uint64)
            s2 = s2 + (c * idx).sum(dtype=np.uint64)
    return np.array([s1, s2], dtype=np.uint64)
