"""TEST INFRASTRUCTURE ONLY -- ctypes binding of the checkers' scenario ABI (tso_abi.h).

Loads either the CPU restatement (``libtorpor_oracle.so``) or the reference's
own headers compiled against a host-memory CUDA stand-in / the real CUDA
runtime (``_ref/libtorpor_ref_{fake,cuda}.so``).  Only tests, the smoke check
and the benchmark's CPU-baseline / reference legs may import this module; the
shipped package never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from typing import List

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

LIBS = {
    "oracle": os.path.join(HERE, "libtorpor_oracle.so"),
    "ref_fake": os.path.join(HERE, "_ref", "libtorpor_ref_fake.so"),
    "ref_cuda": os.path.join(HERE, "_ref", "libtorpor_ref_cuda.so"),
    "ref_exec": os.path.join(HERE, "_ref", "libtorpor_ref_exec.so"),   # ref_fake's contents plus the reference's executor
}


def build(targets=("oracle", "ref")) -> None:
    """Compile the checkers in place (``make -C oracle``).  The ``ref`` target
    is a no-op when the reference tree is not present."""
    subprocess.run(["make", "-C", HERE, *targets], check=True, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)


def available(kind: str) -> bool:
    return os.path.exists(LIBS[kind])


_loaded = {}


def load(kind: str) -> "TsoLib":
    if kind not in _loaded:
        if not available(kind) and kind == "oracle":
            build(("oracle",))
        _loaded[kind] = TsoLib(LIBS[kind])
    return _loaded[kind]


class TsoLib:
    def __init__(self, path: str):
        self.path = path
        L = self.lib = C.CDLL(path)
        u64, i32, i64, vp, cp = C.c_uint64, C.c_int, C.c_int64, C.c_void_p, C.c_char_p
        sig = {
            "tso_reset_world": (None, []),
            "tso_create": (vp, [i32, u64, i32, cp, u64, i32]),
            "tso_destroy": (None, [vp]),
            "tso_track_begin": (None, [vp, cp]),
            "tso_malloc": (u64, [vp, cp, u64, i32]),
            "tso_free": (None, [vp, cp, u64]),
            "tso_memcpy_h2d_model": (i32, [vp, cp, u64, vp, u64]),
            "tso_sync_done": (None, [vp, cp]),
            "tso_mark_access": (i32, [vp, u64]),
            "tso_track_end": (None, [vp, cp]),
            "tso_swap_in": (None, [vp, cp, i32]),
            "tso_wait_ready": (i64, [vp, cp]),
            "tso_swap_in_timed": (i64, [vp, cp, i32]),
            "tso_evict": (None, [vp, cp]),
            "tso_translate": (u64, [vp, cp, u64]),
            "tso_check_alloc": (i32, [vp, cp]),
            "tso_is_model_address": (i32, [vp, cp, u64]),
            "tso_set_model_status": (None, [cp, i32, i32]),
            "tso_total_size": (u64, [cp]),
            "tso_pool_chunks": (i32, [vp, vp, i32]),
            "tso_dump_blocks": (i32, [vp, cp, vp, i32]),
            "tso_dump_params": (i32, [vp, cp, vp, i32]),
            "tso_read_phys": (i32, [vp, u64, vp, u64]),
            "tso_read_host_store": (i32, [vp, cp, u64, vp, u64]),
            "tso_evictor_create": (vp, [cp, i32, u64]),
            "tso_evictor_destroy": (None, [vp]),
            "tso_evictor_check_and_add": (i32, [vp, i32, cp, u64, i32, vp, i32]),
            "tso_evictor_force_evict": (None, [vp, i32, cp]),
            "tso_evictor_lock": (None, [vp, i32, cp]),
            "tso_evictor_unlock": (None, [vp, i32, cp]),
            "tso_impl_name": (cp, []),
            "tso_enable_peer_access": (i32, [i32]),
        }
        sched = {
            "tso_sched_create": (vp, [i32, cp, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
            "tso_sched_destroy": (None, [vp]),
            "tso_sched_set_status": (None, [vp, i32, i32]),
            "tso_sched_set_level": (None, [vp, cp, i32]),
            "tso_sched_decide": (None, [vp, cp, C.POINTER(C.c_int)]),
            "tso_ctrl_create": (vp, [i32, u64, cp, cp, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
            "tso_ctrl_destroy": (None, [vp]),
            "tso_ctrl_request": (i32, [vp, i32, cp, cp, C.c_char_p, i32]),
            "tso_ctrl_complete": (i32, [vp, i32, C.c_char_p, i32]),
        }
        executor = {
            "tso_exec_register_kernel": (None, [cp]),
            "tso_exec_create": (vp, [i32, u64, i32]),
            "tso_exec_manager": (vp, [vp]),
            "tso_exec_destroy": (None, [vp]),
            "tso_exec_signal": (None, [vp, i32, cp]),
            "tso_exec_queries": (i32, [vp, vp, i32, vp, i32]),
            "tso_exec_launches": (i32, [C.c_char_p, i32]),
            "tso_exec_completions": (i32, [C.POINTER(C.c_int), i32]),
            "tso_exec_reset": (None, []),
        }
        if hasattr(L, "tso_pack_timed"):     # the reference's headers only
            sig["tso_pack_timed"] = (i64, [vp, cp])
        self.has_executor = hasattr(L, "tso_exec_create")
        if self.has_executor:
            sig.update(executor)
        self.has_scheduler = hasattr(L, "tso_sched_create")   # the restatement only
        if self.has_scheduler:
            sig.update(sched)
        for name, (res, args) in sig.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args

    @property
    def impl_name(self) -> str:
        return self.lib.tso_impl_name().decode()

    def reset_world(self) -> None:
        self.lib.tso_reset_world()

    def manager(self, server_id=0, budget=0, gpu_count=1, block_manager="Buddy",
                buffer_size=2 << 20, io_threads=4) -> "TsoManager":
        return TsoManager(self, server_id, budget, gpu_count, block_manager, buffer_size, io_threads)

    def evictor(self, kind: str, gpu_count: int, budget: int) -> "TsoEvictor":
        return TsoEvictor(self, kind, gpu_count, budget)

    def scheduler(self, n, policy, pcie_pairs, nvlink) -> "TsoScheduler":
        return TsoScheduler(self, n, policy, pcie_pairs, nvlink)

    def executor(self, server_id=0, budget=0, gpu_count=1) -> "TsoExecutor":
        return TsoExecutor(self, server_id, budget, gpu_count)

    def controller(self, n, mem_limit_bytes, sched_policy, evict_policy, pcie_pairs, nvlink) -> "TsoController":
        return TsoController(self, n, mem_limit_bytes, sched_policy, evict_policy, pcie_pairs, nvlink)

    def enable_peer_access(self, gpu_count: int) -> int:
        return self.lib.tso_enable_peer_access(gpu_count)

    def set_model_status(self, func: str, gpu: int, full: bool) -> None:
        self.lib.tso_set_model_status(func.encode(), gpu, 1 if full else 0)

    def total_size(self, func: str) -> int:
        return self.lib.tso_total_size(func.encode())


class TsoManager:
    """One memory manager of a checker, with the method names of tso_abi.h."""

    def __init__(self, lib: TsoLib, server_id, budget, gpu_count, block_manager, buffer_size, io_threads):
        self.L = lib.lib
        self.server_id = server_id
        self.h = self.L.tso_create(server_id, budget, gpu_count, block_manager.encode(), buffer_size, io_threads)
        if not self.h:
            raise RuntimeError("tso_create failed")

    def close(self):
        if self.h:
            self.L.tso_destroy(self.h)
            self.h = None

    def track_begin(self, f): self.L.tso_track_begin(self.h, f.encode())
    def malloc(self, f, size, is_model): return self.L.tso_malloc(self.h, f.encode(), size, 1 if is_model else 0)
    def free(self, f, vptr): self.L.tso_free(self.h, f.encode(), vptr)

    def memcpy_h2d_model(self, f, dst, data) -> int:
        if not isinstance(data, np.ndarray) and hasattr(data, "nbytes"):   # a size without bytes (TORPOR_ORACLE_TABLES_ONLY=1)
            if os.environ.get("TORPOR_ORACLE_TABLES_ONLY") != "1":
                raise ValueError("a payload without bytes needs TORPOR_ORACLE_TABLES_ONLY=1")
            return self.L.tso_memcpy_h2d_model(self.h, f.encode(), dst, None, int(data.nbytes))
        data = np.ascontiguousarray(data).view(np.uint8)
        return self.L.tso_memcpy_h2d_model(self.h, f.encode(), dst, data.ctypes.data, data.nbytes)

    def sync_done(self, f): self.L.tso_sync_done(self.h, f.encode())
    def mark_access(self, vptr): return self.L.tso_mark_access(self.h, vptr)
    def track_end(self, f): self.L.tso_track_end(self.h, f.encode())
    def swap_in(self, f, src_gpu=-1): self.L.tso_swap_in(self.h, f.encode(), src_gpu)
    def wait_ready(self, f): return self.L.tso_wait_ready(self.h, f.encode())
    def swap_in_timed(self, f, src_gpu=-1): return self.L.tso_swap_in_timed(self.h, f.encode(), src_gpu)
    def evict(self, f): self.L.tso_evict(self.h, f.encode())
    def pack_timed(self, f): return self.L.tso_pack_timed(self.h, f.encode())
    def translate(self, f, vptr): return self.L.tso_translate(self.h, f.encode(), vptr)
    def check_alloc(self, f): return bool(self.L.tso_check_alloc(self.h, f.encode()))
    def is_model_address(self, f, vptr): return bool(self.L.tso_is_model_address(self.h, f.encode(), vptr))

    def pool_chunks(self) -> np.ndarray:
        n = self.L.tso_pool_chunks(self.h, None, 0)
        out = np.zeros(max(n, 1), dtype=np.uint64)
        self.L.tso_pool_chunks(self.h, out.ctypes.data, n)
        return out[:n]

    def dump_blocks(self, f) -> np.ndarray:
        n = self.L.tso_dump_blocks(self.h, f.encode(), None, 0)
        out = np.zeros((max(n, 1), 6), dtype=np.uint64)
        self.L.tso_dump_blocks(self.h, f.encode(), out.ctypes.data, n)
        return out[:n]

    def dump_params(self, f) -> np.ndarray:
        n = self.L.tso_dump_params(self.h, f.encode(), None, 0)
        out = np.zeros((max(n, 1), 7), dtype=np.uint64)
        self.L.tso_dump_params(self.h, f.encode(), out.ctypes.data, n)
        return out[:n]

    def read_phys(self, addr, size) -> np.ndarray:
        out = np.empty(size, dtype=np.uint8)
        rc = self.L.tso_read_phys(self.h, addr, out.ctypes.data, size)
        if rc != 0:
            raise RuntimeError(f"tso_read_phys failed: {rc}")
        return out

    def read_host_store(self, f, vptr, size) -> np.ndarray:
        out = np.empty(size, dtype=np.uint8)
        rc = self.L.tso_read_host_store(self.h, f.encode(), vptr, out.ctypes.data, size)
        if rc != 0:
            raise RuntimeError(f"tso_read_host_store failed: {rc}")
        return out


class TsoScheduler:
    def __init__(self, lib: TsoLib, n, policy, pcie_pairs, nvlink):
        self.L = lib.lib
        pp = (C.c_int * n)(*pcie_pairs)
        nv = (C.c_int * (n * n))(*[v for row in nvlink for v in row])
        self.h = self.L.tso_sched_create(n, policy.encode(), pp, nv)
        if not self.h:
            raise ValueError("this checker only knows the reference's hard-coded 4-GPU topology")

    def close(self):
        if self.h:
            self.L.tso_sched_destroy(self.h)
            self.h = None

    def set_status(self, gpu, status): self.L.tso_sched_set_status(self.h, gpu, status)
    def set_level(self, func, level): self.L.tso_sched_set_level(self.h, func.encode(), level)

    def decide(self, func):
        out = (C.c_int * 3)()
        self.L.tso_sched_decide(self.h, func.encode(), out)
        return out[0], out[1], out[2]


class TsoExecutor:
    """The reference's CUDAExecutor (include/server/cuda_server.hpp) with its loop running on a thread:
    signals as the controller sends them, serialised QueryLists as the clients send them."""

    def __init__(self, lib: TsoLib, server_id, budget, gpu_count):
        self.lib, self.L = lib, lib.lib
        self.server_id = server_id
        self.h = self.L.tso_exec_create(server_id, budget, gpu_count)
        if not self.h:
            raise RuntimeError("tso_exec_create failed")
        # the executor's own memory manager, for the table dumps (a view: never closed through it)
        self.manager = TsoManager.__new__(TsoManager)
        self.manager.L, self.manager.server_id, self.manager.h = self.L, server_id, self.L.tso_exec_manager(self.h)
        self.buf = C.create_string_buffer(1 << 20)

    def close(self):
        if self.h:
            self.manager.h = None
            self.L.tso_exec_destroy(self.h)
            self.h = None

    def register_kernel(self, name: str):
        self.L.tso_exec_register_kernel(name.encode())

    def signal(self, sig: int, func: str):
        self.L.tso_exec_signal(self.h, sig, func.encode())

    def handle(self, query_list: bytes) -> List[bytes]:
        """One serialised QueryList in, the serialised responses the executor sent while handling it out."""
        src = C.create_string_buffer(query_list, len(query_list))
        need = self.L.tso_exec_queries(self.h, src, len(query_list), self.buf, len(self.buf))
        if need > len(self.buf):
            raise RuntimeError("responses larger than the buffer")
        raw, out, pos = self.buf.raw[:need], [], 0
        while pos < need:
            n = int.from_bytes(raw[pos:pos + 4], "little")
            out.append(raw[pos + 4:pos + 4 + n])
            pos += 4 + n
        return out

    def launches(self):
        """[(kernel name, [argument bytes, ...])] since the last call, as passed to cudaLaunchKernel."""
        need = self.L.tso_exec_launches(self.buf, len(self.buf))
        if need > len(self.buf):
            raise RuntimeError("launch list larger than the buffer")
        out = []
        for ln in self.buf.value.decode().splitlines():
            parts = ln.split(" ")
            out.append((parts[0], [b"" if a == "-" else bytes.fromhex(a) for a in parts[1:]]))
        return out

    def completions(self) -> List[int]:
        arr = (C.c_int * 64)()
        n = self.L.tso_exec_completions(arr, 64)
        return list(arr[:min(n, 64)])


class TsoController:
    """One controller of a checker; ``request`` / ``complete`` return the trace lines of that event."""

    def __init__(self, lib: TsoLib, n, mem_limit_bytes, sched_policy, evict_policy, pcie_pairs, nvlink):
        self.L = lib.lib
        pp = (C.c_int * n)(*pcie_pairs)
        nv = (C.c_int * (n * n))(*[v for row in nvlink for v in row])
        self.h = self.L.tso_ctrl_create(n, mem_limit_bytes, sched_policy.encode(), evict_policy.encode(), pp, nv)
        if not self.h:
            raise ValueError("this checker only knows the reference's 4-GPU topology and whole-GiB limits below 25")
        self.buf = C.create_string_buffer(1 << 16)

    def close(self):
        if self.h:
            self.L.tso_ctrl_destroy(self.h)
            self.h = None

    def _lines(self, need):
        if need > len(self.buf):
            raise RuntimeError("controller trace larger than the buffer")
        text = self.buf.value.decode()
        return text.split("\n") if text else []

    def request(self, kind, func, payload=""):
        return self._lines(self.L.tso_ctrl_request(self.h, kind, func.encode(), payload.encode(), self.buf, len(self.buf)))

    def complete(self, executor):
        return self._lines(self.L.tso_ctrl_complete(self.h, executor, self.buf, len(self.buf)))


class TsoEvictor:
    def __init__(self, lib: TsoLib, kind, gpu_count, budget):
        self.L = lib.lib
        self.h = self.L.tso_evictor_create(kind.encode(), gpu_count, budget)

    def close(self):
        if self.h:
            self.L.tso_evictor_destroy(self.h)
            self.h = None

    def check_and_add(self, gpu, func, size, level=1) -> List[str]:
        buf = C.create_string_buffer(1 << 16)
        n = self.L.tso_evictor_check_and_add(self.h, gpu, func.encode(), size, level, buf, len(buf))
        if n < 0:
            raise RuntimeError("victim buffer too small")
        return buf.value.decode().split("\n") if n else []

    def force_evict(self, gpu, func): self.L.tso_evictor_force_evict(self.h, gpu, func.encode())
    def lock(self, gpu, func): self.L.tso_evictor_lock(self.h, gpu, func.encode())
    def unlock(self, gpu, func): self.L.tso_evictor_unlock(self.h, gpu, func.encode())
