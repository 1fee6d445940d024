"""Randomised differential test at the executor level: the random call streams of
tests/test_random_differential.py, expressed as what a client and the controller send -- serialised
cudarpc queries and executor signals -- and replayed on the reference's own CUDAExecutor
(include/server/cuda_server.hpp compiled where it lies, over its own MemoryManager on the
host-memory CUDA stand-in) and on WireExecutor over a plan-only engine.  After every step the tables
must be identical, and so must every response on the way."""
import os
import struct

import pytest

import scenarios
from test_random_differential import random_stream, replay, reuses_a_block_name
from torpor_b200 import wire
from torpor_b200.memory_manager import MemoryManager, repo_reset


class ExecutorAsManager:
    """An executor behind the manager method names ``replay`` drives: every call becomes the wire
    message or signal that causes it (cuda_server.hpp:212-255,951-1065,1226-1310)."""

    def __init__(self, executor, tables, complete, log):
        self.ex, self.tables, self._complete, self.log = executor, tables, complete, log
        self.server_id = 0
        self.active = None

    @staticmethod
    def name(f):                       # executors derive the client's address from the function name
        return f.lstrip("m")

    def _send(self, qtype, message, fields):
        ql = wire.encode("QueryList", {"queries": [{"type": qtype, "query": wire.encode(message, fields), "client_id": 1}]})
        r = self.ex.handle(ql)
        self.log.append((message, r))
        return r

    def _activate(self, f):
        if self.active != f:
            self.ex.signal(wire.SIG_EXECUTE, self.name(f))
            self.active = f

    def track_begin(self, f):
        if f not in self.seen:
            self.seen.add(f)
            self.ex.signal(wire.SIG_STARTUP, self.name(f))      # a cold start
            self.active = f
        else:
            self._activate(f)                                   # a later request of a known function

    seen: set = None

    def malloc(self, f, size, is_model):
        if self.active != f:
            self._activate(f)           # an ordinary request of a known function
        return wire.decode("cudaMallocResponse", self._send(wire.Q_MALLOC, "cudaMallocQuery", {"size": size})[0])["ptr"]

    def memcpy_h2d_model(self, f, dst, data):
        self._send(wire.Q_MEMCPY_ASYNC, "cudaMemcpyAsyncQuery", {"kind": wire.H2D, "dst": dst, "count": int(data.nbytes),
                                                                "payload": data.tobytes(), "stream": bytes(8)})
        return 0

    def sync_done(self, f):
        self._send(wire.Q_DEVICE_SYNCHRONIZE, "genericResponse", {})

    def mark_access(self, p):
        self._send(wire.Q_LAUNCH_KERNEL, "cudaLaunchKernelQuery", {"function": "k", "grid_dim_x": 1, "stream": bytes(8),
                                                                   "args": [struct.pack("<Q", p)]})
        return 1

    def track_end(self, f):
        self._complete()
        self.active = None

    def free(self, f, p):
        self._activate(f)
        self._send(wire.Q_FREE, "cudaFreeQuery", {"ptr": p})
        self._complete()
        self.active = None

    def evict(self, f):
        self.ex.signal(wire.SIG_UNLOAD, self.name(f))

    def swap_in(self, f, src_gpu=-1):
        self.ex.signal(wire.SIG_LOAD + 1 + src_gpu, self.name(f))

    def wait_ready(self, f):
        return self.tables.wait_ready(self.name(f))

    def check_alloc(self, f):
        return self.tables.check_alloc(self.name(f))

    def dump_blocks(self, f, canonical=False):
        return self.tables.dump_blocks(self.name(f))

    def dump_params(self, f, canonical=False):
        return self.tables.dump_params(self.name(f))

    def close(self):
        pass


class ReferenceExecutorBackend:
    def __init__(self, lib):
        self.lib, self.ex, self.log = lib, None, []

    def reset(self):
        if self.ex:
            self.ex.close()
            self.ex = None
        self.lib.reset_world()
        self.lib.lib.tso_exec_reset()

    def manager(self, server_id=0, budget=0, gpu_count=1, block_manager="Buddy"):
        # always written: another checker library of this process may have set it with setenv, behind Python's back
        os.environ["BLOCK_MANAGER"] = block_manager
        self.ex = self.lib.executor(server_id, budget, gpu_count)
        self.ex.register_kernel("k")

        def complete():                    # the result copy ends a request (cuda_server.hpp:1043-1049)
            self.ex.handle(wire.encode("QueryList", {"queries": [{"type": wire.Q_MEMCPY_ASYNC, "client_id": 1, "query": wire.encode(
                "cudaMemcpyAsyncQuery", {"kind": wire.D2H, "src": 0x600000000000, "dst": 0x7000, "count": 0, "stream": bytes(8)})}]}))
            assert self.ex.completions() == [0]
        m = ExecutorAsManager(self.ex, self.ex.manager, complete, self.log)
        m.seen = set()
        return m

    def blocks(self, m, f): return m.dump_blocks(f)
    def params(self, m, f): return m.dump_params(f)


class WireExecutorBackend:
    def __init__(self):
        self.eng, self.log = None, []

    def reset(self):
        if self.eng:
            self.eng.close()
            self.eng = None
        repo_reset()

    def manager(self, server_id=0, budget=0, gpu_count=1, block_manager="Buddy"):
        self.eng = MemoryManager(budget, device=-1, server_id=server_id, gpu_count=gpu_count, block_manager=block_manager)
        ex = wire.WireExecutor(self.eng)
        m = ExecutorAsManager(ex, self.eng, ex.complete, self.log)
        m.seen = set()
        return m

    def blocks(self, m, f): return m.dump_blocks(f)
    def params(self, m, f): return m.dump_params(f)


@pytest.mark.parametrize("block_manager", ["Buddy", "Fixed"])
@pytest.mark.parametrize("seed", range(16))
def test_random_streams_through_both_executors(built, seed, block_manager):
    from oracle import tso
    if not tso.available("ref_exec"):
        pytest.skip("oracle/_ref/libtorpor_ref_exec.so not built (reference tree absent)")
    ops = random_stream(seed, block_manager)
    if reuses_a_block_name(ops):
        pytest.skip("a block's name is granted again in this stream: the reference corrupts its own tables there")
    ref, mine = ReferenceExecutorBackend(tso.load("ref_exec")), WireExecutorBackend()
    want = replay(ref, ops)
    got = replay(mine, ops)
    scenarios.assert_same(got, want, f"executors, seed {seed} / {block_manager}")
    assert len(want) > 30
    assert [m for m, _ in mine.log] == [m for m, _ in ref.log]
    differing = [(i, m) for i, ((m, a), (_, b)) in enumerate(zip(mine.log, ref.log)) if a != b]
    assert not differing, differing[:5]              # every response byte-identical
