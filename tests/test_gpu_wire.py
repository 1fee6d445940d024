"""The remoting surface on a GPU: serialised cudarpc messages into WireExecutor over a CUDA
engine, ending in real cudaLaunchKernel calls on the argument words the executor rewrote
(cuda_server.hpp:1226-1310).  A function is cold-started and run through the wire, evicted,
pushed out of its old pool blocks by another function, swapped back in by a Load signal and run
again with the client's old pointers: the kernel must see the weights at their new address."""
import ctypes as C
import os
import struct

import numpy as np
import pytest

from torpor_b200 import wire
from torpor_b200.memory_manager import MemoryManager, repo_reset

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
KERNELS = os.path.join(ROOT, "tests", "lib", "libwire_kernels.so")
MiB = 1 << 20


class Client:
    """What the client-side interposer sends: one serialised QueryList per call."""

    def __init__(self, ex):
        self.ex = ex

    def call(self, qtype, message, fields):
        body = wire.encode(message, fields) if message else b""
        r = self.ex.handle(wire.encode("QueryList", {"queries": [{"type": qtype, "client_id": 1, "query": body}]}))
        return r[0] if r else None

    def malloc(self, size):
        return wire.decode("cudaMallocResponse", self.call(wire.Q_MALLOC, "cudaMallocQuery", {"size": size}))["ptr"]

    def upload(self, dst, arr):
        self.call(wire.Q_MEMCPY_ASYNC, "cudaMemcpyAsyncQuery",
                  {"kind": wire.H2D, "dst": dst, "count": arr.nbytes, "payload": arr.tobytes()})

    def launch(self, name, args, grid=64, block=256):
        self.call(wire.Q_LAUNCH_KERNEL, "cudaLaunchKernelQuery",
                  {"function": name, "grid_dim_x": grid, "grid_dim_y": 1, "grid_dim_z": 1,
                   "block_dim_x": block, "block_dim_y": 1, "block_dim_z": 1, "args": args})

    def result(self, src, nbytes):
        """The request's result copy (asynchronous D2H) and the stream synchronise that brings it back."""
        assert self.call(wire.Q_MEMCPY_ASYNC, "cudaMemcpyAsyncQuery",
                         {"kind": wire.D2H, "src": src, "dst": 0x7000, "count": nbytes, "stream": bytes(8)}) is None
        back = wire.decode("AsyncResponse", self.call(wire.Q_STREAM_SYNCHRONIZE, None, {}))
        assert back["error"] == 0 and len(back["responses"]) == 1
        return np.frombuffer(back["responses"][0]["payload"], dtype=np.float32)


def make_launcher(lib, name):
    def launch(args, grid, block, shared_mem):
        bufs = [C.create_string_buffer(a, len(a)) for a in args]
        ptrs = (C.c_void_p * len(bufs))(*[C.cast(b, C.c_void_p) for b in bufs])
        rc = lib.wire_launch(name.encode(), ptrs, grid[0], block[0], shared_mem)
        assert rc == 0, f"cudaLaunchKernel({name}) failed with {rc}"
    return launch


def test_launches_run_on_rewritten_addresses(built):
    import torch
    assert torch.cuda.is_available()
    assert os.path.exists(KERNELS), "tests/lib/libwire_kernels.so is missing: run build() first"
    lib = C.CDLL(KERNELS)
    lib.wire_launch.restype = C.c_int
    lib.wire_launch.argtypes = [C.c_char_p, C.POINTER(C.c_void_p), C.c_uint, C.c_uint, C.c_ulonglong]
    torch.cuda.set_device(0)
    rng = np.random.default_rng(11)
    n = 300_000                                   # 1.2 MB of fp32: one 2 MiB model block
    w = rng.standard_normal(n).astype(np.float32)
    w2 = rng.standard_normal(n).astype(np.float32)
    x1, x2 = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)

    repo_reset()
    eng = MemoryManager(0, device=0)
    ex = wire.WireExecutor(eng)
    for k in ("wire_saxpy", "wire_scale_pair"):
        ex.kernels[k] = make_launcher(lib, k)
    cl = Client(ex)

    def first_run(func, weights, x):
        """Cold start over the wire: model.cuda(), the synchronise that ends the model, then the first
        inference, whose launches are tracked."""
        ex.signal(wire.SIG_STARTUP, func)
        wp = cl.malloc(2 * MiB)
        cl.upload(wp, weights)
        cl.call(wire.Q_DEVICE_SYNCHRONIZE, None, {})
        act = cl.malloc(4 * MiB)                    # activations: x at 0, y at 2 MiB
        cl.upload(act, x)
        cl.launch("wire_saxpy", [struct.pack("<Q", wp), struct.pack("<Q", act), struct.pack("<Q", act + 2 * MiB),
                                 struct.pack("<Q", n), struct.pack("<f", 2.0)])
        y = cl.result(act + 2 * MiB, 4 * n)
        return wp, act, y

    wp, act, y = first_run("f", w, x1)
    assert np.array_equal(y, np.float32(2.0) * w + x1)

    # f leaves; g takes over the pool blocks f had (the free list hands them out again); f comes back elsewhere
    ex.signal(wire.SIG_UNLOAD, "f")
    wp_g, act_g, y_g = first_run("g", w2, x1)
    assert np.array_equal(y_g, np.float32(2.0) * w2 + x1)
    ex.signal(wire.SIG_LOAD + 1 - 1, "f")           # Load + 1 + src, src = -1: from the host store
    ex.signal(wire.SIG_EXECUTE, "f")
    ex.launched.clear()
    # A later request allocates its activations afresh, as the client's allocator does once its cached
    # blocks went with the eviction: only the pointer words that named model parameters during the
    # first run are rewritten at launch (valid_memory_address never answers yes, memory_manager.hpp:293-298),
    # so a pointer into a cold-start workspace block would still name that block's old place.
    act2 = cl.malloc(4 * MiB)
    cl.upload(act2, x2)
    cl.launch("wire_saxpy", [struct.pack("<Q", wp), struct.pack("<Q", act2), struct.pack("<Q", act2 + 2 * MiB),
                             struct.pack("<Q", n), struct.pack("<f", 4.0)])
    y = cl.result(act2 + 2 * MiB, 4 * n)
    assert np.array_equal(y, np.float32(4.0) * w + x2)
    name, sent = ex.launched[-1]
    new_w = struct.unpack("<Q", sent[0])[0]
    assert name == "wire_saxpy" and new_w == eng.get_cuda_addr("f", wp)
    assert new_w != wp, "the weights came back at their old address: the test did not exercise the rewrite"
    assert struct.unpack("<Q", sent[1])[0] == act2 and struct.unpack("<Q", sent[2])[0] == act2 + 2 * MiB   # not parameters: as sent
    assert struct.unpack("<Q", sent[3])[0] == n and sent[4] == struct.pack("<f", 4.0)     # scalars untouched

    # pointer words inside one argument (a struct of two pointers and a count)
    ex.signal(wire.SIG_UNLOAD, "f")
    ex.signal(wire.SIG_UNLOAD, "g")
    ex.signal(wire.SIG_STARTUP, "h")
    wp_h = cl.malloc(2 * MiB)
    cl.upload(wp_h, w)
    cl.call(wire.Q_DEVICE_SYNCHRONIZE, None, {})
    act_h = cl.malloc(2 * MiB)
    pair = lambda: [struct.pack("<QQQ", wp_h, act_h, n), struct.pack("<f", 0.5)]
    cl.launch("wire_scale_pair", pair())
    assert np.array_equal(cl.result(act_h, 4 * n), np.float32(0.5) * w)
    ex.signal(wire.SIG_UNLOAD, "h")
    ex.signal(wire.SIG_LOAD + 1 - 1, "g")            # g first, so that h finds its old blocks taken
    ex.signal(wire.SIG_LOAD + 1 - 1, "h")
    ex.signal(wire.SIG_EXECUTE, "h")
    out_h = cl.malloc(2 * MiB)
    cl.launch("wire_scale_pair", [struct.pack("<QQQ", wp_h, out_h, n), struct.pack("<f", 0.25)])
    assert np.array_equal(cl.result(out_h, 4 * n), np.float32(0.25) * w)
    words = struct.unpack("<QQQ", ex.launched[-1][1][0])
    assert words[0] == eng.get_cuda_addr("h", wp_h) and words[1] == out_h and words[2] == n
    eng.close()
    repo_reset()
