"""The C++ drop-in adapter (torpor_b200/adapter: the reference's MemoryManager class over the C
ABI) on a real GPU.  tests/adapter_gpu_probe.cpp drives it with the calls the reference's
executor makes -- cold start, evict, another function taking the freed blocks, the swap signal,
get_cuda_addr for every parameter -- and reads the bytes back from the translated addresses.
The program includes the reference's common headers, so it is compiled where those lie
(oracle/Makefile, target ref) and arrives here built."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PROBE = os.path.join(ROOT, "oracle", "_ref", "adapter_gpu_probe")


def test_adapter_swaps_on_the_gpu(built):
    if not os.path.exists(PROBE):
        pytest.skip("oracle/_ref/adapter_gpu_probe was not built (it needs the reference's headers at compile time)")
    env = dict(os.environ)
    env.pop("TORPOR_SWAP_DEVICE", None)                 # the engine runs on the GPU named by the server id: 0
    r = subprocess.run([PROBE], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env, timeout=300)
    assert r.returncode == 0 and "adapter gpu probe ok" in r.stdout, (r.returncode, r.stdout[-2000:])
    words = r.stdout.split()
    assert int(words[words.index("parameters") - 1]) > 0        # the swap-in really rebound parameters
    assert int(words[words.index("kernel") - 1]) >= 5           # every swap-in was a kernel launch of this library


EXECUTOR = os.path.join(ROOT, "oracle", "_ref", "executor_gpu_probe")


class PipeExecutor:
    """oracle/_ref/executor_gpu_probe: the reference's CUDAExecutor loop, reached over a pipe."""

    def __init__(self, exe, env):
        self.p = subprocess.Popen([exe], stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                                  text=True, env=env, bufsize=1)

    def ask(self, line):
        self.p.stdin.write(line + "\n")
        self.p.stdin.flush()
        out = []
        while True:
            ln = self.p.stdout.readline()
            if not ln:
                raise RuntimeError(f"the executor ended while answering {line[:40]!r}: {self.p.stderr.read()[-1500:]}")
            ln = ln.rstrip("\n")
            if ln == ".":
                return out
            out.append(ln)

    def handle(self, query_list: bytes):
        return [b"" if r[2:] == "-" else bytes.fromhex(r[2:]) for r in self.ask("Q " + query_list.hex())]

    def signal(self, sig, func): assert self.ask(f"S {sig} {func}") == []
    def register_kernel(self, name): assert self.ask(f"K {name}") == []
    def where(self, func, ptr): return int(self.ask(f"G {func} {ptr}")[0].split()[1])
    def stats(self): return [int(v) for v in self.ask("N")[0].split()[1:]]
    def completions(self): return [int(r[2:]) for r in self.ask("C")]

    def close(self):
        try:
            self.p.stdin.write("X\n"); self.p.stdin.flush()
            self.p.wait(60)
        finally:
            if self.p.poll() is None:
                self.p.kill()


def test_reference_executor_loop_runs_on_the_gpu_over_the_adapter(built):
    """include/server/cuda_server.hpp, unmodified and against the real CUDA runtime, with the adapter as
    its memory manager: serialised cudarpc QueryLists and controller signals drive a cold start, a
    first inference (tracked launches), an unload, another function's cold start into the freed blocks,
    a Load signal and a second inference with the client's old weight pointer.  The executor's own
    cudaLaunchKernelService rewrites the pointer word (cuda_server.hpp:1265-1268) and launches a real
    kernel; the result it sends back proves the kernel read the swapped-in bytes at their new place."""
    import struct
    import numpy as np
    from torpor_b200 import wire
    if not os.path.exists(EXECUTOR):
        pytest.skip("oracle/_ref/executor_gpu_probe was not built (it needs the reference's headers at compile time)")
    env = dict(os.environ)
    env.pop("TORPOR_SWAP_DEVICE", None)
    ex = PipeExecutor(EXECUTOR, env)
    MiB = 1 << 20
    zero_stream = bytes(8)

    def call(qtype, message, fields, raw=None):
        body = raw if raw is not None else (wire.encode(message, fields) if message else b"")
        r = ex.handle(wire.encode("QueryList", {"queries": [{"type": qtype, "client_id": 1, "query": body}]}))
        return r[0] if r else None

    def malloc(size):
        return wire.decode("cudaMallocResponse", call(wire.Q_MALLOC, "cudaMallocQuery", {"size": size}))["ptr"]

    def upload(dst, arr):
        call(wire.Q_MEMCPY_ASYNC, "cudaMemcpyAsyncQuery", {"kind": wire.H2D, "dst": dst, "count": arr.nbytes,
                                                            "payload": arr.tobytes(), "stream": zero_stream})

    def saxpy(wp, xp, yp, n, a):
        call(wire.Q_LAUNCH_KERNEL, "cudaLaunchKernelQuery",
             {"function": "wire_saxpy", "grid_dim_x": 64, "grid_dim_y": 1, "grid_dim_z": 1, "block_dim_x": 256,
              "block_dim_y": 1, "block_dim_z": 1, "stream": zero_stream,
              "args": [struct.pack("<Q", wp), struct.pack("<Q", xp), struct.pack("<Q", yp), struct.pack("<Q", n), struct.pack("<f", a)]})

    def result(src, nbytes):
        assert call(wire.Q_MEMCPY_ASYNC, "cudaMemcpyAsyncQuery",
                    {"kind": wire.D2H, "src": src, "dst": 0x7000, "count": nbytes, "stream": zero_stream}) is None
        back = wire.decode("AsyncResponse", call(wire.Q_STREAM_SYNCHRONIZE, None, None, raw=zero_stream))
        assert back["error"] == 0 and len(back["responses"]) == 1
        return np.frombuffer(back["responses"][0]["payload"], dtype=np.float32)

    try:
        ex.register_kernel("wire_saxpy")
        rng = np.random.default_rng(23)
        n = 300_000
        w1, w2 = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
        x1, x2 = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)

        def first_run(func, weights, x):
            ex.signal(wire.SIG_STARTUP, func)
            wp = malloc(2 * MiB)
            upload(wp, weights)
            assert call(wire.Q_DEVICE_SYNCHRONIZE, None, {}) is not None
            act = malloc(4 * MiB)
            upload(act, x)
            saxpy(wp, act, act + 2 * MiB, n, 2.0)
            y = result(act + 2 * MiB, 4 * n)
            assert ex.completions() == [0]
            return wp, y

        wp1, y = first_run("1", w1, x1)                   # the executor takes function names for client ids (stoi)
        assert np.array_equal(y, np.float32(2.0) * w1 + x1)
        ex.signal(wire.SIG_UNLOAD, "1")
        wp2, y = first_run("2", w2, x1)
        assert np.array_equal(y, np.float32(2.0) * w2 + x1)
        launches_before = ex.stats()[0]
        ex.signal(wire.SIG_LOAD + 1 - 1, "1")             # Load + 1 + src with src = -1: from the host store
        ex.signal(wire.SIG_EXECUTE, "1")
        act2 = malloc(4 * MiB)                            # a later request allocates its activations afresh
        upload(act2, x2)
        saxpy(wp1, act2, act2 + 2 * MiB, n, 4.0)          # the client's OLD weight pointer
        y = result(act2 + 2 * MiB, 4 * n)
        assert np.array_equal(y, np.float32(4.0) * w1 + x2)
        assert ex.where("1", wp1) != wp1, "the weights came back at their old address: nothing was rewritten"
        assert ex.stats()[0] > launches_before            # the Load signal was a kernel launch of this library
    finally:
        ex.close()
