"""The header-only C++ adapter (torpor_b200/adapter) keeps the reference's class names,
method names and argument lists: it is compiled here against the reference's own common
headers, in place of include/server/{memory_manager,model_repo,evictor}.hpp, and run on a
plan-only engine.  Needs the reference tree and the CUDA headers at compile time."""
import os
import subprocess
import sysconfig

import pytest

from torpor_b200 import _cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("TORPOR_REFERENCE", "/root/reference")   # same default as oracle/Makefile's REF


def test_adapter_compiles_against_reference_headers_and_runs(built, tmp_path):
    if not os.path.exists(os.path.join(REF, "common", "include", "utils.hpp")):
        pytest.skip("reference tree not present")
    spdlog = os.path.join(sysconfig.get_paths()["purelib"], "flashinfer", "data", "spdlog", "include")
    exe = str(tmp_path / "adapter_probe")
    cmd = ["g++", "-std=c++17", "-O1", "-w", "-o", exe, os.path.join(ROOT, "tests", "adapter_probe.cpp"),
           "-I" + os.path.join(ROOT, "torpor_b200", "adapter"), "-I" + os.path.join(ROOT, "include"),
           "-I" + os.path.join(ROOT, "oracle", "ref_shim"),          # cuda_common.hpp without protoc
           "-I" + os.path.join(REF, "common", "include"), "-I" + spdlog, "-I/usr/local/cuda/include",
           "-L" + os.path.dirname(_cabi.LIB_PATH), "-ltorpor_swap", "-Wl,-rpath," + os.path.dirname(_cabi.LIB_PATH),
           "-L/usr/local/cuda/lib64", "-lcudart", "-pthread"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert r.returncode == 0, r.stdout[-3000:]
    env = dict(os.environ, LD_LIBRARY_PATH="/usr/local/cuda/lib64:" + os.environ.get("LD_LIBRARY_PATH", ""))
    r = subprocess.run([exe], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    assert r.returncode == 0 and "adapter probe ok" in r.stdout, (r.returncode, r.stdout[-2000:])


class _PipeSide:
    """The probe's manager and controller behind the method names tests/controller_cases.py drives."""

    def __init__(self, exe, env):
        self.p = subprocess.Popen([exe], stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env, bufsize=1)

    def ask(self, line):
        self.p.stdin.write(line + "\n")
        self.p.stdin.flush()
        out = []
        while True:
            ln = self.p.stdout.readline()
            if not ln:
                raise RuntimeError(f"probe ended while answering {line!r}")
            ln = ln.rstrip("\n")
            if ln == ".":
                return out
            out.append(ln)

    # manager side (controller_cases.register_sizes)
    def track_begin(self, f): assert self.ask(f"T {f}") == []
    def malloc(self, f, size, is_model): assert self.ask(f"M {f} {size} {1 if is_model else 0}") == []
    def track_end(self, f): assert self.ask(f"U {f}") == []
    # controller side (controller_cases.drive)
    def request(self, kind, func, payload=""): return self.ask(f"R {kind} {func} {payload}")
    def complete(self, executor): return self.ask(f"C {executor}")

    def close(self):
        try:
            self.p.stdin.write("Q\n"); self.p.stdin.flush()
            self.p.wait(30)
        finally:
            if self.p.poll() is None:
                self.p.kill()


def test_reference_controller_runs_unchanged_on_the_adapter(built, tmp_path):
    """include/server/controller.hpp, compiled where it lies with the adapter's model_repo.hpp and
    evictor.hpp in place of its own (and the adapter's MemoryManager registering the models on a
    plan-only engine), sends exactly what the reference alone sent when the recordings were made."""
    import json
    import sys
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import controller_cases as CC
    if not os.path.exists(os.path.join(REF, "include", "server", "controller.hpp")):
        pytest.skip("reference tree not present")
    spdlog = os.path.join(sysconfig.get_paths()["purelib"], "flashinfer", "data", "spdlog", "include")
    exe = str(tmp_path / "controller_on_adapter")
    cmd = ["g++", "-std=c++17", "-O1", "-w", "-DTORPOR_REF_FAKE_CUDA", "-DTORPOR_REF_WITH_CONTROLLER", "-o", exe,
           os.path.join(ROOT, "tests", "controller_on_adapter.cpp"),
           "-I" + os.path.join(ROOT, "torpor_b200", "adapter"), "-I" + os.path.join(ROOT, "include"),
           "-I" + os.path.join(ROOT, "oracle", "ref_shim_ctrl"), "-I" + os.path.join(ROOT, "oracle", "ref_shim"),
           "-I" + os.path.join(REF, "common", "include"), "-I" + os.path.join(REF, "include", "server"), "-I" + spdlog,
           "-L" + os.path.dirname(_cabi.LIB_PATH), "-ltorpor_swap", "-Wl,-rpath," + os.path.dirname(_cabi.LIB_PATH), "-pthread"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert r.returncode == 0, r.stdout[-3000:]
    env = dict(os.environ, LD_LIBRARY_PATH="/usr/local/cuda/lib64:" + os.environ.get("LD_LIBRARY_PATH", ""))
    for sp, ep in CC.COMBOS:
        with open(os.path.join(ROOT, "tests", "golden", f"controller_{sp}_{ep}.json")) as f:
            want = json.load(f)
        for seed, w in zip(CC.SEEDS, want):
            side = _PipeSide(exe, env)                 # a fresh process: fresh repository, rand() reseeded
            try:
                CC.register_sizes(side, CC.model_blocks(seed))
                assert side.ask(f"N {CC.limit_of(seed) >> 30} {sp} {ep}") == []
                got = CC.drive(side, seed)
            finally:
                side.close()
            assert got == w, f"{sp}/{ep} seed {seed}"


class _PipeExecutor:
    """tests/executor_on_adapter.cpp behind the method names of the checker's executor (oracle/tso.py)."""

    def __init__(self, exe, env):
        self.p = subprocess.Popen([exe], stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                                  text=True, env=env, bufsize=1)

    def ask(self, line):
        self.p.stdin.write(line + "\n")
        self.p.stdin.flush()
        out = []
        while True:
            ln = self.p.stdout.readline()
            if not ln:
                raise RuntimeError(f"probe ended while answering {line[:40]!r}")
            ln = ln.rstrip("\n")
            if ln == ".":
                return out
            out.append(ln)

    def register_kernel(self, name): self.ask(f"K {name}")
    def signal(self, sig, func): self.ask(f"S {sig} {func}")
    def handle(self, query_list): return [b"" if r[2:] == "-" else bytes.fromhex(r[2:]) for r in self.ask("Q " + query_list.hex())]
    def completions(self): return [int(r[2:]) for r in self.ask("C")]

    def launches(self):
        out = []
        for r in self.ask("L"):
            parts = r.split(" ")
            out.append((parts[1], [b"" if a == "-" else bytes.fromhex(a) for a in parts[2:]]))
        return out

    # the engine's tables, as the manager handle of the checker gives them
    def _table(self, op, f, width):
        import numpy as np
        rows = [[int(v) for v in r.split(" ")[1:]] for r in self.ask(f"{op} {f}")]
        return np.array(rows, dtype=np.uint64).reshape(len(rows), width)

    def dump_blocks(self, f): return self._table("B", f, 6)
    def dump_params(self, f): return self._table("P", f, 7)
    def check_alloc(self, f): return self.ask(f"A {f}") == ["A 1"]
    def wait_ready(self, f): return 0

    def close(self):
        try:
            self.p.stdin.write("X\n"); self.p.stdin.flush()
            self.p.wait(30)
        finally:
            if self.p.poll() is None:
                self.p.kill()


def test_reference_executor_runs_unchanged_on_the_adapter(built, tmp_path):
    """include/server/cuda_server.hpp, compiled where it lies with the adapter's memory_manager.hpp in
    place of its own, over a plan-only engine: driven with random client streams and controller signals
    it answers, launches and ends up exactly as the reference's executor over the reference's manager."""
    import sys
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from oracle import tso
    import scenarios
    import test_executor_differential as TE
    from test_random_differential import random_stream, replay, reuses_a_block_name
    from torpor_b200 import wire
    if not os.path.exists(os.path.join(REF, "include", "server", "cuda_server.hpp")) or not tso.available("ref_exec"):
        pytest.skip("reference tree not present")
    spdlog = os.path.join(sysconfig.get_paths()["purelib"], "flashinfer", "data", "spdlog", "include")
    exe = str(tmp_path / "executor_on_adapter")
    cmd = ["g++", "-std=c++17", "-O1", "-w", "-DTORPOR_REF_FAKE_CUDA", "-DTORPOR_REF_WITH_EXECUTOR", "-o", exe,
           os.path.join(ROOT, "tests", "executor_on_adapter.cpp"),
           "-I" + os.path.join(ROOT, "torpor_b200", "adapter"), "-I" + os.path.join(ROOT, "include"),
           "-I" + os.path.join(ROOT, "oracle", "ref_shim_exec"), "-I" + os.path.join(ROOT, "oracle", "_ref", "gen"),
           "-I" + os.path.join(ROOT, "oracle", "ref_shim"),
           "-I" + os.path.join(REF, "common", "include"), "-I" + os.path.join(REF, "include", "server"), "-I" + spdlog,
           "-L" + os.path.dirname(_cabi.LIB_PATH), "-ltorpor_swap", "-Wl,-rpath," + os.path.dirname(_cabi.LIB_PATH), "-pthread"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert r.returncode == 0, r.stdout[-3000:]

    class AdapterExecutorBackend:
        def __init__(self):
            self.ex, self.log = None, []

        def reset(self):
            if self.ex:
                self.ex.close()
                self.ex = None

        def manager(self, server_id=0, budget=0, gpu_count=1, block_manager="Buddy"):
            env = dict(os.environ, BLOCK_MANAGER=block_manager,
                       LD_LIBRARY_PATH="/usr/local/cuda/lib64:" + os.environ.get("LD_LIBRARY_PATH", ""))
            self.ex = _PipeExecutor(exe, env)
            self.ex.register_kernel("k")
            ex = self.ex

            def complete():
                ex.handle(wire.encode("QueryList", {"queries": [{"type": wire.Q_MEMCPY_ASYNC, "client_id": 1, "query": wire.encode(
                    "cudaMemcpyAsyncQuery", {"kind": wire.D2H, "src": 0x600000000000, "dst": 0x7000, "count": 0, "stream": bytes(8)})}]}))
                assert ex.completions() == [0]
            m = TE.ExecutorAsManager(ex, ex, complete, self.log)
            m.seen = set()
            return m

        def blocks(self, m, f): return m.dump_blocks(f)
        def params(self, m, f): return m.dump_params(f)

    compared = 0
    for block_manager in ("Buddy", "Fixed"):
        for seed in range(12):
            ops = random_stream(seed, block_manager)
            if reuses_a_block_name(ops):
                continue
            ref, mine = TE.ReferenceExecutorBackend(tso.load("ref_exec")), AdapterExecutorBackend()
            want = replay(ref, ops)
            got = replay(mine, ops)
            scenarios.assert_same(got, want, f"executor on the adapter, seed {seed} / {block_manager}")
            assert [m for m, _ in mine.log] == [m for m, _ in ref.log]
            assert not [i for i, ((_, a), (_, b)) in enumerate(zip(mine.log, ref.log)) if a != b]
            compared += 1
    assert compared >= 12
