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
