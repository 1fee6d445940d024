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
