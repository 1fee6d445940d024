"""The library's host code (allocator, tables, policies, C ABI) under AddressSanitizer +
UndefinedBehaviorSanitizer and under ThreadSanitizer, driven by tests/host_stress.cpp from
several threads on plan-only engines.  The reference has no such check and shares its tables
between threads without locks (include/server/model_repo.hpp:180-185)."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = [os.path.join(ROOT, "tests", "host_stress.cpp")] + [os.path.join(ROOT, "torpor_b200", "csrc", f)
                                                            for f in ("engine.cpp", "engine_swap.cpp", "engine_share.cpp", "pool.cpp", "evictor.cpp", "scheduler.cpp", "controller.cpp")]


@pytest.mark.parametrize("name,flags", [("asan_ubsan", "-fsanitize=address,undefined"), ("tsan", "-fsanitize=thread")])
def test_host_code_is_clean_under_sanitizers(tmp_path, name, flags):
    if not os.path.exists("/usr/local/cuda/include/cuda_runtime.h"):
        pytest.skip("CUDA headers not present")
    exe = str(tmp_path / f"host_stress_{name}")
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", *flags.split(), "-pthread", "-o", exe, *SRC,
           "-I/usr/local/cuda/include", "-L/usr/local/cuda/lib64", "-lcudart", "-lrt", "-ldl"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert r.returncode == 0, r.stdout[-3000:]
    env = dict(os.environ, LD_LIBRARY_PATH="/usr/local/cuda/lib64:" + os.environ.get("LD_LIBRARY_PATH", ""),
               ASAN_OPTIONS="detect_leaks=0:abort_on_error=0", TSAN_OPTIONS="halt_on_error=0:report_signal_unsafe=0",
               UBSAN_OPTIONS="print_stacktrace=1")
    r = subprocess.run([exe, "30"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env, timeout=600)
    out = r.stdout
    assert r.returncode == 0 and "host stress ok" in out, out[-4000:]
    for bad in ("ERROR: AddressSanitizer", "runtime error:", "WARNING: ThreadSanitizer"):
        assert bad not in out, out[-4000:]
