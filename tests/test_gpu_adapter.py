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
