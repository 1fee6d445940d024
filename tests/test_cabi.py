"""The C ABI: the library loads without a GPU, exports every symbol the header declares,
and fails loudly -- no CPU data path -- when asked to move bytes without a device."""
import ctypes
import os
import re

import pytest

from torpor_b200 import _cabi
from torpor_b200.memory_manager import MemoryManager, SwapError

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "torpor_swap.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tsw_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree(built):
    decl = declared_symbols()
    assert len(decl) >= 40
    assert sorted(_cabi.SIGNATURES) == decl


def test_library_exports_every_declared_symbol(built):
    lib = ctypes.CDLL(_cabi.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(lib, name), name


def test_version_and_default_config(built):
    L = _cabi.lib()
    assert b"sm_100a" in L.tsw_version()
    cfg = _cabi.Config()
    L.tsw_config_default(ctypes.byref(cfg))
    assert cfg.budget_bytes == 25 << 30 and cfg.pool_policy == _cabi.POOL_BUDDY and cfg.gpu_count == 1


def test_no_oracle_in_the_product():
    """Nothing under the package may import, load, link or name the checkers."""
    pkg = os.path.join(ROOT, "torpor_b200")
    for dirpath, _, files in os.walk(pkg):
        for fn in files:
            if fn.endswith((".py", ".cpp", ".cu", ".hpp", ".h")) or fn == "Makefile":
                text = open(os.path.join(dirpath, fn), errors="replace").read().lower()
                for word in ("oracle", "tso_", "libtorpor_ref", "_work/"):
                    assert word not in text, (os.path.join(dirpath, fn), word)


def test_cuda_engine_without_a_device_fails_loudly(built):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(SwapError) as e:
        MemoryManager(0, device=0)
    assert e.value.code in (_cabi.ERR_NO_DEVICE, _cabi.ERR_CUDA)
