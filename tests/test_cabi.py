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


def test_null_arguments_are_refused_not_dereferenced(built):
    """Every entry point, called with null for every pointer and zero for every number, answers with an
    error (or does nothing) -- in a child process, so that a crash would be seen and not end the run."""
    import subprocess
    import sys
    child = r'''
import ctypes as C, sys
sys.path.insert(0, sys.argv[1])
from torpor_b200 import _cabi
L = _cabi.lib()
noop = {"signal": _cabi.SIGNAL_FN(lambda *a: None), "ack": _cabi.ACK_FN(lambda *a: None)}
for name, (res, args) in _cabi.SIGNATURES.items():
    vals = []
    for a in args:
        if a is _cabi.SIGNAL_FN: vals.append(noop["signal"])
        elif a is _cabi.ACK_FN: vals.append(noop["ack"])
        elif a in (C.c_void_p, C.c_char_p) or (isinstance(a, type) and issubclass(a, C._Pointer)): vals.append(None)
        else: vals.append(0)
    r = getattr(L, name)(*vals)
    if name in ("tsw_last_error", "tsw_version"):
        assert isinstance(r, bytes)
    elif res is not None:
        assert r <= 0, (name, r)
print("all refused")
'''
    r = subprocess.run([sys.executable, "-c", child, ROOT], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=120)
    assert r.returncode == 0 and "all refused" in r.stdout, (r.returncode, r.stdout[-500:], r.stderr[-1500:])
