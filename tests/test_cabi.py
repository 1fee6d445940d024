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


def header_struct_fields(name):
    """Member names and C types of `typedef struct { ... } <name>;` in the header, in order."""
    text = open(os.path.join(ROOT, "include", "torpor_swap.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    body = re.search(r"typedef\s+struct\s*\{([^}]*)\}\s*" + name + r"\s*;", text).group(1)
    out = []
    for decl in body.split(";"):
        decl = " ".join(decl.split())
        if not decl:
            continue
        m = re.match(r"((?:const )?(?:unsigned )?\w+\s*\*?)\s*(.+)$", decl)
        ctype = m.group(1).replace(" *", "*").strip()
        for d in m.group(2).split(","):
            d = d.strip()
            arr = re.match(r"(\w+)(\[\d+\])$", d)
            out.append((arr.group(1), ctype + arr.group(2)) if arr else (d, ctype))
    return out


@pytest.mark.parametrize("c_name,binding", [("tsw_config", "Config"), ("tsw_segment", "Segment"),
                                            ("tsw_publish", "Publish"), ("tsw_ipc_region", "IpcRegion")])
def test_struct_layouts_of_header_and_binding_agree(c_name, binding):
    """Every struct that crosses the C ABI has the same members, in the same order and of the same
    width, in include/torpor_swap.h and in the ctypes binding."""
    width = {"int": 4, "uint32_t": 4, "uint64_t": 8, "const char*": 8, "unsigned char[64]": 64}
    fields = header_struct_fields(c_name)
    cls = getattr(_cabi, binding)
    assert [f[0] for f in fields] == [f[0] for f in cls._fields_]
    for (name, ctype), bound in zip(fields, cls._fields_):
        assert width[ctype] == ctypes.sizeof(bound[1]), (name, ctype)


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


def test_random_calls_with_wild_values_never_crash(built):
    """Random calls on two plan-only engines with unknown functions, wild pointers and sizes, calls out of
    order: errors are fine, a crash is not.  Run in child processes (six seeds)."""
    import subprocess
    import sys
    child = r'''
import sys, ctypes as C, random
sys.path.insert(0, sys.argv[2])
import numpy as np
from torpor_b200 import _cabi
from torpor_b200.memory_manager import MemoryManager, repo_reset, SwapError, Evictor, Scheduler, Controller
seed = int(sys.argv[1]); rnd = random.Random(seed)
repo_reset()
ms = [MemoryManager(0, device=-1, server_id=g, gpu_count=2, block_manager=rnd.choice(["Buddy", "Fixed"])) for g in range(2)]
funcs = ["a", "b", "c", "", "zz"]
ptrs = [0, 1, 0x600000000000, 0x600138000000, 2**63, 2**64 - 1]
sizes = [0, 1, 512, 2 << 20, 20 << 20, 48 << 20, 130 << 20, (1 << 40), 2**63]
def pick(xs): return rnd.choice(xs)
for step in range(600):
    m = pick(ms); f = pick(funcs)
    op = rnd.randrange(16)
    try:
        if op == 0: m.track_begin(f)
        elif op == 1: m.track_end(f)
        elif op == 2:
            p = m.malloc(f, pick(sizes[:7]), rnd.random() < 0.5); ptrs.append(p); ptrs.append(p + pick([0, 8, 512, 4096]))
        elif op == 3: m.free(f, pick(ptrs))
        elif op == 4: m.memcpy_h2d_model(f, pick(ptrs), np.zeros(pick([0, 1, 64, 4096]), dtype=np.uint8))
        elif op == 5: m.sync_done(f)
        elif op == 6: m.mark_access(pick(ptrs))
        elif op == 7: m.swap_in(f, pick([-1, 0, 1, 5, -7]))
        elif op == 8: m.evict(f)
        elif op == 9: m.get_cuda_addr(f, pick(ptrs), timeout_ns=1000000) if hasattr(m, "get_cuda_addr") else None
        elif op == 10: m.dump_blocks(f); m.dump_params(f, canonical=True)
        elif op == 11: m.check_alloc(f); m.is_model_address(f, pick(ptrs)); m.valid_memory_address(f, pick(ptrs))
        elif op == 12: m.poll_ready(f)
        elif op == 13: m.swap_in_sharded(f, [x for x in ms if x is not m])
        elif op == 14: m.swap_plan(f); m.swap_commit(f)
        elif op == 15: m.canonical_address(f, pick(ptrs))
    except (SwapError, RuntimeError, ValueError, OverflowError, C.ArgumentError):
        pass
for m in ms: m.close()
repo_reset()
print("ok", seed)
'''
    for seed in range(6):
        r = subprocess.run([sys.executable, "-c", child, str(seed), ROOT], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=300)
        assert r.returncode == 0 and f"ok {seed}" in r.stdout, (seed, r.returncode, r.stderr[-1500:])
