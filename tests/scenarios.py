"""Scenario scripts replayed against every implementation of the swap path.

A scenario is a list of executor-level operations (cold start, evict, swap-in,
workspace malloc/free, pointer translation).  ``run`` replays it on a backend and
records, after every step, the canonical block table, parameter table and
translations of the model the step touched.  Two backends produce identical
records iff they made the same placement decisions and rebound the pointer
table identically.

Backends:
  TsoBackend("ref_fake")   the reference's own headers over a host-memory CUDA stand-in
  TsoBackend("oracle")     the CPU restatement under oracle/
  EngineBackend(device)    the shipped engine; device=-1 is the plan-only engine
"""
from __future__ import annotations

import os
import sys
from typing import Callable, Dict, List, Optional

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from torpor_b200 import workloads as W  # noqa: E402

MiB = 1 << 20
GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


# ------------------------------------------------------------------ backends

class TsoBackend:
    def __init__(self, kind: str):
        from oracle import tso
        self.kind = kind
        self.lib = tso.load(kind)
        self.managers = {}

    def reset(self):
        for m in self.managers.values():
            m.close()
        self.managers = {}
        self.lib.reset_world()

    def manager(self, server_id=0, budget=0, gpu_count=1, block_manager="Buddy"):
        m = self.lib.manager(server_id=server_id, budget=budget, gpu_count=gpu_count, block_manager=block_manager)
        self.managers[server_id] = m
        return m

    def set_status(self, func, gpu, full):
        self.lib.set_model_status(func, gpu, full)

    def total_size(self, func):
        return self.lib.total_size(func)

    def blocks(self, m, f):
        return m.dump_blocks(f)

    def params(self, m, f):
        return m.dump_params(f)

    def canon(self, m, addr):
        return addr


class EngineBackend:
    def __init__(self, device: int = -1, **engine_kw):
        from torpor_b200 import memory_manager as MM
        self.MM = MM
        self.device = device
        self.engine_kw = engine_kw
        self.managers = {}

    def reset(self):
        for m in self.managers.values():
            m.close()
        self.managers = {}
        self.MM.repo_reset()

    def manager(self, server_id=0, budget=0, gpu_count=1, block_manager="Buddy"):
        dev = self.device if self.device < 0 else self.device
        m = self.MM.MemoryManager(budget, device=dev, server_id=server_id, gpu_count=gpu_count,
                                  block_manager=block_manager, **self.engine_kw)
        self.managers[server_id] = m
        return m

    def set_status(self, func, gpu, full):
        if full:
            self.MM.ModelRepo.add_model_info(func, gpu)
        else:
            self.MM.ModelRepo.remove_model_info(func, gpu)

    def total_size(self, func):
        return self.MM.ModelRepo.total_size(func)

    def blocks(self, m, f):
        return m.dump_blocks(f, canonical=True)

    def params(self, m, f):
        return m.dump_params(f, canonical=True)


# ------------------------------------------------------------------ recording

class Recorder:
    def __init__(self, backend):
        self.b = backend
        self.out: Dict[str, np.ndarray] = {}
        self.step = 0
        self.loaded: Dict[str, W.LoadedModel] = {}

    def snap(self, m, f, tag):
        key = f"{self.step:03d}_{tag}_{f}_s{m.server_id}"
        self.out[key + "_blocks"] = self.b.blocks(m, f).copy()
        self.out[key + "_params"] = self.b.params(m, f).copy()
        self.step += 1

    def scalar(self, tag, value):
        self.out[f"{self.step:03d}_{tag}"] = np.array([value], dtype=np.uint64)
        self.step += 1


def _zeros(ws):
    return lambda i: np.zeros(ws.tensors[i].nbytes, dtype=np.uint8)


def cold(rec: Recorder, m, f, ws_name, workspace=(W.SMALL_BLOCK,), data=None, access=None):
    ws = W.weight_set(ws_name)
    if access is None:
        lm = W.cold_start(m, f, ws, tensor_data=data or _zeros(ws), workspace_blocks=workspace)
    else:
        lm = cold_start_partial(m, f, ws, data or _zeros(ws), workspace, access)
    rec.loaded[f] = lm
    rec.snap(m, f, "cold")
    return lm


def cold_start_partial(mgr, func, ws, tensor_data, workspace_blocks, access: Callable[[int], bool]):
    """Cold start where only tensors with ``access(i)`` are touched by the first run."""
    blocks, _ = W.pack_blocks(ws)
    bv = [0] * len(blocks)
    wv: List[int] = []
    tv = [0] * len(ws.tensors)
    mgr.track_begin(func)
    for c in W.cold_start_stream(ws, workspace_blocks):
        if c.op == "malloc":
            p = mgr.malloc(func, c.size, c.is_model)
            if c.is_model:
                bv[c.block] = p
            else:
                wv.append(p)
        elif c.op == "memcpy":
            tv[c.tensor] = bv[c.block] + c.offset
            assert mgr.memcpy_h2d_model(func, tv[c.tensor], tensor_data(c.tensor)) == 0
        elif c.op == "sync_done":
            mgr.sync_done(func)
        elif c.op == "access" and access(c.tensor):
            mgr.mark_access(tv[c.tensor])
    mgr.track_end(func)
    return W.LoadedModel(func, ws, bv, wv, tv)


def evict(rec, m, f):
    m.evict(f)
    rec.snap(m, f, "evict")


def swap_in(rec, m, f, src=-1):
    m.swap_in(f, src)
    m.wait_ready(f)
    rec.snap(m, f, "in")


# ------------------------------------------------------------------ scenarios

def s_mixed5(b, rec):
    m = b.manager(budget=0)
    names = ["resnet50", "bert_tiny", "llama_tiny", "vgg19", "bert_base"]
    for k, n in enumerate(names):
        cold(rec, m, f"f{k}", n)
    for k in range(len(names)):
        evict(rec, m, f"f{k}")
    for k in reversed(range(len(names))):
        swap_in(rec, m, f"f{k}")
    evict(rec, m, "f1")
    swap_in(rec, m, "f1")
    for k in range(len(names)):
        rec.scalar(f"check_alloc_f{k}", int(m.check_alloc(f"f{k}")))
        rec.scalar(f"total_size_f{k}", b.total_size(f"f{k}"))


def _churn(b, rec, block_manager, n_ops, seed):
    m = b.manager(budget=0, block_manager=block_manager)
    names = ["resnet50", "bert_tiny", "llama_tiny", "bert_tiny", "resnet50", "llama_tiny", "bert_base"]
    resident = {}
    for k, n in enumerate(names):
        cold(rec, m, f"f{k}", n)
        resident[f"f{k}"] = True
    rng = np.random.default_rng(seed)
    for _ in range(n_ops):
        f = f"f{int(rng.integers(0, len(names)))}"
        if resident[f]:
            evict(rec, m, f)
            resident[f] = False
        else:
            swap_in(rec, m, f)
            resident[f] = True
    for f in resident:
        rec.snap(m, f, "final")


def s_churn_buddy(b, rec):
    _churn(b, rec, "Buddy", 48, 7)


def s_churn_fixed(b, rec):
    _churn(b, rec, "Fixed", 24, 8)


def s_workspace(b, rec):
    """Workspace blocks of every size class, freed and re-requested; pointer translation
    of parameters, block bases and interior pointers across an evict / swap-in cycle."""
    m = b.manager(budget=0)
    ws_sizes = (2 * MiB, 20 * MiB, 48 * MiB, 100 * MiB, 200 * MiB)
    lm = cold(rec, m, "w", "llama_tiny", workspace=ws_sizes)
    cold(rec, m, "other", "bert_tiny")
    probes = [lm.tensor_vaddr[0], lm.tensor_vaddr[5], lm.tensor_vaddr[5] + 4096, lm.block_vaddr[0], lm.block_vaddr[0] + 512,
              lm.workspace_vaddr[0], lm.workspace_vaddr[2] + 12345, lm.workspace_vaddr[4] + (150 * MiB), 0x1234]

    def probe(tag):
        for rnd in range(2):  # an unknown interior pointer is translated only from the second look on
            vals = [_canon_translate(b, m, "w", p) for p in probes]
            rec.out[f"{rec.step:03d}_{tag}_translate{rnd}"] = np.array(vals, dtype=np.uint64)
            rec.step += 1
        rec.scalar(tag + "_is_model", sum(int(m.is_model_address("w", p)) << i for i, p in enumerate(probes)))

    probe("resident")
    m.free("w", lm.workspace_vaddr[1])
    rec.snap(m, "w", "free")
    p_new = m.malloc("w", 2 * MiB, False)
    rec.snap(m, "w", "malloc")
    evict(rec, m, "w")
    evict(rec, m, "other")
    probe("evicted")
    swap_in(rec, m, "other")
    swap_in(rec, m, "w")
    probes.append(p_new)
    probe("back")
    rec.scalar("check_alloc", int(m.check_alloc("w")))


def _canon_translate(b, m, f, p):
    """Translate and express the answer relative to the canonical space, so that CUDA
    engines (whose pool sits at a driver-chosen address) compare with the checkers."""
    out = m.translate(f, p)
    if isinstance(b, EngineBackend):
        return m.canonical_address(f, out)
    return out


def s_partial_access(b, rec):
    m = b.manager(budget=0)
    cold(rec, m, "p", "resnet50", access=lambda i: i % 3 != 1)
    cold(rec, m, "q", "bert_tiny", access=lambda i: i < 10)
    evict(rec, m, "p")
    evict(rec, m, "q")
    swap_in(rec, m, "q")
    swap_in(rec, m, "p")
    evict(rec, m, "p")
    swap_in(rec, m, "p")


def s_two_gpu(b, rec):
    """Replica swap between two GPUs of one process, and the fall-back to the host store
    when the source replica is not marked healthy (memory_manager.hpp:213-224)."""
    m0 = b.manager(server_id=0, budget=0, gpu_count=2)
    m1 = b.manager(server_id=1, budget=0, gpu_count=2)
    cold(rec, m0, "a", "resnet50")
    cold(rec, m1, "b", "llama_tiny")
    b.set_status("a", 0, True)
    swap_in(rec, m1, "a", src=0)         # peer copy
    rec.snap(m0, "a", "src_after")
    swap_in(rec, m0, "b", src=1)         # source not marked Full: falls back to the host store
    evict(rec, m1, "a")
    b.set_status("a", 0, False)
    swap_in(rec, m1, "a", src=0)         # unhealthy again
    evict(rec, m0, "a")
    swap_in(rec, m0, "a")
    b.set_status("b", 1, True)
    evict(rec, m0, "b")
    swap_in(rec, m0, "b", src=1)


SCENARIOS = {
    "mixed5": s_mixed5,
    "churn_buddy": s_churn_buddy,
    "churn_fixed": s_churn_fixed,
    "workspace": s_workspace,
    "partial_access": s_partial_access,
    "two_gpu": s_two_gpu,
}


def run(backend, name: str) -> Dict[str, np.ndarray]:
    backend.reset()
    rec = Recorder(backend)
    try:
        SCENARIOS[name](backend, rec)
    finally:
        backend.reset()
    return rec.out


def golden_path(name: str) -> str:
    return os.path.join(GOLDEN_DIR, f"scenario_{name}.npz")


def load_golden(name: str) -> Dict[str, np.ndarray]:
    with np.load(golden_path(name)) as z:
        return {k: z[k] for k in z.files}


def assert_same(got: Dict[str, np.ndarray], want: Dict[str, np.ndarray], what: str = "") -> None:
    assert sorted(got.keys()) == sorted(want.keys()), f"{what}: step lists differ"
    for k in sorted(want.keys()):
        if not np.array_equal(got[k], want[k]):
            g, w = got[k], want[k]
            detail = f"shape {g.shape} vs {w.shape}"
            if g.shape == w.shape and g.ndim == 2:
                rows = np.nonzero((g != w).any(axis=1))[0]
                r = int(rows[0])
                detail = f"first differing row {r}: got {[hex(int(v)) for v in g[r]]} want {[hex(int(v)) for v in w[r]]}"
            raise AssertionError(f"{what}: step {k} differs ({detail})")
