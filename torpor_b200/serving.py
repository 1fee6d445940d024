"""Controller-level replay of a serverless request stream over the swap engines.

Every request goes through the library's controller (``tsw_ctrl_*``, the request handling of
include/server/controller.hpp:130-262,392-453): it asks the scheduler for a GPU and a source,
pins the source replica, lets the eviction policy make room (victims are unloaded first) and
signals the load; on completion it registers the new replica, releases the pin and serves its
queue.  This module is the executor side: it carries those signals out on real engines.
Swap-ins are asynchronous (``tsw_swap_in`` returns once the kernel is enqueued), so swaps on
different GPUs overlap for real and compete for PCIe / NVLink as they would in service.
Requests arrive on the wall clock (optionally compressed by ``speedup``); the client's
inference itself is not run -- it is modelled as ``exec_ms`` of GPU occupancy per request,
a stated constant per architecture, because only the swap path is under test.

    python -m torpor_b200.serving --gpus 8 --models 64 --rate 200 --duration 120 --cap-gb 40
"""
from __future__ import annotations

import argparse
import collections
import json
import time
from typing import Dict, List, Optional

import numpy as np

from . import workloads as W
from .memory_manager import (Controller, MemoryManager, repo_reset, REQ_EXECUTE, REQ_EXECUTE_AFTER_LOAD,
                             SIGNAL_EXECUTE, SIGNAL_LOAD, SIGNAL_STARTUP, SIGNAL_UNLOAD)

# GPU occupancy per request once the weights are there (ms).  Stand-ins for the client's
# inference, in the range the reference's own node simulator uses (misc/tools/node_simu.py:98-99).
EXEC_MS = {"resnet50": 8.0, "bert_base": 12.0, "bert_large": 25.0, "vgg19": 12.0,
           "bert_tiny": 2.0, "llama_tiny": 4.0, "llama_mid": 20.0, "llama2_7b": 30.0}
LEVEL = {"resnet50": 0, "bert_tiny": 0, "bert_base": 1, "vgg19": 1, "llama_tiny": 1, "bert_large": 2,
         "llama_mid": 2, "llama2_7b": 2}


class SwapServer:
    """N engines under the library's controller (``tsw_ctrl_*``): this class only carries out the
    signals the controller sends -- unload, load (from the host store or a replica), execute -- on
    real engines, and reports completions back, as the reference's executors do
    (include/server/cuda_server.hpp:243-300)."""

    def __init__(self, n_gpus: int, cap_bytes: int, evict_policy: str = "LRU", sched_policy: str = "IA",
                 devices: Optional[List[int]] = None, host_arena_bytes: int = 0, pcie_pairs=None, nvlink=None,
                 shard_min_bytes: int = 0):
        self.n = n_gpus
        self.devices = devices or list(range(n_gpus))
        self.engines = [MemoryManager(cap_bytes, device=self.devices[g], server_id=g, gpu_count=n_gpus,
                                      host_arena_bytes=host_arena_bytes if g == 0 else 0)
                        for g in range(n_gpus)]
        self.ctrl = Controller(n_gpus, cap_bytes, sched_policy, evict_policy, pcie_pairs, nvlink)
        self.arch: Dict[str, str] = {}
        self.nbytes: Dict[str, int] = {}
        self.state = [dict(kind="idle") for _ in range(n_gpus)]
        self.pending = [None] * n_gpus              # a load signalled to GPU g, waiting for its execute signal
        self.arrivals = collections.deque()         # arrival times of queued requests, in the controller's FIFO order
        # 1-link or k-link: a swap-in from the host store of at least this many bytes borrows the PCIe links
        # of the GPUs the scheduler reports free (tsw_sched_helpers); 0 = always one link, as the reference
        self.shard_min_bytes = shard_min_bytes
        self.swaps: List[dict] = []
        self.evictions = 0
        self.local_hits = 0
        self.completed = 0

    def close(self):
        for e in self.engines:
            e.close()
        self.ctrl.close()
        repo_reset()

    # ---- ExecuteAfterLoad (controller.hpp:141-162, 223-227): round-robin placement, load once
    def cold_start(self, func: str, arch: str, seed: int, tensor_data=None):
        ws = W.weight_set(arch, seed=seed)
        self.arch[func], self.nbytes[func] = arch, ws.nbytes
        events = self.ctrl.request(REQ_EXECUTE_AFTER_LOAD, func, str(LEVEL.get(arch, 1)))
        g = next(e[1] for e in events if e[0] == "S" and e[2] == SIGNAL_STARTUP)   # every GPU is idle at this point
        W.cold_start(self.engines[g], func, ws, tensor_data=tensor_data)
        self._carry_out(self.ctrl.complete(g), time.perf_counter())      # registers the replica; may unload others

    def _carry_out(self, events, t_arrival):
        """Executor side of the signals of one controller event."""
        for e in events:
            if e[0] != "S":
                continue
            _, g, sig, func = e
            if sig == SIGNAL_UNLOAD:
                self.engines[g].evict(func)
                self.evictions += 1
            elif sig >= SIGNAL_LOAD:
                src = sig - SIGNAL_LOAD - 1
                if self.engines[g].check_alloc(func):                    # resident: nothing to move (cuda_server.hpp:246)
                    self.pending[g] = None
                else:
                    helpers = []
                    if src < 0 and self.shard_min_bytes and self.nbytes[func] >= self.shard_min_bytes:
                        helpers = [h for h in self.ctrl.helpers(g) if self.state[h]["kind"] == "idle"]
                    self.pending[g] = dict(src=src, t_signal=time.perf_counter(), links=1 + len(helpers))
                    if helpers:                                          # asynchronous either way: kernels enqueued
                        self.engines[g].swap_in_sharded(func, [self.engines[h] for h in helpers])
                    else:
                        self.engines[g].swap_in(func, src)
            elif sig == SIGNAL_EXECUTE:
                st = dict(func=func, t_arrival=t_arrival)
                if self.pending[g] is None:
                    self.local_hits += 1
                    st.update(kind="exec", until=time.perf_counter() + EXEC_MS.get(self.arch[func], 10.0) / 1e3)
                else:
                    st.update(kind="swap", **self.pending[g])
                    self.pending[g] = None
                self.state[g] = st

    # ---- Execute (controller.hpp:163-185)
    def submit(self, func: str, now: float) -> bool:
        events = self.ctrl.request(REQ_EXECUTE, func)
        if not events:                                   # every GPU busy, or pinned replicas in the way: the controller queued it
            self.arrivals.append(now)
            return False
        self._carry_out(events, now)
        return True

    def poll(self):
        """Advance every GPU: finished swaps start executing, finished executions complete."""
        now = time.perf_counter()
        for g in range(self.n):
            st = self.state[g]
            if st["kind"] == "swap" and self.engines[g].poll_ready(st["func"]) == 0:
                self.swaps.append(dict(func=st["func"], gpu=g, src=st["src"], bytes=self.nbytes[st["func"]],
                                       ms=(now - st["t_signal"]) * 1e3, t=st["t_signal"], links=st["links"]))
                st["kind"] = "exec"
                st["until"] = now + EXEC_MS.get(self.arch[st["func"]], 10.0) / 1e3
            if st["kind"] == "exec" and now >= st["until"]:
                self.state[g] = dict(kind="idle")
                self.completed += 1
                events = self.ctrl.complete(g)                           # replica registered, pin released, queue served
                started = any(e[0] == "S" and e[2] == SIGNAL_EXECUTE for e in events)
                self._carry_out(events, self.arrivals.popleft() if started and self.arrivals else now)

    def busy(self) -> bool:
        return any(st["kind"] != "idle" for st in self.state) or self.ctrl.queue_depth() > 0


def run_stream(n_gpus: int, n_models: int, rate: float, duration_s: float, cap_bytes: int, seed: int = 4,
               speedup: float = 1.0, archs=("resnet50", "bert_base", "bert_large", "vgg19"),
               evict_policy: str = "LRU", zero_weights: bool = True, devices: Optional[List[int]] = None,
               shard_min_bytes: int = 0, pcie_pairs=None, nvlink=None) -> dict:
    """The mixed serverless stream: ``n_models`` functions, Zipf popularity, Poisson arrivals."""
    arch_of, times, picks = W.mixed_stream(seed=seed, n_models=n_models, rate=rate, duration_s=duration_s, archs=archs)
    store = sum(W.host_store_bytes(W.weight_set(a)) for a in arch_of)
    srv = SwapServer(n_gpus, cap_bytes, evict_policy=evict_policy, host_arena_bytes=0, devices=devices,
                     shard_min_bytes=shard_min_bytes, pcie_pairs=pcie_pairs, nvlink=nvlink)
    t0 = time.time()
    for i, a in enumerate(arch_of):
        ws = W.weight_set(a)
        data = (lambda k, ws=ws: np.zeros(ws.tensors[k].nbytes, dtype=np.uint8)) if zero_weights else None
        srv.cold_start(f"fn{i}", a, 1000 + i, tensor_data=data)
    cold_s = time.time() - t0
    ev_cold = srv.evictions
    start = time.perf_counter()
    k = 0
    n_req = len(times)
    while k < n_req or srv.busy():
        now = time.perf_counter() - start
        while k < n_req and times[k] / speedup <= now:
            srv.submit(f"fn{int(picks[k])}", now)
            k += 1
        srv.poll()
    wall = time.perf_counter() - start
    ms = np.array([s["ms"] for s in srv.swaps]) if srv.swaps else np.zeros(1)
    by = np.array([s["bytes"] for s in srv.swaps], dtype=np.float64) if srv.swaps else np.zeros(1)
    rel = np.array([s["t"] - start for s in srv.swaps]) if srv.swaps else np.zeros(1)
    fill = rel < wall * 0.25
    host = [s for s in srv.swaps if s["src"] < 0]
    multi = [s for s in host if s["links"] > 1]
    host_ms = np.array([s["ms"] for s in host]) if host else np.zeros(1)
    host_by = np.array([s["bytes"] for s in host], dtype=np.float64) if host else np.zeros(1)
    out = {
        "gpus": n_gpus, "models": n_models, "requests": n_req, "completed": srv.completed, "rate_req_s": rate * speedup,
        "duration_s": wall, "cap_bytes": cap_bytes, "host_store_bytes": store, "cold_start_s": cold_s,
        "evictions_at_cold_start": ev_cold, "evictions_in_service": srv.evictions - ev_cold,
        "local_hits": srv.local_hits, "swaps": len(srv.swaps), "swaps_from_host": len(host),
        "swaps_from_replica": len(srv.swaps) - len(host),
        "host_swaps_over_several_links": len(multi),
        "links_per_host_swap_mean": float(np.mean([s["links"] for s in host])) if host else 0.0,
        "host_swap_ms_p50": float(np.percentile(host_ms, 50)), "host_swap_ms_p99": float(np.percentile(host_ms, 99)),
        "host_swap_gbs_p50": float(np.percentile(host_by / (host_ms / 1e3) / 1e9, 50)) if host else 0.0,
        "swapped_bytes": float(by.sum()) if srv.swaps else 0.0,
        "sustained_swap_gbs": float(by.sum()) / wall / 1e9 if srv.swaps else 0.0,
        "fill_phase_swap_gbs": float(by[fill].sum()) / max(wall * 0.25, 1e-9) / 1e9 if srv.swaps else 0.0,
        "steady_swap_gbs": float(by[~fill].sum()) / max(wall * 0.75, 1e-9) / 1e9 if srv.swaps else 0.0,
        "swap_ms_p50": float(np.percentile(ms, 50)), "swap_ms_p99": float(np.percentile(ms, 99)),
        "swap_ms_max": float(ms.max()),
        "per_swap_gbs_p50": float(np.percentile(by / (ms / 1e3) / 1e9, 50)) if srv.swaps else 0.0,
        "exec_model": "GPU occupancy per request modelled as a constant per architecture (EXEC_MS); inference not run",
    }
    srv.close()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--models", type=int, default=64)
    ap.add_argument("--rate", type=float, default=200.0)
    ap.add_argument("--duration", type=float, default=120.0)
    ap.add_argument("--cap-gb", type=float, default=40.0)
    ap.add_argument("--speedup", type=float, default=1.0)
    ap.add_argument("--policy", default="LRU")
    ap.add_argument("--archs", default="resnet50,bert_base,bert_large,vgg19")
    ap.add_argument("--shard-min-mb", type=float, default=0.0,
                    help="swap-ins from the host store of at least this size borrow idle GPUs' PCIe links (0 = one link)")
    ap.add_argument("--seed", type=int, default=4)
    args = ap.parse_args()
    pairs = nvl = None
    if args.gpus > 1:
        from .memory_manager import discover_topology
        pairs, nvl = discover_topology(args.gpus)        # which GPUs share an uplink, which pairs are NVLink peers
    print(json.dumps(run_stream(args.gpus, args.models, args.rate, args.duration, int(args.cap_gb * (1 << 30)),
                                seed=args.seed, speedup=args.speedup, evict_policy=args.policy,
                                archs=tuple(args.archs.split(",")), shard_min_bytes=int(args.shard_min_mb * (1 << 20)),
                                pcie_pairs=pairs, nvlink=nvl)), flush=True)


if __name__ == "__main__":
    main()
