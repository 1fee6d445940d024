#!/usr/bin/env python
"""Benchmark of the model swap path: swap-in throughput (GB/s) and ms per model.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one swap-in of the workload's weight set from the page-locked host model store
into the target GPU's pool (block placement, pointer-table rebind, data movement over
PCIe, readiness publish) followed by the eviction that makes room for the next step.
Every byte crosses PCIe inside the timed region at every N; at N > 1 each rank's GPU
pulls tiles over its own link and stores them into the target's pool over NVLink.

  value  bytes of the set x K / time of K steps (tsw_swap_in + tsw_wait_ready + tsw_evict);
  e2e    the same through the executor-facing calls: the swap signal, then the translation
         of every parameter in access order as the launch path does it (each waits for its
         row of the pointer table, which the kernel writes into host-mapped memory), evict;
  roofline      the host -> pool launch against the PCIe links of the participating GPUs;
  kernel_hbm    the same kernel with both ends in HBM (a replica on the same GPU), against
                the measured HBM copy peak -- a figure about the kernel, not about the metric;
  gather_stage  (N > 1) each rank's share resident in its HBM, stored into the target over NVLink.

`--impl reference` times the reference's own swap path (its headers compiled where they
lie, oracle/_ref) on the same weight set with its default IO_THREAD_NUM = 4, from the swap
signal to the last parameter's readiness plus the eviction; if that checker is absent the
CPU restatement is timed instead.  Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from concurrent.futures import ThreadPoolExecutor

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

PCIE_GEN5_X16_GBS = 63.0       # 32 GT/s x 16 lanes x 128/130 / 8, one direction, per GPU
NVLINK5_GBS = 900.0            # per direction per GPU (nominal)
HBM_FALLBACK_GBS = 6650.0
# DRAM bytes moved per algorithmic byte by place_kernel with both ends in HBM: dram__bytes_read +
# dram__bytes_write of one launch in an ncu capture of the llama_mid case, over that launch's
# 2 x parameter bytes.  The kernel streams, so the ratio carries to the full-size launch.
DRAM_TRAFFIC_PER_ALGO_BYTE = 0.989
# The same for the host -> pool launch: DRAM bytes written per parameter byte (the reads come over
# PCIe and touch no DRAM of the GPU), from the ncu capture of the llama_mid case.
DRAM_WRITE_PER_ALGO_BYTE_HOST = 0.973


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f), "measured"
    except Exception:
        return {"hbm_gbs": HBM_FALLBACK_GBS}, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms while a region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.idx = device_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.idx)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._pump, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def generate_tensors(ws, threads, with_sums=False):
    """Seeded tensors of `ws`, generated ahead on a thread pool.  Returns the pool and data(i);
    with_sums also returns a dict that fills with every tensor's checksum as it is produced."""
    from torpor_b200 import workloads as W
    from torpor_b200.memory_manager import checksum_host
    pool = ThreadPoolExecutor(max(1, threads))
    sums = {}

    def make(i):
        b = W.tensor_bytes(ws, i)
        if with_sums:
            sums[i] = checksum_host(b)
        return b
    futs = {i: pool.submit(make, i) for i in range(len(ws.tensors))}
    data = lambda i: futs.pop(i).result()
    return (pool, data, sums) if with_sums else (pool, data)


# ------------------------------------------------------------------ reference arm

def _json_line_of(cmd, timeout=1500):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=timeout)
    for ln in r.stdout.splitlines():
        if ln.startswith("{"):
            return json.loads(ln)
    return {"failed": (r.stderr or r.stdout)[-300:]}


def _have_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def run_reference(args):
    """The reference's host-driven swap path (I/O threads packing into pinned memory,
    per-parameter cudaMemcpyAsync, event sync per 2 MiB group; memory_manager.hpp:213-449)
    on the workload itself, with its default IO_THREAD_NUM unless told otherwise.  A step is
    timed where the reference logs it: from the swap signal to the readiness of the last
    parameter in access order (:352,413), plus the eviction (:240-259).  Between the two the
    harness waits, untimed, for the transfer thread to hand its pinned mirrors back (:414-423)."""
    from oracle import tso
    from torpor_b200 import workloads as W
    ncpu = os.cpu_count() or 1
    io_threads = args.ref_io_threads or 4          # default_num_io_thread (memory_manager.hpp:22-23)
    if tso.available("ref_cuda") and _have_gpu():
        kind, lib = "reference", tso.load("ref_cuda")
        what = "reference headers (memory_manager.hpp:213-449) + CUDA runtime"
    else:
        kind, lib, io_threads = "port", tso.load("oracle"), 1
        what = "CPU restatement (oracle/torpor_oracle.cpp), host memcpy into the block layout"
    sample_name = args.ref_sample or args.workload
    ws = W.weight_set(sample_name)
    lib.reset_world()
    src = args.ref_src_gpu
    budget = W.pool_budget_for(ws)
    pool, data = generate_tensors(ws, min(ncpu, 16))
    if src >= 0:
        # the reference's replica swap (memory_manager.hpp:394-396): the model is resident on GPU `src`,
        # GPU 0 copies it parameter by parameter with cudaMemcpyPeerAsync
        if kind != "reference":
            return {"impl": "reference", "unavailable": "the replica-swap baseline needs the reference library and two GPUs"}
        pairs = lib.enable_peer_access(src + 1)          # as the controller does at start-up (controller.hpp:63-75)
        what += f"; peer access enabled for {pairs} directed pairs"
        holder = lib.manager(server_id=src, budget=budget, gpu_count=src + 1, io_threads=io_threads)
        m = lib.manager(server_id=0, budget=budget, gpu_count=src + 1, io_threads=io_threads)
        W.cold_start(holder, "ref", ws, tensor_data=data)
        lib.set_model_status("ref", src, True)
        what += f"; replica swap from GPU {src} (cudaMemcpyPeerAsync per parameter)"
    else:
        m = lib.manager(budget=budget, io_threads=io_threads)
        W.cold_start(m, "ref", ws, tensor_data=data)
        m.evict("ref")
    pool.shutdown()
    for _ in range(args.warmup):
        m.swap_in_timed("ref", src); m.evict("ref")
    t_sig, t_evict = [], []
    t0 = time.perf_counter()
    for _ in range(args.steps):
        t_sig.append(m.swap_in_timed("ref", src))      # microseconds, signal -> last parameter ready
        te = time.perf_counter()
        m.evict("ref")
        t_evict.append((time.perf_counter() - te) * 1e6)
    wall = time.perf_counter() - t0
    step_s = (sum(t_sig) + sum(t_evict)) / 1e6           # what the reference itself spends per step
    gbs = ws.nbytes * args.steps / step_s / 1e9
    cores = io_threads + 1 if kind == "reference" else 1
    sample = (f"{sample_name}: {len(ws.tensors)} tensors, {ws.nbytes} B; {args.warmup} warm-up + {args.steps} swap-ins "
              f"with forced evict between; {what}; IO_THREAD_NUM={io_threads}"
              + (" (the reference's default)" if io_threads == 4 else ""))
    cfg = workload_config(args, args.gpus, sample_name)
    cfg["reference_settings"] = {"IO_THREAD_NUM": io_threads, "BUFFER_SIZE": 2 << 20, "pool_budget_bytes": budget}
    line = {
        # the reference's swap uses one GPU's link whatever N is; n_gpus names the configuration compared
        "impl": "reference", "metric": "model_swap_in_throughput", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": cfg,
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": kind, "sample": sample,
                         "host_cores": ncpu, "signal_to_ready_ms_median": statistics.median(t_sig) / 1e3,
                         "signal_to_ready_ms_mean": statistics.mean(t_sig) / 1e3,
                         "signal_to_ready_gbs": ws.nbytes / (statistics.median(t_sig) / 1e6) / 1e9,
                         "swap_out_metadata_only_us_median": statistics.median(t_evict),
                         "untimed_harness_wait_ms_per_step": (wall - step_s) / args.steps * 1e3},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    return line


def run_reference_pack(args):
    """BASELINE config 1's CPU baseline: the reference's host-side pack of a weight set into the
    pool-block layout -- pageable host store -> pinned block mirrors by its I/O threads alone
    (pinned_io_thread, memory_manager.hpp:311-329) -- nothing crossing to the GPU."""
    from oracle import tso
    from torpor_b200 import workloads as W
    ncpu = os.cpu_count() or 1
    kind = "ref_cuda" if (tso.available("ref_cuda") and _have_gpu()) else ("ref_fake" if tso.available("ref_fake") else None)
    if kind is None:
        return {"impl": "reference", "unavailable": "the reference's headers are not built here (oracle/_ref)"}
    lib = tso.load(kind)
    lib.reset_world()
    name = args.ref_sample or "resnet50"
    ws = W.weight_set(name)
    io_threads = args.ref_io_threads or 4
    m = lib.manager(budget=W.pool_budget_for(ws), io_threads=io_threads)
    W.cold_start(m, "ref", ws)
    m.evict("ref")
    for _ in range(max(1, args.warmup)):
        m.pack_timed("ref")
    us = [m.pack_timed("ref") for _ in range(max(3, args.steps))]
    med = statistics.median(us)
    return {"impl": "reference", "pack": {"value": ws.nbytes / (med / 1e6) / 1e9, "unit": "GB/s", "ms_median": med / 1e3,
                                          "cores": io_threads, "host_cores": ncpu, "kind": "reference",
                                          "sample": f"{name}: {len(ws.tensors)} tensors, {ws.nbytes} B; pageable -> pinned "
                                                    f"memcpy by IO_THREAD_NUM={io_threads} threads, {len(us)} timed packs",
                                          "pinned": "cudaMallocHost" if kind == "ref_cuda" else "host malloc (no GPU here)"}}


def cpu_baselines(args, steps=5, warmup=1):
    """The reported baselines of the bench line, each reference run in its own process (the
    reference's threads and pool cannot be torn down): the full swap-in at the reference's stock
    IO_THREAD_NUM = 4 (the primary one) and with one staging thread per host core, and the
    host-side pack of config 1's ResNet-50 set at both thread counts."""
    ncpu = os.cpu_count() or 1
    me = [sys.executable, os.path.abspath(__file__), "--impl", "reference", "--workload", args.workload]
    if args.ref_sample:
        me += ["--ref-sample", args.ref_sample]
    full = me + ["--steps", str(steps), "--warmup", str(warmup)]
    try:
        primary = _json_line_of(full + ["--ref-io-threads", "4"])
        base = primary.get("cpu_baseline") or {"value": None, "unit": "GB/s", "cores": 0, "kind": "port",
                                               "sample": f"failed: {primary}"}
        if not args.quick_baseline:
            allc = _json_line_of(full + ["--ref-io-threads", str(ncpu)]).get("cpu_baseline")
            if allc:
                base["all_cores_variant"] = {k: allc[k] for k in ("value", "unit", "cores", "signal_to_ready_ms_median", "sample") if k in allc}
        pack = ["--ref-pack", "--ref-sample", "resnet50", "--steps", "10", "--warmup", "2", "--impl", "reference"]
        me0 = [sys.executable, os.path.abspath(__file__)]
        base["config1_host_side_pack"] = {
            "io4": _json_line_of(me0 + pack + ["--ref-io-threads", "4"]).get("pack"),
            f"io{ncpu}": _json_line_of(me0 + pack + ["--ref-io-threads", str(ncpu)]).get("pack"),
            "what": "pinned_io_thread (memory_manager.hpp:311-329) alone on the ResNet-50 set: pageable -> pinned pool-block mirrors"}
        return base
    except Exception as ex:  # reported, never fatal for the GPU arm
        return {"value": None, "unit": "GB/s", "cores": 0, "kind": "port", "sample": f"failed: {ex}"}


# ------------------------------------------------------------------ measured peaks of the box

def feed_matrix(seconds=1.5, chunk=256 << 20):
    """How fast this box feeds its GPUs from page-locked host memory with the copy engines:
    every GPU alone, then groups of GPUs streaming continuously for a fixed time at once
    (the sum of their rates, not equal shares), and every other GPU's copy engine pushing
    into GPU 0 at once.  These are the measured ceilings the swap is compared with."""
    import torch
    n = torch.cuda.device_count()
    host = [torch.empty(chunk, dtype=torch.uint8).pin_memory() for _ in range(n)]
    dev = [torch.empty(chunk, dtype=torch.uint8, device=f"cuda:{g}") for g in range(n)]
    streams = [torch.cuda.Stream(device=g) for g in range(n)]

    def stream_for(gpus, secs, src_of=None):
        """GPUs in `gpus` copy host -> device back to back for `secs`; GB/s per GPU."""
        done = {g: 0 for g in gpus}
        start = threading.Barrier(len(gpus))

        def work(g):
            src = host[g] if src_of is None else host[src_of(g)]
            with torch.cuda.device(g), torch.cuda.stream(streams[g]):
                dev[g].copy_(src, non_blocking=True)
                streams[g].synchronize()
                start.wait()
                t_end = time.perf_counter() + secs
                while time.perf_counter() < t_end:
                    for _ in range(2):
                        dev[g].copy_(src, non_blocking=True)
                    streams[g].synchronize()
                    done[g] += 2 * chunk
        ts = [threading.Thread(target=work, args=(g,)) for g in gpus]
        t0 = time.perf_counter()
        [t.start() for t in ts]
        [t.join() for t in ts]
        return {g: done[g] / secs / 1e9 for g in gpus}

    out = {"gpus": n, "seconds_per_cell": seconds, "chunk_bytes": chunk}
    alone = {}
    for g in range(n):
        alone.update(stream_for([g], seconds / 3))
    out["h2d_alone_gbs"] = [round(alone[g], 2) for g in range(n)]
    out["h2d_alone_sum_gbs"] = round(sum(alone.values()), 1)
    groups = {"all": list(range(n))}
    if n >= 4:
        groups["first_half"] = list(range(n // 2))
        groups["second_half"] = list(range(n // 2, n))
        groups["even"] = list(range(0, n, 2))
    for name, gpus in groups.items():
        r = stream_for(gpus, seconds)
        out[f"h2d_concurrent_{name}"] = {"gpus": gpus, "per_gpu_gbs": [round(r[g], 2) for g in gpus],
                                         "sum_gbs": round(sum(r.values()), 1)}
    # does the rate depend on WHICH page-locked buffer is read?  (a guest that hides its NUMA layout
    # would show it here): GPU g reading each of the n buffers in turn, alone
    if n >= 2:
        by_buf = []
        for g in range(n):
            row = []
            for b in range(n):
                row.append(round(stream_for([g], 0.12, src_of=lambda _g, b=b: b)[g], 1))
            by_buf.append(row)
        out["h2d_alone_by_buffer_gbs"] = by_buf
        # (n-1) -> 1: every other GPU's copy engine pushes into GPU 0 at once
        nb = 1 << 30
        dst = [torch.empty(nb, dtype=torch.uint8, device="cuda:0") for _ in range(n - 1)]
        src = [torch.empty(nb, dtype=torch.uint8, device=f"cuda:{i}") for i in range(1, n)]
        best = 0.0
        for _ in range(4):
            for i in range(n):
                torch.cuda.synchronize(i)
            t0 = time.perf_counter()
            for d, s_, i in zip(dst, src, range(1, n)):
                with torch.cuda.stream(streams[i]):
                    d.copy_(s_, non_blocking=True)
            for i in range(n):
                torch.cuda.synchronize(i)
            best = max(best, nb * (n - 1) / (time.perf_counter() - t0) / 1e9)
        out["peer_gather_to_gpu0_gbs"] = {"value": round(best, 1), "what": f"{n - 1} -> 1 concurrent cudaMemcpyPeerAsync of 1 GiB each, wall clock, best of 4"}
        del dst, src
    return out


def link_probe(seconds=0.4, chunk=64 << 20):
    """Per-GPU rate of page-locked host -> device copies while EVERY GPU of the box copies at once
    (the rate a GPU's link really gets when its neighbours are busy too), for choosing which GPUs
    take part in a swap when fewer are asked for than the box has."""
    import torch
    n = torch.cuda.device_count()
    host = [torch.empty(chunk, dtype=torch.uint8).pin_memory() for _ in range(n)]
    dev = [torch.empty(chunk, dtype=torch.uint8, device=f"cuda:{g}") for g in range(n)]
    streams = [torch.cuda.Stream(device=g) for g in range(n)]
    done = [0] * n
    start = threading.Barrier(n)

    def work(g):
        with torch.cuda.device(g), torch.cuda.stream(streams[g]):
            dev[g].copy_(host[g], non_blocking=True)
            streams[g].synchronize()
            start.wait()
            t_end = time.perf_counter() + seconds
            while time.perf_counter() < t_end:
                for _ in range(4):
                    dev[g].copy_(host[g], non_blocking=True)
                streams[g].synchronize()
                done[g] += 4 * chunk
    ts = [threading.Thread(target=work, args=(g,)) for g in range(n)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    return {"link_probe": {"gpus": n, "concurrent_h2d_gbs": [round(d / seconds / 1e9, 2) for d in done]}}


def run_baselines(args):
    """Reported baselines around the path, each reference run in its own process: swap-in with the
    reference's default IO_THREAD_NUM=4 and with one staging thread per host core, its host-side
    pack alone, its replica swap over cudaMemcpyPeerAsync when a second GPU is there, and the
    copy-engine feed matrix of this box."""
    import torch
    ncpu = os.cpu_count() or 1
    me = os.path.abspath(__file__)
    sample = args.ref_sample or args.workload

    def ref(*extra):
        d = _json_line_of([sys.executable, me, "--impl", "reference", "--steps", str(args.steps), "--warmup",
                           str(args.warmup), "--ref-sample", sample, "--workload", args.workload, *extra])
        return d.get("cpu_baseline", d.get("pack", d))

    out = {"host_cores": ncpu, "gpus": torch.cuda.device_count(), "sample": sample}
    if not args.feed_only and not args.replica_only:
        out["reference_swap_in_io4"] = ref("--ref-io-threads", "4")
        out["reference_swap_in_io_all"] = ref("--ref-io-threads", str(ncpu))
        out["reference_pack_resnet50_io4"] = ref("--ref-pack", "--ref-sample", "resnet50", "--ref-io-threads", "4")
        out["reference_pack_resnet50_io_all"] = ref("--ref-pack", "--ref-sample", "resnet50", "--ref-io-threads", str(ncpu))
    if not args.replica_only:
        out["feed_matrix"] = feed_matrix()
    if torch.cuda.device_count() >= 2 and not args.feed_only:
        out["reference_replica_swap"] = ref("--ref-src-gpu", "1")
        # the same replica swap through this library: GPU 0 places the model from GPU 1's pool over NVLink
        from torpor_b200 import workloads as W
        from torpor_b200.memory_manager import MemoryManager, ModelRepo, repo_reset
        ws = W.weight_set(sample)

        def ours(tile_dev):
            repo_reset()
            holder = MemoryManager(W.pool_budget_for(ws), device=1, server_id=1, gpu_count=2, host_arena_bytes=W.host_store_bytes(ws))
            target = MemoryManager(W.pool_budget_for(ws), device=0, server_id=0, gpu_count=2, tile_bytes_device=tile_dev)
            pool, data = generate_tensors(ws, min(ncpu, 16))
            W.cold_start(holder, "m", ws, tensor_data=data)
            pool.shutdown()
            ModelRepo.add_model_info("m", 1)
            wall, dev = [], []
            for it in range(args.warmup + args.steps):
                t0 = time.perf_counter()
                target.swap_in("m", 1); target.wait_ready("m")
                if it >= args.warmup:
                    wall.append(time.perf_counter() - t0)
                    dev.append(target.stats()["last_swap_device_ns"] / 1e9)
                target.evict("m")
            r = {"signal_to_ready_gbs": ws.nbytes / statistics.median(wall) / 1e9,
                 "signal_to_ready_ms_median": statistics.median(wall) * 1e3,
                 "kernel_gbs": ws.nbytes / statistics.median(dev) / 1e9, "kernel_ms_median": statistics.median(dev) * 1e3,
                 "tile_bytes_device": tile_dev or 512 * 1024,
                 "what": "tsw_swap_in(func, src_gpu=1) + tsw_wait_ready on GPU 0: place_kernel reads GPU 1's pool over NVLink"}
            target.close(); holder.close(); repo_reset()
            return r
        out["ours_replica_swap"] = ours(0)
    return {"baselines": out}


def run_corun(args):
    """What a swap-in from the host store leaves of the GPU to other kernels.  The reference moves
    weights with the copy engine, so the function's first kernels run while its later weights are
    still arriving (cuda_server.hpp:1265-1268 with memory_manager.hpp:527-540); a kernel that reads
    the host store itself occupies SMs instead, and its persistent CTAs hold their registers until
    the swap is over.  Per grid size of the host-side launch: the swap-in alone, a fixed loop of
    bf16 matrix products on another stream alone, and both at once (the swap launched first)."""
    import torch
    from torpor_b200 import workloads as W
    from torpor_b200.memory_manager import MemoryManager, ModelRepo, repo_reset
    torch.cuda.set_device(0)
    ncpu = os.cpu_count() or 1
    ws = W.weight_set(args.workload)
    budget = W.pool_budget_for(ws)
    grids = [int(g) for g in args.corun_grids.split(",")]
    repo_reset()
    holder = MemoryManager(budget, device=0, server_id=len(grids), gpu_count=len(grids) + 1, host_arena_bytes=W.host_store_bytes(ws))
    pool, data = generate_tensors(ws, min(ncpu, 16))
    vaddrs = W.cold_start(holder, "model", ws, tensor_data=data).tensor_vaddr
    pool.shutdown()
    ModelRepo.add_model_info("model", len(grids))
    marks = sorted({0, len(vaddrs) // 4, len(vaddrs) // 2, len(vaddrs) - 1})     # positions in the access order

    side = torch.cuda.Stream()
    a = torch.randn(4096, 4096, dtype=torch.bfloat16, device="cuda")
    b = torch.randn(4096, 4096, dtype=torch.bfloat16, device="cuda")
    c = torch.empty_like(a)

    def products(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(side):
            e0.record()
            for _ in range(reps):
                torch.matmul(a, b, out=c)
            e1.record()
        return e0, e1

    e0, e1 = products(20); torch.cuda.synchronize()            # module load, clocks
    e0, e1 = products(200); torch.cuda.synchronize()
    per = e0.elapsed_time(e1) / 200
    rows = []
    for k, g in enumerate(grids):
        eng = MemoryManager(budget, device=0, server_id=k, gpu_count=len(grids) + 1, grid_ctas_host=g, mover=args.mover)
        for _ in range(max(1, args.warmup)):
            eng.swap_in("model", -1); eng.wait_ready("model"); eng.evict("model")
        alone = []
        for _ in range(max(1, args.steps)):
            eng.swap_in("model", -1); eng.wait_ready("model")
            alone.append(eng.stats()["last_swap_device_ns"] / 1e6)
            eng.evict("model")
        swap_ms = statistics.median(alone)
        # when the launch path gets its parameters: swap signal -> tsw_translate returns, for the first
        # parameter of the access order, the one a quarter and half way in, and the last
        arrive = []
        for _ in range(max(1, args.steps)):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            eng.swap_in("model", -1)
            ts = []
            for i in marks:
                eng.translate("model", vaddrs[i])
                ts.append((time.perf_counter() - t0) * 1e3)
            eng.wait_ready("model"); eng.evict("model")
            arrive.append(ts)
        arrive_ms = [statistics.median(col) for col in zip(*arrive)]
        reps = max(10, int(swap_ms / per))                     # a loop about as long as the swap
        e0, e1 = products(reps); torch.cuda.synchronize()
        loop_alone = e0.elapsed_time(e1)
        both_swap, both_loop = [], []
        for _ in range(max(1, args.steps)):
            torch.cuda.synchronize()
            eng.swap_in("model", -1)                           # returns once the kernel is launched
            e0, e1 = products(reps)
            eng.wait_ready("model")
            torch.cuda.synchronize()
            both_swap.append(eng.stats()["last_swap_device_ns"] / 1e6)
            both_loop.append(e0.elapsed_time(e1))
            eng.evict("model")
        rows.append({"grid_ctas_host": g or "default", "swap_alone_ms": swap_ms, "swap_alone_gbs": ws.nbytes / swap_ms / 1e6,
                     "ready_ms_at_parameter": dict(zip(map(str, marks), arrive_ms)),
                     "products": reps, "loop_alone_ms": loop_alone,
                     "swap_with_loop_ms": statistics.median(both_swap), "swap_with_loop_gbs": ws.nbytes / statistics.median(both_swap) / 1e6,
                     "loop_with_swap_ms": statistics.median(both_loop),
                     "loop_slowdown": statistics.median(both_loop) / loop_alone})
        eng.close()
    holder.close(); repo_reset()
    return {"corun": {"workload": f"{args.workload}: {ws.nbytes} B", "mover": args.mover, "product": "4096^3 bf16 torch.matmul",
                      "product_ms": per, "rows": rows}}


def workload_config(args, n, name=None):
    from torpor_b200 import workloads as W
    name = name or args.workload
    ws = W.weight_set(name)
    return {"workload": f"{name}: {len(ws.tensors)} tensors, {ws.nbytes} B, N(0,0.02) seeded, "
                        f"client-allocator block layout ({len(W.pack_blocks(ws)[0])} model blocks)",
            "target_gpus": 1, "participating_gpus": n, "l2": "inputs larger than L2 (no flush needed)",
            "source": "the host model store (every byte crosses PCIe in the timed region)",
            "step": "swap-in (place, rebind, move, publish) + evict"}


# ------------------------------------------------------------------ checking what was swapped in

class Verifier:
    """Holds what a swap-in must produce -- the checksum of every tensor of the set and, per
    swap-in since the engines were made, the block and pointer tables in canonical addresses
    (worked out beforehand on plan-only engines) -- and compares the target engine with it."""

    def __init__(self, ws, sums, tables):
        self.ws, self.sums, self.tables = ws, sums, tables
        self.swaps = 0          # swap-ins the target has done so far
        self.checks = 0

    def swapped(self):
        self.swaps += 1

    def check(self, eng, func, where):
        got = eng.checksum_resident(func)
        for i in range(len(self.ws.tensors)):
            if not np.array_equal(got[i], self.sums[i]):
                raise RuntimeError(f"{where}: resident bytes of tensor {i} differ from the host store")
        blocks, params = self.tables[self.swaps - 1]
        if not np.array_equal(eng.dump_blocks(func, canonical=True), blocks):
            raise RuntimeError(f"{where}: block table differs from the plan-only engine's after swap-in {self.swaps}")
        if not np.array_equal(eng.dump_params(func, canonical=True), params):
            raise RuntimeError(f"{where}: pointer table differs from the plan-only engine's after swap-in {self.swaps}")
        self.checks += 1

    def record(self, after_timed):
        return {"tensors": len(self.ws.tensors), "table": True, "after_timed": bool(after_timed), "checks": self.checks,
                "how": "64-bit position-weighted checksums of every tensor's resident bytes against the host copy; "
                       "block and pointer tables word for word (canonical addresses) against a plan-only engine "
                       "replaying the same swap sequence; a mismatch fails the run"}


def copy_engine_h2d_gbs(device=0, nbytes=1 << 30, reps=3):
    """cudaMemcpyAsync from page-locked memory on this GPU's link, best of `reps` (CUDA events)."""
    import torch
    x = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    y = torch.empty(nbytes, dtype=torch.uint8, device=f"cuda:{device}")
    best = 0.0
    with torch.cuda.device(device):
        for _ in range(reps + 1):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(); y.copy_(x, non_blocking=True); e.record(); torch.cuda.synchronize()
            best = max(best, nbytes / (s.elapsed_time(e) / 1e3) / 1e9)
    return best


# ------------------------------------------------------------------ our arm, one GPU

def run_single(args):
    import torch
    from torpor_b200 import workloads as W
    from torpor_b200.memory_manager import MemoryManager, ModelRepo, repo_reset

    peaks, peak_kind = measured_peaks()
    ncpu = os.cpu_count() or 1
    # CPU / reference baselines first, in their own processes
    cpu_baseline = None if args.no_cpu_baseline else cpu_baselines(args)

    torch.cuda.set_device(0)
    ws = W.weight_set(args.workload)
    budget = W.pool_budget_for(ws)
    arena = W.host_store_bytes(ws)
    K, Wm = args.steps, args.warmup
    K_hbm = min(K, 10)
    repo_reset()
    total_swaps = 2 + 2 * (Wm + K) + (Wm + K_hbm) + 3 + 4
    tables = W.plan_tables(ws, "model", budget=budget, target_server=0, holder_server=1, gpu_count=2, swaps=total_swaps)
    repo_reset()
    replica = MemoryManager(budget, device=0, server_id=1, gpu_count=2, host_arena_bytes=arena,
                            host_store_mode=args.host_store, tile_bytes_host=args.tile_kib * 1024)
    target = MemoryManager(budget, device=0, server_id=0, gpu_count=2, tile_bytes_host=args.tile_kib * 1024, mover=args.mover,
                           grid_ctas=args.grid_ctas, grid_ctas_host=args.grid_ctas_host)

    pool, data, sums = generate_tensors(ws, min(ncpu, 16), with_sums=True)
    t0 = time.time()
    loaded = W.cold_start(replica, "model", ws, tensor_data=data)
    pool.shutdown()
    torch.cuda.synchronize()
    cold_s = time.time() - t0
    ModelRepo.add_model_info("model", 1)
    ver = Verifier(ws, sums, tables)
    vaddrs = loaded.tensor_vaddr

    def swap(src):
        target.swap_in("model", src)
        ver.swapped()

    def timed(src, steps, warmup, through_translate=False, where=""):
        for _ in range(warmup):
            swap(src); target.wait_ready("model"); target.evict("model")
        dev_ns, ready_s = [], []
        pause = 0.0
        launches0 = target.stats()["kernel_launches"]
        torch.cuda.synchronize()
        t_begin = time.perf_counter()
        for k in range(steps):
            ts = time.perf_counter()
            swap(src)
            if through_translate:
                for v in vaddrs:                     # the launch path: every parameter, in access order
                    target.translate("model", v)
            else:
                target.wait_ready("model")
            ready_s.append(time.perf_counter() - ts)
            dev_ns.append(target.stats()["last_swap_device_ns"])
            if k == steps - 1:                       # the last timed swap-in is the one that is checked; clock paused
                tp = time.perf_counter()
                l1 = target.stats()["kernel_launches"]
                ver.check(target, "model", where)
                launches0 += target.stats()["kernel_launches"] - l1
                pause = time.perf_counter() - tp
            target.evict("model")
        torch.cuda.synchronize()
        wall = time.perf_counter() - t_begin - pause
        return wall, dev_ns, ready_s, target.stats()["kernel_launches"] - launches0

    # correctness of both sources before anything is timed
    swap(-1); target.wait_ready("model"); ver.check(target, "model", "before timing, from the host store"); target.evict("model")
    swap(1); target.wait_ready("model"); ver.check(target, "model", "before timing, from the replica"); target.evict("model")

    sampler = ClockSampler(0)
    sampler.start()
    wall_v, dev_v, ready_v, launches_v = timed(-1, K, Wm, where="after the timed swap-ins from the host store")
    wall_e, dev_e, ready_e, launches_e = timed(-1, K, Wm, through_translate=True, where="after the timed executor-path swap-ins")
    wall_h, dev_h, _, _ = timed(1, K_hbm, Wm, where="after the timed replica swap-ins")
    # swap-out with write-back (no counterpart in the reference, whose swap-out moves nothing):
    # resident bytes -> host store through the same kernel, PCIe D2H bound
    wb = []
    for _ in range(3):
        swap(-1); target.wait_ready("model")
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        target.evict("model", writeback=True)
        wb.append(time.perf_counter() - t0)
    swap(-1); target.wait_ready("model"); ver.check(target, "model", "after the write-back evictions"); target.evict("model")

    # The same executor path with the copy engine carrying the large parameters (tsw_config.mover = 2;
    # the kernel moves the small ones and publishes every row): a fresh engine under the same server id,
    # so the placement sequence -- and the tables it is checked against -- start over.
    assisted = None
    if args.mover == 0:
        target.close()
        target = MemoryManager(budget, device=0, server_id=0, gpu_count=2, tile_bytes_host=args.tile_kib * 1024, mover=2,
                               grid_ctas=args.grid_ctas, grid_ctas_host=args.grid_ctas_host)
        ver.swaps = 0
        swap(-1); target.wait_ready("model"); ver.check(target, "model", "before timing, copy-engine-assisted"); target.evict("model")
        wall_a, dev_a, ready_a, launches_a = timed(-1, K, Wm, through_translate=True,
                                                   where="after the timed copy-engine-assisted swap-ins")
        wb_a = []
        for _ in range(3):
            swap(-1); target.wait_ready("model")
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            target.evict("model", writeback=True)
            wb_a.append(time.perf_counter() - t0)
        swap(-1); target.wait_ready("model"); ver.check(target, "model", "after the copy-engine-assisted write-backs"); target.evict("model")
        assisted = {"value": ws.nbytes * K / wall_a / 1e9, "unit": "GB/s", "ms_per_model": wall_a / K * 1e3,
                    "swap_out_writeback_gbs": ws.nbytes / min(wb_a) / 1e9,
                    "device_ms_per_model": statistics.mean(dev_a) / 1e6, "gpu_launches": launches_a,
                    "frac_of_pcie": ws.nbytes / (statistics.mean(dev_a) / 1e9) / 1e9 / PCIE_GEN5_X16_GBS,
                    "what": "executor path with tsw_config.mover = 2: parameters of 4 MiB and more by cudaMemcpyAsync in "
                            "access order with a publish kernel behind each, the rest by place_kernel at the same time"}
    clocks = sampler.stop()

    ce = copy_engine_h2d_gbs(0)     # measured DMA rate of this box's link, next to the theoretical 63 GB/s

    B = ws.nbytes
    n_params = len(ws.tensors)
    value = B * K / wall_v / 1e9
    e2e = B * K / wall_e / 1e9
    e2e_ms, e2e_dev_ms, e2e_mover = wall_e / K * 1e3, statistics.mean(dev_e) / 1e6, args.mover
    e2e_by_mover = {str(args.mover): e2e}
    if assisted:
        e2e_by_mover["2"] = assisted["value"]
        if assisted["value"] > e2e:      # what a deployment on this box would configure: the faster of the two, as measured here
            e2e, e2e_ms, e2e_dev_ms, e2e_mover = assisted["value"], assisted["ms_per_model"], assisted["device_ms_per_model"], 2
    kern_v = statistics.mean(dev_v) / 1e9
    kern_h = statistics.mean(dev_h) / 1e9
    achieved = B / kern_v / 1e9
    hbm = 2 * B / kern_h / 1e9
    line = {
        "metric": "model_swap_in_throughput", "value": value, "unit": "GB/s", "n_gpus": 1,
        "steps": K, "warmup": Wm, "ms_per_step": wall_v / K * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": workload_config(args, 1),
        "value_arm": "tsw_swap_in from the page-locked host store + tsw_wait_ready + tsw_evict, K steps on the wall clock",
        "signal_to_ready_ms": {"median": statistics.median(ready_v) * 1e3, "mean": statistics.mean(ready_v) * 1e3,
                               "gbs_at_median": B / statistics.median(ready_v) / 1e9},
        "e2e": {"value": e2e, "unit": "GB/s", "ms_per_model": e2e_ms,
                "h2d_bytes_per_step": B + 44 * n_params, "d2h_bytes_per_step": 12 * n_params,
                "device_ms_per_model": e2e_dev_ms, "mover": e2e_mover, "gbs_by_mover": e2e_by_mover,
                "what": "executor path through the C ABI: swap signal (tsw_swap_in), then tsw_translate of every parameter in "
                        "access order (each waits for its pointer-table row, written on the device into host-mapped memory), "
                        "then tsw_evict; source = the page-locked host store; measured with the placement kernel alone "
                        "(mover 0) and with the copy engine carrying the large parameters (mover 2), the faster one reported"},
        "roofline": {"bound": "pcie", "achieved": achieved, "peak": PCIE_GEN5_X16_GBS, "unit": "GB/s",
                     "frac": achieved / PCIE_GEN5_X16_GBS, "peak_kind": "theoretical PCIe Gen5 x16, one direction (no PCIe figure in MEASURED_PEAKS.json)",
                     "kernel": "place_kernel (host store -> pool, zero-copy reads over PCIe)",
                     "algorithmic_bytes_per_launch": B, "launch_ms": kern_v * 1e3,
                     "traffic": DRAM_WRITE_PER_ALGO_BYTE_HOST * B,
                     "copy_engine_same_run_gbs": ce, "frac_of_copy_engine": achieved / ce if ce else None,
                     "frac_wall": value / PCIE_GEN5_X16_GBS},
        "kernel_hbm": {"bound": "hbm", "achieved": hbm, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": hbm / peaks["hbm_gbs"],
                       "peak_kind": f"{peak_kind} copy bandwidth (burst)", "kernel": "place_kernel (replica in HBM -> pool, same GPU)",
                       "algorithmic_bytes_per_launch": 2 * B, "launch_ms": kern_h * 1e3,
                       "traffic": DRAM_TRAFFIC_PER_ALGO_BYTE * 2 * B, "steps": K_hbm,
                       "swap_gbs_wall": B * K_hbm / wall_h / 1e9,
                       "what": "not the metric: the mover with both ends in HBM, no reference path does this on one GPU"},
        "swap_out_writeback": {"value": B / min(wb) / 1e9, "unit": "GB/s", "ms_per_model": min(wb) * 1e3,
                               "frac_of_pcie": B / min(wb) / 1e9 / PCIE_GEN5_X16_GBS,
                               "what": "tsw_evict(writeback=1): pool -> host store, D2H over PCIe; the reference's swap-out is metadata only"},
        "copy_engine_assisted": assisted,
        "verified": ver.record(after_timed=True),
        "cpu_baseline": cpu_baseline,
        "gpu_launches": launches_v, "gpu_launches_e2e": launches_e,
        "clocks": clocks, "host_cores": ncpu, "cold_start_s": cold_s,
        "settings": {"tile_bytes_host": args.tile_kib * 1024 or 65536, "host_store_mode": args.host_store, "mover": args.mover,
                     "grid_ctas_host": args.grid_ctas_host or args.grid_ctas or 32, "grid_ctas": args.grid_ctas or "6 per SM"},
    }
    target.close(); replica.close(); repo_reset()
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama2_7b")
    ap.add_argument("--ref-sample", default=None, help="reference arm: weight set to time (default: the workload itself)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--quick-baseline", action="store_true", help="cpu_baseline without the all-cores variant")
    ap.add_argument("--ref-io-threads", type=int, default=0, help="IO_THREAD_NUM of the reference arm (0 = its default, 4)")
    ap.add_argument("--ref-src-gpu", type=int, default=-1, help="reference arm: swap from a replica on this GPU instead of the host store")
    ap.add_argument("--ref-pack", action="store_true", help="reference arm: time its host-side pack alone (pageable -> pinned)")
    ap.add_argument("--baselines", action="store_true",
                    help="print the reported baselines around the path (reference with its default 4 and with all "
                         "staging threads, its pack, its replica swap, the copy-engine feed matrix) as one JSON line; not the contract line")
    ap.add_argument("--feed-only", action="store_true", help="--baselines: the copy-engine feed matrix only")
    ap.add_argument("--replica-only", action="store_true", help="--baselines: only the replica swap GPU 1 -> GPU 0 over NVLink, "
                                                                "the reference's and this library's, on --ref-sample")
    ap.add_argument("--corun", action="store_true", help="time a loop of matrix products on another stream while a swap-in from "
                                                          "the host store runs, per grid size of the host-side launch; not the contract line")
    ap.add_argument("--corun-grids", default="0,148,296,592,888", help="--corun: CTAs of the host-side launch to try (0 = the library's default)")
    ap.add_argument("--link-probe", action="store_true", help="print every GPU's host-link rate under full contention and exit")
    ap.add_argument("--devices", default="", help="N > 1: comma-separated CUDA ordinals to use, target first "
                                                   "(default: measured -- the best-fed GPUs when the box has more than N)")
    ap.add_argument("--tile-kib", type=int, default=0, help="host-side tile size of the mover in KiB (0 = the library's default, 64)")
    ap.add_argument("--grid-ctas", type=int, default=0, help="persistent CTAs of every placement-kernel launch (0 = the library's defaults: "
                                                             "6 per SM, 32 for single-GPU launches with one end in the host store)")
    ap.add_argument("--grid-ctas-host", type=int, default=0, help="N = 1: CTAs of the launches with one end in the host store only (0 = default)")
    ap.add_argument("--ticket-chunk", type=int, default=0, help="sharded swaps: tiles per draw from the shared counter (0 = 1)")
    ap.add_argument("--mover", type=int, default=0, help="0 placement kernel (default), 1 bulk-copy unit, 2 kernel + copy engine for large parameters")
    ap.add_argument("--host-store", type=int, default=0, help="host store mode: 0 page-locked, 1 write-combined, 2 huge pages")
    ap.add_argument("--sweep", action="store_true", help="N > 1: also time tile sizes and draw sizes of the mover (extra key)")
    ap.add_argument("--nccl-gather", action="store_true", help="N > 1: also time the gather stage over NCCL send/recv (extra key)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.link_probe:
        if rank == 0:
            print(json.dumps(link_probe()), flush=True)
        return 0

    if args.baselines:
        if rank == 0:
            print(json.dumps(run_baselines(args)), flush=True)
        return 0

    if args.corun:
        if rank == 0:
            print(json.dumps(run_corun(args)), flush=True)
        return 0

    if args.impl == "reference":
        if rank != 0:
            return 0
        print(json.dumps(run_reference_pack(args) if args.ref_pack else run_reference(args)), flush=True)
        return 0

    if world > 1 or args.gpus > 1:
        from torpor_b200 import sharded
        line = sharded.bench_main(args, sys.modules[__name__])
        if rank == 0 and line is not None:
            print(json.dumps(line), flush=True)
        return 0

    print(json.dumps(run_single(args)), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
