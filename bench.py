#!/usr/bin/env python
"""Benchmark of the model swap path: swap-in throughput (GB/s) and ms per model.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one swap-in of the workload's weight set into the target GPU's pool
(block placement, pointer-table rebind, data movement, readiness publish) followed
by the eviction that makes room for the next step.  Two arms are timed with the
same engine and kernel:

  value  source = a resident replica in HBM (the reference's replica swap,
         memory_manager.hpp:394-396; at N > 1 each rank's staged share, gathered
         over NVLink) -- inputs already on the device, HBM / NVLink bound;
  e2e    source = the page-locked host model store, through the public swap-in call
         -- every byte crosses PCIe inside the timed region.

`--impl reference` times the reference's own swap path (its headers compiled where
they lie, oracle/_ref) on a bounded sample of the same workload with all host
threads; if that checker is absent the CPU restatement is timed instead.
Prints ONE JSON line on rank 0.
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


def generate_tensors(ws, threads):
    from torpor_b200 import workloads as W
    pool = ThreadPoolExecutor(max(1, threads))
    futs = {i: pool.submit(W.tensor_bytes, ws, i) for i in range(len(ws.tensors))}
    return pool, (lambda i: futs.pop(i).result())


# ------------------------------------------------------------------ reference arm

def run_reference(args, quiet=False):
    """The reference's host-driven swap path (I/O threads staging into pinned memory,
    per-parameter cudaMemcpyAsync, event sync per 2 MiB group) on a bounded sample."""
    from oracle import tso
    from torpor_b200 import workloads as W
    ncpu = os.cpu_count() or 1
    have_gpu = False
    try:
        import torch
        have_gpu = torch.cuda.is_available()
    except Exception:
        pass
    if tso.available("ref_cuda") and have_gpu:
        kind, lib, io_threads = "reference", tso.load("ref_cuda"), (args.ref_io_threads or max(1, ncpu))
        what = "reference headers (memory_manager.hpp:213-449) + CUDA runtime"
    else:
        kind, lib, io_threads = "port", tso.load("oracle"), 1
        what = "CPU restatement (oracle/torpor_oracle.cpp), host memcpy into the block layout"
    ws = W.weight_set(args.ref_sample)
    lib.reset_world()
    src = args.ref_src_gpu
    pool, data = generate_tensors(ws, min(ncpu, 16))
    if src >= 0:
        # the reference's replica swap (memory_manager.hpp:394-396): the model is resident on GPU `src`,
        # GPU 0 copies it parameter by parameter with cudaMemcpyPeerAsync
        if kind != "reference":
            return {"impl": "reference", "unavailable": "the replica-swap baseline needs the reference library and two GPUs"}
        pairs = lib.enable_peer_access(src + 1)          # as the controller does at start-up (controller.hpp:63-75)
        what += f"; peer access enabled for {pairs} directed pairs"
        holder = lib.manager(server_id=src, budget=0, gpu_count=src + 1, io_threads=io_threads)
        m = lib.manager(server_id=0, budget=0, gpu_count=src + 1, io_threads=io_threads)
        W.cold_start(holder, "ref", ws, tensor_data=data)
        lib.set_model_status("ref", src, True)
        what += f"; replica swap from GPU {src} (cudaMemcpyPeerAsync per parameter)"
    else:
        m = lib.manager(budget=0, io_threads=io_threads)
        W.cold_start(m, "ref", ws, tensor_data=data)
        m.evict("ref")
    pool.shutdown()
    for _ in range(args.warmup):
        m.swap_in_timed("ref", src); m.evict("ref")
    t_sig, t_evict = [], []
    t0 = time.perf_counter()
    for _ in range(args.steps):
        t_sig.append(m.swap_in_timed("ref", src))
        te = time.perf_counter()
        m.evict("ref")
        t_evict.append((time.perf_counter() - te) * 1e6)
    wall = time.perf_counter() - t0
    gbs = ws.nbytes * args.steps / wall / 1e9
    cores = io_threads + 1 if kind == "reference" else 1
    sample = (f"{args.ref_sample}: {len(ws.tensors)} tensors, {ws.nbytes} B of the workload's shape; "
              f"{args.warmup} warm-up + {args.steps} swap-ins with forced evict between; {what}; "
              f"IO_THREAD_NUM={io_threads}")
    line = {
        # the reference's swap uses one GPU's link whatever N is; n_gpus names the configuration compared
        "impl": "reference", "metric": "model_swap_in_throughput", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": wall / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": workload_config(args, args.gpus),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": kind, "sample": sample,
                         "host_cores": ncpu, "signal_to_ready_ms_median": statistics.median(t_sig) / 1e3,
                         "signal_to_ready_gbs": ws.nbytes / (statistics.median(t_sig) / 1e6) / 1e9,
                         "swap_out_metadata_only_us_median": statistics.median(t_evict)},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    return line


def run_baselines(args):
    """Reported baselines around the path, each reference run in its own process (the reference's
    threads cannot be joined): swap-in with the reference's default IO_THREAD_NUM=4 and with one
    staging thread per host core, its replica swap over cudaMemcpyPeerAsync when a second GPU is
    there, its metadata-only swap-out, and plain copy-engine rates of this box."""
    import torch
    ncpu = os.cpu_count() or 1
    me = os.path.abspath(__file__)

    def ref(*extra):
        r = subprocess.run([sys.executable, me, "--impl", "reference", "--steps", str(args.steps), "--warmup",
                            str(args.warmup), "--ref-sample", args.ref_sample, "--workload", args.workload, *extra],
                           stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=900)
        for ln in r.stdout.splitlines():
            if ln.startswith("{"):
                d = json.loads(ln)
                return d.get("cpu_baseline", d)
        return {"failed": r.stderr[-300:]}

    out = {"host_cores": ncpu, "gpus": torch.cuda.device_count(), "sample": args.ref_sample,
           "reference_swap_in_io4": ref("--ref-io-threads", "4"),
           "reference_swap_in_io_all": ref("--ref-io-threads", str(ncpu))}
    nbytes = 1 << 30
    host = torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)
    dev0 = torch.empty(nbytes, dtype=torch.uint8, device="cuda:0")

    def timed(fn, dev=0, reps=5):
        torch.cuda.synchronize(dev)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        fn()
        with torch.cuda.device(dev):
            a.record()
            for _ in range(reps):
                fn()
            b.record()
        torch.cuda.synchronize(dev)
        return nbytes * reps / (a.elapsed_time(b) / 1e3) / 1e9

    out["copy_engine_h2d_pinned_gbs"] = timed(lambda: dev0.copy_(host, non_blocking=True))
    out["copy_engine_d2h_pinned_gbs"] = timed(lambda: host.copy_(dev0, non_blocking=True))
    if torch.cuda.device_count() >= 2:
        out["reference_replica_swap"] = ref("--ref-src-gpu", "1")
        dev1 = torch.empty(nbytes, dtype=torch.uint8, device="cuda:1")
        out["copy_engine_peer_gbs"] = timed(lambda: dev0.copy_(dev1, non_blocking=True))
        del dev1
        n = torch.cuda.device_count()
        if n > 2:
            # every other GPU's copy engine pushes 1 GiB into GPU 0 at once: the (n-1) -> 1 gather ceiling
            dst = [torch.empty(nbytes, dtype=torch.uint8, device="cuda:0") for _ in range(n - 1)]
            src = [torch.empty(nbytes, dtype=torch.uint8, device=f"cuda:{i}") for i in range(1, n)]
            streams = [torch.cuda.Stream(device=i) for i in range(1, n)]

            def gather():
                for d, s_, st in zip(dst, src, streams):
                    with torch.cuda.stream(st):
                        d.copy_(s_, non_blocking=True)
            best = 0.0
            for _ in range(4):
                for i in range(n):
                    torch.cuda.synchronize(i)
                t0 = time.perf_counter()
                gather()
                for i in range(n):
                    torch.cuda.synchronize(i)
                best = max(best, nbytes * (n - 1) / (time.perf_counter() - t0) / 1e9)
            out["copy_engine_gather_gbs"] = {"value": best, "what": f"{n - 1} -> 1 concurrent peer copies of 1 GiB each, wall clock, best of 4"}
            del dst, src
        # the same replica swap through this library: GPU 0 places the model from GPU 1's pool over NVLink
        from torpor_b200 import workloads as W
        from torpor_b200.memory_manager import MemoryManager, ModelRepo, repo_reset
        ws = W.weight_set(args.ref_sample)
        repo_reset()
        holder = MemoryManager(W.pool_budget_for(ws), device=1, server_id=1, gpu_count=2, host_arena_bytes=W.host_store_bytes(ws))
        target = MemoryManager(W.pool_budget_for(ws), device=0, server_id=0, gpu_count=2)
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
        out["ours_replica_swap"] = {"signal_to_ready_gbs": ws.nbytes / statistics.median(wall) / 1e9,
                                    "signal_to_ready_ms_median": statistics.median(wall) * 1e3,
                                    "kernel_gbs": ws.nbytes / statistics.median(dev) / 1e9,
                                    "what": "tsw_swap_in(func, src_gpu=1) + tsw_wait_ready on GPU 0: place_kernel reads GPU 1's pool over NVLink"}
        target.close(); holder.close(); repo_reset()
    return {"baselines": out}


def workload_config(args, n):
    from torpor_b200 import workloads as W
    ws = W.weight_set(args.workload)
    return {"workload": f"{args.workload}: {len(ws.tensors)} tensors, {ws.nbytes} B, N(0,0.02) seeded, "
                        f"client-allocator block layout ({len(W.pack_blocks(ws)[0])} model blocks)",
            "target_gpus": 1, "participating_gpus": n, "l2": "inputs larger than L2 (no flush needed)",
            "step": "swap-in (place, rebind, move, publish) + evict"}


# ------------------------------------------------------------------ our arm, one GPU

def run_single(args):
    import torch
    from torpor_b200 import workloads as W
    from torpor_b200.memory_manager import MemoryManager, ModelRepo, repo_reset, checksum_host

    peaks, peak_kind = measured_peaks()
    ncpu = os.cpu_count() or 1

    # CPU / reference baseline first, in its own process (its threads and pool cannot be torn down)
    cpu_baseline = None
    if not args.no_cpu_baseline:
        try:
            r = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference", "--steps", "5",
                                "--warmup", "1", "--ref-sample", args.ref_sample, "--workload", args.workload],
                               stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=600)
            for ln in r.stdout.splitlines():
                if ln.startswith("{"):
                    cpu_baseline = json.loads(ln)["cpu_baseline"]
        except Exception as ex:  # reported, never fatal for the GPU arm
            cpu_baseline = {"value": None, "unit": "GB/s", "cores": 0, "kind": "port", "sample": f"failed: {ex}"}

    torch.cuda.set_device(0)
    ws = W.weight_set(args.workload)
    budget = W.pool_budget_for(ws)
    arena = W.host_store_bytes(ws)
    repo_reset()
    replica = MemoryManager(budget, device=0, server_id=1, gpu_count=2, host_arena_bytes=arena)
    target = MemoryManager(budget, device=0, server_id=0, gpu_count=2)

    pool, data = generate_tensors(ws, min(ncpu, 16))
    sums = {}

    def data_and_sum(i):
        b = data(i)
        if i % 16 == 0:
            sums[i] = checksum_host(b)
        return b

    t0 = time.time()
    W.cold_start(replica, "model", ws, tensor_data=data_and_sum)
    pool.shutdown()
    torch.cuda.synchronize()
    cold_s = time.time() - t0
    ModelRepo.add_model_info("model", 1)

    def verify():
        got = target.checksum_resident("model")
        for i, s in sums.items():
            if not np.array_equal(got[i], s):
                raise RuntimeError(f"resident bytes of tensor {i} differ from the host store")

    def cycle(src):
        target.swap_in("model", src)
        target.wait_ready("model")
        target.evict("model")

    def timed(src, steps, warmup):
        for _ in range(warmup):
            cycle(src)
        dev_ns = []
        launches0 = target.stats()["kernel_launches"]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            target.swap_in("model", src)
            target.wait_ready("model")
            dev_ns.append(target.stats()["last_swap_device_ns"])
            target.evict("model")
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        return wall, dev_ns, target.stats()["kernel_launches"] - launches0

    # correctness of both arms before anything is timed
    target.swap_in("model", 1); target.wait_ready("model"); verify(); target.evict("model")
    target.swap_in("model", -1); target.wait_ready("model"); verify(); target.evict("model")

    sampler = ClockSampler(0)
    sampler.start()
    wall_v, dev_v, launches_v = timed(1, args.steps, args.warmup)
    wall_e, dev_e, launches_e = timed(-1, args.steps, args.warmup)
    # swap-out with write-back (no counterpart in the reference, whose swap-out moves nothing):
    # resident bytes -> host store through the same kernel, PCIe D2H bound
    wb = []
    for _ in range(3):
        target.swap_in("model", 1); target.wait_ready("model")
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        target.evict("model", writeback=True)
        wb.append(time.perf_counter() - t0)
    clocks = sampler.stop()

    # measured DMA peak of this box's link, for context next to the theoretical 63 GB/s
    x = torch.empty(1 << 30, dtype=torch.uint8).pin_memory()
    y = torch.empty(1 << 30, dtype=torch.uint8, device="cuda")
    best = 0.0
    for _ in range(3):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); y.copy_(x, non_blocking=True); e.record(); torch.cuda.synchronize()
        best = max(best, (1 << 30) / (s.elapsed_time(e) / 1e3) / 1e9)
    del x, y

    B = ws.nbytes
    value = B * args.steps / wall_v / 1e9
    e2e = B * args.steps / wall_e / 1e9
    kern_v = statistics.mean(dev_v) / 1e9
    kern_e = statistics.mean(dev_e) / 1e9
    achieved = 2 * B / kern_v / 1e9
    n_params = len(ws.tensors)
    line = {
        "metric": "model_swap_in_throughput", "value": value, "unit": "GB/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": wall_v / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": workload_config(args, 1),
        "value_arm": "swap-in from a resident HBM replica on the same GPU (replica swap path)",
        "e2e": {"value": e2e, "unit": "GB/s", "ms_per_model": wall_e / args.steps * 1e3,
                "h2d_bytes_per_step": B + 44 * n_params, "d2h_bytes_per_step": 12 * n_params,
                "device_ms_per_model": kern_e * 1e3,
                "what": "tsw_swap_in from the page-locked host store + tsw_wait_ready + tsw_evict through the C ABI"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm_gbs"], "peak_kind": f"{peak_kind} copy bandwidth (burst)",
                     "kernel": "place_kernel (HBM -> HBM)", "algorithmic_bytes_per_launch": 2 * B,
                     "launch_ms": kern_v * 1e3,
                     "traffic": (DRAM_TRAFFIC_PER_ALGO_BYTE * 2 * B) if DRAM_TRAFFIC_PER_ALGO_BYTE else None},
        "link_roofline": {"bound": "pcie", "achieved": B / kern_e / 1e9, "achieved_wall": e2e,
                          "peak": PCIE_GEN5_X16_GBS, "unit": "GB/s", "frac": (B / kern_e / 1e9) / PCIE_GEN5_X16_GBS,
                          "frac_wall": e2e / PCIE_GEN5_X16_GBS, "peak_kind": "theoretical PCIe Gen5 x16, one direction",
                          "cudaMemcpyAsync_pinned_h2d_gbs": best, "kernel": "place_kernel (host store -> HBM, zero-copy)"},
        "swap_out_writeback": {"value": ws.nbytes / min(wb) / 1e9, "unit": "GB/s", "ms_per_model": min(wb) * 1e3,
                               "frac_of_pcie": ws.nbytes / min(wb) / 1e9 / PCIE_GEN5_X16_GBS,
                               "what": "tsw_evict(writeback=1): pool -> host store, D2H over PCIe; the reference's swap-out is metadata only"},
        "cpu_baseline": cpu_baseline,
        "gpu_launches": launches_v, "gpu_launches_e2e": launches_e,
        "clocks": clocks, "host_cores": ncpu, "cold_start_s": cold_s,
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
    ap.add_argument("--ref-sample", default="llama_mid")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--ref-io-threads", type=int, default=0, help="IO_THREAD_NUM of the reference arm (0 = host cores)")
    ap.add_argument("--ref-src-gpu", type=int, default=-1, help="reference arm: swap from a replica on this GPU instead of the host store")
    ap.add_argument("--baselines", action="store_true",
                    help="print the reported baselines around the path (reference with its default 4 and with all "
                         "staging threads, its replica swap, copy-engine rates) as one JSON line; not the contract line")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.baselines:
        if rank == 0:
            print(json.dumps(run_baselines(args)), flush=True)
        return 0

    if args.impl == "reference":
        if rank != 0:
            return 0
        print(json.dumps(run_reference(args)), flush=True)
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
