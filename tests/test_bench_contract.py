"""bench.py's lines without a GPU: the reference arm (here the CPU restatement or the reference's
headers over host memory stand in for the GPU run) prints ONE JSON line with the keys the contract
names, labelled with the weight set it really timed; the pack baseline prints its own."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _line(*args):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                       text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-1500:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1, r.stdout[-500:]
    return json.loads(lines[0])


def test_reference_arm_line(built):
    d = _line("--impl", "reference", "--workload", "resnet50", "--steps", "3", "--warmup", "1")
    assert d["impl"] == "reference" and d["metric"] == "model_swap_in_throughput" and d["unit"] == "GB/s"
    assert d["steps"] == 3 and d["warmup"] == 1 and d["higher_is_better"] is True and d["vs_baseline"] is None
    assert d["value"] > 0 and d["ms_per_step"] > 0
    assert "resnet50: 161 tensors, 102228128 B" in d["config"]["workload"]          # the set that was timed, by name and size
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("reference", "port") and cb["cores"] >= 1 and cb["value"] == d["value"]
    assert "resnet50: 161 tensors" in cb["sample"] and "IO_THREAD_NUM" in cb["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    # value = bytes / (signal-to-ready + evict), not the harness's wall clock
    assert abs(d["value"] - 102228128 / (d["ms_per_step"] / 1e3) / 1e9) < 1e-6 * d["value"] + 1e-9


def test_other_ranks_of_the_reference_arm_print_nothing(built):
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--workload", "resnet50"],
                       stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=300, env=env)
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_pack_baseline_line(built):
    from oracle import tso
    import pytest
    if not tso.available("ref_fake"):
        pytest.skip("the reference's headers are not built here")
    d = _line("--impl", "reference", "--ref-pack", "--ref-sample", "resnet50", "--ref-io-threads", "2", "--steps", "4", "--warmup", "1")
    p = d["pack"]
    assert p["cores"] == 2 and p["value"] > 0 and p["kind"] == "reference" and "resnet50: 161 tensors" in p["sample"]
