"""The serverless request stream over plan-only engines (no GPU, no bytes moved): the executor
side of the controller's signals (torpor_b200/serving.py) keeps the engines and the repository
consistent -- every request completes, victims leave the GPU they were evicted from, and every
replica the repository lists is placed on that engine."""
import numpy as np

from torpor_b200 import serving
from torpor_b200 import workloads as W
from torpor_b200.memory_manager import ModelRepo, repo_reset


def test_stream_on_plan_only_engines(built):
    repo_reset()
    out = serving.run_stream(n_gpus=2, n_models=10, rate=300.0, duration_s=1.0, cap_bytes=300 << 20, seed=4,
                             archs=("bert_tiny", "llama_tiny", "resnet50"), devices=[-1, -1], zero_weights=True)
    assert out["completed"] == out["requests"] > 200
    assert out["swaps"] > 20 and out["evictions_in_service"] > 5
    assert out["swaps_from_host"] > 0 and out["swaps_from_replica"] > 0
    assert out["local_hits"] + out["swaps"] == out["requests"]


def test_engines_and_repository_agree_after_churn(built):
    repo_reset()
    srv = serving.SwapServer(3, 200 << 20, devices=[-1, -1, -1], evict_policy="IA")
    archs = ["resnet50", "llama_tiny", "bert_tiny", "resnet50", "llama_tiny", "bert_tiny"]
    for i, a in enumerate(archs):
        srv.cold_start(f"fn{i}", a, 50 + i, tensor_data=lambda k, ws=W.weight_set(a): np.zeros(ws.tensors[k].nbytes, dtype=np.uint8))
    rng = np.random.default_rng(3)
    for step in range(300):
        srv.submit(f"fn{int(rng.integers(0, len(archs)))}", float(step))
        if rng.random() < 0.6:
            for st in srv.state:
                st["until"] = 0.0            # let every running request finish at the next poll
            srv.poll()
    while srv.busy():
        for st in srv.state:
            st["until"] = 0.0
        srv.poll()
    assert srv.completed == 300 and srv.evictions > 0 and srv.ctrl.queue_depth() == 0 and not srv.arrivals
    for i in range(len(archs)):
        homes = set(ModelRepo.active_devices(f"fn{i}"))
        for g in range(3):
            assert srv.engines[g].check_alloc(f"fn{i}") == (g in homes), (i, g, homes)
    srv.close()


def test_large_host_swaps_borrow_idle_links(built):
    repo_reset()
    kw = dict(n_gpus=4, n_models=10, rate=300.0, duration_s=1.0, cap_bytes=300 << 20, seed=4,
              archs=("bert_tiny", "llama_tiny", "resnet50"), devices=[-1] * 4, zero_weights=True,
              pcie_pairs=[0, 1, 2, 3], nvlink=[[0 if i == j else 2 for j in range(4)] for i in range(4)])
    one = serving.run_stream(**kw)
    many = serving.run_stream(shard_min_bytes=50 << 20, **kw)
    assert one["host_swaps_over_several_links"] == 0 and one["links_per_host_swap_mean"] == 1.0
    assert many["completed"] == many["requests"] == one["requests"]
    assert many["host_swaps_over_several_links"] > 5 and 1.0 < many["links_per_host_swap_mean"] <= 4.0
