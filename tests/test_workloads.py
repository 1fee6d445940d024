"""The synthetic weight sets have the tensor counts, parameter counts and byte sizes of
the architectures they stand for, and the client-allocator emulation groups them into
the block shapes the pool is built around."""
from collections import Counter

import numpy as np
import pytest

from torpor_b200 import workloads as W

EXPECT = {
    # name: (tensors, parameters, bytes, model blocks)
    "resnet50": (161, 25_557_032, 102_228_128, 14),
    "bert_base": (199, 109_482_240, 437_928_960, 21),
    "bert_large": (391, 335_141_888, 670_283_776, 31),
    "llama2_7b": (291, 6_738_415_616, 13_476_831_232, 227),
    "vgg19": (38, 143_667_240, 574_668_960, 9),
}


@pytest.mark.parametrize("name", list(EXPECT))
def test_shapes(name):
    ws = W.weight_set(name)
    blocks, where = W.pack_blocks(ws)
    assert (len(ws.tensors), ws.numel, ws.nbytes, len(blocks)) == EXPECT[name]
    for (b, off), t in zip(where, ws.tensors):
        assert off % W.PACK_ALIGN == 0 and off + t.nbytes <= blocks[b].size
    sizes = Counter(b.size for b in blocks)
    assert all(s in (W.SMALL_BLOCK, W.LARGE_BLOCK) or (s >= W.LARGE_LIMIT and s % W.ROUND_LARGE == 0) for s in sizes)


def test_values_are_seeded_and_scaled():
    ws = W.weight_set("resnet50")
    a = W.tensor_values(ws, 3)
    assert np.array_equal(a, W.tensor_values(W.weight_set("resnet50"), 3))
    assert not np.array_equal(a, W.tensor_values(W.weight_set("resnet50", seed=5), 3))
    big = W.tensor_values(ws, len(ws.tensors) - 2)  # fc.weight
    assert big.dtype == np.float32 and abs(float(big.std()) - 0.02) < 5e-4 and abs(float(big.mean())) < 5e-4
    assert W.tensor_values(W.weight_set("bert_large"), 1).dtype == np.float16


def test_cold_start_stream_order():
    ws = W.weight_set("bert_tiny")
    calls = list(W.cold_start_stream(ws))
    ops = [c.op for c in calls]
    assert ops.count("memcpy") == len(ws.tensors) == ops.count("access")
    assert ops.index("sync_done") > max(i for i, o in enumerate(ops) if o == "memcpy")
    assert [c.tensor for c in calls if c.op == "access"] == list(range(len(ws.tensors)))
    seen = set()
    for c in calls:  # a tensor is uploaded only into a block that was malloc'ed before
        if c.op == "malloc" and c.is_model:
            seen.add(c.block)
        if c.op == "memcpy":
            assert c.block in seen


def test_mixed_stream_shape():
    archs, times, picks = W.mixed_stream()
    assert len(archs) == 64 and set(archs) <= {"resnet50", "bert_base", "bert_large", "vgg19"}
    assert 22000 < len(times) < 26000 and times[-1] < 120.0 and (np.diff(times) > 0).all()
    counts = np.bincount(picks, minlength=64)
    assert counts.max() > 8 * np.median(counts)   # Zipf head
