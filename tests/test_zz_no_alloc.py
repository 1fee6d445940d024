"""The allocation-free placement entry point, tsw_place_segments_static.

Some callers sit where a device allocation is not an option: an executor on the
steady-state path of a GPU-sharing server (cudaMalloc would synchronise the device under
the inference kernels it is serving), a process whose device memory has all gone to the
block pool (the allocation would simply fail), or a process whose CUDA calls are
interposed (the allocation would come back to the server).  For them the library keeps the
kernel's descriptor table in a fixed array inside the module.  This test drives that entry
point through the C ABI, twice in a row with different segment lists, and checks that
every byte -- and the published pointer-table rows -- equal what the allocating entry point
tsw_place_segments produces for the same lists, that device memory does not shrink across
the calls, and that a list beyond the fixed limit is refused.  It is collected last on
purpose: a run that stops at the first failure has then already run every other test.
"""
import numpy as np
import pytest

from torpor_b200 import _cabi
from torpor_b200.memory_manager import (MemoryManager, STATIC_MAX_SEGMENTS, SwapError, place_segments_static,
                                        repo_reset)

pytestmark = pytest.mark.gpu


def make_lists(torch, seed, n_seg):
    """Segments of ragged sizes and alignments inside one source and one destination buffer."""
    rng = np.random.default_rng(seed)
    sizes = [int(x) for x in rng.choice([1, 7, 16, 100, 4096, 65536, 65537, 300000, 1 << 20], size=n_seg)]
    span = [((s + 15) // 16) * 16 + 64 for s in sizes]
    offs = np.concatenate([[0], np.cumsum(span)]).astype(np.int64)
    total = int(offs[-1]) + 64
    src = torch.from_numpy(rng.integers(0, 256, size=total, dtype=np.uint8)).cuda()
    shift = [int(x) for x in rng.integers(0, 16, size=n_seg)]
    s_off = [int(offs[i]) + 16 + shift[i] for i in range(n_seg)]
    d_off = [int(offs[i]) + 32 + shift[i] for i in range(n_seg)]   # same alignment class as the source
    return src, total, sizes, s_off, d_off


def run_both(torch, eng, seed, n_seg):
    src, total, sizes, s_off, d_off = make_lists(torch, seed, n_seg)
    outs = []
    for use_static in (False, True):
        dst = torch.full((total,), 0xA5, dtype=torch.uint8, device="cuda")
        done = torch.zeros(n_seg, dtype=torch.int32, device="cuda")
        t_phys = torch.zeros(n_seg, dtype=torch.int64, device="cuda")
        t_flag = torch.zeros(n_seg, dtype=torch.int32, device="cuda")
        pub = _cabi.Publish(done.data_ptr(), t_phys.data_ptr(), t_flag.data_ptr(), 0, 0, _cabi.READY_CUDA, 0)
        s_list = [src.data_ptr() + o for o in s_off]
        d_list = [dst.data_ptr() + o for o in d_off]
        torch.cuda.synchronize()
        if use_static:
            free_before = torch.cuda.mem_get_info()[0]
            place_segments_static(0, s_list, d_list, sizes, tile_bytes=65536, publish=pub, stream=0)
            torch.cuda.synchronize()
            assert torch.cuda.mem_get_info()[0] >= free_before, "the allocation-free entry point shrank free device memory"
        else:
            eng.place_segments(s_list, d_list, sizes, tile_bytes=65536, publish=pub, sync=True)
        rel_phys = (t_phys - dst.data_ptr()).cpu().numpy()
        outs.append((dst.cpu().numpy(), rel_phys, t_flag.cpu().numpy(), done.cpu().numpy()))
    (b0, p0, f0, c0), (b1, p1, f1, c1) = outs
    assert np.array_equal(b0, b1), "bytes differ between the allocating and the allocation-free entry point"
    assert np.array_equal(p0, p1) and np.array_equal(f0, f1) and np.array_equal(c0, c1)
    assert (f1 == _cabi.READY_CUDA).all() and (c1 == 0).all() and np.array_equal(p1, np.array(d_off))
    # and both are right
    want = np.full(total, 0xA5, dtype=np.uint8)
    inp = src.cpu().numpy()
    for so, do, n in zip(s_off, d_off, sizes):
        want[do:do + n] = inp[so:so + n]
    assert np.array_equal(b1, want)


def test_allocation_free_entry_point_matches_the_allocating_one(built):
    import torch
    assert torch.cuda.is_available(), "this test needs a CUDA device"
    repo_reset()
    eng = MemoryManager(0, device=0)
    try:
        run_both(torch, eng, seed=21, n_seg=300)     # first call on the device: looks the scratch address up
        run_both(torch, eng, seed=22, n_seg=57)      # second call: finds the first call's table in the scratch
        # calls that did not overlap leave nothing in the word the kernel reports a clobbered table in,
        # and the entry points give the caller's current device back as they found it
        from torpor_b200.memory_manager import place_segments_static_status
        assert place_segments_static_status(0) == 0
        assert torch.cuda.current_device() == 0
    finally:
        eng.close()
        repo_reset()


def test_allocation_free_entry_point_refuses_oversized_lists(built):
    import torch
    assert torch.cuda.is_available(), "this test needs a CUDA device"
    n = STATIC_MAX_SEGMENTS + 1
    buf = torch.zeros(1024, dtype=torch.uint8, device="cuda")
    with pytest.raises(SwapError) as e:
        place_segments_static(0, [buf.data_ptr()] * n, [buf.data_ptr() + 512] * n, [0] * n)
    assert e.value.code == _cabi.ERR_BUFFER and "16384" in str(e.value)
    with pytest.raises(SwapError):
        place_segments_static(0, [buf.data_ptr()], [buf.data_ptr() + 512], [16], tile_bytes=24)
