"""The activation arena's allocator and liveness rule, on host memory (the same code serves device plans)."""
import ctypes

import torch

from fastdeploy_b200.runtime.arena import ALIGN, Arena


def test_blocks_are_reused_merged_and_never_overlap_live_tensors():
    a = Arena(torch.device("cpu"), slab_bytes=1 << 20)
    t1 = a.alloc((100, 100), torch.float16)            # 20 000 B -> 20 480
    t2 = a.alloc((64, 64), torch.float32)              # 16 384 B
    t3 = a.alloc((10,), torch.float32)                 # rounds up to one ALIGN unit
    assert a.live_bytes == 20480 + 16384 + ALIGN and a.requested == a.live_bytes and len(a.slabs) == 1
    assert (t1 == 0).all() and t1.is_contiguous() and (t2.data_ptr() - a.slabs[0].data_ptr()) % ALIGN == 0
    # a view into t2 keeps t2's block; t1 and t3 go back
    view = t2[3:5]
    freed = a.release_unreferenced([view])
    assert freed == 20480 + ALIGN and a.live_bytes == 16384
    # the hole in front of t2 is taken again (first fit), and the tail merged with the rest of the slab
    t4 = a.alloc((50, 100), torch.float16)             # 10 000 B -> 10 240: fits where t1 was
    assert t4.data_ptr() == t1.data_ptr()
    lo2, hi2 = Arena.span(t2)
    lo4, hi4 = Arena.span(t4)
    assert hi4 <= lo2 or hi2 <= lo4
    assert a.capacity == a.slabs[0].numel() and a.peak_live == 20480 + 16384 + ALIGN
    # nothing needed: everything is free again and one hole spans the slab
    a.release_unreferenced([])
    assert a.live_bytes == 0 and a.free[0] == [(0, a.slabs[0].numel())]
    rep = a.report()
    assert rep["requested_bytes"] == 20480 + 16384 + ALIGN + 10240 and rep["slabs"] == 1


def test_strided_views_count_by_the_bytes_they_can_touch():
    a = Arena(torch.device("cpu"), slab_bytes=1 << 20)
    t1 = a.alloc((8, 16, 16, 64), torch.float16)
    t2 = a.alloc((8, 16, 16, 64), torch.float16)
    sl = t1[..., 8:16]                                  # a channel slice: spans almost the whole block
    lo, hi = Arena.span(sl)
    assert lo == t1.data_ptr() + 16 and hi == t1.data_ptr() + t1.numel() * 2 - 96
    assert a.release_unreferenced([sl]) == t2.numel() * 2
    # a block larger than the slab size gets a slab of its own; slabs grow with the arena
    big = a.alloc((3 << 20,), torch.uint8)
    assert len(a.slabs) == 2 and a.slabs[1].numel() == 3 << 20 and big.numel() == 3 << 20
