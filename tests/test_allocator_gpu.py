"""Caching device / pinned pools: reuse, stream-ordered release, statistics."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_pinned_and_device_pools_reuse_blocks():
    import gc
    from fastdeploy_b200.core import allocator as A
    gc.collect()
    torch.cuda.synchronize()
    A.trim()
    s0 = A.stats()
    a = A.pinned_tensor([1000, 3], torch.float32)
    assert a.is_pinned() and a.shape == (1000, 3)
    a.fill_(2.5)
    d = A.device_tensor([1000, 3], torch.float32)
    d.copy_(a, non_blocking=True)
    torch.cuda.synchronize()
    assert float(d.sum()) == 7500.0
    ptr_a, ptr_d = a.data_ptr(), d.data_ptr()
    s1 = A.stats()
    assert s1["pinned"]["allocated"] - s0["pinned"]["allocated"] == 16384        # 12000 bytes -> 16 KiB class
    assert s1["device"]["allocated"] - s0["device"]["allocated"] == 16384
    del a, d
    torch.cuda.synchronize()
    s_free = A.stats()
    assert s_free["pinned"]["cached"] - s1["pinned"]["cached"] == 16384          # back in the cache, not at the driver
    b = A.pinned_tensor([3000], torch.float32)        # same size class: a cached block comes back, no driver call
    e = A.device_tensor([12000], torch.uint8)
    s2 = A.stats()
    assert s2["pinned"]["driver_calls"] == s1["pinned"]["driver_calls"]
    assert s2["device"]["driver_calls"] == s1["device"]["driver_calls"]
    assert s2["pinned"]["cache_hits"] == s1["pinned"]["cache_hits"] + 1
    assert s2["device"]["cache_hits"] == s1["device"]["cache_hits"] + 1
    assert ptr_a and ptr_d
    del b, e
    torch.cuda.synchronize()
    assert A.trim() >= 32768


def test_block_released_on_a_busy_stream_is_not_handed_out_early():
    from fastdeploy_b200.core import allocator as A
    A.trim()
    side = torch.cuda.Stream()
    big = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    with torch.cuda.stream(side):
        t = A.device_tensor([1 << 20], torch.uint8)
        ptr = t.data_ptr()
        for _ in range(20):
            big.fill_(1)                      # keeps the side stream busy for a few milliseconds
        del t                                 # released with an event on the busy stream
        u = A.device_tensor([1 << 20], torch.uint8)
        assert u.data_ptr() != ptr            # the event has not completed: a fresh block is used instead
    torch.cuda.synchronize()
    v = A.device_tensor([1 << 20], torch.uint8)
    assert v.data_ptr() == ptr                # now it is free again
