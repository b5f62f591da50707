"""Host-side logic of the multi-GPU layer (no GPU)."""
import pytest

from fastdeploy_b200.parallel.comm import ALIGN, HeapLayout, shard_rows


def test_heap_layout_is_deterministic_and_aligned():
    a, b = HeapLayout(1 << 20), HeapLayout(1 << 20)
    seq = [("x", 1000), ("slots", 70000), ("cnt", 16)]
    off_a = [a.alloc(n, s).offset for n, s in seq]
    off_b = [b.alloc(n, s).offset for n, s in seq]
    assert off_a == off_b and all(o % ALIGN == 0 for o in off_a)
    assert a.alloc("x", 500).offset == off_a[0]          # same name -> same block
    with pytest.raises(ValueError):
        a.alloc("x", 2000)
    with pytest.raises(MemoryError):
        a.alloc("huge", 1 << 21)


def test_shard_rows():
    assert shard_rows(8192, 8) == 1024
    with pytest.raises(ValueError):
        shard_rows(1000, 8)
    with pytest.raises(ValueError):
        shard_rows(8 * 64, 8)
