"""Static activation memory plan: one arena per launch plan, blocks handed back when their last reader is lowered.

A launch plan is built once per shape and replayed in a fixed order on one stream, so two buffers whose lifetimes
do not overlap in that order can share memory. The lowering asks the arena for every channel-innermost activation
buffer; after each graph node it tells the arena which address ranges are still needed (values with readers to
come, graph outputs, promised concatenation slices, features held back for a folded gate) and everything else
goes back to the free list. Blocks come from a few large slabs (first fit, neighbours merged on release), so the
plan's activation footprint is ``arena.capacity`` instead of the sum of all buffers (``arena.requested``).

The reference leaves this to its back ends (TensorRT's engine workspace,
fastdeploy/runtime/backends/tensorrt/trt_backend.cc:327-339; Paddle Inference's memory-optimise pass,
fastdeploy/runtime/backends/paddle/paddle_backend.cc).
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Sequence, Tuple

import torch

ALIGN = 512


class Arena:
    def __init__(self, device: torch.device, slab_bytes: int = 256 << 20):
        self.device = device
        self.slab_bytes = int(slab_bytes)
        self.slabs: List[torch.Tensor] = []
        self.free: List[List[Tuple[int, int]]] = []          # per slab: sorted (offset, size) holes
        self.live: Dict[int, Tuple[int, int, int]] = {}      # block id -> (slab, offset, size)
        self._next = 0
        self.requested = 0                                   # bytes asked for in total (= footprint without reuse)
        self.peak_live = 0

    # ------------------------------------------------------------------ allocation
    @property
    def capacity(self) -> int:
        return sum(int(s.numel()) for s in self.slabs)

    @property
    def live_bytes(self) -> int:
        return sum(sz for _, _, sz in self.live.values())

    def _take(self, nbytes: int) -> Tuple[int, int]:
        for si, holes in enumerate(self.free):
            for hi, (off, size) in enumerate(holes):
                if size >= nbytes:
                    if size == nbytes:
                        holes.pop(hi)
                    else:
                        holes[hi] = (off + nbytes, size - nbytes)
                    return si, off
        # slabs grow with the arena (16 MiB, then as much as there already is, up to slab_bytes) so that a small
        # plan does not pay for a large first slab
        size = max(nbytes, min(self.slab_bytes, max(16 << 20, self.capacity)))
        self.slabs.append(torch.zeros(size, dtype=torch.uint8, device=self.device))
        self.free.append([(nbytes, size - nbytes)] if size > nbytes else [])
        return len(self.slabs) - 1, 0

    def alloc(self, shape: Sequence[int], dtype: torch.dtype) -> torch.Tensor:
        """A zeroed contiguous tensor inside the arena (zeroed now; a later tenant of the same bytes sees whatever the
        previous one left, which is what every kernel that writes its whole output expects)."""
        numel = 1
        for d in shape:
            numel *= int(d)
        item = torch.empty(0, dtype=dtype).element_size()
        nbytes = max(ALIGN, (numel * item + ALIGN - 1) // ALIGN * ALIGN)
        si, off = self._take(nbytes)
        self.live[self._next] = (si, off, nbytes)
        self._next += 1
        self.requested += nbytes
        self.peak_live = max(self.peak_live, self.live_bytes)
        t = self.slabs[si][off:off + numel * item].view(dtype).view(list(shape))
        t.zero_()
        return t

    def _release(self, key: int) -> None:
        si, off, size = self.live.pop(key)
        holes = self.free[si]
        holes.append((off, size))
        holes.sort()
        merged: List[Tuple[int, int]] = []
        for o, s in holes:
            if merged and merged[-1][0] + merged[-1][1] == o:
                merged[-1] = (merged[-1][0], merged[-1][1] + s)
            else:
                merged.append((o, s))
        self.free[si] = merged

    # ------------------------------------------------------------------ liveness
    @staticmethod
    def span(t: torch.Tensor) -> Tuple[int, int]:
        """Address range ``[lo, hi)`` that a (possibly strided) tensor can touch."""
        if t.numel() == 0:
            return t.data_ptr(), t.data_ptr()
        last = sum((int(s) - 1) * int(st) for s, st in zip(t.shape, t.stride()))
        return t.data_ptr(), t.data_ptr() + (last + 1) * t.element_size()

    def release_unreferenced(self, needed: Iterable[torch.Tensor]) -> int:
        """Frees every block that none of the ``needed`` tensors overlaps; returns the bytes handed back."""
        if not self.live:
            return 0
        bases = [int(s.data_ptr()) for s in self.slabs]
        ranges: List[Tuple[int, int]] = []
        for t in needed:
            if t is None or t.device.type != self.device.type:
                continue
            lo, hi = self.span(t)
            if hi > lo:
                ranges.append((lo, hi))
        freed = 0
        for key, (si, off, size) in list(self.live.items()):
            lo, hi = bases[si] + off, bases[si] + off + size
            if not any(a < hi and lo < b for a, b in ranges):
                self._release(key)
                freed += size
        return freed

    def report(self) -> Dict[str, int]:
        return {"arena_bytes": self.capacity, "requested_bytes": self.requested, "peak_live_bytes": self.peak_live,
                "slabs": len(self.slabs)}
