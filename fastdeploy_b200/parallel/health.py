"""Rank liveness on the host: heartbeats through a key-value store, checked before every launch that
waits on peers.

A kernel that waits on a peer has a clock budget (a second or so) and reports a status instead of
hanging, but the cheap way to survive a lost rank is not to launch at all: every rank bumps a counter in
the process group's store between steps (``beat``), and ``guard`` - called before a collective or a fused
peer kernel is queued - raises :class:`RankLostError` when a peer's counter has not moved for
``timeout_s``. Ranks leave only between steps, with nothing of theirs in flight; ``leave`` marks that as
orderly so that the others shrink the group instead of reporting a failure. The store is any object with
``set(key, bytes)`` / ``get(key)`` / ``add(key, n)`` (``torch.distributed.TCPStore``, ``FileStore``,
``HashStore``), so the logic runs with plain processes or threads on a CPU-only machine.

The reference has no multi-rank execution and therefore nothing to compare with.
"""
from __future__ import annotations

import time
from typing import Dict, List, Optional


class RankLostError(RuntimeError):
    def __init__(self, ranks: List[int], what: str):
        super().__init__(f"{what}: rank(s) {ranks} stopped answering")
        self.ranks = ranks


class RankHealth:
    def __init__(self, store, rank: int, world: int, timeout_s: float = 2.0, prefix: str = "fdb/health"):
        self.store, self.rank, self.world, self.timeout_s, self.prefix = store, rank, world, timeout_s, prefix
        self._last_seen: Dict[int, tuple] = {}
        self.store.add(self._key(rank), 1)

    def _key(self, r: int) -> str:
        return f"{self.prefix}/beat/{r}"

    def _left_key(self, r: int) -> str:
        return f"{self.prefix}/left/{r}"

    def beat(self) -> None:
        self.store.add(self._key(self.rank), 1)

    def leave(self) -> None:
        """Orderly exit between steps."""
        self.store.add(self._left_key(self.rank), 1)

    def _count(self, key: str) -> int:
        return int(self.store.add(key, 0))

    def wait_for_all(self, timeout_s: Optional[float] = None) -> None:
        """Start-up rendezvous: every rank must have beaten at least once."""
        deadline = time.monotonic() + (timeout_s if timeout_s is not None else self.timeout_s)
        while True:
            missing = [r for r in range(self.world) if self._count(self._key(r)) < 1]
            if not missing:
                return
            if time.monotonic() > deadline:
                raise RankLostError(missing, "start-up")
            time.sleep(0.01)

    def status(self) -> Dict[str, List[int]]:
        """``{"alive": [...], "left": [...], "lost": [...]}`` as seen now."""
        now = time.monotonic()
        alive, left, lost = [], [], []
        for r in range(self.world):
            if r == self.rank:
                alive.append(r)
                continue
            if self._count(self._left_key(r)) > 0:
                left.append(r)
                continue
            c = self._count(self._key(r))
            seen = self._last_seen.get(r)
            if seen is None or seen[0] != c:
                self._last_seen[r] = (c, now)
                alive.append(r)
            elif now - seen[1] > self.timeout_s:
                lost.append(r)
            else:
                alive.append(r)
        return {"alive": alive, "left": left, "lost": lost}

    def guard(self, what: str = "launch") -> List[int]:
        """Raises when a peer is lost; returns the ranks still in the group otherwise."""
        self.beat()
        st = self.status()
        if st["lost"]:
            raise RankLostError(st["lost"], what)
        return st["alive"]
