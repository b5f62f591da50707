"""``TimeCounter`` (fastdeploy/utils/perf.h:22-48): a start / end wall-clock interval in seconds, on the native
steady clock. ``with TimeCounter() as t: ...; t.duration()`` works too."""
from __future__ import annotations

from ..core.scalar import _lib
from . import log


class TimeCounter:
    def __init__(self):
        self._h = _lib().fdb_timer_create()

    def start(self) -> None:
        _lib().fdb_timer_start(self._h)

    def end(self) -> None:
        _lib().fdb_timer_end(self._h)

    def duration(self) -> float:
        return float(_lib().fdb_timer_duration(self._h))

    def print_info(self, prefix: str = "TimeCounter: ", print_out: bool = True) -> None:
        if print_out:
            log.info(f"{prefix} duration = {self.duration()}s.")

    # reference spelling
    Start, End, Duration, PrintInfo = start, end, duration, print_info

    def __enter__(self):
        self.start()
        return self

    def __exit__(self, *exc):
        self.end()
        return False

    def __del__(self):
        try:
            _lib().fdb_timer_destroy(self._h)
        except Exception:
            pass
