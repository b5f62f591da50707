"""Data-parallel serving scheduler: one worker per GPU, dynamic batching in front of them.

The reference scales a model by Triton instance groups (serving/src/fastdeploy_runtime.cc:475-556:
one ``ModelInstanceState`` per instance, each with its own runtime clone on its own stream) and by
thread + ``Clone()`` (tutorials/multi_thread). Here a :class:`Scheduler` owns N workers - each bound to
one device with its own model object (or ``Runtime`` clone) and its own CUDA stream - behind a native
queueing core (``csrc/cpu/scheduler.cc``): per-worker ticket queues, least-loaded dispatch, batches of up
to ``max_batch_size`` that wait at most ``max_queue_delay_us`` (the two knobs of Triton's
``dynamic_batching`` block), request deadlines, cancellation, and the counters behind ``/metrics``.
Worker threads block inside the native core without the interpreter lock, so one process can keep
every GPU of a box busy.

A batch function may return its results directly or a handle with ``result()`` (for instance
``PPYOLOE.predict_async``): then up to ``pipeline_depth`` batches stay in flight per worker, so the
next batch's host->device copy overlaps the current batch's compute.

A worker whose model raises marks the affected requests failed and keeps serving; a worker that dies
(its factory raised, or ``max_failures`` consecutive errors) is taken out of rotation and its queue is
handed to the living workers at once - which the CPU tests drive with fake devices.
"""
from __future__ import annotations

import collections
import ctypes
import threading
import time
from concurrent.futures import Future
from typing import Any, Callable, Deque, Dict, List, Optional, Sequence, Tuple

from .. import _native

_HIST_BOUNDS = [1, 2, 4, 8, 16, 32, 64, 128, 256, 512, 1024, float("inf")]
_I64 = ctypes.c_int64


def _core():
    lib = _native.cpu()
    if not getattr(lib, "_sched_ready", False):
        lib.fdb_sched_create.restype = ctypes.c_void_p
        lib.fdb_sched_create.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int]
        lib.fdb_sched_destroy.argtypes = [ctypes.c_void_p]
        lib.fdb_sched_submit.argtypes = [ctypes.c_void_p, ctypes.c_int, _I64, ctypes.c_int, ctypes.POINTER(_I64),
                                         ctypes.POINTER(ctypes.c_int)]
        lib.fdb_sched_next_batch.argtypes = [ctypes.c_void_p, ctypes.c_int, _I64, ctypes.POINTER(_I64), ctypes.c_int,
                                             ctypes.POINTER(_I64), ctypes.c_int, ctypes.POINTER(ctypes.c_int)]
        lib.fdb_sched_done.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, _I64]
        lib.fdb_sched_cancel.argtypes = [ctypes.c_void_p, _I64]
        lib.fdb_sched_mark_dead.argtypes = [ctypes.c_void_p, ctypes.c_int]
        lib.fdb_sched_take_orphans.argtypes = [ctypes.c_void_p, ctypes.POINTER(_I64), ctypes.c_int]
        lib.fdb_sched_alive.argtypes = [ctypes.c_void_p, ctypes.c_int]
        lib.fdb_sched_pending.argtypes = [ctypes.c_void_p, ctypes.c_int]
        lib.fdb_sched_close.argtypes = [ctypes.c_void_p]
        lib.fdb_sched_stats.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(_I64), ctypes.c_int]
        lib.fdb_cpu_last_error.restype = ctypes.c_char_p
        lib._sched_ready = True
    return lib


_FUTURE_LOCK = threading.Lock()


class RequestFuture:
    """The result handle of one request: the methods of ``concurrent.futures.Future`` that callers of a scheduler use
    (``result``, ``exception``, ``done``, ``cancel``, ``cancelled``, ``running``, ``add_done_callback``), without the
    condition variable that class allocates for every instance - a request that has finished before anybody waits for
    it (the common case of a pipelined client) never allocates a waitable object at all."""

    __slots__ = ("_state", "_value", "_error", "_event", "_callbacks")
    _PENDING, _RUNNING, _CANCELLED, _FINISHED = 0, 1, 2, 3

    def __init__(self):
        self._state = self._PENDING
        self._value = None
        self._error: Optional[BaseException] = None
        self._event: Optional[threading.Event] = None
        self._callbacks = None

    # ---- producer side
    def set_running_or_notify_cancel(self) -> bool:
        with _FUTURE_LOCK:
            if self._state == self._CANCELLED:
                return False
            self._state = self._RUNNING
            return True

    def _finish(self, value, error) -> None:
        with _FUTURE_LOCK:
            if self._state in (self._CANCELLED, self._FINISHED):
                return
            self._value, self._error, self._state = value, error, self._FINISHED
            ev, cbs, self._callbacks = self._event, self._callbacks, None
        if ev is not None:
            ev.set()
        for fn in cbs or ():
            try:
                fn(self)
            except Exception:       # a callback's failure is its own
                pass

    def set_result(self, value) -> None:
        self._finish(value, None)

    def set_exception(self, error: BaseException) -> None:
        self._finish(None, error)

    # ---- consumer side
    def cancel(self) -> bool:
        with _FUTURE_LOCK:
            if self._state in (self._RUNNING, self._FINISHED):
                return False
            self._state = self._CANCELLED
            ev, cbs, self._callbacks = self._event, self._callbacks, None
        if ev is not None:
            ev.set()
        for fn in cbs or ():
            try:
                fn(self)
            except Exception:
                pass
        return True

    def cancelled(self) -> bool:
        return self._state == self._CANCELLED

    def running(self) -> bool:
        return self._state == self._RUNNING

    def done(self) -> bool:
        return self._state in (self._CANCELLED, self._FINISHED)

    def _wait(self, timeout: Optional[float]) -> None:
        with _FUTURE_LOCK:
            if self._state in (self._CANCELLED, self._FINISHED):
                return
            if self._event is None:
                self._event = threading.Event()
            ev = self._event
        if not ev.wait(timeout):
            raise TimeoutError("the request has not finished in time")

    def result(self, timeout: Optional[float] = None):
        self._wait(timeout)
        if self._state == self._CANCELLED:
            from concurrent.futures import CancelledError
            raise CancelledError()
        if self._error is not None:
            raise self._error
        return self._value

    def exception(self, timeout: Optional[float] = None) -> Optional[BaseException]:
        self._wait(timeout)
        if self._state == self._CANCELLED:
            from concurrent.futures import CancelledError
            raise CancelledError()
        return self._error

    def add_done_callback(self, fn) -> None:
        with _FUTURE_LOCK:
            if self._state not in (self._CANCELLED, self._FINISHED):
                self._callbacks = (self._callbacks or []) + [fn]
                return
        fn(self)


class _Item:
    __slots__ = ("payload", "future")

    def __init__(self, payload: Any, future: "RequestFuture"):
        self.payload, self.future = payload, future


class WorkerStats:
    """Snapshot of one worker's counters (read from the native core)."""

    def __init__(self, raw: Sequence[int]):
        (self.requests, self.batches, self.failed, self.expired, self.cancelled, self.queue_wait_us, self.compute_us,
         self.batch_size_sum, self.queued, self.in_flight, alive) = [int(v) for v in raw[:11]]
        self.alive = bool(alive)
        self.batch_histogram = [int(v) for v in raw[11:11 + len(_HIST_BOUNDS)]]

    def as_dict(self) -> Dict[str, Any]:
        b = max(self.batches, 1)
        return {"requests": self.requests, "batches": self.batches, "failed": self.failed, "expired": self.expired,
                "cancelled": self.cancelled, "avg_batch_size": self.batch_size_sum / b,
                "avg_queue_wait_ms": 1e-3 * self.queue_wait_us / max(self.requests, 1),
                "avg_compute_ms": 1e-3 * self.compute_us / b, "queued": self.queued, "in_flight": self.in_flight,
                "batch_histogram": dict(zip(["le_%s" % ("inf" if x == float("inf") else int(x)) for x in _HIST_BOUNDS],
                                            self.batch_histogram))}


class Worker:
    """One device: pulls batches from the native core and runs ``batch_fn(model, [payload, ...])``, which returns
    ``[result, ...]`` or a handle whose ``result()`` does."""

    def __init__(self, sched: "Scheduler", index: int, model_factory: Callable[[int], Any]):
        self.sched, self.index = sched, index
        self.error: Optional[BaseException] = None
        self._consecutive_failures = 0
        self.stream = None
        self.device = None
        try:
            self.model = model_factory(index)
        except BaseException as e:      # the device is unusable: never enters rotation
            self.model, self.error = None, e
            sched._lib.fdb_sched_mark_dead(sched._h, index)
        self.thread = threading.Thread(target=self._loop, name=f"fdb-worker-{index}", daemon=True)
        if self.alive:
            self.thread.start()

    # ------------------------------------------------------------------ introspection
    @property
    def alive(self) -> bool:
        return bool(self.sched._lib.fdb_sched_alive(self.sched._h, self.index))

    def pending(self) -> int:
        return int(self.sched._lib.fdb_sched_pending(self.sched._h, self.index))

    @property
    def stats(self) -> WorkerStats:
        buf = (_I64 * 32)()
        self.sched._lib.fdb_sched_stats(self.sched._h, self.index, buf, 32)
        return WorkerStats(list(buf))

    # ------------------------------------------------------------------ the loop
    def _bind_device(self) -> None:
        """A worker owns its device and one stream on it for everything it launches."""
        rt = getattr(self.model, "runtime", None)
        if rt is not None and getattr(rt, "on_gpu", False):
            import torch
            self.device = rt.device
            torch.cuda.set_device(self.device)
            self.stream = torch.cuda.Stream(self.device)

    def _run(self, payloads: List[Any]):
        if self.stream is not None:
            import torch
            with torch.cuda.stream(self.stream):
                return self.sched.batch_fn(self.model, payloads)
        return self.sched.batch_fn(self.model, payloads)

    def _finish(self, items: List[_Item], handle: Any, t0: float) -> None:
        """Resolves one batch (waiting for an asynchronous handle) and reports it to the core."""
        lib, h = self.sched._lib, self.sched._h
        ok = True
        try:
            results = handle.result() if hasattr(handle, "result") and not isinstance(handle, (list, tuple)) else handle
            if len(results) != len(items):
                raise RuntimeError(f"batch function returned {len(results)} results for {len(items)} requests")
            for it, r in zip(items, results):
                it.future.set_result(r)
            self._consecutive_failures = 0
        except BaseException as e:
            ok = False
            for it in items:
                if not it.future.done():
                    it.future.set_exception(e)
            self._consecutive_failures += 1
            self.error = e
        lib.fdb_sched_done(h, self.index, len(items), 1 if ok else 0, int((time.perf_counter() - t0) * 1e6))
        if not ok and self._consecutive_failures >= self.sched.max_failures:
            self.sched._worker_died(self)

    def _loop(self) -> None:
        sched = self.sched
        lib, h = sched._lib, sched._h
        try:
            self._bind_device()
        except BaseException as e:
            self.error = e
            sched._worker_died(self)
            return
        cap = sched.max_batch_size
        out, exp = (_I64 * cap)(), (_I64 * 256)()
        n_exp = ctypes.c_int(0)
        in_flight: Deque[Tuple[List[_Item], Any, float]] = collections.deque()
        while True:
            if len(in_flight) >= sched.pipeline_depth:
                self._finish(*in_flight.popleft())
                if not self.alive:
                    break
                continue
            # with work in flight do not sleep on an empty queue: go and finish the oldest batch instead
            n = lib.fdb_sched_next_batch(h, self.index, 0 if in_flight else 200000, out, cap, exp, 256,
                                         ctypes.byref(n_exp))
            for k in range(n_exp.value):
                it = sched._take(exp[k])
                if it is not None and not it.future.done():
                    it.future.set_exception(TimeoutError("request deadline passed while queued"))
            if n < 0:
                break
            if n == 0:
                if in_flight:
                    self._finish(*in_flight.popleft())
                    if not self.alive:
                        break
                continue
            items = sched._take_many(out, n)
            live = [it for it in items if it.future.set_running_or_notify_cancel()]
            dropped = n - len(live)
            if dropped:
                lib.fdb_sched_done(h, self.index, dropped, 1, 0)
            if not live:
                continue
            t0 = time.perf_counter()
            try:
                handle = self._run([it.payload for it in live])
            except BaseException as e:
                handle = _Raised(e)
            if sched.pipeline_depth > 1 and hasattr(handle, "result") and not isinstance(handle, (list, tuple)):
                in_flight.append((live, handle, t0))
            else:
                self._finish(live, handle, t0)
                if not self.alive:
                    break
        while in_flight:
            self._finish(*in_flight.popleft())

    def stop(self) -> None:
        if self.thread.is_alive():
            self.thread.join(timeout=10)


class _Raised:
    """Stands in for the handle of a batch whose submission raised."""

    def __init__(self, exc: BaseException):
        self.exc = exc

    def result(self):
        raise self.exc


class Scheduler:
    def __init__(self, model_factory: Callable[[int], Any], batch_fn: Callable[[Any, List[Any]], Any],
                 num_workers: int = 1, max_batch_size: int = 8, max_queue_delay_us: int = 500, max_failures: int = 3,
                 pipeline_depth: int = 1):
        self._lib = _core()
        self._h = ctypes.c_void_p(self._lib.fdb_sched_create(num_workers, max_batch_size, max_queue_delay_us))
        if not self._h:
            raise ValueError(self._lib.fdb_cpu_last_error().decode())
        self.batch_fn, self.max_batch_size, self.max_failures = batch_fn, max_batch_size, max_failures
        self.pipeline_depth = max(1, pipeline_depth)
        self._items: Dict[int, _Item] = {}
        self._items_lock = threading.Lock()
        self._closed = False
        self.workers: List[Worker] = [Worker(self, i, model_factory) for i in range(num_workers)]
        if not any(w.alive for w in self.workers):
            errs = "; ".join(f"worker {w.index}: {w.error!r}" for w in self.workers)
            self.close()
            raise RuntimeError("no worker could be started: " + errs)

    # ------------------------------------------------------------------ tickets
    def _take(self, ticket: int) -> Optional[_Item]:
        with self._items_lock:
            return self._items.pop(int(ticket), None)

    def _take_many(self, tickets, n: int) -> List[_Item]:
        """The items of a whole batch under one acquisition of the lock (tickets whose item is gone are skipped)."""
        pop = self._items.pop
        with self._items_lock:
            found = [pop(tickets[k], None) for k in range(n)]
        return [it for it in found if it is not None]

    def _fail_orphans(self, why: str) -> None:
        buf = (_I64 * 256)()
        while True:
            n = self._lib.fdb_sched_take_orphans(self._h, buf, 256)
            for k in range(n):
                it = self._take(buf[k])
                if it is not None and not it.future.done():
                    it.future.set_exception(RuntimeError(why))
            if n < 256:
                break

    def _worker_died(self, worker: Worker) -> None:
        """Called on the dying worker's own thread: its queue moves to the living workers right away, and
        what cannot be placed any more fails now instead of waiting for ever."""
        self._lib.fdb_sched_mark_dead(self._h, worker.index)
        self._fail_orphans("all workers have failed")

    # ------------------------------------------------------------------ public API
    def alive_workers(self) -> List[Worker]:
        return [w for w in self.workers if w.alive]

    def submit_many(self, payloads: Sequence[Any], timeout: Optional[float] = None,
                    together: bool = False) -> List[RequestFuture]:
        """Enqueues the payloads in one call. ``timeout`` (seconds) is a deadline for leaving the queue: a request
        still waiting when it passes fails with ``TimeoutError`` and is never run. ``together`` sends the whole
        burst to one worker (the least loaded one), keeping its requests adjacent in the executed batches."""
        n = len(payloads)
        futs = [RequestFuture() for _ in range(n)]
        if n == 0:
            return futs
        tickets = (_I64 * n)()
        # Tickets are registered before they can be handed out: the id sequence is only known after the call,
        # so the items are parked under a lock that the workers' lookups also take.
        with self._items_lock:
            if self._closed:
                raise RuntimeError("scheduler is closed")
            done = self._lib.fdb_sched_submit(self._h, n, int((timeout or 0) * 1e6), 1 if together else 0, tickets,
                                              None)
            for k in range(done):
                self._items[int(tickets[k])] = _Item(payloads[k], futs[k])
        if done < n:
            msg = self._lib.fdb_cpu_last_error().decode() or "all workers have failed"
            if done == 0:
                raise RuntimeError(msg)
            for f in futs[done:]:
                f.set_exception(RuntimeError(msg))
        return futs

    def submit(self, payload: Any, timeout: Optional[float] = None) -> RequestFuture:
        return self.submit_many([payload], timeout)[0]

    def infer(self, payload: Any, timeout: Optional[float] = None) -> Any:
        return self.submit(payload).result(timeout)

    def map(self, payloads: Sequence[Any], timeout: Optional[float] = None) -> List[Any]:
        futs = self.submit_many(list(payloads))
        return [f.result(timeout) for f in futs]

    def stats(self) -> dict:
        return {"workers": [dict(index=w.index, alive=w.alive, **w.stats.as_dict()) for w in self.workers]}

    def metrics_text(self, prefix: str = "fdb_scheduler") -> str:
        """Prometheus exposition text of the per-worker counters and the batch-size histogram."""
        lines = []
        snaps = [(w.index, w.stats) for w in self.workers]

        def metric(name, kind, help_, rows):
            lines.append(f"# HELP {prefix}_{name} {help_}")
            lines.append(f"# TYPE {prefix}_{name} {kind}")
            lines.extend(rows)
        metric("requests_total", "counter", "requests finished, per worker",
               [f'{prefix}_requests_total{{worker="{i}"}} {s.requests}' for i, s in snaps])
        metric("failed_total", "counter", "requests whose batch raised",
               [f'{prefix}_failed_total{{worker="{i}"}} {s.failed}' for i, s in snaps])
        metric("expired_total", "counter", "requests dropped at their deadline",
               [f'{prefix}_expired_total{{worker="{i}"}} {s.expired}' for i, s in snaps])
        metric("queue_depth", "gauge", "requests waiting for a batch",
               [f'{prefix}_queue_depth{{worker="{i}"}} {s.queued}' for i, s in snaps])
        metric("in_flight", "gauge", "requests handed to the device and not finished",
               [f'{prefix}_in_flight{{worker="{i}"}} {s.in_flight}' for i, s in snaps])
        metric("worker_alive", "gauge", "1 while the worker is in rotation",
               [f'{prefix}_worker_alive{{worker="{i}"}} {int(s.alive)}' for i, s in snaps])
        metric("queue_wait_seconds_total", "counter", "time requests spent queued",
               [f'{prefix}_queue_wait_seconds_total{{worker="{i}"}} {s.queue_wait_us * 1e-6:.6f}' for i, s in snaps])
        metric("compute_seconds_total", "counter", "time batches spent on the device (submission to results)",
               [f'{prefix}_compute_seconds_total{{worker="{i}"}} {s.compute_us * 1e-6:.6f}' for i, s in snaps])
        rows = []
        for i, s in snaps:
            cum = 0
            for bound, cnt in zip(_HIST_BOUNDS, s.batch_histogram):
                cum += cnt
                le = "+Inf" if bound == float("inf") else str(int(bound))
                rows.append(f'{prefix}_batch_size_bucket{{worker="{i}",le="{le}"}} {cum}')
            rows.append(f'{prefix}_batch_size_sum{{worker="{i}"}} {s.batch_size_sum}')
            rows.append(f'{prefix}_batch_size_count{{worker="{i}"}} {s.batches}')
        metric("batch_size", "histogram", "requests per executed batch", rows)
        return "\n".join(lines) + "\n"

    def close(self) -> None:
        with self._items_lock:
            if self._closed:
                return
            self._closed = True
        self._lib.fdb_sched_close(self._h)
        for w in getattr(self, "workers", []):
            w.stop()
        self._fail_orphans("scheduler is closed")
        with self._items_lock:
            left = list(self._items.values())
            self._items.clear()
        for it in left:                      # nothing may stay pending after close()
            if not it.future.done():
                it.future.set_exception(RuntimeError("scheduler is closed"))

    def __del__(self):
        try:
            self.close()
            if self._h:
                self._lib.fdb_sched_destroy(self._h)
                self._h = None
        except Exception:
            pass
