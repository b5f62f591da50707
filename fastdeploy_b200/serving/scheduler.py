"""Data-parallel serving scheduler: one worker per GPU, dynamic batching in front of them.

The reference scales a model by Triton instance groups (serving/src/fastdeploy_runtime.cc:162-271:
one ``ModelInstanceState`` per instance, each with its own runtime clone) and by thread + ``Clone()``
(examples/runtime/python/multi_thread). Here a :class:`Scheduler` owns N workers - each bound to one
device with its own model object (or ``Runtime`` clone) - and a :class:`DynamicBatcher` that groups
single requests into batches of up to ``max_batch_size`` waiting at most ``max_queue_delay_us``, the two
knobs of Triton's ``dynamic_batching`` block. Requests go to the worker with the fewest queued items.

Workers are plain threads: the model call releases the GIL while the GPU works, and every worker has
its own CUDA stream through its model's runtime. A worker whose model raises marks the affected
requests failed and keeps serving; a worker that dies (its factory raised, or ``max_failures``
consecutive errors) is taken out of rotation and its queue is redistributed - which the CPU tests
drive with fake devices.
"""
from __future__ import annotations

import queue
import threading
import time
from concurrent.futures import Future
from dataclasses import dataclass, field
from typing import Any, Callable, List, Optional, Sequence


@dataclass
class SchedulerStats:
    requests: int = 0
    batches: int = 0
    failed: int = 0
    batch_size_sum: int = 0
    queue_wait_s: float = 0.0
    compute_s: float = 0.0

    def as_dict(self):
        b = max(self.batches, 1)
        return {"requests": self.requests, "batches": self.batches, "failed": self.failed,
                "avg_batch_size": self.batch_size_sum / b, "avg_queue_wait_ms": 1e3 * self.queue_wait_s / max(self.requests, 1),
                "avg_compute_ms": 1e3 * self.compute_s / b}


@dataclass
class _Item:
    payload: Any
    future: Future
    t_enqueue: float = field(default_factory=time.perf_counter)


class Worker:
    """One device: pulls batches from its queue and runs ``batch_fn(model, [payload, ...]) -> [result, ...]``."""

    def __init__(self, index: int, model_factory: Callable[[int], Any], batch_fn: Callable[[Any, List[Any]], Sequence[Any]],
                 max_batch_size: int, max_queue_delay_us: int, max_failures: int = 3,
                 on_death: Optional[Callable[["Worker"], None]] = None):
        self.index = index
        self.on_death = on_death
        self.q: "queue.Queue[Optional[_Item]]" = queue.Queue()
        self.max_batch_size, self.delay_s = max_batch_size, max_queue_delay_us / 1e6
        self.batch_fn, self.max_failures = batch_fn, max_failures
        self.stats = SchedulerStats()
        self.alive = True
        self.error: Optional[BaseException] = None
        self._consecutive_failures = 0
        try:
            self.model = model_factory(index)
        except BaseException as e:      # the device is unusable: never enters rotation
            self.model, self.alive, self.error = None, False, e
        self.thread = threading.Thread(target=self._loop, name=f"fdb-worker-{index}", daemon=True)
        if self.alive:
            self.thread.start()

    def pending(self) -> int:
        return self.q.qsize()

    def _collect(self) -> Optional[List[_Item]]:
        first = self.q.get()
        if first is None:
            return None
        batch = [first]
        deadline = time.perf_counter() + self.delay_s
        while len(batch) < self.max_batch_size:
            remaining = deadline - time.perf_counter()
            try:
                nxt = self.q.get(timeout=max(remaining, 0)) if remaining > 0 else self.q.get_nowait()
            except queue.Empty:
                break
            if nxt is None:
                self.q.put(None)
                break
            batch.append(nxt)
        return batch

    def _loop(self) -> None:
        while True:
            batch = self._collect()
            if batch is None:
                return
            t0 = time.perf_counter()
            for it in batch:
                self.stats.queue_wait_s += t0 - it.t_enqueue
            try:
                results = self.batch_fn(self.model, [it.payload for it in batch])
                if len(results) != len(batch):
                    raise RuntimeError(f"batch function returned {len(results)} results for {len(batch)} requests")
                for it, r in zip(batch, results):
                    it.future.set_result(r)
                self._consecutive_failures = 0
            except BaseException as e:
                self.stats.failed += len(batch)
                for it in batch:
                    if not it.future.done():
                        it.future.set_exception(e)
                self._consecutive_failures += 1
                if self._consecutive_failures >= self.max_failures:
                    self.alive, self.error = False, e
                    # whatever is still queued here must not wait for a later submit(): hand it back now
                    if self.on_death is not None:
                        self.on_death(self)
                    return
            finally:
                self.stats.compute_s += time.perf_counter() - t0
                self.stats.requests += len(batch)
                self.stats.batches += 1
                self.stats.batch_size_sum += len(batch)

    def stop(self) -> None:
        if self.thread.is_alive():
            self.q.put(None)
            self.thread.join(timeout=5)


class Scheduler:
    def __init__(self, model_factory: Callable[[int], Any], batch_fn: Callable[[Any, List[Any]], Sequence[Any]],
                 num_workers: int = 1, max_batch_size: int = 8, max_queue_delay_us: int = 500, max_failures: int = 3):
        self._lock = threading.RLock()
        self.workers: List[Worker] = []
        self.workers = [Worker(i, model_factory, batch_fn, max_batch_size, max_queue_delay_us, max_failures,
                               on_death=self._worker_died) for i in range(num_workers)]
        if not any(w.alive for w in self.workers):
            errs = "; ".join(f"worker {w.index}: {w.error!r}" for w in self.workers)
            raise RuntimeError("no worker could be started: " + errs)
        self._closed = False
        self._rr = 0

    def alive_workers(self) -> List[Worker]:
        return [w for w in self.workers if w.alive]

    def submit(self, payload: Any) -> Future:
        fut: Future = Future()
        with self._lock:
            if self._closed:
                raise RuntimeError("scheduler is closed")
            self._reap()
            alive = self.alive_workers()
            if not alive:
                raise RuntimeError("all workers have failed")
            self._rr += 1      # ties go round the workers instead of always to the first
            n = len(self.workers)
            w = min(alive, key=lambda x: (x.pending(), (x.index - self._rr) % n))
            w.q.put(_Item(payload, fut))
        return fut

    def _worker_died(self, worker: Worker) -> None:
        """Called on the dying worker's own thread: its queued items move to the living workers (or fail when
        none is left) right away. submit() may have picked this worker a moment before it died; such an item
        lands in the dead queue afterwards and is caught by the reap at the next submit() or at close()."""
        with self._lock:
            self._reap()

    def _reap(self) -> None:
        """Moves the queued items of dead workers to the living ones."""
        dead = [w for w in self.workers if not w.alive and not w.q.empty()]
        alive = self.alive_workers()
        for w in dead:
            while True:
                try:
                    it = w.q.get_nowait()
                except queue.Empty:
                    break
                if it is None:
                    continue
                if alive:
                    min(alive, key=lambda x: x.pending()).q.put(it)
                else:
                    it.future.set_exception(RuntimeError("all workers have failed"))

    def infer(self, payload: Any, timeout: Optional[float] = None) -> Any:
        return self.submit(payload).result(timeout)

    def map(self, payloads: Sequence[Any], timeout: Optional[float] = None) -> List[Any]:
        futs = [self.submit(p) for p in payloads]
        return [f.result(timeout) for f in futs]

    def stats(self) -> dict:
        return {"workers": [dict(index=w.index, alive=w.alive, **w.stats.as_dict()) for w in self.workers]}

    def close(self) -> None:
        with self._lock:
            self._closed = True
        for w in self.workers:
            w.stop()
        with self._lock:
            for w in self.workers:          # nothing may stay pending after close()
                while True:
                    try:
                        it = w.q.get_nowait()
                    except queue.Empty:
                        break
                    if it is not None and not it.future.done():
                        it.future.set_exception(RuntimeError("scheduler is closed"))
