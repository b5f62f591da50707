"""Benchmark utilities: the resource monitor and result helpers of benchmark/cpp/{utils,option}.h and
benchmark/python/benchmark_*.py (CPU RSS through ``/proc``, GPU memory / utilisation through
``nvidia-smi`` polled on a thread; tensor diff statistics; runtime vs end-to-end timing loops with the
reference's ``warmup`` / ``repeat`` meaning), plus the profiling loop of
fastdeploy/benchmark/utils.h:28-70 (``RUNTIME_PROFILE_LOOP``)."""
from __future__ import annotations

import os
import subprocess
import threading
import time
from typing import Any, Callable, Dict, List, Optional, Sequence

import numpy as np


class ResourceUsageMonitor:
    def __init__(self, sampling_interval_ms: int = 50, gpu_id: int = 0):
        self.interval = sampling_interval_ms / 1e3
        self.gpu_id = gpu_id
        self.max_cpu_mem_mb = 0.0
        self.max_gpu_mem_mb = 0.0
        self.max_gpu_util = 0.0
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    @staticmethod
    def _rss_mb() -> float:
        try:
            with open("/proc/self/status") as f:
                for line in f:
                    if line.startswith("VmRSS:"):
                        return float(line.split()[1]) / 1024.0
        except OSError:
            pass
        return 0.0

    def _gpu(self):
        try:
            out = subprocess.run(["nvidia-smi", "--query-gpu=memory.used,utilization.gpu", "--format=csv,noheader,nounits",
                                  "-i", str(self.gpu_id)], capture_output=True, text=True, timeout=2).stdout.strip()
            mem, util = (float(v) for v in out.split(","))
            return mem, util
        except Exception:
            return 0.0, 0.0

    def _loop(self):
        while not self._stop.is_set():
            self.max_cpu_mem_mb = max(self.max_cpu_mem_mb, self._rss_mb())
            mem, util = self._gpu()
            self.max_gpu_mem_mb = max(self.max_gpu_mem_mb, mem)
            self.max_gpu_util = max(self.max_gpu_util, util)
            self._stop.wait(self.interval)

    def start(self):
        self._stop.clear()
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=3)

    def get_max_cpu_mem(self) -> float:
        return self.max_cpu_mem_mb

    def get_max_gpu_mem(self) -> float:
        return self.max_gpu_mem_mb

    def get_max_gpu_util(self) -> float:
        return self.max_gpu_util


def tensor_diff(a: np.ndarray, b: np.ndarray) -> Dict[str, float]:
    """Max / min / mean of the element differences (benchmark/cpp/utils: ``CalculateDiffStatis``)."""
    d = np.asarray(a, np.float64) - np.asarray(b, np.float64)
    return {"max": float(d.max()) if d.size else 0.0, "min": float(d.min()) if d.size else 0.0,
            "mean": float(d.mean()) if d.size else 0.0}


def profile_loop(fn: Callable[[], Any], warmup: int = 200, repeat: int = 1000, sync: Optional[Callable[[], None]] = None) -> float:
    """Average seconds per call over ``repeat`` calls after ``warmup`` (the profiling macros re-run the
    wrapped region exactly like this when ``enable_profile`` is set)."""
    for _ in range(warmup):
        fn()
    if sync:
        sync()
    t0 = time.perf_counter()
    for _ in range(repeat):
        fn()
    if sync:
        sync()
    return (time.perf_counter() - t0) / max(repeat, 1)


def benchmark_model(model, images: Sequence[np.ndarray], warmup: int = 20, repeat: int = 100, batch: bool = False,
                    collect_memory: bool = False, gpu_id: int = 0) -> Dict[str, float]:
    """End-to-end latency of ``predict`` / ``batch_predict`` plus the runtime-only share when the model
    records it (``enable_record_time_of_runtime``)."""
    mon = ResourceUsageMonitor(gpu_id=gpu_id) if collect_memory else None
    if mon:
        mon.start()
    call = (lambda: model.batch_predict(images)) if batch else (lambda: [model.predict(im) for im in images])
    for _ in range(warmup):
        call()
    if hasattr(model, "enable_record_time_of_runtime"):
        model.enable_record_time_of_runtime()
    lat = []
    for _ in range(repeat):
        t0 = time.perf_counter()
        call()
        lat.append(time.perf_counter() - t0)
    out = {"e2e_ms_mean": 1e3 * float(np.mean(lat)), "e2e_ms_p50": 1e3 * float(np.percentile(lat, 50)),
           "e2e_ms_p99": 1e3 * float(np.percentile(lat, 99)), "images_per_s": len(images) / float(np.mean(lat))}
    times = getattr(model, "_time_of_runtime", None)
    if times:
        out["runtime_ms_mean"] = 1e3 * float(np.mean(times[len(times) // 5:]))
    if mon:
        mon.stop()
        out.update(cpu_rss_mb=mon.get_max_cpu_mem(), gpu_mem_mb=mon.get_max_gpu_mem(), gpu_util=mon.get_max_gpu_util())
    return out
