"""Process set-up, clock sampling and block timing shared by the benchmark workloads."""
from __future__ import annotations

import os
import subprocess
import threading
import time
from typing import Callable, Dict, List, Optional


class ClockSampler:
    """Samples SM clocks and throttle reasons every 200 ms while the timed regions run. NVML is called in
    process (three light queries per sample); spawning ``nvidia-smi -lms`` instead was seen to stall the
    GPUs of a multi-GPU box for tens of milliseconds per poll, which lands inside short timed regions.
    Falls back to ``nvidia-smi`` when the NVML binding is missing."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.rows = []          # (sm_mhz, max_mhz, set of reason names)
        self.proc = None
        self.thread = None
        self._stop = threading.Event()
        self._nvml = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(self.gpu_index)
            self._max = float(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._poll_nvml, daemon=True)
            self.thread.start()
            return
        except Exception:
            self._nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu_index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read_smi, daemon=True)
        self.thread.start()

    def ready(self) -> bool:
        return bool(self.rows) or (self._nvml is None and self.proc is None)

    def wait_ready(self, limit_s: float = 10.0) -> None:
        t0 = time.time()
        while not self.ready() and time.time() - t0 < limit_s:
            time.sleep(0.05)

    def _poll_nvml(self):
        n = self._nvml
        names = (("hw_slowdown", getattr(n, "nvmlClocksEventReasonHwSlowdown", 0x8)),
                 ("hw_thermal_slowdown", getattr(n, "nvmlClocksEventReasonHwThermalSlowdown", 0x40)),
                 ("sw_thermal_slowdown", getattr(n, "nvmlClocksEventReasonSwThermalSlowdown", 0x20)),
                 ("sw_power_cap", getattr(n, "nvmlClocksEventReasonSwPowerCap", 0x4)))
        get_reasons = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            getattr(n, "nvmlDeviceGetCurrentClocksThrottleReasons", None)
        while not self._stop.is_set():
            try:
                sm = float(n.nvmlDeviceGetClockInfo(self._handle, n.NVML_CLOCK_SM))
                mask = int(get_reasons(self._handle)) if get_reasons else 0
                self.rows.append((sm, self._max, {k for k, bit in names if mask & bit}))
            except Exception:
                pass
            self._stop.wait(0.2)

    def _read_smi(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 8:
                try:
                    reasons = {k for k, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                                  "sw_power_cap"), parts[4:8]) if v.lower().startswith("active")}
                    self.rows.append((float(parts[1]), float(parts[2]), reasons))
                except ValueError:
                    continue

    def stop(self):
        self._stop.set()
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()
        if self.thread is not None:
            self.thread.join(timeout=2)
        sm = sorted(r[0] for r in self.rows)
        mx = max((r[1] for r in self.rows), default=0.0)
        reasons = set().union(*(r[2] for r in self.rows)) if self.rows else set()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm), "source": "nvml" if self._nvml is not None else "nvidia-smi"}


def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except (ValueError, IndexError):
            pass
    return local_rank


def _parse_cpulist(text: str) -> List[int]:
    cpus: List[int] = []
    for part in text.strip().split(","):
        if not part:
            continue
        if "-" in part:
            a, b = part.split("-")
            cpus.extend(range(int(a), int(b) + 1))
        else:
            cpus.append(int(part))
    return cpus


def bind_to_gpu_cpus(local_rank: int, local_world: int) -> Optional[Dict]:
    """Pins this process to CPU cores next to its GPU before any pinned host memory is allocated, so that the
    staging buffers are first touched on the GPU's own NUMA node and the ranks of one box do not migrate over
    each other's cores. The GPU's ``local_cpulist`` comes from sysfs through its PCI address; when several ranks
    share that list (all GPUs under one NUMA node) it is dealt out between them. Returns what was done, or None
    when the topology could not be read (then nothing is changed)."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(physical_gpu_index(local_rank))
        bus = pynvml.nvmlDeviceGetPciInfo(h).busId
        bus = bus.decode() if isinstance(bus, bytes) else bus
        dom, rest = bus.split(":", 1)
        path = f"/sys/bus/pci/devices/{dom[-4:].lower()}:{rest.lower()}"
        with open(path + "/local_cpulist") as f:
            cpus = _parse_cpulist(f.read())
        node = -1
        try:
            with open(path + "/numa_node") as f:
                node = int(f.read().strip())
        except OSError:
            pass
        allowed = sorted(set(cpus) & set(os.sched_getaffinity(0)))
        if not allowed:
            return None
        mine = allowed
        if local_world > 1 and len(allowed) >= 2 * local_world:
            per = len(allowed) // local_world
            mine = allowed[local_rank * per:(local_rank + 1) * per]
        os.sched_setaffinity(0, mine)
        return {"numa_node": node, "cpus": f"{mine[0]}-{mine[-1]}", "n_cpus": len(mine)}
    except Exception:
        return None


class Context:
    """Ranks, device and collectives of one benchmark process."""

    def __init__(self, gpus: int):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        if self.world == 1 and gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
        self.affinity = bind_to_gpu_cpus(self.local_rank, int(os.environ.get("LOCAL_WORLD_SIZE", self.world)))
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        if self.world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=self.dev)

    def barrier(self) -> None:
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize(self.dev)

    def max_over_ranks(self, values: List[float]) -> List[float]:
        if self.world == 1:
            return list(values)
        t = self.torch.tensor(values, device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t]

    def time_blocks(self, run_steps: Callable[[int], object], steps: int, repeats: int) -> List[float]:
        """``repeats`` timed blocks of exactly ``steps`` steps each, every block bracketed by a barrier and a
        device synchronise on both sides and timed with CUDA events on the launching stream. Returns the
        per-block milliseconds as the maximum over ranks."""
        torch = self.torch
        out = []
        for _ in range(repeats):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.barrier()
            e0.record()
            run_steps(steps)
            e1.record()
            self.barrier()
            out.append(e0.elapsed_time(e1))
        return self.max_over_ranks(out)

    def finish(self) -> None:
        if self.world > 1:
            self.dist.destroy_process_group()


def median(xs: List[float]) -> float:
    s = sorted(xs)
    return s[len(s) // 2] if len(s) % 2 else 0.5 * (s[len(s) // 2 - 1] + s[len(s) // 2])


def spread(xs: List[float]) -> Dict[str, float]:
    return {"min": round(min(xs), 3), "median": round(median(xs), 3), "max": round(max(xs), 3), "blocks": len(xs)}
