"""Headline benchmark: end-to-end images/s of PP-YOLOE+-L (fp16, 640x640 from 1080x1920 uint8
frames, batch 32 per GPU, multiclass NMS score 0.01 / IoU 0.6 / keep_top_k 100), data-parallel over N GPUs.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

``value``   : device-timed (CUDA events, max over ranks) images/s of the on-device step: raw uint8 frames
              already on the GPU -> fused pre-processing -> network -> DFL decode -> NMS.
``e2e``     : the same metric through the public API (``fd.vision.detection.PPYOLOE.predict_async``), each
              step copying its frames from pinned host memory and reading its detections back.
Synthetic data, random-initialised weights (no network access here).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PUBLISHED_IMG_S = 64.9     # best published end-to-end PP-YOLOE-L number of the reference: 15.42 ms on a T4
REF_UNAVAILABLE = ("refused by a safety check: building the reference (python setup.py build, which downloads "
                   "ONNX Runtime / Paddle Inference / OpenCV from bj.bcebos.com) was denied; pip install of "
                   "/root/reference fails before that (no setup.py at the root, python/ needs the CMake build)")


class ClockSampler:
    """Polls nvidia-smi for SM clocks and throttle reasons while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu_index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 8:
                self.rows.append(parts)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()
        sm, mx, reasons = [], 0.0, set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx = max(mx, float(r[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except (ValueError, IndexError):
            pass
    return local_rank


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=32, help="images per GPU per step")
    ap.add_argument("--variant", default="l")
    ap.add_argument("--model-dir", default="")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REF_UNAVAILABLE}))
        return 0

    import numpy as np
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    import fastdeploy_b200 as fd
    from fastdeploy_b200.models.ppyoloe import write_ppyoloe
    fd.set_logger(False, True)

    model_dir = args.model_dir or os.path.join(tempfile.gettempdir(), f"fdb200_ppyoloe_{args.variant}_640")
    if rank == 0 and not os.path.exists(os.path.join(model_dir, "model.pdiparams")):
        write_ppyoloe(model_dir, args.variant, image=640, num_classes=80, seed=0, score_threshold=0.01,
                      nms_threshold=0.6, nms_top_k=1000, keep_top_k=100)
    barrier()

    opt = fd.RuntimeOption()
    opt.use_gpu(local_rank)
    opt.enable_trt_fp16()
    model = fd.vision.detection.PPYOLOE(os.path.join(model_dir, "model.pdmodel"),
                                        os.path.join(model_dir, "model.pdiparams"),
                                        os.path.join(model_dir, "infer_cfg.yml"), runtime_option=opt)
    B = args.batch
    H, W = 1080, 1920
    rng = np.random.default_rng(1234 + rank)
    # two alternating sets of pinned host frames, uniform in [0, 255]
    host_sets = []
    for s in range(2):
        t = torch.from_numpy(rng.integers(0, 256, (B, H, W, 3), dtype=np.uint8)).pin_memory()
        host_sets.append([t[i] for i in range(B)])
    dev_sets = [[f.to(dev) for f in frames] for frames in host_sets]

    # The clock sampler starts before the warm-up: the first nvidia-smi query initialises NVML for every GPU
    # of the box and holds driver locks while it does, which must not land inside a timed region.
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    # ---------------- device-timed step (inputs resident on the GPU)
    def run_steps(sets, n):
        """n pipelined steps (the next batch is queued before the previous one is read back)."""
        pend, dets = None, 0
        for i in range(n):
            nxt = model.predict_async(sets[i & 1])
            if pend is not None:
                dets += sum(len(r.boxes) for r in pend.result())
            pend = nxt
        dets += sum(len(r.boxes) for r in pend.result())
        return dets

    t_wait = time.time()
    while not sampler.rows and sampler.proc is not None and time.time() - t_wait < 10.0:
        time.sleep(0.05)                          # NVML is initialised once the first sample is in
    run_steps(dev_sets, max(args.warmup, 3))      # warm-up in the same pipelined pattern as the timed loop
    barrier()                                     # no idle gap from here on: an idle GPU drops its clocks
    sampler.rows.clear()
    launches0 = model.runtime.gpu_launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    run_steps(dev_sets, args.steps)
    e1.record()
    barrier()
    ms_dev = e0.elapsed_time(e1)
    launches = model.runtime.gpu_launches - launches0

    # ---------------- end to end through the public API (pinned host frames in, detections out)
    run_steps(host_sets, max(args.warmup, 3))
    barrier()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    n_det = run_steps(host_sets, args.steps)
    e3.record()
    barrier()
    ms_e2e = e2.elapsed_time(e3)
    clocks = sampler.stop()
    h2d, d2h = model.h2d_bytes_last, model.d2h_bytes_last

    if world > 1:
        t = torch.tensor([ms_dev, ms_e2e], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_dev, ms_e2e = float(t[0]), float(t[1])
    if rank == 0:
        total_imgs = B * world * args.steps
        value = total_imgs / (ms_dev / 1e3)
        e2e = total_imgs / (ms_e2e / 1e3)
        out = {
            "metric": "end-to-end images/sec PP-YOLOE+-L (device-timed)", "value": round(value, 1), "unit": "images/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": round(ms_dev / args.steps, 3), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": round(value / PUBLISHED_IMG_S, 2), "dtype": "fp16", "data": "synthetic",
            "config": {"model": f"PP-YOLOE+-{args.variant.upper()} 640x640 from 1080x1920 uint8, NMS 0.01/0.6/100, "
                                "random-init weights", "global_batch": B * world, "seq_len": None,
                       "parallelism": f"dp{world}",
                       "l2_policy": "inputs larger than L2: 199 MB of raw frames per step, two alternating sets",
                       "baseline_ref": "reference's best published end-to-end PP-YOLOE-L: 15.42 ms on one T4 (TensorRT INT8)"},
            "e2e": {"value": round(e2e, 1), "unit": "images/s", "h2d_bytes_per_step": int(h2d),
                    "d2h_bytes_per_step": int(d2h), "ms_per_step": round(ms_e2e / args.steps, 3),
                    "detections_read": int(n_det)},
            "gpu_launches": int(launches), "clocks": clocks, "impl": "ours",
        }
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
