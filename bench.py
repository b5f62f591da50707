"""Benchmarks of the five headline configurations. The headline (no ``--config``) is end-to-end images/s of
PP-YOLOE+-L (fp16, 640x640 from 1080x1920 uint8 frames, batch 32 per GPU, multiclass NMS score 0.01 / IoU 0.6 /
keep_top_k 100), data-parallel over N GPUs:

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --config ernie | ocr | vit_tp  ...        (same flags, same JSON schema)
    python bench.py --config ppyoloe_library                  (context: the same network on PyTorch / cuDNN fp16)
    python bench.py --config resnet50_cpu                     (ResNet-50 batch-1 latency through the CPU path; no GPU)

``value``   : device-timed (CUDA events, max over ranks) rate of the on-device step, inputs resident on the GPU.
``e2e``     : the same metric through the public API, each step copying its inputs from pinned host memory and
              reading its results back.
Every number is the median of ``--repeats`` timed blocks of exactly ``--steps`` steps. Synthetic data,
random-initialised weights (there is no network access here).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

REF_UNAVAILABLE = ("refused by a safety check: building the reference (its python setup.py build, which downloads "
                   "ONNX Runtime / Paddle Inference / OpenCV binaries from bj.bcebos.com) was denied; a plain pip "
                   "install of the reference tree fails before that (no setup.py at its root, python/ needs the "
                   "CMake build first)")

CONFIGS = ("ppyoloe", "ernie", "ocr", "vit_tp", "ppyoloe_library", "resnet50_cpu")


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repeats", type=int, default=5, help="timed blocks of --steps steps; the median is reported")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="ppyoloe", choices=CONFIGS)
    ap.add_argument("--batch", type=int, default=0, help="per-GPU batch (0 = the configuration's own)")
    ap.add_argument("--variant", default="l")
    ap.add_argument("--model-dir", default="")
    ap.add_argument("--latency-iters", type=int, default=50)
    ap.add_argument("--skip-latency", action="store_true")
    ap.add_argument("--no-scheduler-mode", action="store_true",
                    help="ppyoloe: skip the extra run that drives all N GPUs from ONE process through serving.Scheduler")
    ap.add_argument("--dtype", default="", help="vit_tp: bf16 | fp8")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REF_UNAVAILABLE}))
        return 0

    if args.config == "resnet50_cpu":          # host only: no device context, no process group
        from fastdeploy_b200.benchmarks.resnet50_cpu import run_cpu
        print(json.dumps(run_cpu(args)))
        return 0

    import importlib
    from fastdeploy_b200.benchmarks.common import Context
    ctx = Context(args.gpus)
    mod = importlib.import_module(f"fastdeploy_b200.benchmarks.{args.config}")
    out = mod.run(ctx, args)
    if ctx.rank == 0:
        print(json.dumps(out))
    ctx.finish()
    return 0


if __name__ == "__main__":
    sys.exit(main())
