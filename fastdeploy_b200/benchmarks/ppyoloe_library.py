"""Library baseline for the PP-YOLOE+-L network: the same imported graph (no NMS stage) run by PyTorch operators on the
GPU in fp16, channels-last, with cuDNN choosing its own algorithms - what a user gets from the framework's stock
kernels. Context for the native plan's network time, reported under its own name; it is not the reference arm.
"""
from __future__ import annotations

import os
import tempfile

from .common import ClockSampler, Context, median, physical_gpu_index, spread


def run(ctx: Context, args) -> dict:
    import numpy as np
    torch = ctx.torch
    import fastdeploy_b200 as fd
    from fastdeploy_b200.importer.paddle_import import load_paddle
    from fastdeploy_b200.ir import passes
    from fastdeploy_b200.ir.convert_fp16 import convert_fp32_to_fp16
    from fastdeploy_b200.ir.interp import Interpreter
    from fastdeploy_b200.models.ppyoloe import write_ppyoloe
    fd.set_logger(False, True)
    dev = ctx.dev
    torch.backends.cudnn.benchmark = True
    model_dir = os.path.join(tempfile.gettempdir(), f"fdb200_ppyoloe_{args.variant}_640_nonms")
    if ctx.rank == 0 and not os.path.exists(os.path.join(model_dir, "model.pdiparams")):
        write_ppyoloe(model_dir, args.variant, image=640, num_classes=80, seed=0, with_nms=False)
    ctx.barrier()
    with open(os.path.join(model_dir, "model.pdmodel"), "rb") as f:
        m = f.read()
    with open(os.path.join(model_dir, "model.pdiparams"), "rb") as f:
        p = f.read()
    B = args.batch or 32
    shapes = {"image": [B, 3, 640, 640], "scale_factor": [B, 2]}
    g = passes.optimize(load_paddle(m, p), shapes, level=1)          # constant / batch-norm folding only: stock operators
    g = convert_fp32_to_fp16(g, keep_io_types=False)
    it = Interpreter(g, device=str(dev))
    for k, v in list(it.consts.items()):                              # weights of 4-D convolutions in channels-last
        if v.dim() == 4:
            it.consts[k] = v.contiguous(memory_format=torch.channels_last)
    rng = np.random.default_rng(5)
    sets = []
    for _ in range(2):
        x = torch.from_numpy(rng.standard_normal((B, 3, 640, 640)).astype(np.float32)).to(dev).half()
        sets.append({"image": x.contiguous(memory_format=torch.channels_last),
                     "scale_factor": torch.ones(B, 2, dtype=torch.float16, device=dev)})
    names = [vi.name for vi in g.inputs]
    sampler = ClockSampler(physical_gpu_index(ctx.local_rank))
    sampler.start()

    def steps(n):
        with torch.no_grad():
            for i in range(n):
                it.run({k: sets[i % 2][k] for k in names})
    sampler.wait_ready()
    warm = max(args.warmup, 3)
    steps(warm)
    ctx.barrier()
    sampler.rows.clear()
    ms = ctx.time_blocks(steps, args.steps, args.repeats)
    clocks = sampler.stop()
    med = median(ms)
    return {
        "metric": "images/sec PP-YOLOE+-L network only, PyTorch fp16 channels-last + cuDNN (library baseline)",
        "value": round(B * ctx.world * args.steps / (med / 1e3), 1), "unit": "images/s", "n_gpus": ctx.world,
        "steps": args.steps, "warmup": warm, "ms_per_step": round(med / args.steps, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp16", "data": "synthetic",
        "config": {"model": "PP-YOLOE+-L 640x640 network without pre-processing and NMS, random-init weights",
                   "global_batch": B * ctx.world, "seq_len": None, "parallelism": f"dp{ctx.world}",
                   "what": "the imported graph after constant / batch-norm folding, executed operator by operator with "
                           "torch (cuDNN benchmark mode), eager launches",
                   "l2_policy": "activations of one step exceed L2; two alternating inputs",
                   "timing": f"median of {args.repeats} blocks of {args.steps} steps, CUDA events, max over ranks"},
        "block_ms": spread(ms), "gpu_launches": 0, "clocks": clocks, "impl": "library-baseline",
    }
