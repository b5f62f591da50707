"""The same PP-YOLOE+-L workload driven by ONE process: ``serving.Scheduler`` with one worker thread per GPU,
each owning its device, its stream and its own ``PPYOLOE`` model, fed with single-frame requests that the native
batching core groups into batches of 32 (``PPYOLOE.predict_async``, three batches in flight per GPU). Under
``torch.distributed.run`` only rank 0 runs this part; the other ranks wait for it on the rendezvous store."""
from __future__ import annotations

import os
import time

from .common import Context


class _Timed:
    """Wraps a model so that the worker's stream carries an event before its first and after its last batch."""

    def __init__(self, model, torch):
        self.model, self.torch = model, torch
        self.runtime = model.runtime
        self.first = self.last = None

    def predict_async(self, frames):
        if self.first is None:
            self.first = self.torch.cuda.Event(enable_timing=True)
            self.first.record()
        h = self.model.predict_async(frames)
        self.last = self.torch.cuda.Event(enable_timing=True)
        self.last.record()
        return h

    def reset(self):
        self.first = self.last = None


def run(ctx: Context, args, model_dir: str, host_sets) -> dict:
    torch = ctx.torch
    store = None
    if ctx.world > 1:
        store = ctx.dist.distributed_c10d._get_default_store()
        if ctx.rank != 0:
            store.wait(["fdb_scheduler_mode_done"])
            return {}
    import fastdeploy_b200 as fd
    from fastdeploy_b200.serving import Scheduler
    n_gpu = ctx.world
    B = host_sets[0].shape[0]
    wrapped = {}

    def factory(i):
        opt = fd.RuntimeOption()
        opt.use_gpu(i)
        opt.enable_trt_fp16()
        m = fd.vision.detection.PPYOLOE(os.path.join(model_dir, "model.pdmodel"), os.path.join(model_dir, "model.pdiparams"),
                                        os.path.join(model_dir, "infer_cfg.yml"), runtime_option=opt)
        wrapped[i] = _Timed(m, torch)
        return wrapped[i]
    sched = Scheduler(factory, lambda m, frames: m.predict_async(frames), num_workers=n_gpu, max_batch_size=B,
                      max_queue_delay_us=2000, pipeline_depth=3)
    out = {}
    try:
        def burst(k):
            hs = host_sets[k % len(host_sets)]
            return sched.submit_many([hs[j] for j in range(B)], together=True)

        def run_steps(steps):
            futs = []
            for k in range(steps * n_gpu):
                futs.append(burst(k))
                if len(futs) > 4 * n_gpu:                 # bounded queue: at most four batches waiting per GPU
                    for f in futs.pop(0):
                        f.result(120)
            dets = 0
            for fs in futs:
                for f in fs:
                    dets += len(f.result(120).boxes)
            return dets
        run_steps(max(args.warmup, 3))                    # builds the plans, one per GPU
        for w in wrapped.values():
            w.reset()
        for i in range(n_gpu):
            torch.cuda.synchronize(i)
        t0 = time.perf_counter()
        run_steps(args.steps)
        for i in range(n_gpu):
            torch.cuda.synchronize(i)
        wall_ms = (time.perf_counter() - t0) * 1e3
        dev_ms = max(w.first.elapsed_time(w.last) for w in wrapped.values() if w.first is not None)
        imgs = B * n_gpu * args.steps
        st = sched.stats()["workers"]
        out = {"value": round(imgs / (dev_ms / 1e3), 1), "unit": "images/s", "n_gpus": n_gpu,
               "timing": "CUDA events on each worker's stream, first batch queued to last batch queued + drained, max over GPUs",
               "device_ms": round(dev_ms, 3), "wall_ms": round(wall_ms, 3),
               "wall_images_per_s": round(imgs / (wall_ms / 1e3), 1),
               "avg_batch_size": round(sum(w["avg_batch_size"] for w in st) / len(st), 2),
               "requests_per_worker": [w["requests"] for w in st],
               "what": "one process, serving.Scheduler, one worker thread + stream + model per GPU, single-frame requests"}
    finally:
        sched.close()
        if store is not None:
            store.set("fdb_scheduler_mode_done", "1")
    return out
