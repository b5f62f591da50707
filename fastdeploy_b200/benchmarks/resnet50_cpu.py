"""ResNet-50 v1.5 (ONNX, fp32, random-init, 1000 classes) through ``Runtime`` on the CPU, batch 1: a 224x224x3 uint8
image, ImageNet mean / std and HWC -> CHW in the pre-processor, top-5 after the network. The reference's counterpart
is benchmark/cpp/benchmark_resnet.cc with ``config.x86.ort.fp32.txt`` (ONNX Runtime on the CPU); its published figure is
76.14 ms runtime / 77.43 ms end to end for ResNet50_vd on one thread of a Xeon Gold 6271C.

No GPU is involved: the CPU path of this framework is the graph interpreter on PyTorch's CPU operators (oneDNN
convolutions), used for oracles and for machines without a B200. Times are host wall-clock (``perf_counter``), median
of ``--steps`` calls after ``--warmup``; the machine's CPU model is recorded beside the number.
"""
from __future__ import annotations

import os
import platform
import statistics
import tempfile
import time


def _cpu_name() -> str:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("model name"):
                    return line.split(":", 1)[1].strip()
    except OSError:
        pass
    return platform.processor() or "unknown"


def run_cpu(args) -> dict:
    import numpy as np
    import torch
    import fastdeploy_b200 as fd
    from fastdeploy_b200.models.resnet import resnet50_onnx
    fd.set_logger(False, True)
    d = args.model_dir or tempfile.mkdtemp(prefix="fdb200_resnet50_")
    path = os.path.join(d, "resnet50.onnx")
    if not os.path.exists(path):
        resnet50_onnx(path, seed=0)
    rng = np.random.default_rng(0)
    image = rng.integers(0, 256, (224, 224, 3), dtype=np.uint8)
    warm, steps = max(args.warmup, 3), max(args.steps, 5)
    rows = {}
    for threads in (1, max(1, os.cpu_count() or 1)):
        torch.set_num_threads(threads)
        opt = fd.RuntimeOption()
        opt.use_cpu()
        opt.set_cpu_thread_num(threads)
        model = fd.vision.classification.ResNet(path, runtime_option=opt)
        for _ in range(warm):
            res = model.predict(image, topk=5)
        e2e, net = [], []
        x = np.ascontiguousarray(model.preprocessor.run([image])[0])
        name = model.runtime.get_input_info(0).name
        for _ in range(steps):
            t0 = time.perf_counter()
            res = model.predict(image, topk=5)
            e2e.append((time.perf_counter() - t0) * 1e3)
            t0 = time.perf_counter()
            model.runtime.infer({name: x})
            net.append((time.perf_counter() - t0) * 1e3)
        assert len(res.label_ids) == 5
        rows[threads] = {"e2e_ms": round(statistics.median(e2e), 3), "runtime_ms": round(statistics.median(net), 3)}
    one = rows[1]
    return {
        "metric": "latency ResNet-50 v1.5 batch 1 on CPU (end to end, one thread)", "value": one["e2e_ms"], "unit": "ms",
        "n_gpus": 0, "steps": steps, "warmup": warm, "ms_per_step": one["e2e_ms"], "higher_is_better": False,
        "scaling": "none", "vs_baseline": round(one["e2e_ms"] / 77.43, 3), "dtype": "fp32", "data": "synthetic",
        "config": {"model": "ResNet-50 v1.5 ONNX opset 11, random-init fp32 weights, 1000 classes",
                   "global_batch": 1, "seq_len": None, "parallelism": "cpu",
                   "pipeline": "uint8 224x224x3 -> mean/std + HWC2CHW -> network -> soft-max + top-5",
                   "cpu": _cpu_name(), "threads_measured": sorted(rows),
                   "timing": "host perf_counter, median of the timed calls",
                   "baseline_ref": "reference: 77.43 ms end to end / 76.14 ms runtime, ResNet50_vd, ONNX Runtime, one "
                                   "thread of a Xeon Gold 6271C"},
        "by_threads": {str(k): v for k, v in rows.items()}, "gpu_launches": 0, "impl": "ours",
    }
