"""Per-model benchmark driver with the reference's config-file vocabulary.

    python -m fastdeploy_b200.benchmarks.model_zoo --model ppyoloe --config_path config.gpu.fp16.txt
    python -m fastdeploy_b200.benchmarks.model_zoo --model resnet50 --device gpu --profile_mode runtime

One program stands for the reference's family of ``benchmark/cpp/benchmark_<model>.cc`` files (34 of them, all one
macro: benchmark/cpp/macros.h:20-116): it builds the named model on synthetic weights, feeds a synthetic image (or
token batch), and reports ``Runtime(ms)`` (``profile_mode: runtime`` - the backend call timed inside ``infer`` by the
runtime's own profiling loop, optionally with the host<->device copies) or ``End2End(ms)`` (``profile_mode: end2end``
- warm-up then ``repeat`` full ``predict`` calls under a ``TimeCounter``), plus peak CPU / GPU memory and GPU
utilisation when ``collect_memory_info`` is on. Keys of the config file: device, device_id, cpu_thread_nums, warmup,
repeat, backend, profile_mode, include_h2d_d2h, use_fp16, collect_memory_info, sampling_interval, result_path
(benchmark/cpp/config/config.gpu.paddle_trt.fp16.txt)."""
from __future__ import annotations

import argparse
import os
import sys
import tempfile
from typing import Callable, Dict, Tuple

import numpy as np

DEFAULTS = {"device": "gpu", "device_id": "0", "cpu_thread_nums": "1", "warmup": "20", "repeat": "100", "backend": "native",
            "profile_mode": "runtime", "include_h2d_d2h": "false", "use_fp16": "true", "collect_memory_info": "false",
            "sampling_interval": "1", "result_path": ""}


def load_benchmark_config(path: str) -> Dict[str, str]:
    """``key: value`` lines (ResultManager::LoadBenchmarkConfig, fastdeploy/benchmark/utils.cc)."""
    cfg = dict(DEFAULTS)
    if path:
        with open(path) as f:
            for line in f:
                if ":" in line:
                    k, v = line.split(":", 1)
                    cfg[k.strip()] = v.strip()
    return cfg


def _option(cfg: Dict[str, str]):
    import fastdeploy_b200 as fd
    opt = fd.RuntimeOption()
    if cfg["device"] == "gpu":
        opt.use_gpu(int(cfg["device_id"]))
        if cfg["use_fp16"] == "true":
            opt.enable_trt_fp16()
    else:
        opt.use_cpu()
        opt.set_cpu_thread_num(int(cfg["cpu_thread_nums"]))
    if cfg["profile_mode"] == "runtime":
        opt.enable_profiling(cfg["include_h2d_d2h"] == "true", int(cfg["repeat"]), int(cfg["warmup"]))
    return opt


def _image(h: int, w: int) -> np.ndarray:
    return np.random.default_rng(0).integers(0, 256, (h, w, 3), dtype=np.uint8)


def _build_ppyoloe(cfg, d):
    import fastdeploy_b200 as fd
    from ..models.ppyoloe import write_ppyoloe
    write_ppyoloe(d, "s", image=640, num_classes=80, seed=0)
    m = fd.vision.detection.PPYOLOE(os.path.join(d, "model.pdmodel"), os.path.join(d, "model.pdiparams"),
                                    os.path.join(d, "infer_cfg.yml"), runtime_option=_option(cfg))
    im = _image(720, 1280)
    return m, lambda: m.predict(im)


def _build_resnet50(cfg, d):
    import fastdeploy_b200 as fd
    from ..models.resnet import resnet50_onnx
    path = os.path.join(d, "resnet50.onnx")
    with open(path, "wb") as f:
        f.write(resnet50_onnx())
    opt = _option(cfg)
    opt.set_model_path(path, "", fd.ModelFormat.ONNX)
    rt = fd.Runtime(opt)
    x = np.random.default_rng(0).standard_normal((1, 3, 224, 224)).astype(np.float32)
    name = rt.get_input_info(0).name
    return rt, lambda: rt.infer({name: x})


def _build_ocr(stage: str):
    def build(cfg, d):
        import fastdeploy_b200 as fd
        from ..models import ppocr
        paths = ppocr.write_ppocr(d)
        if stage == "det":
            m = fd.vision.ocr.DBDetector(paths["det_model"], paths["det_params"], runtime_option=_option(cfg))
            im = _image(640, 640)
        elif stage == "cls":
            m = fd.vision.ocr.Classifier(paths["cls_model"], paths["cls_params"], runtime_option=_option(cfg))
            im = _image(48, 192)
        else:
            m = fd.vision.ocr.Recognizer(paths["rec_model"], paths["rec_params"], paths["dict"], runtime_option=_option(cfg))
            im = _image(48, 320)
        return m, lambda: m.predict(im)
    return build


def _build_ernie(cfg, d):
    import fastdeploy_b200 as fd
    from ..models.ernie import write_ernie
    write_ernie(d, "tiny", "seq_cls", seed=0, vocab=False)
    opt = _option(cfg)
    opt.set_model_path(os.path.join(d, "model.pdmodel"), os.path.join(d, "model.pdiparams"))
    rt = fd.Runtime(opt)
    ids = np.random.default_rng(0).integers(1, 100, (8, 128)).astype(np.int64)
    feeds = {rt.get_input_info(i).name: (ids if i == 0 else np.zeros_like(ids)) for i in range(rt.num_inputs())}
    return rt, lambda: rt.infer(feeds)


MODELS: Dict[str, Callable] = {"ppyoloe": _build_ppyoloe, "resnet50": _build_resnet50, "ppocr_det": _build_ocr("det"),
                               "ppocr_cls": _build_ocr("cls"), "ppocr_rec": _build_ocr("rec"), "ernie": _build_ernie}


def run_benchmark(model: str, cfg: Dict[str, str]) -> Dict[str, float]:
    """Builds ``model``, runs it the way the reference's BENCHMARK_MODEL macro does, returns the reported numbers."""
    from ..utils.benchmark import ResourceUsageMonitor
    from ..utils.perf import TimeCounter
    d = tempfile.mkdtemp(prefix=f"fdb200_bench_{model}_")
    obj, step = MODELS[model](cfg, d)
    out: Dict[str, float] = {}
    monitor = None
    if cfg["collect_memory_info"] == "true":
        monitor = ResourceUsageMonitor(int(cfg["sampling_interval"]) * 1000, int(cfg["device_id"]))
        monitor.start()
    if cfg["profile_mode"] == "runtime":
        step()                                         # the runtime's profiling loop runs inside this call
        out["Runtime(ms)"] = obj.get_profile_time() * 1000.0
    else:
        for _ in range(int(cfg["warmup"])):
            step()
        tc = TimeCounter()
        tc.start()
        repeat = int(cfg["repeat"])
        for _ in range(repeat):
            step()
        tc.end()
        out["End2End(ms)"] = tc.duration() / repeat * 1000.0
    if monitor is not None:
        monitor.stop()
        out["cpu_rss_mb"], out["gpu_rss_mb"], out["gpu_util"] = (monitor.get_max_cpu_mem(), monitor.get_max_gpu_mem(),
                                                                monitor.get_max_gpu_util())
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True, choices=sorted(MODELS))
    ap.add_argument("--config_path", default="")
    for k in DEFAULTS:
        ap.add_argument("--" + k, default=None)
    a = ap.parse_args(argv)
    cfg = load_benchmark_config(a.config_path)
    for k in DEFAULTS:
        if getattr(a, k) is not None:
            cfg[k] = str(getattr(a, k))
    res = run_benchmark(a.model, cfg)
    lines = [f"{k}: {v:.6g}{'ms.' if k.endswith('(ms)') else ('MB.' if k.endswith('_mb') else '')}" for k, v in res.items()]
    print("\n".join(lines))
    if cfg["result_path"]:
        with open(cfg["result_path"], "a") as f:       # ResultManager::SaveBenchmarkResult appends
            f.write("\n".join(lines) + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
