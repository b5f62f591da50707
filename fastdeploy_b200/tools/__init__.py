"""Command-line tools: ``python -m fastdeploy_b200.tools {compress, convert, simple_serving, benchmark}``.

The reference's ``fastdeploy`` console script (tools/common_tools/common_tools.py:125-230) has three
sub-commands: ``compress`` (PaddleSlim auto-compression, PTQ / QAT), ``convert`` (X2Paddle: TensorFlow /
Caffe / ONNX -> Paddle) and ``simple_serving`` (uvicorn on a user app). Here:

* ``compress`` is post-training calibration for fp8: it runs calibration batches through the CPU
  interpreter, records the absolute maximum of every GEMM / convolution input and of every weight
  (per output channel), and writes ``quant_scales.json`` plus the weights rounded to e4m3 (stored as the
  original dtype, so the model stays loadable everywhere) next to a copy of the model.
* ``convert`` turns a Paddle inference model into ONNX or an ONNX model into the optimised ONNX graph
  (the importer + IR passes are the converter; TensorFlow / Caffe front ends are not provided).
* ``simple_serving`` starts uvicorn on ``module:app`` exactly like the reference.
* ``benchmark`` times a model file on synthetic inputs (runtime-only latency, like
  benchmark/cpp/benchmark.cc with ``--no_nms``-style raw runtime mode).
"""
from __future__ import annotations

import argparse
import ast
import json
import os
import shutil
import sys
import time
from typing import Dict, List, Optional

import numpy as np


def _load_graph(model: str, params: str = ""):
    from ..importer.onnx_format import load_onnx
    from ..importer.paddle_import import load_paddle
    if model.endswith(".onnx"):
        with open(model, "rb") as f:
            return load_onnx(f.read())
    with open(model, "rb") as f:
        m = f.read()
    p = b""
    if params:
        with open(params, "rb") as f:
            p = f.read()
    return load_paddle(m, p)


def _resolve(model_dir_or_file: str):
    if os.path.isdir(model_dir_or_file):
        for name in ("model.pdmodel", "inference.pdmodel", "model.onnx"):
            p = os.path.join(model_dir_or_file, name)
            if os.path.exists(p):
                return p, p.replace(".pdmodel", ".pdiparams") if p.endswith(".pdmodel") else ""
        raise FileNotFoundError(f"no model file in {model_dir_or_file}")
    if model_dir_or_file.endswith(".pdmodel"):
        return model_dir_or_file, model_dir_or_file.replace(".pdmodel", ".pdiparams")
    return model_dir_or_file, ""


def e4m3_round(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even onto the e4m3 grid (max 448, 3 mantissa bits, subnormals below 2^-6)."""
    import torch
    t = torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32))
    if hasattr(torch, "float8_e4m3fn"):
        return t.clamp(-448, 448).to(torch.float8_e4m3fn).float().numpy()
    m, e = np.frexp(x.astype(np.float64))
    step = np.ldexp(1.0, np.maximum(e, -5) - 4)
    return np.clip(np.round(x / step) * step, -448, 448).astype(np.float32)


def calibrate(graph, feeds_list: List[Dict[str, np.ndarray]]) -> Dict[str, Dict[str, object]]:
    """Per GEMM / convolution node: activation absmax over the calibration set and per-output-channel
    weight absmax. Scales map the absmax onto 448, the largest e4m3 value."""
    from ..ir.interp import Interpreter
    nodes = [n for n in graph.nodes if n.op in ("Conv", "FusedConv", "Gemm", "FusedGemm", "MatMul")]
    amax = {n.name or n.outputs[0]: 0.0 for n in nodes}
    it = Interpreter(graph)
    for feeds in feeds_list:
        env = it.run(feeds, keep_all=True)
        for n in nodes:
            v = env.get(n.inputs[0])
            if v is not None:
                amax[n.name or n.outputs[0]] = max(amax[n.name or n.outputs[0]], float(v.abs().max()))
    out = {}
    for n in nodes:
        key = n.name or n.outputs[0]
        w = graph.initializers.get(n.inputs[1]) if len(n.inputs) > 1 else None
        entry = {"op": n.op, "input": n.inputs[0], "act_absmax": amax[key],
                 "act_scale": (amax[key] / 448.0) if amax[key] > 0 else 1.0}
        if w is not None:
            wa = np.abs(np.asarray(w, np.float32)).reshape(w.shape[0], -1).max(1)
            entry["weight"] = n.inputs[1]
            entry["weight_scale"] = (np.maximum(wa, 1e-12) / 448.0).tolist()
        out[key] = entry
    return out


def cmd_compress(args) -> int:
    model, params = _resolve(args.model or args.config_path)
    g = _load_graph(model, params)
    shapes = ast.literal_eval(args.input_shape_dict) if args.input_shape_dict else {}
    rng = np.random.default_rng(0)
    feeds_list = []
    for _ in range(args.calib_batches):
        feeds = {}
        for vi in g.inputs:
            shp = shapes.get(vi.name) or [d if isinstance(d, int) and d > 0 else 1 for d in vi.shape]
            dt = np.int64 if "int" in str(vi.dtype).lower() else np.float32
            feeds[vi.name] = rng.integers(0, 100, shp).astype(dt) if dt == np.int64 else rng.standard_normal(shp).astype(dt)
        feeds_list.append(feeds)
    if args.calib_npz:
        data = np.load(args.calib_npz)
        feeds_list = [{k: data[k] for k in data.files}]
    scales = calibrate(g, feeds_list)
    os.makedirs(args.save_dir, exist_ok=True)
    for entry in scales.values():
        wn = entry.get("weight")
        if wn is None:
            continue
        w = np.asarray(g.initializers[wn], np.float32)
        s = np.asarray(entry["weight_scale"], np.float32).reshape((-1,) + (1,) * (w.ndim - 1))
        g.initializers[wn] = (e4m3_round(w / s) * s).astype(g.initializers[wn].dtype)
    from ..importer.onnx_format import save_onnx
    with open(os.path.join(args.save_dir, "model.onnx"), "wb") as f:
        f.write(save_onnx(g))
    with open(os.path.join(args.save_dir, "quant_scales.json"), "w") as f:
        json.dump({"format": "e4m3", "method": args.method, "layers": scales}, f, indent=1)
    print(f"calibrated {len(scales)} layers -> {args.save_dir}")
    return 0


def cmd_convert(args) -> int:
    if args.framework not in (None, "paddle", "onnx"):
        print(f"--framework {args.framework} is not supported by this build (paddle and onnx are)", file=sys.stderr)
        return 2
    model, params = _resolve(args.model)
    g = _load_graph(model, params)
    if args.optimize:
        from ..ir.passes import optimize
        shapes = ast.literal_eval(args.input_shape_dict) if args.input_shape_dict else None
        g = optimize(g, shapes, level=1) if shapes else g
    if getattr(args, "to_fp16", False):
        from ..ir.convert_fp16 import convert_fp32_to_fp16
        g = convert_fp32_to_fp16(g, keep_io_types=not getattr(args, "fp16_io", False))
    from ..importer.onnx_format import save_onnx
    os.makedirs(args.save_dir, exist_ok=True)
    out = os.path.join(args.save_dir, "model.onnx")
    with open(out, "wb") as f:
        f.write(save_onnx(g))
    print(f"wrote {out}: {len(g.nodes)} nodes, {len(g.initializers)} initializers")
    return 0


def cmd_simple_serving(args) -> int:
    import uvicorn
    uvicorn.run(args.app, host=args.host, port=args.port, app_dir=".")
    return 0


def cmd_benchmark(args) -> int:
    import fastdeploy_b200 as fd
    from ..core.types import ModelFormat
    model, params = _resolve(args.model)
    opt = fd.RuntimeOption()
    opt.set_model_path(model, params, ModelFormat.ONNX if model.endswith(".onnx") else ModelFormat.PADDLE)
    if args.device == "gpu":
        opt.use_gpu(args.device_id)
        if args.fp16:
            opt.enable_trt_fp16()
    else:
        opt.use_cpu()
    rt = fd.Runtime(opt)
    shapes = ast.literal_eval(args.input_shape_dict) if args.input_shape_dict else {}
    rng = np.random.default_rng(0)
    feeds = {}
    for info in rt.get_input_infos():
        shp = shapes.get(info.name) or [d if isinstance(d, int) and d > 0 else 1 for d in info.shape]
        feeds[info.name] = rng.standard_normal(shp).astype(np.float32)
    for _ in range(args.warmup):
        rt.infer(feeds)
    t0 = time.perf_counter()
    for _ in range(args.repeat):
        rt.infer(feeds)
    ms = 1e3 * (time.perf_counter() - t0) / max(args.repeat, 1)
    print(json.dumps({"model": model, "device": args.device, "runtime_ms": ms, "repeat": args.repeat}))
    return 0


def cmd_export_plan(args) -> int:
    """``fastdeploy export_plan --model dir --input_shape_dict "{...}" --save_dir out``: builds the GPU plan for the
    given shapes and writes ``out/model.fdplan`` for the C++ runner (``fdplan_run``, ``libfdb200_runner.so``)."""
    import fastdeploy_b200 as fd
    from ..core.types import ModelFormat
    model, params = _resolve(args.model)
    opt = fd.RuntimeOption()
    opt.set_model_path(model, params, ModelFormat.ONNX if model.endswith(".onnx") else ModelFormat.PADDLE)
    opt.use_gpu(args.device_id)
    rt = fd.Runtime(opt)
    shapes = ast.literal_eval(args.input_shape_dict) if args.input_shape_dict else None
    if not shapes:
        raise SystemExit("export_plan needs --input_shape_dict with a static shape for every input")
    os.makedirs(args.save_dir, exist_ok=True)
    out = os.path.join(args.save_dir, "model.fdplan")
    info = rt.export_plan(out, shapes)
    print(json.dumps(dict(info, path=out)))
    return 0


def argsparser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="fastdeploy", description=__doc__.split("\n\n")[0])
    p.add_argument("tools", choices=["compress", "convert", "simple_serving", "benchmark", "export_plan", "paddle2coreml"])
    p.add_argument("--config_path", default=None, help="compress: model directory (kept for command compatibility)")
    p.add_argument("--method", default="PTQ", help="compress: PTQ (post-training calibration)")
    p.add_argument("--save_dir", default="./output", help="directory to save the result")
    p.add_argument("--devices", default="gpu")
    p.add_argument("--framework", default=None, help="convert: paddle or onnx")
    p.add_argument("--model", default=None, help="model file or directory")
    p.add_argument("--input_shape_dict", default=None, help="e.g. \"{'image':[1,3,640,640]}\"")
    p.add_argument("--optimize", action="store_true", help="convert: run the IR optimiser before writing")
    p.add_argument("--to_fp16", action="store_true", help="convert: store weights and compute in half precision "
                                                           "(operators that need it stay fp32 between casts)")
    p.add_argument("--fp16_io", action="store_true", help="convert --to_fp16: also make the graph inputs / outputs fp16")
    p.add_argument("--calib_batches", type=int, default=4)
    p.add_argument("--calib_npz", default=None, help="compress: .npz with one array per model input")
    p.add_argument("--app", default="server:app", help="simple_serving: module:attribute of the app")
    p.add_argument("--host", default="127.0.0.1")
    p.add_argument("--port", type=int, default=8000)
    p.add_argument("--device", default="cpu", choices=["cpu", "gpu"])
    p.add_argument("--device_id", type=int, default=0)
    p.add_argument("--fp16", action="store_true")
    # flags of the reference's command line that have no meaning here; accepted so that existing scripts parse
    for flag in ("--prototxt", "--weight", "--caffe_proto", "--p2c_paddle_model_dir", "--p2c_coreml_model_dir",
                 "--p2c_coreml_model_name", "--p2c_input_names", "--p2c_input_dtypes", "--p2c_input_shapes", "--p2c_output_names"):
        p.add_argument(flag, default=None, help=argparse.SUPPRESS)
    p.add_argument("--enable_code_optim", default=None, help=argparse.SUPPRESS)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--repeat", type=int, default=20)
    return p


def cmd_paddle2coreml(args) -> int:
    """The reference converts a Paddle model to Apple's CoreML with an external package
    (tools/common_tools/common_tools.py:165-190). That format has no consumer on this hardware: say so and point at the
    converter that exists."""
    import sys
    print("paddle2coreml is not available in this package: CoreML targets Apple devices. "
          "Use `convert --framework paddle --model <dir> --save_dir <dir>` for an ONNX file.", file=sys.stderr)
    return 2


def main(argv: Optional[List[str]] = None) -> int:
    args = argsparser().parse_args(argv)
    if args.tools == "paddle2coreml":
        return cmd_paddle2coreml(args)
    if args.tools == "convert" and args.framework is not None and args.framework.lower() in ("caffe", "tensorflow"):
        import sys
        print(f"convert: framework {args.framework!r} needs the x2paddle converter, which is not part of this package; "
              "paddle and onnx models are converted", file=sys.stderr)
        return 2
    return {"compress": cmd_compress, "convert": cmd_convert, "simple_serving": cmd_simple_serving,
            "benchmark": cmd_benchmark, "export_plan": cmd_export_plan}[args.tools](args)
