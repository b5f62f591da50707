"""Triton-style model repository: ``<repo>/<model>/config.pbtxt`` + ``<repo>/<model>/<version>/`` files.

The fields read are the ones the reference's Triton backend consumes (serving/src/fastdeploy_runtime.cc:
95-160, 330-520 and the example repositories under examples/*/serving/models): ``name``, ``backend``,
``max_batch_size``, ``input`` / ``output`` (name, data_type, dims), ``instance_group`` (count, kind, gpus),
``dynamic_batching`` (preferred_batch_size, max_queue_delay_microseconds), ``optimization {
execution_accelerators { gpu_execution_accelerator / cpu_execution_accelerator [ { name, parameters } ] } }``
which selects backend and precision (``tensorrt`` + ``precision: trt_fp16``, ``paddle``, ``onnxruntime``,
``openvino``, ``cpu_threads``, ``use_paddle_log`` ...), and ``parameters``. The text format is protobuf
text; the small parser below covers nested messages, repeated fields, strings, numbers, enums and lists.
"""
from __future__ import annotations

import os
import re
from typing import Any, Dict, List, Optional, Tuple

from ..core.types import ModelFormat
from ..runtime.option import RuntimeOption

_TOKEN = re.compile(r'\s*(?:(#[^\n]*)|("(?:\\.|[^"\\])*")|([{}\[\]:,])|([^\s{}\[\]:,"#]+))')


def parse_pbtxt(text: str) -> Dict[str, Any]:
    """Protobuf text -> nested dicts; a field that appears more than once becomes a list."""
    toks: List[str] = []
    pos = 0
    while pos < len(text):
        m = _TOKEN.match(text, pos)
        if not m:
            break
        pos = m.end()
        if m.group(1):
            continue
        toks.append(m.group(2) or m.group(3) or m.group(4))
    idx = 0

    def value():
        nonlocal idx
        t = toks[idx]
        if t == "{":
            idx += 1
            return message("}")
        if t == "[":
            idx += 1
            items = []
            while toks[idx] != "]":
                items.append(value())
                if toks[idx] == ",":
                    idx += 1
            idx += 1
            return items
        idx += 1
        if t.startswith('"'):
            return bytes(t[1:-1], "utf-8").decode("unicode_escape")
        if re.fullmatch(r"-?\d+", t):
            return int(t)
        if re.fullmatch(r"-?\d*\.\d+(e-?\d+)?|-?\d+e-?\d+", t, re.I):
            return float(t)
        return {"true": True, "false": False}.get(t, t)

    def message(end: Optional[str]):
        nonlocal idx
        out: Dict[str, Any] = {}
        while idx < len(toks) and toks[idx] != end:
            if toks[idx] == ",":          # optional separators between fields
                idx += 1
                continue
            key = toks[idx]
            idx += 1
            if idx < len(toks) and toks[idx] == ":":
                idx += 1
            v = value()
            if key in out:
                if not isinstance(out[key], list):
                    out[key] = [out[key]]
                if isinstance(v, list):
                    out[key].extend(v)
                else:
                    out[key].append(v)
            else:
                out[key] = v
        idx += 1
        return out

    return message(None)


def _as_list(v) -> list:
    if v is None:
        return []
    return v if isinstance(v, list) else [v]


class ModelConfig:
    def __init__(self, cfg: Dict[str, Any], model_dir: str):
        self.raw, self.model_dir = cfg, model_dir
        self.name = cfg.get("name", os.path.basename(model_dir))
        self.backend = cfg.get("backend", "fastdeploy")
        self.max_batch_size = int(cfg.get("max_batch_size", 0))
        self.inputs = [dict(name=i["name"], data_type=i.get("data_type", "TYPE_FP32"), dims=_as_list(i.get("dims")))
                       for i in _as_list(cfg.get("input"))]
        self.outputs = [dict(name=o["name"], data_type=o.get("data_type", "TYPE_FP32"), dims=_as_list(o.get("dims")))
                        for o in _as_list(cfg.get("output"))]
        self.instance_groups = [dict(count=int(g.get("count", 1)), kind=g.get("kind", "KIND_GPU"), gpus=_as_list(g.get("gpus")))
                                for g in _as_list(cfg.get("instance_group"))] or [dict(count=1, kind="KIND_GPU", gpus=[0])]
        db = cfg.get("dynamic_batching")
        self.dynamic_batching = db is not None
        self.preferred_batch_size = _as_list((db or {}).get("preferred_batch_size"))
        self.max_queue_delay_us = int((db or {}).get("max_queue_delay_microseconds", 0))
        self.parameters = {}
        for p in _as_list(cfg.get("parameters")):
            val = p.get("value", {})
            self.parameters[p.get("key")] = val.get("string_value") if isinstance(val, dict) else val
        acc = (cfg.get("optimization") or {}).get("execution_accelerators") or {}
        self.gpu_accelerators = _as_list(acc.get("gpu_execution_accelerator"))
        self.cpu_accelerators = _as_list(acc.get("cpu_execution_accelerator"))

    def versions(self) -> List[int]:
        out = []
        for d in os.listdir(self.model_dir):
            if d.isdigit() and os.path.isdir(os.path.join(self.model_dir, d)):
                out.append(int(d))
        return sorted(out)

    def model_files(self, version: Optional[int] = None) -> Tuple[str, str, int]:
        """(model file, params file, format) of a version directory: ``model.pdmodel`` + ``model.pdiparams``
        or ``model.onnx`` (fastdeploy_runtime.cc:208-246)."""
        vs = self.versions()
        if not vs:
            raise FileNotFoundError(f"no version directory under {self.model_dir}")
        v = version if version is not None else vs[-1]
        d = os.path.join(self.model_dir, str(v))
        pd = os.path.join(d, "model.pdmodel")
        if os.path.exists(pd):
            return pd, os.path.join(d, "model.pdiparams"), ModelFormat.PADDLE
        onnx = os.path.join(d, "model.onnx")
        if os.path.exists(onnx):
            return onnx, "", ModelFormat.ONNX
        raise FileNotFoundError(f"neither model.pdmodel nor model.onnx in {d}")

    def instances(self) -> List[Tuple[str, int]]:
        """Flat list of (kind, device id) - one entry per model instance."""
        out = []
        for g in self.instance_groups:
            ids = g["gpus"] or [0]
            for dev in (ids if g["kind"] == "KIND_GPU" else [-1]):
                out += [("gpu" if g["kind"] == "KIND_GPU" else "cpu", int(dev))] * g["count"]
        return out

    def runtime_option(self, kind: str, device_id: int, version: Optional[int] = None) -> RuntimeOption:
        model, params, fmt = self.model_files(version)
        opt = RuntimeOption()
        opt.set_model_path(model, params, fmt)
        accs = self.gpu_accelerators if kind == "gpu" else self.cpu_accelerators
        if kind == "gpu":
            opt.use_gpu(device_id)
        else:
            opt.use_cpu()
        for a in accs:
            name = a.get("name", "")
            params_ = {}
            for p in _as_list(a.get("parameters")):
                params_[p.get("key")] = p.get("value")
            if name in ("tensorrt", "trt"):
                opt.use_trt_backend()
                if str(params_.get("precision", "")).lower() in ("trt_fp16", "fp16"):
                    opt.enable_trt_fp16()
            elif name == "paddle":
                opt.use_paddle_backend()
            elif name == "onnxruntime":
                opt.use_ort_backend()
            elif name == "openvino":
                opt.use_openvino_backend()
            if "cpu_threads" in params_:
                opt.set_cpu_thread_num(int(params_["cpu_threads"]))
        return opt


def load_model_config(model_dir: str) -> ModelConfig:
    with open(os.path.join(model_dir, "config.pbtxt")) as f:
        return ModelConfig(parse_pbtxt(f.read()), model_dir)


def scan_repository(repo: str) -> Dict[str, ModelConfig]:
    out = {}
    for name in sorted(os.listdir(repo)):
        d = os.path.join(repo, name)
        if os.path.isfile(os.path.join(d, "config.pbtxt")):
            cfg = load_model_config(d)
            out[cfg.name] = cfg
    return out
