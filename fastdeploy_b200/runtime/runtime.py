"""``Runtime``: the model-agnostic inference object
(fastdeploy/runtime/runtime.h:37-127, python/fastdeploy/runtime.py:21-158).

``Init`` = read (optionally decrypt) the model, import it into the IR, and - on GPU -
lower it to a launch plan for every input-shape bucket it meets; ``Infer`` copies the
inputs into the plan's static buffers, replays the plan (a CUDA graph when enabled)
and returns the outputs. ``Clone`` shares the imported graph and, on the same device,
the device-resident weights, as the reference's backends do
(fastdeploy/runtime/runtime.cc:396-414).
"""
from __future__ import annotations

import os
import threading
import time
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from ..core.types import Backend, Device, FDDataType, ModelFormat, TensorInfo
from ..importer.onnx_format import load_onnx
from ..importer.paddle_import import load_paddle
from ..ir.graph import Graph
from ..ir.interp import Interpreter
from ..utils import log
from .option import RuntimeOption


def _read(path: str) -> bytes:
    with open(path, "rb") as f:
        return f.read()


def load_graph(option: RuntimeOption) -> Graph:
    """Model file(s) or buffers -> IR, honouring ``model_format`` and the encryption key."""
    fmt = option.model_format
    if option.model_from_memory:
        model, params = option.model_buffer, option.params_buffer or b""
    else:
        if not option.model_file:
            raise ValueError("RuntimeOption has no model: call set_model_path or set_model_buffer")
        model = _read(option.model_file)
        params = _read(option.params_file) if option.params_file else b""
    if option.encryption_key:
        from ..encryption import decrypt
        model = decrypt(model, option.encryption_key)
        if params:
            params = decrypt(params, option.encryption_key)
    if fmt == ModelFormat.AUTOREC:
        name = (option.model_file or "").lower()
        fmt = ModelFormat.ONNX if name.endswith(".onnx") else ModelFormat.PADDLE
    if fmt == ModelFormat.ONNX:
        return load_onnx(model)
    if fmt == ModelFormat.PADDLE:
        return load_paddle(model, params)
    raise ValueError(f"model format {fmt.name} is not supported by this runtime (ONNX and PADDLE are)")


# Plan building allocates, packs weights and captures a CUDA graph: one at a time per process, so that the
# worker threads of a multi-GPU scheduler do not interleave their captures.
_PLAN_BUILD_LOCK = threading.Lock()


_META_READY = False


def _import_meta_kernels() -> None:
    """Shape inference runs the graph on meta tensors. The first meta operation of a process makes PyTorch import
    (and, without a bytecode cache, compile) its Python meta registrations and symbolic-shape modules: seconds that
    belong to process start, not to the first plan. Doing it here keeps the plan-build time that is logged per shape
    free of it, and says what it cost."""
    global _META_READY
    if _META_READY:
        return
    t0 = time.time()
    torch.empty(1, device="meta") + 1
    _META_READY = True
    dt = time.time() - t0
    if dt > 0.2:
        log.info(f"PyTorch meta kernels imported in {dt:.2f}s (once per process)")


class Runtime:
    def __init__(self, runtime_option: Optional[RuntimeOption] = None, _graph: Optional[Graph] = None):
        self.option = runtime_option or RuntimeOption()
        self.option.native_option.apply_env()
        self.graph: Graph = _graph if _graph is not None else load_graph(self.option)
        self._lock = threading.Lock()
        self._plans: Dict[tuple, Any] = {}
        self._interp: Optional[Interpreter] = None
        self._bound_inputs: Dict[str, Any] = {}
        self._bound_outputs: Dict[str, torch.Tensor] = {}
        self._last_outputs: Dict[str, Any] = {}
        self._profile_time = 0.0
        self._last_plan = None
        self._status_host = None
        self._status_event = None
        self.gpu_launches = 0
        self.on_gpu = self.option.device == Device.GPU
        if self.on_gpu:
            if not torch.cuda.is_available():
                raise RuntimeError("RuntimeOption.use_gpu() was requested but no CUDA device is available")
            from .. import _native
            _native.kernels()           # fail loudly when the kernel library is missing
            self.device = torch.device("cuda", self.option.device_id)
            # fp8: 16-bit (bf16) activations between layers, e4m3 operands inside the linear layers
            self.dtype = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp8": torch.bfloat16}[
                self.option.native_option.precision]
            self.fp8 = self.option.native_option.precision == "fp8"
            self.act_scales = self._load_quant_scales() if self.fp8 else {}
            _import_meta_kernels()
            if self.option.trt_shapes:
                shapes = {k: v["opt"] for k, v in self.option.trt_shapes.items()}
                if all(vi.name in shapes for vi in self.graph.inputs):
                    self._plan_for(shapes)
        else:
            self.device = torch.device("cpu")
            if self.option.cpu_thread_num > 0:
                torch.set_num_threads(self.option.cpu_thread_num)
            # the CPU path runs the optimised graph (constant, batch-norm and bias folding, activations fused into
            # their convolutions) with channel-innermost operands and weights packed once for the vendor primitive
            from ..ir.passes import optimize
            self._interp = Interpreter(optimize(self.graph, level=2), channels_last=True)

    # ------------------------------------------------------------------ introspection
    def num_inputs(self) -> int:
        return len(self.graph.inputs)

    def num_outputs(self) -> int:
        return len(self.graph.outputs)

    def get_input_info(self, index: int) -> TensorInfo:
        vi = self.graph.inputs[index]
        shape = [d if isinstance(d, int) else -1 for d in (vi.shape or [])]
        return TensorInfo(vi.name, shape, FDDataType.from_numpy(vi.dtype))

    def get_output_info(self, index: int) -> TensorInfo:
        vi = self.graph.outputs[index]
        shape = [d if isinstance(d, int) else -1 for d in (vi.shape or [])]
        return TensorInfo(vi.name, shape, FDDataType.from_numpy(vi.dtype) if vi.dtype in ("float32", "int32", "int64", "float16", "uint8", "int8", "bool", "float64", "int16") else FDDataType.FP32)

    def get_input_infos(self) -> List[TensorInfo]:
        return [self.get_input_info(i) for i in range(self.num_inputs())]

    def get_output_infos(self) -> List[TensorInfo]:
        return [self.get_output_info(i) for i in range(self.num_outputs())]

    def _load_quant_scales(self) -> Dict[str, float]:
        """Static activation ranges from a calibration file: ``quant_scales.json`` next to the model (what
        ``fastdeploy compress`` writes) or the file named by ``native_option.quant_scales_file``. Layers are keyed by
        node name there; the executor wants the range of each layer's *input tensor*, which the file records as
        ``input``."""
        import json
        import os
        path = getattr(self.option.native_option, "quant_scales_file", "") or ""
        if not path and getattr(self.option, "model_file", ""):
            cand = os.path.join(os.path.dirname(self.option.model_file), "quant_scales.json")
            path = cand if os.path.exists(cand) else ""
        if not path:
            return {}
        with open(path) as f:
            doc = json.load(f)
        out: Dict[str, float] = {}
        for entry in doc.get("layers", {}).values():
            name, amax = entry.get("input"), entry.get("act_absmax")
            if name and amax and amax > 0:
                out[name] = max(out.get(name, 0.0), float(amax))
        log.info(f"loaded {len(out)} calibrated activation ranges from {path}")
        return out

    # ------------------------------------------------------------------ plans
    def _plan_for(self, shapes: Dict[str, Sequence[int]]):
        key = tuple((k, tuple(int(d) for d in shapes[k])) for k in sorted(shapes))
        plan = self._plans.get(key)
        if plan is None:
            from .native_backend import build_plan
            t0 = time.time()
            with _PLAN_BUILD_LOCK:
                plan = build_plan(self.graph, {k: list(v) for k, v in shapes.items()}, self.device, self.dtype,
                                  opt_level=self.option.native_option.opt_level,
                                  cache_dir=self.option.native_option.plan_cache_dir,
                                  fp8=getattr(self, "fp8", False), act_scales=getattr(self, "act_scales", None))
                if self.option.native_option.use_cuda_graph:
                    try:
                        plan.capture()
                    except Exception as e:   # capture is an optimisation; eager replay stays correct
                        log.warning(f"CUDA graph capture failed ({e}); running the plan eagerly")
                        plan.graph = None
            if len(self._plans) >= self.option.native_option.max_plans:
                self._plans.pop(next(iter(self._plans)))
            self._plans[key] = plan
            mem = plan.extra.get("memory")
            log.info(f"built plan for {dict(key)} in {time.time() - t0:.2f}s: {len(plan.steps)} steps, "
                     f"{plan.native_kernel_launches} native kernel launches" +
                     (f", activation arena {mem['arena_bytes'] / 2**20:.0f} MiB for {mem['requested_bytes'] / 2**20:.0f} "
                      f"MiB of buffers" if mem else ""))
        return plan

    def export_plan(self, path: str, shapes: Dict[str, Sequence[int]]) -> Dict[str, Any]:
        """Builds (or takes) the plan for ``shapes`` and writes it as a plan file that ``libfdb200_runner.so`` /
        ``fdplan_run`` replay without Python (runtime/plan_file.py). Returns the export summary."""
        from .plan_file import export_plan
        if not self.on_gpu:
            raise RuntimeError("plan files are written from GPU plans")
        with torch.cuda.device(self.device):
            return export_plan(self._plan_for({k: list(v) for k, v in shapes.items()}), path)

    def memory_report(self) -> Dict[str, Dict[str, int]]:
        """Per built plan (keyed by its input shapes): bytes of the shared activation arena, bytes the same buffers
        would take without reuse, and the largest amount live at once."""
        return {str(dict(k)): dict(p.extra["memory"]) for k, p in self._plans.items() if "memory" in p.extra}

    def plan_for_shapes(self, shapes: Dict[str, Sequence[int]]):
        """Public access for model classes that write inputs straight into plan buffers."""
        with torch.cuda.device(self.device):
            return self._plan_for(shapes)

    # ------------------------------------------------------------------ inference
    def infer(self, data: Union[Dict[str, Any], Sequence[Any]]) -> List[np.ndarray]:
        if not isinstance(data, dict):
            names = [vi.name for vi in self.graph.inputs]
            data = dict(zip(names, data))
        outs = self._infer_dict(data)
        res = [self._to_numpy(outs[vi.name]) for vi in self.graph.outputs]
        self._check_status()
        return res

    def forward(self, *inputs) -> List[np.ndarray]:
        return self.infer(list(inputs))

    @staticmethod
    def _to_numpy(t) -> np.ndarray:
        if isinstance(t, np.ndarray):
            return t
        if t.dtype in (torch.float16, torch.bfloat16):
            t = t.float()
        return t.detach().cpu().numpy()

    def _infer_dict(self, data: Dict[str, Any]) -> Dict[str, Any]:
        with self._lock:
            if not self.on_gpu:
                feeds = {k: (np.ascontiguousarray(v) if isinstance(v, np.ndarray) else v) for k, v in data.items()}
                prof = self.option.profiling
                if prof["enable"]:
                    # the CPU path has no copies to exclude: warm up, then time `repeat` runs on the host clock
                    for _ in range(prof["warmup"]):
                        self._interp.run(feeds)
                    t0 = time.perf_counter()
                    for _ in range(max(prof["repeat"], 1)):
                        res = self._interp.run(feeds)
                    self._profile_time = (time.perf_counter() - t0) / max(prof["repeat"], 1)
                    return res
                return self._interp.run(feeds)
            with torch.cuda.device(self.device):
                shapes = {vi.name: list(data[vi.name].shape) for vi in self.graph.inputs}
                n_valid, bucket = self._batch_bucket(shapes)
                if bucket is not None:
                    shapes = {k: [bucket] + v[1:] for k, v in shapes.items()}
                plan = self._plan_for(shapes)
                self._last_plan = plan
                prof = self.option.profiling
                ev = None
                if prof["enable"] and prof["include_h2d_d2h"]:
                    ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                    ev[0].record()
                for vi in self.graph.inputs:
                    self._copy_in(plan.inputs[vi.name], data[vi.name], n_valid if bucket is not None else None)
                if prof["enable"] and not prof["include_h2d_d2h"]:
                    for _ in range(prof["warmup"]):
                        plan.run()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for _ in range(prof["repeat"]):
                        plan.run()
                    e1.record()
                    torch.cuda.synchronize(self.device)
                    self._profile_time = e0.elapsed_time(e1) / 1e3 / max(prof["repeat"], 1)
                else:
                    plan.run()
                self.gpu_launches += plan.native_kernel_launches
                outs = self._collect_outputs(plan, (n_valid, bucket) if bucket is not None else None)
                if self._status_host is None:
                    self._status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
                    self._status_event = torch.cuda.Event()
                plan.status.snapshot_async(self._status_host)
                self._status_event.record(torch.cuda.current_stream(self.device))
                if ev is not None:
                    ev[1].record()
                    torch.cuda.synchronize(self.device)
                    self._profile_time = ev[0].elapsed_time(ev[1]) / 1e3
                return outs

    def _check_status(self) -> None:
        """Reads the device status word of the plan that just ran. Kernels report a bounded wait that ran out
        (or a rejected shape) through this word instead of trapping, so every inference must look at it: the
        device->host copies of the outputs have already synchronised the stream, the extra 4-byte read is free."""
        plan = self._last_plan
        if plan is not None and self._status_event is not None:
            self._status_event.synchronize()
            plan.status.check_snapshot(self._status_host, "inference")

    def _batch_bucket(self, shapes: Dict[str, List[int]]):
        """``(n, bucket)``: with ``native_option.batch_buckets`` set and every input sharing its first dimension
        ``n``, the smallest bucket that holds ``n`` (``None`` when ``n`` is a bucket itself, exceeds them all, or the
        inputs do not share a batch dimension). The batch then runs in the bucket's plan: rows past ``n`` of the
        plan inputs keep what an earlier batch left there, and outputs are cut back to ``n``."""
        buckets = sorted(self.option.native_option.batch_buckets or [])
        if not buckets or not shapes:
            return None, None
        firsts = {v[0] if len(v) else None for v in shapes.values()}
        if len(firsts) != 1 or None in firsts:
            return None, None
        n = int(next(iter(firsts)))
        for b in buckets:
            if b >= n:
                return n, (int(b) if b != n else None)
        return n, None

    def _copy_in(self, dst, src, n_valid: Optional[int] = None) -> None:
        if isinstance(src, np.ndarray):
            src = torch.from_numpy(np.ascontiguousarray(src))
        if src.device != dst.t.device:
            src = src.to(dst.t.device, non_blocking=True)
        view = dst.t if n_valid is None else dst.t[:n_valid]
        if dst.nhwc:
            view.copy_(src.permute(0, 2, 3, 1))
        else:
            view.copy_(src.reshape(view.shape))

    def _collect_outputs(self, plan, cut: Optional[Tuple[int, int]] = None) -> Dict[str, Any]:
        """``cut = (n, bucket)``: the plan ran a batch of ``n`` padded to ``bucket``; outputs whose first dimension
        is the bucket are cut back to ``n`` (detections of the padding images are dropped)."""
        padded = plan.extra.get("padded_nms_outputs", {})
        outs: Dict[str, Any] = {}
        host: Dict[str, np.ndarray] = {}
        for vi in self.graph.outputs:
            v = plan.outputs[vi.name]
            t = v.logical()
            if vi.name in padded:
                host[vi.name] = self._to_numpy(t)
            else:
                outs[vi.name] = t[:cut[0]] if cut is not None and t.dim() > 0 and t.shape[0] == cut[1] else t
        if host:
            torch.cuda.synchronize(self.device)
            plan.status.check("inference")
            for name, arr in host.items():
                num_name, cap = padded[name]
                counts = self._to_numpy(plan.outputs[num_name].t) if num_name in plan.outputs else \
                    self._to_numpy(plan.extra["nms"][0].out_num)
                rows = arr.reshape(len(counts), cap, -1)
                if cut is not None:
                    counts, rows = counts[:cut[0]], rows[:cut[0]]
                outs[name] = np.concatenate([rows[i, :counts[i]] for i in range(len(counts))], 0) \
                    if len(counts) else rows.reshape(0, rows.shape[-1])
        return outs

    # ------------------------------------------------------------------ zero-copy API
    def bind_input_tensor(self, name: str, tensor) -> None:
        self._bound_inputs[name] = tensor

    def bind_output_tensor(self, name: str, tensor) -> None:
        self._bound_outputs[name] = tensor

    def zero_copy_infer(self) -> None:
        outs = self._infer_dict(self._bound_inputs)
        self._last_outputs = outs
        for name, dst in self._bound_outputs.items():
            src = outs[name]
            src = torch.from_numpy(src) if isinstance(src, np.ndarray) else src
            dst.copy_(src.reshape(dst.shape))
        if self.on_gpu:
            self._check_status()

    def get_output_tensor(self, name: str):
        return self._last_outputs.get(name)

    def compile(self, warm_datas) -> bool:
        """Pre-builds plans for the given sample inputs (the reference compiles TorchScript
        through Poros here, fastdeploy/runtime/runtime.cc:430-449)."""
        for sample in warm_datas:
            self.infer(sample)
        return True

    def get_profile_time(self) -> float:
        return self._profile_time

    def export_trace(self, shapes: Dict[str, Sequence[int]], path: str = "", iters: int = 3) -> Dict[str, Any]:
        """Per-step device timeline of the plan for ``shapes`` as a Chrome-trace JSON document (see ``Plan.trace``)."""
        if not self.on_gpu:
            raise RuntimeError("export_trace needs the GPU back end")
        with torch.cuda.device(self.device):
            return self._plan_for(shapes).trace(path, iters)

    def clone(self, stream=None, device_id: int = -1) -> "Runtime":
        opt = self.option.clone()
        if device_id >= 0:
            opt.device_id = device_id
        if stream is not None:
            opt.external_stream = stream
        return Runtime(opt, _graph=self.graph)
