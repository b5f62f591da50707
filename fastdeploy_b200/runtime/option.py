"""``RuntimeOption`` with the reference's method surface
(python/fastdeploy/runtime.py:160-713, fastdeploy/runtime/runtime_option.h:41-289).

Every backend selector of the reference is accepted and resolves to the single native
backend (GPU) or the reference interpreter (CPU); vendor-specific knobs are stored,
logged once and otherwise ignored. Options that only this runtime has live in
``native_option``.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from ..core.types import Backend, Device, ModelFormat
from ..utils import log


@dataclass
class NativeOption:
    """Knobs of the sm_100a backend."""
    precision: str = "fp16"            # fp16 | bf16 | fp8 (bf16 activations, e4m3 operands with per-channel / per-token scales in the linear layers)
    use_cuda_graph: bool = True
    opt_level: int = 2
    max_plans: int = 8                 # shape buckets kept alive
    batch_buckets: List[int] = field(default_factory=list)   # batch sizes plans are built for: a batch runs padded in the smallest one that holds it
    quant_scales_file: str = ""        # calibrated activation ranges for precision "fp8" (default: quant_scales.json next to the model)
    tp_degree: int = 1
    dp_gpus: List[int] = field(default_factory=list)
    plan_cache_dir: str = ""

    def apply_env(self) -> None:
        self.precision = os.environ.get("FDX_PRECISION", self.precision)
        if "FDX_CUDA_GRAPH" in os.environ:
            self.use_cuda_graph = os.environ["FDX_CUDA_GRAPH"] not in ("0", "false")
        if "FDX_OPT_LEVEL" in os.environ:
            self.opt_level = int(os.environ["FDX_OPT_LEVEL"])


@dataclass
class _VendorOption:
    """Bag of attributes for ``trt_option`` / ``ort_option`` / ... : accepts anything."""
    values: Dict[str, Any] = field(default_factory=dict)

    def __getattr__(self, k):
        if k == "values":
            raise AttributeError(k)
        return self.values.get(k)

    def __setattr__(self, k, v):
        if k == "values":
            object.__setattr__(self, k, v)
        else:
            self.values[k] = v


class RuntimeOption:
    def __init__(self):
        self.model_file = ""
        self.params_file = ""
        self.model_buffer: Optional[bytes] = None
        self.params_buffer: Optional[bytes] = None
        self.model_from_memory = False
        self.model_format = ModelFormat.PADDLE
        self.device = Device.CPU
        self.device_id = 0
        self.backend = Backend.UNKNOWN
        self.cpu_thread_num = -1
        self.encryption_key = ""
        self.enable_pinned_memory_ = False
        self.external_stream = None
        self.enable_valid_backend_check_ = True
        self.profiling = {"enable": False, "include_h2d_d2h": False, "repeat": 100, "warmup": 50}
        self.native_option = NativeOption()
        self.trt_shapes: Dict[str, Dict[str, List[int]]] = {}
        self._vendor = {k: _VendorOption() for k in ("trt", "ort", "paddle_infer", "openvino", "lite", "poros")}
        self._noted = set()

    # ------------------------------------------------------------------ model
    def set_model_path(self, model_path: str, params_path: str = "", model_format: ModelFormat = ModelFormat.PADDLE):
        self.model_file, self.params_file, self.model_format = model_path, params_path, ModelFormat(model_format)
        self.model_from_memory = False

    def set_model_buffer(self, model_buffer: bytes, params_buffer: bytes = b"",
                         model_format: ModelFormat = ModelFormat.PADDLE):
        self.model_buffer, self.params_buffer = model_buffer, params_buffer
        self.model_format = ModelFormat(model_format)
        self.model_from_memory = True

    def set_encryption_key(self, encryption_key: str):
        self.encryption_key = encryption_key

    # ------------------------------------------------------------------ device
    def use_cpu(self):
        self.device = Device.CPU

    def use_gpu(self, device_id: int = 0):
        self.device, self.device_id = Device.GPU, int(device_id)

    def _other_device(self, name: str):
        self._note(f"{name} is not a target of this runtime; falling back to CPU")
        self.device = Device.CPU

    def use_kunlunxin(self, *a, **k): self._other_device("KunlunXin")
    def use_rknpu2(self, *a, **k): self._other_device("RKNPU2")
    def use_sophgo(self): self._other_device("Sophgo")
    def use_ascend(self): self._other_device("Ascend")
    def use_timvx(self): self._other_device("TimVX")
    def use_horizon(self): self._other_device("Horizon")
    def use_directml(self): self._other_device("DirectML")
    def use_ipu(self, *a, **k): self._other_device("IPU")
    def set_ipu_config(self, *a, **k): self._note("IPU options are ignored")

    def set_cpu_thread_num(self, thread_num: int = -1):
        self.cpu_thread_num = int(thread_num)

    def set_external_raw_stream(self, cuda_stream):
        self.external_stream = cuda_stream

    set_external_stream = set_external_raw_stream

    def enable_pinned_memory(self): self.enable_pinned_memory_ = True
    def disable_pinned_memory(self): self.enable_pinned_memory_ = False
    def disable_valid_backend_check(self): self.enable_valid_backend_check_ = False
    def enable_valid_backend_check(self): self.enable_valid_backend_check_ = True

    # ------------------------------------------------------------------ backend selectors
    def _select(self, backend: Backend):
        self.backend = backend
        if backend not in (Backend.UNKNOWN, Backend.NATIVE):
            self._note(f"backend {backend.name} requested: served by the native sm_100a backend on GPU "
                       f"and by the reference interpreter on CPU")

    def use_paddle_backend(self): self._select(Backend.PDINFER)
    def use_paddle_infer_backend(self): self._select(Backend.PDINFER)
    def use_poros_backend(self): self._select(Backend.POROS)
    def use_ort_backend(self): self._select(Backend.ORT)
    def use_tvm_backend(self): self._select(Backend.TVM)
    def use_trt_backend(self): self._select(Backend.TRT)
    def use_openvino_backend(self): self._select(Backend.OPENVINO)
    def use_lite_backend(self): self._select(Backend.LITE)
    def use_paddle_lite_backend(self): self._select(Backend.LITE)
    def use_sophgo_backend(self): self._select(Backend.SOPHGOTPU)
    def use_horizon_npu_backend(self): self._select(Backend.HORIZONNPU)
    def use_native_backend(self): self._select(Backend.NATIVE)

    # ------------------------------------------------------------------ precision & shapes (TensorRT vocabulary)
    def enable_trt_fp16(self): self.native_option.precision = "fp16"
    def disable_trt_fp16(self): self.native_option.precision = "fp16"   # activations are 16-bit on this backend
    def enable_lite_fp16(self): self.native_option.precision = "fp16"
    def disable_lite_fp16(self): pass
    def enable_bf16(self): self.native_option.precision = "bf16"
    def enable_fp8(self): self.native_option.precision = "fp8"

    def set_trt_input_shape(self, tensor_name: str, min_shape, opt_shape=None, max_shape=None):
        """Shape ranges seed the plan cache: a plan is pre-built for ``opt_shape``."""
        self.trt_shapes[tensor_name] = {"min": list(min_shape), "opt": list(opt_shape or min_shape),
                                        "max": list(max_shape or opt_shape or min_shape)}

    def set_batch_buckets(self, buckets) -> None:
        """Batch sizes the native back end builds plans for (e.g. ``[1, 2, 4, 8, 16, 32]``): a batch runs, padded, in
        the smallest bucket that holds it, so a service with ragged batches builds a handful of plans instead of
        one per batch size. The TensorRT back end of the reference covers this with a min / opt / max profile
        (fastdeploy/runtime/backends/tensorrt/trt_backend.cc:327-339)."""
        self.native_option.batch_buckets = sorted(int(b) for b in buckets)

    def set_trt_input_data(self, tensor_name: str, min_data, opt_data=None, max_data=None):
        self._vendor["trt"].values.setdefault("input_data", {})[tensor_name] = (min_data, opt_data, max_data)

    def set_trt_cache_file(self, cache_file_path: str):
        self.native_option.plan_cache_dir = os.path.dirname(cache_file_path) or "."

    def set_trt_max_workspace_size(self, size): self._vendor["trt"].max_workspace_size = size
    def set_trt_max_batch_size(self, size): self._vendor["trt"].max_batch_size = size
    def enable_paddle_to_trt(self): self._note("Paddle-TRT is folded into the native backend")
    def enable_paddle_trt_collect_shape(self): pass
    def disable_paddle_trt_collect_shape(self): pass
    def delete_paddle_backend_pass(self, pass_name): self._vendor["paddle_infer"].values.setdefault("deleted", []).append(pass_name)
    def disable_paddle_trt_ops(self, ops): self._vendor["paddle_infer"].trt_disabled_ops = list(ops)
    def enable_paddle_log_info(self): self._vendor["paddle_infer"].enable_log_info = True
    def disable_paddle_log_info(self): self._vendor["paddle_infer"].enable_log_info = False
    def set_paddle_mkldnn(self, use_mkldnn=True): self._vendor["paddle_infer"].enable_mkldnn = use_mkldnn
    def set_paddle_mkldnn_cache_size(self, cache_size): self._vendor["paddle_infer"].mkldnn_cache_size = cache_size
    def set_ort_graph_opt_level(self, level=-1):
        self._vendor["ort"].graph_optimization_level = level
        if level == 0:
            self.native_option.opt_level = 0
    def set_openvino_device(self, name="CPU"): self._vendor["openvino"].device = name
    def set_openvino_shape_info(self, shape_info): self._vendor["openvino"].shape_infos = shape_info
    def set_openvino_cpu_operators(self, operators): self._vendor["openvino"].cpu_operators = operators
    def set_lite_context_properties(self, v): self._vendor["lite"].nnadapter_context_properties = v
    def set_lite_model_cache_dir(self, v): self._vendor["lite"].nnadapter_model_cache_dir = v
    def set_lite_dynamic_shape_info(self, v): self._vendor["lite"].nnadapter_dynamic_shape_info = v
    def set_lite_subgraph_partition_path(self, v): self._vendor["lite"].nnadapter_subgraph_partition_config_path = v
    def set_lite_subgraph_partition_config_buffer(self, v): self._vendor["lite"].nnadapter_subgraph_partition_config_buffer = v
    def set_lite_mixed_precision_quantization_config_path(self, v): self._vendor["lite"].nnadapter_mixed_precision_quantization_config_path = v
    def set_lite_power_mode(self, mode): self._vendor["lite"].power_mode = mode
    def set_lite_optimized_model_dir(self, v): self._vendor["lite"].optimized_model_dir = v
    def enable_lite_int8(self): self._vendor["lite"].enable_int8 = True
    def disable_lite_int8(self): self._vendor["lite"].enable_int8 = False
    def set_openvino_streams(self, num_streams): self._vendor["openvino"].num_streams = int(num_streams)

    @property
    def trt_option(self): return self._vendor["trt"]
    @property
    def ort_option(self): return self._vendor["ort"]
    @property
    def paddle_infer_option(self): return self._vendor["paddle_infer"]
    @property
    def openvino_option(self): return self._vendor["openvino"]
    @property
    def paddle_lite_option(self): return self._vendor["lite"]
    @property
    def poros_option(self): return self._vendor["poros"]

    # ------------------------------------------------------------------ profiling
    def enable_profiling(self, inclue_h2d_d2h: bool = False, repeat: int = 100, warmup: int = 50):
        """Device-timed (CUDA events) re-execution of the forward, like the reference's
        RUNTIME_PROFILE_LOOP macros (fastdeploy/benchmark/benchmark.h:21-85) but without their
        host-clock-around-an-async-launch weakness."""
        self.profiling = {"enable": True, "include_h2d_d2h": bool(inclue_h2d_d2h), "repeat": int(repeat),
                          "warmup": int(warmup)}

    def disable_profiling(self):
        self.profiling["enable"] = False

    # ------------------------------------------------------------------ misc
    def _note(self, msg: str) -> None:
        if msg not in self._noted:
            self._noted.add(msg)
            log.info(msg)

    def clone(self) -> "RuntimeOption":
        import copy
        o = copy.copy(self)
        o.native_option = copy.deepcopy(self.native_option)
        o.trt_shapes = copy.deepcopy(self.trt_shapes)
        o.profiling = dict(self.profiling)
        return o

    def __repr__(self) -> str:
        return (f"RuntimeOption(model_file={self.model_file!r}, params_file={self.params_file!r}, "
                f"model_format={self.model_format.name}, device={self.device.name}:{self.device_id}, "
                f"backend={self.backend.name}, precision={self.native_option.precision})")
