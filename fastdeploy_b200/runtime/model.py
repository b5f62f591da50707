"""``FastDeployModel``: base class of every model wrapper
(fastdeploy/fastdeploy_model.h:21-160, fastdeploy_model.cc:453-516): owns a ``Runtime``,
records per-call runtime durations on request and prints their statistics with the
first fifth treated as warm-up."""
from __future__ import annotations

import time
from typing import Any, Dict, List, Optional

import numpy as np

from ..core.types import Backend, Device, ModelFormat
from ..utils import log
from .option import RuntimeOption
from .runtime import Runtime


class _Flag(int):
    """A truth value that can also be called: the reference's Python class has ``initialized`` as a property and its C++
    class as a method, and code written for either reads correctly."""

    def __call__(self) -> bool:
        return bool(self)

    def __repr__(self) -> str:
        return repr(bool(self))


class FastDeployModel:
    valid_cpu_backends: List[Backend] = [Backend.ORT, Backend.PDINFER, Backend.OPENVINO, Backend.NATIVE]
    valid_gpu_backends: List[Backend] = [Backend.ORT, Backend.TRT, Backend.PDINFER, Backend.NATIVE]

    def __init__(self, runtime_option: Optional[RuntimeOption] = None):
        self.runtime_option = runtime_option.clone() if runtime_option is not None else RuntimeOption()
        self.runtime: Optional[Runtime] = None
        self.initialized_ = False
        self._record_time = False
        self._time_of_runtime: List[float] = []

    def model_name(self) -> str:
        return type(self).__name__

    ModelName = model_name

    def init_runtime(self) -> bool:
        self.runtime = Runtime(self.runtime_option)
        self.initialized_ = True
        return True

    @property
    def initialized(self) -> _Flag:
        return _Flag(bool(self.initialized_))

    def num_inputs_of_runtime(self) -> int:
        return self.runtime.num_inputs()

    def num_outputs_of_runtime(self) -> int:
        return self.runtime.num_outputs()

    def input_info_of_runtime(self, index: int):
        return self.runtime.get_input_info(index)

    def output_info_of_runtime(self, index: int):
        return self.runtime.get_output_info(index)

    def infer(self, feeds: Dict[str, Any]) -> Dict[str, Any]:
        t0 = time.perf_counter() if self._record_time else 0.0
        outs = self.runtime._infer_dict(feeds)
        if self.runtime.on_gpu:
            self.runtime._check_status()      # a kernel that gave up on a bounded wait raises here, not later
        if self._record_time:
            if self.runtime.on_gpu:
                import torch
                torch.cuda.synchronize(self.runtime.device)
            if len(self._time_of_runtime) < 50000:
                self._time_of_runtime.append(time.perf_counter() - t0)
        return outs

    def enable_record_time_of_runtime(self) -> None:
        self._record_time = True

    def disable_record_time_of_runtime(self) -> None:
        self._record_time = False

    def print_statis_info_of_runtime(self) -> Dict[str, float]:
        n = len(self._time_of_runtime)
        if n < 10:
            log.warning("PrintStatisInfoOfRuntime require the runtime ran 10 times at least, "
                        f"but now you only ran {n} times.")
        warm = n // 5
        rest = self._time_of_runtime[warm:]
        avg = float(np.mean(rest)) if rest else 0.0
        print("============= Runtime Statis Info(" + self.model_name() + ") =============")
        print(f"Total iterations: {n}")
        print(f"Total time of runtime: {sum(self._time_of_runtime):.6f}s.")
        print(f"Warmup iterations: {warm}")
        print(f"Total time of runtime in warmup step: {sum(self._time_of_runtime[:warm]):.6f}s.")
        print(f"Average time of runtime exclude warmup step: {avg * 1000:.6f}ms.")
        return {"iterations": n, "warmup": warm, "avg_ms": avg * 1000}

    def get_profile_time(self) -> float:
        return self.runtime.get_profile_time()

    def clone(self):
        import copy
        m = copy.copy(self)
        m.runtime = self.runtime.clone()
        m._time_of_runtime = []
        return m
