"""Python front of the plan runner (``libfdb200_runner.so``, csrc/runner/plan_runner.cu): loads a plan file written by
``Runtime.export_plan`` and replays it without importing, optimising or lowering the model again - a process that
only serves one exported shape starts in the time it takes to read the file and upload the constants. The same C
functions serve C programs (csrc/runner/fd_plan_runner.h); the reference's counterpart is loading a serialised
engine instead of rebuilding it (fastdeploy/runtime/backends/tensorrt/trt_backend.cc:61-114).

Inputs and outputs are numpy arrays in the plan tensors' own dimension order and type (an fp16 image plan takes
``[N, H, W, 3]`` float16); bfloat16 tensors travel as uint16 bit patterns.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional, Sequence, Union

import numpy as np

_DTYPES = {0: np.float16, 1: np.uint16, 2: np.float32, 3: np.uint8, 4: np.int32, 5: np.int64, 6: np.uint8, 7: np.int8,
           8: np.bool_}
DTYPE_NAMES = {0: "float16", 1: "bfloat16", 2: "float32", 3: "uint8", 4: "int32", 5: "int64", 6: "float8_e4m3", 7: "int8",
               8: "bool"}


class PlanTensorInfo:
    def __init__(self, name: str, dtype_code: int, shape: List[int], nbytes: int):
        self.name, self.dtype_code, self.shape, self.nbytes = name, dtype_code, shape, nbytes
        self.dtype = DTYPE_NAMES.get(dtype_code, "unknown")

    def __repr__(self) -> str:
        return f"PlanTensorInfo({self.name!r}, {self.dtype}, {self.shape})"


class PlanRunner:
    def __init__(self, plan_file: str, kernels_lib: Optional[str] = None, runner_lib: Optional[str] = None):
        from .. import _native
        from .._native import build
        self._lib = ctypes.CDLL(runner_lib or build.RUNNER_LIB)
        lib = self._lib
        P = ctypes.c_void_p
        lib.fdplan_load.restype = P
        lib.fdplan_load.argtypes = [ctypes.c_char_p, ctypes.c_char_p]
        lib.fdplan_last_error.restype = ctypes.c_char_p
        lib.fdplan_io_name.restype = ctypes.c_char_p
        lib.fdplan_io_name.argtypes = [P, ctypes.c_int, ctypes.c_int]
        lib.fdplan_io_bytes.restype = ctypes.c_ulonglong
        lib.fdplan_io_bytes.argtypes = [P, ctypes.c_int, ctypes.c_int]
        lib.fdplan_io_desc.argtypes = [P, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_int),
                                       ctypes.POINTER(ctypes.c_longlong)]
        for fn in ("fdplan_num_ops", "fdplan_num_inputs", "fdplan_num_outputs", "fdplan_run", "fdplan_destroy"):
            getattr(lib, fn).argtypes = [P]
        lib.fdplan_set_input.argtypes = [P, ctypes.c_int, P, ctypes.c_ulonglong]
        lib.fdplan_get_output.argtypes = [P, ctypes.c_int, P, ctypes.c_ulonglong]
        lib.fdplan_time.restype = ctypes.c_double
        lib.fdplan_time.argtypes = [P, ctypes.c_int]
        if not os.path.exists(plan_file):
            raise FileNotFoundError(plan_file)
        self._h = lib.fdplan_load(plan_file.encode(), (kernels_lib or _native.KERNEL_LIB).encode())
        if not self._h:
            raise RuntimeError(f"cannot load {plan_file}: {lib.fdplan_last_error().decode()}")
        self.num_ops = lib.fdplan_num_ops(self._h)
        self.inputs = [self._info(0, k) for k in range(lib.fdplan_num_inputs(self._h))]
        self.outputs = [self._info(1, k) for k in range(lib.fdplan_num_outputs(self._h))]

    def _info(self, is_output: int, k: int) -> PlanTensorInfo:
        dt, dims = ctypes.c_int(), (ctypes.c_longlong * 8)()
        nd = self._lib.fdplan_io_desc(self._h, is_output, k, ctypes.byref(dt), dims)
        return PlanTensorInfo(self._lib.fdplan_io_name(self._h, is_output, k).decode(), dt.value, list(dims[:nd]),
                              int(self._lib.fdplan_io_bytes(self._h, is_output, k)))

    def _fail(self, what: str):
        raise RuntimeError(f"{what}: {self._lib.fdplan_last_error().decode()}")

    def _index(self, infos: List[PlanTensorInfo], key: Union[int, str]) -> int:
        if isinstance(key, str):
            for k, t in enumerate(infos):
                if t.name == key:
                    return k
            raise KeyError(key)
        return int(key)

    # ------------------------------------------------------------------ one step
    def set_input(self, key: Union[int, str], array: np.ndarray) -> None:
        k = self._index(self.inputs, key)
        info = self.inputs[k]
        want = _DTYPES[info.dtype_code]
        a = np.ascontiguousarray(array)
        if a.dtype != want:
            if info.dtype_code == 1:
                raise TypeError(f"input {info.name!r} is bfloat16: pass its bit patterns as uint16")
            a = a.astype(want)
        if a.nbytes != info.nbytes:
            raise ValueError(f"input {info.name!r} takes shape {info.shape} ({info.nbytes} bytes), got {list(a.shape)}")
        if self._lib.fdplan_set_input(self._h, k, a.ctypes.data, a.nbytes) != 0:
            self._fail(f"set_input({info.name})")

    def run(self) -> None:
        if self._lib.fdplan_run(self._h) != 0:
            self._fail("run")

    def get_output(self, key: Union[int, str]) -> np.ndarray:
        k = self._index(self.outputs, key)
        info = self.outputs[k]
        out = np.empty(info.shape, _DTYPES[info.dtype_code])
        if self._lib.fdplan_get_output(self._h, k, out.ctypes.data, out.nbytes) != 0:
            self._fail(f"get_output({info.name})")
        return out

    def infer(self, feeds: Union[Dict[str, np.ndarray], Sequence[np.ndarray]]) -> List[np.ndarray]:
        items = feeds.items() if isinstance(feeds, dict) else enumerate(feeds)
        for key, arr in items:
            self.set_input(key, arr)
        self.run()
        return [self.get_output(k) for k in range(len(self.outputs))]

    def time(self, iters: int = 20) -> float:
        """Milliseconds per replay over ``iters`` launches (device events on the plan's own stream)."""
        ms = float(self._lib.fdplan_time(self._h, int(iters)))
        if ms < 0:
            self._fail("time")
        return ms

    # ------------------------------------------------------------------ lifetime
    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.fdplan_destroy(self._h)
            self._h = None

    def __enter__(self) -> "PlanRunner":
        return self

    def __exit__(self, *exc) -> None:
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
