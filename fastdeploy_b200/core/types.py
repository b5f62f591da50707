"""Enums and small value types of the public API: ``FDDataType`` (integer values equal to
Paddle's ``VarType`` codes, fastdeploy/core/fd_type.h:24-47), ``Backend`` / ``Device`` /
``ModelFormat`` (fastdeploy/runtime/enum_variables.h:30-109) and ``TensorInfo``
(fastdeploy/runtime/backends/backend.h:31-49)."""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import List

import numpy as np


class FDDataType(enum.IntEnum):
    BOOL = 0
    INT16 = 1
    INT32 = 2
    INT64 = 3
    FP16 = 4
    FP32 = 5
    FP64 = 6
    UNKNOWN1 = 7
    UNKNOWN2 = 8
    UINT8 = 20
    INT8 = 21
    BF16 = 22       # extension of this runtime
    FP8E4M3 = 32    # extension of this runtime

    @staticmethod
    def from_numpy(dt) -> "FDDataType":
        return _NP2FD[np.dtype(dt).name]

    def to_numpy(self):
        return np.dtype(_FD2NP[self])

    def size(self) -> int:
        return {0: 1, 1: 2, 2: 4, 3: 8, 4: 2, 5: 4, 6: 8, 20: 1, 21: 1, 22: 2, 32: 1}[int(self)]


_NP2FD = {"bool": FDDataType.BOOL, "int16": FDDataType.INT16, "int32": FDDataType.INT32, "int64": FDDataType.INT64,
          "float16": FDDataType.FP16, "float32": FDDataType.FP32, "float64": FDDataType.FP64, "uint8": FDDataType.UINT8,
          "int8": FDDataType.INT8}
_FD2NP = {v: k for k, v in _NP2FD.items()}


class Backend(enum.IntEnum):
    """Every selector of the reference is accepted; all of them resolve to the native
    backend on GPU and to the reference interpreter on CPU."""
    UNKNOWN = 0
    ORT = 1
    TRT = 2
    PDINFER = 3
    POROS = 4
    OPENVINO = 5
    LITE = 6
    RKNPU2 = 7
    SOPHGOTPU = 8
    HORIZONNPU = 9
    TVM = 10
    NATIVE = 100


class Device(enum.IntEnum):
    CPU = 0
    GPU = 1
    RKNPU = 2
    IPU = 3
    TIMVX = 4
    KUNLUNXIN = 5
    ASCEND = 6
    SOPHGOTPUD = 7
    DIRECTML = 8
    SUNRISENPU = 9


class ModelFormat(enum.IntEnum):
    AUTOREC = 0
    PADDLE = 1
    ONNX = 2
    RKNN = 3
    TORCHSCRIPT = 4
    SOPHGO = 5
    HORIZON = 6
    TVMFormat = 7


@dataclass
class TensorInfo:
    name: str = ""
    shape: List[int] = field(default_factory=list)
    dtype: FDDataType = FDDataType.FP32

    def __repr__(self) -> str:
        return f"TensorInfo(name: {self.name}, shape: {self.shape}, dtype: {self.dtype.name})"


# Which back ends can serve a model format / a device (fastdeploy/runtime/enum_variables.h:82-108). Every selector the
# reference knows is accepted; on this build they all resolve to the native sm_100a executor on a GPU and to the
# reference interpreter on the CPU, so the tables list those two routes under the names a user may ask for.
DEFAULT_BACKENDS_BY_FORMAT = {
    "PADDLE": ["PDINFER", "ORT", "TRT", "NATIVE"],
    "ONNX": ["ORT", "TRT", "NATIVE"],
}
DEFAULT_BACKENDS_BY_DEVICE = {
    "CPU": ["PDINFER", "ORT", "OPENVINO", "NATIVE"],
    "GPU": ["PDINFER", "ORT", "TRT", "NATIVE"],
}


def get_available_backends() -> List["Backend"]:
    """Back ends a ``RuntimeOption`` may select (fastdeploy/runtime/enum_variables.cc:101-134)."""
    return [Backend.ORT, Backend.TRT, Backend.PDINFER, Backend.OPENVINO, Backend.NATIVE]


def is_backend_available(backend) -> bool:
    return Backend(backend) in get_available_backends()


def supported(format_or_device, backend) -> bool:
    """``Supported(format, backend)`` / ``Supported(device, backend)`` of the reference."""
    name = getattr(format_or_device, "name", str(format_or_device)).upper()
    table = DEFAULT_BACKENDS_BY_FORMAT.get(name) or DEFAULT_BACKENDS_BY_DEVICE.get(name)
    return table is not None and Backend(backend).name in table
