"""``FDTensor``: owning-or-borrowing n-d buffer on CPU, pinned host memory or GPU
(fastdeploy/core/fd_tensor.h:31-205). Storage is a torch tensor (CPU / pinned / CUDA) so that
the caching allocators, DLPack and zero-copy numpy views come for free; the API keeps the
reference's method names and semantics (grow-only reallocation, external data sharing,
``CpuData`` staging, ``PrintInfo``)."""
from __future__ import annotations

from typing import List, Optional, Sequence, Union

import numpy as np
import torch

from .types import Device, FDDataType

_FD2TORCH = {FDDataType.BOOL: torch.bool, FDDataType.INT16: torch.int16, FDDataType.INT32: torch.int32,
             FDDataType.INT64: torch.int64, FDDataType.FP16: torch.float16, FDDataType.FP32: torch.float32,
             FDDataType.FP64: torch.float64, FDDataType.UINT8: torch.uint8, FDDataType.INT8: torch.int8,
             FDDataType.BF16: torch.bfloat16}
_TORCH2FD = {v: k for k, v in _FD2TORCH.items()}


class FDTensor:
    def __init__(self, name: str = ""):
        self.name = name
        self.shape: List[int] = []
        self.dtype = FDDataType.FP32
        self.device = Device.CPU
        self.device_id = -1
        self.is_pinned_memory = False
        self._buf: Optional[torch.Tensor] = None      # flat storage, may be larger than the tensor
        self._external = False

    # ------------------------------------------------------------------ construction
    @staticmethod
    def from_numpy(arr: np.ndarray, name: str = "", copy: bool = True) -> "FDTensor":
        t = FDTensor(name)
        a = np.ascontiguousarray(arr)
        t.set_data(list(a.shape), FDDataType.from_numpy(a.dtype), a) if copy else t.set_external_data(
            list(a.shape), FDDataType.from_numpy(a.dtype), torch.from_numpy(a))
        return t

    @staticmethod
    def from_torch(x: torch.Tensor, name: str = "") -> "FDTensor":
        t = FDTensor(name)
        t.set_external_data(list(x.shape), _TORCH2FD[x.dtype], x.contiguous())
        return t

    def nbytes(self) -> int:
        return self.numel() * self.dtype.size()

    Nbytes = nbytes

    def numel(self) -> int:
        return int(np.prod(self.shape)) if self.shape else (1 if self._buf is not None else 0)

    Numel = numel

    def nbytes_allocated(self) -> int:
        return 0 if self._buf is None or self._external else self._buf.numel() * self._buf.element_size()

    def _torch_device(self) -> torch.device:
        return torch.device("cuda", max(self.device_id, 0)) if self.device == Device.GPU else torch.device("cpu")

    def allocate(self, shape: Sequence[int], dtype: FDDataType, name: str = "", device: Device = Device.CPU,
                 device_id: int = -1) -> None:
        self.name = name or self.name
        if device != self.device or device_id != self.device_id:
            self._buf = None
        self.device, self.device_id = device, device_id
        self.resize(shape, dtype)

    Allocate = allocate

    def resize(self, shape: Sequence[int], dtype: Optional[FDDataType] = None) -> None:
        """Grow-only: storage is reallocated only when the request exceeds what is held."""
        dtype = dtype if dtype is not None else self.dtype
        need = int(np.prod(shape)) if len(shape) else 1
        tdt = _FD2TORCH[dtype]
        if self._external or self._buf is None or self._buf.dtype != tdt or self._buf.numel() < need:
            dev = self._torch_device()
            self._buf = torch.empty(need, dtype=tdt, device=dev)
            if self.is_pinned_memory and dev.type == "cpu" and torch.cuda.is_available():
                self._buf = self._buf.pin_memory()
            self._external = False
        self.shape, self.dtype = [int(s) for s in shape], dtype

    Resize = resize

    def set_data(self, shape: Sequence[int], dtype: FDDataType, data) -> None:
        self.resize(shape, dtype)
        src = torch.from_numpy(np.ascontiguousarray(data)) if isinstance(data, np.ndarray) else data
        self.tensor().copy_(src.reshape(self.shape))

    SetData = set_data

    def set_external_data(self, shape: Sequence[int], dtype: FDDataType, data: torch.Tensor,
                          device: Optional[Device] = None, device_id: int = -1) -> None:
        """Borrows ``data`` without copying (``SetExternalData``)."""
        self._buf = data.reshape(-1)
        self._external = True
        self.shape, self.dtype = [int(s) for s in shape], dtype
        self.device = device if device is not None else (Device.GPU if data.is_cuda else Device.CPU)
        self.device_id = device_id if device_id >= 0 else (data.device.index if data.is_cuda else -1)

    SetExternalData = set_external_data

    def stop_sharing(self) -> None:
        if self._external and self._buf is not None:
            self._buf = self._buf[:self.numel()].clone()
            self._external = False

    StopSharing = stop_sharing

    # ------------------------------------------------------------------ views
    def tensor(self) -> torch.Tensor:
        if self._buf is None:
            raise RuntimeError("FDTensor holds no data")
        return self._buf[:self.numel()].view(self.shape)

    def data(self) -> torch.Tensor:
        return self.tensor()

    Data = data
    MutableData = data

    def cpu_data(self) -> np.ndarray:
        """Host view; a device tensor is staged through a host copy first (``CpuData``)."""
        t = self.tensor()
        if t.is_cuda:
            t = t.cpu()
        if t.dtype == torch.bfloat16:
            t = t.float()
        return t.numpy()

    CpuData = cpu_data
    numpy = cpu_data

    def reshape(self, new_shape: Sequence[int]) -> bool:
        new_shape = list(new_shape)
        if -1 in new_shape:
            known = int(np.prod([d for d in new_shape if d != -1]))
            new_shape[new_shape.index(-1)] = self.numel() // max(known, 1)
        if int(np.prod(new_shape)) != self.numel():
            return False
        self.shape = [int(d) for d in new_shape]
        return True

    Reshape = reshape

    def expand_dim(self, axis: int = 0) -> None:
        self.shape.insert(axis, 1)

    ExpandDim = expand_dim

    def squeeze(self, axis: int = 0) -> None:
        assert self.shape[axis] == 1, "The dimension to squeeze must be 1."
        self.shape.pop(axis)

    Squeeze = squeeze

    def copy_buffer(self, other: "FDTensor") -> None:
        self.allocate(other.shape, other.dtype, other.name, other.device, other.device_id)
        self.tensor().copy_(other.tensor())

    def clone(self) -> "FDTensor":
        t = FDTensor(self.name)
        t.is_pinned_memory = self.is_pinned_memory
        t.copy_buffer(self)
        return t

    def to_dlpack(self):
        return torch.utils.dlpack.to_dlpack(self.tensor())

    @staticmethod
    def from_dlpack(capsule, name: str = "") -> "FDTensor":
        return FDTensor.from_torch(torch.utils.dlpack.from_dlpack(capsule), name)

    def print_info(self, prefix: str = "TensorInfo: ") -> str:
        t = self.tensor().double() if self.numel() else torch.zeros(1, dtype=torch.float64)
        msg = (f"{prefix}name={self.name}, shape={' '.join(str(s) for s in self.shape)}, buffer_size={self.nbytes()}, "
               f"dtype={self.dtype.name}, mean={float(t.mean())}, max={float(t.max())}, min={float(t.min())}")
        print(msg)
        return msg

    PrintInfo = print_info
