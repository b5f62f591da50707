"""Common Python-side handle types for native kernel objects."""
from __future__ import annotations

import ctypes
from typing import Any, List, Optional

import torch

from .. import _native

# dtype codes shared with csrc/kernels/fdb_common.h
DT_F16, DT_BF16, DT_F32, DT_U8, DT_I32, DT_I64, DT_F8E4M3, DT_I8 = range(8)

_TORCH_TO_CODE = {
    torch.float16: DT_F16,
    torch.bfloat16: DT_BF16,
    torch.float32: DT_F32,
    torch.uint8: DT_U8,
    torch.int32: DT_I32,
    torch.int64: DT_I64,
    torch.int8: DT_I8,
}
if hasattr(torch, "float8_e4m3fn"):
    _TORCH_TO_CODE[torch.float8_e4m3fn] = DT_F8E4M3

# activation codes shared with csrc/kernels/fdb_common.h
ACT = {
    None: 0, "none": 0, "identity": 0, "relu": 1, "silu": 2, "swish": 2, "hard_swish": 3, "hardswish": 3,
    "hard_sigmoid": 4, "hardsigmoid": 4, "sigmoid": 5, "gelu": 6, "relu6": 7, "leaky_relu": 8, "tanh": 9,
}


def dtype_code(dt: torch.dtype) -> int:
    return _TORCH_TO_CODE[dt]


def current_stream_ptr(device: Optional[torch.device] = None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


class NativeOp:
    """Owns one native ``fdb::Op``; keeps the tensors it points at alive."""

    def __init__(self, handle: int, keep: List[Any], name: str = ""):
        if not handle:
            raise RuntimeError(f"{name or 'native op'}: {_native.last_error()}")
        self.handle = ctypes.c_void_p(handle)
        self.keep = keep
        self.name = name
        # (creation function, kind argument or None, descriptor): what a plan file needs to re-create this op in a
        # process without Python (runtime/plan_file.py); filled in by the wrappers that build the descriptor
        self.create: Optional[tuple] = None

    def launch(self, stream: Optional[int] = None) -> None:
        s = current_stream_ptr() if stream is None else stream
        rc = _native.kernels().fdb_op_launch(self.handle, ctypes.c_void_p(s))
        if rc != 0:
            raise RuntimeError(f"{self.name}: launch failed: {_native.last_error()}")

    __call__ = launch

    def __del__(self):
        try:
            if self.handle:
                _native.kernels().fdb_op_destroy(self.handle)
                self.handle = None
        except Exception:
            pass


class StatusWord:
    """Device int that kernels write a non-zero code to instead of trapping or hanging."""

    MESSAGES = {
        1: "TMA producer wait timed out",
        2: "MMA issuer wait timed out",
        3: "epilogue wait timed out",
        4: "peer signal wait timed out",
        5: "bad shape",
    }

    def __init__(self, device):
        self.t = torch.zeros(1, dtype=torch.int32, device=device)

    @property
    def ptr(self) -> int:
        return self.t.data_ptr()

    def check(self, what: str = "kernel") -> None:
        """Blocking read of the device word (waits for everything queued on the current stream)."""
        v = int(self.t.item())
        if v != 0:
            self.t.zero_()
            raise RuntimeError(f"{what}: device status {v} ({self.MESSAGES.get(v, 'unknown')})")

    def snapshot_async(self, host: torch.Tensor) -> None:
        """Queues a copy of the word into pinned ``host`` (int32[1]) on the current stream. A pipelined
        caller reads it with :meth:`check_snapshot` once its own completion event has fired, so that
        checking one batch never waits for the batches queued behind it."""
        host.copy_(self.t, non_blocking=True)

    def check_snapshot(self, host: torch.Tensor, what: str = "kernel") -> None:
        v = int(host[0])
        if v != 0:
            self.t.zero_()
            raise RuntimeError(f"{what}: device status {v} ({self.MESSAGES.get(v, 'unknown')})")
