"""First-layer 3x3 stride-2 convolution on CUDA cores (csrc/kernels/stem_conv.cu).

A 3-channel stem has K = 27: on the tensor-core path almost every multiplied value is padding, and
the layer is memory bound anyway. This op reads the 8-channel NHWC rows directly and keeps the
weights in the kernel's parameter block. The reference leaves the layer to its inference back ends
(fastdeploy/runtime/backends/), so there is no counterpart kernel there.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import numpy as np
import torch

from .. import _native
from .base import ACT, NativeOp, dtype_code

COUT = 32
MAX_CIN = 3


class _StemDesc(ctypes.Structure):
    _fields_ = [
        ("x", ctypes.c_void_p), ("y", ctypes.c_void_p), ("status", ctypes.c_void_p), ("dtype", ctypes.c_int),
        ("N", ctypes.c_int), ("H", ctypes.c_int), ("W", ctypes.c_int), ("Ho", ctypes.c_int), ("Wo", ctypes.c_int),
        ("x_ld", ctypes.c_int), ("y_ld", ctypes.c_int),
        ("x_n_stride", ctypes.c_longlong), ("y_n_stride", ctypes.c_longlong),
        ("act", ctypes.c_int), ("cin", ctypes.c_int),
        ("w", ctypes.c_float * (9 * MAX_CIN * COUT)), ("bias", ctypes.c_float * COUT),
    ]


def eligible(cout: int, cin: int, kh: int, kw: int, stride: int, pads, act: Optional[str], dtype: torch.dtype) -> bool:
    """True when :class:`StemConv` covers the layer exactly."""
    return (cout == COUT and 1 <= cin <= MAX_CIN and kh == 3 and kw == 3 and stride == 2
            and tuple(pads) == (1, 1, 1, 1) and ACT.get(act, -1) in (0, 1, 2)
            and dtype in (torch.float16, torch.bfloat16))


class StemConv(NativeOp):
    """``y = act(conv3x3_s2_p1(x, w) + bias)`` for NHWC ``x [N,H,W,8]`` (first ``cin`` channels used)."""

    def __init__(self, x: torch.Tensor, weight: np.ndarray, y: torch.Tensor, *, n: int, h: int, w: int,
                 bias: Optional[np.ndarray] = None, act: Optional[str] = None, x_ld: Optional[int] = None,
                 y_ld: Optional[int] = None, x_n_stride: int = 0, y_n_stride: int = 0, name: str = "stem_conv"):
        cout, cin, kh, kw = weight.shape
        assert (cout, kh, kw) == (COUT, 3, 3) and 1 <= cin <= MAX_CIN
        lib = _native.kernels()
        lib.fdb_stem_conv_create.restype = ctypes.c_void_p
        lib.fdb_stem_conv_create.argtypes = [ctypes.POINTER(_StemDesc)]
        d = _StemDesc()
        d.x, d.y, d.status = x.data_ptr(), y.data_ptr(), None
        d.dtype = dtype_code(x.dtype)
        ho, wo = (h - 1) // 2 + 1, (w - 1) // 2 + 1
        d.N, d.H, d.W, d.Ho, d.Wo = n, h, w, ho, wo
        d.x_ld = x_ld if x_ld is not None else x.shape[-1]
        d.y_ld = y_ld if y_ld is not None else y.shape[-1]
        d.x_n_stride = x_n_stride or h * w * d.x_ld
        d.y_n_stride = y_n_stride or ho * wo * d.y_ld
        d.act, d.cin = ACT[act], cin
        wk = np.zeros((3, 3, MAX_CIN, COUT), dtype=np.float32)
        wk[:, :, :cin, :] = np.asarray(weight, dtype=np.float32).transpose(2, 3, 1, 0)
        ctypes.memmove(d.w, wk.ctypes.data, wk.nbytes)
        b = np.zeros(COUT, dtype=np.float32) if bias is None else np.asarray(bias, dtype=np.float32).reshape(COUT)
        ctypes.memmove(d.bias, np.ascontiguousarray(b).ctypes.data, b.nbytes)
        super().__init__(lib.fdb_stem_conv_create(ctypes.byref(d)), [x, y], name)
        self.create = ("fdb_stem_conv_create", None, d)
        self.out_hw = (ho, wo)
