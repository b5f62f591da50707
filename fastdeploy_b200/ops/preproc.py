"""Fused GPU image pre-processing (csrc/kernels/preproc.cu).

Replaces the reference's processor chain on GPU - Resize, Pad/PadToSize/StridePad,
Normalize, HWC2CHW, Cast (fastdeploy/vision/common/processors/*.cc, normalize_and_permute.cu:21-40,
fastdeploy/vision/utils/yolo_preprocess.cu:37-113) - with one launch per batch.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import _native
from .base import NativeOp, dtype_code

INTERP = {"nearest": 0, "linear": 1, "bilinear": 1, "cubic": 2, "bicubic": 2, 0: 0, 1: 1, 2: 2}

# numpy mirror of struct PreprocImage (48 bytes)
IMAGE_META = np.dtype([("src_offset", "<i8"), ("src_h", "<i4"), ("src_w", "<i4"), ("src_stride", "<i4"),
                       ("dst_top", "<i4"), ("dst_left", "<i4"), ("rh", "<i4"), ("rw", "<i4"),
                       ("sx", "<f4"), ("sy", "<f4"), ("pad0", "<i4")], align=False)
assert IMAGE_META.itemsize == 48


class _PreprocDesc(ctypes.Structure):
    _fields_ = [
        ("src", ctypes.c_void_p), ("meta", ctypes.c_void_p), ("dst", ctypes.c_void_p),
        ("N", ctypes.c_int), ("Ho", ctypes.c_int), ("Wo", ctypes.c_int), ("c_out", ctypes.c_int),
        ("interp", ctypes.c_int), ("layout", ctypes.c_int), ("out_dtype", ctypes.c_int), ("swap_rb", ctypes.c_int),
        ("round_u8", ctypes.c_int),
        ("alpha", ctypes.c_float * 3), ("beta", ctypes.c_float * 3), ("pad", ctypes.c_float * 3),
    ]


def _lib():
    lib = _native.kernels()
    if not getattr(lib, "_preproc_ready", False):
        lib.fdb_preproc_create.restype = ctypes.c_void_p
        lib.fdb_preproc_create.argtypes = [ctypes.POINTER(_PreprocDesc)]
        assert lib.fdb_preproc_image_size() == IMAGE_META.itemsize
        lib._preproc_ready = True
    return lib


def normalize_coeffs(mean: Sequence[float], std: Sequence[float], is_scale: bool = True,
                     min_v: Sequence[float] = (0.0, 0.0, 0.0), max_v: Sequence[float] = (255.0, 255.0, 255.0)):
    """alpha/beta of the reference's Normalize (fastdeploy/vision/common/processors/normalize.cc:23-55)."""
    alpha, beta = [], []
    for c in range(3):
        a = 1.0 / (max_v[c] - min_v[c]) if is_scale else 1.0
        b = -min_v[c] * a if is_scale else 0.0
        alpha.append(a / std[c])
        beta.append((b - mean[c]) / std[c])
    return alpha, beta


def fill_meta(meta: np.ndarray, i: int, *, src_offset: int, src_hw: Tuple[int, int], src_stride: int,
              resized_hw: Tuple[int, int], top_left: Tuple[int, int] = (0, 0)) -> None:
    m = meta[i]
    m["src_offset"] = src_offset
    m["src_h"], m["src_w"], m["src_stride"] = src_hw[0], src_hw[1], src_stride
    m["dst_top"], m["dst_left"] = top_left
    m["rh"], m["rw"] = resized_hw
    m["sx"] = src_hw[1] / resized_hw[1]
    m["sy"] = src_hw[0] / resized_hw[0]


class Preprocess(NativeOp):
    """Planned pre-processing launch over fixed ``src`` (uint8 bytes), ``meta`` and ``dst`` buffers."""

    def __init__(self, src: torch.Tensor, meta: torch.Tensor, dst: torch.Tensor, *, n: int, out_hw: Tuple[int, int],
                 layout: str = "nhwc", c_out: int = 3, interp="linear", swap_rb: bool = False,
                 alpha: Sequence[float] = (1.0, 1.0, 1.0), beta: Sequence[float] = (0.0, 0.0, 0.0),
                 pad_value: Sequence[float] = (0.0, 0.0, 0.0), round_u8: bool = True):
        d = _PreprocDesc()
        d.src, d.meta, d.dst = src.data_ptr(), meta.data_ptr(), dst.data_ptr()
        d.N, d.Ho, d.Wo, d.c_out = n, out_hw[0], out_hw[1], c_out if layout == "nhwc" else 3
        d.interp, d.layout, d.out_dtype = INTERP[interp], 0 if layout == "nhwc" else 1, dtype_code(dst.dtype)
        d.swap_rb, d.round_u8 = int(swap_rb), int(round_u8)
        for c in range(3):
            d.alpha[c], d.beta[c], d.pad[c] = alpha[c], beta[c], pad_value[c]
        super().__init__(_lib().fdb_preproc_create(ctypes.byref(d)), [src, meta, dst], "preprocess")
        self.create = ("fdb_preproc_create", None, d)
