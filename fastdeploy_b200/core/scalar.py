"""``Scalar`` (a tagged single value, fastdeploy/core/fd_scalar.h:25-115) and the ue8m0 block-scale format, both
over the native core library (csrc/cpu/core.cc)."""
from __future__ import annotations

import ctypes
from typing import Union

from .. import _native
from .types import FDDataType


def _lib():
    lib = _native.cpu()
    if not getattr(lib, "_core_ready", False):
        lib.fdb_scalar_from_double.argtypes = [ctypes.c_void_p, ctypes.c_double, ctypes.c_int]
        lib.fdb_scalar_from_int64.argtypes = [ctypes.c_void_p, ctypes.c_int64]
        lib.fdb_scalar_from_string.argtypes = [ctypes.c_void_p, ctypes.c_char_p]
        lib.fdb_scalar_dtype.argtypes = [ctypes.c_void_p]
        lib.fdb_scalar_to_double.argtypes = [ctypes.c_void_p]
        lib.fdb_scalar_to_double.restype = ctypes.c_double
        lib.fdb_scalar_to_int64.argtypes = [ctypes.c_void_p]
        lib.fdb_scalar_to_int64.restype = ctypes.c_int64
        lib.fdb_ue8m0_from_float.argtypes = [ctypes.c_float]
        lib.fdb_ue8m0_from_float.restype = ctypes.c_uint8
        lib.fdb_ue8m0_to_float.argtypes = [ctypes.c_uint8]
        lib.fdb_ue8m0_to_float.restype = ctypes.c_float
        lib.fdb_timer_create.restype = ctypes.c_void_p
        for fn in (lib.fdb_timer_destroy, lib.fdb_timer_start, lib.fdb_timer_end, lib.fdb_timer_duration):
            fn.argtypes = [ctypes.c_void_p]
        lib.fdb_timer_duration.restype = ctypes.c_double
        lib._core_ready = True
    return lib


class Scalar:
    """One value with its element type. ``Scalar(3)`` is INT64, ``Scalar(2.5)`` FP64, ``Scalar(True)`` BOOL,
    ``Scalar("-inf")`` FP64; ``Scalar(1, FDDataType.FP32)`` picks the type. ``to(type)`` converts like a C++ cast."""

    def __init__(self, value: Union[bool, int, float, str] = 0, dtype: FDDataType = None):
        lib = _lib()
        self._buf = ctypes.create_string_buffer(lib.fdb_scalar_size())
        if isinstance(value, str):
            if lib.fdb_scalar_from_string(self._buf, value.encode()) != 0:
                raise ValueError(f"Scalar: {value!r} is not a number")
        elif dtype is not None:
            lib.fdb_scalar_from_double(self._buf, float(value), int(dtype))
        elif isinstance(value, bool):
            lib.fdb_scalar_from_double(self._buf, float(value), int(FDDataType.BOOL))
        elif isinstance(value, int):
            lib.fdb_scalar_from_int64(self._buf, value)
        else:
            lib.fdb_scalar_from_double(self._buf, float(value), int(FDDataType.FP64))

    @property
    def dtype(self) -> FDDataType:
        return FDDataType(_lib().fdb_scalar_dtype(self._buf))

    def to(self, kind=float):
        lib = _lib()
        if kind is int:
            return int(lib.fdb_scalar_to_int64(self._buf))
        if kind is bool:
            return lib.fdb_scalar_to_double(self._buf) != 0.0
        return float(lib.fdb_scalar_to_double(self._buf))

    def __float__(self):
        return self.to(float)

    def __int__(self):
        return self.to(int)

    def __repr__(self):
        return f"Scalar({self.to(int) if self.dtype in (FDDataType.INT64, FDDataType.INT32) else self.to(float)}, {self.dtype.name})"


def ue8m0_from_float(v: float) -> int:
    """Smallest power of two >= ``v`` as an 8-bit exponent code (value ``2^(code - 127)``; 255 = NaN)."""
    return int(_lib().fdb_ue8m0_from_float(float(v)))


def ue8m0_to_float(code: int) -> float:
    return float(_lib().fdb_ue8m0_to_float(int(code) & 0xFF))
