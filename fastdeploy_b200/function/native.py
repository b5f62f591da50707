"""ctypes front of the native host function library (csrc/cpu/functions.cc): numpy arrays of any layout go in as
strided views, results come back as fresh contiguous arrays. ``usable(*arrays)`` says whether the native path takes
the operands (host arrays of bool / uint8 / int8 / int32 / int64 / float32 / float64, at most 8 dimensions)."""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence, Tuple

import numpy as np

from .. import _native

MAX_DIMS = 8
_CODES = {np.dtype(np.bool_): 0, np.dtype(np.uint8): 1, np.dtype(np.int8): 2, np.dtype(np.int32): 3,
          np.dtype(np.int64): 4, np.dtype(np.float32): 5, np.dtype(np.float64): 6}
UNARY = {"clip": 0, "sqrt": 1, "log": 2, "round": 3, "exp": 4, "abs": 5, "ceil": 6, "floor": 7, "isnan": 8, "isinf": 9,
         "isfinite": 10}
BINARY = {"add": 0, "subtract": 1, "multiply": 2, "divide": 3, "maximum": 4, "minimum": 5}
REDUCE = {"sum": 0, "mean": 1, "max": 2, "min": 3, "prod": 4, "all": 5, "any": 6}


class _FnTensor(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("dtype", ctypes.c_int), ("ndim", ctypes.c_int),
                ("shape", ctypes.c_longlong * MAX_DIMS), ("strides", ctypes.c_longlong * MAX_DIMS)]


_lib_ready = None


def _lib():
    global _lib_ready
    if _lib_ready is None:
        lib = _native.cpu()
        if lib.fdf_tensor_size() != ctypes.sizeof(_FnTensor):
            raise _native.NativeLibraryError("libfdb200_cpu.so is out of date: FnTensor layout differs")
        P = ctypes.POINTER(_FnTensor)
        lib.fdf_copy.argtypes = [P, P]
        lib.fdf_fill.argtypes = [P, ctypes.c_double]
        lib.fdf_unary.argtypes = [ctypes.c_int, P, P, ctypes.c_double, ctypes.c_double]
        lib.fdf_binary.argtypes = [ctypes.c_int, P, P, P]
        lib.fdf_reduce.argtypes = [ctypes.c_int, P, P, ctypes.c_uint]
        lib.fdf_arg_extreme.argtypes = [ctypes.c_int, P, P, ctypes.c_int]
        lib.fdf_scan.argtypes = [ctypes.c_int, P, P, ctypes.c_int]
        lib.fdf_sort.argtypes = [P, P, P, ctypes.c_int, ctypes.c_int]
        lib.fdf_along_axis.argtypes = [ctypes.c_int, P, P, P, ctypes.c_int]
        lib.fdf_quantile.argtypes = [P, P, ctypes.c_int, ctypes.POINTER(ctypes.c_double), ctypes.c_int]
        lib.fdb_cpu_last_error.restype = ctypes.c_char_p
        _lib_ready = lib
    return _lib_ready


def usable(*arrays) -> bool:
    if not _native.cpu_available():
        return False
    return all(isinstance(a, np.ndarray) and a.dtype in _CODES and a.ndim <= MAX_DIMS for a in arrays)


def _view(a: np.ndarray) -> _FnTensor:
    t = _FnTensor()
    t.data = a.ctypes.data if a.size else None
    t.dtype, t.ndim = _CODES[a.dtype], a.ndim
    for d in range(a.ndim):
        t.shape[d] = a.shape[d]
        t.strides[d] = a.strides[d] // a.itemsize if a.shape[d] > 1 else 0
    return t


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise ValueError(f"{what}: {_lib().fdb_cpu_last_error().decode()}")


def copy(src: np.ndarray, dst: np.ndarray) -> np.ndarray:
    """``dst[...] = src[...]`` for two views of one shape (any layouts, any supported dtypes)."""
    _check(_lib().fdf_copy(ctypes.byref(_view(src)), ctypes.byref(_view(dst))), "copy")
    return dst


def materialise(view: np.ndarray, dtype=None) -> np.ndarray:
    """A contiguous array with the contents of ``view`` (a transpose, a slice, a broadcast ...)."""
    return copy(view, np.empty(view.shape, dtype or view.dtype))


def fill(shape: Sequence[int], value: float, dtype) -> np.ndarray:
    out = np.empty(tuple(shape), dtype)
    _check(_lib().fdf_fill(ctypes.byref(_view(out)), float(value)), "fill")
    return out


def unary(op: str, x: np.ndarray, out_dtype=None, a: float = 0.0, b: float = 0.0) -> np.ndarray:
    out = np.empty(x.shape, out_dtype or x.dtype)
    _check(_lib().fdf_unary(UNARY[op], ctypes.byref(_view(x)), ctypes.byref(_view(out)), a, b), op)
    return out


def binary(op: str, a: np.ndarray, b: np.ndarray, out_dtype=None) -> np.ndarray:
    shape = np.broadcast_shapes(a.shape, b.shape)
    out = np.empty(shape, out_dtype or np.result_type(a.dtype, b.dtype))
    av, bv = np.broadcast_to(a, shape), np.broadcast_to(b, shape)
    _check(_lib().fdf_binary(BINARY[op], ctypes.byref(_view(av)), ctypes.byref(_view(bv)), ctypes.byref(_view(out))), op)
    return out


def reduce(op: str, x: np.ndarray, axes: Sequence[int], keep_dim: bool, out_dtype) -> np.ndarray:
    axes = sorted({a % x.ndim for a in axes}) if x.ndim else []
    kept = [1 if d in axes else x.shape[d] for d in range(x.ndim)]
    out = np.empty(kept, out_dtype)
    mask = 0
    for a in axes:
        mask |= 1 << a
    _check(_lib().fdf_reduce(REDUCE[op], ctypes.byref(_view(x)), ctypes.byref(_view(out)), mask), op)
    return out if keep_dim else out.reshape([x.shape[d] for d in range(x.ndim) if d not in axes])


def arg_extreme(want_max: bool, x: np.ndarray, axis: int, keep_dim: bool, out_dtype) -> np.ndarray:
    axis %= x.ndim
    kept = [1 if d == axis else x.shape[d] for d in range(x.ndim)]
    out = np.empty(kept, out_dtype)
    _check(_lib().fdf_arg_extreme(int(want_max), ctypes.byref(_view(x)), ctypes.byref(_view(out)), axis), "arg")
    return out if keep_dim else out.reshape([x.shape[d] for d in range(x.ndim) if d != axis])


def scan(mode: str, x: np.ndarray, axis: int) -> np.ndarray:
    out = np.empty(x.shape, x.dtype)
    _check(_lib().fdf_scan({"softmax": 0, "cumprod": 1}[mode], ctypes.byref(_view(x)), ctypes.byref(_view(out)),
                           axis % x.ndim), mode)
    return out


def sort(x: np.ndarray, axis: int, descending: bool) -> Tuple[np.ndarray, np.ndarray]:
    vals, idx = np.empty(x.shape, x.dtype), np.empty(x.shape, np.int64)
    _check(_lib().fdf_sort(ctypes.byref(_view(x)), ctypes.byref(_view(vals)), ctypes.byref(_view(idx)), axis % x.ndim,
                           int(descending)), "sort")
    return vals, idx


def gather(x: np.ndarray, index: np.ndarray, axis: int) -> np.ndarray:
    out = np.empty(index.shape, x.dtype)
    _check(_lib().fdf_along_axis(0, ctypes.byref(_view(x)), ctypes.byref(_view(index)), ctypes.byref(_view(out)),
                                 axis % x.ndim), "gather_along_axis")
    return out


def scatter(x: np.ndarray, index: np.ndarray, values: np.ndarray, axis: int) -> np.ndarray:
    out = materialise(x)
    vals = np.broadcast_to(values, index.shape)
    _check(_lib().fdf_along_axis(1, ctypes.byref(_view(out)), ctypes.byref(_view(index)), ctypes.byref(_view(vals)),
                                 axis % x.ndim), "scatter_along_axis")
    return out


def quantile(x: np.ndarray, q: Sequence[float], axis: int, out_dtype) -> np.ndarray:
    """Quantiles along ``axis``; the result has the quantile index as its FIRST dimension and ``axis`` removed."""
    axis %= x.ndim
    shape = [len(q) if d == axis else x.shape[d] for d in range(x.ndim)]
    out = np.empty(shape, out_dtype)
    qs = (ctypes.c_double * len(q))(*[float(v) for v in q])
    _check(_lib().fdf_quantile(ctypes.byref(_view(x)), ctypes.byref(_view(out)), axis, qs, len(q)), "quantile")
    return np.ascontiguousarray(np.moveaxis(out, axis, 0))


def concat(xs: List[np.ndarray], axis: int) -> np.ndarray:
    axis %= xs[0].ndim
    dtype = np.result_type(*[x.dtype for x in xs])
    shape = list(xs[0].shape)
    shape[axis] = sum(x.shape[axis] for x in xs)
    out = np.empty(shape, dtype)
    at = 0
    for x in xs:
        sl = [slice(None)] * out.ndim
        sl[axis] = slice(at, at + x.shape[axis])
        copy(x, out[tuple(sl)])
        at += x.shape[axis]
    return out


def pad(x: np.ndarray, before_after: Sequence[int], value: float) -> np.ndarray:
    shape = [x.shape[d] + before_after[2 * d] + before_after[2 * d + 1] for d in range(x.ndim)]
    out = np.empty(shape, x.dtype)
    _check(_lib().fdf_fill(ctypes.byref(_view(out)), float(value)), "pad")
    sl = tuple(slice(before_after[2 * d], before_after[2 * d] + x.shape[d]) for d in range(x.ndim))
    copy(x, out[sl])
    return out


def tile(x: np.ndarray, reps: Sequence[int]) -> np.ndarray:
    reps = [1] * (x.ndim - len(reps)) + list(reps)
    x = x.reshape([1] * (len(reps) - x.ndim) + list(x.shape))
    # [r0, s0, r1, s1, ...] with stride 0 on the repeat axes, flattened pairwise into the tiled shape
    shape, strides = [], []
    for r, s, st in zip(reps, x.shape, x.strides):
        shape += [r, s]
        strides += [0, st]
    view = np.lib.stride_tricks.as_strided(x, shape=shape, strides=strides, writeable=False)
    out = np.empty(shape, x.dtype)
    copy(view, out)
    return out.reshape([r * s for r, s in zip(reps, x.shape)])
