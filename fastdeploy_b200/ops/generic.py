"""Shape-plumbing kernels of the executor (csrc/kernels/generic_ops.cu): strided copy / cast, broadcasting
elementwise arithmetic and logic, soft-max and reductions over the last axis, row gather.

Every wrapper takes torch tensors as *descriptions* (pointer, shape, element strides, dtype) and returns a
:class:`NativeOp` whose launch touches no framework operator, so that whatever a graph contains besides
convolutions, GEMMs and attention still runs inside the plan's stream and CUDA graph.

The reference runs these as layers of a vendor engine (fastdeploy/runtime/backends/tensorrt/trt_backend.cc:347).
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence, Tuple

import torch

from .. import _native
from .base import NativeOp, dtype_code

DT_BOOL = 8

EW = {
    "add": 0, "sub": 1, "mul": 2, "div": 3, "max": 4, "min": 5, "pow": 6, "eq": 7, "ne": 8, "lt": 9, "le": 10, "gt": 11,
    "ge": 12, "and": 13, "or": 14, "xor": 15, "floordiv": 16, "mod": 17,
    "not": 32, "neg": 33, "abs": 34, "sqrt": 35, "rsqrt": 36, "exp": 37, "log": 38, "tanh": 39, "sigmoid": 40, "relu": 41,
    "erf": 42, "floor": 43, "ceil": 44, "round": 45, "sign": 46, "reciprocal": 47, "affine": 48, "clip": 49, "identity": 50,
    "sin": 51, "cos": 52, "hard_sigmoid": 53, "hard_swish": 54, "silu": 55, "gelu": 56, "leaky_relu": 57, "softplus": 58,
}
REDUCE = {"sum": 0, "mean": 1, "max": 2, "min": 3, "argmax": 4, "argmin": 5, "prod": 6}
MAX_DIMS = 6


class _GenericDesc(ctypes.Structure):
    _fields_ = [("p", ctypes.c_void_p * 4), ("i", ctypes.c_longlong * 48), ("f", ctypes.c_float * 4)]


def _lib():
    lib = _native.kernels()
    if not getattr(lib, "_generic_ready", False):
        lib.fdb_generic_create.restype = ctypes.c_void_p
        lib.fdb_generic_create.argtypes = [ctypes.c_int, ctypes.POINTER(_GenericDesc)]
        lib._generic_ready = True
    return lib


def code_of(dt: torch.dtype) -> int:
    """Element-type code of the generic kernels (the shared codes plus bool)."""
    if dt == torch.bool:
        return DT_BOOL
    return dtype_code(dt)


def supported(dt: torch.dtype) -> bool:
    try:
        code_of(dt)
        return dt != getattr(torch, "float8_e4m3fn", None)
    except KeyError:
        return False


def _make(kind: int, ptrs, ints, floats=(), name="generic") -> NativeOp:
    d = _GenericDesc()
    for k, t in enumerate(ptrs):
        d.p[k] = t.data_ptr() if t is not None else None
    for k, v in enumerate(ints):
        d.i[k] = int(v)
    for k, v in enumerate(floats):
        d.f[k] = float(v)
    op = NativeOp(_lib().fdb_generic_create(kind, ctypes.byref(d)), list(ptrs), name)
    op.create = ("fdb_generic_create", kind, d)
    return op


def coalesce(shape: Sequence[int], strides: Sequence[Sequence[int]]) -> Tuple[List[int], List[List[int]]]:
    """Drops unit dimensions and merges neighbours that every operand walks with one stride
    (``stride[d] == stride[d + 1] * shape[d + 1]``), so that most views fit the kernels' six dimensions."""
    dims = [(s, [st[k] for st in strides]) for k, s in enumerate(shape) if s != 1]
    if not dims:
        return [1], [[0] for _ in strides]
    out = [dims[0]]
    for s, st in dims[1:]:
        ps, pst = out[-1]
        if all(a == b * s for a, b in zip(pst, st)):
            out[-1] = (ps * s, st)
        else:
            out.append((s, st))
    return [s for s, _ in out], [[st[k] for _, st in out] for k in range(len(strides))]


def _pad6(v: Sequence[int]) -> List[int]:
    return list(v) + [0] * (MAX_DIMS - len(v))


def strided_copy(src: torch.Tensor, dst: torch.Tensor, name: str = "copy") -> NativeOp:
    """``dst[...] = cast(src[...])``; ``src`` is broadcast to ``dst``'s shape, both sides may be any strided views."""
    src = src.expand(dst.shape) if tuple(src.shape) != tuple(dst.shape) else src
    shape, (ss, ds) = coalesce(list(dst.shape), [list(src.stride()), list(dst.stride())])
    if len(shape) > MAX_DIMS:
        raise ValueError(f"{name}: view does not collapse to {MAX_DIMS} dimensions")
    nd = len(shape)
    return _make(0, [src, dst], [nd, code_of(src.dtype), code_of(dst.dtype)] + _pad6(shape) + _pad6(ss) + _pad6(ds),
                 name=name)


def elementwise(op: str, a: torch.Tensor, b: Optional[torch.Tensor], out: torch.Tensor, f0: float = 0.0, f1: float = 0.0,
                name: Optional[str] = None) -> NativeOp:
    """``out = op(a, b)`` (``b`` None for unary ops) with numpy broadcasting to ``out``'s shape."""
    a = a.expand(out.shape)
    strides = [list(a.stride())]
    if b is not None:
        b = b.expand(out.shape)
        strides.append(list(b.stride()))
    else:
        strides.append([0] * out.dim())
    strides.append(list(out.stride()))
    shape, (sa, sb, so) = coalesce(list(out.shape), strides)
    if len(shape) > MAX_DIMS:
        raise ValueError(f"{op}: view does not collapse to {MAX_DIMS} dimensions")
    ints = [len(shape), EW[op], code_of(a.dtype), code_of(b.dtype) if b is not None else 0, code_of(out.dtype)]
    ints += _pad6(shape) + _pad6(sa) + _pad6(sb) + _pad6(so)
    return _make(1, [a, b, out], ints, [f0, f1], name=name or f"ew_{op}")


def rows_of(t: torch.Tensor) -> Optional[Tuple[int, int]]:
    """``(rows, row stride)`` when ``t`` is a stack of unit-stride rows at one uniform pitch, else None."""
    if t.dim() == 0 or (t.shape[-1] > 1 and t.stride(-1) != 1):
        return None
    shape, (st,) = coalesce(list(t.shape[:-1]) or [1], [list(t.stride()[:-1]) or [0]])
    if len(shape) != 1:
        return None
    return shape[0], (st[0] if shape[0] > 1 else max(t.shape[-1], 1))


def softmax_last(x: torch.Tensor, y: torch.Tensor, log: bool = False) -> NativeOp:
    """Soft-max over the last axis; both tensors must be stacks of unit-stride rows (see :func:`rows_of`)."""
    rx, ry = rows_of(x), rows_of(y)
    assert rx is not None and ry is not None and rx[0] == ry[0], "softmax_last: rows at one pitch expected"
    return _make(2, [x, y], [rx[0], x.shape[-1], rx[1], ry[1], code_of(x.dtype), code_of(y.dtype), int(log)],
                 name="log_softmax" if log else "softmax")


def reduce_last(mode: str, x: torch.Tensor, y: torch.Tensor) -> NativeOp:
    """``y[row] = reduce(x[row, :])``; ``y`` is contiguous with one element per row."""
    rx = rows_of(x)
    assert rx is not None and y.is_contiguous() and y.numel() == rx[0], "reduce_last: rows at one pitch expected"
    return _make(3, [x, y], [rx[0], x.shape[-1], rx[1], code_of(x.dtype), code_of(y.dtype), REDUCE[mode]],
                 name=f"reduce_{mode}")


def gather_rows(table: torch.Tensor, index: torch.Tensor, out: torch.Tensor) -> NativeOp:
    """``out[i, :] = table[index[i], :]`` for contiguous operands (``index`` int32 / int64, flattened)."""
    assert table.is_contiguous() and index.is_contiguous() and out.is_contiguous()
    row = table[0].numel() if table.dim() > 1 else 1
    assert out.numel() == index.numel() * row
    return _make(4, [table, index, out], [index.numel(), row, table.shape[0], code_of(table.dtype), code_of(index.dtype),
                                         code_of(out.dtype)], name="gather_rows")


def where(cond: torch.Tensor, a: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> NativeOp:
    """``out = cond ? a : b`` with numpy broadcasting to ``out``'s shape."""
    cond, a, b = cond.expand(out.shape), a.expand(out.shape), b.expand(out.shape)
    shape, (sc, sa, sb, so) = coalesce(list(out.shape), [list(cond.stride()), list(a.stride()), list(b.stride()),
                                                         list(out.stride())])
    if len(shape) > MAX_DIMS:
        raise ValueError(f"where: view does not collapse to {MAX_DIMS} dimensions")
    ints = [len(shape), code_of(cond.dtype), code_of(a.dtype), code_of(b.dtype), code_of(out.dtype)]
    ints += _pad6(shape) + _pad6(sc) + _pad6(sa) + _pad6(sb) + _pad6(so)
    return _make(5, [cond, a, b, out], ints, name="where")
