"""Tensor function library on :class:`FDTensor` (fastdeploy/function/functions.h:17-37): the 21
functions of the reference with the same semantics. Host tensors of the plain numeric types run in the native
library (csrc/cpu/functions.cc through ``function/native.py``: strided views, double / int64 arithmetic, stable sort,
first-extreme arg-max, linear-interpolated quantile, integer division toward zero); tensors on a GPU and the
16-bit floating types run on torch operators, so the same call works wherever the operands live. Every function
takes input tensors and writes into / returns an output :class:`FDTensor`."""
from __future__ import annotations

from typing import List, Optional, Sequence, Union

import numpy as np
import torch

from ..core.fd_tensor import _FD2TORCH, FDTensor
from ..core.types import FDDataType
from . import native


def _t(x) -> torch.Tensor:
    if isinstance(x, FDTensor):
        return x.tensor()
    if isinstance(x, np.ndarray):
        return torch.from_numpy(x)
    return x


def _out(res: torch.Tensor, out: Optional[FDTensor] = None, name: str = "") -> FDTensor:
    r = FDTensor.from_torch(res.contiguous(), name)
    r.stop_sharing()
    if out is not None:
        out.copy_buffer(r)
        return out
    return r


def _np(x) -> Optional[np.ndarray]:
    """The operand as a numpy array when the native host library can take it (host memory, a supported dtype)."""
    t = _t(x)
    if isinstance(t, torch.Tensor):
        if t.device.type != "cpu" or t.dtype in (torch.float16, torch.bfloat16) or t.dtype.is_complex:
            return None
        t = t.detach().numpy()
    return t if native.usable(t) else None


def _nout(arr: np.ndarray, out: Optional[FDTensor] = None) -> FDTensor:
    return _out(torch.from_numpy(np.asarray(arr, order="C")), out)      # (ascontiguousarray would make a 0-d result 1-d)


def _unary(name: str, torch_fn, to_bool: bool = False):
    def run(x, out=None):
        a = _np(x)
        if a is not None and (to_bool or a.dtype.kind == "f" or name == "abs"):
            return _nout(native.unary(name, a, np.bool_ if to_bool else None), out)
        return _out(torch_fn(_t(x)), out)
    run.__name__ = name
    run.__doc__ = f"Element-wise ``{name}`` (fastdeploy/function/math.cc, isfinite.cc)."
    return run


def _binary(name: str, torch_fn):
    def run(a, b, out=None):
        x, y = _np(a), _np(b)
        if x is not None and y is not None:
            return _nout(native.binary(name, x, y), out)
        return _out(torch_fn(_t(a), _t(b)), out)
    run.__name__ = name
    run.__doc__ = f"Broadcasting ``{name}`` (fastdeploy/function/elementwise.cc); integer division truncates toward zero."
    return run


def cast(x, dtype: FDDataType, out=None):
    a, tgt = _np(x), _FD2TORCH[dtype]
    if a is not None and tgt not in (torch.float16, torch.bfloat16):
        return _nout(native.materialise(a, torch.empty(0, dtype=tgt).numpy().dtype), out)
    return _out(_t(x).to(tgt), out)


def clip(x, lo: float, hi: float, out=None):
    a = _np(x)
    if a is not None:
        return _nout(native.unary("clip", a, None, lo, hi), out)
    return _out(torch.clamp(_t(x), lo, hi), out)


def concat(xs: Sequence, axis: int = 0, out=None):
    arrs = [_np(x) for x in xs]
    if not [a for a in arrs if a is None]:
        return _nout(native.concat(arrs, axis), out)
    return _out(torch.cat([_t(x) for x in xs], dim=axis), out)


def cumprod(x, axis: int = 0, out=None):
    a = _np(x)
    if a is not None and a.dtype.kind == "f":
        return _nout(native.scan("cumprod", a, axis), out)
    return _out(torch.cumprod(_t(x), dim=axis), out)


add = _binary("add", lambda a, b: a + b)
subtract = _binary("subtract", lambda a, b: a - b)
multiply = _binary("multiply", lambda a, b: a * b)
divide = _binary("divide", lambda a, b: torch.div(a, b, rounding_mode="trunc") if not a.is_floating_point() else a / b)
maximum = _binary("maximum", torch.maximum)


def _native_fill(shape, value, tdtype) -> Optional[np.ndarray]:
    """Filled natively when the type is one the host library stores and the value passes through a double unchanged."""
    if tdtype in (torch.float16, torch.bfloat16) or tdtype.is_complex:
        return None
    ndt = torch.empty(0, dtype=tdtype).numpy().dtype
    if not native.usable(np.empty(0, ndt)) or len(shape) > native.MAX_DIMS:
        return None
    if isinstance(value, int) and not isinstance(value, bool) and _bi.abs(value) > 2 ** 53:
        return None
    return native.fill(list(shape), value, ndt)


def full(value, shape: Sequence[int], dtype: FDDataType = FDDataType.FP32, out=None):
    a = _native_fill(shape, value, _FD2TORCH[dtype])
    if a is not None:
        return _nout(a, out)
    return _out(torch.full(list(shape), value, dtype=_FD2TORCH[dtype]), out)
def full_like(x, value, dtype: Optional[FDDataType] = None, out=None):
    t = _t(x)
    a = _native_fill(list(t.shape), value, _FD2TORCH[dtype] if dtype is not None else t.dtype) if t.device.type == "cpu" else None
    if a is not None:
        return _nout(a, out)
    return _out(torch.full_like(t, value, dtype=_FD2TORCH[dtype] if dtype is not None else t.dtype), out)


def gather_along_axis(x, index, axis: int, out=None):
    a, i = _np(x), _np(index)
    if a is not None and i is not None and i.dtype.kind in "iu" and a.ndim == i.ndim:
        return _nout(native.gather(a, i, axis), out)
    return _out(torch.gather(_t(x), axis, _t(index).long()), out)


def scatter_along_axis(x, index, values, axis: int, out=None):
    a, i, v = _np(x), _np(index), _np(values)
    if a is not None and i is not None and v is not None and i.dtype.kind in "iu" and a.ndim == i.ndim \
            and v.shape == i.shape:
        return _nout(native.scatter(a, i, v.astype(a.dtype, copy=False), axis), out)
    return _out(_t(x).scatter(axis, _t(index).long(), _t(values)), out)


def gaussian_random(shape: Sequence[int], mean: float = 0.0, std: float = 1.0, seed: int = 0,
                    dtype: FDDataType = FDDataType.FP32, out=None):
    g = torch.Generator().manual_seed(seed)
    return _out((torch.randn(list(shape), generator=g) * std + mean).to(_FD2TORCH[dtype]), out)


isnan = _unary("isnan", torch.isnan, to_bool=True)
isinf = _unary("isinf", torch.isinf, to_bool=True)
isfinite = _unary("isfinite", torch.isfinite, to_bool=True)


def linspace(start: float, end: float, num: int, dtype: FDDataType = FDDataType.FP32, out=None):
    return _out(torch.linspace(start, end, num, dtype=torch.float64).to(_FD2TORCH[dtype]), out)


sqrt = _unary("sqrt", torch.sqrt)
log = _unary("log", torch.log)
round = _unary("round", torch.round)     # noqa: A001
exp = _unary("exp", torch.exp)
abs = _unary("abs", torch.abs)           # noqa: A001
ceil = _unary("ceil", torch.ceil)
floor = _unary("floor", torch.floor)


def pad(x, pad_value: Sequence[int], value: float = 0.0, out=None):
    """``pad_value`` = [before_0, after_0, before_1, after_1, ...] (fastdeploy/function/pad.h)."""
    a = _np(x)
    if a is not None and len(pad_value) == 2 * a.ndim and builtins_min(pad_value) >= 0:
        return _nout(native.pad(a, list(pad_value), value), out)
    t = _t(x)
    tp: List[int] = []
    for d in reversed(range(t.dim())):
        tp += [pad_value[2 * d], pad_value[2 * d + 1]]
    return _out(torch.nn.functional.pad(t, tp, value=value), out)


def quantile(x, q: Sequence[float], axis: Sequence[int], out=None):
    """Linear-interpolated quantile along one axis (fastdeploy/function/quantile.cc)."""
    assert len(axis) == 1, "quantile supports a single axis"
    a = _np(x)
    if a is not None:
        return _nout(native.quantile(a, list(q), axis[0], a.dtype if a.dtype.kind == "f" else np.float64), out)
    t = _t(x).double()
    r = torch.quantile(t, torch.tensor(list(q), dtype=torch.float64), dim=axis[0])
    return _out(r.to(_t(x).dtype if _t(x).is_floating_point() else torch.float64), out)


def _native_reduce_dtype(name: str, dt: np.dtype) -> np.dtype:
    """Result type of a reduction, as the torch path gives it: integer sums and products widen to int64, the mean of
    integers is float64, max / min keep the type, all / any are bool."""
    if name in ("all", "any"):
        return np.dtype(np.bool_)
    if name == "mean":
        return dt if dt.kind == "f" else np.dtype(np.float64)
    if name in ("sum", "prod") and dt.kind != "f":
        return np.dtype(np.int64)
    return dt


def _reduce(fn, name: str = ""):
    def run(x, dims: Sequence[int] = (), keep_dim: bool = False, reduce_all: bool = False, out=None):
        a = _np(x)
        if a is not None and name and a.ndim > 0 and not (name in ("max", "min") and a.size == 0):
            d = list(range(a.ndim)) if reduce_all or len(dims) == 0 else [ax % a.ndim for ax in dims]
            return _nout(native.reduce(name, a, d, keep_dim, _native_reduce_dtype(name, a.dtype)), out)
        t = _t(x)
        d = list(range(t.dim())) if reduce_all or len(dims) == 0 else [a % t.dim() for a in dims]
        return _out(fn(t, d, keep_dim), out)
    return run


def _prod(t, d, k):
    for a in sorted(d, reverse=True):
        t = t.prod(dim=a, keepdim=k)
    return t


max = _reduce(lambda t, d, k: t.amax(dim=d, keepdim=k), "max")       # noqa: A001
min = _reduce(lambda t, d, k: t.amin(dim=d, keepdim=k), "min")       # noqa: A001
sum = _reduce(lambda t, d, k: t.sum(dim=d, keepdim=k), "sum")        # noqa: A001
mean = _reduce(lambda t, d, k: t.double().mean(dim=d, keepdim=k).to(t.dtype if t.is_floating_point() else torch.float64),
               "mean")
prod = _reduce(_prod, "prod")
all = _reduce(lambda t, d, k: _prod(t.bool().to(torch.uint8), d, k).bool(), "all")   # noqa: A001
any = _reduce(lambda t, d, k: t.bool().to(torch.uint8).amax(dim=d, keepdim=k).bool(), "any")   # noqa: A001


def argmax(x, axis: int, output_dtype: FDDataType = FDDataType.INT64, keep_dim: bool = False, flatten: bool = False,
           out=None):
    a = _np(x)
    if a is not None and a.size > 0 and _FD2TORCH[output_dtype] in (torch.int32, torch.int64):
        a = a.reshape(-1) if flatten else a
        odt = np.int32 if _FD2TORCH[output_dtype] == torch.int32 else np.int64
        return _nout(native.arg_extreme(True, a, 0 if flatten else axis, keep_dim, odt), out)
    t = _t(x).reshape(-1) if flatten else _t(x)
    return _out(torch.argmax(t, dim=0 if flatten else axis, keepdim=keep_dim).to(_FD2TORCH[output_dtype]), out)


def argmin(x, axis: int, output_dtype: FDDataType = FDDataType.INT64, keep_dim: bool = False, flatten: bool = False,
           out=None):
    a = _np(x)
    if a is not None and a.size > 0 and _FD2TORCH[output_dtype] in (torch.int32, torch.int64):
        a = a.reshape(-1) if flatten else a
        odt = np.int32 if _FD2TORCH[output_dtype] == torch.int32 else np.int64
        return _nout(native.arg_extreme(False, a, 0 if flatten else axis, keep_dim, odt), out)
    t = _t(x).reshape(-1) if flatten else _t(x)
    return _out(torch.argmin(t, dim=0 if flatten else axis, keepdim=keep_dim).to(_FD2TORCH[output_dtype]), out)


def slice(x, axes: Sequence[int], starts: Sequence[int], ends: Optional[Sequence[int]] = None, out=None):   # noqa: A001
    """With ``ends``: ranges per axis; without: picks index ``starts[i]`` on ``axes[i]`` and drops the axis."""
    arr = _np(x)
    t = _t(x) if arr is None else arr
    if ends is None:
        sel = [builtins_slice(None)] * len(t.shape)
        for a, s in zip(axes, starts):
            sel[a] = s
        picked = t[tuple(sel)]
        return _nout(native.materialise(picked), out) if arr is not None else _out(picked, out)
    sl = [builtins_slice(None)] * len(t.shape)
    for a, s, e in zip(axes, starts, ends):
        dim = t.shape[a]
        s = s + dim if s < 0 else s
        e = e + dim if e < 0 else e
        sl[a] = builtins_slice(builtins_max(s, 0), builtins_min(e, dim))
    if arr is not None:
        return _nout(native.materialise(arr[tuple(sl)]), out)
    return _out(t[tuple(sl)], out)


import builtins as _bi   # noqa: E402
builtins_slice, builtins_max, builtins_min = _bi.slice, _bi.max, _bi.min


def softmax(x, axis: int = -1, out=None):
    a = _np(x)
    if a is not None and a.dtype.kind == "f" and a.ndim > 0:
        return _nout(native.scan("softmax", a, axis), out)
    return _out(torch.softmax(_t(x).float(), dim=axis).to(_t(x).dtype), out)


def sort(x, axis: int = -1, descending: bool = False, out=None, out_indices=None):
    a = _np(x)
    if a is not None and a.ndim > 0 and a.dtype != np.bool_:
        v, i = native.sort(a, axis, descending)
        return _nout(v, out), _nout(i, out_indices)
    v, i = torch.sort(_t(x), dim=axis, descending=descending, stable=True)
    return _out(v, out), _out(i, out_indices)


def argsort(x, axis: int = -1, descending: bool = False, out=None):
    a = _np(x)
    if a is not None and a.ndim > 0 and a.dtype != np.bool_:
        return _nout(native.sort(a, axis, descending)[1], out)
    return _out(torch.argsort(_t(x), dim=axis, descending=descending, stable=True), out)


def split(x, num_or_sections: Union[int, Sequence[int]], axis: int = 0) -> List[FDTensor]:
    arr = _np(x)
    t = _t(x)
    if isinstance(num_or_sections, int):
        if arr is None:
            return [_out(p) for p in torch.chunk(t, num_or_sections, dim=axis)]
        each = -(-t.shape[axis] // num_or_sections)            # chunk: equal parts, the last one takes what is left
        secs = [builtins_min(each, t.shape[axis] - i * each) for i in range(num_or_sections) if i * each < t.shape[axis]] or [0]
    else:
        secs = list(num_or_sections)
        if -1 in secs:
            secs[secs.index(-1)] = t.shape[axis] - _bi.sum(s for s in secs if s > 0)
        if arr is None:
            return [_out(p) for p in torch.split(t, secs, dim=axis)]
    if _bi.sum(secs) != arr.shape[axis]:
        raise ValueError(f"split: sections {secs} do not add up to the axis length {arr.shape[axis]}")
    parts, at = [], 0
    for n in secs:
        sel = [builtins_slice(None)] * arr.ndim
        sel[axis] = builtins_slice(at, at + n)
        parts.append(_nout(native.materialise(arr[tuple(sel)])))
        at += n
    return parts


def tile(x, repeat_times: Sequence[int], out=None):
    a = _np(x)
    if a is not None and len(repeat_times) + a.ndim <= 2 * native.MAX_DIMS // 2 and builtins_max(len(repeat_times), a.ndim) <= 4:
        return _nout(native.tile(a, list(repeat_times)), out)
    t = _t(x)
    reps = [1] * (t.dim() - len(repeat_times)) + list(repeat_times)
    return _out(t.repeat(reps), out)


def transpose(x, dims: Sequence[int], out=None):
    a = _np(x)
    if a is not None:
        return _nout(native.materialise(a.transpose(list(dims))), out)
    return _out(_t(x).permute(list(dims)), out)
