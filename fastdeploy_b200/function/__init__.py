"""Tensor function library on :class:`FDTensor` (fastdeploy/function/functions.h:17-37): the 21
functions of the reference with the same semantics, executed by torch on whichever device the
operands live (so the same call works on host tensors and on GPU tensors). Every function takes
input tensors and writes into / returns an output :class:`FDTensor`."""
from __future__ import annotations

from typing import List, Optional, Sequence, Union

import numpy as np
import torch

from ..core.fd_tensor import _FD2TORCH, FDTensor
from ..core.types import FDDataType


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


def cast(x, dtype: FDDataType, out=None): return _out(_t(x).to(_FD2TORCH[dtype]), out)
def clip(x, lo: float, hi: float, out=None): return _out(torch.clamp(_t(x), lo, hi), out)
def concat(xs: Sequence, axis: int = 0, out=None): return _out(torch.cat([_t(x) for x in xs], dim=axis), out)
def cumprod(x, axis: int = 0, out=None): return _out(torch.cumprod(_t(x), dim=axis), out)
def add(a, b, out=None): return _out(_t(a) + _t(b), out)
def subtract(a, b, out=None): return _out(_t(a) - _t(b), out)
def multiply(a, b, out=None): return _out(_t(a) * _t(b), out)
def divide(a, b, out=None):
    ta, tb = _t(a), _t(b)
    return _out(torch.div(ta, tb, rounding_mode="trunc") if not ta.is_floating_point() else ta / tb, out)
def maximum(a, b, out=None): return _out(torch.maximum(_t(a), _t(b)), out)
def full(value, shape: Sequence[int], dtype: FDDataType = FDDataType.FP32, out=None):
    return _out(torch.full(list(shape), value, dtype=_FD2TORCH[dtype]), out)
def full_like(x, value, dtype: Optional[FDDataType] = None, out=None):
    t = _t(x)
    return _out(torch.full_like(t, value, dtype=_FD2TORCH[dtype] if dtype is not None else t.dtype), out)
def gather_along_axis(x, index, axis: int, out=None): return _out(torch.gather(_t(x), axis, _t(index).long()), out)
def scatter_along_axis(x, index, values, axis: int, out=None):
    return _out(_t(x).scatter(axis, _t(index).long(), _t(values)), out)
def gaussian_random(shape: Sequence[int], mean: float = 0.0, std: float = 1.0, seed: int = 0,
                    dtype: FDDataType = FDDataType.FP32, out=None):
    g = torch.Generator().manual_seed(seed)
    return _out((torch.randn(list(shape), generator=g) * std + mean).to(_FD2TORCH[dtype]), out)
def isnan(x, out=None): return _out(torch.isnan(_t(x)), out)
def isinf(x, out=None): return _out(torch.isinf(_t(x)), out)
def isfinite(x, out=None): return _out(torch.isfinite(_t(x)), out)
def linspace(start: float, end: float, num: int, dtype: FDDataType = FDDataType.FP32, out=None):
    return _out(torch.linspace(start, end, num, dtype=torch.float64).to(_FD2TORCH[dtype]), out)
def sqrt(x, out=None): return _out(torch.sqrt(_t(x)), out)
def log(x, out=None): return _out(torch.log(_t(x)), out)
def round(x, out=None): return _out(torch.round(_t(x)), out)   # noqa: A001
def exp(x, out=None): return _out(torch.exp(_t(x)), out)
def abs(x, out=None): return _out(torch.abs(_t(x)), out)       # noqa: A001
def ceil(x, out=None): return _out(torch.ceil(_t(x)), out)
def floor(x, out=None): return _out(torch.floor(_t(x)), out)


def pad(x, pad_value: Sequence[int], value: float = 0.0, out=None):
    """``pad_value`` = [before_0, after_0, before_1, after_1, ...] (fastdeploy/function/pad.h)."""
    t = _t(x)
    tp: List[int] = []
    for d in reversed(range(t.dim())):
        tp += [pad_value[2 * d], pad_value[2 * d + 1]]
    return _out(torch.nn.functional.pad(t, tp, value=value), out)


def quantile(x, q: Sequence[float], axis: Sequence[int], out=None):
    """Linear-interpolated quantile along one axis (fastdeploy/function/quantile.cc)."""
    t = _t(x).double()
    assert len(axis) == 1, "quantile supports a single axis"
    r = torch.quantile(t, torch.tensor(list(q), dtype=torch.float64), dim=axis[0])
    return _out(r.to(_t(x).dtype if _t(x).is_floating_point() else torch.float64), out)


def _reduce(fn):
    def run(x, dims: Sequence[int] = (), keep_dim: bool = False, reduce_all: bool = False, out=None):
        t = _t(x)
        d = list(range(t.dim())) if reduce_all or len(dims) == 0 else [a % t.dim() for a in dims]
        return _out(fn(t, d, keep_dim), out)
    return run


def _prod(t, d, k):
    for a in sorted(d, reverse=True):
        t = t.prod(dim=a, keepdim=k)
    return t


max = _reduce(lambda t, d, k: t.amax(dim=d, keepdim=k))       # noqa: A001
min = _reduce(lambda t, d, k: t.amin(dim=d, keepdim=k))       # noqa: A001
sum = _reduce(lambda t, d, k: t.sum(dim=d, keepdim=k))        # noqa: A001
mean = _reduce(lambda t, d, k: t.double().mean(dim=d, keepdim=k).to(t.dtype if t.is_floating_point() else torch.float64))
prod = _reduce(_prod)
all = _reduce(lambda t, d, k: _prod(t.bool().to(torch.uint8), d, k).bool())   # noqa: A001
any = _reduce(lambda t, d, k: t.bool().to(torch.uint8).amax(dim=d, keepdim=k).bool())   # noqa: A001


def argmax(x, axis: int, output_dtype: FDDataType = FDDataType.INT64, keep_dim: bool = False, flatten: bool = False,
           out=None):
    t = _t(x).reshape(-1) if flatten else _t(x)
    return _out(torch.argmax(t, dim=0 if flatten else axis, keepdim=keep_dim).to(_FD2TORCH[output_dtype]), out)


def argmin(x, axis: int, output_dtype: FDDataType = FDDataType.INT64, keep_dim: bool = False, flatten: bool = False,
           out=None):
    t = _t(x).reshape(-1) if flatten else _t(x)
    return _out(torch.argmin(t, dim=0 if flatten else axis, keepdim=keep_dim).to(_FD2TORCH[output_dtype]), out)


def slice(x, axes: Sequence[int], starts: Sequence[int], ends: Optional[Sequence[int]] = None, out=None):   # noqa: A001
    """With ``ends``: ranges per axis; without: picks index ``starts[i]`` on ``axes[i]`` and drops the axis."""
    t = _t(x)
    if ends is None:
        for a, s in sorted(zip(axes, starts), reverse=True):
            t = t.select(a, s)
        return _out(t, out)
    sl = [builtins_slice(None)] * t.dim()
    for a, s, e in zip(axes, starts, ends):
        dim = t.shape[a]
        s = s + dim if s < 0 else s
        e = e + dim if e < 0 else e
        sl[a] = builtins_slice(builtins_max(s, 0), builtins_min(e, dim))
    return _out(t[tuple(sl)], out)


import builtins as _bi   # noqa: E402
builtins_slice, builtins_max, builtins_min = _bi.slice, _bi.max, _bi.min


def softmax(x, axis: int = -1, out=None): return _out(torch.softmax(_t(x).float(), dim=axis).to(_t(x).dtype), out)


def sort(x, axis: int = -1, descending: bool = False, out=None, out_indices=None):
    v, i = torch.sort(_t(x), dim=axis, descending=descending, stable=True)
    return _out(v, out), _out(i, out_indices)


def argsort(x, axis: int = -1, descending: bool = False, out=None):
    return _out(torch.argsort(_t(x), dim=axis, descending=descending, stable=True), out)


def split(x, num_or_sections: Union[int, Sequence[int]], axis: int = 0) -> List[FDTensor]:
    t = _t(x)
    if isinstance(num_or_sections, int):
        parts = torch.chunk(t, num_or_sections, dim=axis)
    else:
        secs = list(num_or_sections)
        if -1 in secs:
            secs[secs.index(-1)] = t.shape[axis] - _bi.sum(s for s in secs if s > 0)
        parts = torch.split(t, secs, dim=axis)
    return [_out(p) for p in parts]


def tile(x, repeat_times: Sequence[int], out=None):
    t = _t(x)
    reps = [1] * (t.dim() - len(repeat_times)) + list(repeat_times)
    return _out(t.repeat(reps), out)


def transpose(x, dims: Sequence[int], out=None): return _out(_t(x).permute(list(dims)), out)
