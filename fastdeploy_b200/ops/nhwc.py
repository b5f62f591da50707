"""Python handles for the memory-bound NHWC kernels (csrc/kernels/nhwc_ops.cu).

Every factory returns a :class:`NativeOp` bound to fixed tensors; channel strides
(``*_ld``) let an op read or write a channel slice of a wider buffer, which is how
concat and split disappear from the executed plan.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence, Tuple

import torch

from .. import _native
from .base import ACT, DT_BF16, NativeOp, dtype_code

K_GAP_PARTIAL, K_GAP_FINALIZE, K_SE_FC, K_SCALE_CHANNELS, K_MAXPOOL, K_UPSAMPLE, K_COPY, K_DFL, K_BINARY, \
    K_AVGPOOL, K_CAST, K_UNARY = range(12)


class _SimpleDesc(ctypes.Structure):
    _fields_ = [("p", ctypes.c_void_p * 8), ("i", ctypes.c_longlong * 24), ("f", ctypes.c_float * 8)]


def _lib():
    lib = _native.kernels()
    if not getattr(lib, "_simple_ready", False):
        lib.fdb_simple_create.restype = ctypes.c_void_p
        lib.fdb_simple_create.argtypes = [ctypes.c_int, ctypes.POINTER(_SimpleDesc)]
        lib._simple_ready = True
    return lib


def make_simple(kind: int, ptrs: Sequence[Optional[torch.Tensor]], ints: Sequence[int],
                floats: Sequence[float] = (), name: str = "simple") -> NativeOp:
    d = _SimpleDesc()
    for k, t in enumerate(ptrs):
        d.p[k] = t.data_ptr() if t is not None else None
    for k, v in enumerate(ints):
        d.i[k] = int(v)
    for k, v in enumerate(floats):
        d.f[k] = float(v)
    op = NativeOp(_lib().fdb_simple_create(kind, ctypes.byref(d)), list(ptrs), name)
    op.create = ("fdb_simple_create", kind, d)
    return op


def _bf(t: torch.Tensor) -> int:
    return 1 if dtype_code(t.dtype) == DT_BF16 else 0


def gap_splits(hw: int, n: int, c: int, sms: int = 148) -> int:
    """Number of pixel splits so that a global average pool fills the GPU."""
    blocks = n * ((c + 63) // 64)
    return max(1, min((2 * sms + blocks - 1) // blocks, (hw + 255) // 256))


def global_avgpool(x: torch.Tensor, out: torch.Tensor, scratch: torch.Tensor, *, n: int, hw: int, c: int,
                   x_ld: Optional[int] = None, x_n_stride: int = 0, splits: int = 1,
                   out_ld: Optional[int] = None) -> List[NativeOp]:
    """``out[n,c] = mean_p x[n,p,c]``. ``scratch`` holds ``n*splits*c`` fp32 partial sums."""
    assert scratch.dtype == torch.float32 and scratch.numel() >= n * splits * c
    a = make_simple(K_GAP_PARTIAL, [x, scratch], [n, hw, c, x_ld or c, splits, _bf(x), x_n_stride], name="gap_partial")
    b = make_simple(K_GAP_FINALIZE, [scratch, out], [n, c, splits, dtype_code(out.dtype), out_ld or c],
                    [1.0 / hw], name="gap_finalize")
    return [a, b]


def se_fc(v: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, *, n: int, cin: int,
          cout: int, act: Optional[str] = None, alpha: float = 0.0, beta: float = 0.0) -> NativeOp:
    """``out[n,co] = act(bias[co] + sum_ci w[co,ci] v[n,ci])`` with fp32 ``v``/``out`` and 16-bit ``w``."""
    assert v.dtype == torch.float32 and out.dtype == torch.float32
    return make_simple(K_SE_FC, [v, w, bias, out], [n, cin, cout, ACT[act], _bf(w)], [alpha, beta], name="se_fc")


def scale_channels(x: torch.Tensor, s: torch.Tensor, y: torch.Tensor, *, n: int, hw: int, c: int,
                   x_ld: Optional[int] = None, y_ld: Optional[int] = None, residual: Optional[torch.Tensor] = None,
                   r_ld: int = 0, x_n_stride: int = 0, y_n_stride: int = 0, r_n_stride: int = 0) -> NativeOp:
    """``y[n,p,c] = x[n,p,c] * s[n,c] (+ residual[n,p,c])``."""
    assert s.dtype == torch.float32
    return make_simple(K_SCALE_CHANNELS, [x, s, y, residual],
                       [n, hw, c, x_ld or c, y_ld or c, _bf(x), x_n_stride, y_n_stride, r_ld, r_n_stride],
                       name="scale_channels")


def pool2d(x: torch.Tensor, y: torch.Tensor, *, n: int, h: int, w: int, c: int, kernel: Tuple[int, int],
           stride: Tuple[int, int], pad: Tuple[int, int], out_hw: Tuple[int, int], mode: str = "max",
           x_ld: Optional[int] = None, y_ld: Optional[int] = None, x_n_stride: int = 0, y_n_stride: int = 0,
           count_include_pad: bool = False) -> NativeOp:
    kind = K_MAXPOOL if mode == "max" else K_AVGPOOL
    return make_simple(kind, [x, y], [n, h, w, c, x_ld or c, out_hw[0], out_hw[1], y_ld or c, kernel[0], kernel[1],
                                      stride[0], stride[1], pad[0], pad[1], _bf(x), x_n_stride, y_n_stride,
                                      2 if count_include_pad else 1], name=f"{mode}pool")


def upsample_nearest(x: torch.Tensor, y: torch.Tensor, *, n: int, h: int, w: int, c: int, factor: Tuple[int, int],
                     x_ld: Optional[int] = None, y_ld: Optional[int] = None, x_n_stride: int = 0,
                     y_n_stride: int = 0) -> NativeOp:
    return make_simple(K_UPSAMPLE, [x, y], [n, h, w, c, x_ld or c, y_ld or c, factor[0], factor[1], x_n_stride,
                                            y_n_stride], name="upsample_nearest")


def copy_channels(x: torch.Tensor, y: torch.Tensor, *, n: int, h: int, w: int, c: int, x_ld: Optional[int] = None,
                  y_ld: Optional[int] = None, x_n_stride: int = 0, y_n_stride: int = 0) -> NativeOp:
    return make_simple(K_COPY, [x, y], [n, h, w, c, x_ld or c, y_ld or c, 1, 1, x_n_stride, y_n_stride],
                       name="copy_channels")


def dfl_decode(reg: torch.Tensor, boxes: torch.Tensor, scale_factor: Optional[torch.Tensor], *, n: int, anchors: int,
               bins: int, levels: Sequence[Tuple[int, int, int]], offset: float = 0.5, reg_ld: int = 0) -> NativeOp:
    """``levels``: ``(first_anchor, grid_width, stride)`` per pyramid level, in anchor order."""
    ints = [n, anchors, bins, dtype_code(reg.dtype), len(levels)]
    for st, w, s in levels:
        ints += [st, w, s]
    ints += [0] * (20 - len(ints)) + [reg_ld]
    assert boxes.dtype == torch.float32
    return make_simple(K_DFL, [reg, boxes, scale_factor], ints, [offset], name="dfl_decode")


_BIN = {"add": 0, "mul": 1, "sub": 2, "max": 3}


def binary(a: torch.Tensor, b: torch.Tensor, y: torch.Tensor, *, rows: int, c: int, op: str = "add",
           act: Optional[str] = None, a_ld: Optional[int] = None, b_ld: Optional[int] = None,
           y_ld: Optional[int] = None, broadcast_b: bool = False, alpha: float = 0.0, beta: float = 0.0) -> NativeOp:
    return make_simple(K_BINARY, [a, b, y], [rows, c, a_ld or c, b_ld or c, y_ld or c, _bf(a), _BIN[op], ACT[act],
                                             1 if broadcast_b else 0], [alpha, beta], name=f"binary_{op}")


def unary(x: torch.Tensor, y: torch.Tensor, *, rows: int, c: int, act: str, x_ld: Optional[int] = None,
          y_ld: Optional[int] = None, alpha: float = 0.0, beta: float = 0.0) -> NativeOp:
    return make_simple(K_UNARY, [x, y], [rows, c, x_ld or c, y_ld or c, _bf(x), ACT[act]], [alpha, beta],
                       name=f"unary_{act}")


def cast(x: torch.Tensor, y: torch.Tensor) -> NativeOp:
    assert x.numel() == y.numel()
    return make_simple(K_CAST, [x, y], [x.numel(), dtype_code(x.dtype), dtype_code(y.dtype)], name="cast")


K_DEPTHWISE = 12


def depthwise_conv(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], y: torch.Tensor, *, n: int, h: int,
                   w_in: int, c: int, kernel: Tuple[int, int], stride: Tuple[int, int], pad: Tuple[int, int],
                   out_hw: Tuple[int, int], act: Optional[str] = None, act_alpha: float = 0.0, act_beta: float = 0.0,
                   x_ld: Optional[int] = None, y_ld: Optional[int] = None, x_n_stride: int = 0, y_n_stride: int = 0) -> NativeOp:
    """Depthwise convolution on NHWC 16-bit tensors; ``w`` is fp32 ``[KH*KW, C]`` (C padded to 8)."""
    from .base import ACT
    assert w.dtype == torch.float32 and w.shape == (kernel[0] * kernel[1], c)
    return make_simple(K_DEPTHWISE, [x, w, bias, y],
                       [n, h, w_in, c, x_ld or c, out_hw[0], out_hw[1], y_ld or c, kernel[0], kernel[1], stride[0], stride[1],
                        pad[0], pad[1], _bf(x), x_n_stride, y_n_stride, ACT[act]], [act_alpha, act_beta], name="depthwise_conv")


# ---------------------------------------------------------------------- fused small ops (csrc/kernels/fused_small_ops.cu)
def _fused_lib():
    lib = _native.kernels()
    if not getattr(lib, "_fused_ready", False):
        lib.fdb_fused_create.restype = ctypes.c_void_p
        lib.fdb_fused_create.argtypes = [ctypes.c_int, ctypes.POINTER(_SimpleDesc)]
        lib._fused_ready = True
    return lib


def _make_fused(kind: int, ptrs, ints, floats=(), name="fused") -> NativeOp:
    d = _SimpleDesc()
    for k, t in enumerate(ptrs):
        d.p[k] = t.data_ptr() if t is not None else None
    for k, v in enumerate(ints):
        d.i[k] = int(v)
    for k, v in enumerate(floats):
        d.f[k] = float(v)
    op = NativeOp(_fused_lib().fdb_fused_create(kind, ctypes.byref(d)), list(ptrs), name)
    op.create = ("fdb_fused_create", kind, d)
    return op


def gap_splits_v2(hw: int, n: int, c: int, sms: int = 148) -> int:
    """Pixel splits of the bandwidth-bound partial-sum kernel: about eight blocks per SM, at least 128 pixels each."""
    blocks = n * ((c + 63) // 64)
    return max(1, min((8 * sms + blocks - 1) // blocks, (hw + 127) // 128))


def gap_partial(x: torch.Tensor, part: torch.Tensor, *, n: int, hw: int, c: int, x_ld: Optional[int] = None,
                x_n_stride: int = 0, splits: int = 1) -> NativeOp:
    """``part[n, s, c] = sum of x[n, p, c] over the pixels of split s`` (fp32 ``part`` of ``n * splits * c``)."""
    assert part.dtype == torch.float32 and part.numel() >= n * splits * c
    return _make_fused(0, [x, part], [n, hw, c, x_ld or c, splits, _bf(x), x_n_stride], name="gap_partial")


def ese_gate(part: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, *, n: int, cin: int,
             cout: int, splits: int, hw: int, act: Optional[str] = None, alpha: float = 0.0, beta: float = 0.0,
             out_ld: Optional[int] = None) -> NativeOp:
    """``out[n, co] = act(bias[co] + sum_ci w[co, ci] * mean[n, ci])`` where the mean over ``hw`` pixels is finished
    from the per-split partial sums: global-average-pool finalise + the 1x1 "excite" convolution + its activation."""
    assert part.dtype == torch.float32 and out.dtype == torch.float32 and w.dim() == 2 and w.stride(1) == 1
    return _make_fused(1, [part, w, bias, out], [n, cin, cout, splits, w.stride(0), out_ld or cout, ACT[act], _bf(w)],
                       [1.0 / hw, alpha, beta], name="ese_gate")


def spp_maxpool(x: torch.Tensor, outs: Sequence[torch.Tensor], kernels: Sequence[int], *, n: int, h: int, w: int, c: int,
                x_ld: Optional[int] = None, x_n_stride: int = 0, y_lds: Optional[Sequence[int]] = None,
                y_n_strides: Optional[Sequence[int]] = None) -> NativeOp:
    """Stride-1, same-size max pools with odd, increasing ``kernels`` (e.g. 5, 9, 13) of one NHWC input, each written
    to its own destination; the input is read once."""
    ints = [n, h, w, c, x_ld or c, x_n_stride, _bf(x), len(kernels)]
    for k in range(len(kernels)):
        ints += [kernels[k], (y_lds[k] if y_lds else c), (y_n_strides[k] if y_n_strides else 0)]
    return _make_fused(2, [x] + list(outs), ints, name="spp_maxpool")


def spp_fits(h: int, w: int, nk: int) -> bool:
    return h * w * 16 * (1 + nk) <= 96 * 1024


def scale_weights(w_packed: torch.Tensor, gate: torch.Tensor, out: torch.Tensor, *, n: int, cout: int, cin: int,
                  plus: float = 0.0) -> NativeOp:
    """``out[n, co, k] = w_packed[co, k] * (gate[n, k] + plus)``: a channel gate on the input of a 1x1 convolution
    folded into per-image weights (``conv(x * g) = conv_{W diag(g)}(x)``)."""
    kp = w_packed.shape[1]
    assert gate.dtype == torch.float32 and out.dtype == w_packed.dtype and out.numel() == n * cout * kp
    return _make_fused(3, [w_packed, gate, out], [n, cout, kp, cin, gate.stride(0), _bf(w_packed)], [plus],
                       name="scale_weights")


def quantize_e4m3(x: torch.Tensor, y: torch.Tensor, *, rows: int, c: int, scale: float, x_ld: Optional[int] = None,
                  y_ld: Optional[int] = None) -> NativeOp:
    """``y = e4m3(x * scale)`` for 16-bit rows ``x [rows, c]`` (static quantisation: ``scale`` is the reciprocal of
    the activation scale the consuming fp8 GEMM dequantises with)."""
    assert y.dtype == torch.float8_e4m3fn
    return _make_fused(4, [x, y], [rows, c, x_ld or c, y_ld or c, _bf(x)], [scale], name="quantize_e4m3")


def quantize_rows_e4m3_op(x: torch.Tensor, y: torch.Tensor, scales: torch.Tensor, *, rows: int, c: int,
                          x_ld: Optional[int] = None, y_ld: Optional[int] = None, c_padded: Optional[int] = None) -> NativeOp:
    """Dynamic per-row quantisation ``y[r] = e4m3(x[r] * 448 / max|x[r]|)``, ``scales[r] = max|x[r]| / 448``; columns
    ``c .. c_padded - 1`` of ``y`` are zeroed (the consuming fp8 GEMM's K padding)."""
    assert y.dtype == torch.float8_e4m3fn and scales.dtype == torch.float32 and scales.numel() >= rows
    return _make_fused(5, [x, y, scales], [rows, c, x_ld or c, y_ld or c, _bf(x), c_padded or c], name="quantize_rows_e4m3")
