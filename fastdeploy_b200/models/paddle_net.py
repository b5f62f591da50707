"""Layer helpers that emit Paddle operators the way PaddlePaddle's own exporters do
(``conv2d`` + ``batch_norm`` + activation op, bias as ``elementwise_add``), with static
shape bookkeeping in NCHW and ``-1`` for the batch dimension."""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np

from ..importer.paddle_format import ProgramBuilder


class Tensor:
    __slots__ = ("name", "shape")

    def __init__(self, name: str, shape: Sequence[int]):
        self.name, self.shape = name, list(shape)

    @property
    def c(self) -> int:
        return self.shape[1]


class PaddleNet:
    def __init__(self, seed: int = 0):
        self.b = ProgramBuilder()
        self.rng = np.random.default_rng(seed)
        self._names = set()

    def _uname(self, name: str) -> str:
        base, k = name, 1
        while name in self._names:
            name = f"{base}_{k}"
            k += 1
        self._names.add(name)
        return name

    # ---------------------------------------------------------------- parameters
    def weight(self, name: str, shape, scale: Optional[float] = None) -> str:
        fan_in = int(np.prod(shape[1:])) if len(shape) > 1 else shape[0]
        s = scale if scale is not None else np.sqrt(2.0 / max(fan_in, 1))
        return self.b.param(self._uname(name), (self.rng.standard_normal(shape) * s).astype(np.float32))

    def const_param(self, name: str, value: np.ndarray) -> str:
        return self.b.param(self._uname(name), np.ascontiguousarray(value))

    # ---------------------------------------------------------------- layers
    def feed(self, name: str, dtype: str, shape) -> Tensor:
        self.b.feed(name, dtype, shape)
        return Tensor(name, shape)

    def conv(self, x: Tensor, cout: int, k: int, stride: int = 1, pad: Optional[int] = None, groups: int = 1,
             bias: bool = False, name: str = "conv", bias_value: Optional[float] = None) -> Tensor:
        pad = k // 2 if pad is None else pad
        w = self.weight(name + ".w", (cout, x.c // groups, k, k))
        h = (x.shape[2] + 2 * pad - k) // stride + 1
        wd = (x.shape[3] + 2 * pad - k) // stride + 1
        shape = [x.shape[0], cout, h, wd]
        op_type = "depthwise_conv2d" if groups == x.c and groups == cout and groups > 1 else "conv2d"
        y = self.b.op(op_type, {"Input": [x.name], "Filter": [w]}, ("Output",), shape, strides=[stride, stride],
                      paddings=[pad, pad], dilations=[1, 1], groups=groups, padding_algorithm="EXPLICIT",
                      data_format="NCHW")
        if bias:
            if bias_value is None:
                bv = (0.1 * self.rng.standard_normal(cout)).astype(np.float32)
            else:
                bv = np.full(cout, bias_value, np.float32)
            bname = self.const_param(name + ".b", bv)
            y = self.b.op("elementwise_add", {"X": [y], "Y": [bname]}, ("Out",), shape, axis=1)
        return Tensor(y, shape)

    def bn(self, x: Tensor, name: str = "bn") -> Tensor:
        c = x.c
        p = {k: self.const_param(f"{name}.{k}", v) for k, v in dict(
            scale=(1.0 + 0.1 * self.rng.standard_normal(c)).astype(np.float32),
            bias=(0.1 * self.rng.standard_normal(c)).astype(np.float32),
            mean=(0.1 * self.rng.standard_normal(c)).astype(np.float32),
            var=(1.0 + 0.1 * self.rng.random(c)).astype(np.float32)).items()}
        y = self.b.op("batch_norm", {"X": [x.name], "Scale": [p["scale"]], "Bias": [p["bias"]], "Mean": [p["mean"]],
                                     "Variance": [p["var"]]}, ("Y",), x.shape, epsilon=1e-5, momentum=0.9,
                      is_test=True, data_layout="NCHW")
        return Tensor(y, x.shape)

    def act(self, x: Tensor, kind: Optional[str]) -> Tensor:
        if kind in (None, "", "none"):
            return x
        attrs = {}
        if kind == "swish":
            attrs = {"beta": 1.0}
        elif kind == "hard_sigmoid":
            attrs = {"slope": 0.2, "offset": 0.5}
        elif kind == "hard_swish":
            attrs = {"threshold": 6.0, "scale": 6.0, "offset": 3.0}
        elif kind == "relu6":
            attrs = {"threshold": 6.0}
        return Tensor(self.b.op(kind, {"X": [x.name]}, ("Out",), x.shape, **attrs), x.shape)

    def conv_bn_act(self, x: Tensor, cout: int, k: int, stride: int = 1, act: Optional[str] = "swish", groups: int = 1,
                    name: str = "cba", pad: Optional[int] = None) -> Tensor:
        y = self.conv(x, cout, k, stride, pad=pad, groups=groups, name=name + ".conv")
        y = self.bn(y, name + ".bn")
        return self.act(y, act)

    def add(self, a: Tensor, b: Tensor) -> Tensor:
        return Tensor(self.b.op("elementwise_add", {"X": [a.name], "Y": [b.name]}, ("Out",), a.shape, axis=-1), a.shape)

    def mul(self, a: Tensor, b: Tensor) -> Tensor:
        return Tensor(self.b.op("elementwise_mul", {"X": [a.name], "Y": [b.name]}, ("Out",), a.shape, axis=-1), a.shape)

    def concat(self, xs: Sequence[Tensor], axis: int = 1) -> Tensor:
        shape = list(xs[0].shape)
        shape[axis] = sum(t.shape[axis] for t in xs)
        return Tensor(self.b.op("concat", {"X": [t.name for t in xs]}, ("Out",), shape, axis=axis), shape)

    def global_avgpool(self, x: Tensor) -> Tensor:
        shape = [x.shape[0], x.c, 1, 1]
        y = self.b.op("pool2d", {"X": [x.name]}, ("Out",), shape, pooling_type="avg", ksize=[1, 1], adaptive=True,
                      global_pooling=False, strides=[1, 1], paddings=[0, 0], exclusive=True, ceil_mode=False,
                      padding_algorithm="EXPLICIT", data_format="NCHW")
        return Tensor(y, shape)

    def pool(self, x: Tensor, k: int, stride: int, pad: int, kind: str = "max", ceil_mode: bool = False) -> Tensor:
        if ceil_mode:
            h = -(-(x.shape[2] + 2 * pad - k) // stride) + 1
            w = -(-(x.shape[3] + 2 * pad - k) // stride) + 1
        else:
            h = (x.shape[2] + 2 * pad - k) // stride + 1
            w = (x.shape[3] + 2 * pad - k) // stride + 1
        shape = [x.shape[0], x.c, h, w]
        y = self.b.op("pool2d", {"X": [x.name]}, ("Out",), shape, pooling_type=kind, ksize=[k, k], adaptive=False,
                      global_pooling=False, strides=[stride, stride], paddings=[pad, pad], exclusive=True,
                      ceil_mode=ceil_mode, padding_algorithm="EXPLICIT", data_format="NCHW")
        return Tensor(y, shape)

    def upsample2x(self, x: Tensor) -> Tensor:
        shape = [x.shape[0], x.c, x.shape[2] * 2, x.shape[3] * 2]
        y = self.b.op("nearest_interp_v2", {"X": [x.name]}, ("Out",), shape, scale=[2.0, 2.0], out_h=-1, out_w=-1,
                      out_d=-1, interp_method="nearest", align_corners=False, align_mode=1, data_layout="NCHW")
        return Tensor(y, shape)

    def reshape(self, x: Tensor, shape: Sequence[int], out_shape: Sequence[int]) -> Tensor:
        y = self.b.op("reshape2", {"X": [x.name]}, ("Out", "XShape"), out_shape, shape=list(shape))
        return Tensor(y, out_shape)

    def transpose(self, x: Tensor, perm: Sequence[int]) -> Tensor:
        shape = [x.shape[p] for p in perm]
        return Tensor(self.b.op("transpose2", {"X": [x.name]}, ("Out", "XShape"), shape, axis=list(perm)), shape)

    def softmax(self, x: Tensor, axis: int) -> Tensor:
        return Tensor(self.b.op("softmax", {"X": [x.name]}, ("Out",), x.shape, axis=axis), x.shape)

    def fetch(self, x: Tensor) -> None:
        self.b.fetch(x.name)

    def serialize(self) -> Tuple[bytes, bytes]:
        return self.b.serialize()


# ---------------------------------------------------------------------- extra layers (OCR / mobile nets)
def _pn_dwconv_bn_act(self, x, k, stride, act, name):
    return self.conv_bn_act(x, x.c, k, stride, act, groups=x.c, name=name)


def _pn_se(self, x, reduction=4, name="se", gate="hard_sigmoid"):
    mid = max(8, x.c // reduction)
    s = self.global_avgpool(x)
    s = self.act(self.conv(s, mid, 1, 1, bias=True, name=name + ".conv1"), "relu")
    s = self.act(self.conv(s, x.c, 1, 1, bias=True, name=name + ".conv2"), gate)
    return self.mul(x, s)


def _pn_deconv2x(self, x, cout, name, bias=True):
    w = self.weight(name + ".w", (x.c, cout, 2, 2))
    shape = [x.shape[0], cout, x.shape[2] * 2, x.shape[3] * 2]
    y = self.b.op("conv2d_transpose", {"Input": [x.name], "Filter": [w]}, ("Output",), shape, strides=[2, 2],
                  paddings=[0, 0], dilations=[1, 1], groups=1, padding_algorithm="EXPLICIT", data_format="NCHW",
                  output_padding=[], output_size=[])
    if bias:
        bname = self.const_param(name + ".b", (0.1 * self.rng.standard_normal(cout)).astype("float32"))
        y = self.b.op("elementwise_add", {"X": [y], "Y": [bname]}, ("Out",), shape, axis=1)
    return Tensor(y, shape)


def _pn_linear(self, x, cout, name, act=None):
    cin = x.shape[-1]
    w = self.weight(name + ".w", (cin, cout), scale=(1.0 / cin) ** 0.5)
    bname = self.const_param(name + ".b", (0.02 * self.rng.standard_normal(cout)).astype("float32"))
    shape = list(x.shape[:-1]) + [cout]
    y = self.b.op("matmul_v2", {"X": [x.name], "Y": [w]}, ("Out",), shape, trans_x=False, trans_y=False)
    y = self.b.op("elementwise_add", {"X": [y], "Y": [bname]}, ("Out",), shape, axis=-1)
    return self.act(Tensor(y, shape), act)


def _pn_layer_norm(self, x, name):
    c = x.shape[-1]
    g = self.const_param(name + ".w", (1.0 + 0.05 * self.rng.standard_normal(c)).astype("float32"))
    bt = self.const_param(name + ".b", (0.02 * self.rng.standard_normal(c)).astype("float32"))
    y = self.b.op("layer_norm", {"X": [x.name], "Scale": [g], "Bias": [bt]}, ("Y", "Mean", "Variance"), x.shape,
                  begin_norm_axis=len(x.shape) - 1, epsilon=1e-6)
    return Tensor(y, x.shape)


PaddleNet.dwconv_bn_act = _pn_dwconv_bn_act
PaddleNet.se = _pn_se
PaddleNet.deconv2x = _pn_deconv2x
PaddleNet.linear = _pn_linear
PaddleNet.layer_norm = _pn_layer_norm
