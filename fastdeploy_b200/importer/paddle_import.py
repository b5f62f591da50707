"""Paddle ``ProgramDesc`` -> IR. One mapper per Paddle operator, honouring the translation
rules the reference applies in paddle2onnx (paddle2onnx/mapper/**): conv padding
algorithms, pool2d adaptive / ceil / exclusive modes, ``*_interp_v2`` coordinate modes,
elementwise ``axis`` broadcasting, ``mul`` / ``matmul_v2`` flattening rules,
``scale`` bias order, ``lookup_table`` padding index, ``multiclass_nms3``.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional

import numpy as np

from ..ir.graph import Graph, ValueInfo
from .paddle_format import PaddleOp, PaddleProgram, parse_params, parse_program

_MAPPERS: Dict[str, Callable] = {}
NP_TO_ONNX_DT = {"float32": 1, "uint8": 2, "int8": 3, "int16": 5, "int32": 6, "int64": 7, "bool": 9, "float16": 10,
                 "float64": 11, "bfloat16": 16}
PD_DT_TO_NP = {0: "bool", 1: "int16", 2: "int32", 3: "int64", 4: "float16", 5: "float32", 6: "float64", 20: "uint8",
               21: "int8", 22: "bfloat16"}


def mapper(*names):
    def deco(fn):
        for n in names:
            _MAPPERS[n] = fn
        return fn
    return deco


def supported_paddle_ops() -> List[str]:
    return sorted(_MAPPERS)


class Ctx:
    def __init__(self, prog: PaddleProgram, graph: Graph):
        self.prog = prog
        self.g = graph

    def rank(self, name: str) -> Optional[int]:
        if name in self.g.initializers:
            return self.g.initializers[name].ndim
        v = self.prog.vars.get(name)
        return len(v.shape) if v is not None else None

    def shape(self, name: str) -> Optional[List[int]]:
        if name in self.g.initializers:
            return list(self.g.initializers[name].shape)
        v = self.prog.vars.get(name)
        return list(v.shape) if v is not None else None

    def dtype(self, name: str) -> str:
        if name in self.g.initializers:
            return self.g.initializers[name].dtype.name
        v = self.prog.vars.get(name)
        return v.dtype if v is not None else "float32"

    def i64(self, values) -> str:
        return self.g.const(np.asarray(values, dtype=np.int64))

    def f32(self, values) -> str:
        return self.g.const(np.asarray(values, dtype=np.float32))

    def emit(self, op: str, inputs, outputs, **attrs):
        return self.g.add_node(op, inputs, outputs, **attrs)


# ------------------------------------------------------------------------- plumbing
@mapper("feed", "fetch")
def _feed_fetch(c: Ctx, op: PaddleOp):
    pass  # handled by the driver


def _simple(onnx_op: str, **fixed):
    def fn(c: Ctx, op: PaddleOp):
        c.emit(onnx_op, [op.input("X")], [op.output("Out")], **fixed)
    return fn


for _pd, _onnx in [("relu", "Relu"), ("sigmoid", "Sigmoid"), ("tanh", "Tanh"), ("exp", "Exp"), ("log", "Log"),
                   ("sqrt", "Sqrt"), ("abs", "Abs"), ("floor", "Floor"), ("ceil", "Ceil"), ("erf", "Erf"),
                   ("round", "Round"), ("sign", "Sign"), ("sin", "Sin"), ("cos", "Cos"), ("reciprocal", "Reciprocal"),
                   ("silu", "Silu"), ("mish", "Mish"), ("softplus", "Softplus"), ("softsign", "Softsign"),
                   ("logical_not", "Not"), ("assign", "Identity"), ("share_data", "Identity")]:
    _MAPPERS[_pd] = _simple(_onnx)


@mapper("relu6")
def _relu6(c, op):
    c.emit("Clip", [op.input("X"), c.f32(0.0), c.f32(op.attr("threshold", 6.0))], [op.output("Out")])


@mapper("leaky_relu")
def _leaky(c, op):
    c.emit("LeakyRelu", [op.input("X")], [op.output("Out")], alpha=float(op.attr("alpha", 0.02)))


@mapper("elu")
def _elu(c, op):
    c.emit("Elu", [op.input("X")], [op.output("Out")], alpha=float(op.attr("alpha", 1.0)))


@mapper("gelu")
def _gelu(c, op):
    c.emit("Gelu", [op.input("X")], [op.output("Out")], approximate="tanh" if op.attr("approximate", False) else "none")


@mapper("swish")
def _swish(c, op):
    beta = float(op.attr("beta", 1.0))
    if beta == 1.0:
        c.emit("Silu", [op.input("X")], [op.output("Out")])
    else:
        t = c.g.op("Mul", op.input("X"), c.f32(beta))
        s = c.g.op("Sigmoid", t)
        c.emit("Mul", [op.input("X"), s], [op.output("Out")])


@mapper("hard_swish")
def _hard_swish(c, op):
    off, thr, sc = op.attr("offset", 3.0), op.attr("threshold", 6.0), op.attr("scale", 6.0)
    if (off, thr, sc) == (3.0, 6.0, 6.0):
        c.emit("HardSwish", [op.input("X")], [op.output("Out")])
    else:
        t = c.g.op("Add", op.input("X"), c.f32(off))
        t = c.g.op("Clip", t, c.f32(0.0), c.f32(thr))
        t = c.g.op("Mul", op.input("X"), t)
        c.emit("Div", [t, c.f32(sc)], [op.output("Out")])


@mapper("hard_sigmoid")
def _hard_sigmoid(c, op):
    c.emit("HardSigmoid", [op.input("X")], [op.output("Out")], alpha=float(op.attr("slope", 0.2)),
           beta=float(op.attr("offset", 0.5)))


@mapper("clip")
def _clip(c, op):
    lo = op.input("Min") or c.f32(op.attr("min", 0.0))
    hi = op.input("Max") or c.f32(op.attr("max", 0.0))
    c.emit("Clip", [op.input("X"), lo, hi], [op.output("Out")])


@mapper("pow")
def _pow(c, op):
    c.emit("Pow", [op.input("X"), c.f32(op.attr("factor", 1.0))], [op.output("Out")])


@mapper("square")
def _square(c, op):
    c.emit("Mul", [op.input("X"), op.input("X")], [op.output("Out")])


@mapper("rsqrt")
def _rsqrt(c, op):
    c.emit("Reciprocal", [c.g.op("Sqrt", op.input("X"))], [op.output("Out")])


@mapper("dropout")
def _dropout(c, op):
    if op.attr("dropout_implementation", "downgrade_in_infer") == "downgrade_in_infer":
        c.emit("Mul", [op.input("X"), c.f32(1.0 - op.attr("dropout_prob", 0.5))], [op.output("Out")])
    else:
        c.emit("Identity", [op.input("X")], [op.output("Out")])


# ------------------------------------------------------------------------- elementwise with axis
def _elementwise(onnx_op: str):
    def fn(c: Ctx, op: PaddleOp):
        x, y = op.input("X"), op.input("Y")
        axis = op.attr("axis", -1)
        rx, ry = c.rank(x), c.rank(y)
        if axis != -1 and rx is not None and ry is not None and ry < rx and axis + ry < rx:
            ys = c.shape(y)
            if y in c.g.initializers:
                y = c.g.const(c.g.initializers[y].reshape(list(ys) + [1] * (rx - axis - ry)))
            else:
                y = c.g.op("Unsqueeze", y, axes=list(range(ry, ry + rx - axis - ry)))
        c.emit(onnx_op, [x, y], [op.output("Out")])
    return fn


for _pd, _onnx in [("elementwise_add", "Add"), ("elementwise_sub", "Sub"), ("elementwise_mul", "Mul"),
                   ("elementwise_div", "Div"), ("elementwise_pow", "Pow"), ("elementwise_max", "Max"),
                   ("elementwise_min", "Min"), ("elementwise_mod", "Mod"), ("equal", "Equal"), ("less_than", "Less"),
                   ("greater_than", "Greater"), ("less_equal", "LessOrEqual"), ("greater_equal", "GreaterOrEqual"),
                   ("logical_and", "And"), ("logical_or", "Or"), ("logical_xor", "Xor")]:
    _MAPPERS[_pd] = _elementwise(_onnx)


@mapper("elementwise_floordiv")
def _floordiv(c, op):
    d = c.g.op("Div", op.input("X"), op.input("Y"))
    if c.dtype(op.input("X")).startswith("float"):
        c.emit("Floor", [d], [op.output("Out")])
    else:
        c.emit("Identity", [d], [op.output("Out")])


@mapper("not_equal")
def _not_equal(c, op):
    c.emit("Not", [c.g.op("Equal", op.input("X"), op.input("Y"))], [op.output("Out")])


@mapper("sum")
def _sum(c, op):
    c.emit("Sum", op.inputs["X"], [op.output("Out")])


@mapper("where")
def _where(c, op):
    c.emit("Where", [op.input("Condition"), op.input("X"), op.input("Y")], [op.output("Out")])


@mapper("scale")
def _scale(c, op):
    x = op.input("X")
    s = op.input("ScaleTensor") or c.f32(op.attr("scale", 1.0))
    b = float(op.attr("bias", 0.0))
    is_float = c.dtype(x).startswith("float") or c.dtype(x) == "bfloat16"
    if not is_float:
        x = c.g.op("Cast", x, to=1)
    if op.attr("bias_after_scale", True):
        t = c.g.op("Mul", x, s)
        out = c.g.op("Add", t, c.f32(b)) if b != 0.0 else t
    else:
        t = c.g.op("Add", x, c.f32(b)) if b != 0.0 else x
        out = c.g.op("Mul", t, s)
    if not is_float:
        c.emit("Cast", [out], [op.output("Out")], to=NP_TO_ONNX_DT[c.dtype(op.input("X"))])
    else:
        c.emit("Identity", [out], [op.output("Out")])


# ------------------------------------------------------------------------- conv / pool / norm
def _conv_pads(op: PaddleOp, nd: int = 2):
    algo = op.attr("padding_algorithm", "EXPLICIT")
    pads = list(op.attr("paddings", [0] * nd))
    if algo == "SAME":
        return {"auto_pad": "SAME_UPPER"}
    if algo == "VALID":
        return {"pads": [0] * (2 * nd)}
    if len(pads) == nd:
        return {"pads": pads + pads}
    # [before0, after0, before1, after1] -> ONNX [before0, before1, after0, after1]
    return {"pads": [pads[2 * i] for i in range(nd)] + [pads[2 * i + 1] for i in range(nd)]}


@mapper("conv2d", "depthwise_conv2d", "conv3d")
def _conv2d(c, op):
    nd = 3 if op.type == "conv3d" else 2
    ins = [op.input("Input"), op.input("Filter")]
    if op.input("Bias"):
        ins.append(op.input("Bias"))
    if op.attr("data_format", "NCHW") not in ("NCHW", "NCDHW", "AnyLayout"):
        raise NotImplementedError("conv2d: only NCHW models are supported")
    c.emit("Conv", ins, [op.output("Output")], strides=list(op.attr("strides", [1] * nd)),
           dilations=list(op.attr("dilations", [1] * nd)), group=int(op.attr("groups", 1)), **_conv_pads(op, nd))


@mapper("conv2d_transpose", "depthwise_conv2d_transpose")
def _conv2d_transpose(c, op):
    attrs = dict(strides=list(op.attr("strides", [1, 1])), dilations=list(op.attr("dilations", [1, 1])),
                 group=int(op.attr("groups", 1)), **_conv_pads(op))
    if op.attr("output_padding"):
        attrs["output_padding"] = list(op.attr("output_padding"))
    c.emit("ConvTranspose", [op.input("Input"), op.input("Filter")], [op.output("Output")], **attrs)


@mapper("batch_norm")
def _batch_norm(c, op):
    c.emit("BatchNormalization", [op.input("X"), op.input("Scale"), op.input("Bias"), op.input("Mean"),
                                  op.input("Variance")], [op.output("Y")], epsilon=float(op.attr("epsilon", 1e-5)))


@mapper("instance_norm")
def _instance_norm(c, op):
    c.emit("InstanceNormalization", [op.input("X"), op.input("Scale"), op.input("Bias")], [op.output("Y")],
           epsilon=float(op.attr("epsilon", 1e-5)))


@mapper("layer_norm")
def _layer_norm(c, op):
    x = op.input("X")
    axis = int(op.attr("begin_norm_axis", 1))
    ins = [x, op.input("Scale") or "", op.input("Bias") or ""]
    c.emit("LayerNormalization", ins, [op.output("Y")], axis=axis, epsilon=float(op.attr("epsilon", 1e-5)))


@mapper("pool2d", "max_pool2d_with_index")
def _pool2d(c, op):
    x, out = op.input("X"), op.output("Out")
    ptype = "max" if op.type == "max_pool2d_with_index" else op.attr("pooling_type", "max")
    k = list(op.attr("ksize", [1, 1]))
    shape = c.shape(x) or [-1, -1, -1, -1]
    if op.attr("global_pooling", False) or (op.attr("adaptive", False) and k == [1, 1]):
        c.emit("GlobalMaxPool" if ptype == "max" else "GlobalAveragePool", [x], [out])
        return
    if op.attr("adaptive", False):
        h, w = shape[2], shape[3]
        if h > 0 and w > 0 and h % k[0] == 0 and w % k[1] == 0:
            st = [h // k[0], w // k[1]]
            ks = [h - (k[0] - 1) * st[0], w - (k[1] - 1) * st[1]]
            c.emit("MaxPool" if ptype == "max" else "AveragePool", [x], [out], kernel_shape=ks, strides=st,
                   pads=[0, 0, 0, 0])
        else:
            c.emit("AdaptivePool2d", [x], [out], pooling_type=ptype, output_size=k, domain="Paddle")
        return
    attrs = dict(kernel_shape=k, strides=list(op.attr("strides", [1, 1])), ceil_mode=int(op.attr("ceil_mode", False)))
    algo = op.attr("padding_algorithm", "EXPLICIT")
    pads = list(op.attr("paddings", [0, 0]))
    if algo == "SAME":
        attrs["auto_pad"] = "SAME_UPPER"
    elif algo == "VALID":
        attrs["pads"] = [0, 0, 0, 0]
    else:
        attrs["pads"] = pads + pads if len(pads) == 2 else [pads[0], pads[2], pads[1], pads[3]]
    if ptype == "max":
        c.emit("MaxPool", [x], [out], **attrs)
    else:
        attrs["count_include_pad"] = 0 if op.attr("exclusive", True) else 1
        c.emit("AveragePool", [x], [out], **attrs)


def _interp(mode: str):
    def fn(c: Ctx, op: PaddleOp):
        x = op.input("X")
        attrs = {"mode": mode}
        if op.attr("align_corners", False):
            attrs["coordinate_transformation_mode"] = "align_corners"
        elif mode == "nearest":
            attrs["coordinate_transformation_mode"] = "asymmetric"
            attrs["nearest_mode"] = "floor"
        elif op.attr("align_mode", 1) == 1 and mode != "cubic":
            attrs["coordinate_transformation_mode"] = "asymmetric"
        else:
            attrs["coordinate_transformation_mode"] = "half_pixel"
        nd = (c.rank(x) or 4) - 2
        sizes = scales = ""
        if op.input("OutSize"):
            head = c.g.op("Slice", c.g.op("Shape", x), c.i64([0]), c.i64([2]), c.i64([0]))
            sizes = c.g.op("Concat", head, c.g.op("Cast", op.input("OutSize"), to=7), axis=0)
        elif op.inputs.get("SizeTensor"):
            head = c.g.op("Slice", c.g.op("Shape", x), c.i64([0]), c.i64([2]), c.i64([0]))
            parts = [c.g.op("Cast", c.g.op("Reshape", t, c.i64([1])), to=7) for t in op.inputs["SizeTensor"]]
            sizes = c.g.op("Concat", head, *parts, axis=0)
        elif op.input("Scale"):
            scales = c.g.op("Concat", c.f32([1.0, 1.0]), op.input("Scale"), axis=0)
        else:
            out_dims = [op.attr(k, -1) for k in (("out_d", "out_h", "out_w")[3 - nd:])]
            if all(d is not None and d > 0 for d in out_dims):
                head = c.g.op("Slice", c.g.op("Shape", x), c.i64([0]), c.i64([2]), c.i64([0]))
                sizes = c.g.op("Concat", head, c.i64(out_dims), axis=0)
            else:
                sc = op.attr("scale", [])
                sc = list(sc) if isinstance(sc, (list, tuple)) else [sc] * nd
                if len(sc) == 1:
                    sc = sc * nd
                scales = c.f32([1.0, 1.0] + [float(s) for s in sc])
        c.emit("Resize", [x, "", scales, sizes] if sizes else [x, "", scales], [op.output("Out")], **attrs)
    return fn


for _pd, _mode in [("nearest_interp_v2", "nearest"), ("nearest_interp", "nearest"), ("bilinear_interp_v2", "linear"),
                   ("bilinear_interp", "linear"), ("bicubic_interp_v2", "cubic"), ("linear_interp_v2", "linear"),
                   ("trilinear_interp_v2", "linear")]:
    _MAPPERS[_pd] = _interp(_mode)


@mapper("pixel_shuffle")
def _pixel_shuffle(c, op):
    c.emit("DepthToSpace", [op.input("X")], [op.output("Out")], blocksize=int(op.attr("upscale_factor", 1)), mode="CRD")


@mapper("pad3d", "pad2d")
def _pad3d(c, op):
    p = list(op.attr("paddings", []))
    rank = c.rank(op.input("X")) or (5 if op.type == "pad3d" else 4)
    nd = rank - 2
    # paddle order: innermost dim first, (before, after) pairs
    before = [0, 0] + [p[2 * (nd - 1 - i)] for i in range(nd)]
    after = [0, 0] + [p[2 * (nd - 1 - i) + 1] for i in range(nd)]
    mode = {"constant": "constant", "reflect": "reflect", "replicate": "edge", "edge": "edge"}[op.attr("mode", "constant")]
    c.emit("Pad", [op.input("X"), c.i64(before + after), c.f32(op.attr("value", op.attr("pad_value", 0.0)))],
           [op.output("Out")], mode=mode)


@mapper("pad")
def _pad(c, op):
    p = list(op.attr("paddings", []))
    nd = len(p) // 2
    c.emit("Pad", [op.input("X"), c.i64([p[2 * i] for i in range(nd)] + [p[2 * i + 1] for i in range(nd)]),
                   c.f32(op.attr("pad_value", 0.0))], [op.output("Out")], mode="constant")


# ------------------------------------------------------------------------- matmul family
@mapper("matmul_v2")
def _matmul_v2(c, op):
    x, y = op.input("X"), op.input("Y")
    if op.attr("trans_x", False):
        r = c.rank(x)
        perm = list(range(r)); perm[-1], perm[-2] = perm[-2], perm[-1]
        x = c.g.op("Transpose", x, perm=perm)
    if op.attr("trans_y", False):
        r = c.rank(y)
        if y in c.g.initializers and r == 2:
            y = c.g.const(np.ascontiguousarray(c.g.initializers[y].T))
        else:
            perm = list(range(r)); perm[-1], perm[-2] = perm[-2], perm[-1]
            y = c.g.op("Transpose", y, perm=perm)
    c.emit("MatMul", [x, y], [op.output("Out")])


@mapper("matmul")
def _matmul(c, op):
    x, y = op.input("X"), op.input("Y")
    if op.attr("transpose_X", False):
        r = c.rank(x); perm = list(range(r)); perm[-1], perm[-2] = perm[-2], perm[-1]
        x = c.g.op("Transpose", x, perm=perm)
    if op.attr("transpose_Y", False):
        r = c.rank(y); perm = list(range(r)); perm[-1], perm[-2] = perm[-2], perm[-1]
        y = c.g.op("Transpose", y, perm=perm)
    alpha = float(op.attr("alpha", 1.0))
    if alpha == 1.0:
        c.emit("MatMul", [x, y], [op.output("Out")])
    else:
        c.emit("Mul", [c.g.op("MatMul", x, y), c.f32(alpha)], [op.output("Out")])


@mapper("bmm")
def _bmm(c, op):
    c.emit("MatMul", [op.input("X"), op.input("Y")], [op.output("Out")])


@mapper("mul")
def _mul(c, op):
    x, y = op.input("X"), op.input("Y")
    xn, yn = int(op.attr("x_num_col_dims", 1)), int(op.attr("y_num_col_dims", 1))
    xf = c.g.op("Flatten", x, axis=xn)
    yf = c.g.op("Flatten", y, axis=yn) if (c.rank(y) or 2) != 2 or yn != 1 else y
    mm = c.g.op("MatMul", xf, yf)
    xs = c.g.op("Slice", c.g.op("Shape", x), c.i64([0]), c.i64([xn]), c.i64([0]))
    ys = c.g.op("Slice", c.g.op("Shape", y), c.i64([yn]), c.i64([1 << 30]), c.i64([0]))
    c.emit("Reshape", [mm, c.g.op("Concat", xs, ys, axis=0)], [op.output("Out")])


@mapper("fc")
def _fc(c, op):
    x = c.g.op("Flatten", op.input("Input"), axis=int(op.attr("in_num_col_dims", 1)))
    ins = [x, op.input("W")] + ([op.input("Bias")] if op.input("Bias") else [])
    out = c.g.op("Gemm", *ins)
    act = op.attr("activation_type", "")
    c.emit("Relu" if act == "relu" else "Identity", [out], [op.output("Out")])


@mapper("softmax")
def _softmax(c, op):
    # the IR is opset 13: Softmax normalises along one arbitrary axis
    c.emit("Softmax", [op.input("X")], [op.output("Out")], axis=int(op.attr("axis", -1)), _opset=13)


@mapper("log_softmax")
def _log_softmax(c, op):
    c.emit("LogSoftmax", [op.input("X")], [op.output("Out")], axis=int(op.attr("axis", -1)))


@mapper("lookup_table_v2", "lookup_table")
def _lookup(c, op):
    ids, w = op.input("Ids"), op.input("W")
    pad = int(op.attr("padding_idx", -1))
    if pad != -1 and w in c.g.initializers:
        tab = c.g.initializers[w].copy()
        tab[pad if pad >= 0 else tab.shape[0] + pad] = 0
        w = c.g.const(tab)
    if op.type == "lookup_table":
        ids = c.g.op("Squeeze", ids, axes=[-1])
    c.emit("Gather", [w, ids], [op.output("Out")], axis=0)


# ------------------------------------------------------------------------- shape manipulation
@mapper("reshape2", "reshape")
def _reshape(c, op):
    x = op.input("X")
    if op.inputs.get("ShapeTensor"):
        parts = [c.g.op("Cast", c.g.op("Reshape", t, c.i64([1])), to=7) for t in op.inputs["ShapeTensor"]]
        shape = c.g.op("Concat", *parts, axis=0)
    elif op.input("Shape"):
        shape = c.g.op("Cast", op.input("Shape"), to=7)
    else:
        shape = c.i64(op.attr("shape", []))
    c.emit("Reshape", [x, shape], [op.output("Out")])


@mapper("transpose2", "transpose")
def _transpose(c, op):
    c.emit("Transpose", [op.input("X")], [op.output("Out")], perm=list(op.attr("axis", [])))


@mapper("flatten_contiguous_range")
def _flatten_range(c, op):
    x = op.input("X")
    start, stop = int(op.attr("start_axis", 1)), int(op.attr("stop_axis", -1))
    r = c.rank(x)
    if r is None:
        raise NotImplementedError("flatten_contiguous_range needs a known input rank")
    start = start if start >= 0 else r + start
    stop = stop if stop >= 0 else r + stop
    shape = [0] * start + [-1] + [0] * (r - 1 - stop)
    if r - 1 - stop > 0:
        # trailing zeros would refer to the wrong input dims: build the shape at run time
        sh = c.g.op("Shape", x)
        head = c.g.op("Slice", sh, c.i64([0]), c.i64([start]), c.i64([0]))
        tail = c.g.op("Slice", sh, c.i64([stop + 1]), c.i64([r]), c.i64([0]))
        c.emit("Reshape", [x, c.g.op("Concat", head, c.i64([-1]), tail, axis=0)], [op.output("Out")])
    else:
        c.emit("Reshape", [x, c.i64(shape)], [op.output("Out")])


@mapper("flatten2", "flatten")
def _flatten2(c, op):
    c.emit("Flatten", [op.input("X")], [op.output("Out")], axis=int(op.attr("axis", 1)))


@mapper("squeeze2", "squeeze")
def _squeeze(c, op):
    axes = list(op.attr("axes", []))
    if axes:
        c.emit("Squeeze", [op.input("X")], [op.output("Out")], axes=axes)
    else:
        c.emit("Squeeze", [op.input("X")], [op.output("Out")])


@mapper("unsqueeze2", "unsqueeze")
def _unsqueeze(c, op):
    c.emit("Unsqueeze", [op.input("X")], [op.output("Out")], axes=list(op.attr("axes", [])))


@mapper("concat")
def _concat(c, op):
    c.emit("Concat", op.inputs["X"], [op.output("Out")], axis=int(op.attr("axis", 0)))


@mapper("stack")
def _stack(c, op):
    axis = int(op.attr("axis", 0))
    parts = [c.g.op("Unsqueeze", x, axes=[axis]) for x in op.inputs["X"]]
    c.emit("Concat", parts, [op.output("Y")], axis=axis)


@mapper("unstack")
def _unstack(c, op):
    axis = int(op.attr("axis", 0))
    outs = op.outputs["Y"]
    parts = c.g.add_node("Split", [op.input("X")], n_out=len(outs), axis=axis) if len(outs) > 1 else [op.input("X")]
    for p, o in zip(parts, outs):
        c.emit("Squeeze", [p], [o], axes=[axis])


@mapper("split")
def _split(c, op):
    axis = int(op.attr("axis", 0))
    sections = list(op.attr("sections", []))
    outs = op.outputs["Out"]
    if sections and -1 in sections:
        total = (c.shape(op.input("X")) or [])[axis]
        sections[sections.index(-1)] = total - sum(s for s in sections if s > 0)
    if sections:
        c.emit("Split", [op.input("X"), c.i64(sections)], outs, axis=axis)
    else:
        c.emit("Split", [op.input("X")], outs, axis=axis)


@mapper("slice")
def _slice(c, op):
    axes = list(op.attr("axes", []))
    starts = op.input("StartsTensor") or c.i64(op.attr("starts", []))
    ends = op.input("EndsTensor") or c.i64(op.attr("ends", []))
    dec = list(op.attr("decrease_axis", []) or [])
    if dec:
        t = c.g.op("Slice", op.input("Input"), starts, ends, c.i64(axes))
        c.emit("Squeeze", [t], [op.output("Out")], axes=dec)
    else:
        c.emit("Slice", [op.input("Input"), starts, ends, c.i64(axes)], [op.output("Out")])


@mapper("strided_slice")
def _strided_slice(c, op):
    c.emit("Slice", [op.input("Input"), c.i64(op.attr("starts", [])), c.i64(op.attr("ends", [])),
                     c.i64(op.attr("axes", [])), c.i64(op.attr("strides", []))], [op.output("Out")])


@mapper("gather")
def _gather(c, op):
    c.emit("Gather", [op.input("X"), op.input("Index")], [op.output("Out")], axis=int(op.attr("axis", 0)))


@mapper("gather_nd")
def _gather_nd(c, op):
    c.emit("GatherND", [op.input("X"), op.input("Index")], [op.output("Out")])


@mapper("index_select")
def _index_select(c, op):
    c.emit("Gather", [op.input("X"), op.input("Index")], [op.output("Out")], axis=int(op.attr("dim", 0)))


@mapper("take_along_axis")
def _take_along(c, op):
    c.emit("GatherElements", [op.input("Input"), op.input("Index")], [op.output("Result")], axis=int(op.attr("Axis", 0)))


@mapper("shape")
def _shape(c, op):
    c.emit("Cast", [c.g.op("Shape", op.input("Input"))], [op.output("Out")], to=6)


@mapper("size")
def _size(c, op):
    c.emit("Size", [op.input("Input")], [op.output("Out")])


@mapper("cast")
def _cast(c, op):
    c.emit("Cast", [op.input("X")], [op.output("Out")], to=NP_TO_ONNX_DT[PD_DT_TO_NP[int(op.attr("out_dtype", 5))]])


@mapper("fill_constant")
def _fill_constant(c, op):
    dtype = PD_DT_TO_NP[int(op.attr("dtype", 5))]
    sval = op.attr("str_value", "")
    value = float(sval) if sval not in ("", None) else op.attr("value", 0.0)
    if op.input("ShapeTensor") or op.inputs.get("ShapeTensorList"):
        if op.input("ShapeTensor"):
            shape = c.g.op("Cast", op.input("ShapeTensor"), to=7)
        else:
            parts = [c.g.op("Cast", c.g.op("Reshape", t, c.i64([1])), to=7) for t in op.inputs["ShapeTensorList"]]
            shape = c.g.op("Concat", *parts, axis=0)
        c.emit("ConstantOfShape", [shape], [op.output("Out")], value=np.asarray([value], dtype=dtype))
    else:
        c.g.initializers[op.output("Out")] = np.full(list(op.attr("shape", [])), value, dtype=dtype)


@mapper("fill_any_like", "fill_zeros_like")
def _fill_like(c, op):
    dt = int(op.attr("dtype", -1))
    dtype = PD_DT_TO_NP[dt] if dt >= 0 else c.dtype(op.input("X"))
    value = 0.0 if op.type == "fill_zeros_like" else op.attr("value", 0.0)
    c.emit("ConstantOfShape", [c.g.op("Shape", op.input("X"))], [op.output("Out")],
           value=np.asarray([value], dtype=dtype))


@mapper("assign_value")
def _assign_value(c, op):
    dtype = PD_DT_TO_NP[int(op.attr("dtype", 5))]
    for key in ("fp32_values", "int32_values", "int64_values", "bool_values"):
        vals = op.attr(key, None)
        if vals:
            break
    c.g.initializers[op.output("Out")] = np.asarray(vals, dtype=dtype).reshape(list(op.attr("shape", [])))


@mapper("expand_v2")
def _expand_v2(c, op):
    shape = op.input("Shape") or c.i64([1 if d == -1 else d for d in op.attr("shape", [])])
    c.emit("Expand", [op.input("X"), shape], [op.output("Out")])


@mapper("expand_as_v2")
def _expand_as(c, op):
    c.emit("Expand", [op.input("X"), c.i64(op.attr("target_shape", []))], [op.output("Out")])


@mapper("tile")
def _tile(c, op):
    reps = list(op.attr("repeat_times", []))
    r = c.rank(op.input("X")) or len(reps)
    reps = [1] * (r - len(reps)) + reps
    c.emit("Tile", [op.input("X"), c.i64(reps)], [op.output("Out")])


@mapper("range")
def _range(c, op):
    sq = [c.g.op("Squeeze", op.input(k)) for k in ("Start", "End", "Step")]
    c.emit("Range", sq, [op.output("Out")])


@mapper("arg_max", "arg_min")
def _argmax(c, op):
    x = op.input("X")
    if op.attr("flatten", False):
        x = c.g.op("Reshape", x, c.i64([-1]))
    t = c.g.op("ArgMax" if op.type == "arg_max" else "ArgMin", x, axis=int(op.attr("axis", 0)),
               keepdims=int(op.attr("keepdims", False)))
    dt = int(op.attr("dtype", 3))
    c.emit("Cast", [t], [op.output("Out")], to=NP_TO_ONNX_DT[PD_DT_TO_NP.get(dt, "int64")])


@mapper("top_k_v2", "top_k")
def _topk(c, op):
    k = op.input("K") or c.i64([op.attr("k", 1)])
    if op.input("K"):
        k = c.g.op("Cast", c.g.op("Reshape", k, c.i64([1])), to=7)
    c.emit("TopK", [op.input("X"), k], [op.output("Out"), op.output("Indices")], axis=int(op.attr("axis", -1)),
           largest=int(op.attr("largest", True)))


@mapper("cumsum")
def _cumsum(c, op):
    c.emit("CumSum", [op.input("X"), c.i64(op.attr("axis", -1))], [op.output("Out")])


def _reduce(onnx_op: str):
    def fn(c: Ctx, op: PaddleOp):
        dims = list(op.attr("dim", [0]))
        attrs = {"keepdims": int(op.attr("keep_dim", False))}
        if not op.attr("reduce_all", False):
            attrs["axes"] = dims
        c.emit(onnx_op, [op.input("X")], [op.output("Out")], **attrs)
    return fn


for _pd, _onnx in [("reduce_mean", "ReduceMean"), ("reduce_sum", "ReduceSum"), ("reduce_max", "ReduceMax"),
                   ("reduce_min", "ReduceMin"), ("reduce_prod", "ReduceProd")]:
    _MAPPERS[_pd] = _reduce(_onnx)


@mapper("mean")
def _mean(c, op):
    c.emit("ReduceMean", [op.input("X")], [op.output("Out")], keepdims=0)


@mapper("p_norm")
def _p_norm(c, op):
    p = float(op.attr("porder", 2.0))
    onnx_op = "ReduceL2" if p == 2.0 else "ReduceL1"
    c.emit(onnx_op, [op.input("X")], [op.output("Out")], axes=[int(op.attr("axis", -1))],
           keepdims=int(op.attr("keepdim", False)))


@mapper("norm")
def _norm(c, op):
    n = c.g.op("ReduceL2", op.input("X"), axes=[int(op.attr("axis", 1))], keepdims=1)
    n = c.g.op("Add", n, c.f32(op.attr("epsilon", 1e-10)))
    c.emit("Div", [op.input("X"), n], [op.output("Out")])


@mapper("multiclass_nms3", "multiclass_nms2", "multiclass_nms")
def _multiclass_nms(c, op):
    outs = [op.output("Out"), op.output("Index") or c.g.unique("nms_index"), op.output("NmsRoisNum") or c.g.unique("nms_num")]
    c.emit("MultiClassNMS", [op.input("BBoxes"), op.input("Scores")], outs, domain="Paddle",
           background_label=int(op.attr("background_label", -1)), keep_top_k=int(op.attr("keep_top_k", 100)),
           nms_eta=float(op.attr("nms_eta", 1.0)), nms_threshold=float(op.attr("nms_threshold", 0.5)),
           nms_top_k=int(op.attr("nms_top_k", 1000)), normalized=int(op.attr("normalized", True)),
           score_threshold=float(op.attr("score_threshold", 0.01)))


# ------------------------------------------------------------------------- driver
def _custom_mapper(export_name: str):
    """A Paddle operator the caller deploys as a custom operator of its own (paddle2onnx/converter.h:24-34): it goes
    through as one node of domain ``custom`` with every input and output in the order of the op's slots and the
    scalar / list attributes copied."""
    def fn(c: Ctx, op: PaddleOp):
        ins = [a for k in sorted(op.inputs) for a in op.inputs[k]]
        outs = [a for k in sorted(op.outputs) for a in op.outputs[k]]
        attrs = {k: v for k, v in op.attrs.items()
                 if isinstance(v, (bool, int, float, str)) or (isinstance(v, list) and v and not isinstance(v[0], dict))}
        attrs["input_slots"] = [f"{k}:{len(op.inputs[k])}" for k in sorted(op.inputs)]
        attrs["output_slots"] = [f"{k}:{len(op.outputs[k])}" for k in sorted(op.outputs)]
        c.g.add_node(export_name, ins, outs, domain="custom", **attrs)
    return fn


def import_program(prog: PaddleProgram, params: Dict[str, np.ndarray], name: str = "paddle_model",
                   custom_ops: Optional[Dict[str, str]] = None) -> Graph:
    g = Graph(name, opset=13)
    c = Ctx(prog, g)
    from . import paddle_control_flow as cf
    mappers = dict(_MAPPERS)
    for pd_type, export_name in (custom_ops or {}).items():
        mappers[pd_type] = _custom_mapper(export_name or pd_type)
    for name, fn in cf.CONTROL_MAPPERS.items():
        mappers[name] = (lambda f: lambda ctx, op: f(ctx, op, mappers))(fn)
    all_ops = list(prog.ops) + [op for _, ops in prog.sub_blocks for op in ops]
    unsupported = sorted({op.type for op in all_ops if op.type not in mappers})
    if unsupported:
        raise NotImplementedError(f"paddle importer: unsupported operators {unsupported}")
    for k, v in params.items():
        g.initializers[k] = v
    for fname in prog.feed_names():
        v = prog.vars[fname]
        g.inputs.append(ValueInfo(fname, v.dtype, [d if d >= 0 else "dyn" for d in v.shape]))
    # Programs with control flow (or in-place ops) are not in single-assignment form: rename as we go.
    in_place = any(op.type in cf.CONTROL_MAPPERS for op in all_ops)
    if in_place:
        c.prog = cf._scope_program(prog, {}, {})
        c.renamer = cf.Renamer(set(params) | set(prog.feed_names()) | {"feed", "fetch"})
        for op in prog.ops:
            if op.type in ("feed", "fetch"):
                continue
            cf.run_op(c, op, mappers)
    else:
        for op in prog.ops:
            mappers[op.type](c, op)
    for fname in prog.fetch_names():
        v = prog.vars.get(fname)
        out_name = c.renamer.read(fname) if in_place else fname
        g.outputs.append(ValueInfo(out_name, v.dtype if v else "float32",
                                   [d if d >= 0 else "dyn" for d in v.shape] if v else None))
    for vname, v in prog.vars.items():
        if not v.persistable and v.shape:
            g.value_info[vname] = ValueInfo(vname, v.dtype, [d if d >= 0 else "dyn" for d in v.shape])
    g.metadata["source_format"] = "paddle"
    return g


def load_paddle(model_bytes: bytes, params_bytes: Optional[bytes], name: str = "paddle_model",
                custom_ops: Optional[Dict[str, str]] = None) -> Graph:
    """``custom_ops``: Paddle operator type -> name of the custom operator it is exported as (for operators the
    deployment provides itself)."""
    prog = parse_program(model_bytes)
    params = parse_params(prog, params_bytes) if params_bytes else {}
    return import_program(prog, params, name, custom_ops)


from . import paddle_ops_extra  # noqa: E402,F401  (registers the second batch of mappers)
