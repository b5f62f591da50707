"""Second batch of Paddle operator mappers: quantise / dequantise, detection heads (``yolo_box``, ``roi_align``),
recurrent layers (``rnn``), normalisations, indexing and a long tail of activations and tensor utilities.

Each mapper cites the reference's converter for the same operator (paths under paddle2onnx/mapper/); semantics
follow the Paddle kernels those converters translate. Compositions use operators the interpreter and the executor
already know, so a model that contains them needs nothing new at run time.
"""
from __future__ import annotations

import numpy as np

from .paddle_import import _MAPPERS, Ctx, PaddleOp, _simple, mapper

INT_MAX = 2 ** 31 - 1

# paddle2onnx/mapper/activation/activation.cc: one ONNX operator each
for _pd, _onnx in [("acos", "Acos"), ("asin", "Asin"), ("atan", "Atan"), ("cosh", "Cosh"), ("sinh", "Sinh"), ("tan", "Tan")]:
    _MAPPERS[_pd] = _simple(_onnx)


# ------------------------------------------------------------------------- quantisation
def _onnx_scale(c: Ctx, name: str, bits: int):
    """Paddle stores the clipping range (absolute maximum); ONNX wants the step: range / (2^(bits-1) - 1)
    (paddle2onnx/mapper/quantize/quantize_linear.cc:40-70)."""
    qmax = float(2 ** (bits - 1) - 1)
    if name in c.g.initializers:
        return c.g.const((np.asarray(c.g.initializers[name], np.float32) / qmax).astype(np.float32), prefix="qscale")
    return c.g.op("Div", name, c.f32(qmax))


@mapper("quantize_linear")
def _quantize_linear(c: Ctx, op: PaddleOp):
    bits = int(op.attr("bit_length", 8))
    axis = int(op.attr("quant_axis", -1))
    scale = _onnx_scale(c, op.input("Scale"), bits)
    ins = [op.input("X"), scale]
    if op.input("ZeroPoint") and op.input("ZeroPoint") in c.g.initializers:
        ins.append(c.g.const(np.asarray(c.g.initializers[op.input("ZeroPoint")]).astype(np.int8), prefix="qzp"))
    c.emit("QuantizeLinear", ins, [op.output("Y")], axis=axis if axis >= 0 else 1)


@mapper("dequantize_linear")
def _dequantize_linear(c: Ctx, op: PaddleOp):
    """paddle2onnx/mapper/quantize/dequantize_linear.cc:18-80. An int8 weight with a per-channel range becomes
    ``DequantizeLinear(w, range / 127, axis)``, which constant folding turns into float weights."""
    bits = int(op.attr("bit_length", 8))
    axis = int(op.attr("quant_axis", -1))
    scale = _onnx_scale(c, op.input("Scale"), bits)
    ins = [op.input("X"), scale]
    if op.input("ZeroPoint") and op.input("ZeroPoint") in c.g.initializers:
        ins.append(c.g.const(np.asarray(c.g.initializers[op.input("ZeroPoint")]).astype(np.int8), prefix="qzp"))
    c.emit("DequantizeLinear", ins, [op.output("Y")], axis=axis if axis >= 0 else 1)


# ------------------------------------------------------------------------- activations
@mapper("atan2")
def _atan2(c, op):
    c.emit("Atan2", [op.input("X1"), op.input("X2")], [op.output("Out")], domain="fdb")


@mapper("brelu")
def _brelu(c, op):
    c.emit("Clip", [op.input("X"), c.f32(op.attr("t_min", 0.0)), c.f32(op.attr("t_max", 24.0))], [op.output("Out")])


@mapper("hard_shrink")
def _hard_shrink(c, op):
    c.emit("Shrink", [op.input("X")], [op.output("Out")], lambd=float(op.attr("threshold", 0.5)), bias=0.0)


@mapper("softshrink")
def _softshrink(c, op):
    lam = float(op.attr("lambda", 0.5))
    c.emit("Shrink", [op.input("X")], [op.output("Out")], lambd=lam, bias=lam)


@mapper("tanh_shrink")
def _tanh_shrink(c, op):
    c.emit("Sub", [op.input("X"), c.g.op("Tanh", op.input("X"))], [op.output("Out")])


@mapper("thresholded_relu")
def _thresholded_relu(c, op):
    c.emit("ThresholdedRelu", [op.input("X")], [op.output("Out")], alpha=float(op.attr("threshold", 1.0)))


@mapper("logsigmoid")
def _logsigmoid(c, op):
    # log(sigmoid(x)) = -softplus(-x), stable for large |x|
    c.emit("Neg", [c.g.op("Softplus", c.g.op("Neg", op.input("X")))], [op.output("Out")])


@mapper("log10", "log2")
def _log_base(c, op):
    base = 10.0 if op.type == "log10" else 2.0
    c.emit("Div", [c.g.op("Log", op.input("X")), c.f32(np.log(base))], [op.output("Out")])


@mapper("log1p")
def _log1p(c, op):
    c.emit("Log", [c.g.op("Add", op.input("X"), c.f32(1.0))], [op.output("Out")])


@mapper("selu")
def _selu(c, op):
    c.emit("Selu", [op.input("X")], [op.output("Out")], alpha=float(op.attr("alpha", 1.6732632423543772)),
           gamma=float(op.attr("scale", 1.0507009873554805)))


@mapper("prelu")
def _prelu(c, op):
    """paddle2onnx/mapper/activation/activation.cc PReluMapper: the slope broadcasts over the trailing dimensions."""
    alpha = op.input("Alpha")
    rank = c.rank(op.input("X")) or 4
    if op.attr("mode", "all") == "channel" and alpha in c.g.initializers and rank > 2:
        a = np.asarray(c.g.initializers[alpha]).reshape(-1)
        alpha = c.g.const(a.reshape([-1] + [1] * (rank - 2)).astype(np.float32), prefix="prelu_alpha")
    c.emit("PRelu", [op.input("X"), alpha], [op.output("Out")])


# ------------------------------------------------------------------------- creation / shape utilities
@mapper("expand")
def _expand_v1(c, op):
    times = op.input("ExpandTimes") or c.i64(op.attr("expand_times", []))
    c.emit("Tile", [op.input("X"), times], [op.output("Out")])


@mapper("eye")
def _eye(c, op):
    from .paddle_import import PD_DT_TO_NP as PD_DTYPE
    rows = int(op.attr("num_rows"))
    cols = int(op.attr("num_columns", -1))
    dt = PD_DTYPE.get(int(op.attr("dtype", 5)), "float32")
    val = np.eye(rows, cols if cols > 0 else rows).astype(dt)
    c.emit("Identity", [c.g.const(val, prefix="eye")], [op.output("Out")])


@mapper("fill_constant_batch_size_like")
def _fill_bsl(c, op):
    """Output shape = attr ``shape`` with dimension ``output_dim_idx`` taken from the input's ``input_dim_idx``
    (paddle2onnx/mapper/tensor/fill_like.cc)."""
    from .paddle_import import PD_DT_TO_NP as PD_DTYPE
    shape = [int(d) for d in op.attr("shape")]
    i_idx, o_idx = int(op.attr("input_dim_idx", 0)), int(op.attr("output_dim_idx", 0))
    dt = PD_DTYPE.get(int(op.attr("dtype", 5)), "float32")
    value = op.attr("str_value", "") or op.attr("value", 0.0)
    batch = c.g.op("Slice", c.g.op("Shape", op.input("Input")), c.i64([i_idx]), c.i64([i_idx + 1]), c.i64([0]))
    parts = []
    if o_idx > 0:
        parts.append(c.i64(shape[:o_idx]))
    parts.append(batch)
    if o_idx + 1 < len(shape):
        parts.append(c.i64(shape[o_idx + 1:]))
    full = parts[0] if len(parts) == 1 else c.g.op("Concat", *parts, axis=0)
    c.emit("ConstantOfShape", [full], [op.output("Out")], value=np.asarray([float(value)], dtype=dt))


@mapper("flip")
def _flip(c, op):
    c.emit("Flip", [op.input("X")], [op.output("Out")], axes=[int(a) for a in op.attr("axis", [])], domain="fdb")


@mapper("gaussian_random")
def _gaussian_random(c, op):
    from .paddle_import import PD_DT_TO_NP as PD_DTYPE
    dt = {"float32": 1, "float64": 11, "float16": 10}[PD_DTYPE.get(int(op.attr("dtype", 5)), "float32")]
    c.emit("RandomNormal", [], [op.output("Out")], shape=[int(d) for d in op.attr("shape")], mean=float(op.attr("mean", 0.0)),
           scale=float(op.attr("std", 1.0)), seed=int(op.attr("seed", 0)), dtype=dt)


@mapper("linspace")
def _linspace(c, op):
    """start + arange(num) * (stop - start) / (num - 1) (paddle2onnx/mapper/tensor/linspace.cc)."""
    start, stop, num = op.input("Start"), op.input("Stop"), op.input("Num")
    if all(n in c.g.initializers for n in (start, stop, num)):
        a, b = float(c.g.initializers[start].reshape(-1)[0]), float(c.g.initializers[stop].reshape(-1)[0])
        n = int(c.g.initializers[num].reshape(-1)[0])
        c.emit("Identity", [c.g.const(np.linspace(a, b, n).astype(np.float32), prefix="linspace")], [op.output("Out")])
        return
    n = c.g.op("Cast", c.g.op("Reshape", num, c.i64([])), to=7)
    idx = c.g.op("Cast", c.g.op("Range", c.i64(0), n, c.i64(1)), to=1)
    s = c.g.op("Cast", c.g.op("Reshape", start, c.i64([])), to=1)
    e = c.g.op("Cast", c.g.op("Reshape", stop, c.i64([])), to=1)
    denom = c.g.op("Max", c.g.op("Sub", c.g.op("Cast", n, to=1), c.f32(1.0)), c.f32(1.0))
    step = c.g.op("Div", c.g.op("Sub", e, s), denom)
    c.emit("Add", [c.g.op("Mul", idx, step), s], [op.output("Out")])


@mapper("meshgrid")
def _meshgrid(c, op):
    xs, outs = op.inputs["X"], op.outputs["Out"]
    sizes = [c.g.op("Reshape", c.g.op("Size", x), c.i64([1])) for x in xs]
    full = c.g.op("Concat", *sizes, axis=0)
    for i, (x, o) in enumerate(zip(xs, outs)):
        shape = [1] * len(xs)
        shape[i] = -1
        c.emit("Expand", [c.g.op("Reshape", x, c.i64(shape)), full], [o])


@mapper("mv")
def _mv(c, op):
    c.emit("MatMul", [op.input("X"), op.input("Vec")], [op.output("Out")])


@mapper("dot")
def _dot(c, op):
    c.emit("ReduceSum", [c.g.op("Mul", op.input("X"), op.input("Y"))], [op.output("Out")], axes=[-1], keepdims=0)


@mapper("dist")
def _dist(c, op):
    """p-norm of x - y over all elements (paddle2onnx/mapper/tensor/dist.cc)."""
    p = float(op.attr("p", 2.0))
    d = c.g.op("Abs", c.g.op("Sub", op.input("X"), op.input("Y")))
    if p == float("inf"):
        r = c.g.op("ReduceMax", d, keepdims=0)
    elif p == float("-inf"):
        r = c.g.op("ReduceMin", d, keepdims=0)
    elif p == 0.0:
        r = c.g.op("ReduceSum", c.g.op("Cast", c.g.op("Greater", d, c.f32(0.0)), to=1), keepdims=0)
    else:
        r = c.g.op("Pow", c.g.op("ReduceSum", c.g.op("Pow", d, c.f32(p)), keepdims=0), c.f32(1.0 / p))
    c.emit("Reshape", [r, c.i64([1])], [op.output("Out")])


@mapper("one_hot_v2")
def _one_hot_v2(c, op):
    depth = op.input("depth_tensor") or c.i64([int(op.attr("depth"))])
    c.emit("OneHot", [op.input("X"), depth, c.f32([0.0, 1.0])], [op.output("Out")], axis=-1)


def _reduce_bool(onnx_op: str):
    def fn(c: Ctx, op: PaddleOp):
        attrs = {"keepdims": int(op.attr("keep_dim", False))}
        if not op.attr("reduce_all", False):
            attrs["axes"] = list(op.attr("dim", [0]))
        t = c.g.op(onnx_op, c.g.op("Cast", op.input("X"), to=6), **attrs)
        c.emit("Cast", [t], [op.output("Out")], to=9)
    return fn


_MAPPERS["reduce_all"] = _reduce_bool("ReduceMin")
_MAPPERS["reduce_any"] = _reduce_bool("ReduceMax")


@mapper("logsumexp")
def _logsumexp(c, op):
    attrs = {"keepdims": int(op.attr("keepdim", False))}
    if not op.attr("reduce_all", False):
        attrs["axes"] = list(op.attr("axis", [0]))
    c.emit("ReduceLogSumExp", [op.input("X")], [op.output("Out")], **attrs)


@mapper("index_sample")
def _index_sample(c, op):
    c.emit("GatherElements", [op.input("X"), op.input("Index")], [op.output("Out")], axis=1)


@mapper("argsort")
def _argsort(c, op):
    """TopK over the whole axis (paddle2onnx/mapper/tensor/argsort.cc)."""
    axis = int(op.attr("axis", -1))
    k = c.g.op("Slice", c.g.op("Shape", op.input("X")), c.i64([axis]), c.i64([axis + 1 if axis != -1 else INT_MAX]), c.i64([0]))
    c.emit("TopK", [op.input("X"), k], [op.output("Out"), op.output("Indices")], axis=axis,
           largest=int(bool(op.attr("descending", False))))


@mapper("where_index")
def _where_index(c, op):
    c.emit("Transpose", [c.g.op("NonZero", op.input("Condition"))], [op.output("Out")], perm=[1, 0])


@mapper("scatter")
def _scatter(c, op):
    """Rows ``Ids`` of ``X`` replaced (``overwrite``) or accumulated (paddle2onnx/mapper/tensor/scatter.cc)."""
    ids = c.g.op("Reshape", c.g.op("Cast", op.input("Ids"), to=7), c.i64([-1, 1]))
    if op.attr("overwrite", True):
        c.emit("ScatterND", [op.input("X"), ids, op.input("Updates")], [op.output("Out")])
    else:
        # accumulate mode first zeroes the touched rows, then adds every update
        zero = c.g.op("Mul", op.input("Updates"), c.f32(0.0))
        base = c.g.op("ScatterND", op.input("X"), ids, zero)
        c.emit("ScatterND", [base, ids, op.input("Updates")], [op.output("Out")], reduction="add")


@mapper("scatter_nd_add")
def _scatter_nd_add(c, op):
    c.emit("ScatterND", [op.input("X"), c.g.op("Cast", op.input("Index"), to=7), op.input("Updates")], [op.output("Out")],
           reduction="add")


@mapper("unique")
def _unique(c, op):
    axis = op.attr("axis", [])
    attrs = {"sorted": 1}
    if axis:
        attrs["axis"] = int(axis[0])
    outs = [op.output("Out"), op.output("Indices") or "", op.output("Index") or "", op.output("Counts") or ""]
    c.emit("Unique", [op.input("X")], outs, **attrs)


@mapper("partial_concat", "partial_sum")
def _partial(c, op):
    start, length = int(op.attr("start_index", 0)), int(op.attr("length", -1))
    end = INT_MAX if length < 0 else start + length
    parts = [c.g.op("Slice", x, c.i64([start]), c.i64([end]), c.i64([1])) for x in op.inputs["X"]]
    if op.type == "partial_concat":
        c.emit("Concat", parts, [op.output("Out")], axis=1)
    else:
        c.emit("Sum", parts, [op.output("Out")])


# ------------------------------------------------------------------------- normalisation / affine
@mapper("group_norm")
def _group_norm(c, op):
    """paddle2onnx/mapper/nn/group_norm.cc: NCHW input, per-channel scale and bias."""
    x = op.input("X")
    cdim = (c.shape(x) or [0, 0])[1]
    scale = op.input("Scale") or c.f32(np.ones(cdim, np.float32))
    bias = op.input("Bias") or c.f32(np.zeros(cdim, np.float32))
    c.emit("GroupNormalization", [x, scale, bias], [op.output("Y")], epsilon=float(op.attr("epsilon", 1e-5)),
           num_groups=int(op.attr("groups")))


@mapper("affine_channel")
def _affine_channel(c, op):
    rank = c.rank(op.input("X")) or 4
    shape = [1, -1] + [1] * (rank - 2)
    s = c.g.op("Reshape", op.input("Scale"), c.i64(shape))
    b = c.g.op("Reshape", op.input("Bias"), c.i64(shape))
    c.emit("Add", [c.g.op("Mul", op.input("X"), s), b], [op.output("Out")])


@mapper("data_norm")
def _data_norm(c, op):
    """(x - BatchSum / BatchSize) * sqrt(BatchSize / BatchSquareSum) (paddle2onnx/mapper/nn/data_norm.cc)."""
    size, total, sq = op.input("BatchSize"), op.input("BatchSum"), op.input("BatchSquareSum")
    mean = c.g.op("Div", total, size)
    scale = c.g.op("Sqrt", c.g.op("Div", size, sq))
    c.emit("Mul", [c.g.op("Sub", op.input("X"), mean), scale], [op.output("Y")])


@mapper("temporal_shift")
def _temporal_shift(c, op):
    c.emit("TemporalShift", [op.input("X")], [op.output("Out")], seg_num=int(op.attr("seg_num")),
           shift_ratio=float(op.attr("shift_ratio", 0.25)), domain="fdb")


@mapper("softmax_with_cross_entropy")
def _softmax_ce(c, op):
    axis = int(op.attr("axis", -1))
    sm = c.g.op("Softmax", op.input("Logits"), axis=axis)
    c.emit("Identity", [sm], [op.output("Softmax")])
    logp = c.g.op("Log", sm)
    if op.attr("soft_label", False):
        loss = c.g.op("Neg", c.g.op("ReduceSum", c.g.op("Mul", logp, op.input("Label")), axes=[axis], keepdims=1))
    else:
        loss = c.g.op("Neg", c.g.op("GatherElements", logp, c.g.op("Cast", op.input("Label"), to=7), axis=axis))
    c.emit("Identity", [loss], [op.output("Loss")])


# ------------------------------------------------------------------------- pooling in 3-D
@mapper("pool3d", "max_pool3d_with_index")
def _pool3d(c, op):
    """paddle2onnx/mapper/nn/pool3d.cc: explicit symmetric padding, global and adaptive forms."""
    ptype = "max" if op.type == "max_pool3d_with_index" else op.attr("pooling_type", "max")
    x, out = op.input("X"), op.output("Out")
    if op.attr("global_pooling", False) or (op.attr("adaptive", False) and list(op.attr("ksize")) == [1, 1, 1]):
        c.emit("GlobalMaxPool" if ptype == "max" else "GlobalAveragePool", [x], [out])
        return
    if op.attr("adaptive", False):
        raise NotImplementedError("pool3d: adaptive pooling to a size other than 1 is not supported")
    k = [int(v) for v in op.attr("ksize")]
    s = [int(v) for v in op.attr("strides", [1, 1, 1])]
    p = [int(v) for v in op.attr("paddings", [0, 0, 0])]
    pads = p + p if len(p) == 3 else [p[0], p[2], p[4], p[1], p[3], p[5]]
    attrs = dict(kernel_shape=k, strides=s, pads=pads, ceil_mode=int(op.attr("ceil_mode", False)))
    if ptype == "max":
        outs = [out] + ([op.output("Mask")] if op.type == "max_pool3d_with_index" and op.output("Mask") else [])
        c.emit("MaxPool", [x], outs, **attrs)
    else:
        c.emit("AveragePool", [x], [out], count_include_pad=int(not op.attr("exclusive", True)), **attrs)


# ------------------------------------------------------------------------- sampling / detection heads
@mapper("grid_sampler")
def _grid_sampler(c, op):
    c.emit("GridSample", [op.input("X"), op.input("Grid")], [op.output("Output")], mode=op.attr("mode", "bilinear"),
           padding_mode=op.attr("padding_mode", "zeros"), align_corners=int(op.attr("align_corners", True)))


@mapper("set_value")
def _set_value(c, op):
    """Slice assignment with constant bounds (paddle2onnx/mapper/tensor/set_value.h); tensor-valued bounds are rejected."""
    if op.input("StartsTensorList") or op.input("EndsTensorList") or op.input("StepsTensorList"):
        raise NotImplementedError("set_value: tensor-valued slice bounds are not supported")
    attrs = dict(axes=[int(a) for a in op.attr("axes", [])], starts=[int(a) for a in op.attr("starts", [])],
                 ends=[int(a) for a in op.attr("ends", [])], steps=[int(a) for a in op.attr("steps", [])],
                 decrease_axes=[int(a) for a in op.attr("decrease_axes", []) or []],
                 none_axes=[int(a) for a in op.attr("none_axes", []) or []])
    ins = [op.input("Input")]
    if op.input("ValueTensor"):
        ins.append(op.input("ValueTensor"))
    else:
        for key in ("fp32_values", "int32_values", "int64_values", "bool_values", "fp64_values", "values"):
            v = op.attr(key, None)
            if v is not None and len(v):
                attrs["values"] = [float(t) for t in v]
                break
        attrs["shape"] = [int(d) for d in op.attr("shape", []) or []]
    c.emit("SetValue", ins, [op.output("Out")], domain="fdb", **attrs)


@mapper("yolo_box")
def _yolo_box(c, op):
    """paddle2onnx/mapper/detection/yolo_box.cc: kept as one operator whose semantics are the Paddle kernel's."""
    c.emit("YoloBox", [op.input("X"), op.input("ImgSize")], [op.output("Boxes"), op.output("Scores")], domain="fdb",
           anchors=[int(a) for a in op.attr("anchors")], class_num=int(op.attr("class_num")),
           conf_thresh=float(op.attr("conf_thresh", 0.01)), downsample_ratio=int(op.attr("downsample_ratio", 32)),
           clip_bbox=int(op.attr("clip_bbox", True)), scale_x_y=float(op.attr("scale_x_y", 1.0)),
           iou_aware=int(op.attr("iou_aware", False)), iou_aware_factor=float(op.attr("iou_aware_factor", 0.5)))


@mapper("roi_align")
def _roi_align(c, op):
    """paddle2onnx/mapper/detection/roi_align.cc: ``RoisNum`` (boxes per image) becomes the per-box image index."""
    rois_num = op.input("RoisNum")
    if rois_num:
        n = c.g.op("Cast", rois_num, to=7)
        ends = c.g.op("CumSum", n, c.i64(0))
        total = c.g.op("Slice", c.g.op("Shape", op.input("ROIs")), c.i64([0]), c.i64([1]), c.i64([0]))
        pos = c.g.op("Range", c.i64(0), c.g.op("Reshape", total, c.i64([])), c.i64(1))
        # image index of box r = number of images whose boxes end at or before r
        ge = c.g.op("GreaterOrEqual", c.g.op("Unsqueeze", pos, axes=[1]), c.g.op("Unsqueeze", ends, axes=[0]))
        batch = c.g.op("ReduceSum", c.g.op("Cast", ge, to=7), axes=[1], keepdims=0)
    else:
        total = c.g.op("Slice", c.g.op("Shape", op.input("ROIs")), c.i64([0]), c.i64([1]), c.i64([0]))
        batch = c.g.op("ConstantOfShape", total, value=np.asarray([0], np.int64))
    c.emit("RoiAlign", [op.input("X"), op.input("ROIs"), batch], [op.output("Out")],
           output_height=int(op.attr("pooled_height", 1)), output_width=int(op.attr("pooled_width", 1)),
           sampling_ratio=max(int(op.attr("sampling_ratio", -1)), 0), spatial_scale=float(op.attr("spatial_scale", 1.0)),
           coordinate_transformation_mode="half_pixel" if op.attr("aligned", False) else "output_half_pixel", mode="avg")


# ------------------------------------------------------------------------- recurrent layers
@mapper("rnn")
def _rnn(c, op):
    """Multi-layer, optionally bidirectional LSTM (paddle2onnx/mapper/nn/rnn.cc): ``WeightList`` holds, for every layer
    and direction, W_ih and W_hh (all of them first) and then b_ih and b_hh; Paddle's gate order i, f, c, o is
    re-ordered to ONNX's i, o, f, c; the initial states ``[layers * directions, batch, hidden]`` are split per layer."""
    mode = op.attr("mode", "LSTM")
    if mode != "LSTM":
        raise NotImplementedError(f"rnn: mode {mode} is not supported (LSTM is)")
    layers, hidden = int(op.attr("num_layers", 1)), int(op.attr("hidden_size"))
    ndir = 2 if op.attr("is_bidirec", False) else 1
    wl = op.inputs["WeightList"]
    nw = layers * ndir * 2

    def reorder(a: np.ndarray) -> np.ndarray:
        i, f, g, o = np.split(a, 4, axis=0)
        return np.concatenate([i, o, f, g], axis=0)

    def weight(name):
        if name not in c.g.initializers:
            raise NotImplementedError("rnn: weights must be constants")
        return np.asarray(c.g.initializers[name], np.float32)
    x = op.input("Input")
    pre = op.inputs.get("PreState", [])
    h_all, c_all = (pre[0], pre[1]) if len(pre) >= 2 else (None, None)
    hs, cs = [], []
    for layer in range(layers):
        w_ih, w_hh, bias = [], [], []
        for d in range(ndir):
            k = (layer * ndir + d) * 2
            w_ih.append(reorder(weight(wl[k])))
            w_hh.append(reorder(weight(wl[k + 1])))
            b = np.concatenate([reorder(weight(wl[nw + k])), reorder(weight(wl[nw + k + 1]))]) if len(wl) >= 2 * nw \
                else np.zeros(8 * hidden, np.float32)
            bias.append(b)
        ins = [x, c.g.const(np.stack(w_ih), prefix="lstm_w"), c.g.const(np.stack(w_hh), prefix="lstm_r"),
               c.g.const(np.stack(bias), prefix="lstm_b"), ""]
        if h_all is not None:
            lo, hi = layer * ndir, (layer + 1) * ndir
            ins += [c.g.op("Slice", h_all, c.i64([lo]), c.i64([hi]), c.i64([0])),
                    c.g.op("Slice", c_all, c.i64([lo]), c.i64([hi]), c.i64([0]))]
        y, h, cc = c.g.add_node("LSTM", ins, n_out=3, hidden_size=hidden,
                                direction="bidirectional" if ndir == 2 else "forward")
        # [seq, directions, batch, hidden] -> [seq, batch, directions * hidden]
        x = c.g.op("Reshape", c.g.op("Transpose", y, perm=[0, 2, 1, 3]), c.i64([0, 0, -1]))
        hs.append(h)
        cs.append(cc)
    c.emit("Identity", [x], [op.output("Out")])
    states = op.outputs.get("State", [])
    if len(states) >= 2:
        c.emit("Concat" if len(hs) > 1 else "Identity", hs, [states[0]], **({"axis": 0} if len(hs) > 1 else {}))
        c.emit("Concat" if len(cs) > 1 else "Identity", cs, [states[1]], **({"axis": 0} if len(cs) > 1 else {}))
