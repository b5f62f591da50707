"""Rewrites an fp32 graph to fp16 storage and arithmetic: weights become half precision, operators on a keep-fp32
list stay in single precision between inserted ``Cast`` nodes, graph inputs and outputs keep their types.

The executor does not need this pass (it chooses 16-bit kernels itself); it exists for users who export a smaller
model file or hand the graph to another runtime. Counterpart: paddle2onnx/optimizer/convert_fp32_to_fp16.cc
(keep-fp32 operator list :50-90, value clamping :300-340, boundary casts :520-700)."""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Set

import numpy as np

from .graph import Graph, Node
from .shape_infer import VALUE_ARGS

FP16_MAX = 65504.0
FP16_MIN_POSITIVE = 1e-7          # magnitudes below this are raised to it so that they do not flush to zero
# operators whose arithmetic or whose float arguments must stay fp32
DEFAULT_KEEP_FP32 = {"Resize", "Upsample", "TopK", "NonMaxSuppression", "MultiClassNMS", "PPYOLOEPost", "RoiAlign", "Range",
                     "CumSum", "Pow", "Exp", "ReduceLogSumExp", "Softmax", "LogSoftmax", "LayerNormalization",
                     "InstanceNormalization", "GroupNormalization", "YoloBox", "QuantizeLinear", "DequantizeLinear",
                     "EmbedLayerNorm", "RandomNormal"}
ONNX_FLOAT, ONNX_FLOAT16 = 1, 10


def _to_half(a: np.ndarray) -> np.ndarray:
    a = np.asarray(a, np.float32)
    tiny = (np.abs(a) < FP16_MIN_POSITIVE) & (a != 0)
    a = np.where(tiny, np.sign(a) * FP16_MIN_POSITIVE, a)
    return np.clip(a, -FP16_MAX, FP16_MAX).astype(np.float16)


def convert_fp32_to_fp16(graph: Graph, keep_io_types: bool = True, keep_fp32_ops: Optional[Iterable[str]] = None) -> Graph:
    """Returns a converted copy of ``graph``."""
    g = graph.clone()
    keep: Set[str] = set(DEFAULT_KEEP_FP32 if keep_fp32_ops is None else keep_fp32_ops)
    float_inputs = {vi.name for vi in g.inputs if vi.dtype == "float32"}
    float_outputs = {vi.name for vi in g.outputs if vi.dtype in ("float32", None)}
    # 1. which values live in fp16: everything float except what a kept operator produces or consumes as a value
    kept_nodes = [n for n in g.nodes if n.op in keep]
    kept_outputs = {o for n in kept_nodes for o in n.outputs if o}
    # initializers used by a kept node, or as a shape / scale argument of any node, stay fp32
    pinned: Set[str] = set()
    for n in g.nodes:
        for k, name in enumerate(n.inputs):
            if name in g.initializers and (n.op in keep or k in VALUE_ARGS.get(n.op, ())):
                pinned.add(name)
    for name, arr in list(g.initializers.items()):
        if arr.dtype == np.float32 and name not in pinned:
            g.initializers[name] = _to_half(arr)
    # 2. casts around the kept operators
    new_nodes: List[Node] = []
    cast_cache: Dict[str, str] = {}

    def cast(name: str, to: int) -> str:
        key = f"{name}->{to}"
        if key not in cast_cache:
            out = g.unique(name + ("_fp32" if to == ONNX_FLOAT else "_fp16"))
            new_nodes.append(Node("Cast", [name], [out], {"to": to}, g.unique("n_Cast"), ""))
            cast_cache[key] = out
        return cast_cache[key]

    def is_float_value(name: str) -> bool:
        if name in g.initializers:
            return g.initializers[name].dtype in (np.float32, np.float16)
        return True          # activations of unknown type are treated as float; integer tensors never reach a Cast below

    int_values = _integer_values(g)
    for vi in g.inputs:
        if keep_io_types and vi.name in float_inputs:
            # the graph keeps its fp32 input; consumers in the fp16 region read a cast
            pass
    rename_in: Dict[str, str] = {}
    if keep_io_types:
        for name in float_inputs:
            rename_in[name] = cast(name, ONNX_FLOAT16)
    for n in g.nodes:
        if n.op in keep:
            ins = []
            for k, name in enumerate(n.inputs):
                if not name or name in int_values or name in pinned or name in kept_outputs or \
                        (keep_io_types and name in float_inputs):
                    ins.append(name)
                elif name in g.initializers and g.initializers[name].dtype != np.float16:
                    ins.append(name)
                else:
                    ins.append(cast(name, ONNX_FLOAT))
            n.inputs = ins
        else:
            ins = []
            for k, name in enumerate(n.inputs):
                if name in rename_in:
                    ins.append(rename_in[name])
                elif name in kept_outputs and name not in int_values and k not in VALUE_ARGS.get(n.op, ()):
                    ins.append(cast(name, ONNX_FLOAT16))
                else:
                    ins.append(name)
            n.inputs = ins
            if n.op == "Cast" and n.attr("to") == ONNX_FLOAT:
                n.attrs["to"] = ONNX_FLOAT16
            if n.op == "ConstantOfShape" and isinstance(n.attr("value", None), np.ndarray) and n.attr("value").dtype == np.float32:
                n.attrs["value"] = n.attr("value").astype(np.float16)
        new_nodes.append(n)
    # 3. fp32 graph outputs
    if keep_io_types:
        for vi in g.outputs:
            if vi.name in float_outputs and vi.name not in kept_outputs and vi.name not in int_values:
                inner = g.unique(vi.name + "_fp16")
                for n in new_nodes:
                    n.outputs = [inner if o == vi.name else o for o in n.outputs]
                    n.inputs = [inner if i == vi.name else i for i in n.inputs]
                new_nodes.append(Node("Cast", [inner], [vi.name], {"to": ONNX_FLOAT}, g.unique("n_Cast"), ""))
    else:
        for vi in list(g.inputs) + list(g.outputs):
            if vi.dtype == "float32":
                vi.dtype = "float16"
    g.nodes = new_nodes
    g.toposort()
    g.metadata["converted_fp16"] = "1"
    return g


def _integer_values(g: Graph) -> Set[str]:
    """Names of values that are certainly not floating point (shape arithmetic, indices, masks)."""
    out: Set[str] = {name for name, a in g.initializers.items() if a.dtype.kind in "iub"}
    out |= {vi.name for vi in g.inputs if vi.dtype not in ("float32", "float16", "float64", None)}
    int_ops = {"Shape", "Size", "ArgMax", "ArgMin", "NonZero", "Equal", "Less", "Greater", "LessOrEqual", "GreaterOrEqual",
               "Not", "And", "Or", "Xor"}
    passthrough = {"Reshape", "Squeeze", "Unsqueeze", "Slice", "Gather", "Concat", "Identity", "Transpose", "Expand",
                   "Tile", "Flatten", "Split", "Add", "Sub", "Mul", "Div", "Max", "Min", "Neg", "Abs", "Mod", "Where"}
    changed = True
    while changed:
        changed = False
        for n in g.nodes:
            outs = [o for o in n.outputs if o and o not in out]
            if not outs:
                continue
            if n.op in int_ops or (n.op == "Cast" and n.attr("to") not in (1, 10, 11, 16)) or \
                    (n.op == "TopK" and False):
                out.update(outs)
                changed = True
            elif n.op in passthrough:
                data = [i for k, i in enumerate(n.inputs) if i and not (n.op in VALUE_ARGS and k in VALUE_ARGS[n.op])]
                if n.op == "Where":
                    data = data[1:]
                if n.op == "Gather":
                    data = data[:1]
                if data and all(i in out for i in data):
                    out.update(outs)
                    changed = True
    # second outputs that are indices
    for n in g.nodes:
        if n.op == "TopK" and len(n.outputs) > 1 and n.outputs[1]:
            out.add(n.outputs[1])
        if n.op in ("MultiClassNMS", "PPYOLOEPost") and len(n.outputs) > 1:
            out.update(o for o in n.outputs[1:] if o)
    return out
