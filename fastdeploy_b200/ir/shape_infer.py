"""Shape propagation for concrete input shapes.

Activations run as ``meta`` tensors (no storage, no math) through the interpreter's own
operator implementations, while small integer "shape tensors" (outputs of Shape, Slice
of a shape, Concat of dims ...) stay real so that Reshape / Resize / Expand targets are
known. The result is the static shape and dtype of every value plus the concrete
contents of every shape tensor - the information the reference obtains from TensorRT's
shape profile collection (fastdeploy/runtime/backends/tensorrt/trt_backend.cc:442-504).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import interp
from .graph import Graph

# argument positions whose VALUES (not just shapes) an operator reads
VALUE_ARGS = {
    "Reshape": (1,), "Slice": (1, 2, 3, 4), "Expand": (1,), "Tile": (1,), "Resize": (1, 2, 3), "Upsample": (1,),
    "Pad": (1, 2), "ConstantOfShape": (0,), "Range": (0, 1, 2), "TopK": (1,), "Split": (1,), "Squeeze": (1,),
    "Unsqueeze": (1,), "CumSum": (1,), "Clip": (1, 2), "OneHot": (1,), "ReduceSum": (1,), "ReduceMean": (1,),
    "ReduceMax": (1,), "ReduceMin": (1,),
}


def _meta(shape, dtype=torch.float32):
    return torch.empty([int(d) for d in shape], dtype=dtype, device="meta")


# output shapes of operators whose reference implementation loops over values and cannot run on meta tensors
SHAPE_RULES = {
    "RoiAlign": lambda node, x, rois, idx: _meta([rois.shape[0], x.shape[1], node.attr("output_height", 1),
                                                  node.attr("output_width", 1)], x.dtype),
    "YoloBox": lambda node, x, img: (
        _meta([x.shape[0], (len(node.attr("anchors")) // 2) * x.shape[2] * x.shape[3], 4], x.dtype),
        _meta([x.shape[0], (len(node.attr("anchors")) // 2) * x.shape[2] * x.shape[3], node.attr("class_num")], x.dtype)),
    "SetValue": lambda node, x, *v: _meta(x.shape, x.dtype),
    "TemporalShift": lambda node, x: _meta(x.shape, x.dtype),
    "PackedAttention": lambda node, q, *rest: _meta(q.shape, q.dtype),
}
# a real tensor larger than this is treated as data, not as a shape tensor
MAX_REAL_ELEMS = 4096

_TORCH2NP = {v: k for k, v in interp.NP2TORCH.items()}


class ShapeInfo:
    def __init__(self):
        self.shapes: Dict[str, List[int]] = {}
        self.dtypes: Dict[str, str] = {}
        self.values: Dict[str, np.ndarray] = {}   # known contents (shape tensors and small constants)

    def shape(self, name: str) -> List[int]:
        return self.shapes[name]


def _to_meta(t: torch.Tensor) -> torch.Tensor:
    return t if t.device.type == "meta" else torch.empty_like(t, device="meta")


def infer_shapes(graph: Graph, input_shapes: Dict[str, Sequence[int]],
                 input_values: Optional[Dict[str, np.ndarray]] = None) -> ShapeInfo:
    """Runs the graph on meta tensors. ``input_values`` may pin small inputs (e.g. scale factors)."""
    env: Dict[str, Optional[torch.Tensor]] = {"": None}
    for k, v in graph.initializers.items():
        t = torch.from_numpy(np.ascontiguousarray(v))
        if t.dtype in (torch.float16, torch.float64):
            t = t.float()
        if t.numel() > MAX_REAL_ELEMS:
            t = _to_meta(t)
        env[k] = t
    for vi in graph.inputs:
        if input_values and vi.name in input_values:
            env[vi.name] = torch.from_numpy(np.ascontiguousarray(input_values[vi.name]))
            continue
        if vi.name not in input_shapes:
            raise KeyError(f"shape of input {vi.name!r} not given")
        dt = interp.NP2TORCH[vi.dtype]
        if dt in (torch.float16, torch.bfloat16, torch.float64):
            dt = torch.float32
        env[vi.name] = torch.empty(list(input_shapes[vi.name]), dtype=dt, device="meta")
    with torch.no_grad():
        for node in graph.nodes:
            fn = interp._OPS.get(node.op)
            if fn is None:
                raise NotImplementedError(f"shape inference: unsupported op {node.op}")
            args = [env[i] for i in node.inputs]
            while args and args[-1] is None:
                args.pop()
            value_pos = VALUE_ARGS.get(node.op, ())
            data_args = [a for k, a in enumerate(args) if a is not None and k not in value_pos]
            any_meta = any(a.device.type == "meta" for a in data_args)
            if node.op == "Shape":
                res = torch.tensor(list(args[0].shape), dtype=torch.int64)
            elif node.op == "Size":
                res = torch.tensor(args[0].numel(), dtype=torch.int64)
            elif node.op in ("MultiClassNMS", "PPYOLOEPost"):
                n = args[0].shape[0]
                k = node.attr("keep_top_k", 100)
                if node.op == "PPYOLOEPost":
                    m = sum(h * w for h, w in zip(node.attr("grid_h"), node.attr("grid_w")))
                else:
                    m = args[0].shape[1]
                k = k if k > 0 else m
                res = (torch.empty(n * k, 6, device="meta"), torch.empty(n * k, 1, dtype=torch.int64, device="meta"),
                       torch.empty(n, dtype=torch.int32, device="meta"))
            elif any_meta and node.op in SHAPE_RULES:
                res = SHAPE_RULES[node.op](node, *args)
            else:
                if any_meta:
                    args = [(_to_meta(a) if (a is not None and k not in value_pos) else a) for k, a in enumerate(args)]
                for k in value_pos:
                    if k < len(args) and args[k] is not None and args[k].device.type == "meta":
                        raise ValueError(f"{node.op} {node.name!r}: argument {k} must have a known value "
                                         f"for static shape inference")
                node.attrs.setdefault("_opset", graph.opset)
                res = fn(node, *args)
            if not isinstance(res, tuple):
                res = (res,)
            for name, val in zip(node.outputs, res):
                if name:
                    env[name] = val
    info = ShapeInfo()
    for name, t in env.items():
        if t is None or not name:
            continue
        info.shapes[name] = [int(d) for d in t.shape]
        info.dtypes[name] = _TORCH2NP.get(t.dtype, "float32")
        if t.device.type != "meta" and t.numel() <= MAX_REAL_ELEMS:
            info.values[name] = t.numpy()
    return info
