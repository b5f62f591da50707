"""Model readers, writers and the converter entry points (paddle2onnx/converter.h:36-130):

``export`` (Paddle inference model -> ONNX bytes, optionally optimised / converted to fp16), ``is_exportable``,
``remove_multiclass_nms`` (cut the NMS tail off a detector so that a caller can run its own),
``convert_fp32_to_fp16``, and the two readers that list a model's inputs and outputs without building a runtime.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from ..ir.graph import Graph, ValueInfo
from .onnx_format import load_onnx, save_onnx
from .paddle_format import parse_program
from .paddle_import import _MAPPERS, load_paddle


@dataclass
class ModelTensorInfo:
    name: str
    shape: List[int]            # -1 for a dynamic dimension
    dtype: str                  # numpy dtype name


@dataclass
class NMSParameters:
    """Attributes of the ``MultiClassNMS`` node that ``remove_multiclass_nms`` took out (paddle2onnx/converter.h:87-95)."""
    background_label: int = -1
    keep_top_k: int = 300
    nms_eta: float = 1.0
    nms_threshold: float = 0.7
    score_threshold: float = 0.01
    nms_top_k: int = 10000
    normalized: bool = True


def _infos(values: Sequence[ValueInfo]) -> List[ModelTensorInfo]:
    return [ModelTensorInfo(v.name, [d if isinstance(d, (int, np.integer)) and d >= 0 else -1 for d in (v.shape or [])],
                            v.dtype) for v in values]


class OnnxReader:
    """Inputs and outputs of an ONNX model given as bytes."""

    def __init__(self, model: bytes):
        g = load_onnx(model)
        self.inputs, self.outputs = _infos(g.inputs), _infos(g.outputs)
        self.num_inputs, self.num_outputs = len(self.inputs), len(self.outputs)


class PaddleReader:
    """Inputs and outputs of a Paddle ``.pdmodel`` given as bytes, plus whether it carries quantisation ops."""

    def __init__(self, model: bytes):
        prog = parse_program(model)
        def info(name):
            v = prog.vars.get(name)
            return ModelTensorInfo(name, list(v.shape) if v else [], v.dtype if v else "float32")
        self.inputs = [info(n) for n in prog.feed_names()]
        self.outputs = [info(n) for n in prog.fetch_names()]
        self.num_inputs, self.num_outputs = len(self.inputs), len(self.outputs)
        all_ops = list(prog.ops) + [op for _, ops in prog.sub_blocks for op in ops]
        self.has_nms = any(op.type in ("multiclass_nms3", "multiclass_nms2", "multiclass_nms", "matrix_nms") for op in all_ops)
        self.is_quantize_model = any(op.type.startswith(("quantize_linear", "dequantize_linear", "fake_quantize",
                                                         "fake_channel_wise", "fake_dequantize")) for op in all_ops)


def unsupported_ops(model: bytes) -> List[str]:
    """Operator types of the program (sub-blocks included) that the importer has no mapper for."""
    from .paddle_control_flow import CONTROL_MAPPERS
    prog = parse_program(model)
    all_ops = list(prog.ops) + [op for _, ops in prog.sub_blocks for op in ops]
    return sorted({op.type for op in all_ops if op.type not in _MAPPERS and op.type not in CONTROL_MAPPERS})


def is_exportable(model: bytes, params: Optional[bytes] = None) -> bool:
    try:
        return not unsupported_ops(model)
    except Exception:
        return False


def export(model: bytes, params: Optional[bytes], enable_optimize: bool = True, export_fp16_model: bool = False,
           input_shapes: Optional[Dict[str, Sequence[int]]] = None, keep_io_types: bool = True,
           custom_ops: Optional[Dict[str, str]] = None) -> bytes:
    """Paddle inference model -> ONNX model bytes. ``enable_optimize`` runs the numerically safe graph rewrites
    (constant, batch-norm and bias folding); ``export_fp16_model`` stores weights and computes in half precision with
    casts around the operators that need fp32; ``custom_ops`` passes the named Paddle operators through as custom
    nodes (the graph is then written as imported: the rewrites evaluate nodes, and a custom node has no evaluator)."""
    g = load_paddle(model, params, custom_ops=custom_ops)
    if enable_optimize and not custom_ops:
        from ..ir.passes import optimize
        g = optimize(g, dict(input_shapes) if input_shapes else None, level=1)
    if export_fp16_model:
        from ..ir.convert_fp16 import convert_fp32_to_fp16
        g = convert_fp32_to_fp16(g, keep_io_types=keep_io_types)
    return save_onnx(g)


def convert_fp32_to_fp16(onnx_model: bytes, keep_io_types: bool = True) -> bytes:
    from ..ir.convert_fp16 import convert_fp32_to_fp16 as conv
    return save_onnx(conv(load_onnx(onnx_model), keep_io_types=keep_io_types))


def remove_multiclass_nms(onnx_model: bytes) -> Tuple[bytes, Optional[NMSParameters]]:
    """Cuts the (single) ``MultiClassNMS`` node out of a detector: the graph's outputs become the node's box and
    score inputs, and the node's attributes are returned so that the caller can apply NMS itself
    (paddle2onnx/converter.h:112-114, used by the TensorRT back end of the reference). A model without the node
    comes back unchanged with ``None``."""
    g = load_onnx(onnx_model)
    nms = [n for n in g.nodes if n.op == "MultiClassNMS"]
    if len(nms) != 1:
        return onnx_model, None
    node = nms[0]
    p = NMSParameters(int(node.attr("background_label", -1)), int(node.attr("keep_top_k", 300)),
                      float(node.attr("nms_eta", 1.0)), float(node.attr("nms_threshold", 0.7)),
                      float(node.attr("score_threshold", 0.01)), int(node.attr("nms_top_k", 10000)),
                      bool(node.attr("normalized", True)))
    info = g.value_info
    g.outputs = []
    for name in node.inputs[:2]:
        vi = info.get(name)
        g.outputs.append(ValueInfo(name, vi.dtype if vi else "float32", list(vi.shape) if vi and vi.shape else None))
    g.nodes.remove(node)
    g.prune()
    g.toposort()
    return save_onnx(g), p
