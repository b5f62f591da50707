"""ONNX ``ModelProto`` reader and writer on top of the wire codec (no ``onnx`` package).

Covers what the reference reads through ONNX Runtime / nvonnxparser / its own
``OnnxReader`` (paddle2onnx/onnx_reader.cc): graph nodes with all attribute kinds,
initializers in raw or typed storage, value infos with symbolic dims, opset imports.
"""
from __future__ import annotations

from typing import Any, Dict, List

import numpy as np

from ..ir.graph import Graph, Node, ValueInfo, body_outer_refs
from . import protowire as pw

# ---- TensorProto.DataType <-> numpy
ONNX_DTYPES = {1: "float32", 2: "uint8", 3: "int8", 4: "uint16", 5: "int16", 6: "int32", 7: "int64", 9: "bool",
               10: "float16", 11: "float64", 12: "uint32", 13: "uint64", 16: "bfloat16"}
NP_TO_ONNX = {v: k for k, v in ONNX_DTYPES.items()}

DIM = {1: ("dim_value", "int", False), 2: ("dim_param", "str", False)}
SHAPE = {1: ("dim", DIM, True)}
TENSOR_TYPE = {1: ("elem_type", "int", False), 2: ("shape", SHAPE, False)}
TYPE = {1: ("tensor_type", TENSOR_TYPE, False)}
VALUE_INFO = {1: ("name", "str", False), 2: ("type", TYPE, False), 3: ("doc_string", "str", False)}
TENSOR = {1: ("dims", "int", True), 2: ("data_type", "int", False), 4: ("float_data", "float", True),
          5: ("int32_data", "int", True), 6: ("string_data", "bytes", True), 7: ("int64_data", "int", True),
          8: ("name", "str", False), 9: ("raw_data", "bytes", False), 10: ("double_data", "double", True),
          11: ("uint64_data", "uint", True), 12: ("doc_string", "str", False)}
ATTRIBUTE: Dict[int, Any] = {1: ("name", "str", False), 20: ("type", "int", False), 2: ("f", "float", False),
                             3: ("i", "int", False), 4: ("s", "bytes", False), 5: ("t", TENSOR, False),
                             7: ("floats", "float", True), 8: ("ints", "int", True), 9: ("strings", "bytes", True),
                             10: ("tensors", TENSOR, True), 13: ("doc_string", "str", False)}
NODE = {1: ("input", "str", True), 2: ("output", "str", True), 3: ("name", "str", False), 4: ("op_type", "str", False),
        5: ("attribute", ATTRIBUTE, True), 6: ("doc_string", "str", False), 7: ("domain", "str", False)}
GRAPH: Dict[int, Any] = {1: ("node", NODE, True), 2: ("name", "str", False), 5: ("initializer", TENSOR, True),
                         10: ("doc_string", "str", False), 11: ("input", VALUE_INFO, True),
                         12: ("output", VALUE_INFO, True), 13: ("value_info", VALUE_INFO, True)}
ATTRIBUTE[6] = ("g", GRAPH, False)
ATTRIBUTE[11] = ("graphs", GRAPH, True)
OPSET = {1: ("domain", "str", False), 2: ("version", "int", False)}
STRING_ENTRY = {1: ("key", "str", False), 2: ("value", "str", False)}
MODEL = {1: ("ir_version", "int", False), 2: ("producer_name", "str", False), 3: ("producer_version", "str", False),
         4: ("domain", "str", False), 5: ("model_version", "int", False), 6: ("doc_string", "str", False),
         7: ("graph", GRAPH, False), 8: ("opset_import", OPSET, True), 14: ("metadata_props", STRING_ENTRY, True)}

A_FLOAT, A_INT, A_STRING, A_TENSOR, A_GRAPH, A_FLOATS, A_INTS, A_STRINGS, A_TENSORS = 1, 2, 3, 4, 5, 6, 7, 8, 9


def _bf16_to_f32(raw: np.ndarray) -> np.ndarray:
    return (raw.astype(np.uint32) << 16).view(np.float32)


def tensor_to_numpy(t: Dict[str, Any]) -> np.ndarray:
    dims = [int(d) for d in t.get("dims", [])]
    dt = int(t.get("data_type", 1))
    name = ONNX_DTYPES.get(dt)
    if name is None:
        raise ValueError(f"unsupported ONNX tensor data_type {dt}")
    raw = t.get("raw_data")
    if raw:
        if name == "bfloat16":
            arr = _bf16_to_f32(np.frombuffer(raw, dtype=np.uint16))
        else:
            arr = np.frombuffer(raw, dtype=np.dtype(name))
    elif name == "float32":
        arr = np.asarray(t.get("float_data", []), dtype=np.float32)
    elif name == "float64":
        arr = np.asarray(t.get("double_data", []), dtype=np.float64)
    elif name == "int64":
        arr = np.asarray(t.get("int64_data", []), dtype=np.int64)
    elif name in ("uint32", "uint64"):
        arr = np.asarray(t.get("uint64_data", []), dtype=np.dtype(name))
    elif name == "float16":
        arr = np.asarray(t.get("int32_data", []), dtype=np.uint16).view(np.float16)
    elif name == "bfloat16":
        arr = _bf16_to_f32(np.asarray(t.get("int32_data", []), dtype=np.uint16))
    else:
        arr = np.asarray(t.get("int32_data", []), dtype=np.int32).astype(np.dtype(name))
    n = int(np.prod(dims)) if dims else 1
    if arr.size != n:
        raise ValueError(f"tensor {t.get('name')!r}: {arr.size} elements for dims {dims}")
    return arr.reshape(dims).copy()


def numpy_to_tensor(name: str, arr: np.ndarray) -> Dict[str, Any]:
    arr = np.ascontiguousarray(arr)
    dt = NP_TO_ONNX.get(arr.dtype.name)
    if dt is None:
        raise ValueError(f"unsupported numpy dtype {arr.dtype}")
    return {"name": name, "dims": list(arr.shape), "data_type": dt, "raw_data": arr.tobytes()}


def _attr_value(a: Dict[str, Any]):
    t = int(a.get("type", 0))
    if t == A_FLOAT:
        return float(a.get("f", 0.0))
    if t == A_INT:
        return int(a.get("i", 0))
    if t == A_STRING:
        return a.get("s", b"").decode("utf-8", errors="replace")
    if t == A_TENSOR:
        return tensor_to_numpy(a["t"])
    if t == A_FLOATS:
        return [float(x) for x in a.get("floats", [])]
    if t == A_INTS:
        return [int(x) for x in a.get("ints", [])]
    if t == A_STRINGS:
        return [s.decode("utf-8", errors="replace") for s in a.get("strings", [])]
    if t == A_GRAPH:
        return _graph_from_msg(a["g"], 11)
    if t == A_TENSORS:
        return [tensor_to_numpy(x) for x in a.get("tensors", [])]
    # type omitted by old exporters: infer from the populated field
    for key in ("f", "i", "s", "t"):
        if key in a:
            return a[key] if key != "t" else tensor_to_numpy(a["t"])
    if a.get("ints"):
        return [int(x) for x in a["ints"]]
    if a.get("floats"):
        return [float(x) for x in a["floats"]]
    return None


def _value_info(v: Dict[str, Any]) -> ValueInfo:
    tt = v.get("type", {}).get("tensor_type", {})
    dtype = ONNX_DTYPES.get(int(tt.get("elem_type", 1)), "float32")
    shape = None
    if "shape" in tt:
        shape = []
        for d in tt["shape"].get("dim", []):
            if "dim_value" in d:
                shape.append(int(d["dim_value"]))
            else:
                shape.append(d.get("dim_param", "?") or "?")
    return ValueInfo(v.get("name", ""), dtype, shape)


def _graph_from_msg(g: Dict[str, Any], opset: int) -> Graph:
    graph = Graph(g.get("name", "graph"), opset)
    for t in g.get("initializer", []):
        graph.initializers[t.get("name", "")] = tensor_to_numpy(t)
    for v in g.get("input", []):
        vi = _value_info(v)
        if vi.name not in graph.initializers:
            graph.inputs.append(vi)
    for v in g.get("output", []):
        graph.outputs.append(_value_info(v))
    for v in g.get("value_info", []):
        vi = _value_info(v)
        graph.value_info[vi.name] = vi
    for n in g.get("node", []):
        attrs = {a["name"]: _attr_value(a) for a in n.get("attribute", [])}
        bodies = [a for a in attrs.values() if isinstance(a, Graph)]
        if bodies and "outer_refs" not in attrs:
            # Loop / If from another exporter: note what the bodies read from this scope, so that pruning and
            # sorting see those dependencies
            refs: List[str] = []
            for b in bodies:
                refs += [r for r in body_outer_refs(b) if r not in refs]
            attrs["outer_refs"] = refs
        graph.nodes.append(Node(n.get("op_type", ""), list(n.get("input", [])), list(n.get("output", [])), attrs,
                                n.get("name", ""), n.get("domain", "")))
    return graph


def load_onnx(data: bytes) -> Graph:
    model = pw.decode(data, MODEL)
    if "graph" not in model:
        raise ValueError("not an ONNX ModelProto: no graph")
    opset = 11
    for o in model.get("opset_import", []):
        if o.get("domain", "") in ("", "ai.onnx"):
            opset = int(o.get("version", 11))
    graph = _graph_from_msg(model["graph"], opset)
    graph.metadata["producer_name"] = model.get("producer_name", "")
    graph.metadata["ir_version"] = int(model.get("ir_version", 0))
    for kv in model.get("metadata_props", []):
        graph.metadata[kv.get("key", "")] = kv.get("value", "")
    # hoist Constant nodes into initializers: the rest of the stack sees one kind of constant
    kept: List[Node] = []
    for n in graph.nodes:
        if n.op == "Constant" and isinstance(n.attrs.get("value"), np.ndarray):
            graph.initializers[n.outputs[0]] = n.attrs["value"]
        else:
            kept.append(n)
    graph.nodes = kept
    return graph


def _attr_msg(name: str, v) -> Dict[str, Any]:
    if isinstance(v, bool):
        return {"name": name, "type": A_INT, "i": int(v)}
    if isinstance(v, (int, np.integer)):
        return {"name": name, "type": A_INT, "i": int(v)}
    if isinstance(v, (float, np.floating)):
        return {"name": name, "type": A_FLOAT, "f": float(v)}
    if isinstance(v, str):
        return {"name": name, "type": A_STRING, "s": v.encode("utf-8")}
    if isinstance(v, bytes):
        return {"name": name, "type": A_STRING, "s": v}
    if isinstance(v, np.ndarray):
        return {"name": name, "type": A_TENSOR, "t": numpy_to_tensor("", v)}
    if isinstance(v, Graph):
        return {"name": name, "type": A_GRAPH, "g": _graph_to_msg(v)}
    if isinstance(v, (list, tuple)):
        if len(v) and all(isinstance(x, str) for x in v):
            return {"name": name, "type": A_STRINGS, "strings": [x.encode("utf-8") for x in v]}
        if len(v) and any(isinstance(x, (float, np.floating)) for x in v):
            return {"name": name, "type": A_FLOATS, "floats": [float(x) for x in v]}
        return {"name": name, "type": A_INTS, "ints": [int(x) for x in v]}
    raise ValueError(f"cannot encode attribute {name!r} of type {type(v)}")


def _vi_msg(v: ValueInfo) -> Dict[str, Any]:
    tt: Dict[str, Any] = {"elem_type": NP_TO_ONNX.get(v.dtype, 1)}
    if v.shape is not None:
        dims = []
        for d in v.shape:
            if isinstance(d, (int, np.integer)) and d >= 0:
                dims.append({"dim_value": int(d)})
            else:
                dims.append({"dim_param": str(d) if not isinstance(d, (int, np.integer)) else "dyn"})
        tt["shape"] = {"dim": dims}
    return {"name": v.name, "type": {"tensor_type": tt}}


def _graph_to_msg(graph: Graph) -> Dict[str, Any]:
    return {
        "name": graph.name,
        "node": [{"input": n.inputs, "output": n.outputs, "name": n.name, "op_type": n.op, "domain": n.domain,
                  "attribute": [_attr_msg(k, v) for k, v in n.attrs.items() if v is not None and not k.startswith("_")]} for n in graph.nodes],
        "initializer": [numpy_to_tensor(k, v) for k, v in graph.initializers.items()],
        "input": [_vi_msg(v) for v in graph.inputs],
        "output": [_vi_msg(v) for v in graph.outputs],
        "value_info": [_vi_msg(v) for v in graph.value_info.values()],
    }


def save_onnx(graph: Graph, producer: str = "fastdeploy_b200") -> bytes:
    domains = sorted({n.domain for n in graph.nodes if n.domain})
    model = {
        "ir_version": 7, "producer_name": producer, "producer_version": "1",
        "graph": _graph_to_msg(graph),
        "opset_import": [{"domain": "", "version": graph.opset}] + [{"domain": d, "version": 1} for d in domains],
        "metadata_props": [{"key": k, "value": str(v)} for k, v in graph.metadata.items()
                           if k not in ("producer_name", "ir_version")],
    }
    return pw.encode(model, MODEL)
