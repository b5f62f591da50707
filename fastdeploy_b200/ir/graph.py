"""Graph IR of the native backend.

The IR uses ONNX operator semantics (opset 11-17 subset) plus a handful of fused or
custom operators (domain ``fdb``): both importers - ONNX ``ModelProto`` and Paddle
``ProgramDesc`` - produce this IR, the CPU interpreter executes it in fp32 and the
sm_100a executor lowers it to kernel launches. It plays the role that the ONNX graph
plays inside the reference, where every Paddle model is first converted by
paddle2onnx (fastdeploy/runtime/backends/ort/ort_backend.cc:194-218).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, Iterable, List, Optional, Sequence

import numpy as np


@dataclass
class ValueInfo:
    name: str
    dtype: str = "float32"            # numpy dtype name
    shape: Optional[List[Any]] = None  # ints, or str / -1 for dynamic dims

    def static_shape(self) -> Optional[List[int]]:
        if self.shape is None:
            return None
        if all(isinstance(d, (int, np.integer)) and d >= 0 for d in self.shape):
            return [int(d) for d in self.shape]
        return None


@dataclass
class Node:
    op: str
    inputs: List[str]
    outputs: List[str]
    attrs: Dict[str, Any] = field(default_factory=dict)
    name: str = ""
    domain: str = ""

    def attr(self, key: str, default: Any = None) -> Any:
        return self.attrs.get(key, default)


def body_outer_refs(body: "Graph") -> List[str]:
    """Names that a Loop / If body graph reads from the enclosing scope: what it neither defines nor takes as an
    input (bodies nested inside it included)."""
    defined = set(body.initializers) | {v.name for v in body.inputs} | {""}
    refs: List[str] = []
    for n in body.nodes:
        nested = [r for a in n.attrs.values() if isinstance(a, Graph) for r in body_outer_refs(a)]
        for i in list(n.inputs) + list(n.attrs.get("outer_refs", [])) + nested:
            if i not in defined and i not in refs:
                refs.append(i)
        defined.update(n.outputs)
    for v in body.outputs:
        if v.name not in defined and v.name not in refs:
            refs.append(v.name)
    return refs


class Graph:
    def __init__(self, name: str = "graph", opset: int = 11):
        self.name = name
        self.opset = opset
        self.nodes: List[Node] = []
        self.inputs: List[ValueInfo] = []
        self.outputs: List[ValueInfo] = []
        self.initializers: Dict[str, np.ndarray] = {}
        self.value_info: Dict[str, ValueInfo] = {}
        self.metadata: Dict[str, Any] = {}
        self._uid = 0

    # ------------------------------------------------------------------ building
    def unique(self, prefix: str) -> str:
        self._uid += 1
        return f"{prefix}_{self._uid}"

    def add_input(self, name: str, dtype: str, shape: Sequence[Any]) -> str:
        self.inputs.append(ValueInfo(name, dtype, list(shape)))
        return name

    def add_output(self, name: str, dtype: str = "float32", shape: Optional[Sequence[Any]] = None) -> str:
        self.outputs.append(ValueInfo(name, dtype, list(shape) if shape is not None else None))
        return name

    def add_initializer(self, name: str, value: np.ndarray) -> str:
        self.initializers[name] = np.ascontiguousarray(value)
        return name

    def const(self, value, dtype=None, prefix: str = "const") -> str:
        arr = np.asarray(value, dtype=dtype)
        return self.add_initializer(self.unique(prefix), arr)

    def add_node(self, op: str, inputs: Sequence[str], outputs: Optional[Sequence[str]] = None, n_out: int = 1,
                 name: str = "", domain: str = "", **attrs) -> List[str]:
        if outputs is None:
            outputs = [self.unique(op.lower())] if n_out == 1 else [self.unique(op.lower()) for _ in range(n_out)]
        node = Node(op, list(inputs), list(outputs), dict(attrs), name or self.unique("n_" + op), domain)
        self.nodes.append(node)
        return list(outputs)

    def op(self, op: str, *inputs: str, **attrs) -> str:
        """Adds a single-output node and returns the output name."""
        return self.add_node(op, inputs, **attrs)[0]

    # ------------------------------------------------------------------ queries
    def producers(self) -> Dict[str, Node]:
        prod = {}
        for n in self.nodes:
            for o in n.outputs:
                if o:
                    prod[o] = n
        return prod

    def consumers(self) -> Dict[str, List[Node]]:
        cons: Dict[str, List[Node]] = {}
        for n in self.nodes:
            for i in n.inputs:
                if i:
                    cons.setdefault(i, []).append(n)
        return cons

    def input_names(self) -> List[str]:
        return [v.name for v in self.inputs]

    def output_names(self) -> List[str]:
        return [v.name for v in self.outputs]

    def toposort(self) -> None:
        """Stable topological sort of ``self.nodes``."""
        known = set(self.initializers) | {v.name for v in self.inputs} | {""}
        pending = list(self.nodes)
        ordered: List[Node] = []
        while pending:
            rest = []
            progressed = False
            for n in pending:
                if all(i in known for i in list(n.inputs) + list(n.attrs.get("outer_refs", []))):
                    ordered.append(n)
                    known.update(n.outputs)
                    progressed = True
                else:
                    rest.append(n)
            if not progressed:
                missing = {i for n in rest for i in list(n.inputs) + list(n.attrs.get("outer_refs", [])) if i not in known}
                raise ValueError(f"graph has a cycle or undefined values: {sorted(missing)[:5]}")
            pending = rest
        self.nodes = ordered

    def prune(self) -> None:
        """Drops nodes and initializers that do not reach a graph output."""
        needed = set(self.output_names())
        keep: List[Node] = []
        for n in reversed(self.nodes):
            if any(o in needed for o in n.outputs):
                keep.append(n)
                needed.update(i for i in n.inputs if i)
                needed.update(n.attrs.get("outer_refs", []))      # what the bodies of Loop / If read from this scope
        keep.reverse()
        self.nodes = keep
        self.initializers = {k: v for k, v in self.initializers.items() if k in needed}

    def clone(self) -> "Graph":
        g = Graph(self.name, self.opset)
        g.nodes = [Node(n.op, list(n.inputs), list(n.outputs), copy.deepcopy(n.attrs), n.name, n.domain) for n in self.nodes]
        g.inputs = [ValueInfo(v.name, v.dtype, list(v.shape) if v.shape is not None else None) for v in self.inputs]
        g.outputs = [ValueInfo(v.name, v.dtype, list(v.shape) if v.shape is not None else None) for v in self.outputs]
        g.initializers = dict(self.initializers)
        g.value_info = dict(self.value_info)
        g.metadata = copy.deepcopy(self.metadata)
        g._uid = self._uid
        return g

    def num_params(self) -> int:
        return int(sum(v.size for v in self.initializers.values()))

    def op_histogram(self) -> Dict[str, int]:
        h: Dict[str, int] = {}
        for n in self.nodes:
            h[n.op] = h.get(n.op, 0) + 1
        return dict(sorted(h.items()))

    def __repr__(self) -> str:
        return (f"Graph({self.name!r}, nodes={len(self.nodes)}, params={self.num_params()}, "
                f"inputs={[v.name for v in self.inputs]}, outputs={[v.name for v in self.outputs]})")
