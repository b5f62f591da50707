"""Paddle inference model files: ``.pdmodel`` (serialized ``ProgramDesc``) and combined
``.pdiparams``; reader, writer and a small program builder.

File layout follows what the reference's parser reads
(paddle2onnx/parser/parser.cc:60-178, paddle2onnx/proto/p2o_paddle.proto):
``.pdiparams`` is the concatenation, in sorted persistable-variable-name order, of
``u32 version | u64 lod_level | u32 version | i32 desc_size | TensorDesc | raw data``.
"""
from __future__ import annotations

import struct
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np

from . import protowire as pw

# ---- VarType.Type
VT_BOOL, VT_INT16, VT_INT32, VT_INT64, VT_FP16, VT_FP32, VT_FP64 = 0, 1, 2, 3, 4, 5, 6
VT_LOD_TENSOR, VT_FEED_MINIBATCH, VT_FETCH_LIST = 7, 9, 10
VT_UINT8, VT_INT8, VT_BF16 = 20, 21, 22
VT_SELECTED_ROWS, VT_READER, VT_RAW = 8, 15, 17

PD_DTYPES = {VT_BOOL: "bool", VT_INT16: "int16", VT_INT32: "int32", VT_INT64: "int64", VT_FP16: "float16",
             VT_FP32: "float32", VT_FP64: "float64", VT_UINT8: "uint8", VT_INT8: "int8", VT_BF16: "bfloat16"}
NP_TO_PD = {v: k for k, v in PD_DTYPES.items()}

# ---- AttrType
AT_INT, AT_FLOAT, AT_STRING, AT_INTS, AT_FLOATS, AT_STRINGS, AT_BOOLEAN, AT_BOOLEANS, AT_BLOCK, AT_LONG, AT_BLOCKS, \
    AT_LONGS, AT_FLOAT64S, AT_VAR, AT_VARS, AT_FLOAT64 = range(16)

TENSOR_DESC = {1: ("data_type", "int", False), 2: ("dims", "int", True)}
LOD_TENSOR_DESC = {1: ("tensor", TENSOR_DESC, False), 2: ("lod_level", "int", False)}
VAR_TYPE = {1: ("type", "int", False), 2: ("selected_rows", TENSOR_DESC, False), 3: ("lod_tensor", LOD_TENSOR_DESC, False),
            4: ("tensor_array", LOD_TENSOR_DESC, False)}
ATTR = {1: ("name", "str", False), 2: ("type", "int", False), 3: ("i", "int", False), 4: ("f", "float", False),
        5: ("s", "str", False), 6: ("ints", "int", True), 7: ("floats", "float", True), 8: ("strings", "str", True),
        10: ("b", "bool", False), 11: ("bools", "bool", True), 12: ("block_idx", "int", False), 13: ("l", "int", False),
        14: ("blocks_idx", "int", True), 15: ("longs", "int", True), 16: ("float64s", "double", True),
        17: ("var_name", "str", False), 18: ("vars_name", "str", True), 19: ("float64", "double", False)}
OP_VAR = {1: ("parameter", "str", False), 2: ("arguments", "str", True)}
OP_DESC = {1: ("inputs", OP_VAR, True), 2: ("outputs", OP_VAR, True), 3: ("type", "str", False), 4: ("attrs", ATTR, True),
           5: ("is_target", "bool", False)}
VAR_DESC = {1: ("name", "str", False), 2: ("type", VAR_TYPE, False), 3: ("persistable", "bool", False),
            4: ("need_check_feed", "bool", False), 5: ("is_parameter", "bool", False), 6: ("stop_gradient", "bool", False)}
BLOCK_DESC = {1: ("idx", "int", False), 2: ("parent_idx", "int", False), 3: ("vars", VAR_DESC, True),
              4: ("ops", OP_DESC, True), 5: ("forward_block_idx", "int", False)}
VERSION = {1: ("version", "int", False)}
PROGRAM_DESC = {1: ("blocks", BLOCK_DESC, True), 4: ("version", VERSION, False)}


class BlockRef(int):
    """Index of a sub-block of the program (the value of a ``sub_block`` attribute of ``while`` / ``conditional_block``)."""


class PaddleOp:
    __slots__ = ("type", "inputs", "outputs", "attrs")

    def __init__(self, type_: str, inputs: Dict[str, List[str]], outputs: Dict[str, List[str]], attrs: Dict[str, Any]):
        self.type, self.inputs, self.outputs, self.attrs = type_, inputs, outputs, attrs

    def input(self, key: str, idx: int = 0) -> Optional[str]:
        v = self.inputs.get(key, [])
        return v[idx] if len(v) > idx else None

    def output(self, key: str, idx: int = 0) -> Optional[str]:
        v = self.outputs.get(key, [])
        return v[idx] if len(v) > idx else None

    def attr(self, key: str, default=None):
        return self.attrs.get(key, default)

    def __repr__(self):
        return f"PaddleOp({self.type}, in={self.inputs}, out={self.outputs})"


class PaddleVar:
    __slots__ = ("name", "dtype", "shape", "persistable", "var_type")

    def __init__(self, name, dtype, shape, persistable, var_type=VT_LOD_TENSOR):
        self.name, self.dtype, self.shape, self.persistable, self.var_type = name, dtype, shape, persistable, var_type


class PaddleProgram:
    """In-memory ProgramDesc (block 0 only is executed; sub-blocks are kept for control flow ops)."""

    def __init__(self):
        self.vars: Dict[str, PaddleVar] = {}
        self.ops: List[PaddleOp] = []
        self.sub_blocks: List[Tuple[Dict[str, PaddleVar], List[PaddleOp]]] = []
        self.version = 0

    # ---------------------------------------------------------------- building
    def add_var(self, name: str, dtype: str = "float32", shape: Sequence[int] = (), persistable: bool = False,
                var_type: int = VT_LOD_TENSOR) -> str:
        self.vars[name] = PaddleVar(name, dtype, list(shape), persistable, var_type)
        return name

    def add_op(self, type_: str, inputs: Dict[str, Sequence[str]], outputs: Dict[str, Sequence[str]], **attrs) -> PaddleOp:
        op = PaddleOp(type_, {k: list(v) for k, v in inputs.items()}, {k: list(v) for k, v in outputs.items()}, attrs)
        self.ops.append(op)
        return op

    def feed_names(self) -> List[str]:
        feeds = [(op.attr("col", 0), op.output("Out")) for op in self.ops if op.type == "feed"]
        return [n for _, n in sorted(feeds)]

    def fetch_names(self) -> List[str]:
        fetches = [(op.attr("col", 0), op.input("X")) for op in self.ops if op.type == "fetch"]
        return [n for _, n in sorted(fetches)]

    def param_names(self) -> List[str]:
        """Sorted persistable variable names = record order of ``.pdiparams``."""
        names = []
        for v in self.vars.values():
            if v.var_type in (VT_FEED_MINIBATCH, VT_FETCH_LIST, VT_READER, VT_RAW):
                continue
            if v.var_type == VT_SELECTED_ROWS:
                raise ValueError("SELECTED_ROWS variables are not supported")
            if v.persistable:
                names.append(v.name)
        return sorted(names)


# ------------------------------------------------------------------------ decode
def _attr_value(a: Dict[str, Any]):
    t = int(a.get("type", 0))
    if t == AT_INT: return int(a.get("i", 0))
    if t == AT_FLOAT: return float(a.get("f", 0.0))
    if t == AT_STRING: return a.get("s", "")
    if t == AT_INTS: return [int(x) for x in a.get("ints", [])]
    if t == AT_FLOATS: return [float(x) for x in a.get("floats", [])]
    if t == AT_STRINGS: return list(a.get("strings", []))
    if t == AT_BOOLEAN: return bool(a.get("b", False))
    if t == AT_BOOLEANS: return [bool(x) for x in a.get("bools", [])]
    if t == AT_BLOCK: return BlockRef(a.get("block_idx", 0))
    if t == AT_LONG: return int(a.get("l", 0))
    if t == AT_BLOCKS: return [int(x) for x in a.get("blocks_idx", [])]
    if t == AT_LONGS: return [int(x) for x in a.get("longs", [])]
    if t == AT_FLOAT64S: return [float(x) for x in a.get("float64s", [])]
    if t == AT_VAR: return a.get("var_name", "")
    if t == AT_VARS: return list(a.get("vars_name", []))
    if t == AT_FLOAT64: return float(a.get("float64", 0.0))
    return None


def _decode_block(b: Dict[str, Any]):
    vars_: Dict[str, PaddleVar] = {}
    for v in b.get("vars", []):
        vt = v.get("type", {})
        kind = int(vt.get("type", VT_LOD_TENSOR))
        dtype, shape = "float32", []
        td = vt.get("lod_tensor", {}).get("tensor") or vt.get("selected_rows") or vt.get("tensor_array", {}).get("tensor")
        if td:
            dtype = PD_DTYPES.get(int(td.get("data_type", VT_FP32)), "float32")
            shape = [int(d) for d in td.get("dims", [])]
        vars_[v["name"]] = PaddleVar(v["name"], dtype, shape, bool(v.get("persistable", False)), kind)
    ops = []
    for o in b.get("ops", []):
        ins = {x["parameter"]: list(x.get("arguments", [])) for x in o.get("inputs", [])}
        outs = {x["parameter"]: list(x.get("arguments", [])) for x in o.get("outputs", [])}
        attrs = {a["name"]: _attr_value(a) for a in o.get("attrs", [])}
        ops.append(PaddleOp(o.get("type", ""), ins, outs, attrs))
    return vars_, ops


def parse_program(model_bytes: bytes) -> PaddleProgram:
    msg = pw.decode(model_bytes, PROGRAM_DESC)
    blocks = msg.get("blocks", [])
    if not blocks:
        raise ValueError("not a Paddle ProgramDesc: no blocks")
    prog = PaddleProgram()
    prog.vars, prog.ops = _decode_block(blocks[0])
    for b in blocks[1:]:
        prog.sub_blocks.append(_decode_block(b))
    prog.version = int(msg.get("version", {}).get("version", 0))
    return prog


def parse_params(prog: PaddleProgram, params_bytes: bytes) -> Dict[str, np.ndarray]:
    names = prog.param_names()
    params: Dict[str, np.ndarray] = {}
    pos, total = 0, len(params_bytes)
    buf = memoryview(params_bytes)
    while pos < total:
        idx = len(params)
        if idx >= len(names):
            raise ValueError("more parameter records than persistable variables")
        if pos + 20 > total:
            raise ValueError("truncated parameter record header")
        _ver, lod_level, _ver2, desc_size = struct.unpack_from("<IQIi", buf, pos)
        pos += 20
        if lod_level != 0:
            raise ValueError("only weights with lod_level = 0 are supported")
        td = pw.decode(bytes(buf[pos:pos + desc_size]), TENSOR_DESC)
        pos += desc_size
        dtype = PD_DTYPES.get(int(td.get("data_type", VT_FP32)))
        if dtype is None:
            raise ValueError(f"unsupported parameter dtype {td.get('data_type')}")
        dims = [int(d) for d in td.get("dims", [])]
        numel = int(np.prod(dims)) if dims else 1
        if dtype == "bfloat16":
            nbytes = numel * 2
            raw = np.frombuffer(buf[pos:pos + nbytes], dtype=np.uint16)
            arr = (raw.astype(np.uint32) << 16).view(np.float32)
        else:
            nbytes = numel * np.dtype(dtype).itemsize
            arr = np.frombuffer(buf[pos:pos + nbytes], dtype=np.dtype(dtype))
        if pos + nbytes > total:
            raise ValueError("truncated parameter data")
        pos += nbytes
        params[names[idx]] = arr.reshape(dims).copy()
    if len(params) != len(names):
        raise ValueError(f"parameter file holds {len(params)} tensors, program declares {len(names)}")
    return params


# ------------------------------------------------------------------------ encode
def _attr_msg(name: str, v) -> Dict[str, Any]:
    if isinstance(v, BlockRef):
        return {"name": name, "type": AT_BLOCK, "block_idx": int(v)}
    if isinstance(v, bool):
        return {"name": name, "type": AT_BOOLEAN, "b": v}
    if isinstance(v, (int, np.integer)):
        if -(1 << 31) <= int(v) < (1 << 31):
            return {"name": name, "type": AT_INT, "i": int(v)}
        return {"name": name, "type": AT_LONG, "l": int(v)}
    if isinstance(v, (float, np.floating)):
        return {"name": name, "type": AT_FLOAT, "f": float(v)}
    if isinstance(v, str):
        return {"name": name, "type": AT_STRING, "s": v}
    if isinstance(v, (list, tuple)):
        if len(v) and all(isinstance(x, bool) for x in v):
            return {"name": name, "type": AT_BOOLEANS, "bools": list(v)}
        if len(v) and all(isinstance(x, str) for x in v):
            return {"name": name, "type": AT_STRINGS, "strings": list(v)}
        if len(v) and any(isinstance(x, (float, np.floating)) for x in v):
            return {"name": name, "type": AT_FLOATS, "floats": [float(x) for x in v]}
        return {"name": name, "type": AT_INTS, "ints": [int(x) for x in v]}
    raise ValueError(f"cannot encode paddle attribute {name!r}: {type(v)}")


def _block_msg(idx: int, parent: int, vars_: Dict[str, "PaddleVar"], ops: List[PaddleOp]) -> Dict[str, Any]:
    vars_msg = []
    for v in vars_.values():
        vt: Dict[str, Any] = {"type": v.var_type}
        if v.var_type == VT_LOD_TENSOR:
            vt["lod_tensor"] = {"tensor": {"data_type": NP_TO_PD[v.dtype], "dims": list(v.shape)}, "lod_level": 0}
        vars_msg.append({"name": v.name, "type": vt, "persistable": v.persistable})
    ops_msg = []
    for op in ops:
        ops_msg.append({
            "type": op.type,
            "inputs": [{"parameter": k, "arguments": v} for k, v in op.inputs.items()],
            "outputs": [{"parameter": k, "arguments": v} for k, v in op.outputs.items()],
            "attrs": [_attr_msg(k, v) for k, v in op.attrs.items() if v is not None],
        })
    return {"idx": idx, "parent_idx": parent, "vars": vars_msg, "ops": ops_msg}


def serialize_program(prog: PaddleProgram) -> bytes:
    blocks = [_block_msg(0, -1, prog.vars, prog.ops)]
    for k, (vars_, ops) in enumerate(prog.sub_blocks):
        blocks.append(_block_msg(k + 1, 0, vars_, ops))
    msg = {"blocks": blocks, "version": {"version": prog.version}}
    # proto2 files written by Paddle do not pack repeated scalars
    return pw.encode(msg, PROGRAM_DESC, packed=False)


def serialize_params(prog: PaddleProgram, params: Dict[str, np.ndarray]) -> bytes:
    out = bytearray()
    for name in prog.param_names():
        arr = np.ascontiguousarray(params[name])
        desc = pw.encode({"data_type": NP_TO_PD[arr.dtype.name], "dims": list(arr.shape)}, TENSOR_DESC, packed=False)
        out += struct.pack("<IQIi", 0, 0, 0, len(desc))
        out += desc
        out += arr.tobytes()
    return bytes(out)


class ProgramBuilder:
    """Convenience layer used by the synthetic model generators: keeps parameters next
    to the program and emits feed / fetch ops the way Paddle's ``save_inference_model`` does."""

    def __init__(self):
        self.prog = PaddleProgram()
        self.params: Dict[str, np.ndarray] = {}
        self._uid = 0
        self.prog.add_var("feed", var_type=VT_FEED_MINIBATCH, persistable=True)
        self.prog.add_var("fetch", var_type=VT_FETCH_LIST, persistable=True)
        self._n_feed = 0
        self._n_fetch = 0

    def tmp(self, prefix: str = "tmp", dtype: str = "float32", shape: Sequence[int] = ()) -> str:
        self._uid += 1
        return self.prog.add_var(f"{prefix}_{self._uid}", dtype, shape)

    def feed(self, name: str, dtype: str, shape: Sequence[int]) -> str:
        self.prog.add_var(name, dtype, shape)
        self.prog.add_op("feed", {"X": ["feed"]}, {"Out": [name]}, col=self._n_feed)
        self._n_feed += 1
        return name

    def fetch(self, name: str) -> None:
        self.prog.add_op("fetch", {"X": [name]}, {"Out": ["fetch"]}, col=self._n_fetch)
        self._n_fetch += 1

    def param(self, name: str, value: np.ndarray) -> str:
        self.prog.add_var(name, value.dtype.name, value.shape, persistable=True)
        self.params[name] = value
        return name

    def op(self, type_: str, inputs: Dict[str, Sequence[str]], out_keys: Sequence[str] = ("Out",),
           out_shape: Sequence[int] = (), var_dtype: str = "float32", **attrs) -> str:
        """Adds an op with fresh output variables; returns the first output name."""
        outs = {k: [self.tmp(type_, var_dtype, out_shape)] for k in out_keys}
        self.prog.add_op(type_, inputs, outs, **attrs)
        return outs[out_keys[0]][0]

    def sub_block(self, ops: Sequence[Tuple[str, Dict[str, Sequence[str]], Dict[str, Sequence[str]], Dict[str, Any]]],
                  new_vars: Sequence[Tuple[str, str, Sequence[int]]] = ()) -> BlockRef:
        """Adds a sub-block made of ``(type, inputs, outputs, attrs)`` ops; ``new_vars`` = ``(name, dtype, shape)`` of
        the variables that only live inside it. Returns the reference to put into a ``sub_block`` attribute."""
        vars_ = {n: PaddleVar(n, dt, list(shape), False) for n, dt, shape in new_vars}
        block_ops = [PaddleOp(t, {k: list(v) for k, v in i.items()}, {k: list(v) for k, v in o.items()}, dict(a))
                     for t, i, o, a in ops]
        self.prog.sub_blocks.append((vars_, block_ops))
        return BlockRef(len(self.prog.sub_blocks))

    def serialize(self) -> Tuple[bytes, bytes]:
        return serialize_program(self.prog), serialize_params(self.prog, self.params)
