"""Paddle control flow -> graph IR: ``while`` becomes ``Loop``, ``conditional_block`` becomes ``If``, ``select_input``
picks one of its operands at run time (paddle2onnx/mapper/loop.cc:20-195 exports ``while`` the same way; the
conditional forms go beyond it).

Paddle blocks are not in single-assignment form: a ``while`` block overwrites the loop variables (and its own
condition) under their outer names, ``increment`` works in place. The importer therefore renames as it goes
(``Renamer``): every later write of a name gets a fresh value name and later reads follow it.

* ``while(X, Condition) -> Out``: ``Loop("", cond, carried...)`` whose body graph takes ``(iteration, cond, carried...)``
  and returns ``(cond', carried'...)``; the carried values are the block's ``Out`` variables, everything else the
  block reads is taken from the enclosing scope by name (recorded in the node's ``outer_refs`` so that pruning and
  sorting keep the producers).
* ``conditional_block(Cond, Input) -> Out``: ``If(cond)`` with the sub-block as ``then_branch``; the ``else_branch``
  hands back the previous value of a variable that already existed and an empty tensor for one that did not (Paddle
  leaves it unset; the ``select_input`` that follows never picks it).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Set

import numpy as np

from ..ir.graph import Graph, Node, ValueInfo, body_outer_refs
from .paddle_format import PaddleOp, PaddleProgram, PaddleVar

CONTROL_OPS = ("while", "conditional_block", "select_input")


class Renamer:
    """Single-assignment renaming of Paddle variable names within one scope."""

    def __init__(self, defined: Set[str], current: Optional[Dict[str, str]] = None):
        self.defined = set(defined)
        self.cur: Dict[str, str] = dict(current or {})
        self._n = 0

    def read(self, name: str) -> str:
        return self.cur.get(name, name)

    def write(self, name: str) -> str:
        if name not in self.defined:
            self.defined.add(name)
            self.cur.pop(name, None)
            return name
        self._n += 1
        new = f"{name}@{self._n}"
        while new in self.defined:
            self._n += 1
            new = f"{name}@{self._n}"
        self.defined.add(new)
        self.cur[name] = new
        return new

    def apply(self, op: PaddleOp) -> PaddleOp:
        ins = {k: [self.read(a) for a in v] for k, v in op.inputs.items()}
        outs = {k: [self.write(a) for a in v] for k, v in op.outputs.items()}
        return PaddleOp(op.type, ins, outs, dict(op.attrs))


def _scope_program(prog: PaddleProgram, block_vars: Dict[str, PaddleVar], aliases: Dict[str, str]) -> PaddleProgram:
    """A program view whose variable table also knows the sub-block's variables and the renamed names."""
    view = PaddleProgram()
    view.vars = dict(prog.vars)
    view.vars.update(block_vars)
    for new, old in aliases.items():
        if old in view.vars and new not in view.vars:
            v = view.vars[old]
            view.vars[new] = PaddleVar(new, v.dtype, list(v.shape), False, v.var_type)
    view.sub_blocks = prog.sub_blocks
    view.version = prog.version
    return view


def run_op(ctx, op: PaddleOp, mappers) -> None:
    """Renames ``op`` into single-assignment form in ``ctx``'s scope and maps it. The mapper of a control-flow op
    also needs the op as written (``ctx.raw_op``) and the scope as it was before the op's own outputs were renamed."""
    r: Renamer = ctx.renamer
    ctx.raw_op, ctx.cur_before, ctx.defined_before = op, dict(r.cur), set(r.defined)
    renamed = r.apply(op)
    for key, old_names in op.outputs.items():
        for new, old in zip(renamed.outputs[key], old_names):
            if new != old and old in ctx.prog.vars and new not in ctx.prog.vars:
                v = ctx.prog.vars[old]
                ctx.prog.vars[new] = PaddleVar(new, v.dtype, list(v.shape), False, v.var_type)
    if op.type not in mappers:
        raise NotImplementedError(f"paddle importer: unsupported operator {op.type!r}")
    mappers[op.type](ctx, renamed)


def _import_block(ctx, block_idx: int, body: Graph, renamer: Renamer, mappers) -> None:
    """Maps the ops of sub-block ``block_idx`` into ``body`` (recursively for nested control flow)."""
    from .paddle_import import Ctx
    block_vars, ops = ctx.prog.sub_blocks[block_idx - 1]
    sub = Ctx(_scope_program(ctx.prog, block_vars, {}), body)
    sub.renamer = renamer
    body._uid = ctx.g._uid                                   # one counter for generated names in every scope
    for op in ops:
        run_op(sub, op, mappers)
    ctx.g._uid = body._uid


_outer_refs = body_outer_refs


def map_while(ctx, op: PaddleOp, mappers) -> None:
    r: Renamer = ctx.renamer
    block = int(op.attr("sub_block"))
    cond_name = op.inputs["Condition"][0]                    # already renamed to the current outer value
    raw = getattr(ctx, "raw_op", op)                          # the op before renaming: original variable names
    cond_var = raw.inputs["Condition"][0]
    carried_vars = [v for v in dict.fromkeys(raw.outputs.get("Out", [])) if v != cond_var]
    known = set(raw.inputs.get("X", [])) | {cond_var}
    missing = [v for v in carried_vars if v not in known]
    if missing:
        raise NotImplementedError(f"while: outputs {missing} are not among the inputs (tensor arrays are not supported)")
    uid = ctx.g.unique("loop")
    body = Graph(f"{uid}_body", ctx.g.opset)
    it_in, cond_in = f"{uid}@iter", f"{uid}@cond_in"
    body.inputs.append(ValueInfo(it_in, "int64", []))
    body.inputs.append(ValueInfo(cond_in, "bool", []))
    before = dict(getattr(ctx, "cur_before", r.cur))           # the scope before this op's own outputs were renamed
    start = dict(before)                                      # reads of other outer names follow the outer renaming
    start[cond_var] = cond_in
    outer_now = {}
    for v in carried_vars:
        name_in = f"{uid}@{v}"
        pv = ctx.prog.vars.get(v)
        body.inputs.append(ValueInfo(name_in, pv.dtype if pv else "float32", None))
        start[v] = name_in
        outer_now[v] = before.get(v, v)                       # value of the variable just before the loop
    inner = Renamer(r.defined | {it_in, cond_in} | set(start.values()), start)
    _import_block(ctx, block, body, inner, mappers)
    body.outputs.append(ValueInfo(inner.read(cond_var), "bool", None))
    for v in carried_vars:
        pv = ctx.prog.vars.get(v)
        body.outputs.append(ValueInfo(inner.read(v), pv.dtype if pv else "float32", None))
    r.defined |= inner.defined
    outs = []
    for v in carried_vars:
        # the names `r.apply` gave to the while op's outputs stand for the values after the loop
        idx = raw.outputs["Out"].index(v)
        outs.append(op.outputs["Out"][idx])
    ctx.g.add_node("Loop", ["", cond_name] + [outer_now[v] for v in carried_vars], outs, body=body,
                   outer_refs=_outer_refs(body))
    # after the loop the condition is false
    false_name = ctx.g.const(np.zeros(1, np.bool_))
    if cond_var in raw.outputs.get("Out", []):
        idx = raw.outputs["Out"].index(cond_var)
        ctx.g.add_node("Identity", [false_name], [op.outputs["Out"][idx]])


def map_conditional_block(ctx, op: PaddleOp, mappers) -> None:
    r: Renamer = ctx.renamer
    raw = getattr(ctx, "raw_op", op)
    block = int(op.attr("sub_block"))
    cond_name = op.inputs["Cond"][0]
    out_vars = list(dict.fromkeys(raw.outputs.get("Out", [])))
    uid = ctx.g.unique("if")
    then_g = Graph(f"{uid}_then", ctx.g.opset)
    # inside the block the outer names still mean the values from before the op (its own outputs were renamed already)
    before = dict(getattr(ctx, "cur_before", r.cur))
    inner = Renamer(r.defined, before)
    _import_block(ctx, block, then_g, inner, mappers)
    else_g = Graph(f"{uid}_else", ctx.g.opset)
    for v in out_vars:
        pv = ctx.prog.vars.get(v) or ctx.prog.sub_blocks[block - 1][0].get(v)
        dt = pv.dtype if pv else "float32"
        then_g.outputs.append(ValueInfo(inner.read(v), dt, None))
        prev = before.get(v, v)
        if prev in getattr(ctx, "defined_before", set()):
            else_name = f"{uid}@{v}@else"
            else_g.add_node("Identity", [prev], [else_name])
        else:
            else_name = else_g.const(np.zeros((0,), np.dtype(dt) if dt != "bfloat16" else np.float32))
            alias = f"{uid}@{v}@unset"
            else_g.add_node("Identity", [else_name], [alias])
            else_name = alias
        else_g.outputs.append(ValueInfo(else_name, dt, None))
    r.defined |= inner.defined
    outs = [op.outputs["Out"][raw.outputs["Out"].index(v)] for v in out_vars]
    refs = _outer_refs(then_g)
    refs += [x for x in _outer_refs(else_g) if x not in refs]
    ctx.g.add_node("If", [cond_name], outs, then_branch=then_g, else_branch=else_g, outer_refs=refs)


def map_select_input(ctx, op: PaddleOp, mappers) -> None:
    ctx.g.add_node("SelectInput", [op.inputs["Mask"][0]] + list(op.inputs["X"]), [op.outputs["Out"][0]], domain="fdb")


def map_increment(ctx, op: PaddleOp, mappers) -> None:
    x = op.inputs["X"][0]
    dt = ctx.dtype(getattr(ctx, "raw_op", op).inputs["X"][0])
    step = ctx.g.const(np.asarray([op.attr("step", 1.0)], np.dtype(dt if dt != "bfloat16" else "float32")))
    ctx.g.add_node("Add", [x, step], [op.outputs["Out"][0]])


CONTROL_MAPPERS = {"while": map_while, "conditional_block": map_conditional_block, "select_input": map_select_input,
                   "increment": map_increment}
