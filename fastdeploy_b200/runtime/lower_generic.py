"""Native lowering of the "small change" operators: views, casts, broadcasting arithmetic and logic, soft-max,
reductions, gathers, concatenation along any axis, constant padding.

A plan is static - every buffer has a fixed address - so an operator whose result is only another way of
indexing its input (Reshape, Transpose, Squeeze, Slice, Expand, Split ...) becomes a torch *view* recorded at build
time and costs no launch at all; the rest runs on the stride-generic kernels of :mod:`fastdeploy_b200.ops.generic`.
Compile-time-known values (shape arithmetic) are baked in as constants.

The interpreter's torch implementation of each operator is evaluated once while the plan is built: it gives the
result's shape and element type, and it is the fallback for the operators this module does not cover.

The reference hands these operators to its vendor engines (fastdeploy/runtime/backends/tensorrt/trt_backend.cc:347,
fastdeploy/runtime/backends/ort/ort_backend.cc:296).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..ir import interp
from ..ir.graph import Node
from ..ops import generic as G

VIEW_OPS = {"Reshape", "Flatten", "Squeeze", "Unsqueeze", "Transpose", "Identity", "Slice", "Expand", "Split", "Dropout"}
_COPY_IF_NOT_VIEW = {"Reshape", "Flatten"}

BINARY = {"Add": "add", "Sub": "sub", "Mul": "mul", "Div": "div", "Max": "max", "Min": "min", "Pow": "pow", "Equal": "eq",
          "Less": "lt", "LessOrEqual": "le", "Greater": "gt", "GreaterOrEqual": "ge", "And": "and", "Or": "or",
          "Xor": "xor", "Mod": "mod", "Sum": "add"}
UNARY = {"Not": "not", "Neg": "neg", "Abs": "abs", "Sqrt": "sqrt", "Exp": "exp", "Log": "log", "Tanh": "tanh",
         "Sigmoid": "sigmoid", "Relu": "relu", "Erf": "erf", "Floor": "floor", "Ceil": "ceil", "Round": "round",
         "Sign": "sign", "Reciprocal": "reciprocal", "Cast": "identity", "Sin": "sin", "Cos": "cos",
         "HardSwish": "hard_swish", "Silu": "silu", "Swish": "silu", "Softplus": "softplus"}
REDUCE = {"ReduceSum": "sum", "ReduceMean": "mean", "ReduceMax": "max", "ReduceMin": "min", "ReduceProd": "prod",
          "ArgMax": "argmax", "ArgMin": "argmin"}


def _same_storage(a: torch.Tensor, b: torch.Tensor) -> bool:
    return a.untyped_storage().data_ptr() == b.untyped_storage().data_ptr()


class GenericLowering:
    """Mixed into :class:`fastdeploy_b200.runtime.native_backend.Lowering`."""

    # ------------------------------------------------------------------ helpers
    def copy(self, src: torch.Tensor, dst: torch.Tensor, name: str, node: Optional[Node] = None) -> None:
        """Emits ``dst = cast(src)`` (any strided views, ``src`` broadcast to ``dst``) as one native launch."""
        try:
            op = G.strided_copy(src, dst, name=name)
        except (ValueError, KeyError):
            # more than six non-mergeable dimensions, or an element type the kernels do not know
            def cp(src=src, dst=dst):
                dst.copy_(src)
            self.plan.add_py(cp, f"torch:{name}", node)
            cp()
            return
        self.plan.add_native(op, node)
        op.launch()

    def _emit(self, op, node: Optional[Node]) -> None:
        self.plan.add_native(op, node)
        op.launch()

    def _torch_args(self, node: Node, upcast: bool):
        """Input tensors of ``node`` as the interpreter wants them (value arguments on the host)."""
        from ..ir.shape_infer import VALUE_ARGS
        ins = [None if nm == "" else self.as_torch(nm) for nm in node.inputs]
        while ins and ins[-1] is None:
            ins.pop()
        args = []
        for k, t in enumerate(ins):
            if k in VALUE_ARGS.get(node.op, ()) and node.inputs[k] in self.info.values:
                args.append(torch.from_numpy(np.ascontiguousarray(self.info.values[node.inputs[k]])))
            elif upcast and t is not None and t.dtype in (torch.float16, torch.bfloat16):
                args.append(t.float())
            else:
                args.append(t)
        return ins, args

    def _oracle(self, node: Node):
        """Runs the interpreter's implementation once at build time: result tensors (shape, dtype, values)."""
        fn = interp._OPS.get(node.op)
        if fn is None:
            return None
        node.attrs.setdefault("_opset", self.g.opset)
        _, args = self._torch_args(node, upcast=True)
        with torch.no_grad():
            r = fn(node, *args)
        return r if isinstance(r, tuple) else (r,)

    def _flows_16bit(self, node: Node) -> bool:
        return any(nm in self.vals and self.vals[nm].nhwc and self.vals[nm].t.dtype == self.dtype for nm in node.inputs)

    def _alloc_out(self, node: Node, name: str, like: torch.Tensor):
        """Destination of a generic op: ``(Val, logical tensor to write through)``. A 4-D float result that continues
        a 16-bit NHWC activation stays NHWC (or lands in its promised concatenation slice); everything else is a
        contiguous tensor of the interpreter's element type."""
        from .native_backend import Val
        if like.dim() == 4 and like.is_floating_point() and (name in self.preassigned or self._flows_16bit(node)):
            v = self.out_nhwc(name)
            return v, v.logical()
        t = torch.zeros(like.shape, dtype=like.dtype, device=self.device)
        return Val(t, False), t

    # ------------------------------------------------------------------ entry
    def lower_generic(self, node: Node) -> bool:
        """Tries the native generic paths for ``node``; False sends it to the torch fallback."""
        outs = [o for o in node.outputs if o]
        if outs and all(o in self.info.values for o in outs) and node.op not in ("MultiClassNMS", "PPYOLOEPost"):
            return self._bake_constants(node)
        try:
            if node.op in VIEW_OPS:
                return self._lower_view(node)
            if node.op in BINARY:
                return self._lower_ew_binary(node)
            if node.op in UNARY or node.op in ("Clip", "HardSigmoid", "LeakyRelu", "Gelu"):
                return self._lower_ew_unary(node)
            if node.op in ("Softmax", "LogSoftmax"):
                return self._lower_softmax(node)
            if node.op in REDUCE:
                return self._lower_reduce(node)
            if node.op == "Where":
                return self._lower_where(node)
            if node.op == "Gather":
                return self._lower_gather(node)
            if node.op == "Concat":
                return self._lower_concat_any(node)
            if node.op == "Pad":
                return self._lower_pad(node)
        except (ValueError, KeyError, AssertionError):
            return False
        return False

    def _bake_constants(self, node: Node) -> bool:
        from .native_backend import Val
        for o in node.outputs:
            if o:
                t = torch.from_numpy(np.ascontiguousarray(self.info.values[o]))
                if t.dtype == torch.float64:
                    t = t.float()
                self.vals[o] = Val(t.to(self.device), False)
        return True

    # ------------------------------------------------------------------ views
    def _lower_view(self, node: Node) -> bool:
        from .native_backend import Val
        fn = interp._OPS[node.op]
        node.attrs.setdefault("_opset", self.g.opset)
        ins, args = self._torch_args(node, upcast=False)
        data = ins[0]
        with torch.no_grad():
            r = fn(node, *args)
        res = r if isinstance(r, tuple) else (r,)
        staged = []
        for name, o in zip(node.outputs, res):
            if not name:
                continue
            if _same_storage(o, data):
                staged.append((name, o, None))
            elif node.op in _COPY_IF_NOT_VIEW and o.numel() == data.numel():
                staged.append((name, o, data))
            else:
                return False
        for name, o, src in staged:
            if src is None:
                self.vals[name] = Val(o, False)
            else:
                dst = torch.zeros(o.shape, dtype=o.dtype, device=self.device)
                self.copy(src, dst.view(src.shape), f"reshape_copy({name})", node)
                self.vals[name] = Val(dst, False)
            if name in self.preassigned:
                self._copy_into_slice(name)
        return True

    # ------------------------------------------------------------------ elementwise
    def _lower_ew_binary(self, node: Node) -> bool:
        if node.op == "Mod" and node.attr("fmod", 0):
            return False
        names = [nm for nm in node.inputs if nm]
        if len(names) != 2:
            return False
        ref = self._oracle(node)[0]
        a, b = self.as_torch(names[0]), self.as_torch(names[1])
        if not all(G.supported(t.dtype) for t in (a, b, ref)):
            return False
        val, out = self._alloc_out(node, node.outputs[0], ref)
        self._emit(G.elementwise(BINARY[node.op], a, b, out, name=f"ew_{BINARY[node.op]}:{node.name}"), node)
        self.vals[node.outputs[0]] = val
        return True

    def _lower_ew_unary(self, node: Node) -> bool:
        ref = self._oracle(node)[0]
        x = self.as_torch(node.inputs[0])
        if not (G.supported(x.dtype) and G.supported(ref.dtype)):
            return False
        f0 = f1 = 0.0
        if node.op == "Clip":
            def bound(k, attr, default):
                if len(node.inputs) > k and node.inputs[k]:
                    v = self.info.values.get(node.inputs[k])
                    if v is None and node.inputs[k] in self.g.initializers:
                        v = self.g.initializers[node.inputs[k]]
                    if v is None:
                        raise ValueError("Clip bound is not a constant")
                    return float(np.asarray(v).reshape(-1)[0])
                return float(node.attr(attr, default))
            f0, f1 = bound(1, "min", -3.4028234e38), bound(2, "max", 3.4028234e38)
            opname = "clip"
        elif node.op == "HardSigmoid":
            f0, f1, opname = node.attr("alpha", 0.2), node.attr("beta", 0.5), "hard_sigmoid"
        elif node.op == "LeakyRelu":
            f0, opname = node.attr("alpha", 0.01), "leaky_relu"
        elif node.op == "Gelu":
            if node.attr("approximate", "none") == "tanh":
                return False
            opname = "gelu"
        else:
            opname = UNARY[node.op]
        val, out = self._alloc_out(node, node.outputs[0], ref)
        self._emit(G.elementwise(opname, x, None, out, f0, f1, name=f"ew_{opname}:{node.name}"), node)
        self.vals[node.outputs[0]] = val
        return True

    def _lower_where(self, node: Node) -> bool:
        ref = self._oracle(node)[0]
        c, a, b = (self.as_torch(nm) for nm in node.inputs[:3])
        if not all(G.supported(t.dtype) for t in (c, a, b, ref)):
            return False
        val, out = self._alloc_out(node, node.outputs[0], ref)
        self._emit(G.where(c, a, b, out), node)
        self.vals[node.outputs[0]] = val
        return True

    # ------------------------------------------------------------------ soft-max / reductions
    def _rows_contiguous(self, x: torch.Tensor, name: str, node: Node) -> torch.Tensor:
        """``x`` itself when it is a stack of unit-stride rows at one pitch, else a contiguous copy (one launch)."""
        if G.rows_of(x) is not None:
            return x
        tmp = torch.zeros(x.shape, dtype=x.dtype, device=self.device)
        self.copy(x, tmp, f"to_rows({name})", node)
        return tmp

    def _lower_softmax(self, node: Node) -> bool:
        from .native_backend import Val
        x = self.as_torch(node.inputs[0])
        nd = x.dim()
        opset = node.attr("_opset", self.g.opset)
        axis = node.attr("axis", -1 if opset >= 13 else 1)
        axis = axis if axis >= 0 else nd + axis
        if opset < 13 and axis != nd - 1:
            return False                # "flatten from axis" semantics of the old opsets
        if not G.supported(x.dtype) or nd == 0:
            return False
        xm = x.movedim(axis, -1)
        xr = self._rows_contiguous(xm, node.inputs[0], node)
        y = torch.zeros(xm.shape, dtype=torch.float32, device=self.device)
        self._emit(G.softmax_last(xr, y, log=node.op == "LogSoftmax"), node)
        self.vals[node.outputs[0]] = Val(y.movedim(-1, axis), False)
        return True

    def _lower_reduce(self, node: Node) -> bool:
        from .native_backend import Val
        ref = self._oracle(node)[0]
        x = self.as_torch(node.inputs[0])
        nd = x.dim()
        if nd == 0 or not (G.supported(x.dtype) and G.supported(ref.dtype)):
            return False
        if node.op in ("ArgMax", "ArgMin"):
            if node.attr("select_last_index", 0):
                return False
            axes = [node.attr("axis", 0)]
            keep = bool(node.attr("keepdims", 1))
        else:
            axes = None
            if len(node.inputs) > 1 and node.inputs[1]:
                v = self.info.values.get(node.inputs[1])
                if v is None:
                    return False
                axes = [int(a) for a in np.asarray(v).reshape(-1)]
            if axes is None:
                axes = node.attr("axes", None)
            if not axes:
                if node.attr("noop_with_empty_axes", 0):
                    return False
                axes = list(range(nd))
            keep = bool(node.attr("keepdims", 1))
        axes = sorted(a if a >= 0 else nd + a for a in axes)
        kept = [d for d in range(nd) if d not in axes]
        xp = x.permute(kept + axes)
        red = int(np.prod([x.shape[a] for a in axes]))
        lead = [x.shape[d] for d in kept]
        # [kept dims..., reduced elements] with unit stride over the reduced block
        if len(axes) == 1 and xp.stride(-1) == 1 and G.rows_of(xp) is not None:
            x2 = xp
        else:
            tmp = torch.zeros(list(xp.shape), dtype=x.dtype, device=self.device)
            self.copy(xp, tmp, f"to_rows({node.inputs[0]})", node)
            x2 = tmp.view(lead + [red])
        y = torch.zeros(lead if lead else [1], dtype=ref.dtype, device=self.device)
        self._emit(G.reduce_last(REDUCE[node.op], x2, y), node)
        out = y.view(lead) if lead else y.view([])
        if keep:
            for a in axes:
                out = out.unsqueeze(a)
        if list(out.shape) != list(ref.shape):
            raise ValueError("reduce: unexpected result shape")
        self.vals[node.outputs[0]] = Val(out, False)
        return True

    # ------------------------------------------------------------------ gather / concat / pad
    def _lower_gather(self, node: Node) -> bool:
        from .native_backend import Val
        x = self.as_torch(node.inputs[0])
        axis = node.attr("axis", 0)
        axis = axis if axis >= 0 else x.dim() + axis
        idx_name = node.inputs[1]
        const = self.info.values.get(idx_name)
        if const is None and idx_name in self.g.initializers:
            const = self.g.initializers[idx_name]
        if const is not None and np.asarray(const).ndim == 0:         # constant scalar index: a view
            i = int(const)
            i = i + x.shape[axis] if i < 0 else i
            self.vals[node.outputs[0]] = Val(x.select(axis, i), False)
            return True
        if axis != 0 or not G.supported(x.dtype):
            return False
        idx = self.as_torch(idx_name)
        if idx.dtype not in (torch.int64, torch.int32):
            return False
        if not x.is_contiguous():
            t = torch.zeros(x.shape, dtype=x.dtype, device=self.device)
            self.copy(x, t, f"gather_table({node.inputs[0]})", node)
            x = t
        if not idx.is_contiguous():
            t = torch.zeros(idx.shape, dtype=idx.dtype, device=self.device)
            self.copy(idx, t, f"gather_index({idx_name})", node)
            idx = t
        out_dt = torch.float32 if x.dtype in (torch.float16, torch.bfloat16) else x.dtype
        out = torch.zeros(list(idx.shape) + list(x.shape[1:]), dtype=out_dt, device=self.device)
        self._emit(G.gather_rows(x, idx, out), node)
        self.vals[node.outputs[0]] = Val(out, False)
        return True

    def _lower_concat_any(self, node: Node) -> bool:
        ref = self._oracle(node)[0]
        if not G.supported(ref.dtype):
            return False
        axis = node.attr("axis", 0)
        axis = axis if axis >= 0 else ref.dim() + axis
        val, out = self._alloc_out(node, node.outputs[0], ref)
        off = 0
        for nm in node.inputs:
            src = self.as_torch(nm)
            k = src.shape[axis]
            if k:
                self.copy(src, out.narrow(axis, off, k), f"concat_copy({nm})", node)
            off += k
        self.vals[node.outputs[0]] = val
        return True

    def _lower_pad(self, node: Node) -> bool:
        if node.attr("mode", "constant") != "constant":
            return False
        ref = self._oracle(node)[0]
        x = self.as_torch(node.inputs[0])
        if not (G.supported(ref.dtype) and G.supported(x.dtype)):
            return False
        pads = self.info.values.get(node.inputs[1]) if len(node.inputs) > 1 and node.inputs[1] else node.attr("pads", None)
        if pads is None and len(node.inputs) > 1 and node.inputs[1] in self.g.initializers:
            pads = self.g.initializers[node.inputs[1]]
        if pads is None or (len(node.inputs) > 3 and node.inputs[3]):
            return False
        pads = [int(p) for p in np.asarray(pads).reshape(-1)]
        nd = x.dim()
        if len(pads) != 2 * nd or any(p < 0 for p in pads):
            return False
        val, out = self._alloc_out(node, node.outputs[0], ref)
        # the border never changes between replays: fill it once, from the interpreter's result
        out.copy_(ref.to(self.device))
        inner = out
        for d in range(nd):
            inner = inner.narrow(d, pads[d], x.shape[d])
        self.copy(x, inner, f"pad_copy({node.inputs[0]})", node)
        self.vals[node.outputs[0]] = val
        return True
