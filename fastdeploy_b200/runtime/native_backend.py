"""The single native backend: lowers an optimised IR graph to a static launch plan of
sm_100a kernels for one concrete set of input shapes ("shape bucket"), optionally
captured into a CUDA graph.

It replaces the reference's ten vendor backends behind ``BaseBackend``
(fastdeploy/runtime/backends/backend.h:51-97): where TensorRT rebuilds an engine when
an unseen shape arrives (fastdeploy/runtime/backends/tensorrt/trt_backend.cc:327-339),
this backend keeps one plan per shape bucket and builds a new one in milliseconds.

Layout and precision: 4-D activations live as NHWC fp16/bf16 tensors (logically NCHW),
channel counts are padded to multiples of 8, concat / split along channels are
realised as channel-slice views so producers write straight into the concatenated
buffer. View-like operators (Reshape, Transpose, Slice ...) become torch views recorded at
build time; casts, broadcasting arithmetic, soft-max, reductions and gathers run on the
stride-generic kernels of ``lower_generic.py``. Only operators that neither path covers
(LSTM, TopK, NonZero ...) run through the interpreter's torch implementation; such a step
shows up in the plan under the name ``torch:<op>``.
"""
from __future__ import annotations

import ctypes
import math
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import _native
from ..ir import interp, passes
from ..ir.graph import Graph, Node
from ..ir.shape_infer import ShapeInfo, infer_shapes
from ..ops import nhwc as K
from ..utils import log
from ..ops import stem_conv
from ..ops.base import NativeOp, StatusWord, current_stream_ptr
from ..ops.conv_gemm import ConvGemm, pack_conv_weight, pack_linear_weight
from ..ops.nms import MulticlassNMS
from .lower_generic import GenericLowering


_NVTX = __import__("os").environ.get("FDX_NVTX", "0") not in ("", "0")


def _round8(c: int) -> int:
    return (c + 7) // 8 * 8


@dataclass
class Val:
    """A value on the device. ``nhwc``: ``t`` is ``[N,H,W,C]`` (maybe a channel slice of a
    wider buffer, ``t.stride(2)`` = channel stride) holding the logical ``[N,C,H,W]`` tensor;
    otherwise ``t`` is a torch tensor in the logical layout."""
    t: torch.Tensor
    nhwc: bool = False

    @property
    def logical_shape(self) -> List[int]:
        if self.nhwc:
            n, h, w, c = self.t.shape
            return [n, c, h, w]
        return list(self.t.shape)

    def logical(self) -> torch.Tensor:
        return self.t.permute(0, 3, 1, 2) if self.nhwc else self.t

    @property
    def ld(self) -> int:
        return self.t.stride(2)

    @property
    def n_stride(self) -> int:
        return self.t.stride(0)


class Step:
    """One plan entry: a native op or a python callable."""
    __slots__ = ("fn", "native", "name", "node")

    def __init__(self, fn: Callable[[], None], native: Optional[NativeOp], name: str, node: Optional[Node]):
        self.fn, self.native, self.name, self.node = fn, native, name, node


class Plan:
    """Static launch list for one shape bucket."""

    def __init__(self, device: torch.device):
        self.device = device
        self.steps: List[Step] = []
        self.inputs: Dict[str, Val] = {}
        self.outputs: Dict[str, Val] = {}
        self.status = StatusWord(device)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.native_plan = None
        self._segments: List[Any] = []
        self.native_kernel_launches = 0
        self.extra: Dict[str, Any] = {}

    # ------------------------------------------------------------------ building
    def add_native(self, op: NativeOp, node: Optional[Node] = None, launches: int = 1) -> None:
        self.steps.append(Step(op.launch, op, op.name, node))
        self.native_kernel_launches += launches

    def add_py(self, fn: Callable[[], None], name: str, node: Optional[Node] = None) -> None:
        self.steps.append(Step(fn, None, name, node))

    def finalize(self) -> None:
        """Groups consecutive native ops into native sub-plans (one ctypes call each)."""
        lib = _native.kernels()
        self._segments = []
        run: List[Step] = []

        def flush():
            if not run:
                return
            handle = ctypes.c_void_p(lib.fdb_plan_create())
            for s in run:
                lib.fdb_plan_add(handle, s.native.handle, 0)
            self._segments.append(("native", handle, list(run)))
            run.clear()
        for s in self.steps:
            if s.native is not None:
                run.append(s)
            else:
                flush()
                self._segments.append(("py", s.fn, s))
        flush()

    # ------------------------------------------------------------------ running
    def run(self) -> None:
        if self.graph is not None:
            self.graph.replay()
            return
        self._run_eager()

    def _run_eager(self) -> None:
        lib = _native.kernels()
        stream = ctypes.c_void_p(current_stream_ptr(self.device))
        if _NVTX:
            for s in self.steps:                   # one range per step instead of one native call per segment
                torch.cuda.nvtx.range_push(s.name)
                s.fn()
                torch.cuda.nvtx.range_pop()
            return
        for kind, obj, _ in self._segments:
            if kind == "native":
                if lib.fdb_plan_run(obj, stream) != 0:
                    raise RuntimeError(f"native plan failed: {_native.last_error()}")
            else:
                obj()

    def trace(self, path: str = "", iters: int = 3) -> Dict[str, Any]:
        """Runs the plan step by step with a CUDA event pair around every step and returns (and optionally writes) a
        Chrome-trace document (``chrome://tracing`` / Perfetto): one complete event per step with its device time, on
        a time axis of cumulative device time. With ``FDX_NVTX=1`` in the environment every step of an eager run is
        also an NVTX range, so an external timeline tool shows the same names."""
        import json
        names = [s.name for s in self.steps]
        best = [float("inf")] * len(self.steps)
        for _ in range(max(1, iters)):
            evs = []
            for s in self.steps:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                s.fn()
                e1.record()
                evs.append((e0, e1))
            torch.cuda.synchronize(self.device)
            for k, (e0, e1) in enumerate(evs):
                best[k] = min(best[k], e0.elapsed_time(e1) * 1e3)      # microseconds
        events, ts = [], 0.0
        for k, (name, dur) in enumerate(zip(names, best)):
            node = self.steps[k].node
            events.append({"name": name, "cat": "native" if self.steps[k].native is not None else "framework", "ph": "X",
                           "ts": round(ts, 3), "dur": round(dur, 3), "pid": 0, "tid": int(self.device.index or 0),
                           "args": {"step": k, "op": node.op if node is not None else ""}})
            ts += dur
        doc = {"traceEvents": events, "displayTimeUnit": "ms",
               "otherData": {"steps": len(events), "sum_us": round(ts, 1), "launches": self.native_kernel_launches}}
        if path:
            with open(path, "w") as f:
                json.dump(doc, f)
        return doc

    def capture(self, warmup: int = 2) -> None:
        """Captures the whole plan into one CUDA graph (replay = one launch)."""
        s = torch.cuda.Stream(self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(s):
            for _ in range(warmup):
                self._run_eager()
        torch.cuda.current_stream(self.device).wait_stream(s)
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        # thread-local capture: worker threads of other GPUs keep allocating and launching meanwhile
        with torch.cuda.graph(g, stream=s, capture_error_mode="thread_local"):
            self._run_eager()
        self.graph = g

    def __del__(self):
        try:
            lib = _native.kernels()
            for kind, obj, _ in self._segments:
                if kind == "native":
                    lib.fdb_plan_destroy(obj)
        except Exception:
            pass


class Lowering(GenericLowering):
    """Builds a :class:`Plan` from an optimised graph and concrete input shapes."""

    def __init__(self, graph: Graph, input_shapes: Dict[str, Sequence[int]], device: torch.device,
                 dtype: torch.dtype = torch.float16, input_values: Optional[Dict[str, np.ndarray]] = None,
                 fp8: bool = False, act_scales: Optional[Dict[str, float]] = None, reuse_buffers: bool = False):
        self.g = graph
        self.device = device
        self.dtype = dtype
        # fp8: linear layers run as e4m3 GEMMs (per-output-channel weight scales; activations quantised with the
        # calibrated static range when one is known for the tensor, else per row on the fly)
        self.fp8 = fp8
        self.act_scales = dict(passes.get_act_scales(graph))
        self.act_scales.update(act_scales or {})
        self.q8: Dict[str, Tuple[torch.Tensor, Optional[torch.Tensor], float]] = {}
        self.fp8_gemms = 0
        self.info: ShapeInfo = infer_shapes(graph, input_shapes, input_values)
        self.plan = Plan(device)
        self.vals: Dict[str, Val] = {}
        self.consts: Dict[str, torch.Tensor] = {}
        self.packed: Dict[Tuple[str, str], torch.Tensor] = {}
        self.cons = graph.consumers()
        self.prod = graph.producers()
        self.preassigned: Dict[str, Val] = {}
        self.fused_away: set = set()        # ids of nodes that an earlier node's lowering has already covered
        self.pending_gate: Dict[str, Tuple[str, str]] = {}   # gated map -> (feature, gate) folded into its consumer
        # static memory plan (runtime/arena.py): activation buffers whose readers are all lowered are handed back
        from .arena import Arena
        self.arena: Optional[Arena] = Arena(device) if reuse_buffers else None
        self.arena_open = False              # buffers made before the node loop (promised slices, heads) stay private
        self.remaining: Dict[str, int] = {}
        self.input_shapes = {k: list(v) for k, v in input_shapes.items()}

    # ------------------------------------------------------------------ helpers
    def const_f32(self, name: str) -> torch.Tensor:
        key = name
        if key not in self.consts:
            arr = self.g.initializers[name]
            t = torch.from_numpy(np.ascontiguousarray(arr))
            if t.dtype in (torch.float16, torch.float64):
                t = t.float()
            self.consts[key] = t.to(self.device)
        return self.consts[key]

    def new_nhwc(self, n: int, h: int, w: int, c: int, dtype: Optional[torch.dtype] = None) -> Val:
        cp = _round8(c)
        if self.arena is not None and self.arena_open and cp == c:
            # (padding channels must read as zero for good, so padded buffers stay out of the shared arena)
            return Val(self.arena.alloc((n, h, w, c), dtype or self.dtype), True)
        buf = torch.zeros(n, h, w, cp, dtype=dtype or self.dtype, device=self.device)
        return Val(buf[..., :c], True)

    def _release_dead(self, node: Node) -> None:
        """After ``node`` (lowered or covered by an earlier one): its inputs have one reader fewer; arena blocks that
        no value with readers to come, output, promised slice or held-back gate operand touches are handed back."""
        for nm in set(i for i in node.inputs if i):
            if nm in self.remaining:
                self.remaining[nm] -= 1
        needed = []
        outs = set(self.g.output_names())
        held = set()
        for gated, (feat, gate) in self.pending_gate.items():
            if self.remaining.get(gated, 0) > 0:
                held.update((feat, gate))
        for nm, v in self.vals.items():
            if self.remaining.get(nm, 0) > 0 or nm in outs or nm in held or nm in self.plan.inputs:
                needed.append(v.t)
        for nm, v in self.preassigned.items():
            if self.remaining.get(nm, 0) > 0 or nm in outs:
                needed.append(v.t)
        self.arena.release_unreferenced(needed)

    def out_nhwc(self, name: str, dtype: Optional[torch.dtype] = None) -> Val:
        """Destination of a 4-D op output: the pre-assigned concat slice or a fresh buffer."""
        if name in self.preassigned:
            return self.preassigned[name]
        n, c, h, w = self.info.shapes[name]
        return self.new_nhwc(n, h, w, c, dtype)

    def as_nhwc(self, name: str) -> Val:
        """Value as a 16-bit NHWC tensor with 8-aligned channel stride (converting if needed)."""
        v = self.get(name)
        if v.nhwc and v.t.dtype == self.dtype and v.t.stride(3) == 1 and v.ld % 8 == 0 \
                and v.t.data_ptr() % 16 == 0:
            return v
        if not v.nhwc and v.t.dim() == 4:
            # a view whose memory already is channel-innermost (e.g. a reshape of an NHWC buffer)
            p = v.t.permute(0, 2, 3, 1)
            if p.dtype == self.dtype and p.stride(3) == 1 and p.stride(2) % 8 == 0 and p.data_ptr() % 16 == 0 \
                    and p.stride(1) == p.stride(2) * p.shape[2]:
                nv = Val(p, True)
                self.vals[name] = nv
                return nv
        n, c, h, w = v.logical_shape
        dst = self.new_nhwc(n, h, w, c)
        self.copy(v.logical(), dst.logical(), f"to_nhwc({name})")
        self.vals[name] = dst
        return dst

    def as_torch(self, name: str, fp32: bool = True) -> torch.Tensor:
        """Logical-layout view for fallback ops (no copy; 16-bit floats are upcast lazily by the op)."""
        if name in self.g.initializers:
            return self.const_f32(name)
        return self.get(name).logical()

    def get(self, name: str) -> Val:
        if name in self.vals:
            return self.vals[name]
        if name in self.g.initializers:
            v = Val(self.const_f32(name), False)
            self.vals[name] = v
            return v
        raise KeyError(f"value {name!r} not produced yet")

    def is4d(self, name: str) -> bool:
        return len(self.info.shapes.get(name, [])) == 4

    # ------------------------------------------------------------------ driver
    def build(self) -> Plan:
        g = self.g
        # graph inputs
        for vi in g.inputs:
            shape = self.input_shapes[vi.name]
            tdt = interp.NP2TORCH[vi.dtype]
            if len(shape) == 4 and tdt.is_floating_point:
                n, c, h, w = shape
                v = self.new_nhwc(n, h, w, c)
            else:
                if tdt.is_floating_point:
                    tdt = torch.float32
                v = Val(torch.zeros(shape, dtype=tdt, device=self.device), False)
            self.vals[vi.name] = v
            self.plan.inputs[vi.name] = v
        self._plan_concats()
        for node in g.nodes:
            for nm in set(i for i in node.inputs if i):
                self.remaining[nm] = self.remaining.get(nm, 0) + 1
        self.arena_open = True
        for node in g.nodes:
            if id(node) not in self.fused_away:
                fn = getattr(self, "lower_" + node.op, None)
                done = False
                if fn is not None:
                    done = fn(node) is not False
                if not done:
                    self.lower_fallback(node)
            if self.arena is not None:
                self._release_dead(node)
        self.arena_open = False
        if self.arena is not None:
            self.plan.extra["memory"] = self.arena.report()
            self.plan.extra["arena"] = self.arena
        for vi in g.outputs:
            self.plan.outputs[vi.name] = self.get(vi.name)
        self.plan.finalize()
        torch.cuda.synchronize(self.device)
        self.plan.status.check("plan build")
        return self.plan

    def _plan_concats(self) -> None:
        """Pre-assigns channel slices of concat outputs to their producers (concat fusion)."""
        nhwc_producers = {"FusedConv", "MaxPool", "AveragePool", "Resize", "Mul", "Add", "Concat"}
        for node in self.g.nodes:
            if node.op != "Concat" or not self.is4d(node.outputs[0]):
                continue
            axis = node.attr("axis", 1)
            if axis not in (1, -3):
                continue
            n, c, h, w = self.info.shapes[node.outputs[0]]
            if node.outputs[0] in self.preassigned:
                dst = self.preassigned[node.outputs[0]]
            else:
                dst = self.new_nhwc(n, h, w, c)
                self.preassigned[node.outputs[0]] = dst
            off = 0
            for i in node.inputs:
                ci = self.info.shapes[i][1]
                p = self.prod.get(i)
                aligned = off % 8 == 0
                if (p is not None and p.op in nhwc_producers and i not in self.preassigned and aligned
                        and i not in self.g.output_names()):
                    self.preassigned[i] = Val(dst.t[..., off:off + ci], True)
                off += ci

    # ------------------------------------------------------------------ fallback
    def lower_fallback(self, node: Node) -> None:
        if self.lower_generic(node):
            return
        fn = interp._OPS.get(node.op)
        if fn is None:
            raise NotImplementedError(f"native backend: unsupported op {node.op}")
        args_names = list(node.inputs)
        ins = [None if nm == "" else self.as_torch(nm) for nm in args_names]
        while ins and ins[-1] is None:
            ins.pop()
        value_pos = {}
        from ..ir.shape_infer import VALUE_ARGS
        for k in VALUE_ARGS.get(node.op, ()):
            if k < len(node.inputs) and node.inputs[k] in self.info.values:
                value_pos[k] = torch.from_numpy(np.ascontiguousarray(self.info.values[node.inputs[k]]))
        node.attrs.setdefault("_opset", self.g.opset)

        def compute():
            a = []
            for k, t in enumerate(ins):
                if k in value_pos:
                    a.append(value_pos[k])
                elif t is not None and t.dtype in (torch.float16, torch.bfloat16):
                    a.append(t.float())
                else:
                    a.append(t)
            r = fn(node, *a)
            return r if isinstance(r, tuple) else (r,)
        with torch.no_grad():
            first = compute()
        outs = [torch.empty_like(r, memory_format=torch.contiguous_format).copy_(r) for r in first]

        def step():
            with torch.no_grad():
                for o, r in zip(outs, compute()):
                    o.copy_(r)
        self.plan.add_py(step, f"torch:{node.op}", node)
        for name, o in zip(node.outputs, outs):
            if name:
                self.vals[name] = Val(o, False)
                if name in self.preassigned:       # a concat slice was promised: copy into it
                    self._copy_into_slice(name)

    def _copy_into_slice(self, name: str) -> None:
        dst = self.preassigned[name]
        self.copy(self.vals[name].logical(), dst.logical(), f"to_slice({name})")
        self.vals[name] = dst

    # ------------------------------------------------------------------ conv
    def lower_FusedConv(self, node: Node):
        x_name, w_name = node.inputs[0], node.inputs[1]
        w = self.g.initializers[w_name]
        if w.ndim != 4 or any(d != 1 for d in node.attr("dilations", [1, 1])):
            return False
        if not self.is4d(x_name):
            return False
        group = node.attr("group", 1)
        if group != 1:
            return self._lower_depthwise(node, w, group)
        strides = node.attr("strides", [1, 1])
        if strides[0] != strides[1]:
            return False
        cout, cin, kh, kw = w.shape
        gated = self.pending_gate.pop(x_name, None)
        if gated is not None:
            x_name = gated[0]             # read the un-gated feature map; the gate goes into per-image weights
        x = self.as_nhwc(x_name)
        n, cx, h, wd = x.logical_shape
        n_o, c_o, ho, wo = self.info.shapes[node.outputs[0]]
        pads = interp._pads_2d(node, x.logical(), [kh, kw], strides, node.attr("dilations", [1, 1]))
        pad_t, pad_l = pads[0], pads[1]
        if stem_conv.eligible(cout, cin, kh, kw, strides[0], pads, node.attr("activation", "none"), self.dtype) \
                and not (len(node.inputs) > 3 and node.inputs[3]) and x.ld == 8 \
                and node.outputs[0] not in self.preassigned:
            y = self.out_nhwc(node.outputs[0], None)
            bias_np = np.asarray(self.g.initializers[node.inputs[2]], dtype=np.float32) \
                if len(node.inputs) > 2 and node.inputs[2] else None
            op = stem_conv.StemConv(x.t, np.asarray(w), y.t, n=n, h=h, w=wd, bias=bias_np,
                                    act=node.attr("activation", "none"), x_ld=x.ld, y_ld=y.ld,
                                    x_n_stride=x.n_stride, y_n_stride=y.n_stride, name=f"stem_conv:{node.name}")
            self.plan.add_native(op, node)
            op.launch()
            self.vals[node.outputs[0]] = y
            return None
        cin_phys = _round8(cin)
        key = (w_name, f"conv{cin_phys}")
        if key not in self.packed:
            wt = torch.from_numpy(np.ascontiguousarray(w)).float()
            if cin_phys != cin:
                wt = torch.nn.functional.pad(wt, (0, 0, 0, 0, 0, cin_phys - cin))
            self.packed[key] = pack_conv_weight(wt.to(self.device), self.dtype)
        wp = self.packed[key]
        bias = None
        if len(node.inputs) > 2 and node.inputs[2]:
            bias = self.const_f32(node.inputs[2]).float().contiguous()
        # an ESE gate ([N,C,1,1] multiplied into a feature map) is produced in fp32
        out_name = node.outputs[0]
        gate = ho == 1 and wo == 1 and all(c.op == "Mul" for c in self.cons.get(out_name, [])) \
            and len(self.cons.get(out_name, [])) > 0 and out_name not in self.preassigned
        y = self.out_nhwc(out_name, torch.float32 if gate else None)
        res = None
        if len(node.inputs) > 3 and node.inputs[3]:
            res = self.as_nhwc(node.inputs[3])
        if h == 1 and wd == 1 and kh == 1 and kw == 1 and res is None and n > 1:
            # a 1x1 map per image (squeeze-excite gates): the images become the rows of one GEMM
            # tile instead of one nearly empty 128-row tile each
            op = ConvGemm(x.t, wp, y.t, in_shape=(1, 1, n, cin_phys), out_hw=(1, n), cout=cout, bias=bias,
                          act=node.attr("activation", "none"), act_alpha=node.attr("act_alpha", 0.0),
                          act_beta=node.attr("act_beta", 0.0), x_ld=x.n_stride, y_ld=y.n_stride,
                          status=self.plan.status, name=f"conv:{node.name}")
            self.plan.add_native(op, node)
            op.launch()
            self.vals[out_name] = y
            return None
        wkw = {}
        if gated is not None:
            gate = self.get(gated[1]).t                        # fp32 [n, 1, 1, c]
            kp = wp.shape[1]
            wn = torch.zeros(n, cout, kp, dtype=self.dtype, device=self.device)
            sw = K.scale_weights(wp, gate.reshape(n, -1), wn, n=n, cout=cout, cin=cin)
            self.plan.add_native(sw, node)
            sw.launch()
            wp = wn
            wkw = dict(w_batched=2, w_ld=kp, w_n_stride=cout * kp)
        op = ConvGemm(x.t, wp, y.t, in_shape=(n, h, wd, cin_phys), out_hw=(ho, wo), cout=cout, kernel=(kh, kw),
                      stride=strides[0], pad=(pad_t, pad_l), bias=bias, **wkw,
                      residual=res.t if res is not None else None, res_mode=node.attr("res_mode", 0),
                      act=node.attr("activation", "none"), act_alpha=node.attr("act_alpha", 0.0),
                      act_beta=node.attr("act_beta", 0.0), x_ld=x.ld, y_ld=y.ld,
                      res_ld=res.ld if res is not None else None, status=self.plan.status,
                      x_n_stride=x.n_stride, y_n_stride=y.n_stride,
                      res_n_stride=res.n_stride if res is not None else 0, name=f"conv:{node.name}")
        self.plan.add_native(op, node)
        op.launch()
        self.vals[out_name] = y

    lower_Conv = lower_FusedConv

    def lower_ConvTranspose(self, node: Node):
        """Transposed convolution whose kernel equals its stride (the 2x2 / stride-2 up-sampling of segmentation and
        text-detection heads): every output pixel has exactly one contributing tap, so the layer is ``kh * kw`` 1x1
        GEMMs on the tensor cores, each writing the output pixels ``(kh * y + i, kw * x + j)`` through a strided
        output view, with bias and activation fused."""
        x_name, w_name = node.inputs[0], node.inputs[1]
        w = self.g.initializers.get(w_name)
        if w is None or w.ndim != 4 or not self.is4d(x_name) or node.attr("group", 1) != 1:
            return False
        cin, cout, kh, kw = w.shape
        strides = node.attr("strides", [1, 1])
        if list(strides) != [kh, kw] or any(p != 0 for p in node.attr("pads", [0, 0, 0, 0])) \
                or any(p != 0 for p in node.attr("output_padding", [0, 0])) \
                or any(d != 1 for d in node.attr("dilations", [1, 1])) \
                or node.attr("auto_pad", "NOTSET") not in ("NOTSET", ""):
            return False
        x = self.as_nhwc(x_name)
        n, cx, h, wd = x.logical_shape
        cin_phys = _round8(cin)
        bias = self.const_f32(node.inputs[2]).float().contiguous() if len(node.inputs) > 2 and node.inputs[2] else None
        y = self.out_nhwc(node.outputs[0])
        for i in range(kh):
            for j in range(kw):
                key = (w_name, f"deconv{cin_phys}_{i}_{j}")
                if key not in self.packed:
                    wt = torch.from_numpy(np.ascontiguousarray(w[:, :, i, j].T)).float().reshape(cout, cin, 1, 1)
                    if cin_phys != cin:
                        wt = torch.nn.functional.pad(wt, (0, 0, 0, 0, 0, cin_phys - cin))
                    self.packed[key] = pack_conv_weight(wt.to(self.device), self.dtype)
                yv = y.t[:, i::kh, j::kw, :]
                op = ConvGemm(x.t, self.packed[key], yv, in_shape=(n, h, wd, cin_phys), out_hw=(h, wd), cout=cout,
                              bias=bias, act=node.attr("activation", "none"), act_alpha=node.attr("act_alpha", 0.0),
                              act_beta=node.attr("act_beta", 0.0), x_ld=x.ld, y_ld=yv.stride(2), x_n_stride=x.n_stride,
                              y_n_stride=yv.stride(0), y_h_stride=yv.stride(1), status=self.plan.status,
                              name=f"deconv{i}{j}:{node.name}")
                self.plan.add_native(op, node)
                op.launch()
        self.vals[node.outputs[0]] = y

    def _lower_depthwise(self, node: Node, w: np.ndarray, group: int):
        """Depthwise convolution (one filter per channel): CUDA-core kernel, bias and activation fused."""
        cout, cpg, kh, kw = w.shape
        x = self.as_nhwc(node.inputs[0])
        n, cx, h, wd = x.logical_shape
        if cpg != 1 or group != cx or cout != cx or (len(node.inputs) > 3 and node.inputs[3]):
            return False
        strides = node.attr("strides", [1, 1])
        pads = interp._pads_2d(node, x.logical(), [kh, kw], strides, node.attr("dilations", [1, 1]))
        n_o, c_o, ho, wo = self.info.shapes[node.outputs[0]]
        cp = _round8(cx)
        key = (node.inputs[1], "dw")
        if key not in self.packed:
            wk = np.zeros((kh * kw, cp), np.float32)
            wk[:, :cx] = np.asarray(w, np.float32).reshape(cx, kh * kw).T
            self.packed[key] = torch.from_numpy(wk).to(self.device)
        bias = None
        if len(node.inputs) > 2 and node.inputs[2]:
            b = np.zeros(cp, np.float32)
            b[:cx] = np.asarray(self.g.initializers[node.inputs[2]], np.float32).reshape(-1)
            bias = torch.from_numpy(b).to(self.device)
        y = self.out_nhwc(node.outputs[0], None)
        if x.ld < cp or y.ld < cp:
            return False
        op = K.depthwise_conv(x.t, self.packed[key], bias, y.t, n=n, h=h, w_in=wd, c=cp, kernel=(kh, kw),
                              stride=(strides[0], strides[1]), pad=(pads[0], pads[1]), out_hw=(ho, wo),
                              act=node.attr("activation", "none"), act_alpha=node.attr("act_alpha", 0.0),
                              act_beta=node.attr("act_beta", 0.0), x_ld=x.ld, y_ld=y.ld, x_n_stride=x.n_stride,
                              y_n_stride=y.n_stride)
        op.keep.append(bias)
        self.plan.add_native(op, node)
        op.launch()
        self.vals[node.outputs[0]] = y
        return None

    # ------------------------------------------------------------------ gemm
    def lower_FusedGemm(self, node: Node):
        x_name, w_name = node.inputs[0], node.inputs[1]
        w = self.g.initializers[w_name]
        nout, kdim = w.shape
        xv = self.get(x_name)
        shp = xv.logical_shape
        if shp[-1] != kdim or kdim % 8 != 0:
            return False
        rows = int(np.prod(shp[:-1]))
        x2 = self.rows_view(x_name, rows, kdim)
        key = (w_name, "lin")
        if key not in self.packed:
            self.packed[key] = pack_linear_weight(torch.from_numpy(np.ascontiguousarray(w)).float().to(self.device),
                                                  self.dtype)
        bias = self.const_f32(node.inputs[2]).float().contiguous() if len(node.inputs) > 2 and node.inputs[2] else None
        out_shape = self.info.shapes[node.outputs[0]]
        is_output = node.outputs[0] in self.g.output_names()
        y = torch.zeros(rows, _round8(nout), dtype=torch.float32 if is_output else self.dtype, device=self.device)
        if self.fp8 and not (len(node.inputs) > 3 and node.inputs[3]) and kdim % 16 == 0 and nout >= 16 and kdim >= 64:
            self._lower_gemm_fp8(node, x_name, x2, w, w_name, bias, y, rows, kdim, nout)
            self.vals[node.outputs[0]] = Val(y[:, :nout].unflatten(0, out_shape[:-1]), False)
            return None
        res = None
        if len(node.inputs) > 3 and node.inputs[3]:
            res = self.rows_view(node.inputs[3], rows, nout)
        op = ConvGemm(x2, self.packed[key], y, in_shape=(1, 1, rows, kdim), out_hw=(1, rows), cout=nout, bias=bias,
                      residual=res, res_mode=node.attr("res_mode", 0), act=node.attr("activation", "none"),
                      act_alpha=node.attr("act_alpha", 0.0), act_beta=node.attr("act_beta", 0.0),
                      x_ld=x2.stride(0), y_ld=y.stride(0), res_ld=res.stride(0) if res is not None else None,
                      status=self.plan.status, name=f"gemm:{node.name}")
        self.plan.add_native(op, node)
        op.launch()
        self.vals[node.outputs[0]] = Val(y[:, :nout].unflatten(0, out_shape[:-1]), False)

    def _lower_gemm_fp8(self, node: Node, x_name: str, x2: torch.Tensor, w: np.ndarray, w_name: str, bias, y: torch.Tensor,
                        rows: int, kdim: int, nout: int) -> None:
        """Linear layer on e4m3 operands (``kind::f8f6f4`` MMAs, fp32 accumulation). Weights: one scale per output
        channel. Activations: the tensor's calibrated range when the graph or a calibration file gives one (static
        quantisation, the scale folds into the per-channel scale and the epilogue takes its straight path), else a
        per-row range found on the fly. The quantised copy of an activation is shared by all its consumers.
        The reference's int8 counterpart is TensorRT's calibrated engine build
        (fastdeploy/runtime/backends/tensorrt/trt_backend.cc:619-631)."""
        from ..ops.conv_gemm import FP8_MAX, pack_linear_weight_fp8
        key = (w_name, "lin8")
        if key not in self.packed:
            wq, sw = pack_linear_weight_fp8(torch.from_numpy(np.ascontiguousarray(w)).float().to(self.device))
            self.packed[key] = (wq, sw.float().contiguous())
        wq, sw = self.packed[key]
        if x_name not in self.q8:
            xq = torch.zeros(rows, kdim, dtype=torch.float8_e4m3fn, device=self.device)
            amax = self.act_scales.get(x_name)
            if amax is not None and amax > 0:
                s_act = float(amax) / FP8_MAX
                op = K.quantize_e4m3(x2, xq, rows=rows, c=kdim, scale=1.0 / s_act, x_ld=x2.stride(0), y_ld=kdim)
                self.q8[x_name] = (xq, None, s_act)
            else:
                sa = torch.zeros(rows, dtype=torch.float32, device=self.device)
                op = K.quantize_rows_e4m3_op(x2, xq, sa, rows=rows, c=kdim, x_ld=x2.stride(0), y_ld=kdim)
                self.q8[x_name] = (xq, sa, 1.0)
            self.plan.add_native(op, node)
            op.launch()
        xq, sa, s_act = self.q8[x_name]
        scale_b = sw if sa is not None else (sw * s_act).contiguous()
        op = ConvGemm(xq, wq, y, in_shape=(1, 1, rows, kdim), out_hw=(1, rows), cout=nout, bias=bias,
                      act=node.attr("activation", "none"), act_alpha=node.attr("act_alpha", 0.0),
                      act_beta=node.attr("act_beta", 0.0), x_ld=kdim, y_ld=y.stride(0), scale_a=sa, scale_b=scale_b,
                      status=self.plan.status, name=f"gemm_fp8:{node.name}")
        self.plan.add_native(op, node)
        op.launch()
        self.fp8_gemms += 1

    def rows_view(self, name: str, rows: int, cols: int) -> torch.Tensor:
        """``[rows, cols]`` 16-bit view with unit inner stride and 8-aligned row stride."""
        v = self.get(name)
        t = v.t
        if v.nhwc:
            n, h, w, c = t.shape
            if h == 1 and w == 1 and c == cols and t.dtype == self.dtype:
                return t.reshape(n, c) if t.is_contiguous() else t[:, 0, 0, :]
            t = v.logical()
        if t.dtype == self.dtype and t.stride(-1) == 1:
            try:
                t2 = t.view(rows, cols)
                if t2.stride(0) % 8 == 0 and t2.data_ptr() % 16 == 0:
                    return t2
            except RuntimeError:
                pass
        dst = torch.zeros(rows, cols, dtype=self.dtype, device=self.device)
        self.copy(t, dst.view(t.shape), f"to_rows({name})")
        return dst

    # ------------------------------------------------------------------ pooling / resize / elementwise
    def _lower_pool(self, node: Node, mode: str):
        x_name = node.inputs[0]
        if not self.is4d(x_name):
            return False
        k = node.attr("kernel_shape")
        if len(k) != 2 or node.attr("ceil_mode", 0):
            return False
        x = self.as_nhwc(x_name)
        n, c, h, w = x.logical_shape
        strides = node.attr("strides", [1, 1])
        pads = interp._pads_2d(node, x.logical(), k, strides)
        _, _, ho, wo = self.info.shapes[node.outputs[0]]
        y = self.out_nhwc(node.outputs[0])
        op = K.pool2d(x.t, y.t, n=n, h=h, w=w, c=_round8(c) if x.ld >= _round8(c) and y.ld >= _round8(c) else c,
                      kernel=(k[0], k[1]), stride=(strides[0], strides[1]), pad=(pads[0], pads[1]), out_hw=(ho, wo),
                      mode=mode, x_ld=x.ld, y_ld=y.ld, x_n_stride=x.n_stride, y_n_stride=y.n_stride,
                      count_include_pad=bool(node.attr("count_include_pad", 0)))
        self.plan.add_native(op, node)
        op.launch()
        self.vals[node.outputs[0]] = y

    def lower_MaxPool(self, node: Node):
        if len(node.outputs) > 1 and node.outputs[1]:
            return False
        if self._lower_spp(node):
            return None
        return self._lower_pool(node, "max")

    def _same_size_pool(self, node: Node):
        """Kernel size of a stride-1 max pool that keeps the spatial size (odd k, pad k // 2), else 0."""
        k = node.attr("kernel_shape")
        if node.op != "MaxPool" or len(k) != 2 or k[0] != k[1] or k[0] % 2 == 0 or node.attr("ceil_mode", 0):
            return 0
        if list(node.attr("strides", [1, 1])) != [1, 1] or (len(node.outputs) > 1 and node.outputs[1]):
            return 0
        if any(d != 1 for d in node.attr("dilations", [1, 1])):
            return 0
        pads = node.attr("pads", [0, 0, 0, 0])
        if node.attr("auto_pad", "NOTSET") not in ("NOTSET", "") or list(pads) != [k[0] // 2] * 4:
            return 0
        return k[0]

    def _lower_spp(self, node: Node) -> bool:
        """Spatial pyramid pooling: the stride-1 max pools that share this node's input become one launch."""
        x_name = node.inputs[0]
        if not self.is4d(x_name) or not self._same_size_pool(node):
            return False
        group = [c for c in self.cons.get(x_name, []) if self._same_size_pool(c) and id(c) not in self.fused_away]
        group.sort(key=self._same_size_pool)
        sizes = [self._same_size_pool(c) for c in group]
        n, c, h, w = self.info.shapes[x_name]
        if len(group) < 2 or len(group) > 3 or len(set(sizes)) != len(sizes) or not K.spp_fits(h, w, len(group)):
            return False
        x = self.as_nhwc(x_name)
        cp = _round8(c)
        outs = [self.out_nhwc(g.outputs[0]) for g in group]
        if x.ld < cp or any(o.ld < cp for o in outs):
            return False
        op = K.spp_maxpool(x.t, [o.t for o in outs], sizes, n=n, h=h, w=w, c=cp, x_ld=x.ld, x_n_stride=x.n_stride,
                           y_lds=[o.ld for o in outs], y_n_strides=[o.n_stride for o in outs])
        self.plan.add_native(op, node)
        op.launch()
        for g, o in zip(group, outs):
            self.vals[g.outputs[0]] = o
            if g is not node:
                self.fused_away.add(id(g))
        return True

    def lower_AveragePool(self, node: Node):
        return self._lower_pool(node, "avg")

    def lower_GlobalAveragePool(self, node: Node):
        x_name = node.inputs[0]
        if not self.is4d(x_name):
            return False
        x = self.as_nhwc(x_name)
        n, c, h, w = x.logical_shape
        cp = _round8(c) if x.ld >= _round8(c) else c
        splits = K.gap_splits_v2(h * w, n, cp)
        scratch = torch.empty(n * splits * cp, dtype=torch.float32, device=self.device)
        part = K.gap_partial(x.t, scratch, n=n, hw=h * w, c=cp, x_ld=x.ld, x_n_stride=x.n_stride, splits=splits)
        self.plan.add_native(part, node)
        part.launch()
        gates = self._ese_consumers(node, c, cp)
        if gates:
            # squeeze-excite: the pooled vector only feeds 1x1 convolutions whose results scale feature maps;
            # one kernel per gate finishes the mean, applies the 1x1 weights, the bias and the activation
            for conv, wt, bias, cout in gates:
                y = self.new_nhwc(n, 1, 1, cout, torch.float32)
                op = K.ese_gate(scratch, wt, bias, y.t, n=n, cin=cp, cout=cout, splits=splits, hw=h * w,
                                act=conv.attr("activation", "none"), alpha=conv.attr("act_alpha", 0.0),
                                beta=conv.attr("act_beta", 0.0), out_ld=y.t.stride(0))
                op.keep += [wt, bias]
                self.plan.add_native(op, conv)
                op.launch()
                self.fused_away.add(id(conv))
                self.vals[conv.outputs[0]] = y
            return None
        y = self.out_nhwc(node.outputs[0])
        fin = K.make_simple(K.K_GAP_FINALIZE, [scratch, y.t], [n, cp, splits, K.dtype_code(y.t.dtype), y.t.stride(0)],
                            [1.0 / (h * w)], name="gap_finalize")
        self.plan.add_native(fin, node)
        fin.launch()
        self.vals[node.outputs[0]] = y

    def _ese_consumers(self, node: Node, c: int, cp: int):
        """The 1x1 convolutions that turn this pooled vector into channel gates, if that is all it feeds."""
        out = node.outputs[0]
        cons = self.cons.get(out, [])
        if not cons or out in self.g.output_names() or out in self.preassigned:
            return None
        gates = [self._ese_gate_of(conv, out, c, cp) for conv in cons]
        return gates if all(g is not None for g in gates) else None

    def _ese_gate_of(self, conv: Node, out: str, c: int, cp: int):
        if conv.op not in ("FusedConv", "Conv") or conv.inputs[0] != out or conv.attr("group", 1) != 1:
            return None
        if len(conv.inputs) > 3 and conv.inputs[3]:
            return None
        w = self.g.initializers.get(conv.inputs[1])
        if w is None or w.ndim != 4 or w.shape[2:] != (1, 1) or w.shape[1] != c:
            return None
        gate_out = conv.outputs[0]
        users = self.cons.get(gate_out, [])
        if not users or any(u.op != "Mul" for u in users) or gate_out in self.preassigned \
                or gate_out in self.g.output_names() or conv.attr("activation", "none") == "gelu":
            return None
        cout = w.shape[0]
        if cout % 8 != 0:
            return None
        key = (conv.inputs[1], f"gate{cp}")
        if key not in self.packed:
            wt = torch.zeros(cout, cp, dtype=self.dtype, device=self.device)
            wt[:, :c] = torch.from_numpy(np.ascontiguousarray(w.reshape(cout, c))).to(self.device).to(self.dtype)
            self.packed[key] = wt
        bias = self.const_f32(conv.inputs[2]).float().contiguous() if len(conv.inputs) > 2 and conv.inputs[2] else None
        return conv, self.packed[key], bias, cout

    def lower_Resize(self, node: Node):
        x_name = node.inputs[0]
        if not self.is4d(x_name) or node.attr("mode", "nearest") != "nearest":
            return False
        n, c, h, w = self.info.shapes[x_name]
        _, _, ho, wo = self.info.shapes[node.outputs[0]]
        if ho % h or wo % w:
            return False
        ctm = node.attr("coordinate_transformation_mode", "half_pixel")
        if not (ctm == "asymmetric" or (ho // h in (1, 2) and wo // w in (1, 2))):
            return False
        x = self.as_nhwc(x_name)
        y = self.out_nhwc(node.outputs[0])
        cc = _round8(c) if x.ld >= _round8(c) and y.ld >= _round8(c) else c
        op = K.upsample_nearest(x.t, y.t, n=n, h=h, w=w, c=cc, factor=(ho // h, wo // w), x_ld=x.ld, y_ld=y.ld,
                                x_n_stride=x.n_stride, y_n_stride=y.n_stride)
        self.plan.add_native(op, node)
        op.launch()
        self.vals[node.outputs[0]] = y

    def lower_Concat(self, node: Node):
        out = node.outputs[0]
        if out not in self.preassigned or not self.is4d(out):
            return False
        dst = self.preassigned[out]
        off = 0
        for i in node.inputs:
            ci = self.info.shapes[i][1]
            v = self.get(i)
            sl = dst.t[..., off:off + ci]
            same = v.nhwc and v.t.data_ptr() == sl.data_ptr() and v.t.stride() == sl.stride()
            if not same:
                self.copy(v.logical(), sl.permute(0, 3, 1, 2), f"concat_copy({i})", node)
            off += ci
        self.vals[out] = dst

    def _lower_binary(self, node: Node, opname: str):
        a_name, b_name = node.inputs
        if not (self.is4d(a_name) and self.is4d(b_name)):
            return False
        if a_name in self.g.initializers or b_name in self.g.initializers:
            return False
        sa, sb = self.info.shapes[a_name], self.info.shapes[b_name]
        if sa != sb:
            # feature map times per-image channel gate [N,C,1,1]
            if opname == "mul" and sb[2:] == [1, 1] and sa[:2] == sb[:2]:
                return self._lower_scale(node, a_name, b_name)
            if opname == "mul" and sa[2:] == [1, 1] and sa[:2] == sb[:2]:
                return self._lower_scale(node, b_name, a_name)
            return False
        a, b = self.as_nhwc(a_name), self.as_nhwc(b_name)
        n, c, h, w = a.logical_shape
        if a.n_stride != h * w * a.ld or b.n_stride != h * w * b.ld:
            return False
        y = self.out_nhwc(node.outputs[0])
        if y.n_stride != h * w * y.ld:
            return False
        op = K.binary(a.t, b.t, y.t, rows=n * h * w, c=_round8(c) if min(a.ld, b.ld, y.ld) >= _round8(c) else c,
                      op=opname, a_ld=a.ld, b_ld=b.ld, y_ld=y.ld)
        self.plan.add_native(op, node)
        op.launch()
        self.vals[node.outputs[0]] = y

    def _gate_folds_into_consumer(self, node: Node, x_name: str, s_name: str) -> bool:
        """True when ``x * gate`` only feeds a 1x1 convolution and scaling that convolution's weights per image is
        cheaper than writing and re-reading the scaled map (pixels per image well above the output channels)."""
        out = node.outputs[0]
        cons = self.cons.get(out, [])
        if len(cons) != 1 or out in self.g.output_names() or out in self.preassigned:
            return False
        conv = cons[0]
        if conv.op not in ("FusedConv", "Conv") or conv.inputs[0] != out or conv.attr("group", 1) != 1:
            return False
        if len(conv.inputs) > 3 and conv.inputs[3] == out:
            return False
        w = self.g.initializers.get(conv.inputs[1])
        if w is None or w.ndim != 4 or tuple(w.shape[2:]) != (1, 1):
            return False
        if list(conv.attr("strides", [1, 1])) != [1, 1] or any(p != 0 for p in conv.attr("pads", [0, 0, 0, 0])) \
                or conv.attr("auto_pad", "NOTSET") not in ("NOTSET", ""):
            return False
        n, c, h, wd = self.info.shapes[x_name]
        s = self.vals.get(s_name)
        if s is None or not s.nhwc or s.t.dtype != torch.float32 or c % 8 != 0 or w.shape[1] != c:
            return False
        if s.t.shape[1:3] != (1, 1) or s.t.stride(3) != 1:
            return False
        return h * wd >= 2 * w.shape[0] and n > 1 and stem_conv is not None

    def _lower_scale(self, node: Node, x_name: str, s_name: str):
        if self._gate_folds_into_consumer(node, x_name, s_name):
            self.pending_gate[node.outputs[0]] = (x_name, s_name)
            return None
        x = self.as_nhwc(x_name)
        s = self.get(s_name)
        n, c, h, w = x.logical_shape
        if not (s.nhwc and s.t.dtype == torch.float32 and s.t.stride(0) == _round8(c) and _round8(c) == c):
            sv = torch.zeros(n, c, dtype=torch.float32, device=self.device)
            self.copy(s.logical(), sv.view(n, c, 1, 1), f"gate_to_f32({s_name})", node)
            s_t = sv
        else:
            s_t = s.t
        y = self.out_nhwc(node.outputs[0])
        op = K.scale_channels(x.t, s_t, y.t, n=n, hw=h * w, c=c, x_ld=x.ld, y_ld=y.ld, x_n_stride=x.n_stride,
                              y_n_stride=y.n_stride) if c % 8 == 0 else None
        if op is None:
            return False
        self.plan.add_native(op, node)
        op.launch()
        self.vals[node.outputs[0]] = y

    def lower_Add(self, node: Node):
        return self._lower_binary(node, "add")

    def lower_Mul(self, node: Node):
        return self._lower_binary(node, "mul")

    def lower_Sub(self, node: Node):
        return self._lower_binary(node, "sub")

    def _lower_unary(self, node: Node, act: str, alpha: float = 0.0, beta: float = 0.0):
        x_name = node.inputs[0]
        if not self.is4d(x_name):
            return False
        x = self.as_nhwc(x_name)
        n, c, h, w = x.logical_shape
        y = self.out_nhwc(node.outputs[0])
        if x.n_stride != h * w * x.ld or y.n_stride != h * w * y.ld:
            return False
        op = K.unary(x.t, y.t, rows=n * h * w, c=_round8(c) if min(x.ld, y.ld) >= _round8(c) else c, act=act,
                     x_ld=x.ld, y_ld=y.ld, alpha=alpha, beta=beta)
        self.plan.add_native(op, node)
        op.launch()
        self.vals[node.outputs[0]] = y

    def lower_Relu(self, node): return self._lower_unary(node, "relu")
    def lower_Silu(self, node): return self._lower_unary(node, "silu")
    def lower_Sigmoid(self, node): return self._lower_unary(node, "sigmoid")
    def lower_HardSwish(self, node): return self._lower_unary(node, "hard_swish")
    def lower_Tanh(self, node): return self._lower_unary(node, "tanh")

    def lower_HardSigmoid(self, node):
        return self._lower_unary(node, "hard_sigmoid", node.attr("alpha", 0.2), node.attr("beta", 0.5))

    def lower_LeakyRelu(self, node):
        return self._lower_unary(node, "leaky_relu", node.attr("alpha", 0.01))

    def lower_Flatten(self, node: Node):
        v = self.get(node.inputs[0])
        if v.nhwc and v.t.shape[1] == 1 and v.t.shape[2] == 1 and node.attr("axis", 1) == 1:
            self.vals[node.outputs[0]] = Val(v.t[:, 0, 0, :], False)
            return True
        return False

    # ------------------------------------------------------------------ detection post-processing
    def lower_MultiClassNMS(self, node: Node):
        top_k, keep = node.attr("nms_top_k", 1000), node.attr("keep_top_k", 100)
        if node.attr("nms_eta", 1.0) < 1.0 or top_k == 0 or (min(keep, top_k) if keep > 0 and top_k > 0 else max(keep, top_k)) \
                > MulticlassNMS.MAX_KEEP or (keep <= 0 and top_k < 0):
            return False
        boxes = self.as_torch(node.inputs[0])
        scores = self.as_torch(node.inputs[1])
        n, m, _ = boxes.shape
        if boxes.dtype == torch.float32 and boxes.is_contiguous():
            bx = boxes
        else:
            bx = torch.zeros(n, m, 4, dtype=torch.float32, device=self.device)
            self.copy(boxes, bx, "nms_boxes_f32", node)
        if not scores.is_contiguous():
            sc = torch.zeros(scores.shape, dtype=scores.dtype, device=self.device)
            self.copy(scores, sc, "nms_scores", node)
            scores = sc
        self._emit_nms(node, bx, scores, class_major=True)

    def _emit_nms(self, node: Node, boxes: torch.Tensor, scores: torch.Tensor, class_major: bool) -> None:
        nms = MulticlassNMS(boxes, scores, class_major=class_major,
                            score_threshold=node.attr("score_threshold", 0.01),
                            nms_threshold=node.attr("nms_threshold", 0.5), nms_top_k=node.attr("nms_top_k", 1000),
                            keep_top_k=node.attr("keep_top_k", 100), normalized=bool(node.attr("normalized", 1)),
                            background_label=node.attr("background_label", -1))
        self.plan.add_native(nms.op, node, launches=nms.launches)
        nms.launch()
        self.plan.extra.setdefault("nms", []).append(nms)
        n = boxes.shape[0]
        cap = nms.out.shape[1]
        # padded outputs; the runtime compacts them with the per-image counts after the D2H copy
        self.vals[node.outputs[0]] = Val(nms.out.view(n * cap, 6), False)
        if len(node.outputs) > 1 and node.outputs[1]:
            self.vals[node.outputs[1]] = Val(nms.out_index.view(n * cap, 1), False)
        if len(node.outputs) > 2 and node.outputs[2]:
            self.vals[node.outputs[2]] = Val(nms.out_num, False)
        self.plan.extra.setdefault("padded_nms_outputs", {})[node.outputs[0]] = (node.outputs[2] if len(node.outputs) > 2 else None, cap)
        if len(node.outputs) > 1 and node.outputs[1]:
            self.plan.extra["padded_nms_outputs"][node.outputs[1]] = (node.outputs[2] if len(node.outputs) > 2 else None, cap)

    def plan_PPYOLOEPost(self, node: Node) -> None:
        """Allocates the anchor-major score / regression buffers and hands their per-level row
        ranges to the producing convolutions."""
        nl = node.attr("num_levels")
        gh, gw = node.attr("grid_h"), node.attr("grid_w")
        a_total = sum(h * w for h, w in zip(gh, gw))
        n, c = self.info.shapes[node.inputs[0]][:2]
        rc = self.info.shapes[node.inputs[nl]][1]
        # class scores stay in the network's 16-bit type when that is fp16 (11 significant bits, what an fp16 engine
        # yields); bf16 would leave 8 bits, too coarse to rank detections, so bf16 plans keep fp32 scores
        score_dt = torch.float16 if self.dtype == torch.float16 else torch.float32
        scores = torch.zeros(n, a_total, _round8(c), dtype=score_dt, device=self.device)
        regs = torch.zeros(n, a_total, _round8(rc), dtype=self.dtype, device=self.device)
        off = 0
        for i in range(nl):
            h, w = gh[i], gw[i]
            for name, buf, ch in ((node.inputs[i], scores, c), (node.inputs[nl + i], regs, rc)):
                p = self.prod.get(name)
                if p is not None and p.op in ("FusedConv", "Conv") and len(self.cons.get(name, [])) == 1 \
                        and name not in self.preassigned:
                    view = buf[:, off:off + h * w, :ch].unflatten(1, (h, w))
                    self.preassigned[name] = Val(view, True)
            off += h * w
        self.plan.extra[("ppyoloe_post", node.name)] = (scores, regs)

    def lower_PPYOLOEPost(self, node: Node):
        nl = node.attr("num_levels")
        gh, gw = node.attr("grid_h"), node.attr("grid_w")
        scores, regs = self.plan.extra[("ppyoloe_post", node.name)]
        n, a_total = scores.shape[:2]
        c = self.info.shapes[node.inputs[0]][1]
        rc = self.info.shapes[node.inputs[nl]][1]
        off = 0
        levels = []
        for i in range(nl):
            h, w = gh[i], gw[i]
            for name, buf, ch in ((node.inputs[i], scores, c), (node.inputs[nl + i], regs, rc)):
                v = self.get(name)
                view = buf[:, off:off + h * w, :ch].unflatten(1, (h, w))
                if not (v.nhwc and v.t.data_ptr() == view.data_ptr()):
                    self.copy(v.logical(), view.permute(0, 3, 1, 2), "ppyoloe_gather", node)
            levels.append((off, w, node.attr("strides")[i]))
            off += h * w
        sf = self.get(node.inputs[2 * nl]).t
        boxes = torch.zeros(n, a_total, 4, dtype=torch.float32, device=self.device)
        op = K.dfl_decode(regs, boxes, sf, n=n, anchors=a_total, bins=node.attr("bins"), levels=levels,
                          offset=node.attr("offset", 0.5), reg_ld=regs.shape[2])
        self.plan.add_native(op, node)
        op.launch()
        self._emit_nms(node, boxes, scores[:, :, :c], class_major=False)


def graph_fingerprint(graph: Graph, input_shapes: Dict[str, Sequence[int]], dtype, opt_level: int) -> str:
    """Cache key of an optimised graph: structure, attributes, shapes, and for every weight its shape,
    dtype and a sample of its bytes (hashing 600 MB of weights on every start would cost more than the passes)."""
    import hashlib
    h = hashlib.sha256()
    h.update(repr((sorted((k, tuple(v)) for k, v in input_shapes.items()), str(dtype), opt_level)).encode())
    for n in graph.nodes:
        h.update(repr((n.op, n.inputs, n.outputs, sorted((k, repr(v)[:200]) for k, v in n.attrs.items()))).encode())
    for name in sorted(graph.initializers):
        a = np.ascontiguousarray(graph.initializers[name])
        raw = a.view(np.uint8).reshape(-1)
        h.update(repr((name, a.shape, str(a.dtype))).encode())
        h.update(raw[:256].tobytes())
        h.update(raw[-256:].tobytes())
        if raw.size > 4096:
            h.update(raw[::max(1, raw.size // 1024)].tobytes())
    return h.hexdigest()[:32]


def optimize_cached(graph: Graph, input_shapes, input_values, opt_level: int, dtype, cache_dir: str) -> Graph:
    """``passes.optimize`` behind an on-disk cache (the counterpart of the reference's serialized TensorRT engine,
    fastdeploy/runtime/backends/tensorrt/trt_backend.cc:240-300 ``serialize_file``): the optimised graph, fused
    ops included, is stored in this package's ONNX writer format under ``cache_dir`` and reloaded on the next
    start instead of re-running constant folding, BN / RepVGG folding and the pattern matchers."""
    if not cache_dir or input_values:
        return passes.optimize(graph, input_shapes, input_values, level=opt_level)
    import os
    from ..importer.onnx_format import load_onnx, save_onnx
    path = os.path.join(cache_dir, graph_fingerprint(graph, input_shapes, dtype, opt_level) + ".fdbgraph")
    if os.path.exists(path):
        try:
            with open(path, "rb") as f:
                g = load_onnx(f.read())
            log.info(f"optimised graph loaded from {path}")
            return g
        except Exception as e:      # a damaged cache entry is rebuilt, never fatal
            log.warning(f"ignoring unreadable plan cache entry {path}: {e}")
    g = passes.optimize(graph, input_shapes, input_values, level=opt_level)
    try:
        os.makedirs(cache_dir, exist_ok=True)
        tmp = path + f".tmp{os.getpid()}"
        with open(tmp, "wb") as f:
            f.write(save_onnx(g))
        os.replace(tmp, path)
    except OSError as e:
        log.warning(f"could not write plan cache entry {path}: {e}")
    return g


def build_plan(graph: Graph, input_shapes: Dict[str, Sequence[int]], device, dtype=torch.float16,
               input_values: Optional[Dict[str, np.ndarray]] = None, opt_level: int = 2, cache_dir: str = "",
               fp8: bool = False, act_scales: Optional[Dict[str, float]] = None,
               reuse_buffers: Optional[bool] = None) -> Plan:
    """Optimises ``graph`` for the given shapes and lowers it to a plan on ``device``. ``fp8`` runs the linear layers on
    e4m3 operands; ``act_scales`` (tensor name -> calibrated absolute maximum) adds to the ranges the graph carries."""
    device = torch.device(device)
    if any(n.op in ("Loop", "If", "Scan") for n in graph.nodes):
        raise NotImplementedError("graphs with control flow (Loop / If / Scan) have no static launch plan: run them on the CPU "
                                  "path (RuntimeOption.use_cpu())")
    with torch.cuda.device(device):
        g = optimize_cached(graph, input_shapes, input_values, opt_level, dtype, cache_dir)
        if reuse_buffers is None:
            reuse_buffers = os.environ.get("FDX_REUSE_BUFFERS", "1") not in ("0", "false")
        low = Lowering(g, input_shapes, device, dtype, input_values, fp8=fp8, act_scales=act_scales,
                       reuse_buffers=reuse_buffers)
        for node in g.nodes:
            if node.op == "PPYOLOEPost":
                low.plan_PPYOLOEPost(node)
        plan = low.build()
        plan.extra["graph"] = g
        plan.extra["fp8_gemms"] = low.fp8_gemms
    return plan


# ---------------------------------------------------------------------- transformer lowering
def _rows_of(shape: Sequence[int]) -> int:
    return int(np.prod(shape[:-1])) if len(shape) > 1 else 1


def _lower_LayerNormalization(self: Lowering, node: Node):
    from ..ops import transformer as T
    x_name = node.inputs[0]
    shp = self.info.shapes[x_name]
    axis = node.attr("axis", -1)
    if axis not in (-1, len(shp) - 1) or shp[-1] % 8 != 0:
        return False
    c, rows = shp[-1], _rows_of(shp)
    x2 = self.rows_view(x_name, rows, c)
    gamma = self.const_f32(node.inputs[1]).float().contiguous() if len(node.inputs) > 1 and node.inputs[1] else None
    beta = self.const_f32(node.inputs[2]).float().contiguous() if len(node.inputs) > 2 and node.inputs[2] else None
    y = torch.zeros(rows, c, dtype=self.dtype, device=self.device)
    op = T.layernorm(x2, y, gamma, beta, rows=rows, c=c, eps=node.attr("epsilon", 1e-5), x_ld=x2.stride(0), y_ld=c)
    self.plan.add_native(op, node)
    op.launch()
    self.vals[node.outputs[0]] = Val(y.unflatten(0, shp[:-1]), False)


def _lower_EmbedLayerNorm(self: Lowering, node: Node):
    from ..ops import transformer as T
    k = node.attr("num_tables")
    ids_names, tab_names = node.inputs[:k], node.inputs[k:2 * k]
    gamma, beta = self.const_f32(node.inputs[2 * k]), self.const_f32(node.inputs[2 * k + 1])
    out_shape = self.info.shapes[node.outputs[0]]
    c, rows = out_shape[-1], _rows_of(out_shape)
    if c % 8 != 0 or c > 1536 or k > 4:
        return False
    seq = out_shape[-2]
    ids: List[Optional[torch.Tensor]] = []
    for nm in ids_names:
        if nm in self.g.initializers:
            arr = self.g.initializers[nm].reshape(-1)
            # constant position ids 0..S-1 (broadcast over the batch) become the implicit index
            if arr.size == seq and np.array_equal(arr, np.arange(seq)):
                ids.append(None)
                continue
            full = np.broadcast_to(self.g.initializers[nm], out_shape[:-1]).reshape(-1)
            ids.append(torch.from_numpy(np.array(full, dtype=np.int64)).to(self.device))
            continue
        v = self.get(nm).t
        if v.dtype != torch.int64 or not v.is_contiguous() or v.numel() != rows:
            buf = torch.zeros(rows, dtype=torch.int64, device=self.device)
            self.copy(v, buf.view(out_shape[:-1]), f"ids_i64({nm})", node)
            v = buf
        ids.append(v.reshape(-1))
    tabs = []
    for nm in tab_names:
        key = (nm, "emb")
        if key not in self.packed:
            self.packed[key] = self.const_f32(nm).to(self.dtype).contiguous()
        tabs.append(self.packed[key])
    y = torch.zeros(rows, c, dtype=self.dtype, device=self.device)
    op = T.embed_layernorm(ids, tabs, y, gamma, beta, rows=rows, c=c, seq=seq, eps=node.attr("epsilon", 1e-5))
    self.plan.add_native(op, node)
    op.launch()
    self.vals[node.outputs[0]] = Val(y.unflatten(0, out_shape[:-1]), False)


def _lower_Attention(self: Lowering, node: Node):
    from ..ops.transformer import Attention
    shp = self.info.shapes[node.inputs[0]]
    if len(shp) != 3:
        return False
    b, s, hd = shp
    heads = node.attr("num_heads")
    d = hd // heads
    if s > 1024:
        return False
    dp = _round8(d)

    def view3(name):
        v = self.get(name).t
        if d != dp:
            # head size not a multiple of 8 (SVTR: 120 / 8 = 15): zero-padded per head; zeros change neither the
            # scores nor the first d output columns
            buf = torch.zeros(b, s, heads * dp, dtype=self.dtype, device=self.device)
            self.copy(self.as_torch(name).unflatten(2, (heads, d)), buf.view(b, s, heads, dp)[..., :d],
                      f"pad_heads({name})", node)
            return buf
        if v.dtype == self.dtype and v.dim() == 3 and v.stride(2) == 1 and v.stride(1) % 8 == 0 \
                and v.data_ptr() % 16 == 0:
            return v
        return self.rows_view(name, b * s, hd).unflatten(0, (b, s))
    q, k, v = view3(node.inputs[0]), view3(node.inputs[1]), view3(node.inputs[2])
    mask = None
    if len(node.inputs) > 3 and node.inputs[3]:
        mshape = self.info.shapes[node.inputs[3]]
        if int(np.prod(mshape)) not in (b * s, b * s * s):
            return False
        mv = self.as_torch(node.inputs[3])
        if mv.dtype == torch.float32 and mv.is_contiguous():
            mask = mv
        else:
            mask = torch.zeros(mshape, dtype=torch.float32, device=self.device)
            self.copy(mv, mask, "attn_mask_f32", node)
    out = torch.zeros(b, s, heads * dp, dtype=self.dtype, device=self.device)
    att = Attention(q, k, v, out, heads=heads, scale=node.attr("scale", 1.0 / math.sqrt(d)), mask=mask,
                    status=self.plan.status)
    for op in att.ops:
        self.plan.add_native(op, node)
        op.launch()
    self.plan.extra.setdefault("attention", []).append(att)
    if d != dp:
        trimmed = torch.zeros(b, s, hd, dtype=self.dtype, device=self.device)
        self.copy(out.view(b, s, heads, dp)[..., :d], trimmed.view(b, s, heads, d), "trim_heads", node)
        out = trimmed
    self.vals[node.outputs[0]] = Val(out, False)


def _lower_PackedAttention(self: Lowering, node: Node):
    """Padding-free self-attention (ir/packing.py): q / k / v are ``[1, T, H*D]``; the starts and lengths are int32
    plan inputs read by the kernel at every launch."""
    from ..ops.transformer import PackedAttention, fused_attention_fits
    shp = self.info.shapes[node.inputs[0]]
    heads = node.attr("num_heads")
    max_len = int(node.attr("max_len", 512))
    if len(shp) != 3 or shp[0] != 1:
        return False
    t, hd = shp[1], shp[2]
    d = hd // heads
    if t % 8 or not fused_attention_fits(max_len, max_len, d):
        raise ValueError(f"packed attention: {t} rows (multiple of 8), head dim {d} (multiple of 16), "
                         f"longest sequence {max_len} (<= 512) do not fit the fused kernel")
    q, k, v = (self.rows_view(nm, t, hd) for nm in node.inputs[:3])
    start, lens = self.get(node.inputs[3]).t, self.get(node.inputs[4]).t
    if start.dtype != torch.int32 or lens.dtype != torch.int32:
        raise ValueError("packed attention: seq_start and seq_len must be int32 plan inputs")
    out = torch.zeros(t, hd, dtype=self.dtype, device=self.device)
    att = PackedAttention(q, k, v, out, heads=heads, scale=node.attr("scale", 1.0 / math.sqrt(d)), max_len=max_len,
                          seq_start=start.reshape(-1), seq_len=lens.reshape(-1), status=self.plan.status)
    for op in att.ops:
        self.plan.add_native(op, node)
        op.launch()
    self.plan.extra.setdefault("attention", []).append(att)
    self.vals[node.outputs[0]] = Val(out.view(1, t, hd), False)


def _lower_Gelu(self: Lowering, node: Node):
    if node.attr("approximate", "none") == "tanh":
        return False
    shp = self.info.shapes[node.inputs[0]]
    if shp[-1] % 8 != 0:
        return False
    rows, c = _rows_of(shp), shp[-1]
    x2 = self.rows_view(node.inputs[0], rows, c)
    y = torch.zeros(rows, c, dtype=self.dtype, device=self.device)
    op = K.unary(x2, y, rows=rows, c=c, act="gelu", x_ld=x2.stride(0), y_ld=c)
    self.plan.add_native(op, node)
    op.launch()
    self.vals[node.outputs[0]] = Val(y.unflatten(0, shp[:-1]), False)


Lowering.lower_LayerNormalization = _lower_LayerNormalization
Lowering.lower_EmbedLayerNorm = _lower_EmbedLayerNorm
Lowering.lower_Attention = _lower_Attention
Lowering.lower_PackedAttention = _lower_PackedAttention
Lowering.lower_Gelu = _lower_Gelu
