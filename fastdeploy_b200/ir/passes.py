"""Graph rewrites applied before lowering: constant folding, BatchNorm / bias folding,
RepVGG branch folding, activation and residual fusion into convolutions and GEMMs,
LayerNorm / GELU / attention recognition.

They take over the jobs of the optimisers inside the reference's vendor engines and of
the paddle2onnx graph passes (paddle2onnx/optimizer/fuse_paddle_conv_bias.h,
fuse_constant_reshape.h, ...). Every pass keeps the graph executable by the reference
interpreter, which is how the tests prove pass-on == pass-off.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np
import torch

from . import interp
from .graph import Graph, Node
from .shape_infer import ShapeInfo, infer_shapes

ACT_OPS = {"Relu": "relu", "Silu": "silu", "Swish": "silu", "Sigmoid": "sigmoid", "HardSwish": "hard_swish",
           "Tanh": "tanh", "Gelu": "gelu"}


def _single_consumer(cons: Dict[str, List[Node]], graph: Graph, name: str) -> Optional[Node]:
    c = cons.get(name, [])
    if len(c) == 1 and name not in graph.output_names():
        return c[0]
    return None


def _remove(graph: Graph, dead: Sequence[Node]) -> None:
    ids = {id(n) for n in dead}
    graph.nodes = [n for n in graph.nodes if id(n) not in ids]


def _replace_uses(graph: Graph, old: str, new: str) -> None:
    for n in graph.nodes:
        n.inputs = [new if i == old else i for i in n.inputs]
    for o in graph.outputs:
        if o.name == old:
            o.name = new


def _act_of(node: Node, graph: Graph):
    """(activation, alpha, beta) if ``node`` is a fusable unary activation."""
    if node.op in ACT_OPS and not (node.op == "Gelu" and node.attr("approximate", "none") == "tanh"):
        return ACT_OPS[node.op], 0.0, 0.0
    if node.op == "LeakyRelu":
        return "leaky_relu", float(node.attr("alpha", 0.01)), 0.0
    if node.op == "HardSigmoid":
        return "hard_sigmoid", float(node.attr("alpha", 0.2)), float(node.attr("beta", 0.5))
    if node.op == "Clip":
        lo = graph.initializers.get(node.inputs[1]) if len(node.inputs) > 1 and node.inputs[1] else node.attr("min")
        hi = graph.initializers.get(node.inputs[2]) if len(node.inputs) > 2 and node.inputs[2] else node.attr("max")
        if lo is not None and hi is not None and float(np.asarray(lo)) == 0.0 and float(np.asarray(hi)) == 6.0:
            return "relu6", 0.0, 0.0
    return None


# --------------------------------------------------------------------------- constants
def fold_constants(graph: Graph, info: Optional[ShapeInfo] = None) -> int:
    """Evaluates nodes whose inputs are all constants; with ``info`` also replaces values
    that shape inference proved constant (shape arithmetic)."""
    changed = 0
    keep: List[Node] = []
    for node in graph.nodes:
        if info is not None and all(o in info.values for o in node.outputs if o) and node.op not in ("Constant",):
            small = all(info.values[o].size <= 4096 for o in node.outputs if o)
            dyn_free = node.op in ("Shape", "Size") or all((i in graph.initializers or i == "") for i in node.inputs)
            if small and dyn_free:
                for o in node.outputs:
                    if o:
                        graph.initializers[o] = np.ascontiguousarray(info.values[o])
                changed += 1
                continue
        big_gather = node.op == "Gather" and node.inputs[0] in graph.initializers and \
            graph.initializers[node.inputs[0]].ndim == 2 and node.inputs[1] in graph.initializers and \
            graph.initializers[node.inputs[1]].size * graph.initializers[node.inputs[0]].shape[1] > 1024
        if node.inputs and all((i in graph.initializers or i == "") for i in node.inputs) and node.op in interp._OPS \
                and node.op not in ("MultiClassNMS",) and not big_gather:
            args = []
            for i in node.inputs:
                if i == "":
                    args.append(None)
                else:
                    t = torch.from_numpy(np.ascontiguousarray(graph.initializers[i]))
                    args.append(t.float() if t.dtype in (torch.float16, torch.float64) else t)
            while args and args[-1] is None:
                args.pop()
            node.attrs.setdefault("_opset", graph.opset)
            with torch.no_grad():
                res = interp._OPS[node.op](node, *args)
            res = res if isinstance(res, tuple) else (res,)
            for o, r in zip(node.outputs, res):
                if o:
                    graph.initializers[o] = np.ascontiguousarray(r.numpy())
            changed += 1
            continue
        keep.append(node)
    graph.nodes = keep
    return changed


def eliminate_identity(graph: Graph) -> int:
    changed = 0
    for node in list(graph.nodes):
        if node.op in ("Identity", "Dropout") and node.inputs[0] not in graph.initializers:
            if node.outputs[0] in graph.output_names() and node.inputs[0] in graph.input_names():
                continue
            if node.outputs[0] in graph.output_names():
                # keep the public output name: rename the producer's output instead
                prod = graph.producers().get(node.inputs[0])
                if prod is None or len(graph.consumers().get(node.inputs[0], [])) != 1:
                    continue
                prod.outputs = [node.outputs[0] if o == node.inputs[0] else o for o in prod.outputs]
            else:
                _replace_uses(graph, node.outputs[0], node.inputs[0])
            _remove(graph, [node])
            changed += 1
    return changed


# --------------------------------------------------------------------------- quantised models
ACT_SCALES_KEY = "fdb_act_scales"


def get_act_scales(graph: Graph) -> Dict[str, float]:
    """Static activation ranges recorded by :func:`fold_qdq` (or loaded from a calibration file): tensor name ->
    absolute maximum the tensor was calibrated to. Kept as a JSON string so that it survives the on-disk graph cache."""
    import json
    raw = graph.metadata.get(ACT_SCALES_KEY, "")
    return {k: float(v) for k, v in json.loads(raw).items()} if raw else {}


def set_act_scales(graph: Graph, scales: Dict[str, float]) -> None:
    import json
    graph.metadata[ACT_SCALES_KEY] = json.dumps({k: float(v) for k, v in scales.items()})


_QLINEAR_UNARY = {"QLinearGlobalAveragePool": "GlobalAveragePool", "QLinearAveragePool": "AveragePool",
                  "QLinearLeakyRelu": "LeakyRelu", "QLinearSigmoid": "Sigmoid", "QLinearSoftmax": "Softmax"}
_QLINEAR_BINARY = {"QLinearAdd": "Add", "QLinearMul": "Mul"}


def expand_qlinear(graph: Graph) -> int:
    """Integer operators of quantised ONNX models (``QLinearConv`` / ``QLinearMatMul`` of the standard set and the
    ``QLinear*`` operators ONNX Runtime's quantiser writes in the ``com.microsoft`` domain) rewritten as
    ``DequantizeLinear -> float operator -> QuantizeLinear``. Constant weights become float weights here, the int32
    bias is scaled by ``x_scale * w_scale``; the ``Quantize -> Dequantize`` pairs between consecutive layers are then
    removed by :func:`fold_qdq`, which leaves a float graph with a calibrated range per activation - the form the
    e4m3 path takes. The reference runs such models through ONNX Runtime's int8 kernels
    (fastdeploy/runtime/backends/ort/ort_backend.cc:391)."""
    changed = 0
    for node in list(graph.nodes):
        op_name = node.op
        if op_name not in ("QLinearConv", "QLinearMatMul", "QLinearConcat") and op_name not in _QLINEAR_UNARY \
                and op_name not in _QLINEAR_BINARY:
            continue
        new_nodes: List[Node] = []

        def dq(x, s_name, z_name):
            out = graph.unique("dq")
            new_nodes.append(Node("DequantizeLinear", [x, s_name] + ([z_name] if z_name else []), [out], {},
                                  graph.unique("n_DequantizeLinear")))
            return out

        def const_float(x, s_name, z_name, axis):
            """Float value of a quantised constant (None when it is not constant)."""
            if x not in graph.initializers or s_name not in graph.initializers:
                return None
            v = graph.initializers[x].astype(np.float64)
            sc = np.asarray(graph.initializers[s_name], np.float64).reshape(-1)
            zp = np.asarray(graph.initializers[z_name], np.float64).reshape(-1) if z_name and z_name in graph.initializers \
                else np.zeros(1)
            shape = [1] * v.ndim
            if sc.size > 1:
                shape[axis] = sc.size
            return ((v - zp.reshape(shape if zp.size > 1 else [1] * v.ndim)) * sc.reshape(shape)).astype(np.float32)
        i = node.inputs
        attrs = {k: v for k, v in node.attrs.items() if not k.startswith("_")}
        if op_name == "QLinearConv":
            x = dq(i[0], i[1], i[2])
            wf = const_float(i[3], i[4], i[5], 0)
            w = graph.const(wf, prefix="w_deq") if wf is not None else dq(i[3], i[4], i[5])
            ins = [x, w]
            if len(i) > 8 and i[8]:
                if i[8] not in graph.initializers or i[1] not in graph.initializers or i[4] not in graph.initializers:
                    continue
                bias = graph.initializers[i[8]].astype(np.float64) * float(np.asarray(graph.initializers[i[1]]).reshape(-1)[0]) * \
                    np.asarray(graph.initializers[i[4]], np.float64).reshape(-1)
                ins.append(graph.const(bias.astype(np.float32), prefix="b_deq"))
            y = graph.unique("conv_f")
            new_nodes.append(Node("Conv", ins, [y], attrs, graph.unique("n_Conv")))
            ys, yz = i[6], i[7]
        elif op_name == "QLinearMatMul":
            a = dq(i[0], i[1], i[2])
            bf = const_float(i[3], i[4], i[5], -1)
            b = graph.const(bf, prefix="w_deq") if bf is not None else dq(i[3], i[4], i[5])
            y = graph.unique("matmul_f")
            new_nodes.append(Node("MatMul", [a, b], [y], {}, graph.unique("n_MatMul")))
            ys, yz = i[6], i[7]
        elif op_name in _QLINEAR_BINARY:
            a, b = dq(i[0], i[1], i[2] if len(i) > 2 else ""), dq(i[3], i[4], i[5] if len(i) > 5 else "")
            y = graph.unique("bin_f")
            new_nodes.append(Node(_QLINEAR_BINARY[op_name], [a, b], [y], {}, graph.unique("n_" + _QLINEAR_BINARY[op_name])))
            ys, yz = i[6], i[7] if len(i) > 7 else ""
        elif op_name == "QLinearConcat":
            ys, yz = i[0], i[1]
            parts = [dq(i[k], i[k + 1], i[k + 2]) for k in range(2, len(i), 3)]
            y = graph.unique("concat_f")
            new_nodes.append(Node("Concat", parts, [y], {"axis": attrs.get("axis", 1)}, graph.unique("n_Concat")))
        else:
            if attrs.pop("channels_last", 0):
                continue                                    # NHWC variant of the contrib pools: left as it is
            x = dq(i[0], i[1], i[2] if len(i) > 2 else "")
            y = graph.unique("unary_f")
            new_nodes.append(Node(_QLINEAR_UNARY[op_name], [x], [y], attrs, graph.unique("n_" + _QLINEAR_UNARY[op_name])))
            ys, yz = i[3], i[4] if len(i) > 4 else ""
        new_nodes.append(Node("QuantizeLinear", [y, ys] + ([yz] if yz else []), list(node.outputs), {},
                              graph.unique("n_QuantizeLinear")))
        at = graph.nodes.index(node)
        graph.nodes[at:at + 1] = new_nodes
        changed += 1
    if changed:
        graph.toposort()
    return changed


_LAYOUT_ONLY = ("Flatten", "Reshape", "Transpose", "Squeeze", "Unsqueeze", "Identity")


def hoist_dequantize_over_layout_ops(graph: Graph) -> int:
    """``q -> Flatten / Reshape / Transpose / ... -> DequantizeLinear(per-tensor)``  =>  ``q -> DequantizeLinear ->
    the same layout operator``: moving elements around commutes with a per-tensor dequantisation, and afterwards the
    quantise / dequantise pair is adjacent and :func:`fold_qdq` can take it out."""
    changed = 0
    again = True
    while again:
        again = False
        prod, cons = graph.producers(), graph.consumers()
        for dq in list(graph.nodes):
            if dq.op != "DequantizeLinear" or len(dq.inputs) < 2:
                continue
            sc = graph.initializers.get(dq.inputs[1])
            if sc is None or np.asarray(sc).size != 1:
                continue
            view = prod.get(dq.inputs[0])
            if view is None or view.op not in _LAYOUT_ONLY or len(cons.get(view.outputs[0], [])) != 1 or \
                    view.outputs[0] in graph.output_names():
                continue
            moved = graph.unique("dq_moved")
            new_dq = Node("DequantizeLinear", [view.inputs[0]] + list(dq.inputs[1:]), [moved], dict(dq.attrs),
                          graph.unique("n_DequantizeLinear"))
            new_view = Node(view.op, [moved] + list(view.inputs[1:]), list(dq.outputs), dict(view.attrs),
                            graph.unique("n_" + view.op), view.domain)
            at = graph.nodes.index(view)
            graph.nodes[at] = new_dq
            graph.nodes[graph.nodes.index(dq)] = new_view
            changed += 1
            again = True
            break
    if changed:
        graph.toposort()
    return changed


def fold_qdq(graph: Graph) -> int:
    """``x -> QuantizeLinear(s) -> DequantizeLinear(s) -> consumer``  =>  ``x -> consumer`` with the calibrated range
    ``s * 127`` of ``x`` recorded for the executor, which quantises ``x`` to e4m3 with that static range when it runs
    the consumer as an fp8 GEMM (and simply drops the fake quantisation at 16-bit precision). Weight-side
    ``DequantizeLinear`` nodes have constant inputs and are folded into float weights by constant folding before this
    pass. The reference rewrites the same pattern for TensorRT / ONNX Runtime int8
    (paddle2onnx/mapper/quantize_helper.cc:80-190, 348-620)."""
    changed = 0
    prod = graph.producers()
    scales = get_act_scales(graph)

    def const_scalar(name):
        v = graph.initializers.get(name) if name else None
        return None if v is None or np.asarray(v).size != 1 else np.asarray(v).reshape(-1)[0]
    for q in list(graph.nodes):
        if q.op != "QuantizeLinear" or q not in graph.nodes or q.inputs[1] not in graph.initializers:
            continue
        s_q = const_scalar(q.inputs[1])
        if s_q is None:
            continue                      # per-channel activation scales: keep the fake quantisation
        readers = graph.consumers().get(q.outputs[0], [])
        if not readers or q.outputs[0] in graph.output_names():
            continue
        zp_q = const_scalar(q.inputs[2]) if len(q.inputs) > 2 and q.inputs[2] else None

        def same(dq):
            if dq.op != "DequantizeLinear" or len(dq.inputs) < 2:
                return False
            s_d = const_scalar(dq.inputs[1])
            zp_d = const_scalar(dq.inputs[2]) if len(dq.inputs) > 2 and dq.inputs[2] else None
            return dq.op == "DequantizeLinear" and dq.inputs[0] == q.outputs[0] and s_d is not None and \
                abs(float(s_d) - float(s_q)) <= 1e-12 * max(1.0, abs(float(s_q))) and \
                int(zp_d if zp_d is not None else 0) == int(zp_q if zp_q is not None else 0)
        if not all(same(dq) for dq in readers):
            continue                      # a re-scaling pair or a reader that wants the integers: keep it
        x = q.inputs[0]
        if zp_q is not None and np.asarray(graph.initializers[q.inputs[2]]).dtype == np.uint8:
            reach = max(int(zp_q), 255 - int(zp_q))           # asymmetric uint8: the larger side of the zero point
        else:
            z = int(zp_q) if zp_q is not None else 0
            reach = max(128 + z, 127 - z) if z else 127
        scales[x] = float(s_q) * float(reach)
        dead = [q]
        for dq in readers:
            if dq.outputs[0] in graph.output_names():
                # a graph output keeps its name: the pair becomes a plain copy of the float value
                graph.nodes[graph.nodes.index(dq)] = Node("Identity", [x], list(dq.outputs), {}, graph.unique("n_Identity"))
            else:
                _replace_uses(graph, dq.outputs[0], x)
                dead.append(dq)
        _remove(graph, dead)
        prod = graph.producers()
        changed += 1
    if changed:
        set_act_scales(graph, scales)
    return changed


# --------------------------------------------------------------------------- conv folding
def fold_batchnorm(graph: Graph) -> int:
    """Conv / ConvTranspose -> BatchNormalization  =>  the convolution with scaled weights and folded bias."""
    changed = 0
    cons = graph.consumers()
    for conv in list(graph.nodes):
        if conv.op not in ("Conv", "ConvTranspose") or conv.inputs[1] not in graph.initializers:
            continue
        if conv.op == "ConvTranspose" and conv.attr("group", 1) != 1:
            continue
        bn = _single_consumer(cons, graph, conv.outputs[0])
        if bn is None or bn.op != "BatchNormalization" or bn.inputs[0] != conv.outputs[0]:
            continue
        if not all(i in graph.initializers for i in bn.inputs[1:5]):
            continue
        w = graph.initializers[conv.inputs[1]].astype(np.float64)
        b = graph.initializers[conv.inputs[2]].astype(np.float64) if len(conv.inputs) > 2 and conv.inputs[2] else 0.0
        scale, bias, mean, var = (graph.initializers[i].astype(np.float64) for i in bn.inputs[1:5])
        k = scale / np.sqrt(var + bn.attr("epsilon", 1e-5))
        # output channels are dimension 0 of a Conv weight and dimension 1 of a ConvTranspose weight
        kshape = [-1] + [1] * (w.ndim - 1) if conv.op == "Conv" else [1, -1] + [1] * (w.ndim - 2)
        w2 = (w * k.reshape(kshape)).astype(np.float32)
        b2 = ((b - mean) * k + bias).astype(np.float32)
        conv.inputs = [conv.inputs[0], graph.const(w2, prefix="w_bnfold"), graph.const(b2, prefix="b_bnfold")]
        conv.outputs = [bn.outputs[0]]
        _remove(graph, [bn])
        cons = graph.consumers()
        changed += 1
    return changed


def fold_conv_bias_add(graph: Graph) -> int:
    """Conv -> Add(per-channel constant)  =>  Conv with bias (Paddle exports bias as elementwise_add)."""
    changed = 0
    cons = graph.consumers()
    for conv in list(graph.nodes):
        if conv.op not in ("Conv", "ConvTranspose") or conv.inputs[1] not in graph.initializers:
            continue
        add = _single_consumer(cons, graph, conv.outputs[0])
        if add is None or add.op != "Add":
            continue
        other = add.inputs[1] if add.inputs[0] == conv.outputs[0] else add.inputs[0]
        if other not in graph.initializers:
            continue
        w = graph.initializers[conv.inputs[1]]
        cout = w.shape[0] if conv.op == "Conv" else w.shape[1] * conv.attr("group", 1)
        bv = graph.initializers[other]
        if bv.size != cout or (bv.ndim > 1 and bv.shape[1 if bv.ndim == w.ndim else 0] != cout and bv.size != 1):
            continue
        bv = bv.reshape(-1).astype(np.float32)
        if len(conv.inputs) > 2 and conv.inputs[2]:
            bv = bv + graph.initializers[conv.inputs[2]].astype(np.float32)
        conv.inputs = [conv.inputs[0], conv.inputs[1], graph.const(bv, prefix="b_fold")]
        conv.outputs = [add.outputs[0]]
        _remove(graph, [add])
        cons = graph.consumers()
        changed += 1
    return changed


def fold_repvgg(graph: Graph) -> int:
    """Add(Conv3x3(x), Conv1x1(x) [, x via identity BN]) => one Conv3x3 (re-parameterisation)."""
    changed = 0
    prod = graph.producers()
    cons = graph.consumers()
    for add in list(graph.nodes):
        if add.op != "Add":
            continue
        a, b = prod.get(add.inputs[0]), prod.get(add.inputs[1])
        if a is None or b is None or a.op != "Conv" or b.op != "Conv" or a.inputs[0] != b.inputs[0]:
            continue
        if _single_consumer(cons, graph, a.outputs[0]) is not add or _single_consumer(cons, graph, b.outputs[0]) is not add:
            continue
        wa, wb = graph.initializers.get(a.inputs[1]), graph.initializers.get(b.inputs[1])
        if wa is None or wb is None:
            continue
        if wa.shape[2:] == (1, 1) and wb.shape[2:] == (3, 3):
            a, b, wa, wb = b, a, wb, wa
        if wa.shape[2:] != (3, 3) or wb.shape[2:] != (1, 1) or wa.shape[:2] != wb.shape[:2]:
            continue
        if a.attr("strides", [1, 1]) != b.attr("strides", [1, 1]) or a.attr("group", 1) != b.attr("group", 1):
            continue
        if list(a.attr("pads", [0] * 4)) != [1, 1, 1, 1] or any(b.attr("pads", [0] * 4)):
            continue
        w = wa.astype(np.float32).copy()
        w[:, :, 1, 1] += wb[:, :, 0, 0]
        bias = np.zeros(w.shape[0], np.float32)
        for cnode in (a, b):
            if len(cnode.inputs) > 2 and cnode.inputs[2]:
                bias = bias + graph.initializers[cnode.inputs[2]].astype(np.float32)
        a.inputs = [a.inputs[0], graph.const(w, prefix="w_rep"), graph.const(bias, prefix="b_rep")]
        a.outputs = [add.outputs[0]]
        _remove(graph, [b, add])
        prod, cons = graph.producers(), graph.consumers()
        changed += 1
    return changed


# --------------------------------------------------------------------------- activation patterns
def recognize_silu(graph: Graph) -> int:
    """Mul(x, Sigmoid(x)) => Silu(x);  Mul(x, HardSigmoid(x; 1/6, 0.5)) => HardSwish(x)."""
    changed = 0
    prod = graph.producers()
    cons = graph.consumers()
    for mul in list(graph.nodes):
        if mul.op != "Mul":
            continue
        for xi, si in ((0, 1), (1, 0)):
            s = prod.get(mul.inputs[si])
            if s is None or s.inputs[0] != mul.inputs[xi] or _single_consumer(cons, graph, s.outputs[0]) is not mul:
                continue
            if s.op == "Sigmoid":
                new = "Silu"
            elif s.op == "HardSigmoid" and abs(s.attr("alpha", 0.2) - 1 / 6) < 1e-6 and abs(s.attr("beta", 0.5) - 0.5) < 1e-6:
                new = "HardSwish"
            else:
                continue
            mul.op, mul.inputs, mul.attrs = new, [mul.inputs[xi]], {}
            _remove(graph, [s])
            prod, cons = graph.producers(), graph.consumers()
            changed += 1
            break
    return changed


def recognize_gelu(graph: Graph) -> int:
    """x * 0.5 * (1 + erf(x / sqrt(2))) in any multiplication order => Gelu(x)."""
    changed = 0
    prod = graph.producers()
    cons = graph.consumers()

    def const_val(name):
        v = graph.initializers.get(name)
        return float(v.reshape(-1)[0]) if v is not None and v.size == 1 else None

    for erf in [n for n in graph.nodes if n.op == "Erf"]:
        div = prod.get(erf.inputs[0])
        if div is None:
            continue
        if div.op == "Div" and const_val(div.inputs[1]) is not None and abs(const_val(div.inputs[1]) - math.sqrt(2)) < 1e-3:
            x = div.inputs[0]
        elif div.op == "Mul" and any(const_val(i) is not None and abs(const_val(i) - 1 / math.sqrt(2)) < 1e-3 for i in div.inputs):
            x = div.inputs[0] if const_val(div.inputs[1]) is not None else div.inputs[1]
        else:
            continue
        add = _single_consumer(cons, graph, erf.outputs[0])
        if add is None or add.op != "Add" or not any(const_val(i) == 1.0 for i in add.inputs):
            continue
        # collect the multiplication chain that follows: needs x and 0.5
        chain, cur, have_x, have_half = [], add, False, False
        while True:
            nxt = _single_consumer(cons, graph, cur.outputs[0])
            if nxt is None or nxt.op != "Mul":
                break
            other = nxt.inputs[1] if nxt.inputs[0] == cur.outputs[0] else nxt.inputs[0]
            if other == x:
                have_x = True
            elif const_val(other) == 0.5:
                have_half = True
            else:
                p = prod.get(other)
                if p is not None and p.op == "Mul" and x in p.inputs and any(const_val(i) == 0.5 for i in p.inputs) \
                        and _single_consumer(cons, graph, p.outputs[0]) is nxt:
                    have_x = have_half = True
                    chain.append(p)
                else:
                    break
            chain.append(nxt)
            cur = nxt
            if have_x and have_half:
                break
        if not (have_x and have_half):
            continue
        last = chain[-1]
        graph.nodes[graph.nodes.index(last)] = Node("Gelu", [x], [last.outputs[0]], {"approximate": "none"}, last.name)
        _remove(graph, [div, erf, add] + chain[:-1])
        prod, cons = graph.producers(), graph.consumers()
        changed += 1
    return changed


def recognize_layernorm(graph: Graph) -> int:
    """ReduceMean / Sub / Pow|Mul / ReduceMean / Add eps / Sqrt / Div / Mul gamma / Add beta => LayerNormalization."""
    changed = 0
    prod = graph.producers()
    cons = graph.consumers()
    for sqrt in [n for n in graph.nodes if n.op == "Sqrt"]:
        add_eps = prod.get(sqrt.inputs[0])
        if add_eps is None or add_eps.op != "Add":
            continue
        eps_name = next((i for i in add_eps.inputs if i in graph.initializers and graph.initializers[i].size == 1), None)
        var_name = next((i for i in add_eps.inputs if i != eps_name), None)
        var = prod.get(var_name)
        if eps_name is None or var is None or var.op != "ReduceMean":
            continue
        sq = prod.get(var.inputs[0])
        if sq is None or sq.op not in ("Pow", "Mul"):
            continue
        sub = prod.get(sq.inputs[0])
        if sub is None or sub.op != "Sub":
            continue
        mean = prod.get(sub.inputs[1])
        if mean is None or mean.op != "ReduceMean" or mean.inputs[0] != sub.inputs[0]:
            continue
        axes = mean.attr("axes", [-1])
        if list(axes) not in ([-1],) and not (len(axes) == 1):
            continue
        div = _single_consumer(cons, graph, sqrt.outputs[0])
        if div is None or div.op != "Div" or div.inputs[0] != sub.outputs[0]:
            continue
        x = sub.inputs[0]
        out, dead = div.outputs[0], [mean, sub, sq, var, add_eps, sqrt, div]
        gamma = beta = ""
        mul = _single_consumer(cons, graph, out)
        if mul is not None and mul.op == "Mul":
            g = next((i for i in mul.inputs if i in graph.initializers), None)
            if g is not None:
                gamma, out = g, mul.outputs[0]
                dead.append(mul)
                addb = _single_consumer(cons, graph, out)
                if addb is not None and addb.op == "Add":
                    bname = next((i for i in addb.inputs if i in graph.initializers), None)
                    if bname is not None:
                        beta, out = bname, addb.outputs[0]
                        dead.append(addb)
        eps = float(graph.initializers[eps_name].reshape(-1)[0])
        idx = graph.nodes.index(dead[-1])
        graph.nodes[idx] = Node("LayerNormalization", [x, gamma, beta], [out], {"axis": int(axes[0]), "epsilon": eps},
                                graph.unique("n_LayerNorm"))
        _remove(graph, dead[:-1])
        prod, cons = graph.producers(), graph.consumers()
        changed += 1
    return changed


# --------------------------------------------------------------------------- fusion into conv / gemm
def fuse_conv_activation(graph: Graph) -> int:
    """Conv (+Add residual) + activation (+Add residual) => FusedConv (domain fdb)."""
    changed = 0
    cons = graph.consumers()
    for conv in list(graph.nodes):
        if conv.op != "Conv" or conv.inputs[1] not in graph.initializers:
            continue
        if conv.attr("auto_pad", "NOTSET") not in ("NOTSET", "VALID") and False:
            continue
        out = conv.outputs[0]
        attrs = dict(conv.attrs)
        attrs.update(activation="none", act_alpha=0.0, act_beta=0.0, res_mode=0)
        dead: List[Node] = []
        residual = ""
        nxt = _single_consumer(cons, graph, out)
        # residual before activation (ResNet): Conv -> Add(res) -> Relu
        if nxt is not None and nxt.op == "Add":
            other = nxt.inputs[1] if nxt.inputs[0] == out else nxt.inputs[0]
            after = _single_consumer(cons, graph, nxt.outputs[0])
            if other not in graph.initializers and other != out and after is not None and _act_of(after, graph):
                residual, attrs["res_mode"] = other, 1
                dead.append(nxt)
                out = nxt.outputs[0]
                nxt = after
        if nxt is not None:
            act = _act_of(nxt, graph)
            if act is not None:
                attrs["activation"], attrs["act_alpha"], attrs["act_beta"] = act
                dead.append(nxt)
                out = nxt.outputs[0]
                nxt = _single_consumer(cons, graph, out)
        # residual after activation (CSPRes basic block): act(Conv) + x
        if attrs["res_mode"] == 0 and nxt is not None and nxt.op == "Add":
            other = nxt.inputs[1] if nxt.inputs[0] == out else nxt.inputs[0]
            if other not in graph.initializers and other != out:
                residual, attrs["res_mode"] = other, 2
                dead.append(nxt)
                out = nxt.outputs[0]
        bias = conv.inputs[2] if len(conv.inputs) > 2 else ""
        conv.op, conv.domain = "FusedConv", "fdb"
        conv.inputs = [conv.inputs[0], conv.inputs[1], bias] + ([residual] if residual else [])
        conv.outputs = [out]
        conv.attrs = attrs
        if dead:
            # the fused node must come after the residual's producer
            _remove(graph, dead)
            if residual:
                graph.nodes.remove(conv)
                graph.nodes.append(conv)
                graph.toposort()
            cons = graph.consumers()
        changed += 1
    return changed


def fuse_deconv_activation(graph: Graph) -> int:
    """ConvTranspose + activation => ConvTranspose carrying ``activation`` / ``act_alpha`` / ``act_beta`` attributes
    (applied by the interpreter and fused into the epilogue by the native backend)."""
    changed = 0
    cons = graph.consumers()
    for dc in list(graph.nodes):
        if dc.op != "ConvTranspose" or dc.attr("activation", None) is not None:
            continue
        nxt = _single_consumer(cons, graph, dc.outputs[0])
        act = _act_of(nxt, graph) if nxt is not None else None
        if act is None:
            continue
        dc.attrs["activation"], dc.attrs["act_alpha"], dc.attrs["act_beta"] = act
        dc.outputs = [nxt.outputs[0]]
        _remove(graph, [nxt])
        cons = graph.consumers()
        changed += 1
    return changed


def fuse_gemm(graph: Graph, info: Optional[ShapeInfo] = None) -> int:
    """MatMul(x, W) | Gemm (+Add bias) (+activation) (+Add residual) => FusedGemm with W as [N, K]."""
    changed = 0
    cons = graph.consumers()
    for mm in list(graph.nodes):
        if mm.op == "MatMul":
            wname = mm.inputs[1]
            w = graph.initializers.get(wname)
            if w is None or w.ndim != 2:
                continue
            w_nk = np.ascontiguousarray(w.T)
            bias = ""
        elif mm.op == "Gemm":
            w = graph.initializers.get(mm.inputs[1])
            if w is None or mm.attr("transA", 0) or mm.attr("alpha", 1.0) != 1.0 or mm.attr("beta", 1.0) != 1.0:
                continue
            w_nk = np.ascontiguousarray(w if mm.attr("transB", 0) else w.T)
            bias = mm.inputs[2] if len(mm.inputs) > 2 else ""
            if bias and (bias not in graph.initializers or graph.initializers[bias].size != w_nk.shape[0]):
                continue
        else:
            continue
        out = mm.outputs[0]
        dead: List[Node] = []
        attrs = dict(activation="none", act_alpha=0.0, act_beta=0.0, res_mode=0)
        nxt = _single_consumer(cons, graph, out)
        if not bias and nxt is not None and nxt.op == "Add":
            other = nxt.inputs[1] if nxt.inputs[0] == out else nxt.inputs[0]
            if other in graph.initializers and graph.initializers[other].size == w_nk.shape[0]:
                bias = graph.const(graph.initializers[other].reshape(-1).astype(np.float32), prefix="b_gemm")
                dead.append(nxt)
                out = nxt.outputs[0]
                nxt = _single_consumer(cons, graph, out)
        elif bias:
            bias = graph.const(graph.initializers[bias].reshape(-1).astype(np.float32), prefix="b_gemm")
        if nxt is not None:
            act = _act_of(nxt, graph)
            if act is not None:
                attrs["activation"], attrs["act_alpha"], attrs["act_beta"] = act
                dead.append(nxt)
                out = nxt.outputs[0]
                nxt = _single_consumer(cons, graph, out)
        residual = ""
        if nxt is not None and nxt.op == "Add":
            other = nxt.inputs[1] if nxt.inputs[0] == out else nxt.inputs[0]
            same_shape = info is None or info.shapes.get(other) == info.shapes.get(out)
            if other not in graph.initializers and other != out and same_shape:
                residual, attrs["res_mode"] = other, 2
                dead.append(nxt)
                out = nxt.outputs[0]
        mm.op, mm.domain = "FusedGemm", "fdb"
        mm.inputs = [mm.inputs[0], graph.const(w_nk, prefix="w_nk"), bias] + ([residual] if residual else [])
        mm.outputs = [out]
        mm.attrs = attrs
        _remove(graph, dead)
        if residual:
            graph.nodes.remove(mm)
            graph.nodes.append(mm)
            graph.toposort()
        cons = graph.consumers()
        changed += 1
    return changed


def fuse_qkv_gemms(graph: Graph) -> int:
    """The query / key / value projections of an attention layer are three linear layers of the same input: one
    FusedGemm with the weights stacked along the output dimension, and three Slice views of its output, reads the
    activations once and gives the tensor cores a wider tile. Only projections whose sole reader is one
    (Packed)Attention node are merged."""
    changed = 0
    cons = graph.consumers()
    prod = graph.producers()
    for att in [n for n in graph.nodes if n.op in ("Attention", "PackedAttention")]:
        gemms = [prod.get(nm) for nm in att.inputs[:3]]
        if any(g is None or g.op != "FusedGemm" or len(g.inputs) != 3 for g in gemms) or len({id(g) for g in gemms}) != 3:
            continue
        x = gemms[0].inputs[0]
        if any(g.inputs[0] != x or g.attrs != gemms[0].attrs or g.attr("activation", "none") != "none" or
               len(cons.get(g.outputs[0], [])) != 1 or g.outputs[0] in graph.output_names() for g in gemms):
            continue
        ws = [graph.initializers.get(g.inputs[1]) for g in gemms]
        if any(w is None or w.ndim != 2 or w.shape[1] != ws[0].shape[1] or w.shape[0] % 8 for w in ws):
            continue
        bs = []
        for g, w in zip(gemms, ws):
            b = graph.initializers.get(g.inputs[2]) if g.inputs[2] else np.zeros(w.shape[0], np.float32)
            if b is None:
                break
            bs.append(np.asarray(b, np.float32).reshape(-1))
        if len(bs) != 3:
            continue
        w_all = graph.const(np.ascontiguousarray(np.concatenate(ws, 0)), prefix="w_qkv")
        b_all = graph.const(np.concatenate(bs, 0), prefix="b_qkv")
        fused_out = graph.unique("qkv")
        first = min(graph.nodes.index(g) for g in gemms)
        fused = Node("FusedGemm", [x, w_all, b_all], [fused_out], dict(gemms[0].attrs), graph.unique("n_FusedGemm_qkv"),
                     "fdb")
        slices, at = [], 0
        for g, w in zip(gemms, ws):
            st = graph.const(np.asarray([at], np.int64), prefix="qkv_start")
            en = graph.const(np.asarray([at + w.shape[0]], np.int64), prefix="qkv_end")
            ax = graph.const(np.asarray([-1], np.int64), prefix="qkv_axis")
            slices.append(Node("Slice", [fused_out, st, en, ax], [g.outputs[0]], {}, graph.unique("n_Slice_qkv")))
            at += w.shape[0]
        for g in gemms:
            graph.nodes.remove(g)
        graph.nodes[first:first] = [fused] + slices
        changed += 1
    if changed:
        graph.toposort()
    return changed


# --------------------------------------------------------------------------- transformer blocks
def fuse_attention(graph: Graph, info: ShapeInfo) -> int:
    """Recognises multi-head self-attention written with Reshape/Transpose/MatMul/Softmax:

        q,k,v [B,S,H*D] -Reshape-> [B,S,H,D] -Transpose(0,2,1,3)-> [B,H,S,D]
        softmax(q @ k^T * scale (+ mask)) @ v -Transpose(0,2,1,3)-> Reshape [B,S,H*D]

    and replaces it by one ``Attention`` node (domain fdb). The scale may sit on q, on k or on the scores."""
    changed = 0
    prod = graph.producers()
    cons = graph.consumers()

    def scalar(name):
        v = graph.initializers.get(name)
        return float(v.reshape(-1)[0]) if v is not None and v.size == 1 else None

    def peel_scale(name):
        """value name -> (source name, multiplicative scale)"""
        p = prod.get(name)
        if p is not None and p.op in ("Mul", "Div"):
            for a, b in ((0, 1), (1, 0)):
                s = scalar(p.inputs[b])
                if s is not None and (p.op == "Mul" or b == 1):
                    return p.inputs[a], (s if p.op == "Mul" else 1.0 / s), [p]
        return name, 1.0, []

    def head_split(name):
        """[B,H,S,D] value produced by Transpose(0,2,1,3)(Reshape(x)) -> (x, heads, dead nodes)"""
        t = prod.get(name)
        if t is None or t.op != "Transpose" or list(t.attr("perm", [])) != [0, 2, 1, 3]:
            return None
        r = prod.get(t.inputs[0])
        if r is None or r.op != "Reshape":
            return None
        shp = info.shapes.get(r.outputs[0])
        if shp is None or len(shp) != 4:
            return None
        return r.inputs[0], shp[2], [t, r]

    for sm in [n for n in graph.nodes if n.op == "Softmax"]:
        dead: List[Node] = [sm]
        scale = 1.0
        src = sm.inputs[0]
        mask = ""
        p = prod.get(src)
        if p is not None and p.op == "Add":
            a, b = p.inputs
            pa, pb = prod.get(a), prod.get(b)
            # the branch that leads to a MatMul is the scores; the other is the additive mask
            def leads_to_mm(nm):
                q = prod.get(nm)
                while q is not None and q.op in ("Mul", "Div"):
                    q = prod.get(q.inputs[0])
                return q is not None and q.op == "MatMul"
            if leads_to_mm(a):
                src, mask = a, b
            elif leads_to_mm(b):
                src, mask = b, a
            else:
                continue
            dead.append(p)
        src, s1, d1 = peel_scale(src)
        scale *= s1
        dead += d1
        qk = prod.get(src)
        if qk is None or qk.op != "MatMul":
            continue
        dead.append(qk)
        qn, s2, d2 = peel_scale(qk.inputs[0])
        scale *= s2
        dead += d2
        kn = qk.inputs[1]
        kt = prod.get(kn)
        if kt is None or kt.op != "Transpose":
            continue
        perm = list(kt.attr("perm", []))
        if perm == [0, 1, 3, 2]:
            kn2, s3, d3 = peel_scale(kt.inputs[0])
            ksplit = head_split(kn2)
            dead += [kt] + d3
            scale *= s3
        elif perm == [0, 2, 3, 1]:      # Transpose straight from [B,S,H,D] to [B,H,D,S]
            r = prod.get(kt.inputs[0])
            if r is None or r.op != "Reshape":
                continue
            shp = info.shapes.get(r.outputs[0])
            ksplit = (r.inputs[0], shp[2], [kt, r])
        else:
            continue
        qsplit = head_split(qn)
        pv = _single_consumer(cons, graph, sm.outputs[0])
        if pv is None or pv.op != "MatMul" or pv.inputs[0] != sm.outputs[0]:
            continue
        vsplit = head_split(pv.inputs[1])
        if qsplit is None or ksplit is None or vsplit is None:
            continue
        t_out = _single_consumer(cons, graph, pv.outputs[0])
        if t_out is None or t_out.op != "Transpose" or list(t_out.attr("perm", [])) != [0, 2, 1, 3]:
            continue
        r_out = _single_consumer(cons, graph, t_out.outputs[0])
        if r_out is None or r_out.op != "Reshape":
            continue
        heads = qsplit[1]
        dead += [pv, t_out] + qsplit[2] + ksplit[2] + vsplit[2]
        # every removed node must feed only this pattern
        dead_ids = {id(n) for n in dead} | {id(r_out)}
        ok = True
        for n in dead:
            for o in n.outputs:
                if any(id(cn) not in dead_ids for cn in cons.get(o, [])) or o in graph.output_names():
                    ok = False
        if not ok:
            continue
        node = Node("Attention", [qsplit[0], ksplit[0], vsplit[0]] + ([mask] if mask else []), [r_out.outputs[0]],
                    {"num_heads": int(heads), "scale": float(scale)}, graph.unique("n_Attention"), "fdb")
        graph.nodes[graph.nodes.index(r_out)] = node
        _remove(graph, dead)
        graph.toposort()
        prod, cons = graph.producers(), graph.consumers()
        changed += 1
    return changed


def fuse_embed_layernorm(graph: Graph) -> int:
    """LayerNormalization(Gather(T0, ids0) + Gather(T1, ids1) + ...) => EmbedLayerNorm (domain fdb)."""
    changed = 0
    prod = graph.producers()
    cons = graph.consumers()
    for ln in [n for n in graph.nodes if n.op == "LayerNormalization"]:
        leaves, dead, stack = [], [], [ln.inputs[0]]
        ok = True
        while stack:
            name = stack.pop()
            p = prod.get(name)
            if p is None:
                ok = False
                break
            if p.op == "Add" and _single_consumer(cons, graph, p.outputs[0]) is not None:
                dead.append(p)
                stack += [p.inputs[1], p.inputs[0]]
            elif p.op == "Gather" and p.inputs[0] in graph.initializers and p.attr("axis", 0) == 0 \
                    and graph.initializers[p.inputs[0]].ndim == 2 and _single_consumer(cons, graph, p.outputs[0]) is not None:
                dead.append(p)
                leaves.append((p.inputs[1], p.inputs[0]))
            else:
                ok = False
                break
        if not ok or len(leaves) < 2 or not ln.inputs[1] or not ln.inputs[2]:
            continue
        ids = [l[0] for l in leaves]
        tabs = [l[1] for l in leaves]
        node = Node("EmbedLayerNorm", ids + tabs + [ln.inputs[1], ln.inputs[2]], [ln.outputs[0]],
                    {"num_tables": len(leaves), "epsilon": float(ln.attr("epsilon", 1e-5))},
                    graph.unique("n_EmbedLayerNorm"), "fdb")
        graph.nodes[graph.nodes.index(ln)] = node
        _remove(graph, dead)
        graph.toposort()
        prod, cons = graph.producers(), graph.consumers()
        changed += 1
    return changed


# --------------------------------------------------------------------------- pipelines
def optimize(graph: Graph, input_shapes: Optional[Dict[str, Sequence[int]]] = None,
             input_values: Optional[Dict[str, np.ndarray]] = None, level: int = 2) -> Graph:
    """Runs the standard pipeline on a copy of ``graph``.

    level 0: nothing; 1: constant folding and BN / bias folding (numerically safe rewrites);
    2: + operator fusion into FusedConv / FusedGemm / Attention / EmbedLayerNorm."""
    g = graph.clone()
    if level <= 0:
        return g
    if any(n.op in ("Loop", "If", "Scan") for n in g.nodes):
        # the bodies of control-flow nodes read values of this scope by name: rewrites that rename or remove values
        # would have to follow them into the bodies, so such graphs run as imported
        return g
    g.toposort()
    eliminate_identity(g)
    expand_qlinear(g)                      # before shape inference: the integer operators have no shape rules of their own
    info = None
    if input_shapes is not None:
        info = infer_shapes(g, input_shapes, input_values)
    for _ in range(4):
        if not fold_constants(g, info):
            break
    hoist_dequantize_over_layout_ops(g)
    if fold_qdq(g):
        for _ in range(2):
            if not fold_constants(g, info):
                break
    fold_conv_bias_add(g)
    fold_batchnorm(g)
    fold_conv_bias_add(g)
    fold_repvgg(g)
    recognize_silu(g)
    recognize_gelu(g)
    recognize_layernorm(g)
    if level >= 2:
        if info is not None:
            info = infer_shapes(g, input_shapes, input_values)
            fuse_attention(g, info)
        fuse_embed_layernorm(g)
        fuse_conv_activation(g)
        fuse_deconv_activation(g)
        fuse_gemm(g, info)
        fuse_qkv_gemms(g)
        if info is not None and any(n.op == "MultiClassNMS" for n in g.nodes):
            info = infer_shapes(g, input_shapes, input_values)
            fuse_ppyoloe_head(g, info)
    g.prune()
    g.toposort()
    return g


# --------------------------------------------------------------------------- PP-YOLOE head
def fuse_ppyoloe_head(graph: Graph, info: ShapeInfo) -> int:
    """Collapses the exported PP-YOLOE ET-head tail - per level Reshape/Transpose/Softmax/projection
    conv (DFL integral), distance->box with constant anchor points and strides, division by the
    scale factor, score concat and ``MultiClassNMS`` - into one ``PPYOLOEPost`` node (domain fdb)
    that consumes the per-level class-score maps ``[b,C,H,W]`` and regression maps ``[b,4*bins,H,W]``."""
    changed = 0
    prod = graph.producers()

    def const(name):
        return graph.initializers.get(name)

    for nms in [n for n in graph.nodes if n.op == "MultiClassNMS"]:
        try:
            boxes_name, scores_name = nms.inputs[:2]
            sc = prod[scores_name]
            assert sc.op == "Concat"
            cls_src, grids = [], []
            for nm in sc.inputs:
                r = prod[nm]
                assert r.op == "Reshape"
                shp = info.shapes[r.inputs[0]]
                assert len(shp) == 4 and info.shapes[nm] == [shp[0], shp[1], shp[2] * shp[3]]
                cls_src.append(r.inputs[0])
                grids.append((shp[2], shp[3]))
            div = prod[boxes_name]
            assert div.op == "Div"
            # scale factor expression: Reshape(Concat(sx, sy, sx, sy)) with (sy, sx) = Split(scale_factor)
            rs = prod[div.inputs[1]]
            assert rs.op == "Reshape"
            cc = prod[rs.inputs[0]]
            assert cc.op == "Concat" and len(cc.inputs) == 4
            sp = prod[cc.inputs[0]]
            assert sp.op == "Split" and sp.inputs[0] in graph.input_names()
            assert cc.inputs == [sp.outputs[1], sp.outputs[0], sp.outputs[1], sp.outputs[0]]
            sf_input = sp.inputs[0]
            mul = prod[div.inputs[0]]
            assert mul.op == "Mul"
            stride_c = const(mul.inputs[1]) if const(mul.inputs[1]) is not None else const(mul.inputs[0])
            cat_name = mul.inputs[0] if const(mul.inputs[1]) is not None else mul.inputs[1]
            cat = prod[cat_name]
            assert cat.op == "Concat" and len(cat.inputs) == 2
            sub, add = prod[cat.inputs[0]], prod[cat.inputs[1]]
            assert sub.op == "Sub" and add.op == "Add"
            anchor = const(sub.inputs[0])
            assert anchor is not None
            lt = sub.inputs[1]
            rb = add.inputs[0] if const(add.inputs[1]) is not None else add.inputs[1]
            spl = prod[lt]
            assert spl.op == "Split" and spl.outputs == [lt, rb]
            dcat = prod[spl.inputs[0]]
            assert dcat.op == "Concat"
            reg_src, bins = [], None
            for nm in dcat.inputs:
                sq = prod[nm]
                assert sq.op == "Squeeze"
                cv = prod[sq.inputs[0]]
                assert cv.op in ("Conv", "FusedConv") and cv.attr("activation", "none") == "none"
                w = const(cv.inputs[1])
                assert w is not None and w.shape[0] == 1 and np.allclose(w.reshape(-1), np.arange(w.size))
                bins = int(w.size)
                sm = prod[cv.inputs[0]]
                assert sm.op == "Softmax"
                tr = prod[sm.inputs[0]]
                assert tr.op == "Transpose" and list(tr.attr("perm")) == [0, 2, 3, 1]
                rr = prod[tr.inputs[0]]
                assert rr.op == "Reshape"
                rshape = info.shapes[rr.inputs[0]]
                assert len(rshape) == 4 and rshape[1] == 4 * bins
                reg_src.append(rr.inputs[0])
            assert len(reg_src) == len(cls_src)
            # anchors / strides must be the canonical grid
            strides, pos = [], 0
            for (h, w) in grids:
                l = h * w
                ys, xs = np.meshgrid(np.arange(h, dtype=np.float32) + 0.5, np.arange(w, dtype=np.float32) + 0.5, indexing="ij")
                pts = np.stack([xs.reshape(-1), ys.reshape(-1)], -1)
                assert np.allclose(anchor[pos:pos + l], pts)
                s = stride_c.reshape(-1)[pos:pos + l]
                assert np.all(s == s[0])
                strides.append(int(s[0]))
                pos += l
            assert pos == anchor.shape[0]
        except (AssertionError, KeyError, IndexError):
            continue
        attrs = {k: v for k, v in nms.attrs.items() if not k.startswith("_")}
        attrs.update(strides=strides, grid_h=[g[0] for g in grids], grid_w=[g[1] for g in grids], bins=bins,
                     offset=0.5, num_levels=len(grids))
        node = Node("PPYOLOEPost", cls_src + reg_src + [sf_input], list(nms.outputs), attrs,
                    graph.unique("n_PPYOLOEPost"), "fdb")
        graph.nodes[graph.nodes.index(nms)] = node
        graph.prune()
        prod = graph.producers()
        changed += 1
    return changed
