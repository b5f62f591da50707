"""Reference interpreter for the IR (fp32, PyTorch CPU tensors - or any torch device).

It is the numerical oracle for every fused pass and every CUDA kernel, and it is the
engine behind ``RuntimeOption.use_cpu()`` - the role ONNX Runtime's CPU provider plays
in the reference (fastdeploy/runtime/backends/ort/ort_backend.cc:366-407).
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np
import torch
import torch.nn.functional as F

from .graph import Graph, Node

_OPS: Dict[str, Callable] = {}

NP2TORCH = {"float32": torch.float32, "float64": torch.float64, "float16": torch.float16, "int64": torch.int64,
            "int32": torch.int32, "int16": torch.int16, "int8": torch.int8, "uint8": torch.uint8, "bool": torch.bool,
            "bfloat16": torch.bfloat16}
ONNX_DT2TORCH = {1: torch.float32, 2: torch.uint8, 3: torch.int8, 5: torch.int16, 6: torch.int32, 7: torch.int64,
                 9: torch.bool, 10: torch.float16, 11: torch.float64, 16: torch.bfloat16}


def op(*names):
    def deco(fn):
        for n in names:
            _OPS[n] = fn
        return fn
    return deco


def supported_ops() -> List[str]:
    return sorted(_OPS)


def _ints(t) -> List[int]:
    if t is None:
        return []
    if isinstance(t, torch.Tensor):
        return [int(v) for v in t.flatten().tolist()]
    return [int(v) for v in t]


def _pads_2d(node: Node, x, kernel, strides, dilations=(1, 1)):
    """ONNX pads/auto_pad -> (top, left, bottom, right)."""
    auto = node.attr("auto_pad", "NOTSET")
    nd = len(kernel)
    if auto in ("SAME_UPPER", "SAME_LOWER"):
        pads_b, pads_e = [], []
        for i in range(nd):
            size = x.shape[2 + i]
            out = math.ceil(size / strides[i])
            total = max((out - 1) * strides[i] + (kernel[i] - 1) * dilations[i] + 1 - size, 0)
            lo = total // 2 if auto == "SAME_UPPER" else total - total // 2
            pads_b.append(lo)
            pads_e.append(total - lo)
        return pads_b + pads_e
    if auto == "VALID":
        return [0] * (2 * nd)
    return list(node.attr("pads", [0] * (2 * nd)))


def _apply_pad_nd(x, pads, value=0.0):
    nd = len(pads) // 2
    if not any(pads):
        return x
    tp = []
    for i in reversed(range(nd)):
        tp += [pads[i], pads[nd + i]]
    return F.pad(x, tp, value=value)


ACTIVATIONS = {
    None: lambda x, a, b: x, "": lambda x, a, b: x, "none": lambda x, a, b: x,
    "relu": lambda x, a, b: torch.relu(x),
    "silu": lambda x, a, b: F.silu(x),
    "hard_swish": lambda x, a, b: F.hardswish(x),
    "hard_sigmoid": lambda x, a, b: torch.clamp(a * x + b, 0, 1),
    "sigmoid": lambda x, a, b: torch.sigmoid(x),
    "gelu": lambda x, a, b: F.gelu(x),
    "relu6": lambda x, a, b: F.relu6(x),
    "leaky_relu": lambda x, a, b: F.leaky_relu(x, a),
    "tanh": lambda x, a, b: torch.tanh(x),
}


# ------------------------------------------------------------------------- NN ops
@op("Conv")
def _conv(node, x, w, b=None):
    nd = w.dim() - 2
    strides = node.attr("strides", [1] * nd)
    dil = node.attr("dilations", [1] * nd)
    group = node.attr("group", 1)
    pads = _pads_2d(node, x, list(w.shape[2:]), strides, dil)
    sym = all(pads[i] == pads[nd + i] for i in range(nd))
    if not sym:
        x = _apply_pad_nd(x, pads)
        pad = [0] * nd
    else:
        pad = pads[:nd]
    if nd == 2 and node.attrs.get("_cpu_fast") and x.device.type == "cpu" and x.dtype == torch.float32 \
            and w.dtype == torch.float32 and x.dim() == 4:
        y = _cpu_packed_conv(node, x, w, b, pad, strides, dil, group, "none")
        if y is not None:
            return y
    fn = {1: F.conv1d, 2: F.conv2d, 3: F.conv3d}[nd]
    return fn(x, w, b, stride=strides, padding=pad, dilation=dil, groups=group)


def _cpu_packed_conv(node, x, w, b, pad, strides, dil, group, act):
    """CPU fast path of the interpreter (``Interpreter(channels_last=True)``): the vendor primitive with the weights
    re-ordered ONCE per input shape into the layout it wants (a plain ``conv2d`` re-orders them at every call; a
    64 -> 256 1x1 layer of ResNet-50 takes 1.1 ms instead of 4.9 ms on one core) and the activation applied inside
    the primitive. Returns None when the primitive is not in this PyTorch build or rejects the case."""
    prim = getattr(getattr(torch.ops, "mkldnn", None), "_convolution_pointwise", None)
    reorder = getattr(getattr(torch.ops, "mkldnn", None), "_reorder_convolution_weight", None)
    if prim is None or reorder is None or node.attrs.get("_cpu_fast") == "off":
        return None
    try:
        cache = node.attrs.setdefault("_cpu_packed", {})
        key = tuple(x.shape)
        if key not in cache:
            cache[key] = reorder(w, list(pad), list(strides), list(dil), group, list(x.shape))
        return prim(x, cache[key], b, list(pad), list(strides), list(dil), group, act, [], "")
    except (RuntimeError, TypeError):
        node.attrs["_cpu_fast"] = "off"
        return None


@op("FusedConv")
def _fused_conv(node, x, w, b=None, res=None):
    """Conv + bias (+ residual before/after activation) + activation; domain fdb."""
    mode = node.attr("res_mode", 0)
    act = node.attr("activation", "none")
    if act == "relu" and node.attrs.get("_cpu_fast") is True and not (res is not None and mode == 1) \
            and x.device.type == "cpu" and x.dtype == torch.float32 and w.dim() == 4 and x.dim() == 4:
        nd = 2
        strides, dil, group = node.attr("strides", [1, 1]), node.attr("dilations", [1, 1]), node.attr("group", 1)
        pads = _pads_2d(node, x, list(w.shape[2:]), strides, dil)
        if all(pads[i] == pads[nd + i] for i in range(nd)):
            y = _cpu_packed_conv(node, x, w, b, pads[:nd], strides, dil, group, "relu")
            if y is not None:
                return y + res if res is not None else y
    y = _conv(node, x, w, b)
    if res is not None and mode == 1:
        y = y + res
    y = ACTIVATIONS[act](y, node.attr("act_alpha", 0.0), node.attr("act_beta", 0.0))
    if res is not None and mode == 2:
        y = y + res
    return y


@op("ConvTranspose")
def _conv_transpose(node, x, w, b=None):
    nd = w.dim() - 2
    strides = node.attr("strides", [1] * nd)
    dil = node.attr("dilations", [1] * nd)
    group = node.attr("group", 1)
    pads = node.attr("pads", [0] * (2 * nd))
    out_pad = node.attr("output_padding", [0] * nd)
    fn = {1: F.conv_transpose1d, 2: F.conv_transpose2d, 3: F.conv_transpose3d}[nd]
    y = fn(x, w, b, stride=strides, padding=0, output_padding=out_pad, groups=group, dilation=dil)
    sl = [slice(None), slice(None)]
    for i in range(nd):
        end = y.shape[2 + i] - pads[nd + i]
        sl.append(slice(pads[i], end))
    y = y[tuple(sl)]
    if node.attr("activation", None) is not None:       # set by the deconvolution + activation fusion pass
        y = ACTIVATIONS[node.attr("activation")](y, node.attr("act_alpha", 0.0), node.attr("act_beta", 0.0))
    return y


@op("BatchNormalization")
def _bn(node, x, scale, bias, mean, var):
    eps = node.attr("epsilon", 1e-5)
    shape = [1, -1] + [1] * (x.dim() - 2)
    return (x - mean.reshape(shape)) / torch.sqrt(var.reshape(shape) + eps) * scale.reshape(shape) + bias.reshape(shape)


@op("InstanceNormalization")
def _inorm(node, x, scale, bias):
    return F.instance_norm(x, weight=scale, bias=bias, eps=node.attr("epsilon", 1e-5))


@op("LayerNormalization")
def _ln(node, x, scale=None, bias=None):
    axis = node.attr("axis", -1)
    axis = axis if axis >= 0 else x.dim() + axis
    shape = list(x.shape[axis:])
    return F.layer_norm(x, shape, scale.reshape(shape) if scale is not None else None,
                        bias.reshape(shape) if bias is not None else None, node.attr("epsilon", 1e-5))


def _pool_common(node, x, kind):
    k = node.attr("kernel_shape")
    nd = len(k)
    strides = node.attr("strides", [1] * nd)
    ceil_mode = bool(node.attr("ceil_mode", 0))
    pads = _pads_2d(node, x, k, strides)
    if kind == "max":
        x = _apply_pad_nd(x, pads, value=float("-inf"))
        fn = {1: F.max_pool1d, 2: F.max_pool2d, 3: F.max_pool3d}[nd]
        return fn(x, k, strides, 0, ceil_mode=ceil_mode)
    include = bool(node.attr("count_include_pad", 0))
    sym = all(pads[i] == pads[nd + i] for i in range(nd))
    fn = {1: F.avg_pool1d, 2: F.avg_pool2d, 3: F.avg_pool3d}[nd]
    if sym:
        return fn(x, k, strides, pads[:nd], ceil_mode=ceil_mode, count_include_pad=include)
    ones = torch.ones_like(x)
    xs = fn(_apply_pad_nd(x, pads), k, strides, 0, ceil_mode=ceil_mode) * float(np.prod(k))
    if include:
        return xs / float(np.prod(k))
    cnt = fn(_apply_pad_nd(ones, pads), k, strides, 0, ceil_mode=ceil_mode) * float(np.prod(k))
    return xs / cnt


@op("MaxPool")
def _maxpool(node, x):
    return _pool_common(node, x, "max")


@op("AveragePool")
def _avgpool(node, x):
    return _pool_common(node, x, "avg")


@op("GlobalAveragePool")
def _gap(node, x):
    return x.mean(dim=tuple(range(2, x.dim())), keepdim=True)


@op("GlobalMaxPool")
def _gmp(node, x):
    return x.amax(dim=tuple(range(2, x.dim())), keepdim=True)


@op("AdaptivePool2d")
def _adaptive_pool(node, x):
    """Paddle custom op: windows [floor(i*in/out), ceil((i+1)*in/out))
    (fastdeploy/runtime/backends/common/cuda/adaptive_pool2d_kernel.cu:20-59)."""
    size = node.attr("output_size")
    if node.attr("pooling_type", "avg") == "max":
        return F.adaptive_max_pool2d(x, size)
    return F.adaptive_avg_pool2d(x, size)


@op("Gemm")
def _gemm(node, a, b, c=None):
    if node.attr("transA", 0):
        a = a.t()
    if node.attr("transB", 0):
        b = b.t()
    y = node.attr("alpha", 1.0) * (a @ b)
    if c is not None:
        y = y + node.attr("beta", 1.0) * c
    return y


@op("FusedGemm")
def _fused_gemm(node, x, w, b=None, res=None):
    """act(x @ w^T + b) (+ residual); w is [N, K]; domain fdb."""
    y = x @ w.t()
    if b is not None:
        y = y + b
    mode = node.attr("res_mode", 0)
    if res is not None and mode == 1:
        y = y + res
    y = ACTIVATIONS[node.attr("activation", "none")](y, node.attr("act_alpha", 0.0), node.attr("act_beta", 0.0))
    if res is not None and mode == 2:
        y = y + res
    return y


@op("MatMul")
def _matmul(node, a, b):
    return torch.matmul(a, b)


@op("Attention")
def _attention(node, q, k, v, mask=None):
    """softmax(q k^T * scale + mask) v with q,k,v [B, S, heads*dh]; domain fdb.

    ``mask`` is additive, broadcastable to [B, heads, S, S] (e.g. [B,1,1,S])."""
    heads = node.attr("num_heads")
    b, s, hd = q.shape
    dh = hd // heads
    scale = node.attr("scale", 1.0 / math.sqrt(dh))

    def split(t):
        return t.reshape(b, -1, heads, dh).permute(0, 2, 1, 3)
    att = torch.matmul(split(q), split(k).transpose(-1, -2)) * scale
    if mask is not None:
        att = att + mask
    att = torch.softmax(att, dim=-1)
    return torch.matmul(att, split(v)).permute(0, 2, 1, 3).reshape(b, s, hd)


@op("PackedAttention")
def _packed_attention(node, q, k, v, seq_start, seq_len):
    """Self-attention inside each of the sequences stored back to back in ``q``/``k``/``v`` ``[1, T, heads*dh]``:
    sequence ``i`` is rows ``seq_start[i] .. seq_start[i] + seq_len[i]``; rows outside every sequence are zero;
    domain fdb."""
    heads = node.attr("num_heads")
    hd = q.shape[-1]
    dh = hd // heads
    scale = node.attr("scale", 1.0 / math.sqrt(dh))
    out = torch.zeros_like(q)
    q2, k2, v2, o2 = q.reshape(-1, hd), k.reshape(-1, hd), v.reshape(-1, hd), out.view(-1, hd)
    for st, n in zip(seq_start.reshape(-1).tolist(), seq_len.reshape(-1).tolist()):
        if n <= 0:
            continue
        def split(t):
            return t[st:st + n].reshape(n, heads, dh).permute(1, 0, 2)
        att = torch.softmax(torch.matmul(split(q2), split(k2).transpose(-1, -2)) * scale, dim=-1)
        o2[st:st + n] = torch.matmul(att, split(v2)).permute(1, 0, 2).reshape(n, hd)
    return out


@op("SelectInput")
def _select_input(node, mask, *xs):
    """Paddle ``select_input``: the operand whose index ``mask`` holds; domain fdb."""
    return xs[int(mask.reshape(-1)[0])]


@op("Loop", "If", "Scan")
def _control_flow(node, *args):
    raise RuntimeError(f"{node.op} needs the enclosing scope: it is executed by Interpreter.run, not as a free function")


@op("EmbedLayerNorm")
def _embed_ln(node, ids, *rest):
    """sum of embedding lookups followed by LayerNorm; domain fdb.

    inputs: ids_0..ids_{k-1}, table_0..table_{k-1}, gamma, beta"""
    k = node.attr("num_tables")
    id_list = [ids] + list(rest[:k - 1])
    tables = rest[k - 1:2 * k - 1]
    gamma, beta = rest[2 * k - 1], rest[2 * k]
    x = sum(F.embedding(i.long(), t) for i, t in zip(id_list, tables))
    return F.layer_norm(x, [x.shape[-1]], gamma, beta, node.attr("epsilon", 1e-5))


# ------------------------------------------------------------------------- activations / elementwise
@op("Relu")
def _relu(node, x): return torch.relu(x)
@op("Sigmoid")
def _sigmoid(node, x): return torch.sigmoid(x)
@op("Tanh")
def _tanh(node, x): return torch.tanh(x)
@op("Erf")
def _erf(node, x): return torch.erf(x)
@op("Exp")
def _exp(node, x): return torch.exp(x)
@op("Log")
def _log(node, x): return torch.log(x)
@op("Sqrt")
def _sqrt(node, x): return torch.sqrt(x)
@op("Reciprocal")
def _recip(node, x): return 1.0 / x
@op("Abs")
def _abs(node, x): return torch.abs(x)
@op("Neg")
def _neg(node, x): return -x
@op("Floor")
def _floor(node, x): return torch.floor(x)
@op("Ceil")
def _ceil(node, x): return torch.ceil(x)
@op("Round")
def _round(node, x): return torch.round(x)
@op("Sign")
def _sign(node, x): return torch.sign(x)
@op("Sin")
def _sin(node, x): return torch.sin(x)
@op("Cos")
def _cos(node, x): return torch.cos(x)
@op("Softplus")
def _softplus(node, x): return F.softplus(x)
@op("Softsign")
def _softsign(node, x): return F.softsign(x)
@op("Mish")
def _mish(node, x): return F.mish(x)
@op("Identity", "Dropout")
def _identity(node, x, *_): return x
@op("Not")
def _not(node, x): return ~x
@op("Gelu")
def _gelu(node, x): return F.gelu(x, approximate="tanh" if node.attr("approximate", "none") == "tanh" else "none")
@op("Silu", "Swish")
def _silu(node, x): return F.silu(x)
@op("HardSwish")
def _hswish(node, x): return F.hardswish(x)


@op("LeakyRelu")
def _leaky(node, x): return F.leaky_relu(x, node.attr("alpha", 0.01))


@op("Elu")
def _elu(node, x): return F.elu(x, node.attr("alpha", 1.0))


@op("Selu")
def _selu(node, x):
    a, g = node.attr("alpha", 1.6732632), node.attr("gamma", 1.0507010)
    return g * torch.where(x > 0, x, a * (torch.exp(x) - 1))


@op("PRelu")
def _prelu(node, x, slope):
    return torch.where(x > 0, x, x * slope)


@op("HardSigmoid")
def _hsigmoid(node, x):
    return torch.clamp(node.attr("alpha", 0.2) * x + node.attr("beta", 0.5), 0, 1)


@op("Clip")
def _clip(node, x, lo=None, hi=None):
    lo_v = float(lo) if lo is not None else node.attr("min", None)
    hi_v = float(hi) if hi is not None else node.attr("max", None)
    return torch.clamp(x, lo_v, hi_v)


def _binary(fn):
    def run(node, a, b):
        if a.dtype != b.dtype and a.is_floating_point() != b.is_floating_point():
            tgt = a.dtype if a.is_floating_point() else b.dtype
            a, b = a.to(tgt), b.to(tgt)
        return fn(a, b)
    return run


_OPS["Add"] = _binary(torch.add)
_OPS["Sub"] = _binary(torch.sub)
_OPS["Mul"] = _binary(torch.mul)
_OPS["Pow"] = _binary(torch.pow)
_OPS["Equal"] = _binary(torch.eq)
_OPS["Less"] = _binary(torch.lt)
_OPS["Greater"] = _binary(torch.gt)
_OPS["LessOrEqual"] = _binary(torch.le)
_OPS["GreaterOrEqual"] = _binary(torch.ge)
_OPS["And"] = _binary(torch.logical_and)
_OPS["Or"] = _binary(torch.logical_or)
_OPS["Xor"] = _binary(torch.logical_xor)


@op("Div")
def _div(node, a, b):
    if not a.is_floating_point() and not b.is_floating_point():
        return torch.div(a, b, rounding_mode="trunc")
    return a / b


@op("Mod")
def _mod(node, a, b):
    return torch.fmod(a, b) if node.attr("fmod", 0) else torch.remainder(a, b)


@op("Max")
def _max(node, *xs):
    y = xs[0]
    for x in xs[1:]:
        y = torch.maximum(y, x)
    return y


@op("Min")
def _min(node, *xs):
    y = xs[0]
    for x in xs[1:]:
        y = torch.minimum(y, x)
    return y


@op("Sum")
def _sum(node, *xs):
    y = xs[0]
    for x in xs[1:]:
        y = y + x
    return y


@op("Where")
def _where(node, c, a, b): return torch.where(c, a, b)


@op("Softmax")
def _softmax(node, x):
    axis = node.attr("axis", -1 if node.attr("_opset", 13) >= 13 else 1)
    if node.attr("_opset", 13) < 13 and axis not in (-1, x.dim() - 1):
        shape = x.shape
        flat = x.reshape(int(np.prod(shape[:axis])), -1)
        return torch.softmax(flat, dim=1).reshape(shape)
    return torch.softmax(x, dim=axis)


@op("LogSoftmax")
def _logsoftmax(node, x): return torch.log_softmax(x, dim=node.attr("axis", -1))


# ------------------------------------------------------------------------- shape ops
@op("Reshape")
def _reshape(node, x, shape):
    tgt = _ints(shape)
    if not node.attr("allowzero", 0):
        tgt = [x.shape[i] if d == 0 else d for i, d in enumerate(tgt)]
    return x.reshape(tgt)


@op("Flatten")
def _flatten(node, x):
    axis = node.attr("axis", 1)
    axis = axis if axis >= 0 else x.dim() + axis
    lead = int(np.prod(x.shape[:axis])) if axis > 0 else 1
    return x.reshape(lead, -1)


@op("Transpose")
def _transpose(node, x):
    perm = node.attr("perm", list(reversed(range(x.dim()))))
    return x.permute(perm)


@op("Squeeze")
def _squeeze(node, x, axes=None):
    ax = _ints(axes) if axes is not None else node.attr("axes", None)
    if ax is None:
        return x.squeeze()
    for a in sorted([a if a >= 0 else x.dim() + a for a in ax], reverse=True):
        x = x.squeeze(a)
    return x


@op("Unsqueeze")
def _unsqueeze(node, x, axes=None):
    ax = _ints(axes) if axes is not None else node.attr("axes")
    out_rank = x.dim() + len(ax)
    for a in sorted([a if a >= 0 else out_rank + a for a in ax]):
        x = x.unsqueeze(a)
    return x


@op("Concat")
def _concat(node, *xs):
    xs = [x for x in xs if x.numel() > 0 or x.dim() > 1]
    dt = xs[0].dtype
    return torch.cat([x.to(dt) for x in xs], dim=node.attr("axis", 0))


@op("Split")
def _split(node, x, split=None):
    axis = node.attr("axis", 0)
    sizes = _ints(split) if split is not None else node.attr("split", None)
    n_out = len(node.outputs)
    if sizes is None:
        sizes = [x.shape[axis] // n_out] * n_out
    return tuple(torch.split(x, sizes, dim=axis))


@op("Slice")
def _slice(node, x, starts=None, ends=None, axes=None, steps=None):
    st = _ints(starts) if starts is not None else node.attr("starts")
    en = _ints(ends) if ends is not None else node.attr("ends")
    ax = _ints(axes) if axes is not None else node.attr("axes", list(range(len(st))))
    sp = _ints(steps) if steps is not None else [1] * len(st)
    sl = [slice(None)] * x.dim()
    flips = []
    for s, e, a, p in zip(st, en, ax, sp):
        a = a if a >= 0 else x.dim() + a
        dim = x.shape[a]
        if p > 0:
            s = max(s + dim, 0) if s < 0 else min(s, dim)
            e = max(e + dim, 0) if e < 0 else min(e, dim)
            sl[a] = slice(s, e, p)
        else:
            s = s + dim if s < 0 else min(s, dim - 1)
            e = e + dim if -dim <= e < 0 else (-1 if e < -dim else min(e, dim - 1))
            idx = torch.arange(s, e, p, device=x.device)
            x = x.index_select(a, idx)
            flips.append(a)
    return x[tuple(sl)]


@op("Gather")
def _gather(node, x, idx):
    axis = node.attr("axis", 0)
    axis = axis if axis >= 0 else x.dim() + axis
    idx = idx.long()
    idx = torch.where(idx < 0, idx + x.shape[axis], idx)
    out = x.index_select(axis, idx.flatten())
    return out.reshape(list(x.shape[:axis]) + list(idx.shape) + list(x.shape[axis + 1:]))


@op("GatherND")
def _gather_nd(node, x, idx):
    idx = idx.long()
    k = idx.shape[-1]
    flat = idx.reshape(-1, k)
    out = x[tuple(flat[:, i] for i in range(k))]
    return out.reshape(list(idx.shape[:-1]) + list(x.shape[k:]))


@op("GatherElements")
def _gather_el(node, x, idx): return torch.gather(x, node.attr("axis", 0), idx.long())


@op("ScatterND")
def _scatter_nd(node, x, idx, upd):
    y = x.clone()
    idx = idx.long()
    k = idx.shape[-1]
    flat = idx.reshape(-1, k)
    where = tuple(flat[:, i] for i in range(k))
    upd = upd.reshape([-1] + list(x.shape[k:])).to(x.dtype)
    if node.attr("reduction", "none") == "add":
        y.index_put_(where, upd, accumulate=True)
    else:
        y[where] = upd
    return y


@op("Shape")
def _shape(node, x): return torch.tensor(list(x.shape), dtype=torch.int64)


@op("Size")
def _size(node, x): return torch.tensor(x.numel(), dtype=torch.int64)


@op("Cast")
def _cast(node, x): return x.to(ONNX_DT2TORCH[node.attr("to")])


@op("ConstantOfShape")
def _const_of_shape(node, shape):
    v = node.attr("value", None)
    if v is None:
        return torch.zeros(_ints(shape), dtype=torch.float32)
    t = torch.from_numpy(np.asarray(v))
    return torch.full(_ints(shape), t.flatten()[0].item(), dtype=t.dtype)


@op("Expand")
def _expand(node, x, shape):
    tgt = _ints(shape)
    rank = max(len(tgt), x.dim())
    xs = [1] * (rank - x.dim()) + list(x.shape)
    tgt = [1] * (rank - len(tgt)) + tgt
    out = [max(a, b) if b != -1 else a for a, b in zip(xs, tgt)]
    return x.reshape(xs).expand(out)


@op("Tile")
def _tile(node, x, reps): return x.repeat(_ints(reps))


@op("Range")
def _range(node, start, limit, delta):
    return torch.arange(start.item(), limit.item(), delta.item(), dtype=start.dtype)


@op("Pad")
def _pad(node, x, pads=None, value=None):
    p = _ints(pads) if pads is not None else node.attr("pads")
    mode = node.attr("mode", "constant")
    v = float(value) if value is not None and value.numel() else node.attr("value", 0.0)
    nd = len(p) // 2
    tp = []
    for i in reversed(range(nd)):
        tp += [p[i], p[nd + i]]
    if mode == "constant":
        return F.pad(x, tp, value=v)
    while len(tp) > 2 and tp[-1] == 0 and tp[-2] == 0:   # torch wants only the padded trailing dims
        tp = tp[:-2]
    return F.pad(x, tp, mode="reflect" if mode == "reflect" else "replicate")


def _reduce(fn, default_keep=1):
    def run(node, x, axes=None):
        ax = _ints(axes) if axes is not None else node.attr("axes", None)
        keep = bool(node.attr("keepdims", default_keep))
        if ax is None or len(ax) == 0:
            ax = list(range(x.dim()))
        return fn(x, tuple(ax), keep)
    return run


_OPS["ReduceMean"] = _reduce(lambda x, a, k: x.mean(dim=a, keepdim=k))
_OPS["ReduceSum"] = _reduce(lambda x, a, k: x.sum(dim=a, keepdim=k))
_OPS["ReduceMax"] = _reduce(lambda x, a, k: x.amax(dim=a, keepdim=k))
_OPS["ReduceMin"] = _reduce(lambda x, a, k: x.amin(dim=a, keepdim=k))
_OPS["ReduceProd"] = _reduce(lambda x, a, k: _prod(x, a, k))
_OPS["ReduceL2"] = _reduce(lambda x, a, k: torch.sqrt((x * x).sum(dim=a, keepdim=k)))
_OPS["ReduceL1"] = _reduce(lambda x, a, k: x.abs().sum(dim=a, keepdim=k))
_OPS["ReduceLogSumExp"] = _reduce(lambda x, a, k: torch.logsumexp(x, dim=a, keepdim=k))
_OPS["ReduceSumSquare"] = _reduce(lambda x, a, k: (x * x).sum(dim=a, keepdim=k))


def _prod(x, axes, keep):
    for a in sorted([a if a >= 0 else x.dim() + a for a in axes], reverse=True):
        x = x.prod(dim=a, keepdim=keep)
    return x


@op("ArgMax")
def _argmax(node, x):
    return torch.argmax(x, dim=node.attr("axis", 0), keepdim=bool(node.attr("keepdims", 1)))


@op("ArgMin")
def _argmin(node, x):
    return torch.argmin(x, dim=node.attr("axis", 0), keepdim=bool(node.attr("keepdims", 1)))


@op("TopK")
def _topk(node, x, k):
    v, i = torch.topk(x, int(k.flatten()[0]), dim=node.attr("axis", -1), largest=bool(node.attr("largest", 1)),
                      sorted=True)
    return v, i


@op("CumSum")
def _cumsum(node, x, axis):
    return torch.cumsum(x, dim=int(axis))


@op("NonZero")
def _nonzero(node, x): return torch.nonzero(x).t().contiguous()


@op("OneHot")
def _onehot(node, idx, depth, values):
    d = int(depth.flatten()[0])
    oh = F.one_hot(idx.long() % d, d).to(values.dtype)
    return oh * (values[1] - values[0]) + values[0]


@op("Resize", "Upsample")
def _resize(node, x, *rest):
    roi = scales = sizes = None
    if node.op == "Upsample":
        scales = rest[0] if rest else None
    else:
        if len(rest) >= 1: roi = rest[0]
        if len(rest) >= 2: scales = rest[1]
        if len(rest) >= 3: sizes = rest[2]
    mode = node.attr("mode", "nearest")
    ctm = node.attr("coordinate_transformation_mode", "half_pixel")
    nd = x.dim() - 2
    if sizes is not None and sizes.numel():
        out = _ints(sizes)[2:]
    else:
        sc = [float(v) for v in scales.flatten().tolist()] if scales is not None and scales.numel() else \
            node.attr("scales")
        out = [int(math.floor(x.shape[2 + i] * sc[2 + i])) for i in range(nd)]
    if mode == "nearest":
        if ctm == "asymmetric" and node.attr("nearest_mode", "round_prefer_floor") == "floor":
            idx = []
            y = x
            for i in range(nd):
                src = (torch.arange(out[i]) * (x.shape[2 + i] / out[i])).floor().long().clamp(max=x.shape[2 + i] - 1)
                y = y.index_select(2 + i, src.to(x.device))
            return y
        return F.interpolate(x, size=out, mode="nearest")
    tmode = {1: "linear", 2: "bilinear", 3: "trilinear"}[nd] if mode == "linear" else "bicubic"
    if ctm == "align_corners":
        return F.interpolate(x, size=out, mode=tmode, align_corners=True)
    if ctm == "asymmetric" and nd == 2 and mode == "linear":
        return _resize_asymmetric_linear(x, out)
    return F.interpolate(x, size=out, mode=tmode, align_corners=False)


def _resize_asymmetric_linear(x, out):
    n, c, h, w = x.shape
    ys = torch.arange(out[0], dtype=torch.float32, device=x.device) * (h / out[0])
    xs = torch.arange(out[1], dtype=torch.float32, device=x.device) * (w / out[1])
    y0 = ys.floor().long().clamp(max=h - 1); y1 = (y0 + 1).clamp(max=h - 1); fy = (ys - y0).view(1, 1, -1, 1)
    x0 = xs.floor().long().clamp(max=w - 1); x1 = (x0 + 1).clamp(max=w - 1); fx = (xs - x0).view(1, 1, 1, -1)
    top = x[:, :, y0][:, :, :, x0] * (1 - fx) + x[:, :, y0][:, :, :, x1] * fx
    bot = x[:, :, y1][:, :, :, x0] * (1 - fx) + x[:, :, y1][:, :, :, x1] * fx
    return top * (1 - fy) + bot * fy


@op("DepthToSpace")
def _d2s(node, x):
    b = node.attr("blocksize")
    if node.attr("mode", "DCR") == "CRD":
        return F.pixel_shuffle(x, b)
    n, c, h, w = x.shape
    return x.reshape(n, b, b, c // (b * b), h, w).permute(0, 3, 4, 1, 5, 2).reshape(n, c // (b * b), h * b, w * b)


@op("MultiClassNMS")
def _mc_nms(node, boxes, scores):
    """Paddle ``multiclass_nms3`` as exported for ONNX Runtime
    (fastdeploy/runtime/backends/ort/ops/multiclass_nms.cc:86-284): outputs Out [K,6], Index [K,1], NmsRoisNum [N]."""
    from ..ops.nms import multiclass_nms_reference
    out, idx, num = multiclass_nms_reference(
        boxes.float().cpu().numpy(), scores.float().cpu().numpy(), node.attr("score_threshold", 0.01),
        node.attr("nms_threshold", 0.5), node.attr("nms_top_k", 1000), node.attr("keep_top_k", 100),
        bool(node.attr("normalized", 1)), node.attr("background_label", -1), node.attr("nms_eta", 1.0))
    return (torch.from_numpy(out), torch.from_numpy(idx.astype(np.int64)).reshape(-1, 1),
            torch.from_numpy(num.astype(np.int32)))


@op("PPYOLOEPost")
def _ppyoloe_post(node, *args):
    """DFL integral + distance->box + stride + scale-factor division + multiclass NMS; domain fdb.

    inputs: cls_0..cls_{L-1} [b,C,H,W] (scores), reg_0..reg_{L-1} [b,4*bins,H,W] (logits), scale_factor [b,2]"""
    nl = node.attr("num_levels")
    cls, reg, sf = args[:nl], args[nl:2 * nl], args[2 * nl]
    bins = node.attr("bins")
    boxes, scores = [], []
    for i in range(nl):
        b, c, h, w = cls[i].shape
        scores.append(cls[i].float().reshape(b, c, h * w))
        r = reg[i].float().reshape(b, 4, bins, h * w).permute(0, 3, 1, 2)          # [b, l, 4, bins]
        dist = (torch.softmax(r, -1) * torch.arange(bins, dtype=torch.float32, device=r.device)).sum(-1)
        ys, xs = torch.meshgrid(torch.arange(h, device=r.device) + node.attr("offset", 0.5),
                                torch.arange(w, device=r.device) + node.attr("offset", 0.5), indexing="ij")
        pts = torch.stack([xs.reshape(-1), ys.reshape(-1)], -1).float()
        bx = torch.cat([pts - dist[..., :2], pts + dist[..., 2:]], -1) * float(node.attr("strides")[i])
        boxes.append(bx)
    boxes = torch.cat(boxes, 1)
    sf = sf.float()
    boxes = boxes / torch.stack([sf[:, 1], sf[:, 0], sf[:, 1], sf[:, 0]], -1)[:, None, :]
    return _mc_nms(node, boxes, torch.cat(scores, 2))


@op("LSTM")
def _lstm(node, x, w, r, b=None, seq_lens=None, h0=None, c0=None, *_):
    """Single-layer forward/bidirectional LSTM, ONNX gate order i,o,f,c."""
    hidden = node.attr("hidden_size")
    ndir = w.shape[0]
    seq, batch, _ = x.shape
    ys, hs, cs = [], [], []
    for d in range(ndir):
        wi, ri = w[d], r[d]
        bi = b[d] if b is not None else torch.zeros(8 * hidden)
        h = h0[d] if h0 is not None else torch.zeros(batch, hidden)
        c = c0[d] if c0 is not None else torch.zeros(batch, hidden)
        steps = range(seq) if d == 0 else reversed(range(seq))
        out = [None] * seq
        for t in steps:
            g = x[t] @ wi.t() + h @ ri.t() + bi[:4 * hidden] + bi[4 * hidden:]
            i, o, f, cc = g.split(hidden, dim=1)
            c = torch.sigmoid(f) * c + torch.sigmoid(i) * torch.tanh(cc)
            h = torch.sigmoid(o) * torch.tanh(c)
            out[t] = h
        ys.append(torch.stack(out))
        hs.append(h)
        cs.append(c)
    return torch.stack(ys, dim=1), torch.stack(hs), torch.stack(cs)


# ------------------------------------------------------------------------- driver
class Interpreter:
    """Executes a :class:`Graph` node by node with torch tensors on ``device``."""

    def __init__(self, graph: Graph, device: str = "cpu", channels_last: bool = False):
        """``channels_last``: on the CPU, 4-D fp32 weights and inputs are held channel-innermost, the layout in which
        the vendor convolution primitives run without re-ordering their operands at every call (same values, same
        logical shapes; a 3x3 layer of ResNet-50 takes 1.9 ms instead of 3.1 ms on one core)."""
        self.graph = graph
        self.device = torch.device(device)
        self.channels_last = bool(channels_last) and self.device.type == "cpu"
        if self.channels_last:
            for n in graph.nodes:
                if n.op in ("Conv", "FusedConv"):
                    n.attrs["_cpu_fast"] = True
        missing = sorted({n.op for n in graph.nodes if n.op not in _OPS})
        if missing:
            raise NotImplementedError(f"interpreter: unsupported ops {missing}")
        self.consts = {}
        for k, v in graph.initializers.items():
            t = torch.from_numpy(np.ascontiguousarray(v))
            # half-precision weights are computed in fp32 (this is the reference path) unless the graph was
            # converted to fp16 on purpose, in which case it carries its own casts
            keep_half = str(graph.metadata.get("converted_fp16", "")) == "1"
            if t.dtype == torch.float64 or (t.dtype == torch.float16 and not keep_half):
                t = t.float()
            if self.channels_last and t.dim() == 4 and t.dtype == torch.float32:
                t = t.contiguous(memory_format=torch.channels_last)
            self.consts[k] = t.to(self.device)

    # ------------------------------------------------------------------ execution
    def _exec(self, nodes, env, opset: int) -> None:
        for node in nodes:
            if node.op in ("Loop", "If", "Scan"):
                res = self._control(node, env, opset)
            else:
                args = [env[i] for i in node.inputs]
                while args and args[-1] is None:
                    args.pop()
                node.attrs.setdefault("_opset", opset)
                res = _OPS[node.op](node, *args)
            if not isinstance(res, tuple):
                res = (res,)
            for name, val in zip(node.outputs, res):
                if name:
                    env[name] = val

    def _body_env(self, body: Graph, outer) -> "collections.ChainMap":
        import collections
        local = {}
        for k, v in body.initializers.items():
            t = torch.from_numpy(np.ascontiguousarray(v))
            local[k] = (t.float() if t.dtype in (torch.float16, torch.float64) else t).to(self.device)
        return collections.ChainMap(local, outer)

    def _control(self, node: Node, env, opset: int):
        """ONNX ``Loop`` / ``If``: the body graphs read this scope by name (a ChainMap keeps their writes local)."""
        if node.op == "If":
            cond = bool(env[node.inputs[0]].reshape(-1)[0])
            body = node.attr("then_branch") if cond else node.attr("else_branch")
            scope = self._body_env(body, env)
            self._exec(body.nodes, scope, opset)
            return tuple(scope[v.name] for v in body.outputs)
        if node.op == "Scan":
            return self._scan(node, env, opset)
        body = node.attr("body")
        m = env[node.inputs[0]] if node.inputs[0] else None
        cond_t = env[node.inputs[1]] if len(node.inputs) > 1 and node.inputs[1] else None
        carried = [env[i] for i in node.inputs[2:]]
        n_carried = len(carried)
        trips = int(m.reshape(-1)[0]) if m is not None else None
        keep_going = bool(cond_t.reshape(-1)[0]) if cond_t is not None else True
        scans = [[] for _ in range(len(body.outputs) - 1 - n_carried)]
        it = 0
        limit = int(node.attr("max_iterations", 1 << 20))          # a bound on runaway loops, not an ONNX attribute
        while keep_going and (trips is None or it < trips):
            if it >= limit:
                raise RuntimeError(f"Loop {node.name!r} ran {limit} iterations without its condition turning false")
            scope = self._body_env(body, env)
            scope[body.inputs[0].name] = torch.tensor(it, dtype=torch.int64, device=self.device)
            scope[body.inputs[1].name] = torch.tensor(keep_going, device=self.device)
            for vi, val in zip(body.inputs[2:], carried):
                scope[vi.name] = val
            self._exec(body.nodes, scope, opset)
            outs = [scope[v.name] for v in body.outputs]
            keep_going = bool(outs[0].reshape(-1)[0])
            carried = outs[1:1 + n_carried]
            for k, s in enumerate(outs[1 + n_carried:]):
                scans[k].append(s)
            it += 1
        stacked = [torch.stack(s) if s else torch.zeros(0, device=self.device) for s in scans]
        return tuple(carried) + tuple(stacked)

    def _scan(self, node: Node, env, opset: int):
        """ONNX ``Scan`` (opset 9+): ``N`` state values and ``M`` scanned inputs; the body maps
        ``(states..., slices...)`` to ``(states..., output slices...)``; the slices of every scan output are stacked."""
        body = node.attr("body")
        m = int(node.attr("num_scan_inputs"))
        args = [env[i] for i in node.inputs]
        n = len(args) - m
        states, scans = args[:n], args[n:]
        in_axes = node.attr("scan_input_axes", [0] * m)
        in_dirs = node.attr("scan_input_directions", [0] * m)
        k_out = len(body.outputs) - n
        out_axes = node.attr("scan_output_axes", [0] * k_out)
        out_dirs = node.attr("scan_output_directions", [0] * k_out)
        steps = scans[0].shape[in_axes[0]] if scans else 0
        collected = [[] for _ in range(k_out)]
        for t in range(steps):
            scope = self._body_env(body, env)
            for vi, val in zip(body.inputs[:n], states):
                scope[vi.name] = val
            for j, (vi, val) in enumerate(zip(body.inputs[n:], scans)):
                idx = steps - 1 - t if in_dirs[j] else t
                scope[vi.name] = val.select(in_axes[j], idx)
            self._exec(body.nodes, scope, opset)
            outs = [scope[v.name] for v in body.outputs]
            states = outs[:n]
            for j, o in enumerate(outs[n:]):
                collected[j].append(o)
        stacked = []
        for j, parts in enumerate(collected):
            if out_dirs[j]:
                parts = parts[::-1]
            stacked.append(torch.stack(parts, dim=out_axes[j]) if parts else torch.zeros(0, device=self.device))
        return tuple(states) + tuple(stacked)

    def run(self, feeds: Dict[str, "np.ndarray | torch.Tensor"], outputs: Optional[Sequence[str]] = None,
            keep_all: bool = False) -> Dict[str, torch.Tensor]:
        env: Dict[str, Optional[torch.Tensor]] = dict(self.consts)
        env[""] = None
        for vi in self.graph.inputs:
            if vi.name not in feeds:
                raise KeyError(f"missing input {vi.name!r}")
            t = feeds[vi.name]
            t = torch.from_numpy(np.ascontiguousarray(t)) if isinstance(t, np.ndarray) else t
            # the reference path computes in fp32; a graph converted to fp16 takes the dtype it declares
            if str(self.graph.metadata.get("converted_fp16", "")) == "1":
                t = t.to(NP2TORCH.get(vi.dtype, t.dtype)) if t.is_floating_point() else t
            elif t.dtype in (torch.float16, torch.bfloat16, torch.float64):
                t = t.float()
            t = t.to(self.device)
            if self.channels_last and t.dim() == 4 and t.dtype == torch.float32:
                t = t.contiguous(memory_format=torch.channels_last)
            env[vi.name] = t
        opset = self.graph.opset
        with torch.no_grad():
            self._exec(self.graph.nodes, env, opset)
        names = list(outputs) if outputs is not None else self.graph.output_names()
        if keep_all:
            return {k: v for k, v in env.items() if v is not None}
        return {n: env[n] for n in names}


from . import interp_extra  # noqa: E402,F401  (registers the second batch of operators)
from . import interp_onnx_more  # noqa: E402,F401  (the rest of the standard ONNX operator set)
