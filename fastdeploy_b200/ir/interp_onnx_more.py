"""The rest of the standard ONNX operator set in the interpreter: quantised linear algebra (QLinearConv,
QLinearMatMul, ConvInteger, MatMulInteger, DynamicQuantizeLinear - what ONNX Runtime's int8 models are made of,
fastdeploy/runtime/backends/ort/ort_backend.cc:391), NonMaxSuppression, Einsum, recurrent layers (RNN, GRU), and
the smaller tensor, pooling, normalisation and random operators. Semantics follow the ONNX operator definitions;
each is the fp32 reference on the CPU path and the oracle for anything lowered natively later.
"""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn.functional as F

from .interp import ONNX_DT2TORCH, _ints, op


# --------------------------------------------------------------------------------------------- small tensor operators
@op("IsNaN")
def _isnan(node, x):
    return torch.isnan(x)


@op("IsInf")
def _isinf(node, x):
    pos, neg = node.attr("detect_positive", 1), node.attr("detect_negative", 1)
    out = torch.zeros_like(x, dtype=torch.bool)
    if pos:
        out |= x == float("inf")
    if neg:
        out |= x == float("-inf")
    return out


@op("Mean")
def _mean(node, *xs):
    out = xs[0]
    for t in xs[1:]:
        out = out + t
    return out / len(xs)


@op("Celu")
def _celu(node, x):
    return F.celu(x, alpha=node.attr("alpha", 1.0))


@op("Hardmax")
def _hardmax(node, x):
    axis = node.attr("axis", -1)
    idx = torch.argmax(x, dim=axis, keepdim=True)            # the first maximum
    return torch.zeros_like(x).scatter_(axis, idx, 1.0)


@op("EyeLike")
def _eyelike(node, x):
    dt = ONNX_DT2TORCH[node.attr("dtype")] if node.attr("dtype") is not None else x.dtype
    n, m, k = x.shape[0], x.shape[1], node.attr("k", 0)
    out = torch.zeros(n, m, dtype=dt)
    rows = torch.arange(n)
    cols = rows + k
    ok = (cols >= 0) & (cols < m)
    out[rows[ok], cols[ok]] = 1
    return out


@op("Constant")
def _constant(node):
    """Normally hoisted into the initializers by the ONNX reader; kept for graphs built by hand."""
    v = node.attr("value")
    if v is not None:
        return torch.from_numpy(np.ascontiguousarray(v))
    for key, dt in (("value_float", torch.float32), ("value_int", torch.int64)):
        if node.attr(key) is not None:
            return torch.tensor(node.attr(key), dtype=dt)
    for key, dt in (("value_floats", torch.float32), ("value_ints", torch.int64)):
        if node.attr(key) is not None:
            return torch.tensor(list(node.attr(key)), dtype=dt)
    raise ValueError("Constant without a value")


@op("Trilu")
def _trilu(node, x, k=None):
    kk = int(k.reshape(-1)[0]) if k is not None else 0
    return torch.triu(x, kk) if node.attr("upper", 1) else torch.tril(x, kk)


@op("BitShift")
def _bitshift(node, x, y):
    return torch.bitwise_left_shift(x, y) if node.attr("direction") == "LEFT" else torch.bitwise_right_shift(x, y)


@op("Det")
def _det(node, x):
    return torch.linalg.det(x)


@op("Compress")
def _compress(node, x, cond):
    axis = node.attr("axis", None)
    keep = torch.nonzero(cond.reshape(-1).bool()).reshape(-1)
    if axis is None:
        return x.reshape(-1)[keep[keep < x.numel()]]
    return torch.index_select(x, axis, keep[keep < x.shape[axis]])


@op("ReverseSequence")
def _reverse_sequence(node, x, lens):
    b_axis, t_axis = node.attr("batch_axis", 1), node.attr("time_axis", 0)
    out = x.clone()
    for b, n in enumerate(lens.reshape(-1).tolist()):
        src = x.select(b_axis, b)
        t = t_axis if t_axis < b_axis else t_axis - 1
        seg = src.narrow(t, 0, int(n)).flip(t)
        out.select(b_axis, b).narrow(t, 0, int(n)).copy_(seg)
    return out


@op("ScatterElements", "Scatter")
def _scatter_elements(node, x, idx, upd):
    axis = node.attr("axis", 0)
    idx = torch.where(idx < 0, idx + x.shape[axis], idx).long()
    red = node.attr("reduction", "none")
    out = x.clone()
    if red == "none":
        return out.scatter_(axis, idx, upd)
    how = {"add": "sum", "mul": "prod", "max": "amax", "min": "amin"}[red]
    return out.scatter_reduce_(axis, idx, upd, how, include_self=True)


@op("SpaceToDepth")
def _space_to_depth(node, x):
    bs = node.attr("blocksize")
    n, c, h, w = x.shape
    t = x.reshape(n, c, h // bs, bs, w // bs, bs).permute(0, 3, 5, 1, 2, 4)
    return t.reshape(n, c * bs * bs, h // bs, w // bs)


@op("ConcatFromSequence")
def _concat_from_sequence(node, *xs):
    axis = node.attr("axis", 0)
    return torch.stack(xs, dim=axis) if node.attr("new_axis", 0) else torch.cat(xs, dim=axis)


# --------------------------------------------------------------------------------------------- pooling / normalisation
@op("LRN")
def _lrn(node, x):
    return F.local_response_norm(x, node.attr("size"), alpha=node.attr("alpha", 1e-4), beta=node.attr("beta", 0.75),
                                 k=node.attr("bias", 1.0))


@op("LpNormalization")
def _lp_normalization(node, x):
    p, axis = node.attr("p", 2), node.attr("axis", -1)
    n = torch.linalg.vector_norm(x, ord=p, dim=axis, keepdim=True)
    return x / torch.where(n == 0, torch.ones_like(n), n)


@op("MeanVarianceNormalization")
def _mvn(node, x):
    axes = node.attr("axes", [0, 2, 3])
    mean = x.mean(dim=axes, keepdim=True)
    var = ((x - mean) ** 2).mean(dim=axes, keepdim=True)
    return (x - mean) / torch.sqrt(var + 1e-9)


@op("LpPool")
def _lp_pool(node, x):
    p = node.attr("p", 2)
    k = node.attr("kernel_shape")
    strides = node.attr("strides", [1] * len(k))
    pads = node.attr("pads", [0] * (2 * len(k)))
    xp = F.pad(x.abs() ** p, [pads[1], pads[3], pads[0], pads[2]] if len(k) == 2 else [pads[0], pads[1]])
    pooled = F.avg_pool2d(xp, k, strides) * (k[0] * k[1]) if len(k) == 2 else F.avg_pool1d(xp, k[0], strides[0]) * k[0]
    return pooled ** (1.0 / p)


@op("GlobalLpPool")
def _global_lp_pool(node, x):
    p = node.attr("p", 2)
    dims = list(range(2, x.dim()))
    return (x.abs() ** p).sum(dim=dims, keepdim=True) ** (1.0 / p)


@op("ReduceLogSum")
def _reduce_log_sum(node, x, axes=None):
    ax = _ints(axes) if axes is not None else node.attr("axes", None)
    keep = bool(node.attr("keepdims", 1))
    s = x.sum(dim=tuple(ax), keepdim=keep) if ax else x.sum().reshape([1] * x.dim() if keep else [])
    return torch.log(s)


@op("MaxUnpool")
def _max_unpool(node, x, idx, out_shape=None):
    k, strides = node.attr("kernel_shape"), node.attr("strides", None)
    pads = node.attr("pads", [0] * (2 * len(k)))
    size = _ints(out_shape) if out_shape is not None else None
    n, c = x.shape[:2]
    if size is None:
        st = strides or k
        size = [n, c] + [(x.shape[2 + d] - 1) * st[d] - pads[d] - pads[len(k) + d] + k[d] for d in range(len(k))]
    out = torch.zeros(size, dtype=x.dtype).reshape(-1)
    out[idx.reshape(-1).long()] = x.reshape(-1)               # ONNX indices are flat over the whole output tensor
    return out.reshape(size)


@op("MaxRoiPool")
def _max_roi_pool(node, x, rois):
    ph, pw = node.attr("pooled_shape")
    scale = node.attr("spatial_scale", 1.0)
    out = torch.zeros(rois.shape[0], x.shape[1], ph, pw, dtype=x.dtype)
    h, w = x.shape[2], x.shape[3]
    for r in range(rois.shape[0]):
        b, x1, y1, x2, y2 = [float(v) for v in rois[r]]
        x1, y1, x2, y2 = [int(round(v * scale)) for v in (x1, y1, x2, y2)]
        rw, rh = max(x2 - x1 + 1, 1), max(y2 - y1 + 1, 1)
        for i in range(ph):
            for j in range(pw):
                hs, he = int(math.floor(i * rh / ph)) + y1, int(math.ceil((i + 1) * rh / ph)) + y1
                ws, we = int(math.floor(j * rw / pw)) + x1, int(math.ceil((j + 1) * rw / pw)) + x1
                hs, he, ws, we = max(hs, 0), min(he, h), max(ws, 0), min(we, w)
                if he > hs and we > ws:
                    out[r, :, i, j] = x[int(b), :, hs:he, ws:we].amax(dim=(1, 2))
    return out


# --------------------------------------------------------------------------------------------- Einsum / NMS
@op("Einsum")
def _einsum(node, *xs):
    return torch.einsum(node.attr("equation"), *xs)


@op("NonMaxSuppression")
def _onnx_nms(node, boxes, scores, max_out=None, iou_thr=None, score_thr=None):
    """boxes [N, M, 4], scores [N, C, M] -> selected [K, 3] = (batch, class, box), per (batch, class) greedy over
    descending scores; ``center_point_box`` = 1 reads (cx, cy, w, h), else two opposite corners in any order."""
    limit = int(max_out.reshape(-1)[0]) if max_out is not None and max_out.numel() else 0
    iou_t = float(iou_thr.reshape(-1)[0]) if iou_thr is not None and iou_thr.numel() else 0.0
    sc_t = float(score_thr.reshape(-1)[0]) if score_thr is not None and score_thr.numel() else None
    if limit == 0:
        return torch.zeros(0, 3, dtype=torch.int64)
    b = boxes.float()
    if node.attr("center_point_box", 0):
        cx, cy, w, h = b.unbind(-1)
        x1, y1, x2, y2 = cx - w / 2, cy - h / 2, cx + w / 2, cy + h / 2
    else:
        y1, x1 = torch.minimum(b[..., 0], b[..., 2]), torch.minimum(b[..., 1], b[..., 3])
        y2, x2 = torch.maximum(b[..., 0], b[..., 2]), torch.maximum(b[..., 1], b[..., 3])
    area = (x2 - x1) * (y2 - y1)
    picked = []
    for n in range(scores.shape[0]):
        for c in range(scores.shape[1]):
            s = scores[n, c]
            order = torch.argsort(s, descending=True, stable=True).tolist()
            kept = []
            for i in order:
                if sc_t is not None and float(s[i]) <= sc_t:
                    break
                ok = True
                for j in kept:
                    iw = max(0.0, float(min(x2[n, i], x2[n, j]) - max(x1[n, i], x1[n, j])))
                    ih = max(0.0, float(min(y2[n, i], y2[n, j]) - max(y1[n, i], y1[n, j])))
                    inter = iw * ih
                    union = float(area[n, i] + area[n, j]) - inter
                    if union > 0 and inter / union > iou_t:
                        ok = False
                        break
                if ok:
                    kept.append(i)
                    picked.append([n, c, i])
                    if len(kept) >= limit:
                        break
    return torch.tensor(picked, dtype=torch.int64).reshape(-1, 3)


# --------------------------------------------------------------------------------------------- quantised linear algebra
def _zp(t, like):
    return torch.zeros((), dtype=torch.int32) if t is None else t.to(torch.int32)


def _per_channel(t, rank: int, axis: int):
    """A scale / zero point that is a scalar or a vector over ``axis`` as a tensor that broadcasts over ``rank`` dims."""
    if t.numel() == 1:
        return t.reshape([1] * rank)
    shape = [1] * rank
    shape[axis] = t.numel()
    return t.reshape(shape)


def _saturate(v, zero_point, dtype):
    """saturate(round(v) + zero_point): rounding (half to even) comes before the zero point is added."""
    lo, hi = (0, 255) if dtype == torch.uint8 else (-128, 127)
    return torch.clamp(torch.round(v) + zero_point, lo, hi).to(dtype)


@op("DynamicQuantizeLinear")
def _dynamic_quantize(node, x):
    lo, hi = min(float(x.min()), 0.0), max(float(x.max()), 0.0)
    scale = (hi - lo) / 255.0 if hi > lo else 1.0
    zp = min(255.0, max(0.0, round(-lo / scale)))             # round half to even, as ONNX asks
    y = _saturate(x / scale, zp, torch.uint8)
    return y, torch.tensor(scale, dtype=torch.float32), torch.tensor(int(zp), dtype=torch.uint8)


@op("MatMulInteger")
def _matmul_integer(node, a, b, a_zp=None, b_zp=None):
    ai = a.to(torch.int32) - (_per_channel(a_zp.to(torch.int32), a.dim(), a.dim() - 2) if a_zp is not None else 0)
    bi = b.to(torch.int32) - (_per_channel(b_zp.to(torch.int32), b.dim(), b.dim() - 1) if b_zp is not None else 0)
    return torch.matmul(ai.double(), bi.double()).to(torch.int32)


@op("ConvInteger")
def _conv_integer(node, x, w, x_zp=None, w_zp=None):
    from .interp import _conv
    xi = x.to(torch.int32) - (x_zp.to(torch.int32).reshape(()) if x_zp is not None else 0)
    wi = w.to(torch.int32) - (_per_channel(w_zp.to(torch.int32), w.dim(), 0) if w_zp is not None else 0)
    return _conv(node, xi.double(), wi.double()).to(torch.int32)


@op("QLinearMatMul")
def _qlinear_matmul(node, a, a_s, a_zp, b, b_s, b_zp, y_s, y_zp):
    af = (a.to(torch.int32) - _per_channel(a_zp.to(torch.int32), a.dim(), a.dim() - 2)).double() * \
        _per_channel(a_s.double(), a.dim(), a.dim() - 2)
    bf = (b.to(torch.int32) - _per_channel(b_zp.to(torch.int32), b.dim(), b.dim() - 1)).double() * \
        _per_channel(b_s.double(), b.dim(), b.dim() - 1)
    y = torch.matmul(af, bf) / y_s.double()
    return _saturate(y, y_zp.double(), y_zp.dtype)


@op("QLinearConv")
def _qlinear_conv(node, x, x_s, x_zp, w, w_s, w_zp, y_s, y_zp, bias=None):
    from .interp import _conv
    xf = (x.to(torch.int32) - x_zp.to(torch.int32).reshape(())).double() * x_s.double().reshape(())
    wf = (w.to(torch.int32) - _per_channel(w_zp.to(torch.int32), w.dim(), 0)).double() * _per_channel(w_s.double(), w.dim(), 0)
    bf = None
    if bias is not None:                                      # int32 bias, scale = x_scale * w_scale
        bf = bias.double() * (x_s.double().reshape(()) * w_s.double().reshape(-1))
    y = _conv(node, xf, wf, bf) / y_s.double().reshape(())
    return _saturate(y, y_zp.double().reshape(()), y_zp.dtype)


# --------------------------------------------------------------------------------------------- recurrent layers
_ACT = {"Tanh": torch.tanh, "Sigmoid": torch.sigmoid, "Relu": torch.relu}


def _directions(node, n_dir):
    d = node.attr("direction", "forward")
    return {"forward": [False], "reverse": [True], "bidirectional": [False, True]}[d][:n_dir]


@op("RNN")
def _rnn(node, x, w, r, b=None, seq_lens=None, h0=None):
    """Elman RNN, layout 0: x [T, B, I], w [D, H, I], r [D, H, H], b [D, 2H]; returns (Y [T, D, B, H], Y_h [D, B, H])."""
    t_len, bsz, _ = x.shape
    n_dir, hid = w.shape[0], w.shape[1]
    acts = node.attr("activations", ["Tanh"] * n_dir)
    ys, hs = [], []
    for d, rev in enumerate(_directions(node, n_dir)):
        f = _ACT[acts[d] if d < len(acts) else acts[0]]
        h = h0[d] if h0 is not None else torch.zeros(bsz, hid, dtype=x.dtype)
        bias = (b[d, :hid] + b[d, hid:]) if b is not None else 0
        out = [None] * t_len
        for t in (range(t_len - 1, -1, -1) if rev else range(t_len)):
            h = f(x[t] @ w[d].T + h @ r[d].T + bias)
            out[t] = h
        ys.append(torch.stack(out))
        hs.append(h)
    return torch.stack(ys, dim=1), torch.stack(hs)


@op("GRU")
def _gru(node, x, w, r, b=None, seq_lens=None, h0=None):
    """ONNX GRU, layout 0, gate order z, r, h: returns (Y [T, D, B, H], Y_h [D, B, H])."""
    t_len, bsz, _ = x.shape
    n_dir, hid = w.shape[0], w.shape[1] // 3
    lbr = node.attr("linear_before_reset", 0)
    ys, hs = [], []
    for d, rev in enumerate(_directions(node, n_dir)):
        wz, wr, wh = w[d].split(hid, 0)
        rz, rr, rh = r[d].split(hid, 0)
        if b is not None:
            wbz, wbr, wbh, rbz, rbr, rbh = b[d].split(hid, 0)
        else:
            wbz = wbr = wbh = rbz = rbr = rbh = torch.zeros(hid, dtype=x.dtype)
        h = h0[d] if h0 is not None else torch.zeros(bsz, hid, dtype=x.dtype)
        out = [None] * t_len
        for t in (range(t_len - 1, -1, -1) if rev else range(t_len)):
            z = torch.sigmoid(x[t] @ wz.T + h @ rz.T + wbz + rbz)
            rg = torch.sigmoid(x[t] @ wr.T + h @ rr.T + wbr + rbr)
            if lbr:
                hh = torch.tanh(x[t] @ wh.T + rg * (h @ rh.T + rbh) + wbh)
            else:
                hh = torch.tanh(x[t] @ wh.T + (rg * h) @ rh.T + rbh + wbh)
            h = (1 - z) * hh + z * h
            out[t] = h
        ys.append(torch.stack(out))
        hs.append(h)
    return torch.stack(ys, dim=1), torch.stack(hs)


# --------------------------------------------------------------------------------------------- random operators
def _generator(node):
    g = torch.Generator()
    seed = node.attr("seed", None)
    g.manual_seed(int(seed) if seed is not None else 0)
    return g


@op("RandomUniform")
def _random_uniform(node):
    dt = ONNX_DT2TORCH[node.attr("dtype", 1)]
    lo, hi = node.attr("low", 0.0), node.attr("high", 1.0)
    return (torch.rand(node.attr("shape"), generator=_generator(node)) * (hi - lo) + lo).to(dt)


@op("RandomUniformLike")
def _random_uniform_like(node, x):
    dt = ONNX_DT2TORCH[node.attr("dtype")] if node.attr("dtype") is not None else x.dtype
    lo, hi = node.attr("low", 0.0), node.attr("high", 1.0)
    return (torch.rand(list(x.shape), generator=_generator(node)) * (hi - lo) + lo).to(dt)


@op("RandomNormalLike")
def _random_normal_like(node, x):
    dt = ONNX_DT2TORCH[node.attr("dtype")] if node.attr("dtype") is not None else x.dtype
    return (torch.randn(list(x.shape), generator=_generator(node)) * node.attr("scale", 1.0) + node.attr("mean", 0.0)).to(dt)


@op("Multinomial")
def _multinomial(node, x):
    dt = ONNX_DT2TORCH[node.attr("dtype", 6)]
    p = torch.softmax(x.float(), dim=-1)                      # the input holds unnormalised log-probabilities
    return torch.multinomial(p, node.attr("sample_size", 1), replacement=True, generator=_generator(node)).to(dt)


# --------------------------------------------------------------------------------------------- newer opsets (17 - 20)
for _name, _fn in (("BitwiseAnd", torch.bitwise_and), ("BitwiseOr", torch.bitwise_or), ("BitwiseXor", torch.bitwise_xor)):
    op(_name)((lambda f: (lambda node, a, b: f(a, b)))(_fn))


@op("BitwiseNot")
def _bitwise_not(node, x):
    return torch.bitwise_not(x)


@op("CastLike")
def _cast_like(node, x, target):
    return x.to(target.dtype)


@op("Bernoulli")
def _bernoulli(node, x):
    dt = ONNX_DT2TORCH[node.attr("dtype")] if node.attr("dtype") is not None else x.dtype
    return torch.bernoulli(x.float(), generator=_generator(node)).to(dt)


def _window(node, size, a0: float, a1: float, a2: float):
    n = int(size.reshape(-1)[0])
    dt = ONNX_DT2TORCH[node.attr("output_datatype", 1)]
    denom = n if node.attr("periodic", 1) else max(n - 1, 1)
    k = torch.arange(n, dtype=torch.float64)
    w = a0 - a1 * torch.cos(2 * math.pi * k / denom) + a2 * torch.cos(4 * math.pi * k / denom)
    return w.to(dt)


@op("HannWindow")
def _hann(node, size):
    return _window(node, size, 0.5, 0.5, 0.0)


@op("HammingWindow")
def _hamming(node, size):
    return _window(node, size, 25.0 / 46.0, 21.0 / 46.0, 0.0)


@op("BlackmanWindow")
def _blackman(node, size):
    return _window(node, size, 0.42, 0.5, 0.08)


@op("CenterCropPad")
def _center_crop_pad(node, x, shape):
    axes = node.attr("axes", list(range(x.dim())))
    out = x
    for ax, want in zip(axes, _ints(shape)):
        have = out.shape[ax]
        if want < have:
            start = (have - want) // 2
            out = out.narrow(ax, start, want)
        elif want > have:
            before = (want - have) // 2
            pad = [0, 0] * out.dim()
            pad[2 * (out.dim() - 1 - ax)] = before
            pad[2 * (out.dim() - 1 - ax) + 1] = want - have - before
            out = F.pad(out, pad)
    return out


@op("Col2Im")
def _col2im(node, x, image_shape, block_shape):
    return F.fold(x, _ints(image_shape), _ints(block_shape), dilation=node.attr("dilations", 1),
                  padding=node.attr("pads", [0, 0, 0, 0])[:2], stride=node.attr("strides", 1))


@op("DFT")
def _dft(node, x, dft_length=None, axis=None):
    """Input [..., 1] (real) or [..., 2] (real, imaginary); the transformed axis is ``axis`` (attribute before opset 20)."""
    ax = int(axis.reshape(-1)[0]) if axis is not None else node.attr("axis", 1)
    n = int(dft_length.reshape(-1)[0]) if dft_length is not None else None
    z = torch.complex(x[..., 0], x[..., 1]) if x.shape[-1] == 2 else x[..., 0].to(torch.complex64 if x.dtype == torch.float32 else torch.complex128)
    ax = ax if ax >= 0 else ax + x.dim()
    if node.attr("inverse", 0):
        out = torch.fft.ifft(z, n=n, dim=ax)
    elif node.attr("onesided", 0):
        out = torch.fft.fft(z, n=n, dim=ax)
        keep = out.shape[ax] // 2 + 1
        out = out.narrow(ax, 0, keep)
    else:
        out = torch.fft.fft(z, n=n, dim=ax)
    return torch.view_as_real(out).to(x.dtype)
