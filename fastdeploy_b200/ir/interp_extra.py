"""Interpreter operators added for the second batch of importer mappers: quantise / dequantise, trigonometric
and shrink activations, group normalisation, grid sampling, RoI align, YOLOv3 box decoding, ``set_value`` slicing
assignment, ``unique``, temporal shift, random normal.

Each is the fp32 reference the GPU executor is tested against. Operator semantics follow the ONNX definitions where
ONNX has the operator; the Paddle-only ones (``YoloBox``, ``SetValue``, ``TemporalShift``, ``Atan2``, ``Flip``) carry
the Paddle kernel's semantics and cite it.
"""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn.functional as F

from .interp import NP2TORCH, ONNX_DT2TORCH, _OPS, _ints, op

for _name, _fn in (("Acos", torch.acos), ("Asin", torch.asin), ("Atan", torch.atan), ("Cosh", torch.cosh),
                   ("Sinh", torch.sinh), ("Tan", torch.tan), ("Acosh", torch.acosh), ("Asinh", torch.asinh),
                   ("Atanh", torch.atanh)):
    if _name not in _OPS:
        _OPS[_name] = (lambda f: (lambda node, x: f(x)))(_fn)


@op("Atan2")
def _atan2(node, a, b):
    return torch.atan2(a, b)


@op("Shrink")
def _shrink(node, x):
    """ONNX Shrink: x - bias above lambd, x + bias below -lambd, else 0."""
    lambd, bias = node.attr("lambd", 0.5), node.attr("bias", 0.0)
    return torch.where(x > lambd, x - bias, torch.where(x < -lambd, x + bias, torch.zeros_like(x)))


@op("ThresholdedRelu")
def _thresholded_relu(node, x):
    return torch.where(x > node.attr("alpha", 1.0), x, torch.zeros_like(x))


@op("Flip")
def _flip(node, x):
    return torch.flip(x, dims=[int(a) for a in node.attr("axes")])


def _axis_view(t: torch.Tensor, like: torch.Tensor, axis: int) -> torch.Tensor:
    if t.dim() == 0 or t.numel() == 1:
        return t.reshape(())
    shape = [1] * like.dim()
    shape[axis if axis >= 0 else like.dim() + axis] = -1
    return t.reshape(shape)


@op("QuantizeLinear")
def _quantize_linear(node, x, scale, zp=None):
    """``clamp(round_half_even(x / scale) + zero_point)`` to int8 (uint8 when the zero point is uint8)."""
    axis = node.attr("axis", 1)
    s = _axis_view(scale.float(), x, axis)
    z = _axis_view(zp.float(), x, axis) if zp is not None else 0.0
    unsigned = zp is not None and zp.dtype == torch.uint8
    lo, hi = (0, 255) if unsigned else (-128, 127)
    q = torch.clamp(torch.round(x.float() / s) + z, lo, hi)
    return q.to(torch.uint8 if unsigned else torch.int8)


@op("DequantizeLinear")
def _dequantize_linear(node, x, scale, zp=None):
    axis = node.attr("axis", 1)
    s = _axis_view(scale.float(), x, axis)
    z = _axis_view(zp.float(), x, axis) if zp is not None else 0.0
    return (x.float() - z) * s


@op("GroupNormalization")
def _group_norm(node, x, scale, bias):
    return F.group_norm(x, int(node.attr("num_groups")), scale, bias, float(node.attr("epsilon", 1e-5)))


@op("GridSample")
def _grid_sample(node, x, grid):
    mode = {"linear": "bilinear", "bilinear": "bilinear", "nearest": "nearest", "cubic": "bicubic",
            "bicubic": "bicubic"}[node.attr("mode", "bilinear")]
    return F.grid_sample(x, grid, mode=mode, padding_mode=node.attr("padding_mode", "zeros"),
                         align_corners=bool(node.attr("align_corners", 0)))


@op("RoiAlign")
def _roi_align(node, x, rois, batch_idx):
    """ONNX RoiAlign (average mode): every output bin averages ``sampling_ratio^2`` bilinear samples
    (adaptive count ``ceil(roi / bins)`` when the ratio is 0). ``coordinate_transformation_mode = half_pixel`` shifts
    the box by half a pixel, which is Paddle's ``aligned = True``."""
    ph, pw = int(node.attr("output_height", 1)), int(node.attr("output_width", 1))
    ratio = int(node.attr("sampling_ratio", 0))
    scale = float(node.attr("spatial_scale", 1.0))
    aligned = node.attr("coordinate_transformation_mode", "half_pixel") == "half_pixel"
    n, c, h, w = x.shape
    out = x.new_zeros((rois.shape[0], c, ph, pw))
    off = 0.5 if aligned else 0.0
    for r in range(rois.shape[0]):
        img = x[int(batch_idx[r])]
        x1, y1, x2, y2 = [float(v) * scale - off for v in rois[r]]
        rw, rh = x2 - x1, y2 - y1
        if not aligned:
            rw, rh = max(rw, 1.0), max(rh, 1.0)
        bw, bh = rw / pw, rh / ph
        gx = ratio if ratio > 0 else max(int(math.ceil(rw / pw)), 1)
        gy = ratio if ratio > 0 else max(int(math.ceil(rh / ph)), 1)
        ys = y1 + (torch.arange(ph).view(ph, 1) + (torch.arange(gy).view(1, gy) + 0.5) / gy) * bh      # [ph, gy]
        xs = x1 + (torch.arange(pw).view(pw, 1) + (torch.arange(gx).view(1, gx) + 0.5) / gx) * bw      # [pw, gx]
        ys, xs = ys.reshape(-1).to(x.dtype), xs.reshape(-1).to(x.dtype)
        valid_y = (ys >= -1.0) & (ys <= h)
        valid_x = (xs >= -1.0) & (xs <= w)
        yc, xc = ys.clamp(0, h - 1), xs.clamp(0, w - 1)
        y0, x0 = yc.floor().long(), xc.floor().long()
        y1i, x1i = (y0 + 1).clamp(max=h - 1), (x0 + 1).clamp(max=w - 1)
        ly, lx = (yc - y0).view(-1, 1), (xc - x0).view(1, -1)
        v = (img[:, y0][:, :, x0] * (1 - ly) * (1 - lx) + img[:, y0][:, :, x1i] * (1 - ly) * lx +
             img[:, y1i][:, :, x0] * ly * (1 - lx) + img[:, y1i][:, :, x1i] * ly * lx)
        v = v * (valid_y.view(-1, 1) & valid_x.view(1, -1)).to(x.dtype)
        out[r] = v.reshape(c, ph, gy, pw, gx).mean(dim=(2, 4))
    return out


@op("YoloBox")
def _yolo_box(node, x, img_size):
    """YOLOv3 head decoding (paddle/phi/kernels/funcs/yolo_box_util.h): per anchor and cell, centre = (sigmoid(t) *
    scale - (scale - 1) / 2 + cell) / grid, size = exp(t) * anchor / input size, both times the image size;
    confidence below ``conf_thresh`` zeroes the box and its scores; boxes as x1 y1 x2 y2, optionally clipped."""
    anchors = [float(a) for a in node.attr("anchors")]
    na = len(anchors) // 2
    cnum = int(node.attr("class_num"))
    thresh = float(node.attr("conf_thresh", 0.01))
    ds = int(node.attr("downsample_ratio", 32))
    clip = bool(node.attr("clip_bbox", True))
    sxy = float(node.attr("scale_x_y", 1.0))
    iou_aware = bool(node.attr("iou_aware", False))
    iou_factor = float(node.attr("iou_aware_factor", 0.5))
    n, _, h, w = x.shape
    if iou_aware:
        ioup = torch.sigmoid(x[:, :na].reshape(n, na, 1, h, w))
        x = x[:, na:]
    x = x.reshape(n, na, 5 + cnum, h, w)
    img_h = img_size[:, 0].float().view(n, 1, 1, 1)
    img_w = img_size[:, 1].float().view(n, 1, 1, 1)
    gx = torch.arange(w, dtype=x.dtype).view(1, 1, 1, w)
    gy = torch.arange(h, dtype=x.dtype).view(1, 1, h, 1)
    bias = -0.5 * (sxy - 1.0)
    cx = (torch.sigmoid(x[:, :, 0]) * sxy + bias + gx) / w * img_w
    cy = (torch.sigmoid(x[:, :, 1]) * sxy + bias + gy) / h * img_h
    aw = torch.tensor(anchors[0::2], dtype=x.dtype).view(1, na, 1, 1)
    ah = torch.tensor(anchors[1::2], dtype=x.dtype).view(1, na, 1, 1)
    bw = torch.exp(x[:, :, 2]) * aw / (ds * w) * img_w
    bh = torch.exp(x[:, :, 3]) * ah / (ds * h) * img_h
    conf = torch.sigmoid(x[:, :, 4])
    if iou_aware:
        conf = conf.pow(1.0 - iou_factor) * ioup[:, :, 0].pow(iou_factor)
    keep = (conf >= thresh).to(x.dtype)
    boxes = torch.stack([cx - bw / 2, cy - bh / 2, cx + bw / 2, cy + bh / 2], dim=-1)
    if clip:
        boxes = torch.stack([boxes[..., 0].clamp(min=0), boxes[..., 1].clamp(min=0),
                             torch.minimum(boxes[..., 2], img_w - 1), torch.minimum(boxes[..., 3], img_h - 1)], dim=-1)
    boxes = boxes * keep.unsqueeze(-1)
    scores = (conf * keep).unsqueeze(2) * torch.sigmoid(x[:, :, 5:])
    return boxes.reshape(n, na * h * w, 4), scores.permute(0, 1, 3, 4, 2).reshape(n, na * h * w, cnum)


@op("SetValue")
def _set_value(node, x, value=None):
    """``x[slices] = value`` on a copy (paddle/phi/kernels/set_value_kernel.h): ``axes / starts / ends / steps``
    select the region, ``decrease_axes`` are dimensions the value lacks, ``none_axes`` dimensions it has extra."""
    y = x.clone()
    axes, starts = node.attr("axes", []), node.attr("starts", [])
    ends, steps = node.attr("ends", []), node.attr("steps", []) or [1] * len(axes)
    sl = [slice(None)] * x.dim()
    for a, s, e, p in zip(axes, starts, ends, steps):
        sl[a] = slice(int(s), int(e), int(p))
    if value is None:
        vals = node.attr("values")
        shape = node.attr("shape", None) or [len(vals)]
        value = torch.tensor(vals, dtype=x.dtype).reshape([int(d) for d in shape])
    region = y[tuple(sl)]
    v = value.to(x.dtype)
    for a in sorted(node.attr("decrease_axes", []) or []):
        v = v.unsqueeze(a) if v.dim() < region.dim() else v
    y[tuple(sl)] = v.expand(region.shape) if v.numel() != region.numel() else v.reshape(region.shape)
    return y


@op("Unique")
def _unique(node, x):
    """ONNX Unique: values, first-occurrence indices, inverse indices, counts (sorted unless ``sorted = 0``)."""
    axis = node.attr("axis", None)
    flat = x.reshape(-1) if axis is None else x
    vals, inv, counts = torch.unique(flat, sorted=True, return_inverse=True, return_counts=True, dim=None if axis is None else axis)
    n = vals.shape[0] if axis is None else vals.shape[axis]
    inv_flat = inv.reshape(-1)
    first = torch.full((n,), inv_flat.numel(), dtype=torch.int64)
    first = first.scatter_reduce(0, inv_flat, torch.arange(inv_flat.numel()), reduce="amin")
    if not node.attr("sorted", 1):
        order = torch.argsort(first)
        rank = torch.empty_like(order)
        rank[order] = torch.arange(n)
        vals = vals.index_select(0 if axis is None else axis, order)
        first, counts, inv = first[order], counts[order], rank[inv]
    return vals, first, inv, counts


@op("TemporalShift")
def _temporal_shift(node, x):
    """``[N * T, C, H, W]``: the first ``C * ratio`` channels take the previous frame's values, the next ``C * ratio``
    the following frame's, the rest stay (paddle/phi/kernels/cpu/temporal_shift_kernel.cc)."""
    t = int(node.attr("seg_num"))
    ratio = float(node.attr("shift_ratio", 0.25))
    nt, c, h, w = x.shape
    v = x.reshape(nt // t, t, c, h, w)
    c1, c2 = int(c * ratio), int(c * 2 * ratio)
    out = torch.zeros_like(v)
    out[:, 1:, :c1] = v[:, :-1, :c1]
    out[:, :-1, c1:c2] = v[:, 1:, c1:c2]
    out[:, :, c2:] = v[:, :, c2:]
    return out.reshape(nt, c, h, w)


@op("RandomNormal")
def _random_normal(node):
    g = torch.Generator().manual_seed(int(node.attr("seed", 0)))
    shape = [int(d) for d in node.attr("shape")]
    dt = ONNX_DT2TORCH.get(node.attr("dtype", 1), torch.float32)
    return (torch.randn(shape, generator=g) * float(node.attr("scale", 1.0)) + float(node.attr("mean", 0.0))).to(dt)
