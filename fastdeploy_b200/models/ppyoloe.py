"""Synthetic PP-YOLOE+ generator: CSPRepResNet backbone, CustomCSPPAN neck with SPP,
ET-head with DFL, exported as a Paddle inference model (``.pdmodel`` + ``.pdiparams``)
plus ``infer_cfg.yml`` - the three files the reference's ``PPYOLOE`` class loads
(fastdeploy/vision/detection/ppdet/model.h:24-60, ppdet/preprocessor.cc:53-127).

The operator sequence mirrors a PaddleDetection deploy export: RepVGG blocks already
re-parameterised into one 3x3 ``conv2d`` + bias, ``batch_norm`` kept as separate ops,
``swish`` activations, ESE attention as ``pool2d``(adaptive 1x1) -> ``conv2d`` ->
``hard_sigmoid`` / ``sigmoid`` -> ``elementwise_mul``, DFL as ``softmax`` + 1x1 projection
conv, box decoding with constant anchor points / strides, division by ``scale_factor``
and (optionally) ``multiclass_nms3`` inside the graph.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from .paddle_net import PaddleNet, Tensor

VARIANTS = {
    # depth_mult, width_mult
    "s": (0.33, 0.50), "m": (0.67, 0.75), "l": (1.0, 1.0), "x": (1.33, 1.25),
    "tiny": (0.33, 0.25),   # test-size network, not a published variant
}


def _basic_block(net: PaddleNet, x: Tensor, ch: int, shortcut: bool, name: str) -> Tensor:
    y = net.conv_bn_act(x, ch, 3, 1, "swish", name=name + ".conv1")
    # RepVGG block in deploy form: one 3x3 conv with bias + swish
    y = net.conv(y, ch, 3, 1, bias=True, name=name + ".conv2.rep")
    y = net.act(y, "swish")
    return net.add(x, y) if shortcut else y


def _ese(net: PaddleNet, x: Tensor, name: str) -> Tensor:
    s = net.global_avgpool(x)
    s = net.conv(s, x.c, 1, 1, bias=True, name=name + ".fc")
    s = net.act(s, "hard_sigmoid")      # slope 0.2, offset 0.5 (paddle.nn.Hardsigmoid)
    return net.mul(x, s)


def _csp_res_stage(net: PaddleNet, x: Tensor, ch_out: int, n: int, name: str) -> Tensor:
    ch_mid = (x.c + ch_out) // 2
    x = net.conv_bn_act(x, ch_mid, 3, 2, "swish", name=name + ".conv_down")
    y1 = net.conv_bn_act(x, ch_mid // 2, 1, 1, "swish", name=name + ".conv1")
    y2 = net.conv_bn_act(x, ch_mid // 2, 1, 1, "swish", name=name + ".conv2")
    for i in range(n):
        y2 = _basic_block(net, y2, ch_mid // 2, True, f"{name}.blocks.{i}")
    y = net.concat([y1, y2], 1)
    y = _ese(net, y, name + ".attn")
    return net.conv_bn_act(y, ch_out, 1, 1, "swish", name=name + ".conv3")


def _spp(net: PaddleNet, x: Tensor, ch_out: int, name: str) -> Tensor:
    outs = [x] + [net.pool(x, k, 1, k // 2, "max") for k in (5, 9, 13)]
    return net.conv_bn_act(net.concat(outs, 1), ch_out, 1, 1, "swish", name=name + ".conv")


def _csp_stage(net: PaddleNet, x: Tensor, ch_out: int, n: int, spp: bool, name: str) -> Tensor:
    ch_mid = ch_out // 2
    y1 = net.conv_bn_act(x, ch_mid, 1, 1, "swish", name=name + ".conv1")
    y2 = net.conv_bn_act(x, ch_mid, 1, 1, "swish", name=name + ".conv2")
    for i in range(n):
        y2 = _basic_block(net, y2, ch_mid, False, f"{name}.convs.{i}")
        if spp and i == (n - 1) // 2:
            y2 = _spp(net, y2, ch_mid, f"{name}.spp")
    return net.conv_bn_act(net.concat([y1, y2], 1), ch_out, 1, 1, "swish", name=name + ".conv3")


def _ese_attn(net: PaddleNet, feat: Tensor, avg: Tensor, name: str) -> Tensor:
    w = net.conv(avg, feat.c, 1, 1, bias=True, name=name + ".fc")
    w = net.act(w, "sigmoid")
    return net.conv_bn_act(net.mul(feat, w), feat.c, 1, 1, "swish", name=name + ".conv")


def build_ppyoloe(variant: str = "l", num_classes: int = 80, image: int = 640, seed: int = 0, with_nms: bool = True,
                  reg_max: int = 16, score_threshold: float = 0.01, nms_threshold: float = 0.6,
                  nms_top_k: int = 1000, keep_top_k: int = 100) -> PaddleNet:
    depth, width = VARIANTS[variant]
    layers = [max(round(n * depth), 1) for n in (3, 6, 6, 3)]
    chans = [max(round(c * width), 1) for c in (64, 128, 256, 512, 1024)]
    # keep every channel count a multiple of 16 so that ch_mid // 2 stays a multiple of 8
    chans = [max(16, (c + 15) // 16 * 16) for c in chans]
    net = PaddleNet(seed)
    img = net.feed("image", "float32", [-1, 3, image, image])
    scale_factor = net.feed("scale_factor", "float32", [-1, 2])

    # ---------------- backbone: CSPRepResNet with a 3-conv stem
    x = net.conv_bn_act(img, chans[0] // 2, 3, 2, "swish", name="backbone.stem.conv1")
    x = net.conv_bn_act(x, chans[0] // 2, 3, 1, "swish", name="backbone.stem.conv2")
    x = net.conv_bn_act(x, chans[0], 3, 1, "swish", name="backbone.stem.conv3")
    feats: List[Tensor] = []
    for i in range(4):
        x = _csp_res_stage(net, x, chans[i + 1], layers[i], f"backbone.stages.{i}")
        if i >= 1:
            feats.append(x)
    c3, c4, c5 = feats

    # ---------------- neck: CustomCSPPAN
    neck_ch = [max(16, (round(c * width) + 15) // 16 * 16) for c in (768, 384, 192)]
    nblk = max(round(3 * depth), 1)
    fpn: List[Tensor] = []
    route = None
    for i, (f, ch) in enumerate(zip((c5, c4, c3), neck_ch)):
        if route is not None:
            f = net.concat([route, f], 1)
        f = _csp_stage(net, f, ch, nblk, spp=(i == 0), name=f"neck.fpn_stages.{i}")
        fpn.append(f)
        if i < 2:
            route = net.conv_bn_act(f, ch // 2, 1, 1, "swish", name=f"neck.fpn_routes.{i}")
            route = net.upsample2x(route)
    pan = [fpn[-1]]
    route = fpn[-1]
    for i in reversed(range(2)):
        route = net.conv_bn_act(route, route.c, 3, 2, "swish", name=f"neck.pan_routes.{i}")
        f = net.concat([route, fpn[i]], 1)
        route = _csp_stage(net, f, neck_ch[i], nblk, spp=False, name=f"neck.pan_stages.{i}")
        pan.append(route)
    neck_feats = pan[::-1]          # strides 32, 16, 8
    strides = [32, 16, 8]

    # ---------------- head: PPYOLOEHead.forward_eval
    bins = reg_max + 1
    proj = net.const_param("head.proj_conv.w", np.arange(bins, dtype=np.float32).reshape(1, bins, 1, 1))
    cls_list, reg_list, points, stride_rows = [], [], [], []
    bias_cls = float(-np.log((1 - 0.01) / 0.01))
    for i, (feat, s) in enumerate(zip(neck_feats, strides)):
        h, w = feat.shape[2], feat.shape[3]
        l = h * w
        avg = net.global_avgpool(feat)
        cls_feat = net.add(_ese_attn(net, feat, avg, f"head.stem_cls.{i}"), feat)
        cls_logit = net.conv(cls_feat, num_classes, 3, 1, bias=True, name=f"head.pred_cls.{i}", bias_value=bias_cls)
        cls_score = net.act(cls_logit, "sigmoid")
        cls_list.append(net.reshape(cls_score, [-1, num_classes, l], [-1, num_classes, l]))
        reg_feat = _ese_attn(net, feat, avg, f"head.stem_reg.{i}")
        reg = net.conv(reg_feat, 4 * bins, 3, 1, bias=True, name=f"head.pred_reg.{i}", bias_value=1.0)
        reg = net.reshape(reg, [-1, 4, bins, l], [-1, 4, bins, l])
        reg = net.transpose(reg, [0, 2, 3, 1])                       # [b, bins, l, 4]
        reg = net.softmax(reg, 1)
        dist = net.b.op("conv2d", {"Input": [reg.name], "Filter": [proj]}, ("Output",), [-1, 1, l, 4], strides=[1, 1],
                        paddings=[0, 0], dilations=[1, 1], groups=1, padding_algorithm="EXPLICIT", data_format="NCHW")
        dist = net.b.op("squeeze2", {"X": [dist]}, ("Out", "XShape"), [-1, l, 4], axes=[1])
        reg_list.append(Tensor(dist, [-1, l, 4]))
        ys, xs = np.meshgrid(np.arange(h, dtype=np.float32) + 0.5, np.arange(w, dtype=np.float32) + 0.5, indexing="ij")
        points.append(np.stack([xs.reshape(-1), ys.reshape(-1)], -1))
        stride_rows.append(np.full((l, 1), s, np.float32))
    scores = net.concat(cls_list, 2)                                 # [b, C, A]
    dists = net.concat(reg_list, 1)                                  # [b, A, 4]
    a_total = sum(p.shape[0] for p in points)
    anchor = net.const_param("head.anchor_points", np.concatenate(points).astype(np.float32))
    stride_t = net.const_param("head.stride_tensor", np.concatenate(stride_rows).astype(np.float32))
    b = net.b
    lt = b.tmp("lt", "float32", [-1, a_total, 2])
    rb = b.tmp("rb", "float32", [-1, a_total, 2])
    b.prog.add_op("split", {"X": [dists.name]}, {"Out": [lt, rb]}, axis=-1, num=2, sections=[])
    x1y1 = b.op("elementwise_sub", {"X": [anchor], "Y": [lt]}, ("Out",), [-1, a_total, 2], axis=-1)
    x2y2 = b.op("elementwise_add", {"X": [rb], "Y": [anchor]}, ("Out",), [-1, a_total, 2], axis=-1)
    boxes = b.op("concat", {"X": [x1y1, x2y2]}, ("Out",), [-1, a_total, 4], axis=-1)
    boxes = b.op("elementwise_mul", {"X": [boxes], "Y": [stride_t]}, ("Out",), [-1, a_total, 4], axis=-1)
    sy = b.tmp("sy", "float32", [-1, 1])
    sx = b.tmp("sx", "float32", [-1, 1])
    b.prog.add_op("split", {"X": [scale_factor.name]}, {"Out": [sy, sx]}, axis=-1, num=2, sections=[])
    sf = b.op("concat", {"X": [sx, sy, sx, sy]}, ("Out",), [-1, 4], axis=-1)
    sf = b.op("reshape2", {"X": [sf]}, ("Out", "XShape"), [-1, 1, 4], shape=[-1, 1, 4])
    boxes = b.op("elementwise_div", {"X": [boxes], "Y": [sf]}, ("Out",), [-1, a_total, 4], axis=-1)
    if with_nms:
        out = b.tmp("nms_out", "float32", [-1, 6])
        idx = b.tmp("nms_index", "int32", [-1, 1])
        num = b.tmp("nms_num", "int32", [-1])
        b.prog.add_op("multiclass_nms3", {"BBoxes": [boxes], "Scores": [scores.name]},
                      {"Out": [out], "Index": [idx], "NmsRoisNum": [num]}, background_label=-1,
                      keep_top_k=keep_top_k, nms_eta=1.0, nms_threshold=nms_threshold, nms_top_k=nms_top_k,
                      normalized=True, score_threshold=score_threshold)
        b.fetch(out)
        b.fetch(num)
    else:
        b.fetch(boxes)
        b.fetch(scores.name)
    return net


INFER_CFG = """mode: paddle
draw_threshold: 0.5
metric: COCO
use_dynamic_shape: false
arch: YOLO
min_subgraph_size: 3
Preprocess:
- interp: 2
  keep_ratio: false
  target_size:
  - {size}
  - {size}
  type: Resize
- mean:
  - 0.0
  - 0.0
  - 0.0
  norm_type: none
  std:
  - 1.0
  - 1.0
  - 1.0
  type: NormalizeImage
- type: Permute
label_list:
{labels}
"""


def write_ppyoloe(out_dir: str, variant: str = "l", image: int = 640, num_classes: int = 80, seed: int = 0,
                  **kw) -> Dict[str, str]:
    """Writes ``model.pdmodel``, ``model.pdiparams`` and ``infer_cfg.yml`` into ``out_dir``."""
    os.makedirs(out_dir, exist_ok=True)
    net = build_ppyoloe(variant, num_classes, image, seed, **kw)
    model, params = net.serialize()
    paths = {"model": os.path.join(out_dir, "model.pdmodel"), "params": os.path.join(out_dir, "model.pdiparams"),
             "config": os.path.join(out_dir, "infer_cfg.yml")}
    with open(paths["model"], "wb") as f:
        f.write(model)
    with open(paths["params"], "wb") as f:
        f.write(params)
    labels = "\n".join(f"- class_{i}" for i in range(num_classes))
    with open(paths["config"], "w") as f:
        f.write(INFER_CFG.format(size=image, labels=labels))
    return paths
