"""Synthetic PP-OCRv3 generators (Paddle inference format), one per stage of the pipeline:

* ``det``: DBNet - MobileNetV3-large x0.5 backbone, RSE-FPN neck (96 channels), DBHead with two 2x2
  stride-2 transposed convolutions -> probability map ``[N,1,H,W]``.
* ``cls``: MobileNetV3-small x0.35 angle classifier on ``[N,3,48,192]`` crops -> ``[N,2]`` (softmax).
* ``rec``: SVTR-LCNet - MobileNetV1-Enhance backbone (height collapsed to 1), SVTR neck with two global
  mixing blocks, CTC head over a 6625-character vocabulary -> ``[N, W/8, 6625]`` (softmax).

They stand in for the files the reference downloads (ch_PP-OCRv3_det / cls / rec inference models)."""
from __future__ import annotations

import os
from typing import Dict, List

import numpy as np

from .paddle_net import PaddleNet, Tensor


def _mv3_block(net: PaddleNet, x: Tensor, k: int, exp: int, cout: int, use_se: bool, act: str, stride, name: str) -> Tensor:
    y = net.conv_bn_act(x, exp, 1, 1, act, name=name + ".expand")
    y = net.conv_bn_act(y, exp, k, stride, act, groups=exp, name=name + ".dw")
    if use_se:
        y = net.se(y, 4, name + ".se")
    y = net.conv_bn_act(y, cout, 1, 1, None, name=name + ".linear")
    if stride == 1 and x.c == cout:
        y = net.add(x, y)
    return y


def _c(v: float, scale: float) -> int:
    return max(8, int(v * scale + 4) // 8 * 8)


MV3_LARGE = [  # k, exp, c, se, act, stride
    (3, 16, 16, False, "relu", 1), (3, 64, 24, False, "relu", 2), (3, 72, 24, False, "relu", 1),
    (5, 72, 40, True, "relu", 2), (5, 120, 40, True, "relu", 1), (5, 120, 40, True, "relu", 1),
    (3, 240, 80, False, "hard_swish", 2), (3, 200, 80, False, "hard_swish", 1), (3, 184, 80, False, "hard_swish", 1),
    (3, 184, 80, False, "hard_swish", 1), (3, 480, 112, True, "hard_swish", 1), (3, 672, 112, True, "hard_swish", 1),
    (5, 672, 160, True, "hard_swish", 2), (5, 960, 160, True, "hard_swish", 1), (5, 960, 160, True, "hard_swish", 1)]
MV3_SMALL = [
    (3, 16, 16, True, "relu", 2), (3, 72, 24, False, "relu", 2), (3, 88, 24, False, "relu", 1),
    (5, 96, 40, True, "hard_swish", 2), (5, 240, 40, True, "hard_swish", 1), (5, 240, 40, True, "hard_swish", 1),
    (5, 120, 48, True, "hard_swish", 1), (5, 144, 48, True, "hard_swish", 1), (5, 288, 96, True, "hard_swish", 2),
    (5, 576, 96, True, "hard_swish", 1), (5, 576, 96, True, "hard_swish", 1)]


def build_det(image_hw=(-1, -1), seed: int = 0, scale: float = 0.5) -> PaddleNet:
    net = PaddleNet(seed)
    h, w = image_hw
    x = net.feed("x", "float32", [-1, 3, h, w])
    y = net.conv_bn_act(x, _c(16, scale), 3, 2, "hard_swish", name="backbone.conv1")
    feats: List[Tensor] = []
    for i, (k, e, c, se, act, s) in enumerate(MV3_LARGE):
        if s == 2 and i > 1:
            feats.append(y)
        y = _mv3_block(net, y, k, _c(e, scale), _c(c, scale), se, act, s, f"backbone.blocks.{i}")
    y = net.conv_bn_act(y, _c(960, scale), 1, 1, "hard_swish", name="backbone.conv_last")
    feats.append(y)
    # after block 1 the stride is 4: collect [s4, s8, s16, s32]
    feats = feats[-4:] if len(feats) >= 4 else feats
    # RSE-FPN
    oc = 96
    ins = []
    for i, f in enumerate(feats):
        t = net.conv(f, oc, 1, 1, name=f"neck.ins_conv.{i}")
        ins.append(net.add(t, net.se(t, 4, f"neck.ins_conv.{i}.se")))
    for i in (2, 1, 0):
        ins[i] = net.add(ins[i], net.upsample2x(ins[i + 1]))
    outs = []
    for i, f in enumerate(ins):
        t = net.conv(f, oc // 4, 3, 1, name=f"neck.inp_conv.{i}")
        t = net.add(t, net.se(t, 4, f"neck.inp_conv.{i}.se"))
        for _ in range(i):
            t = net.upsample2x(t)
        outs.append(t)
    fuse = net.concat(outs[::-1], 1)
    # DBHead (binarize branch)
    t = net.act(net.bn(net.conv(fuse, oc // 4, 3, 1, name="head.conv1"), "head.bn1"), "relu")
    t = net.act(net.bn(net.deconv2x(t, oc // 4, "head.deconv1"), "head.bn2"), "relu")
    t = net.act(net.deconv2x(t, 1, "head.deconv2"), "sigmoid")
    net.fetch(t)
    return net


def build_cls(seed: int = 0, scale: float = 0.35) -> PaddleNet:
    net = PaddleNet(seed)
    x = net.feed("x", "float32", [-1, 3, 48, 192])
    y = net.conv_bn_act(x, _c(16, scale), 3, 2, "hard_swish", name="backbone.conv1")
    for i, (k, e, c, se, act, s) in enumerate(MV3_SMALL):
        stride = (2, 1)[0] if s == 2 else 1
        y = _mv3_block(net, y, k, _c(e, scale), _c(c, scale), se, act, stride, f"backbone.blocks.{i}")
    y = net.conv_bn_act(y, _c(576, scale), 1, 1, "hard_swish", name="backbone.conv_last")
    y = net.global_avgpool(y)
    y = net.reshape(y, [0, -1], [-1, y.c])
    y = net.linear(y, 2, "head.fc")
    y = net.softmax(y, -1)
    net.fetch(y)
    return net


def build_rec(width: int = -1, vocab: int = 6625, seed: int = 0, scale: float = 0.5, dim: int = 120) -> PaddleNet:
    net = PaddleNet(seed)
    x = net.feed("x", "float32", [-1, 3, 48, width])

    def ds(t, cout, stride, name, k=3):
        """depthwise separable unit of MobileNetV1-Enhance; ``stride`` may be (sh, sw)."""
        sh, sw = stride if isinstance(stride, tuple) else (stride, stride)
        if sh == sw:
            t = net.dwconv_bn_act(t, k, sh, "hard_swish", name + ".dw")
        else:
            # (2,1) stride: depthwise conv at stride 1 then a (2,1) max-pool keeps the builder square-strided
            t = net.dwconv_bn_act(t, k, 1, "hard_swish", name + ".dw")
            shape = [t.shape[0], t.c, t.shape[2] // 2 if t.shape[2] > 0 else -1, t.shape[3]]
            y = net.b.op("pool2d", {"X": [t.name]}, ("Out",), shape, pooling_type="avg", ksize=[2, 1], adaptive=False,
                         global_pooling=False, strides=[2, 1], paddings=[0, 0], exclusive=True, ceil_mode=False,
                         padding_algorithm="EXPLICIT", data_format="NCHW")
            t = Tensor(y, shape)
        return net.conv_bn_act(t, cout, 1, 1, "hard_swish", name=name + ".pw")
    c = lambda v: _c(v, scale)
    y = net.conv_bn_act(x, c(32), 3, 2, "hard_swish", name="backbone.conv1")          # 24 x W/2
    y = ds(y, c(64), 1, "backbone.block2_1")
    y = ds(y, c(128), 1, "backbone.block2_2")
    y = ds(y, c(128), 1, "backbone.block3_1")
    y = ds(y, c(256), (2, 1), "backbone.block3_2")                                      # 12
    y = ds(y, c(256), 1, "backbone.block4_1")
    y = ds(y, c(512), 2, "backbone.block4_2")                                           # 6 x W/4
    for i in range(5):
        y = ds(y, c(512), 1, f"backbone.block5.{i}", k=5)
    y = ds(y, c(1024), (2, 1), "backbone.block5.5", k=5)                               # 3
    y = net.se(y, 4, "backbone.se")
    y = ds(y, c(1024), 2, "backbone.block6", k=5)                                       # 2 x W/8
    shape = [y.shape[0], y.c, 1, y.shape[3]]
    y = Tensor(net.b.op("pool2d", {"X": [y.name]}, ("Out",), shape, pooling_type="max", ksize=[2, 1], adaptive=False,
                        global_pooling=False, strides=[2, 1], paddings=[0, 0], exclusive=True, ceil_mode=False,
                        padding_algorithm="EXPLICIT", data_format="NCHW"), shape)      # 1 x W/8
    # SVTR neck
    hdim = y.c
    t = net.conv_bn_act(y, hdim // 8, 3, 1, "swish", name="neck.conv1")
    t = net.conv_bn_act(t, dim, 1, 1, "swish", name="neck.conv2")
    wtok = t.shape[3]
    seq = net.reshape(t, [0, dim, -1], [-1, dim, wtok])
    seq = net.transpose(seq, [0, 2, 1])                                                 # [B, T, dim]
    heads = 8
    for i in range(2):
        p = f"neck.svtr.{i}"
        hln = net.layer_norm(seq, p + ".norm1")
        qkv = []
        for nm in ("q", "k", "v"):
            tq = net.linear(hln, dim, f"{p}.attn.{nm}")
            tq = net.reshape(tq, [0, 0, heads, dim // heads], [-1, wtok, heads, dim // heads])
            qkv.append(net.transpose(tq, [0, 2, 1, 3]))
        q = Tensor(net.b.op("scale", {"X": [qkv[0].name]}, ("Out",), qkv[0].shape, scale=float(dim // heads) ** -0.5,
                            bias=0.0, bias_after_scale=True), qkv[0].shape)
        sc = net.b.op("matmul_v2", {"X": [q.name], "Y": [qkv[1].name]}, ("Out",), [-1, heads, wtok, wtok],
                      trans_x=False, trans_y=True)
        pr = net.b.op("softmax", {"X": [sc]}, ("Out",), [-1, heads, wtok, wtok], axis=-1)
        ctx = net.b.op("matmul_v2", {"X": [pr], "Y": [qkv[2].name]}, ("Out",), qkv[2].shape, trans_x=False,
                       trans_y=False)
        ctx = net.transpose(Tensor(ctx, qkv[2].shape), [0, 2, 1, 3])
        ctx = net.reshape(ctx, [0, 0, dim], [-1, wtok, dim])
        seq = net.add(seq, net.linear(ctx, dim, f"{p}.attn.proj"))
        f = net.linear(net.layer_norm(seq, p + ".norm2"), dim * 2, f"{p}.mlp.fc1", act="swish")
        seq = net.add(seq, net.linear(f, dim, f"{p}.mlp.fc2"))
    seq = net.layer_norm(seq, "neck.norm")
    t = net.transpose(seq, [0, 2, 1])
    t = net.reshape(t, [0, dim, 1, -1], [-1, dim, 1, wtok])
    t = net.conv_bn_act(t, hdim // 8, 1, 1, "swish", name="neck.conv3")
    t = net.concat([y, t], 1)
    t = net.conv_bn_act(t, hdim // 8, 3, 1, "swish", name="neck.conv4")
    t = net.conv_bn_act(t, 64, 1, 1, "swish", name="neck.conv1x1")
    seq = net.reshape(t, [0, 64, -1], [-1, 64, wtok])
    seq = net.transpose(seq, [0, 2, 1])
    logits = net.linear(seq, vocab, "head.fc")
    probs = net.softmax(logits, -1)
    net.fetch(probs)
    return net


def write_ppocr(out_dir: str, seed: int = 0, vocab: int = 6625, rec_width: int = -1) -> Dict[str, str]:
    """Writes det / cls / rec model pairs and the character dictionary (``vocab - 2`` lines, as the
    recogniser's label list is ``blank + dict + space``)."""
    os.makedirs(out_dir, exist_ok=True)
    paths: Dict[str, str] = {}
    for name, net in (("det", build_det(seed=seed)), ("cls", build_cls(seed=seed + 1)),
                      ("rec", build_rec(rec_width, vocab, seed=seed + 2))):
        model, params = net.serialize()
        paths[name + "_model"] = os.path.join(out_dir, f"{name}.pdmodel")
        paths[name + "_params"] = os.path.join(out_dir, f"{name}.pdiparams")
        with open(paths[name + "_model"], "wb") as f:
            f.write(model)
        with open(paths[name + "_params"], "wb") as f:
            f.write(params)
    paths["dict"] = os.path.join(out_dir, "ppocr_keys_v1.txt")
    with open(paths["dict"], "w", encoding="utf-8") as f:
        chars = []
        cp = 0x4E00
        while len(chars) < vocab - 2:
            chars.append(chr(cp))
            cp += 1
        f.write("\n".join(chars) + "\n")
    return paths
