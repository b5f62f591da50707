"""Vision Transformer generator (PaddleClas ``VisionTransformer`` export layout): patch-embedding convolution,
class token + learned position embedding, pre-LayerNorm encoder blocks (multi-head attention with separate
q / k / v projections, GELU feed-forward), final LayerNorm and a linear head on the class token.

``ViT-H/14``: patch 14, 32 layers, hidden 1280, 16 heads, MLP 5120, 224 x 224 input -> 257 tokens, about
632 M parameters. The reference runs such a model through ``PaddleClasModel`` with an ``inference_cls.yaml``
(fastdeploy/vision/classification/ppcls/model.cc:23-119); weights here are random (no network access).
"""
from __future__ import annotations

import os
from typing import Dict

import numpy as np

from ..importer.paddle_format import ProgramBuilder
from .ernie import _B

SIZES = {
    "huge14": dict(patch=14, layers=32, hidden=1280, heads=16, mlp=5120),
    "large16": dict(patch=16, layers=24, hidden=1024, heads=16, mlp=4096),
    "base16": dict(patch=16, layers=12, hidden=768, heads=12, mlp=3072),
    "tiny": dict(patch=8, layers=2, hidden=64, heads=4, mlp=128),       # test size
}


def build_vit(size: str = "huge14", image: int = 224, num_classes: int = 1000, seed: int = 0) -> ProgramBuilder:
    cfg = SIZES[size]
    P, L, H, NH, F = cfg["patch"], cfg["layers"], cfg["hidden"], cfg["heads"], cfg["mlp"]
    D = H // NH
    G = image // P
    T = G * G + 1
    m = _B(seed)
    b = m.b
    x = b.feed("x", "float32", [-1, 3, image, image])
    w = m.w("patch_embed.proj.w_0", (H, 3, P, P))
    bias = m.vec("patch_embed.proj.b_0", H)
    y = b.op("conv2d", {"Input": [x], "Filter": [w]}, ("Output",), [-1, H, G, G], strides=[P, P], paddings=[0, 0],
             dilations=[1, 1], groups=1, padding_algorithm="EXPLICIT", data_format="NCHW")
    bias4 = b.op("reshape2", {"X": [bias]}, ("Out", "XShape"), [1, H, 1, 1], shape=[1, H, 1, 1])
    y = b.op("elementwise_add", {"X": [y], "Y": [bias4]}, ("Out",), [-1, H, G, G], axis=-1)
    y = b.op("flatten_contiguous_range", {"X": [y]}, ("Out", "XShape"), [-1, H, G * G], start_axis=2, stop_axis=3)
    y = b.op("transpose2", {"X": [y]}, ("Out", "XShape"), [-1, G * G, H], axis=[0, 2, 1])
    cls = m.w("cls_token", (1, 1, H))
    shape_ref = b.op("slice", {"Input": [y]}, ("Out",), [-1, 1, H], axes=[1], starts=[0], ends=[1], decrease_axis=[],
                     infer_flags=[1])
    cls_b = b.op("scale", {"X": [shape_ref]}, ("Out",), [-1, 1, H], scale=0.0, bias=0.0, bias_after_scale=True)
    cls_b = b.op("elementwise_add", {"X": [cls_b], "Y": [cls]}, ("Out",), [-1, 1, H], axis=-1)
    s3 = [-1, T, H]
    xseq = b.op("concat", {"X": [cls_b, y]}, ("Out",), s3, axis=1)
    pos = m.w("pos_embed", (1, T, H))
    xseq = b.op("elementwise_add", {"X": [xseq], "Y": [pos]}, ("Out",), s3, axis=-1)
    for l in range(L):
        p = f"blocks.{l}"
        h = m.layer_norm(xseq, H, f"{p}.norm1", s3)
        qkv = []
        for nm in ("q", "k", "v"):
            t = m.linear(h, H, H, f"{p}.attn.{nm}", s3)
            t = b.op("reshape2", {"X": [t]}, ("Out", "XShape"), [-1, T, NH, D], shape=[0, 0, NH, D])
            t = b.op("transpose2", {"X": [t]}, ("Out", "XShape"), [-1, NH, T, D], axis=[0, 2, 1, 3])
            qkv.append(t)
        q = b.op("scale", {"X": [qkv[0]]}, ("Out",), [-1, NH, T, D], scale=float(D) ** -0.5, bias=0.0, bias_after_scale=True)
        sc = b.op("matmul_v2", {"X": [q], "Y": [qkv[1]]}, ("Out",), [-1, NH, T, T], trans_x=False, trans_y=True)
        pr = b.op("softmax", {"X": [sc]}, ("Out",), [-1, NH, T, T], axis=-1)
        ctx = b.op("matmul_v2", {"X": [pr], "Y": [qkv[2]]}, ("Out",), [-1, NH, T, D], trans_x=False, trans_y=False)
        ctx = b.op("transpose2", {"X": [ctx]}, ("Out", "XShape"), [-1, T, NH, D], axis=[0, 2, 1, 3])
        ctx = b.op("reshape2", {"X": [ctx]}, ("Out", "XShape"), s3, shape=[0, 0, H])
        att = m.linear(ctx, H, H, f"{p}.attn.proj", s3)
        xseq = b.op("elementwise_add", {"X": [xseq], "Y": [att]}, ("Out",), s3, axis=-1)
        h = m.layer_norm(xseq, H, f"{p}.norm2", s3)
        f1 = m.linear(h, H, F, f"{p}.mlp.fc1", [-1, T, F])
        f1 = b.op("gelu", {"X": [f1]}, ("Out",), [-1, T, F], approximate=False)
        f2 = m.linear(f1, F, H, f"{p}.mlp.fc2", s3)
        xseq = b.op("elementwise_add", {"X": [xseq], "Y": [f2]}, ("Out",), s3, axis=-1)
    xseq = m.layer_norm(xseq, H, "norm", s3)
    c = b.op("slice", {"Input": [xseq]}, ("Out",), [-1, H], axes=[1], starts=[0], ends=[1], decrease_axis=[1], infer_flags=[1])
    logits = m.linear(c, H, num_classes, "head", [-1, num_classes])
    b.fetch(b.op("softmax", {"X": [logits]}, ("Out",), [-1, num_classes], axis=-1))
    return b


def write_vit(out_dir: str, size: str = "huge14", image: int = 224, num_classes: int = 1000, seed: int = 0) -> Dict[str, str]:
    os.makedirs(out_dir, exist_ok=True)
    model, params = build_vit(size, image, num_classes, seed).serialize()
    paths = {"model": os.path.join(out_dir, "inference.pdmodel"), "params": os.path.join(out_dir, "inference.pdiparams"),
             "config": os.path.join(out_dir, "inference_cls.yaml")}
    with open(paths["model"], "wb") as f:
        f.write(model)
    with open(paths["params"], "wb") as f:
        f.write(params)
    with open(paths["config"], "w") as f:
        f.write("PreProcess:\n  transform_ops:\n"
                f"  - ResizeImage:\n      resize_short: {int(image * 256 / 224)}\n"
                f"  - CropImage:\n      size: {image}\n"
                "  - NormalizeImage:\n      mean: [0.5, 0.5, 0.5]\n      std: [0.5, 0.5, 0.5]\n      scale: 0.00392157\n      order: ''\n"
                "  - ToCHWImage: null\nPostProcess:\n  Topk:\n    topk: 5\n")
    return paths
