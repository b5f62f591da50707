"""Synthetic SER model in the shape of PP-StructureV2's visual-feature-independent LayoutXLM (Paddle inference format).

Inputs, in the order the reference binds them (python/fastdeploy/vision/ocr/ppocr/__init__.py:1275-1292):
``input_ids [B, S]``, ``bbox [B, S, 4]`` (x0, y0, x1, y1 on the 0..1000 grid), ``attention_mask [B, S]``,
``token_type_ids [B, S]``, all int64. The embedding is the LayoutLMv2 sum - word + position + left + upper + right +
lower + height + width + token type - followed by LayerNorm; the encoder is the BERT-style stack of
``models/ernie.py``; the head is a per-token linear classifier over the BIO labels. The spatial-aware relative
attention bias of the original is left out (random weights would make it noise): the operator set that a real
export needs around it (slices of the box tensor, coordinate differences, nine embedding lookups, additive mask from
the attention mask) is all here.
"""
from __future__ import annotations

import os
from typing import Dict

import numpy as np

from .ernie import _B

SIZES = {
    "base": dict(layers=12, hidden=768, heads=12, ffn=3072, vocab=250002, max_pos=514, coord=1024, types=1),
    "tiny": dict(layers=2, hidden=64, heads=4, ffn=128, vocab=300, max_pos=514, coord=1024, types=1),   # test size
}


def build_ser_vi_layoutxlm(size: str = "tiny", num_labels: int = 7, seed: int = 0):
    cfg = SIZES[size]
    L, H, NH, F = cfg["layers"], cfg["hidden"], cfg["heads"], cfg["ffn"]
    D = H // NH
    m = _B(seed)
    b = m.b
    ids = b.feed("input_ids", "int64", [-1, -1])
    bbox = b.feed("bbox", "int64", [-1, -1, 4])
    att_mask = b.feed("attention_mask", "int64", [-1, -1])
    tids = b.feed("token_type_ids", "int64", [-1, -1])
    s3 = [-1, -1, H]
    tabs = {"word": m.w("word_embeddings", (cfg["vocab"], H)), "pos": m.w("position_embeddings", (cfg["max_pos"], H)),
            "x": m.w("x_position_embeddings", (cfg["coord"], H)), "y": m.w("y_position_embeddings", (cfg["coord"], H)),
            "h": m.w("h_position_embeddings", (cfg["coord"], H)), "w": m.w("w_position_embeddings", (cfg["coord"], H)),
            "type": m.w("token_type_embeddings", (cfg["types"], H))}

    def coord(k):
        return b.op("slice", {"Input": [bbox]}, ("Out",), [-1, -1], axes=[2], starts=[k], ends=[k + 1], decrease_axis=[2],
                    infer_flags=[1])
    x0, y0, x1, y1 = coord(0), coord(1), coord(2), coord(3)
    hh = b.op("elementwise_sub", {"X": [y1], "Y": [y0]}, ("Out",), [-1, -1], "int64", axis=-1)
    ww = b.op("elementwise_sub", {"X": [x1], "Y": [x0]}, ("Out",), [-1, -1], "int64", axis=-1)
    ones = b.op("fill_any_like", {"X": [ids]}, ("Out",), [-1, -1], "int64", value=1.0, dtype=3)
    csum = b.op("cumsum", {"X": [ones]}, ("Out",), [-1, -1], "int64", axis=-1, exclusive=False, reverse=False)
    pos_ids = b.op("elementwise_sub", {"X": [csum], "Y": [ones]}, ("Out",), [-1, -1], "int64", axis=-1)

    def look(idx, table):
        return b.op("lookup_table_v2", {"Ids": [idx], "W": [table]}, ("Out",), s3, padding_idx=-1)
    parts = [look(ids, tabs["word"]), look(pos_ids, tabs["pos"]), look(x0, tabs["x"]), look(y0, tabs["y"]),
             look(x1, tabs["x"]), look(y1, tabs["y"]), look(hh, tabs["h"]), look(ww, tabs["w"]), look(tids, tabs["type"])]
    x = parts[0]
    for p in parts[1:]:
        x = b.op("elementwise_add", {"X": [x], "Y": [p]}, ("Out",), s3, axis=-1)
    x = m.layer_norm(x, H, "embeddings.layer_norm", s3)
    mask_f = b.op("cast", {"X": [att_mask]}, ("Out",), [-1, -1], in_dtype=3, out_dtype=5)
    am = b.op("scale", {"X": [mask_f]}, ("Out",), [-1, -1], scale=1e4, bias=-1.0, bias_after_scale=False)
    am = b.op("unsqueeze2", {"X": [am]}, ("Out", "XShape"), [-1, 1, 1, -1], axes=[1, 2])
    for l in range(L):
        p = f"encoder.layer.{l}"
        qkv = []
        for nm in ("query", "key", "value"):
            t = m.linear(x, H, H, f"{p}.attention.self.{nm}", s3)
            t = b.op("reshape2", {"X": [t]}, ("Out", "XShape"), [-1, -1, NH, D], shape=[0, 0, NH, D])
            t = b.op("transpose2", {"X": [t]}, ("Out", "XShape"), [-1, NH, -1, D], axis=[0, 2, 1, 3])
            qkv.append(t)
        q = b.op("scale", {"X": [qkv[0]]}, ("Out",), [-1, NH, -1, D], scale=float(D) ** -0.5, bias=0.0,
                 bias_after_scale=True)
        sc = b.op("matmul_v2", {"X": [q], "Y": [qkv[1]]}, ("Out",), [-1, NH, -1, -1], trans_x=False, trans_y=True)
        sc = b.op("elementwise_add", {"X": [sc], "Y": [am]}, ("Out",), [-1, NH, -1, -1], axis=-1)
        pr = b.op("softmax", {"X": [sc]}, ("Out",), [-1, NH, -1, -1], axis=-1)
        ctx = b.op("matmul_v2", {"X": [pr], "Y": [qkv[2]]}, ("Out",), [-1, NH, -1, D], trans_x=False, trans_y=False)
        ctx = b.op("transpose2", {"X": [ctx]}, ("Out", "XShape"), [-1, -1, NH, D], axis=[0, 2, 1, 3])
        ctx = b.op("reshape2", {"X": [ctx]}, ("Out", "XShape"), s3, shape=[0, 0, H])
        att = m.linear(ctx, H, H, f"{p}.attention.output.dense", s3)
        x = m.layer_norm(b.op("elementwise_add", {"X": [x], "Y": [att]}, ("Out",), s3, axis=-1), H,
                         f"{p}.attention.output.LayerNorm", s3)
        f1 = m.linear(x, H, F, f"{p}.intermediate.dense", [-1, -1, F])
        f1 = b.op("gelu", {"X": [f1]}, ("Out",), [-1, -1, F], approximate=False)
        f2 = m.linear(f1, F, H, f"{p}.output.dense", s3)
        x = m.layer_norm(b.op("elementwise_add", {"X": [x], "Y": [f2]}, ("Out",), s3, axis=-1), H,
                         f"{p}.output.LayerNorm", s3)
    b.fetch(m.linear(x, H, num_labels, "classifier", [-1, -1, num_labels]))
    return b


def write_ser_vi_layoutxlm(out_dir: str, size: str = "tiny", num_labels: int = 7, seed: int = 0) -> Dict[str, str]:
    """Writes ``model.pdmodel`` / ``model.pdiparams`` and a class list matching ``num_labels`` (``O`` + B-/I- pairs)."""
    os.makedirs(out_dir, exist_ok=True)
    model, params = build_ser_vi_layoutxlm(size, num_labels, seed).serialize()
    paths = {"model": os.path.join(out_dir, "model.pdmodel"), "params": os.path.join(out_dir, "model.pdiparams"),
             "classes": os.path.join(out_dir, "class_list.txt")}
    with open(paths["model"], "wb") as f:
        f.write(model)
    with open(paths["params"], "wb") as f:
        f.write(params)
    names = ["OTHER"] + ["QUESTION", "ANSWER", "HEADER", "FOOTER", "TITLE", "TABLE"][:(num_labels - 1) // 2]
    with open(paths["classes"], "w") as f:
        f.write("\n".join(names) + "\n")
    return paths
