"""Synthetic ERNIE-3.0 / UIE encoder generator (Paddle inference format).

12 layers, hidden 768, 12 heads, FFN 3072, vocab 40000 for the ``base`` size; post-LayerNorm
BERT-style blocks with erf-GELU. ``task="seq_cls"`` adds pooler(tanh) + linear and takes
``input_ids, token_type_ids`` (examples/text/ernie-3.0/python/seq_cls_infer.py); ``task="uie"`` takes
``input_ids, token_type_ids, pos_ids, att_mask`` and ends in two sigmoid span heads
(fastdeploy/text/uie/model.cc:565-609). The op sequence follows a PaddleNLP export: ``lookup_table_v2``
embeddings, ``matmul_v2`` + ``elementwise_add`` linears, ``reshape2``/``transpose2`` head split,
``scale``d scores, additive mask built from the ids, ``softmax``, ``layer_norm``.
"""
from __future__ import annotations

import os
from typing import Dict, Optional

import numpy as np

from ..importer.paddle_format import ProgramBuilder

SIZES = {
    "base": dict(layers=12, hidden=768, heads=12, ffn=3072, vocab=40000, max_pos=2048, types=4),
    "medium": dict(layers=6, hidden=768, heads=12, ffn=3072, vocab=40000, max_pos=2048, types=4),
    "mini": dict(layers=6, hidden=384, heads=12, ffn=1536, vocab=40000, max_pos=2048, types=4),
    "tiny": dict(layers=2, hidden=64, heads=4, ffn=128, vocab=1000, max_pos=128, types=4),   # test size
}


class _B:
    def __init__(self, seed: int):
        self.b = ProgramBuilder()
        self.rng = np.random.default_rng(seed)

    def w(self, name, shape, scale=0.02):
        return self.b.param(name, (self.rng.standard_normal(shape) * scale).astype(np.float32))

    def vec(self, name, n, value=None):
        v = np.full(n, value, np.float32) if value is not None else (0.02 * self.rng.standard_normal(n)).astype(np.float32)
        return self.b.param(name, v)

    def linear(self, x, cin, cout, name, shape):
        w = self.w(name + ".w_0", (cin, cout))
        bias = self.vec(name + ".b_0", cout)
        y = self.b.op("matmul_v2", {"X": [x], "Y": [w]}, ("Out",), shape, trans_x=False, trans_y=False)
        return self.b.op("elementwise_add", {"X": [y], "Y": [bias]}, ("Out",), shape, axis=-1)

    def layer_norm(self, x, c, name, shape):
        g = self.b.param(name + ".w_0", (1.0 + 0.05 * self.rng.standard_normal(c)).astype(np.float32))
        bt = self.vec(name + ".b_0", c)
        return self.b.op("layer_norm", {"X": [x], "Scale": [g], "Bias": [bt]}, ("Y", "Mean", "Variance"), shape,
                         begin_norm_axis=len(shape) - 1, epsilon=1e-12)


def build_ernie(size: str = "base", task: str = "seq_cls", num_labels: int = 2, seed: int = 0) -> ProgramBuilder:
    cfg = SIZES[size]
    L, H, NH, F, V = cfg["layers"], cfg["hidden"], cfg["heads"], cfg["ffn"], cfg["vocab"]
    D = H // NH
    m = _B(seed)
    b = m.b
    ids = b.feed("input_ids", "int64", [-1, -1])
    tids = b.feed("token_type_ids", "int64", [-1, -1])
    s3 = [-1, -1, H]
    word = m.w("word_embeddings", (V, H))
    pos = m.w("position_embeddings", (cfg["max_pos"], H))
    typ = m.w("token_type_embeddings", (cfg["types"], H))
    if task == "uie":
        pos_ids = b.feed("pos_ids", "int64", [-1, -1])
        att_mask = b.feed("att_mask", "int64", [-1, -1])
        mask_f = b.op("cast", {"X": [att_mask]}, ("Out",), [-1, -1], in_dtype=3, out_dtype=5)
    else:
        # position ids = cumsum(ones) - 1 ; mask from pad id 0
        ones = b.op("fill_any_like", {"X": [ids]}, ("Out",), [-1, -1], "int64", value=1.0, dtype=3)
        csum = b.op("cumsum", {"X": [ones]}, ("Out",), [-1, -1], "int64", axis=-1, exclusive=False, reverse=False)
        pos_ids = b.op("elementwise_sub", {"X": [csum], "Y": [ones]}, ("Out",), [-1, -1], "int64", axis=-1)
        zero = b.param("pad_token_id", np.zeros(1, np.int64))
        neq = b.op("not_equal", {"X": [ids], "Y": [zero]}, ("Out",), [-1, -1], "bool", axis=-1)
        mask_f = b.op("cast", {"X": [neq]}, ("Out",), [-1, -1], in_dtype=0, out_dtype=5)
    # additive mask [B,1,1,S]: (mask - 1) * 1e4
    am = b.op("scale", {"X": [mask_f]}, ("Out",), [-1, -1], scale=1e4, bias=-1.0, bias_after_scale=False)
    am = b.op("unsqueeze2", {"X": [am]}, ("Out", "XShape"), [-1, 1, 1, -1], axes=[1, 2])
    e = b.op("lookup_table_v2", {"Ids": [ids], "W": [word]}, ("Out",), s3, padding_idx=-1)
    pe = b.op("lookup_table_v2", {"Ids": [pos_ids], "W": [pos]}, ("Out",), s3, padding_idx=-1)
    te = b.op("lookup_table_v2", {"Ids": [tids], "W": [typ]}, ("Out",), s3, padding_idx=-1)
    x = b.op("elementwise_add", {"X": [e], "Y": [pe]}, ("Out",), s3, axis=-1)
    x = b.op("elementwise_add", {"X": [x], "Y": [te]}, ("Out",), s3, axis=-1)
    x = m.layer_norm(x, H, "embeddings.layer_norm", s3)
    for l in range(L):
        p = f"encoder.layers.{l}"
        qkv = []
        for nm in ("q_proj", "k_proj", "v_proj"):
            t = m.linear(x, H, H, f"{p}.self_attn.{nm}", s3)
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
        att = m.linear(ctx, H, H, f"{p}.self_attn.out_proj", s3)
        x = m.layer_norm(b.op("elementwise_add", {"X": [x], "Y": [att]}, ("Out",), s3, axis=-1), H, f"{p}.norm1", s3)
        f1 = m.linear(x, H, F, f"{p}.linear1", [-1, -1, F])
        f1 = b.op("gelu", {"X": [f1]}, ("Out",), [-1, -1, F], approximate=False)
        f2 = m.linear(f1, F, H, f"{p}.linear2", s3)
        x = m.layer_norm(b.op("elementwise_add", {"X": [x], "Y": [f2]}, ("Out",), s3, axis=-1), H, f"{p}.norm2", s3)
    if task == "seq_cls":
        cls = b.op("slice", {"Input": [x]}, ("Out",), [-1, H], axes=[1], starts=[0], ends=[1], decrease_axis=[1],
                   infer_flags=[1])
        pooled = m.linear(cls, H, H, "pooler.dense", [-1, H])
        pooled = b.op("tanh", {"X": [pooled]}, ("Out",), [-1, H])
        logits = m.linear(pooled, H, num_labels, "classifier", [-1, num_labels])
        b.fetch(logits)
    elif task == "uie":
        for nm in ("linear_start", "linear_end"):
            t = m.linear(x, H, 1, nm, [-1, -1, 1])
            t = b.op("squeeze2", {"X": [t]}, ("Out", "XShape"), [-1, -1], axes=[-1])
            t = b.op("sigmoid", {"X": [t]}, ("Out",), [-1, -1])
            b.fetch(t)
    elif task == "token_cls":
        b.fetch(m.linear(x, H, num_labels, "classifier", [-1, -1, num_labels]))
    else:
        b.fetch(x)
    return b


def write_ernie(out_dir: str, size: str = "base", task: str = "seq_cls", seed: int = 0, vocab: bool = True,
                **kw) -> Dict[str, str]:
    os.makedirs(out_dir, exist_ok=True)
    b = build_ernie(size, task, seed=seed, **kw)
    model, params = b.serialize()
    paths = {"model": os.path.join(out_dir, "model.pdmodel"), "params": os.path.join(out_dir, "model.pdiparams"),
             "vocab": os.path.join(out_dir, "vocab.txt")}
    with open(paths["model"], "wb") as f:
        f.write(model)
    with open(paths["params"], "wb") as f:
        f.write(params)
    if vocab:
        from ..text.tokenizer import write_synthetic_vocab
        write_synthetic_vocab(paths["vocab"], SIZES[size]["vocab"])
    return paths
