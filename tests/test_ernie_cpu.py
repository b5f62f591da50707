"""ERNIE generator -> Paddle importer -> fusion passes keep the outputs (CPU)."""
import numpy as np
import pytest


@pytest.mark.parametrize("task", ["seq_cls", "uie"])
def test_ernie_tiny_fusion_equivalence(task):
    from fastdeploy_b200.importer.paddle_import import load_paddle
    from fastdeploy_b200.ir.interp import Interpreter
    from fastdeploy_b200.ir.passes import optimize
    from fastdeploy_b200.models.ernie import build_ernie
    g = load_paddle(*build_ernie("tiny", task).serialize())
    B, S = 2, 16
    rng = np.random.RandomState(0)
    ids = rng.randint(1, 1000, (B, S)).astype(np.int64)
    ids[1, 10:] = 0
    feeds = {"input_ids": ids, "token_type_ids": np.zeros((B, S), np.int64)}
    if task == "uie":
        feeds["pos_ids"] = np.tile(np.arange(S), (B, 1)).astype(np.int64)
        feeds["att_mask"] = (ids != 0).astype(np.int64)
    shapes = {k: list(v.shape) for k, v in feeds.items()}
    ref = Interpreter(g).run(feeds)
    g2 = optimize(g, shapes, level=2)
    hist = g2.op_histogram()
    assert hist.get("Attention") == 2 and hist.get("EmbedLayerNorm") == 1 and hist.get("FusedGemm", 0) >= 10, hist
    assert "Softmax" not in hist and "Transpose" not in hist and "Erf" not in hist
    out = Interpreter(g2).run(feeds)
    for k in ref:
        assert float((ref[k] - out[k]).abs().max()) < 1e-5


def test_vit_tiny_fusion_equivalence():
    from fastdeploy_b200.importer.paddle_import import load_paddle
    from fastdeploy_b200.ir.interp import Interpreter
    from fastdeploy_b200.ir.passes import optimize
    from fastdeploy_b200.models.vit import build_vit
    g = load_paddle(*build_vit("tiny", image=32, num_classes=10).serialize())
    x = np.random.RandomState(0).randn(2, 3, 32, 32).astype(np.float32)
    ref = Interpreter(g).run({"x": x})
    g2 = optimize(g, {"x": [2, 3, 32, 32]}, level=2)
    hist = g2.op_histogram()
    assert hist.get("Attention") == 2 and hist.get("FusedGemm", 0) >= 9 and hist.get("LayerNormalization", 0) >= 5, hist
    out = Interpreter(g2).run({"x": x})
    for k in ref:
        assert float((ref[k] - out[k]).abs().max()) < 1e-5
        assert abs(float(out[k].sum()) - 2.0) < 1e-4        # two softmax rows
