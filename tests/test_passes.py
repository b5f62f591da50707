"""Graph passes keep the numerics: pass-on == pass-off through the reference interpreter (CPU)."""
import numpy as np
import pytest


def _run(g, feeds):
    from fastdeploy_b200.ir.interp import Interpreter
    return {k: v.float().numpy() for k, v in Interpreter(g).run(feeds).items()}


def test_resnet_fusion_equivalence():
    from fastdeploy_b200.ir.passes import optimize
    from fastdeploy_b200.models.resnet import build_resnet
    g = build_resnet((1, 1, 1, 1), num_classes=10, width=16, image=64)
    x = np.random.RandomState(0).rand(2, 3, 64, 64).astype(np.float32)
    ref = _run(g, {"input": x})["output"]
    g2 = optimize(g, {"input": [2, 3, 64, 64]}, level=2)
    hist = g2.op_histogram()
    assert "BatchNormalization" not in hist and "Relu" not in hist and "Add" not in hist
    assert hist["FusedConv"] == 17 and hist["FusedGemm"] == 1
    out = _run(g2, {"input": x})["output"]
    assert np.abs(out - ref).max() < 1e-5
    # residual add before the activation for the ResNet pattern
    assert any(n.attr("res_mode") == 1 for n in g2.nodes if n.op == "FusedConv")


@pytest.mark.parametrize("level", [1, 2])
def test_ppyoloe_tiny_equivalence(level):
    from fastdeploy_b200.importer.paddle_import import load_paddle
    from fastdeploy_b200.ir.passes import optimize
    from fastdeploy_b200.models.ppyoloe import build_ppyoloe
    net = build_ppyoloe("tiny", image=96, num_classes=6, score_threshold=0.005)
    g = load_paddle(*net.serialize())
    x = np.random.RandomState(1).rand(2, 3, 96, 96).astype(np.float32)
    sf = np.array([[1.0, 1.0], [0.5, 0.75]], np.float32)
    ref = _run(g, {"image": x, "scale_factor": sf})
    g2 = optimize(g, {"image": [2, 3, 96, 96], "scale_factor": [2, 2]}, level=level)
    out = _run(g2, {"image": x, "scale_factor": sf})
    if level == 2:
        assert g2.op_histogram().get("PPYOLOEPost") == 1
        assert "Softmax" not in g2.op_histogram() and "Silu" not in g2.op_histogram()
    for k in ref:
        assert out[k].shape == ref[k].shape and ref[k].size > 0
        assert np.abs(out[k] - ref[k]).max() < 5e-4


def test_repvgg_and_silu_patterns():
    from fastdeploy_b200.ir.graph import Graph
    from fastdeploy_b200.ir.passes import optimize
    rng = np.random.RandomState(3)
    g = Graph()
    g.add_input("x", "float32", [1, 8, 10, 10])
    w3 = g.add_initializer("w3", rng.randn(8, 8, 3, 3).astype(np.float32) * 0.1)
    w1 = g.add_initializer("w1", rng.randn(8, 8, 1, 1).astype(np.float32) * 0.1)
    b3 = g.add_initializer("b3", rng.randn(8).astype(np.float32))
    a = g.op("Conv", "x", w3, b3, pads=[1, 1, 1, 1], strides=[1, 1], kernel_shape=[3, 3])
    b = g.op("Conv", "x", w1, pads=[0, 0, 0, 0], strides=[1, 1], kernel_shape=[1, 1])
    s = g.op("Add", a, b)
    y = g.op("Mul", s, g.op("Sigmoid", s))
    g.nodes[-1].outputs = ["y"]
    g.add_output("y")
    x = rng.randn(1, 8, 10, 10).astype(np.float32)
    ref = _run(g, {"x": x})["y"]
    g2 = optimize(g, {"x": [1, 8, 10, 10]}, level=2)
    assert [n.op for n in g2.nodes] == ["FusedConv"] and g2.nodes[0].attr("activation") == "silu"
    assert np.abs(_run(g2, {"x": x})["y"] - ref).max() < 1e-5


def test_gelu_layernorm_attention_recognition():
    import math
    from fastdeploy_b200.ir.graph import Graph
    from fastdeploy_b200.ir.passes import optimize
    rng = np.random.RandomState(4)
    B, S, H, D = 2, 6, 2, 4
    g = Graph(opset=13)
    g.add_input("x", "float32", [B, S, H * D])
    g.add_input("mask", "float32", [B, 1, 1, S])

    def lin(inp, name):
        w = g.add_initializer(name + ".w", rng.randn(H * D, H * D).astype(np.float32) * 0.3)
        b = g.add_initializer(name + ".b", rng.randn(H * D).astype(np.float32) * 0.1)
        return g.op("Add", g.op("MatMul", inp, w), b)

    def heads(t):
        r = g.op("Reshape", t, g.const(np.array([0, 0, H, D], np.int64)))
        return g.op("Transpose", r, perm=[0, 2, 1, 3])
    q, k, v = lin("x", "q"), lin("x", "k"), lin("x", "v")
    att = g.op("MatMul", heads(q), g.op("Transpose", heads(k), perm=[0, 1, 3, 2]))
    att = g.op("Mul", att, g.const(np.float32(1 / math.sqrt(D))))
    att = g.op("Softmax", g.op("Add", att, "mask"), axis=-1)
    ctx = g.op("Transpose", g.op("MatMul", att, heads(v)), perm=[0, 2, 1, 3])
    ctx = g.op("Reshape", ctx, g.const(np.array([0, 0, H * D], np.int64)))
    h = g.op("Add", lin(ctx, "o"), "x")
    # decomposed LayerNorm
    mean = g.op("ReduceMean", h, axes=[-1], keepdims=1)
    d = g.op("Sub", h, mean)
    var = g.op("ReduceMean", g.op("Pow", d, g.const(np.float32(2.0))), axes=[-1], keepdims=1)
    nrm = g.op("Div", d, g.op("Sqrt", g.op("Add", var, g.const(np.float32(1e-5)))))
    gamma = g.add_initializer("gamma", rng.rand(H * D).astype(np.float32) + 0.5)
    beta = g.add_initializer("beta", rng.randn(H * D).astype(np.float32))
    ln = g.op("Add", g.op("Mul", nrm, gamma), beta)
    # erf GELU
    f = lin(ln, "ffn")
    e = g.op("Erf", g.op("Div", f, g.const(np.float32(math.sqrt(2)))))
    ge = g.op("Mul", g.op("Mul", f, g.op("Add", e, g.const(np.float32(1.0)))), g.const(np.float32(0.5)))
    g.nodes[-1].outputs = ["y"]
    g.add_output("y")
    x = rng.randn(B, S, H * D).astype(np.float32)
    mask = np.zeros((B, 1, 1, S), np.float32)
    mask[1, ..., 4:] = -1e4
    ref = _run(g, {"x": x, "mask": mask})["y"]
    g2 = optimize(g, {"x": [B, S, H * D], "mask": [B, 1, 1, S]}, level=2)
    hist = g2.op_histogram()
    assert hist.get("Attention") == 1 and hist.get("LayerNormalization") == 1, hist
    assert "Erf" not in hist and "Softmax" not in hist and "Transpose" not in hist
    gem = [n for n in g2.nodes if n.op == "FusedGemm"]
    # q / k / v projections are one stacked GEMM (+ three channel slices), then out-proj and the two FFN layers
    assert len(gem) == 3 and hist.get("Slice") == 3
    assert any(n.attr("activation") == "gelu" for n in gem) and any(n.attr("res_mode") == 2 for n in gem)
    assert np.abs(_run(g2, {"x": x, "mask": mask})["y"] - ref).max() < 1e-5


def test_optimised_graph_disk_cache_round_trip(tmp_path):
    """The on-disk plan cache stores the optimised graph (fused ops included) and a second start loads it
    instead of running the passes; both graphs compute the same outputs."""
    import os
    import numpy as np
    import torch
    from fastdeploy_b200.importer.paddle_import import load_paddle
    from fastdeploy_b200.ir import passes
    from fastdeploy_b200.ir.interp import Interpreter
    from fastdeploy_b200.models.ernie import build_ernie
    from fastdeploy_b200.runtime import native_backend as nb
    g = load_paddle(*build_ernie("tiny").serialize())
    shapes = {"input_ids": [2, 16], "token_type_ids": [2, 16]}
    g1 = nb.optimize_cached(g, shapes, None, 2, torch.float16, str(tmp_path))
    files = os.listdir(tmp_path)
    assert len(files) == 1 and files[0].endswith(".fdbgraph")
    calls = []
    orig = passes.optimize
    passes.optimize = lambda *a, **k: calls.append(1) or orig(*a, **k)
    try:
        g2 = nb.optimize_cached(load_paddle(*build_ernie("tiny").serialize()), shapes, None, 2, torch.float16, str(tmp_path))
    finally:
        passes.optimize = orig
    assert not calls, "second start must come from the cache"
    assert nb.graph_fingerprint(g, shapes, torch.float16, 2) != nb.graph_fingerprint(g, shapes, torch.bfloat16, 2)
    feeds = {"input_ids": np.random.default_rng(0).integers(1, 1000, (2, 16)).astype(np.int64),
             "token_type_ids": np.zeros((2, 16), np.int64)}
    a, b = Interpreter(g1).run(feeds), Interpreter(g2).run(feeds)
    for k in a:
        assert np.array_equal(np.asarray(a[k]), np.asarray(b[k]))


def test_fp32_to_fp16_converter_keeps_io_and_blocked_ops():
    import numpy as np
    import torch
    from fastdeploy_b200.importer.onnx_format import load_onnx, save_onnx
    from fastdeploy_b200.ir.convert_fp16 import convert_fp32_to_fp16
    from fastdeploy_b200.ir.graph import Graph
    from fastdeploy_b200.ir.interp import Interpreter
    rng = np.random.RandomState(0)
    g = Graph()
    g.add_input("x", "float32", [2, 8, 12, 12])
    w1 = g.const((rng.randn(16, 8, 3, 3) * 0.1).astype(np.float32), prefix="w1")
    b1 = g.const(np.array([1e-9] * 8 + [0.1] * 8, np.float32), prefix="b1")         # tiny values must not flush to zero
    g.add_node("Conv", ["x", w1, b1], ["c1"], kernel_shape=[3, 3], pads=[1, 1, 1, 1])
    g.add_node("Relu", ["c1"], ["r1"])
    scales = g.const(np.array([1, 1, 2, 2], np.float32), prefix="scales")
    g.add_node("Resize", ["r1", "", scales], ["up"], mode="nearest")                    # stays fp32, its scales too
    g.add_node("GlobalAveragePool", ["up"], ["gap"])
    g.add_node("Flatten", ["gap"], ["flat"], axis=1)
    w2 = g.const((rng.randn(16, 5) * 0.2).astype(np.float32), prefix="w2")
    g.add_node("MatMul", ["flat", w2], ["logits"])
    g.add_node("Softmax", ["logits"], ["prob"], axis=-1)                                 # stays fp32
    g.add_node("ArgMax", ["prob"], ["label"], axis=1, keepdims=0)
    g.add_output("prob", "float32", [2, 5])
    g.add_output("label", "int64", [2])
    h = convert_fp32_to_fp16(g)
    assert h.initializers[w1].dtype == np.float16 and h.initializers[w2].dtype == np.float16
    assert h.initializers[scales].dtype == np.float32
    assert float(np.abs(h.initializers[b1][:8]).min()) > 0            # raised to the smallest kept magnitude
    ops = [n.op for n in h.nodes]
    assert ops.count("Cast") >= 4 and [vi.dtype for vi in h.inputs] == ["float32"]
    x = rng.rand(2, 8, 12, 12).astype(np.float32)
    ref = Interpreter(g).run({"x": x})
    got = Interpreter(load_onnx(save_onnx(h))).run({"x": x})          # survives serialisation
    assert got["prob"].dtype == torch.float32 and got["label"].dtype == torch.int64
    assert torch.allclose(got["prob"], ref["prob"], atol=3e-3)
    resize = [n for n in h.nodes if n.op == "Resize"][0]
    prod = h.producers()
    assert prod[resize.inputs[0]].op == "Cast" and prod[resize.inputs[0]].attr("to") == 1
    # without kept i/o types the graph takes and returns half precision
    h2 = convert_fp32_to_fp16(g, keep_io_types=False)
    assert h2.inputs[0].dtype == "float16"


def test_qlinear_model_becomes_a_float_graph_with_calibrated_ranges():
    """A quantised ONNX model in operator form (QuantizeLinear -> QLinearConv x 2 -> QLinearGlobalAveragePool ->
    QLinearMatMul -> DequantizeLinear, with a branch through QLinearAdd): the expansion gives the same integers as
    the integer operators, and the optimiser turns it into a float graph that stays within quantisation noise."""
    from fastdeploy_b200.ir.graph import Graph, ValueInfo
    from fastdeploy_b200.ir.interp import Interpreter
    from fastdeploy_b200.ir.passes import expand_qlinear, get_act_scales, optimize
    rng = np.random.RandomState(7)
    g = Graph("q", 13)
    g.inputs.append(ValueInfo("x", "float32", [2, 3, 8, 8]))

    def c(name, v):
        g.initializers[name] = np.asarray(v)
        return name
    xs, xz = c("xs", np.float32(0.02)), c("xz", np.uint8(128))
    g.add_node("QuantizeLinear", ["x", xs, xz], ["xq"])
    w1 = c("w1", rng.randint(-90, 90, (4, 3, 3, 3)).astype(np.int8))
    w1s, w1z = c("w1s", (rng.rand(4) * 0.0005 + 0.0008).astype(np.float32)), c("w1z", np.zeros(4, np.int8))
    b1 = c("b1", rng.randint(-3000, 3000, 4).astype(np.int32))
    y1s, y1z = c("y1s", np.float32(0.012)), c("y1z", np.uint8(125))
    g.add_node("QLinearConv", ["xq", xs, xz, w1, w1s, w1z, y1s, y1z, b1], ["y1q"], pads=[1, 1, 1, 1])
    w2 = c("w2", rng.randint(-90, 90, (4, 4, 1, 1)).astype(np.int8))
    w2s, w2z = c("w2s", np.float32(0.01)), c("w2z", np.int8(0))
    y2s, y2z = c("y2s", np.float32(0.025)), c("y2z", np.uint8(128))
    g.add_node("QLinearConv", ["y1q", y1s, y1z, w2, w2s, w2z, y2s, y2z], ["y2q"])
    ys3, yz3 = c("y3s", np.float32(0.035)), c("y3z", np.uint8(127))
    g.add_node("QLinearAdd", ["y1q", y1s, y1z, "y2q", y2s, y2z, ys3, yz3], ["y3q"], domain="com.microsoft")
    ps, pz = c("ps", np.float32(0.03)), c("pz", np.uint8(118))
    g.add_node("QLinearGlobalAveragePool", ["y3q", ys3, yz3, ps, pz], ["pq"], domain="com.microsoft", channels_last=0)
    g.add_node("Flatten", ["pq"], ["fq"], axis=1)
    w3 = c("w3", rng.randint(0, 255, (4, 5)).astype(np.uint8))
    w3s, w3z = c("w3s", np.float32(0.004)), c("w3z", np.uint8(127))
    os_, oz = c("os", np.float32(0.01)), c("oz", np.uint8(128))
    g.add_node("QLinearMatMul", ["fq", ps, pz, w3, w3s, w3z, os_, oz], ["oq"])
    g.add_node("DequantizeLinear", ["oq", os_, oz], ["out"])
    g.outputs.append(ValueInfo("out", "float32", [2, 5]))
    x = (rng.rand(2, 3, 8, 8).astype(np.float32) - 0.5) * 4

    # (1) the expansion alone keeps the integer arithmetic to within one step of the last scale
    e = g.clone()
    assert expand_qlinear(e) == 5
    assert not any(n.op.startswith("QLinear") for n in e.nodes)
    out_e = Interpreter(e).run({"x": x})["out"].numpy()
    # the standard-set operators exist in the interpreter: run the two convolutions of the original as a cross-check
    head = Graph("head", 13)
    head.inputs, head.initializers = list(g.inputs), dict(g.initializers)
    head.nodes = [n for n in g.clone().nodes[:3]]
    head.outputs.append(ValueInfo("y2q", "uint8", None))
    head_e = Graph("head_e", 13)
    head_e.inputs, head_e.initializers = list(e.inputs), dict(e.initializers)
    head_e.nodes = list(e.clone().nodes)
    head_e.outputs.append(ValueInfo("y2q", "uint8", None))
    head_e.prune()
    a = Interpreter(head).run({"x": x})["y2q"].numpy().astype(int)
    b = Interpreter(head_e).run({"x": x})["y2q"].numpy().astype(int)
    assert np.abs(a - b).max() <= 1
    # (2) the optimiser leaves a float graph: no quantise / dequantise node, ranges recorded for the activations
    f = optimize(g, {"x": [2, 3, 8, 8]}, level=2)
    ops = {n.op for n in f.nodes}
    assert not any(o in ops for o in ("QuantizeLinear", "DequantizeLinear", "QLinearConv", "QLinearMatMul")), ops
    ranges = get_act_scales(f)
    assert abs(ranges["x"] - 0.02 * 128) < 1e-6 and len(ranges) >= 5
    out_f = Interpreter(f).run({"x": x})["out"].numpy()
    assert out_f.shape == (2, 5) and np.abs(out_f - out_e).max() < 0.06                # a few output steps of 0.01
    assert np.abs(out_e).max() > 0.05                                                    # (and the outputs are not all zero)
