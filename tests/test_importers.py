"""Wire codec, ONNX and Paddle readers/writers, importer -> interpreter round trips (CPU)."""
import struct

import numpy as np
import pytest


def test_protowire_roundtrip_and_unknown_fields():
    from fastdeploy_b200.importer import protowire as pw
    inner = {1: ("a", "int", False), 2: ("b", "str", False)}
    schema = {1: ("i", "int", False), 2: ("f", "float", True), 3: ("s", "str", True), 4: ("m", inner, True),
              5: ("d", "double", False), 6: ("neg", "int", True), 7: ("raw", "bytes", False), 8: ("flag", "bool", False)}
    msg = {"i": 1 << 40, "f": [1.5, -2.25], "s": ["x", "héllo"], "m": [{"a": -7, "b": "q"}, {"a": 3}], "d": 3.5,
           "neg": [-1, -(1 << 62), 5], "raw": b"\x00\xff", "flag": True}
    for packed in (True, False):
        back = pw.decode(pw.encode(msg, schema, packed=packed), schema)
        assert back["i"] == msg["i"] and back["f"] == msg["f"] and back["s"] == msg["s"]
        assert back["m"][0] == {"a": -7, "b": "q"} and back["m"][1]["a"] == 3
        assert back["neg"] == msg["neg"] and back["raw"] == msg["raw"] and back["flag"] is True and back["d"] == 3.5
    # a reader with a smaller schema skips what it does not know
    small = {1: ("i", "int", False)}
    assert pw.decode(pw.encode(msg, schema), small) == {"i": 1 << 40}
    with pytest.raises(pw.WireError):
        pw.decode(b"\x0a\x05abc", schema)          # truncated length-delimited field


def test_onnx_roundtrip_and_interpreter():
    from fastdeploy_b200.importer.onnx_format import load_onnx, save_onnx
    from fastdeploy_b200.ir.interp import Interpreter
    from fastdeploy_b200.models.resnet import build_resnet
    g = build_resnet((1, 1, 1, 1), num_classes=10, width=8, image=32, softmax=True)
    data = save_onnx(g)
    g2 = load_onnx(data)
    assert [n.op for n in g2.nodes] == [n.op for n in g.nodes]
    assert g2.opset == 11 and g2.inputs[0].shape == ["N", 3, 32, 32]
    x = np.random.RandomState(0).rand(2, 3, 32, 32).astype(np.float32)
    a = Interpreter(g).run({"input": x})["output"]
    b = Interpreter(g2).run({"input": x})["output"]
    assert np.array_equal(a.numpy(), b.numpy())
    assert np.allclose(a.sum(1).numpy(), 1.0, atol=1e-5)


def test_interpreter_conv_matches_torch():
    import torch
    from fastdeploy_b200.ir.graph import Graph
    from fastdeploy_b200.ir.interp import Interpreter
    rng = np.random.RandomState(1)
    g = Graph()
    g.add_input("x", "float32", [1, 4, 9, 9])
    w = g.add_initializer("w", rng.randn(6, 2, 3, 3).astype(np.float32))
    b = g.add_initializer("b", rng.randn(6).astype(np.float32))
    y = g.op("Conv", "x", w, b, strides=[2, 2], pads=[1, 0, 1, 2], group=2, dilations=[1, 1], kernel_shape=[3, 3])
    g.nodes[-1].outputs = ["y"]
    g.add_output("y")
    x = rng.randn(1, 4, 9, 9).astype(np.float32)
    got = Interpreter(g).run({"x": x})["y"]
    xp = torch.nn.functional.pad(torch.from_numpy(x), (0, 2, 1, 1))
    ref = torch.nn.functional.conv2d(xp, torch.from_numpy(g.initializers["w"]), torch.from_numpy(g.initializers["b"]),
                                     stride=2, groups=2)
    assert torch.allclose(got, ref, atol=1e-5)


def test_paddle_write_read_roundtrip_sorted_params():
    from fastdeploy_b200.importer.paddle_format import ProgramBuilder, parse_params, parse_program
    b = ProgramBuilder()
    b.feed("x", "float32", [-1, 4])
    w2 = b.param("zeta.w", np.arange(8, dtype=np.float32).reshape(4, 2))
    w1 = b.param("alpha.b", np.array([1.0, -1.0], np.float32))
    y = b.op("matmul_v2", {"X": ["x"], "Y": [w2]}, ("Out",), [-1, 2], trans_x=False, trans_y=False)
    z = b.op("elementwise_add", {"X": [y], "Y": [w1]}, ("Out",), [-1, 2], axis=-1)
    b.fetch(z)
    model, params = b.serialize()
    prog = parse_program(model)
    assert prog.param_names() == ["alpha.b", "zeta.w"]           # sorted by name = record order
    assert prog.feed_names() == ["x"] and prog.fetch_names() == [z]
    p = parse_params(prog, params)
    assert np.array_equal(p["zeta.w"], np.arange(8, dtype=np.float32).reshape(4, 2))
    # first record in the file is alpha.b: header (20 bytes) + desc, then 2 floats
    _, lod, _, dsz = struct.unpack_from("<IQIi", params, 0)
    assert lod == 0 and np.frombuffer(params[20 + dsz:20 + dsz + 8], np.float32).tolist() == [1.0, -1.0]
    # lod_level != 0 is rejected
    bad = bytearray(params)
    struct.pack_into("<Q", bad, 4, 1)
    with pytest.raises(ValueError):
        parse_params(prog, bytes(bad))
    with pytest.raises(ValueError):
        parse_params(prog, params[:-3])


def test_paddle_import_semantics():
    """scale bias order, hard_sigmoid slope/offset, pool2d adaptive, elementwise axis, flatten range."""
    import torch
    from fastdeploy_b200.importer.paddle_format import ProgramBuilder
    from fastdeploy_b200.importer.paddle_import import load_paddle
    from fastdeploy_b200.ir.interp import Interpreter
    b = ProgramBuilder()
    b.feed("x", "float32", [-1, 4, 6, 6])
    bias = b.param("bias", np.array([1, 2, 3, 4], np.float32))
    t = b.op("elementwise_add", {"X": ["x"], "Y": [bias]}, ("Out",), [-1, 4, 6, 6], axis=1)
    t = b.op("scale", {"X": [t]}, ("Out",), [-1, 4, 6, 6], scale=2.0, bias=1.0, bias_after_scale=False)
    t = b.op("hard_sigmoid", {"X": [t]}, ("Out",), [-1, 4, 6, 6], slope=0.1, offset=0.3)
    t = b.op("pool2d", {"X": [t]}, ("Out",), [-1, 4, 3, 3], pooling_type="avg", ksize=[3, 3], adaptive=True,
             global_pooling=False, strides=[1, 1], paddings=[0, 0], exclusive=True, ceil_mode=False,
             padding_algorithm="EXPLICIT")
    t = b.op("flatten_contiguous_range", {"X": [t]}, ("Out", "XShape"), [-1, 36], start_axis=1, stop_axis=3)
    b.fetch(t)
    g = load_paddle(*b.serialize())
    x = np.random.RandomState(2).randn(2, 4, 6, 6).astype(np.float32)
    got = Interpreter(g).run({"x": x})[g.output_names()[0]]
    xt = torch.from_numpy(x) + torch.tensor([1., 2., 3., 4.]).view(1, 4, 1, 1)
    xt = torch.clamp(0.1 * ((xt + 1.0) * 2.0) + 0.3, 0, 1)
    ref = torch.nn.functional.adaptive_avg_pool2d(xt, 3).reshape(2, -1)
    assert torch.allclose(got, ref, atol=1e-6)


def test_paddle_importer_rejects_unknown_op():
    from fastdeploy_b200.importer.paddle_format import ProgramBuilder
    from fastdeploy_b200.importer.paddle_import import load_paddle, supported_paddle_ops
    b = ProgramBuilder()
    b.feed("x", "float32", [-1, 4])
    t = b.op("some_future_op", {"X": ["x"]}, ("Out",), [-1, 4])
    b.fetch(t)
    with pytest.raises(NotImplementedError):
        load_paddle(*b.serialize())
    assert len(supported_paddle_ops()) >= 120


def test_converter_entry_points():
    """export / is_exportable / readers / remove_multiclass_nms / fp16 conversion, as the reference's converter offers."""
    from fastdeploy_b200 import importer as I
    from fastdeploy_b200.ir.interp import Interpreter
    from fastdeploy_b200.models.ppyoloe import build_ppyoloe
    net = build_ppyoloe("tiny", image=64, num_classes=4, with_nms=True, score_threshold=0.05)
    model, params = net.serialize()
    assert I.is_exportable(model, params) and I.unsupported_ops(model) == []
    pr = I.PaddleReader(model)
    assert [t.name for t in pr.inputs] == ["image", "scale_factor"] and pr.num_outputs == 2 and pr.has_nms
    assert not pr.is_quantize_model and pr.inputs[0].shape[1:] == [3, 64, 64]
    onnx_bytes = I.export(model, params)
    orr = I.OnnxReader(onnx_bytes)
    assert orr.num_inputs == 2 and orr.num_outputs == 2 and orr.inputs[0].dtype == "float32"
    cut, p = I.remove_multiclass_nms(onnx_bytes)
    assert p is not None and abs(p.score_threshold - 0.05) < 1e-9 and p.keep_top_k > 0
    g = I.load_onnx(cut)
    assert not any(n.op == "MultiClassNMS" for n in g.nodes) and len(g.outputs) == 2
    x = np.random.RandomState(0).rand(1, 3, 64, 64).astype(np.float32)
    out = Interpreter(g).run({"image": x, "scale_factor": np.ones((1, 2), np.float32)})
    boxes, scores = (out[v.name].numpy() for v in g.outputs)
    assert boxes.shape[0] == 1 and boxes.shape[-1] == 4 and scores.shape[1] == 4          # [N, M, 4] and [N, C, M]
    again, none = I.remove_multiclass_nms(cut)
    assert none is None and again == cut
    half = I.convert_fp32_to_fp16(cut)
    gh = I.load_onnx(half)
    assert any(v.dtype == np.float16 for v in gh.initializers.values())
    out_h = Interpreter(gh).run({"image": x, "scale_factor": np.ones((1, 2), np.float32)})
    assert np.abs(out_h[g.outputs[1].name].float().numpy() - scores).max() < 5e-2
    # an operator the importer does not know makes the model non-exportable, and is named
    from fastdeploy_b200.importer.paddle_format import ProgramBuilder
    b = ProgramBuilder()
    xin = b.feed("x", "float32", [1, 4])
    b.fetch(b.op("some_future_op", {"X": [xin]}, ("Out",), [1, 4]))
    m2, _ = b.serialize()
    assert not I.is_exportable(m2) and I.unsupported_ops(m2) == ["some_future_op"]


def test_custom_operators_pass_through_the_export():
    from fastdeploy_b200 import importer as I
    from fastdeploy_b200.importer.paddle_format import ProgramBuilder
    b = ProgramBuilder()
    x = b.feed("x", "float32", [1, 4])
    y = b.op("relu", {"X": [x]}, ("Out",), [1, 4])
    z = b.op("my_plugin", {"X": [y], "Aux": [x]}, ("Out",), [1, 4], radius=3, mode="fast", taps=[1, 2, 3])
    b.fetch(b.op("scale", {"X": [z]}, ("Out",), [1, 4], scale=2.0, bias=0.0, bias_after_scale=True))
    model, params = b.serialize()
    assert not I.is_exportable(model)
    g = I.load_onnx(I.export(model, params, custom_ops={"my_plugin": "MyPluginV2"}))
    node = [n for n in g.nodes if n.op == "MyPluginV2"][0]
    assert node.domain == "custom" and node.inputs == [x, y] and node.attr("radius") == 3 and node.attr("mode") == "fast"
    assert node.attr("taps") == [1, 2, 3] and node.attr("input_slots") == ["Aux:1", "X:1"]
    assert [n.op for n in g.nodes] == ["Relu", "MyPluginV2", "Mul"] or len(g.nodes) >= 3
