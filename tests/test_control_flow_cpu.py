"""Paddle control flow (while, conditional_block + select_input) through the importer, the ONNX writer / reader and
the interpreter. The reference exports ``while`` as an ONNX Loop (paddle2onnx/mapper/loop.cc)."""
import numpy as np
import pytest

from fastdeploy_b200.importer.onnx_format import load_onnx, save_onnx
from fastdeploy_b200.importer.paddle_format import ProgramBuilder
from fastdeploy_b200.importer.paddle_import import load_paddle
from fastdeploy_b200.ir.interp import Interpreter


def _while_program():
    """acc = x; i = 0; while i < n: acc = acc * w + 1; i += 1   (w a parameter read from the enclosing scope)"""
    b = ProgramBuilder()
    x = b.feed("x", "float32", [-1, 3])
    n = b.feed("n", "int64", [1])
    w = b.param("w", np.asarray([0.5, 2.0, -1.0], np.float32))
    i = b.op("fill_constant", {}, ("Out",), [1], "int64", shape=[1], value=0.0, dtype=3)
    acc = b.op("assign", {"X": [x]}, ("Out",), [-1, 3])
    cond = b.op("less_than", {"X": [i], "Y": [n]}, ("Out",), [1], "bool", axis=-1)
    block = b.sub_block([
        ("elementwise_mul", {"X": [acc], "Y": [w]}, {"Out": ["t0"]}, {"axis": -1}),
        ("scale", {"X": ["t0"]}, {"Out": [acc]}, {"scale": 1.0, "bias": 1.0, "bias_after_scale": True}),
        ("increment", {"X": [i]}, {"Out": [i]}, {"step": 1.0}),
        ("less_than", {"X": [i], "Y": [n]}, {"Out": [cond]}, {"axis": -1}),
    ], new_vars=[("t0", "float32", [-1, 3])])
    b.prog.add_var("scopes", var_type=17)
    b.prog.add_op("while", {"X": [acc, i, n, w], "Condition": [cond]}, {"Out": [acc, i, cond], "StepScopes": ["scopes"]},
                  sub_block=block, is_test=True)
    out = b.op("scale", {"X": [acc]}, ("Out",), [-1, 3], scale=2.0, bias=0.0, bias_after_scale=True)
    b.fetch(out)
    b.fetch(i)
    return b.serialize()


def _reference_while(x, n):
    acc, w = x.copy(), np.asarray([0.5, 2.0, -1.0], np.float32)
    for _ in range(n):
        acc = acc * w + 1
    return acc * 2


@pytest.mark.parametrize("trips", [0, 1, 5])
def test_while_becomes_a_loop_and_runs(trips):
    model, params = _while_program()
    g = load_paddle(model, params)
    loops = [nd for nd in g.nodes if nd.op == "Loop"]
    assert len(loops) == 1 and "w" in loops[0].attr("outer_refs")
    body = loops[0].attr("body")
    assert len(body.inputs) == 2 + 2 and len(body.outputs) == 1 + 2          # (iter, cond, acc, i) -> (cond, acc, i)
    x = np.random.default_rng(0).standard_normal((2, 3)).astype(np.float32)
    feeds = {"x": x, "n": np.asarray([trips], np.int64)}
    outs = Interpreter(g).run(feeds)
    names = g.output_names()
    assert np.allclose(outs[names[0]].numpy(), _reference_while(x, trips), atol=1e-5)
    assert int(outs[names[1]].numpy().reshape(-1)[0]) == trips
    # pruning keeps what only the body reads, and the graph survives the ONNX writer and reader
    g.prune()
    assert "w" in g.initializers
    g2 = load_onnx(save_onnx(g))
    outs2 = Interpreter(g2).run(feeds)
    assert np.allclose(outs2[names[0]].numpy(), _reference_while(x, trips), atol=1e-5)


def test_runtime_runs_a_model_with_a_loop_on_the_cpu(tmp_path):
    import fastdeploy_b200 as fd
    model, params = _while_program()
    (tmp_path / "m.pdmodel").write_bytes(model)
    (tmp_path / "m.pdiparams").write_bytes(params)
    opt = fd.RuntimeOption()
    opt.use_cpu()
    opt.set_model_path(str(tmp_path / "m.pdmodel"), str(tmp_path / "m.pdiparams"))
    rt = fd.Runtime(opt)
    x = np.ones((4, 3), np.float32)
    res = rt.infer({"x": x, "n": np.asarray([3], np.int64)})
    assert np.allclose(res[0], _reference_while(x, 3), atol=1e-5) and int(res[1].reshape(-1)[0]) == 3


def _cond_program():
    """y = x * 3 if sum(x) > 0 else x - 10   (the two-block form that paddle.static.nn.cond writes)"""
    b = ProgramBuilder()
    x = b.feed("x", "float32", [-1, 2])
    s = b.op("reduce_sum", {"X": [x]}, ("Out",), [1], dim=[0], keep_dim=False, reduce_all=True)
    zero = b.op("fill_constant", {}, ("Out",), [1], shape=[1], value=0.0, dtype=5)
    c = b.op("greater_than", {"X": [s], "Y": [zero]}, ("Out",), [1], "bool", axis=-1)
    nc = b.op("logical_not", {"X": [c]}, ("Out",), [1], "bool")
    b.prog.add_var("y_true", "float32", [-1, 2])
    b.prog.add_var("y_false", "float32", [-1, 2])
    b.prog.add_var("sc0", var_type=17)
    b.prog.add_var("sc1", var_type=17)
    t_block = b.sub_block([("scale", {"X": [x]}, {"Out": ["y_true"]}, {"scale": 3.0, "bias": 0.0, "bias_after_scale": True})])
    f_block = b.sub_block([("scale", {"X": [x]}, {"Out": ["y_false"]}, {"scale": 1.0, "bias": -10.0, "bias_after_scale": True})])
    b.prog.add_op("conditional_block", {"Cond": [c], "Input": [x]}, {"Out": ["y_true"], "Scope": ["sc0"]},
                  sub_block=t_block, is_scalar_condition=True)
    b.prog.add_op("conditional_block", {"Cond": [nc], "Input": [x]}, {"Out": ["y_false"], "Scope": ["sc1"]},
                  sub_block=f_block, is_scalar_condition=True)
    mask = b.op("cast", {"X": [c]}, ("Out",), [1], "int32", in_dtype=0, out_dtype=2)
    y = b.op("select_input", {"X": ["y_false", "y_true"], "Mask": [mask]}, ("Out",), [-1, 2])
    b.fetch(y)
    return b.serialize()


def test_conditional_blocks_become_if_nodes():
    model, params = _cond_program()
    g = load_paddle(model, params)
    hist = g.op_histogram()
    assert hist.get("If") == 2 and hist.get("SelectInput") == 1
    interp = Interpreter(load_onnx(save_onnx(g)))
    name = g.output_names()[0]
    for x in (np.asarray([[1.0, 2.0]], np.float32), np.asarray([[-4.0, 1.0], [0.5, 0.5]], np.float32)):
        want = x * 3 if x.sum() > 0 else x - 10
        assert np.allclose(interp.run({"x": x})[name].numpy(), want)


def test_gpu_lowering_refuses_control_flow_with_a_clear_message():
    from fastdeploy_b200.ir.passes import optimize
    model, params = _while_program()
    g = load_paddle(model, params)
    assert [n.op for n in optimize(g, level=2).nodes] == [n.op for n in g.nodes]      # runs as imported
    from fastdeploy_b200.runtime.native_backend import build_plan
    with pytest.raises(NotImplementedError, match="control flow"):
        build_plan(g, {"x": [2, 3], "n": [1]}, "cpu")


def test_onnx_loop_with_trip_count_and_scan_outputs():
    """ONNX Loop semantics beyond what Paddle's while needs: a trip count, no condition input, scan outputs."""
    from fastdeploy_b200.ir.graph import Graph, ValueInfo
    body = Graph("body", 13)
    body.inputs += [ValueInfo("it", "int64", []), ValueInfo("c_in", "bool", []), ValueInfo("acc_in", "float32", [2])]
    body.add_node("Cast", ["it"], ["it_f"], to=1)
    body.add_node("Add", ["acc_in", "it_f"], ["acc_out"])
    body.add_node("Mul", ["acc_out", "outer_scale"], ["scan0"])               # reads the enclosing scope
    body.add_node("Identity", ["c_in"], ["c_out"])
    body.outputs += [ValueInfo("c_out", "bool", []), ValueInfo("acc_out", "float32", [2]), ValueInfo("scan0", "float32", [2])]
    g = Graph("main", 13)
    g.inputs.append(ValueInfo("x", "float32", [2]))
    g.initializers["trips"] = np.asarray(4, np.int64)
    g.initializers["outer_scale"] = np.asarray([10.0, 100.0], np.float32)
    g.add_node("Loop", ["trips", "", "x"], ["acc", "scans"], body=body)       # no outer_refs: the reader works them out
    g.outputs += [ValueInfo("acc", "float32", [2]), ValueInfo("scans", "float32", [4, 2])]
    g2 = load_onnx(save_onnx(g))
    out = Interpreter(g2).run({"x": np.asarray([1.0, 2.0], np.float32)})
    assert out["acc"].tolist() == [7.0, 8.0]                                   # + 0 + 1 + 2 + 3
    want = np.asarray([[1, 2], [2, 3], [4, 5], [7, 8]], np.float32) * np.asarray([10.0, 100.0], np.float32)
    assert np.allclose(out["scans"].numpy(), want)
    assert g2.nodes[0].attr("outer_refs") == ["outer_scale"]
    g2.prune()
    assert "outer_scale" in g2.initializers


def test_onnx_scan_running_sum_with_a_reversed_input():
    """The ONNX operator's own example (running sum of the rows of x), plus a second, reversed scan input."""
    from fastdeploy_b200.ir.graph import Graph, ValueInfo
    body = Graph("scan_body", 13)
    body.inputs += [ValueInfo("sum_in", "float32", [2]), ValueInfo("row", "float32", [2]), ValueInfo("rev_row", "float32", [2])]
    body.add_node("Add", ["sum_in", "row"], ["sum_out"])
    body.add_node("Identity", ["sum_out"], ["scan_out"])
    body.add_node("Mul", ["rev_row", "two"], ["scaled"])
    body.initializers["two"] = np.asarray(2.0, np.float32)
    body.outputs += [ValueInfo("sum_out", "float32", [2]), ValueInfo("scan_out", "float32", [2]), ValueInfo("scaled", "float32", [2])]
    g = Graph("main", 13)
    g.inputs += [ValueInfo("init", "float32", [2]), ValueInfo("x", "float32", [3, 2])]
    g.add_node("Scan", ["init", "x", "x"], ["final", "sums", "scaled_rev"], body=body, num_scan_inputs=2,
               scan_input_directions=[0, 1])
    g.outputs += [ValueInfo("final", "float32", [2]), ValueInfo("sums", "float32", [3, 2]), ValueInfo("scaled_rev", "float32", [3, 2])]
    x = np.asarray([[1, 2], [3, 4], [5, 6]], np.float32)
    out = Interpreter(load_onnx(save_onnx(g))).run({"init": np.zeros(2, np.float32), "x": x})
    assert out["final"].tolist() == [9.0, 12.0]
    assert out["sums"].tolist() == [[1, 2], [4, 6], [9, 12]]
    assert out["scaled_rev"].tolist() == (x[::-1] * 2).tolist()
