"""Stride-generic executor kernels against plain PyTorch, and the plans of the bundled model families:
none of them may contain a step that runs a framework operator."""
import tempfile

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev(t):
    return t.cuda()


def test_strided_copy_transposes_casts_and_broadcasts():
    from fastdeploy_b200.ops import generic as G
    g = torch.Generator().manual_seed(0)
    x = _dev(torch.randn(3, 5, 7, 9, generator=g))
    # NCHW fp32 -> NHWC fp16 through views
    dst = torch.zeros(3, 7, 9, 8, dtype=torch.float16, device="cuda")
    G.strided_copy(x, dst[..., :5].permute(0, 3, 1, 2)).launch()
    torch.cuda.synchronize()
    assert torch.equal(dst[..., :5], x.permute(0, 2, 3, 1).half())
    assert float(dst[..., 5:].abs().max()) == 0.0
    # broadcast + int64 -> int32 + slice of a wider destination
    ids = _dev(torch.arange(7, dtype=torch.int64)).view(1, 7)
    out = torch.full((4, 10), -1, dtype=torch.int32, device="cuda")
    G.strided_copy(ids, out[:, 2:9]).launch()
    torch.cuda.synchronize()
    assert torch.equal(out[:, 2:9].long(), ids.expand(4, 7)) and int(out[0, 0]) == -1 and int(out[3, 9]) == -1
    # bf16 bits survive a same-type move; seven non-mergeable dimensions are refused
    b = _dev(torch.randn(4, 6, generator=g)).bfloat16()
    o = torch.zeros(6, 4, dtype=torch.bfloat16, device="cuda")
    G.strided_copy(b.t(), o).launch()
    torch.cuda.synchronize()
    assert torch.equal(o, b.t())
    big = torch.zeros([2] * 14, device="cuda")[:, 0, :, 0, :, 0, :, 0, :, 0, :, 0, :, 0]
    with pytest.raises(ValueError):
        G.strided_copy(big, torch.zeros([2] * 7, device="cuda").permute(6, 5, 4, 3, 2, 1, 0))


@pytest.mark.parametrize("op,fn", [("add", torch.add), ("sub", torch.sub), ("mul", torch.mul), ("div", torch.div),
                                   ("max", torch.maximum), ("min", torch.minimum), ("pow", None)])
def test_elementwise_binary_broadcast_fp32(op, fn):
    from fastdeploy_b200.ops import generic as G
    g = torch.Generator().manual_seed(1)
    a = _dev(torch.rand(4, 1, 6, generator=g) + 0.5)
    b = _dev(torch.rand(5, 1, generator=g) + 0.5)
    out = torch.zeros(4, 5, 6, device="cuda")
    G.elementwise(op, a, b, out).launch()
    torch.cuda.synchronize()
    ref = torch.pow(a, b) if fn is None else fn(a, b)
    torch.testing.assert_close(out, ref.expand(4, 5, 6), rtol=1e-6, atol=1e-6)


def test_elementwise_integer_logic_and_unary():
    from fastdeploy_b200.ops import generic as G
    ids = _dev(torch.tensor([[5, 0, 7, 0], [0, 0, 123456789012, 1]], dtype=torch.int64))
    zero = _dev(torch.zeros((), dtype=torch.int64))
    eq = torch.zeros(2, 4, dtype=torch.bool, device="cuda")
    G.elementwise("eq", ids, zero, eq).launch()
    ne = torch.zeros(2, 4, dtype=torch.bool, device="cuda")
    G.elementwise("not", eq, None, ne).launch()
    f = torch.zeros(2, 4, device="cuda")
    G.elementwise("identity", ne, None, f).launch()
    big = torch.zeros(2, 4, dtype=torch.int64, device="cuda")
    G.elementwise("add", ids, _dev(torch.tensor(1, dtype=torch.int64)), big).launch()
    torch.cuda.synchronize()
    assert torch.equal(eq, ids == 0) and torch.equal(ne, ids != 0) and torch.equal(f, (ids != 0).float())
    assert torch.equal(big, ids + 1)
    x = _dev(torch.linspace(-4, 4, 97))
    for op, ref in (("sigmoid", torch.sigmoid(x)), ("tanh", torch.tanh(x)), ("gelu", torch.nn.functional.gelu(x)),
                    ("silu", torch.nn.functional.silu(x)), ("hard_swish", torch.nn.functional.hardswish(x)),
                    ("relu", torch.relu(x)), ("abs", x.abs()), ("erf", torch.erf(x)), ("floor", x.floor()),
                    ("sign", torch.sign(x)), ("exp", x.exp())):
        y = torch.zeros_like(x)
        G.elementwise(op, x, None, y).launch()
        torch.cuda.synchronize()
        torch.testing.assert_close(y, ref, rtol=2e-6, atol=2e-6)
    y = torch.zeros_like(x)
    G.elementwise("clip", x, None, y, -1.5, 2.0).launch()
    G.elementwise("affine", y, None, y, 2.0, 1.0).launch()
    torch.cuda.synchronize()
    torch.testing.assert_close(y, x.clamp(-1.5, 2.0) * 2 + 1)


def test_where_softmax_reduce_gather():
    from fastdeploy_b200.ops import generic as G
    g = torch.Generator().manual_seed(2)
    c = _dev(torch.rand(3, 1, 8, generator=g) > 0.5)
    a = _dev(torch.randn(3, 4, 8, generator=g))
    b = _dev(torch.full((1,), float("-inf")))
    out = torch.zeros(3, 4, 8, device="cuda")
    G.where(c, a, b, out).launch()
    torch.cuda.synchronize()
    assert torch.equal(out, torch.where(c, a, b))
    # soft-max over rows of a padded fp16 matrix (row pitch > row length), fp32 result
    buf = _dev(torch.randn(6, 5, 6632, generator=g)).half()
    x = buf[..., :6625]
    y = torch.zeros(6, 5, 6625, device="cuda")
    G.softmax_last(x, y).launch()
    ly = torch.zeros(6, 5, 6625, device="cuda")
    G.softmax_last(x, ly, log=True).launch()
    torch.cuda.synchronize()
    torch.testing.assert_close(y, torch.softmax(x.float(), -1), rtol=1e-4, atol=1e-7)
    torch.testing.assert_close(ly, torch.log_softmax(x.float(), -1), rtol=1e-4, atol=1e-4)
    # masked entries (-inf) at the front, in the middle and at the end of long and short rows, every dtype pair
    for cols in (6625, 40):
        for din, dout in ((torch.float16, torch.float16), (torch.bfloat16, torch.float32), (torch.float32, torch.bfloat16)):
            xm = _dev(torch.randn(4, cols, generator=g)).to(din)
            xm[0, :3] = float("-inf")
            xm[1, cols // 2:cols // 2 + 5] = float("-inf")
            xm[2, -2:] = float("-inf")
            ym = torch.zeros(4, cols, device="cuda", dtype=dout)
            G.softmax_last(xm, ym).launch()
            torch.cuda.synchronize()
            want = torch.softmax(xm.float(), -1)
            tol = 1e-5 if dout == torch.float32 else 4e-3
            assert (ym.float() - want).abs().max().item() < tol and not torch.isnan(ym.float()).any()
    xs = _dev(torch.randn(7, 33, generator=g))
    for mode, ref in (("sum", xs.sum(-1)), ("mean", xs.mean(-1)), ("max", xs.amax(-1)), ("min", xs.amin(-1))):
        r = torch.zeros(7, device="cuda")
        G.reduce_last(mode, xs, r).launch()
        torch.cuda.synchronize()
        torch.testing.assert_close(r, ref, rtol=1e-5, atol=1e-5)
    xs[2, 5] = xs[2, 20] = 99.0        # a tie: the first index wins
    am = torch.zeros(7, dtype=torch.int64, device="cuda")
    G.reduce_last("argmax", xs, am).launch()
    torch.cuda.synchronize()
    assert torch.equal(am, xs.argmax(-1)) and int(am[2]) == 5
    table = _dev(torch.randn(50, 16, generator=g))
    idx = _dev(torch.tensor([[3, 49], [0, -1]], dtype=torch.int64))
    o = torch.zeros(2, 2, 16, device="cuda")
    G.gather_rows(table, idx, o).launch()
    torch.cuda.synchronize()
    assert torch.equal(o, table[idx])


# ---------------------------------------------------------------------------------------------- plans
def _feed(plan, feeds):
    for k, v in feeds.items():
        dst = plan.inputs[k]
        t = torch.from_numpy(v).cuda()
        if dst.nhwc:
            dst.t.copy_(t.permute(0, 2, 3, 1))
        else:
            dst.t.copy_(t)


def _framework_steps(plan):
    return [s.name for s in plan.steps if s.native is None]


def _check_plan(g, feeds, tol=4e-2, skip_outputs=(), mean_tol=None):
    from fastdeploy_b200.ir.interp import Interpreter
    from fastdeploy_b200.runtime.native_backend import build_plan
    ref = Interpreter(g).run(feeds)
    plan = build_plan(g, {k: list(v.shape) for k, v in feeds.items()}, "cuda:0")
    assert _framework_steps(plan) == [], _framework_steps(plan)
    _feed(plan, feeds)
    plan.run()
    torch.cuda.synchronize()
    plan.status.check()
    for name, r in ref.items():
        if name in skip_outputs:
            continue
        out = plan.outputs[name].logical().float().cpu()
        r = torch.as_tensor(r).float()
        assert list(out.shape) == list(r.shape), (name, out.shape, r.shape)
        if mean_tol is not None:
            # a sigmoid over wide-range logits: single pixels near the decision boundary move a lot for a small
            # relative error of the logit, so the mean error and the binarised map are compared instead
            assert (out - r).abs().mean().item() < mean_tol, (name, (out - r).abs().mean().item())
            assert ((out > 0.5) == (r > 0.5)).float().mean().item() > 0.97
            continue
        err = (out - r).abs().max().item()
        assert err <= tol * r.abs().max().item() + 1e-3, (name, err)
    # a captured replay is bit-identical: nothing in the plan depends on host state
    first = {n: plan.outputs[n].logical().float().cpu().clone() for n in ref}
    plan.capture()
    plan.run()
    torch.cuda.synchronize()
    for n in ref:
        assert torch.equal(first[n], plan.outputs[n].logical().float().cpu()), n
    return plan


@pytest.mark.parametrize("task", ["seq_cls", "uie"])
def test_ernie_plans_have_no_framework_steps(task):
    from fastdeploy_b200.importer.paddle_import import load_paddle
    from fastdeploy_b200.models.ernie import build_ernie
    m, p = build_ernie("tiny", task).serialize()
    g = load_paddle(m, p)
    rng = np.random.RandomState(0)
    ids = rng.randint(1, 100, size=(4, 32)).astype(np.int64)
    ids[1, 20:] = 0
    ids[3, 7:] = 0
    feeds = {"input_ids": ids, "token_type_ids": np.zeros((4, 32), np.int64)}
    if task == "uie":
        feeds["pos_ids"] = np.tile(np.arange(32, dtype=np.int64), (4, 1))
        feeds["att_mask"] = (ids != 0).astype(np.int64)
    feeds = {vi.name: feeds[vi.name] for vi in g.inputs}
    _check_plan(g, feeds)


@pytest.mark.parametrize("kind,shape", [("det", [1, 3, 160, 160]), ("cls", [2, 3, 48, 192]), ("rec", [2, 3, 48, 160])])
def test_ocr_plans_have_no_framework_steps(kind, shape):
    from fastdeploy_b200.importer.paddle_import import load_paddle
    from fastdeploy_b200.models import ppocr
    paths = ppocr.write_ppocr(tempfile.mkdtemp())
    g = load_paddle(open(paths[kind + "_model"], "rb").read(), open(paths[kind + "_params"], "rb").read())
    x = np.random.RandomState(3).rand(*shape).astype(np.float32)
    _check_plan(g, {g.inputs[0].name: x}, mean_tol=0.03 if kind == "det" else None)


def test_resnet_and_ppyoloe_plans_have_no_framework_steps():
    from fastdeploy_b200.importer.onnx_format import load_onnx
    from fastdeploy_b200.importer.paddle_import import load_paddle
    from fastdeploy_b200.models.ppyoloe import build_ppyoloe
    from fastdeploy_b200.models.resnet import resnet18_like_onnx
    from fastdeploy_b200.runtime.native_backend import build_plan
    g = load_onnx(resnet18_like_onnx())
    _check_plan(g, {"input": np.random.RandomState(0).rand(4, 3, 64, 64).astype(np.float32)})
    m, p = build_ppyoloe("tiny", image=128, num_classes=8, with_nms=True, score_threshold=0.005).serialize()
    plan = build_plan(load_paddle(m, p), {"image": [2, 3, 128, 128], "scale_factor": [2, 2]}, "cuda:0")
    assert _framework_steps(plan) == [], _framework_steps(plan)


def test_deconvolution_with_folded_batchnorm_matches_interpreter():
    """ConvTranspose 2x2 / stride 2 -> BatchNormalization -> Relu -> ConvTranspose -> Sigmoid (a DB text-detection
    head): four strided-output GEMMs per layer, nothing left for the framework."""
    from fastdeploy_b200.ir.graph import Graph
    from fastdeploy_b200.ir import passes
    rng = np.random.RandomState(5)
    g = Graph()
    g.add_input("x", "float32", [2, 24, 20, 28])
    w1 = g.const((rng.randn(24, 16, 2, 2) * 0.2).astype(np.float32), prefix="w1")
    b1 = g.const(rng.randn(16).astype(np.float32) * 0.1, prefix="b1")
    bn = [g.const(v.astype(np.float32), prefix="bn") for v in (rng.rand(16) + 0.5, rng.randn(16) * 0.1, rng.randn(16) * 0.1,
                                                               rng.rand(16) + 0.5)]
    w2 = g.const((rng.randn(16, 1, 2, 2) * 0.3).astype(np.float32), prefix="w2")
    g.add_node("ConvTranspose", ["x", w1, b1], ["d1"], strides=[2, 2], kernel_shape=[2, 2])
    g.add_node("BatchNormalization", ["d1"] + bn, ["n1"], epsilon=1e-5)
    g.add_node("Relu", ["n1"], ["r1"])
    g.add_node("ConvTranspose", ["r1", w2], ["d2"], strides=[2, 2], kernel_shape=[2, 2])
    g.add_node("Sigmoid", ["d2"], ["y"])
    g.add_output("y", "float32", [2, 1, 80, 112])
    opt = passes.optimize(g, {"x": [2, 24, 20, 28]})
    assert [n.op for n in opt.nodes] == ["ConvTranspose", "ConvTranspose"]
    plan = _check_plan(g, {"x": rng.rand(2, 24, 20, 28).astype(np.float32)}, tol=2e-2)
    assert sum(1 for s in plan.steps if s.name.startswith("deconv")) == 8
