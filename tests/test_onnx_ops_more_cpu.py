"""The rest of the standard ONNX operator set in the interpreter, each against a reference written out with numpy or
torch (operator definitions: github.com/onnx/onnx, docs/Operators.md)."""
import numpy as np
import pytest
import torch

from fastdeploy_b200.ir.graph import Node
from fastdeploy_b200.ir.interp import _OPS


def run(op, inputs, **attrs):
    node = Node(op, [f"i{k}" for k in range(len(inputs))], ["o"], dict(attrs, _opset=13), op)
    args = [None if a is None else (torch.from_numpy(np.ascontiguousarray(a)) if isinstance(a, np.ndarray) else a)
            for a in inputs]
    while args and args[-1] is None:
        args.pop()
    out = _OPS[op](node, *args)
    return [o.numpy() for o in out] if isinstance(out, tuple) else out.numpy()


rng = np.random.default_rng(0)


def test_small_tensor_operators():
    x = np.array([[1.0, np.inf, -np.inf, np.nan]], np.float32)
    assert run("IsNaN", [x]).tolist() == [[False, False, False, True]]
    assert run("IsInf", [x]).tolist() == [[False, True, True, False]]
    assert run("IsInf", [x], detect_negative=0).tolist() == [[False, True, False, False]]
    a, b, c = (rng.standard_normal((2, 3)).astype(np.float32) for _ in range(3))
    assert np.allclose(run("Mean", [a, b, c]), (a + b + c) / 3)
    assert np.allclose(run("Celu", [a], alpha=2.0), np.maximum(0, a) + np.minimum(0, 2.0 * (np.exp(a / 2.0) - 1)), atol=1e-6)
    h = run("Hardmax", [np.array([[1.0, 3.0, 3.0], [2.0, 0.0, 1.0]], np.float32)], axis=1)
    assert h.tolist() == [[0, 1, 0], [1, 0, 0]]
    assert run("EyeLike", [np.zeros((3, 4), np.float32)], k=1).tolist() == np.eye(3, 4, 1).tolist()
    assert run("EyeLike", [np.zeros((3, 3), np.int64)], k=-1, dtype=1).dtype == np.float32
    m = np.arange(16, dtype=np.float32).reshape(4, 4)
    assert np.array_equal(run("Trilu", [m, np.array(1, np.int64)], upper=1), np.triu(m, 1))
    assert np.array_equal(run("Trilu", [m], upper=0), np.tril(m))
    assert run("BitShift", [np.array([1, 4], np.uint8), np.array([3, 1], np.uint8)], direction="LEFT").tolist() == [8, 8]
    assert run("BitShift", [np.array([16, 4], np.uint8), np.array([3, 1], np.uint8)], direction="RIGHT").tolist() == [2, 2]
    sq = rng.standard_normal((2, 3, 3)).astype(np.float32)
    assert np.allclose(run("Det", [sq]), np.linalg.det(sq), atol=1e-5)
    v = np.arange(12, dtype=np.float32).reshape(3, 4)
    assert np.array_equal(run("Compress", [v, np.array([0, 1, 1], bool)], axis=0), v[1:])
    assert np.array_equal(run("Compress", [v, np.array([1, 0, 0, 0, 1], bool)]), np.array([0.0, 4.0], np.float32))
    seq = np.arange(24, dtype=np.float32).reshape(4, 3, 2)                       # [T, B, C]
    want = seq.copy()
    for item, n in enumerate([4, 2, 1]):
        want[:n, item] = seq[:n, item][::-1]
    assert np.array_equal(run("ReverseSequence", [seq, np.array([4, 2, 1], np.int64)], batch_axis=1, time_axis=0), want)
    base = np.zeros((3, 3), np.float32)
    idx = np.array([[1, 0, 2], [0, 2, 1]], np.int64)
    upd = np.array([[1.0, 1.1, 1.2], [2.0, 2.1, 2.2]], np.float32)
    got = run("ScatterElements", [base, idx, upd], axis=0)
    assert np.allclose(got, [[2.0, 1.1, 0.0], [1.0, 0.0, 2.2], [0.0, 2.1, 1.2]])
    add = run("ScatterElements", [np.ones((1, 5), np.float32), np.array([[1, 1]], np.int64), np.array([[2.0, 3.0]], np.float32)],
              axis=1, reduction="add")
    assert add.tolist() == [[1.0, 6.0, 1.0, 1.0, 1.0]]
    x4 = rng.standard_normal((1, 2, 4, 6)).astype(np.float32)
    std = run("SpaceToDepth", [x4], blocksize=2)
    assert std.shape == (1, 8, 2, 3) and np.array_equal(run("DepthToSpace", [std], blocksize=2, mode="DCR"), x4)
    assert run("Constant", [], value=np.array([1, 2], np.int64)).tolist() == [1, 2] and float(run("Constant", [], value_float=2.5)) == 2.5
    assert run("Einsum", [a, b.T.copy()], equation="ij,jk->ik").shape == (2, 2)
    assert np.allclose(run("Einsum", [a, b.T.copy()], equation="ij,jk->ik"), a @ b.T, atol=1e-6)


def test_pooling_and_normalisation_operators():
    x = rng.standard_normal((2, 6, 5, 5)).astype(np.float32)
    lrn = run("LRN", [x], size=3, alpha=1e-3, beta=0.75, bias=2.0)
    sq = np.pad(x ** 2, [(0, 0), (1, 1), (0, 0), (0, 0)])
    acc = sq[:, 0:6] + sq[:, 1:7] + sq[:, 2:8]
    assert np.allclose(lrn, x / (2.0 + 1e-3 / 3 * acc) ** 0.75, atol=1e-5)
    l2 = run("LpNormalization", [x], p=2, axis=1)
    assert np.allclose(l2, x / np.sqrt((x ** 2).sum(1, keepdims=True)), atol=1e-6)
    l1 = run("LpNormalization", [x], p=1, axis=-1)
    assert np.allclose(np.abs(l1).sum(-1), 1.0, atol=1e-5)
    mvn = run("MeanVarianceNormalization", [x])
    assert np.allclose(mvn.mean((0, 2, 3)), 0, atol=1e-5) and np.allclose(mvn.std((0, 2, 3)), 1, atol=1e-3)
    glp = run("GlobalLpPool", [x], p=2)
    assert glp.shape == (2, 6, 1, 1) and np.allclose(glp.reshape(2, 6), np.sqrt((x ** 2).sum((2, 3))), atol=1e-5)
    lp = run("LpPool", [x], p=2, kernel_shape=[2, 2], strides=[2, 2])
    want = np.sqrt(sum(x[:, :, i:4:2, j:4:2] ** 2 for i in range(2) for j in range(2)))
    assert np.allclose(lp, want, atol=1e-5)
    pos = np.abs(x) + 0.1
    assert np.allclose(run("ReduceLogSum", [pos], axes=[1, 3], keepdims=0), np.log(pos.sum((1, 3))), atol=1e-5)
    pooled, idx = torch.nn.functional.max_pool2d(torch.from_numpy(x[:, :, :4, :4]), 2, return_indices=True)
    flat = idx + (torch.arange(12).reshape(2, 6, 1, 1) * 16)                     # ONNX indices run over the whole tensor
    un = run("MaxUnpool", [pooled.numpy(), flat.numpy()], kernel_shape=[2, 2], strides=[2, 2])
    ref = torch.nn.functional.max_unpool2d(pooled, idx, 2).numpy()
    assert un.shape == (2, 6, 4, 4) and np.array_equal(un, ref)
    feat = np.arange(2 * 1 * 6 * 6, dtype=np.float32).reshape(2, 1, 6, 6)
    rois = np.array([[0, 0, 0, 3, 3], [1, 2, 2, 5, 5]], np.float32)
    rp = run("MaxRoiPool", [feat, rois], pooled_shape=[2, 2], spatial_scale=1.0)
    assert rp.shape == (2, 1, 2, 2) and rp[0, 0].tolist() == [[7.0, 9.0], [19.0, 21.0]] and rp[1, 0, 1, 1] == feat[1, 0, 5, 5]


def test_non_max_suppression_and_integer_linear_algebra():
    boxes = np.array([[[0, 0, 1, 1], [0, 0.1, 1, 1.1], [0, -0.1, 1, 0.9], [0, 10, 1, 11], [0, 10.1, 1, 11.1], [0, 100, 1, 101]]],
                     np.float32)
    scores = np.array([[[0.9, 0.75, 0.6, 0.95, 0.5, 0.3]]], np.float32)
    sel = run("NonMaxSuppression", [boxes, scores, np.array([3], np.int64), np.array([0.5], np.float32),
                                    np.array([0.0], np.float32)])
    assert sel.tolist() == [[0, 0, 3], [0, 0, 0], [0, 0, 5]]                     # the ONNX operator's own example
    sel2 = run("NonMaxSuppression", [boxes, scores, np.array([2], np.int64), np.array([0.5], np.float32),
                                     np.array([0.4], np.float32)])
    assert sel2.tolist() == [[0, 0, 3], [0, 0, 0]]
    centre = np.array([[[0.5, 0.5, 1, 1], [0.5, 0.6, 1, 1], [0.5, 10.5, 1, 1]]], np.float32)
    sel3 = run("NonMaxSuppression", [centre, np.array([[[0.9, 0.8, 0.7]]], np.float32), np.array([3], np.int64),
                                     np.array([0.5], np.float32)], center_point_box=1)
    assert sel3.tolist() == [[0, 0, 0], [0, 0, 2]]
    assert run("NonMaxSuppression", [boxes, scores]).shape == (0, 3)             # no output budget, nothing selected
    # integer matmul / conv with zero points
    a = rng.integers(0, 255, (3, 4)).astype(np.uint8)
    b = rng.integers(-128, 127, (4, 5)).astype(np.int8)
    mm = run("MatMulInteger", [a, b, np.array(12, np.uint8), np.array(-3, np.int8)])
    assert mm.dtype == np.int32 and np.array_equal(mm, (a.astype(np.int32) - 12) @ (b.astype(np.int32) + 3))
    x = rng.integers(0, 255, (1, 2, 5, 5)).astype(np.uint8)
    w = rng.integers(0, 255, (3, 2, 3, 3)).astype(np.uint8)
    ci = run("ConvInteger", [x, w, np.array(7, np.uint8), np.array(100, np.uint8)], pads=[1, 1, 1, 1])
    ref = torch.nn.functional.conv2d(torch.from_numpy(x.astype(np.float64) - 7), torch.from_numpy(w.astype(np.float64) - 100), padding=1)
    assert ci.dtype == np.int32 and np.array_equal(ci, ref.numpy().astype(np.int32))
    # dynamic quantisation: the ONNX operator's own example
    y, scale, zp = run("DynamicQuantizeLinear", [np.array([0, 2, -3, -2.5, 1.34, 0.5], np.float32)])
    assert y.tolist() == [153, 255, 0, 26, 221, 179] and abs(float(scale) - 0.0196078438) < 1e-7 and int(zp) == 153
    # QLinearMatMul: the ONNX operator's own example
    qa = np.array([[208, 236, 0, 238], [3, 214, 255, 29]], np.uint8)
    qb = np.array([[152, 51, 244], [60, 26, 255], [0, 127, 246], [127, 254, 247]], np.uint8)
    qy = run("QLinearMatMul", [qa, np.array(0.0066, np.float32), np.array(113, np.uint8), qb, np.array(0.00705, np.float32),
                               np.array(114, np.uint8), np.array(0.0107, np.float32), np.array(118, np.uint8)])
    assert qy.tolist() == [[168, 115, 255], [1, 66, 151]]
    # QLinearConv against the dequantise -> conv -> quantise chain, per-channel weight scales and an int32 bias
    xs, xz = np.array(0.02, np.float32), np.array(128, np.uint8)
    ws, wz = np.array([0.01, 0.02, 0.005], np.float32), np.array([0, 0, 0], np.int8)
    wq = rng.integers(-100, 100, (3, 2, 3, 3)).astype(np.int8)
    bias = rng.integers(-500, 500, 3).astype(np.int32)
    ys, yz = np.array(0.05, np.float32), np.array(100, np.uint8)
    got = run("QLinearConv", [x, xs, xz, wq, ws, wz, ys, yz, bias], pads=[1, 1, 1, 1])
    xf = (x.astype(np.float64) - 128) * 0.02
    wf = wq.astype(np.float64) * ws.astype(np.float64).reshape(3, 1, 1, 1)
    bf = bias.astype(np.float64) * 0.02 * ws.astype(np.float64)
    ref = torch.nn.functional.conv2d(torch.from_numpy(xf), torch.from_numpy(wf), torch.from_numpy(bf), padding=1).numpy()
    want = np.clip(np.rint(ref / float(ys)) + 100, 0, 255).astype(np.uint8)
    assert got.dtype == np.uint8 and np.abs(got.astype(int) - want.astype(int)).max() <= 1


def test_recurrent_layers_match_torch():
    t_len, bsz, inp, hid = 5, 3, 4, 6
    x = rng.standard_normal((t_len, bsz, inp)).astype(np.float32)
    for bidir in (False, True):
        d = 2 if bidir else 1
        gru = torch.nn.GRU(inp, hid, bidirectional=bidir)
        # torch stacks gates r, z, n; ONNX wants z, r, h
        def reorder(p):
            r, z, n = p.detach().split(hid, 0)
            return torch.cat([z, r, n], 0)
        sfx = ["", "_reverse"][:d]
        w = torch.stack([reorder(getattr(gru, "weight_ih_l0" + s)) for s in sfx]).numpy()
        r = torch.stack([reorder(getattr(gru, "weight_hh_l0" + s)) for s in sfx]).numpy()
        b = torch.stack([torch.cat([reorder(getattr(gru, "bias_ih_l0" + s)), reorder(getattr(gru, "bias_hh_l0" + s))]) for s in sfx]).numpy()
        y, yh = run("GRU", [x, w, r, b], hidden_size=hid, linear_before_reset=1,
                    direction="bidirectional" if bidir else "forward")
        ref_y, ref_h = gru(torch.from_numpy(x))
        assert y.shape == (t_len, d, bsz, hid) and np.allclose(yh, ref_h.detach().numpy(), atol=1e-5)
        assert np.allclose(y.transpose(0, 2, 1, 3).reshape(t_len, bsz, d * hid), ref_y.detach().numpy(), atol=1e-5)
        rnn = torch.nn.RNN(inp, hid, bidirectional=bidir)
        w = torch.stack([getattr(rnn, "weight_ih_l0" + s).detach() for s in sfx]).numpy()
        r = torch.stack([getattr(rnn, "weight_hh_l0" + s).detach() for s in sfx]).numpy()
        b = torch.stack([torch.cat([getattr(rnn, "bias_ih_l0" + s), getattr(rnn, "bias_hh_l0" + s)]).detach() for s in sfx]).numpy()
        y, yh = run("RNN", [x, w, r, b], hidden_size=hid, direction="bidirectional" if bidir else "forward")
        ref_y, ref_h = rnn(torch.from_numpy(x))
        assert np.allclose(yh, ref_h.detach().numpy(), atol=1e-5)
        assert np.allclose(y.transpose(0, 2, 1, 3).reshape(t_len, bsz, d * hid), ref_y.detach().numpy(), atol=1e-5)


def test_random_operators_have_the_asked_shape_type_and_range():
    u = run("RandomUniform", [], shape=[4, 5], low=2.0, high=3.0, seed=7.0, dtype=1)
    assert u.shape == (4, 5) and u.dtype == np.float32 and (u >= 2).all() and (u < 3).all()
    assert np.array_equal(u, run("RandomUniform", [], shape=[4, 5], low=2.0, high=3.0, seed=7.0, dtype=1))
    like = np.zeros((3, 2), np.float64)
    assert run("RandomUniformLike", [like], seed=1.0).dtype == np.float64 and run("RandomNormalLike", [like], dtype=1).dtype == np.float32
    n = run("RandomNormalLike", [np.zeros((2000,), np.float32)], mean=5.0, scale=2.0, seed=3.0)
    assert abs(n.mean() - 5.0) < 0.2 and abs(n.std() - 2.0) < 0.2
    logits = np.log(np.array([[0.0001, 0.0001, 0.9998]], np.float32))
    m = run("Multinomial", [logits], sample_size=20, seed=2.0)
    assert m.shape == (1, 20) and m.dtype == np.int32 and (m == 2).mean() > 0.9


def test_newer_opset_operators():
    a, b = np.array([12, 10, 255], np.uint8), np.array([10, 3, 15], np.uint8)
    assert run("BitwiseAnd", [a, b]).tolist() == (a & b).tolist() and run("BitwiseOr", [a, b]).tolist() == (a | b).tolist()
    assert run("BitwiseXor", [a, b]).tolist() == (a ^ b).tolist() and run("BitwiseNot", [a]).tolist() == (~a).tolist()
    assert run("CastLike", [np.array([1.7, -2.2], np.float32), np.zeros(1, np.int64)]).tolist() == [1, -2]
    bern = run("Bernoulli", [np.full((4000,), 0.25, np.float32)], seed=1.0)
    assert bern.dtype == np.float32 and abs(bern.mean() - 0.25) < 0.03
    n = np.array(8, np.int64)
    assert np.allclose(run("HannWindow", [n]), np.hanning(9)[:8], atol=1e-6)                  # periodic by default
    assert np.allclose(run("HannWindow", [n], periodic=0), np.hanning(8), atol=1e-6)
    assert np.allclose(run("HammingWindow", [n], periodic=0), 25 / 46 - 21 / 46 * np.cos(2 * np.pi * np.arange(8) / 7), atol=1e-6)
    assert np.allclose(run("BlackmanWindow", [n], periodic=0), np.blackman(8), atol=1e-6)
    x = np.arange(20, dtype=np.float32).reshape(4, 5)
    assert np.array_equal(run("CenterCropPad", [x, np.array([2, 7], np.int64)]), np.pad(x[1:3], [(0, 0), (1, 1)]))
    img = rng.standard_normal((1, 2, 5, 5)).astype(np.float32)
    cols = torch.nn.functional.unfold(torch.from_numpy(img), (2, 2)).numpy()
    back = run("Col2Im", [cols, np.array([5, 5], np.int64), np.array([2, 2], np.int64)])
    ones = torch.nn.functional.fold(torch.nn.functional.unfold(torch.ones(1, 2, 5, 5), (2, 2)), (5, 5), (2, 2)).numpy()
    assert np.allclose(back / ones, img, atol=1e-6)
    sig = rng.standard_normal((2, 16, 1)).astype(np.float32)
    spec = run("DFT", [sig], axis=1)
    ref = np.fft.fft(sig[..., 0], axis=1)
    assert spec.shape == (2, 16, 2) and np.allclose(spec[..., 0], ref.real, atol=1e-4) and np.allclose(spec[..., 1], ref.imag, atol=1e-4)
    half = run("DFT", [sig], axis=1, onesided=1)
    assert half.shape == (2, 9, 2) and np.allclose(half[..., 0], ref.real[:, :9], atol=1e-4)
    inv = run("DFT", [spec], axis=1, inverse=1)
    assert np.allclose(inv[..., 0], sig[..., 0], atol=1e-5)
