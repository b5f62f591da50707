"""Second batch of Paddle operator mappers: every operator is imported from a serialized program and run through
the fp32 interpreter against a NumPy / PyTorch statement of the Paddle semantics."""
import numpy as np
import pytest
import torch


def _run(b, feeds, fetch):
    from fastdeploy_b200.importer.paddle_import import load_paddle
    from fastdeploy_b200.ir.interp import Interpreter
    for f in fetch:
        b.fetch(f)
    g = load_paddle(*b.serialize())
    out = Interpreter(g).run(feeds)
    return [out[n] for n in g.output_names()]


def _builder():
    from fastdeploy_b200.importer.paddle_format import ProgramBuilder
    return ProgramBuilder()


X = np.random.RandomState(0).uniform(-0.9, 0.9, (3, 5)).astype(np.float32)
XT = torch.from_numpy(X)
UNARY = [
    ("acos", {}, torch.acos(XT)), ("asin", {}, torch.asin(XT)), ("atan", {}, torch.atan(XT)), ("cosh", {}, torch.cosh(XT)),
    ("sinh", {}, torch.sinh(XT)), ("tan", {}, torch.tan(XT)), ("brelu", dict(t_min=-0.2, t_max=0.5), XT.clamp(-0.2, 0.5)),
    ("hard_shrink", dict(threshold=0.3), torch.nn.functional.hardshrink(XT, 0.3)),
    ("softshrink", {"lambda": 0.3}, torch.nn.functional.softshrink(XT, 0.3)),
    ("tanh_shrink", {}, XT - torch.tanh(XT)), ("thresholded_relu", dict(threshold=0.2), torch.where(XT > 0.2, XT, torch.zeros(()))),
    ("logsigmoid", {}, torch.nn.functional.logsigmoid(XT)), ("log10", {}, torch.log10(XT.abs() + 1)),
    ("log2", {}, torch.log2(XT.abs() + 1)), ("log1p", {}, torch.log1p(XT.abs() + 1)), ("selu", {}, torch.selu(XT)),
    ("flip", dict(axis=[1]), torch.flip(XT, [1])), ("logsumexp", dict(axis=[1], keepdim=False), torch.logsumexp(XT, 1)),
]


@pytest.mark.parametrize("name,attrs,ref", UNARY, ids=[u[0] for u in UNARY])
def test_unary_and_reduction_mappers(name, attrs, ref):
    b = _builder()
    b.feed("x", "float32", [3, 5])
    src = "x"
    if name in ("log10", "log2", "log1p"):
        src = b.op("abs", {"X": ["x"]}, ("Out",), [3, 5])
        src = b.op("scale", {"X": [src]}, ("Out",), [3, 5], scale=1.0, bias=1.0, bias_after_scale=True)
    y = b.op(name, {"X": [src]}, ("Out",), [3, 5], **attrs)
    got, = _run(b, {"x": X}, [y])
    torch.testing.assert_close(got.float(), ref, rtol=1e-5, atol=1e-6)


def test_quantize_dequantize_linear_follow_the_paddle_range_convention():
    b = _builder()
    b.feed("x", "float32", [4, 6])
    sx = b.param("sx", np.array([2.0], np.float32))                      # clipping range, not step
    zp = b.param("zp", np.zeros(1, np.float32))
    q = b.prog.add_var("q", "float32", [4, 6])
    b.prog.add_op("quantize_linear", {"X": ["x"], "Scale": [sx], "ZeroPoint": [zp]}, {"Y": [q]}, quant_axis=-1, bit_length=8)
    d = b.prog.add_var("d", "float32", [4, 6])
    b.prog.add_op("dequantize_linear", {"X": [q], "Scale": [sx], "ZeroPoint": [zp]}, {"Y": [d]}, quant_axis=-1, bit_length=8)
    # a per-channel int8 weight: range per output column (quant_axis 1)
    w8 = np.random.RandomState(1).randint(-127, 128, (6, 3)).astype(np.int8)
    sw = np.array([0.5, 1.0, 2.0], np.float32)
    wq = b.param("w8", w8)
    sws = b.param("sw", sw)
    zw = b.param("zw", np.zeros(3, np.float32))
    wf = b.prog.add_var("wf", "float32", [6, 3])
    b.prog.add_op("dequantize_linear", {"X": [wq], "Scale": [sws], "ZeroPoint": [zw]}, {"Y": [wf]}, quant_axis=1, bit_length=8)
    y = b.op("matmul_v2", {"X": [d], "Y": [wf]}, ("Out",), [4, 3], trans_x=False, trans_y=False)
    x = np.random.RandomState(2).uniform(-3, 3, (4, 6)).astype(np.float32)
    got, = _run(b, {"x": x}, [y])
    xq = np.clip(np.round(x / (2.0 / 127)), -128, 127) * (2.0 / 127)
    ref = xq @ (w8.astype(np.float32) * (sw / 127)[None, :])
    np.testing.assert_allclose(got.numpy(), ref, rtol=1e-5, atol=1e-5)


def test_yolo_box_matches_a_direct_statement_of_the_kernel():
    rng = np.random.RandomState(3)
    n, a, c, h, w = 2, 3, 4, 5, 6
    anchors = [10, 13, 16, 30, 33, 23]
    x = rng.randn(n, a * (5 + c), h, w).astype(np.float32)
    img = np.array([[320, 480], [416, 416]], np.int32)
    b = _builder()
    b.feed("x", "float32", [n, a * (5 + c), h, w])
    b.feed("im", "int32", [n, 2])
    boxes = b.prog.add_var("boxes", "float32", [n, a * h * w, 4])
    scores = b.prog.add_var("scores", "float32", [n, a * h * w, c])
    b.prog.add_op("yolo_box", {"X": ["x"], "ImgSize": ["im"]}, {"Boxes": [boxes], "Scores": [scores]}, anchors=anchors,
                  class_num=c, conf_thresh=0.4, downsample_ratio=32, clip_bbox=True, scale_x_y=1.05)
    gb, gs = _run(b, {"x": x, "im": img}, [boxes, scores])
    sig = lambda v: 1 / (1 + np.exp(-v))
    xr = x.reshape(n, a, 5 + c, h, w)
    rb, rs = np.zeros((n, a, h, w, 4), np.float32), np.zeros((n, a, h, w, c), np.float32)
    for i in range(n):
        ih, iw = img[i]
        for k in range(a):
            for yy in range(h):
                for xx in range(w):
                    t = xr[i, k, :, yy, xx]
                    conf = sig(t[4])
                    if conf < 0.4:
                        continue
                    cx = (xx + sig(t[0]) * 1.05 - 0.025) * iw / w
                    cy = (yy + sig(t[1]) * 1.05 - 0.025) * ih / h
                    bw = np.exp(t[2]) * anchors[2 * k] * iw / (32 * w)
                    bh = np.exp(t[3]) * anchors[2 * k + 1] * ih / (32 * h)
                    rb[i, k, yy, xx] = [max(cx - bw / 2, 0), max(cy - bh / 2, 0), min(cx + bw / 2, iw - 1), min(cy + bh / 2, ih - 1)]
                    rs[i, k, yy, xx] = conf * sig(t[5:])
    np.testing.assert_allclose(gb.numpy(), rb.reshape(n, -1, 4), rtol=1e-4, atol=1e-3)
    np.testing.assert_allclose(gs.numpy(), rs.reshape(n, -1, c), rtol=1e-4, atol=1e-5)


def test_roi_align_on_constant_and_linear_images():
    n, c, h, w = 2, 3, 16, 20
    yy, xx = np.mgrid[0:h, 0:w].astype(np.float32)
    x = np.zeros((n, c, h, w), np.float32)
    x[0] = 7.0                                   # constant image
    x[1, 0], x[1, 1], x[1, 2] = xx, yy, 2 * xx + 3 * yy        # linear ramps: bilinear sampling is exact
    rois = np.array([[2.0, 3.0, 10.0, 9.0], [4.0, 2.0, 16.0, 12.0], [1.0, 1.0, 5.0, 13.0]], np.float32)
    b = _builder()
    b.feed("x", "float32", [n, c, h, w])
    b.feed("rois", "float32", [3, 4])
    b.feed("num", "int32", [n])
    y = b.op("roi_align", {"X": ["x"], "ROIs": ["rois"], "RoisNum": ["num"]}, ("Out",), [3, c, 2, 4], pooled_height=2,
             pooled_width=4, spatial_scale=0.5, sampling_ratio=2, aligned=True)
    got, = _run(b, {"x": x, "rois": rois, "num": np.array([1, 2], np.int32)}, [y])
    got = got.numpy()
    np.testing.assert_allclose(got[0], 7.0, rtol=1e-6)
    for r in (1, 2):
        x1, y1, x2, y2 = rois[r] * 0.5 - 0.5
        bw, bh = (x2 - x1) / 4, (y2 - y1) / 2
        cx = x1 + (np.arange(4) + 0.5) * bw            # a bin's mean of a linear function = its value at the bin centre
        cy = y1 + (np.arange(2) + 0.5) * bh
        np.testing.assert_allclose(got[r, 0], np.broadcast_to(cx[None, :], (2, 4)), rtol=1e-5, atol=1e-5)
        np.testing.assert_allclose(got[r, 1], np.broadcast_to(cy[:, None], (2, 4)), rtol=1e-5, atol=1e-5)
        np.testing.assert_allclose(got[r, 2], 2 * cx[None, :] + 3 * cy[:, None], rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("bidirec", [False, True])
def test_rnn_lstm_matches_torch(bidirec):
    torch.manual_seed(0)
    seq, batch, inp, hid, layers = 5, 3, 6, 4, 2
    ref = torch.nn.LSTM(inp, hid, num_layers=layers, bidirectional=bidirec)
    b = _builder()
    b.feed("x", "float32", [seq, batch, inp])
    ndir = 2 if bidirec else 1
    weights, biases = [], []
    for layer in range(layers):
        for d in range(ndir):
            sfx = f"_l{layer}" + ("_reverse" if d else "")
            weights += [b.param(f"w_ih{sfx}", getattr(ref, "weight_ih" + sfx).detach().numpy()),
                        b.param(f"w_hh{sfx}", getattr(ref, "weight_hh" + sfx).detach().numpy())]
            biases += [b.param(f"b_ih{sfx}", getattr(ref, "bias_ih" + sfx).detach().numpy()),
                       b.param(f"b_hh{sfx}", getattr(ref, "bias_hh" + sfx).detach().numpy())]
    h0 = np.random.RandomState(1).randn(layers * ndir, batch, hid).astype(np.float32)
    c0 = np.random.RandomState(2).randn(layers * ndir, batch, hid).astype(np.float32)
    b.feed("h0", "float32", list(h0.shape))
    b.feed("c0", "float32", list(c0.shape))
    out = b.prog.add_var("out", "float32", [seq, batch, ndir * hid])
    hn = b.prog.add_var("hn", "float32", list(h0.shape))
    cn = b.prog.add_var("cn", "float32", list(c0.shape))
    b.prog.add_op("rnn", {"Input": ["x"], "PreState": ["h0", "c0"], "WeightList": weights + biases},
                  {"Out": [out], "State": [hn, cn]}, mode="LSTM", num_layers=layers, is_bidirec=bidirec, hidden_size=hid,
                  input_size=inp)
    x = np.random.RandomState(3).randn(seq, batch, inp).astype(np.float32)
    gy, gh, gc = _run(b, {"x": x, "h0": h0, "c0": c0}, [out, hn, cn])
    ry, (rh, rc) = ref(torch.from_numpy(x), (torch.from_numpy(h0), torch.from_numpy(c0)))
    torch.testing.assert_close(gy, ry.detach(), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(gh, rh.detach(), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(gc, rc.detach(), rtol=1e-4, atol=1e-5)


def test_group_norm_prelu_affine_channel_grid_sampler():
    rng = np.random.RandomState(4)
    x = rng.randn(2, 6, 5, 7).astype(np.float32)
    b = _builder()
    b.feed("x", "float32", [2, 6, 5, 7])
    b.feed("grid", "float32", [2, 3, 4, 2])
    sc, bi = rng.rand(6).astype(np.float32) + 0.5, rng.randn(6).astype(np.float32)
    gn = b.op("group_norm", {"X": ["x"], "Scale": [b.param("gs", sc)], "Bias": [b.param("gb", bi)]}, ("Y",), [2, 6, 5, 7],
              groups=3, epsilon=1e-5)
    al = rng.rand(6).astype(np.float32)
    pr = b.op("prelu", {"X": ["x"], "Alpha": [b.param("alpha", al)]}, ("Out",), [2, 6, 5, 7], mode="channel")
    ac = b.op("affine_channel", {"X": ["x"], "Scale": [b.param("as", sc)], "Bias": [b.param("ab", bi)]}, ("Out",), [2, 6, 5, 7])
    gs = b.op("grid_sampler", {"X": ["x"], "Grid": ["grid"]}, ("Output",), [2, 6, 3, 4], mode="bilinear",
              padding_mode="zeros", align_corners=True)
    grid = rng.uniform(-1.1, 1.1, (2, 3, 4, 2)).astype(np.float32)
    g1, g2, g3, g4 = _run(b, {"x": x, "grid": grid}, [gn, pr, ac, gs])
    xt = torch.from_numpy(x)
    torch.testing.assert_close(g1, torch.nn.functional.group_norm(xt, 3, torch.from_numpy(sc), torch.from_numpy(bi)), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(g2, torch.nn.functional.prelu(xt, torch.from_numpy(al)))
    torch.testing.assert_close(g3, xt * torch.from_numpy(sc).view(1, 6, 1, 1) + torch.from_numpy(bi).view(1, 6, 1, 1))
    torch.testing.assert_close(g4, torch.nn.functional.grid_sample(xt, torch.from_numpy(grid), align_corners=True))


def test_indexing_and_creation_mappers():
    rng = np.random.RandomState(5)
    x = rng.randn(4, 5).astype(np.float32)
    idx = np.array([[0, 4, 2], [1, 1, 3], [4, 0, 0], [2, 3, 1]], np.int64)
    b = _builder()
    b.feed("x", "float32", [4, 5])
    b.feed("idx", "int64", [4, 3])
    b.feed("ids", "int64", [2])
    b.feed("upd", "float32", [2, 5])
    b.feed("lab", "int64", [4])
    isamp = b.op("index_sample", {"X": ["x"], "Index": ["idx"]}, ("Out",), [4, 3])
    srt = b.prog.add_var("srt", "float32", [4, 5])
    sidx = b.prog.add_var("sidx", "int64", [4, 5])
    b.prog.add_op("argsort", {"X": ["x"]}, {"Out": [srt], "Indices": [sidx]}, axis=-1, descending=True)
    sc = b.op("scatter", {"X": ["x"], "Ids": ["ids"], "Updates": ["upd"]}, ("Out",), [4, 5], overwrite=True)
    sca = b.op("scatter", {"X": ["x"], "Ids": ["ids"], "Updates": ["upd"]}, ("Out",), [4, 5], overwrite=False)
    oh = b.op("one_hot_v2", {"X": ["lab"]}, ("Out",), [4, 6], depth=6)
    ey = b.op("eye", {}, ("Out",), [3, 4], num_rows=3, num_columns=4, dtype=5)
    anyv = b.op("reduce_any", {"X": [b.op("greater_than", {"X": ["x"], "Y": [b.param("one", np.array([1.0], np.float32))]},
                                           ("Out",), [4, 5], var_dtype="bool")]}, ("Out",), [4], var_dtype="bool", dim=[1],
                keep_dim=False)
    sv = b.op("set_value", {"Input": ["x"]}, ("Out",), [4, 5], axes=[0, 1], starts=[1, 0], ends=[3, 2], steps=[1, 1],
              decrease_axes=[], none_axes=[], shape=[1], fp32_values=[9.0])
    wi = b.op("where_index", {"Condition": [b.op("greater_than", {"X": ["x"], "Y": [b.param("one2", np.array([0.5], np.float32))]},
                                                 ("Out",), [4, 5], var_dtype="bool")]}, ("Out",), [-1, 2], var_dtype="int64")
    dt = b.op("dot", {"X": ["x"], "Y": ["x"]}, ("Out",), [4])
    ds = b.op("dist", {"X": ["x"], "Y": [b.op("scale", {"X": ["x"]}, ("Out",), [4, 5], scale=0.5, bias=0.0)]}, ("Out",), [1], p=2.0)
    ids = np.array([3, 1], np.int64)
    upd = rng.randn(2, 5).astype(np.float32)
    lab = np.array([0, 5, 2, 2], np.int64)
    outs = _run(b, {"x": x, "idx": idx, "ids": ids, "upd": upd, "lab": lab}, [isamp, srt, sidx, sc, sca, oh, ey, anyv, sv, wi, dt, ds])
    g = [o.numpy() for o in outs]
    np.testing.assert_array_equal(g[0], np.take_along_axis(x, idx, 1))
    order = np.argsort(-x, axis=1, kind="stable")
    np.testing.assert_array_equal(g[1], np.take_along_axis(x, order, 1))
    np.testing.assert_array_equal(g[2], order)
    ref = x.copy(); ref[ids] = upd
    np.testing.assert_array_equal(g[3], ref)
    np.testing.assert_allclose(g[4], ref)                  # distinct ids: accumulate over a zeroed row = overwrite
    np.testing.assert_array_equal(g[5], np.eye(6, dtype=np.float32)[lab])
    np.testing.assert_array_equal(g[6], np.eye(3, 4, dtype=np.float32))
    np.testing.assert_array_equal(g[7], (x > 1.0).any(1))
    ref = x.copy(); ref[1:3, 0:2] = 9.0
    np.testing.assert_array_equal(g[8], ref)
    np.testing.assert_array_equal(g[9], np.argwhere(x > 0.5))
    np.testing.assert_allclose(g[10], (x * x).sum(1), rtol=1e-5)
    np.testing.assert_allclose(g[11], [np.sqrt(((0.5 * x) ** 2).sum())], rtol=1e-5)


def test_meshgrid_linspace_temporal_shift_partial_ops():
    rng = np.random.RandomState(6)
    b = _builder()
    b.feed("a", "float32", [3])
    b.feed("c", "float32", [4])
    b.feed("v", "float32", [6, 8, 2, 2])
    m0 = b.prog.add_var("m0", "float32", [3, 4])
    m1 = b.prog.add_var("m1", "float32", [3, 4])
    b.prog.add_op("meshgrid", {"X": ["a", "c"]}, {"Out": [m0, m1]})
    ls = b.op("linspace", {"Start": [b.param("ls0", np.array([1.0], np.float32))], "Stop": [b.param("ls1", np.array([3.0], np.float32))],
                           "Num": [b.param("lsn", np.array([5], np.int32))]}, ("Out",), [5], dtype=5)
    ts = b.op("temporal_shift", {"X": ["v"]}, ("Out",), [6, 8, 2, 2], seg_num=3, shift_ratio=0.25)
    pc = b.op("partial_concat", {"X": [m0, m1]}, ("Out",), [3, 4], start_index=1, length=2)
    ps = b.op("partial_sum", {"X": [m0, m1]}, ("Out",), [3, 2], start_index=1, length=2)
    a, c = rng.randn(3).astype(np.float32), rng.randn(4).astype(np.float32)
    v = rng.randn(6, 8, 2, 2).astype(np.float32)
    g = [o.numpy() for o in _run(b, {"a": a, "c": c, "v": v}, [m0, m1, ls, ts, pc, ps])]
    r0, r1 = np.meshgrid(a, c, indexing="ij")
    np.testing.assert_array_equal(g[0], r0)
    np.testing.assert_array_equal(g[1], r1)
    np.testing.assert_allclose(g[2], np.linspace(1, 3, 5), rtol=1e-6)
    vv = v.reshape(2, 3, 8, 2, 2)
    ref = np.zeros_like(vv)
    ref[:, 1:, :2] = vv[:, :-1, :2]
    ref[:, :-1, 2:4] = vv[:, 1:, 2:4]
    ref[:, :, 4:] = vv[:, :, 4:]
    np.testing.assert_array_equal(g[3], ref.reshape(6, 8, 2, 2))
    np.testing.assert_array_equal(g[4], np.concatenate([r0[:, 1:3], r1[:, 1:3]], 1))
    np.testing.assert_array_equal(g[5], r0[:, 1:3] + r1[:, 1:3])


def _qdq_mlp(seed=0, hidden=64, out=32):
    """x -> QDQ -> matmul(int8 weight, per-channel) + bias -> relu -> QDQ -> matmul -> out, as PaddleSlim exports it."""
    rng = np.random.RandomState(seed)
    b = _builder()
    b.feed("x", "float32", [-1, hidden])
    w1 = rng.randn(hidden, hidden).astype(np.float32) * 0.2
    w2 = rng.randn(hidden, out).astype(np.float32) * 0.2
    cur = "x"
    floats = []
    for k, (w, act_range) in enumerate(((w1, 3.0), (w2, 4.0))):
        rng_w = np.abs(w).max(0)
        w8 = np.clip(np.round(w / rng_w * 127), -127, 127).astype(np.int8)
        floats.append(w8.astype(np.float32) * rng_w / 127)
        sx = b.param(f"sx{k}", np.array([act_range], np.float32))
        zx = b.param(f"zx{k}", np.zeros(1, np.float32))
        q = b.prog.add_var(f"q{k}", "float32", [-1, hidden])
        b.prog.add_op("quantize_linear", {"X": [cur], "Scale": [sx], "ZeroPoint": [zx]}, {"Y": [q]}, quant_axis=-1, bit_length=8)
        d = b.prog.add_var(f"d{k}", "float32", [-1, hidden])
        b.prog.add_op("dequantize_linear", {"X": [q], "Scale": [sx], "ZeroPoint": [zx]}, {"Y": [d]}, quant_axis=-1, bit_length=8)
        wf = b.prog.add_var(f"wf{k}", "float32", list(w.shape))
        b.prog.add_op("dequantize_linear", {"X": [b.param(f"w8_{k}", w8)], "Scale": [b.param(f"sw{k}", rng_w.astype(np.float32))],
                                            "ZeroPoint": [b.param(f"zw{k}", np.zeros(w.shape[1], np.float32))]}, {"Y": [wf]},
                      quant_axis=1, bit_length=8)
        cur = b.op("matmul_v2", {"X": [d], "Y": [wf]}, ("Out",), [-1, w.shape[1]], trans_x=False, trans_y=False)
        if k == 0:
            bias = b.param("b0", rng.randn(hidden).astype(np.float32) * 0.1)
            cur = b.op("elementwise_add", {"X": [cur], "Y": [bias]}, ("Out",), [-1, hidden], axis=-1)
            cur = b.op("relu", {"X": [cur]}, ("Out",), [-1, hidden])
            floats.append(rng.randn(0))     # placeholder keeps indices simple
    b.fetch(cur)
    return b, floats


def test_qdq_pass_removes_fake_quantisation_and_records_ranges():
    from fastdeploy_b200.importer.paddle_import import load_paddle
    from fastdeploy_b200.ir import passes
    b, _ = _qdq_mlp()
    g = load_paddle(*b.serialize())
    assert sum(n.op == "QuantizeLinear" for n in g.nodes) == 2 and sum(n.op == "DequantizeLinear" for n in g.nodes) == 4
    opt = passes.optimize(g, {"x": [8, 64]})
    assert [n.op for n in opt.nodes] == ["FusedGemm", "FusedGemm"]
    scales = passes.get_act_scales(opt)
    assert sorted(round(v, 4) for v in scales.values()) == [3.0, 4.0]
    assert set(scales) == {n.inputs[0] for n in opt.nodes}
    # the ranges survive the serialised form the plan cache uses
    from fastdeploy_b200.importer.onnx_format import load_onnx, save_onnx
    assert passes.get_act_scales(load_onnx(save_onnx(opt))) == scales
