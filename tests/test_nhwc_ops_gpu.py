"""Memory-bound NHWC kernels, fused pre-processing and device NMS vs plain references."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
F = torch.nn.functional


def _close(a, b, tol):
    err = (a.float() - b.float()).abs().max().item()
    assert err <= tol, f"max abs err {err} > {tol}"


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_gap_se_scale(dtype):
    from fastdeploy_b200.ops import nhwc
    torch.manual_seed(0)
    n, h, w, c = 3, 20, 24, 96
    buf = torch.randn(n, h, w, 128, device="cuda").to(dtype)
    x = buf[..., 32:]
    splits = 4
    scratch = torch.empty(n * splits * c, device="cuda")
    avg = torch.empty(n, c, device="cuda")
    for op in nhwc.global_avgpool(x, avg, scratch, n=n, hw=h * w, c=c, x_ld=128, splits=splits):
        op.launch()
    _close(avg, x.float().mean((1, 2)), 2e-3)
    wt = (torch.randn(c, c, device="cuda") * 0.1).to(dtype)
    b = torch.randn(c, device="cuda")
    s = torch.empty(n, c, device="cuda")
    nhwc.se_fc(avg, wt, b, s, n=n, cin=c, cout=c, act="hard_sigmoid", alpha=1 / 6.0, beta=0.5).launch()
    ref_s = F.hardsigmoid(avg @ wt.float().t() + b)
    _close(s, ref_s, 2e-3)
    y = torch.zeros(n, h, w, c, device="cuda", dtype=dtype)
    nhwc.scale_channels(x, s, y, n=n, hw=h * w, c=c, x_ld=128).launch()
    _close(y, x.float() * ref_s[:, None, None, :], 5e-2)


@pytest.mark.parametrize("k,s,p", [(5, 1, 2), (9, 1, 4), (13, 1, 6), (3, 2, 1), (2, 2, 0)])
def test_maxpool(k, s, p):
    from fastdeploy_b200.ops import nhwc
    torch.manual_seed(1)
    n, h, w, c = 2, 20, 20, 64
    x = torch.randn(n, h, w, c, device="cuda").half()
    ho, wo = (h + 2 * p - k) // s + 1, (w + 2 * p - k) // s + 1
    ybuf = torch.zeros(n, ho, wo, 2 * c, device="cuda", dtype=torch.float16)
    nhwc.pool2d(x, ybuf[..., c:], n=n, h=h, w=w, c=c, kernel=(k, k), stride=(s, s), pad=(p, p), out_hw=(ho, wo),
                y_ld=2 * c).launch()
    ref = F.max_pool2d(x.float().permute(0, 3, 1, 2), k, s, p).permute(0, 2, 3, 1)
    _close(ybuf[..., c:], ref, 0)
    assert float(ybuf[..., :c].abs().max()) == 0


def test_avgpool_exclusive():
    from fastdeploy_b200.ops import nhwc
    torch.manual_seed(2)
    x = torch.randn(2, 15, 15, 32, device="cuda").half()
    y = torch.zeros(2, 8, 8, 32, device="cuda", dtype=torch.float16)
    nhwc.pool2d(x, y, n=2, h=15, w=15, c=32, kernel=(3, 3), stride=(2, 2), pad=(1, 1), out_hw=(8, 8), mode="avg").launch()
    ref = F.avg_pool2d(x.float().permute(0, 3, 1, 2), 3, 2, 1, count_include_pad=False).permute(0, 2, 3, 1)
    _close(y, ref, 2e-3)


def test_upsample_binary_unary_cast():
    from fastdeploy_b200.ops import nhwc
    torch.manual_seed(3)
    x = torch.randn(2, 10, 12, 64, device="cuda").half()
    y = torch.zeros(2, 20, 24, 96, device="cuda", dtype=torch.float16)
    nhwc.upsample_nearest(x, y, n=2, h=10, w=12, c=64, factor=(2, 2), y_ld=96).launch()
    ref = F.interpolate(x.float().permute(0, 3, 1, 2), scale_factor=2, mode="nearest").permute(0, 2, 3, 1)
    _close(y[..., :64], ref, 0)
    a = torch.randn(100, 64, device="cuda").half()
    b = torch.randn(100, 64, device="cuda").half()
    o = torch.empty_like(a)
    nhwc.binary(a, b, o, rows=100, c=64, op="add", act="relu").launch()
    _close(o, torch.relu(a.float() + b.float()), 2e-3)
    nhwc.unary(a, o, rows=100, c=64, act="hard_swish").launch()
    _close(o, F.hardswish(a.float()), 2e-3)
    f = torch.randn(1000, device="cuda")
    hh = torch.empty(1000, device="cuda", dtype=torch.float16)
    nhwc.cast(f, hh).launch()
    _close(hh, f, 2e-3)
    i64 = torch.randint(0, 40000, (777,), device="cuda")
    i32 = torch.empty(777, device="cuda", dtype=torch.int32)
    nhwc.cast(i64, i32).launch()
    assert torch.equal(i32.long(), i64)


def test_dfl_decode():
    from fastdeploy_b200.ops import nhwc
    torch.manual_seed(4)
    n, bins = 2, 17
    levels = [(0, 4, 32), (16, 8, 16), (80, 16, 8)]
    a = 16 + 64 + 256
    reg = torch.randn(n, a, 4 * bins, device="cuda").half()
    sf = torch.tensor([[0.5, 0.25], [2.0, 1.5]], device="cuda")
    boxes = torch.empty(n, a, 4, device="cuda")
    nhwc.dfl_decode(reg, boxes, sf, n=n, anchors=a, bins=bins, levels=levels).launch()
    prob = torch.softmax(reg.float().reshape(n, a, 4, bins), -1)
    dist = (prob * torch.arange(bins, device="cuda")).sum(-1)
    pts, strides = [], []
    for st, w, s in levels:
        ys, xs = torch.meshgrid(torch.arange(w), torch.arange(w), indexing="ij")
        pts.append(torch.stack([xs.flatten() + 0.5, ys.flatten() + 0.5], -1))
        strides.append(torch.full((w * w, 1), float(s)))
    pts = torch.cat(pts).cuda()
    strides = torch.cat(strides).cuda()
    ref = torch.cat([pts - dist[..., :2], pts + dist[..., 2:]], -1) * strides
    ref = ref / torch.stack([sf[:, 1], sf[:, 0], sf[:, 1], sf[:, 0]], -1)[:, None, :]
    _close(boxes, ref, 2e-2)


@pytest.mark.parametrize("interp,cvflag", [("nearest", 0), ("linear", 1), ("cubic", 2)])
@pytest.mark.parametrize("layout", ["nhwc", "nchw"])
def test_preprocess_vs_opencv(interp, cvflag, layout):
    import cv2
    from fastdeploy_b200.ops import preproc
    rng = np.random.RandomState(0)
    imgs = [rng.randint(0, 256, (108, 192, 3), dtype=np.uint8), rng.randint(0, 256, (90, 160, 3), dtype=np.uint8)]
    ho, wo = 64, 80
    mean, std = [0.485, 0.456, 0.406], [0.229, 0.224, 0.225]
    alpha, beta = preproc.normalize_coeffs(mean, std)
    meta = np.zeros(2, dtype=preproc.IMAGE_META)
    off = 0
    blobs = []
    geo = [((64, 80), (0, 0)), ((45, 80), (5, 0))]
    for i, im in enumerate(imgs):
        preproc.fill_meta(meta, i, src_offset=off, src_hw=im.shape[:2], src_stride=im.shape[1] * 3,
                          resized_hw=geo[i][0], top_left=geo[i][1])
        blobs.append(im.reshape(-1))
        off += im.size
    src = torch.from_numpy(np.concatenate(blobs)).cuda()
    meta_d = torch.from_numpy(meta.view(np.uint8)).cuda()
    c_out = 8 if layout == "nhwc" else 3
    dst = torch.zeros((2, ho, wo, c_out) if layout == "nhwc" else (2, 3, ho, wo), device="cuda", dtype=torch.float32)
    preproc.Preprocess(src, meta_d, dst, n=2, out_hw=(ho, wo), layout=layout, c_out=c_out, interp=interp,
                       swap_rb=True, alpha=alpha, beta=beta, pad_value=(0.0, 0.0, 0.0)).launch()
    out = dst.cpu().numpy()
    for i, im in enumerate(imgs):
        (rh, rw), (top, left) = geo[i]
        r = cv2.resize(im, (rw, rh), interpolation=cvflag)[..., ::-1].astype(np.float32)
        ref = np.zeros((ho, wo, 3), np.float32)
        ref[top:top + rh, left:left + rw] = r * np.array(alpha, np.float32) + np.array(beta, np.float32)
        got = out[i][..., :3] if layout == "nhwc" else out[i].transpose(1, 2, 0)
        # one uint8 step of the resized image
        tol = 1.01 * max(alpha)
        bad = np.abs(got - ref) > tol
        assert bad.mean() < 1e-3, f"{bad.mean()} of pixels differ by more than one step"
        if layout == "nhwc":
            assert np.all(out[i][..., 3:] == 0)


def _nms_inputs(n, m, c, seed, dense):
    rng = np.random.RandomState(seed)
    ctr = rng.rand(n, m, 2).astype(np.float32) * 600
    wh = rng.rand(n, m, 2).astype(np.float32) * 120 + 4
    boxes = np.concatenate([ctr - wh / 2, ctr + wh / 2], -1).astype(np.float32)
    scores = rng.rand(n, c, m).astype(np.float32)
    if not dense:
        scores = scores ** 8
    # force ties
    scores[:, :, ::7] = np.round(scores[:, :, ::7], 2)
    return boxes, scores


@pytest.mark.parametrize("dense", [False, True])
@pytest.mark.parametrize("class_major", [True, False])
def test_multiclass_nms_matches_reference(dense, class_major):
    from fastdeploy_b200.ops.nms import MulticlassNMS, multiclass_nms_reference
    n, m, c = 2, 1500, 6
    boxes, scores = _nms_inputs(n, m, c, 5, dense)
    thr = 0.01 if dense else 0.3
    kw = dict(score_threshold=thr, nms_threshold=0.6, nms_top_k=300, keep_top_k=50)
    ref_out, ref_idx, ref_num = multiclass_nms_reference(boxes, scores, normalized=True, **kw)
    tb = torch.from_numpy(boxes).cuda()
    ts = torch.from_numpy(scores).cuda()
    if not class_major:
        ts = ts.permute(0, 2, 1).contiguous()
    nms = MulticlassNMS(tb, ts, class_major=class_major, **kw)
    nms.launch()
    torch.cuda.synchronize()
    num = nms.out_num.cpu().numpy()
    assert list(num) == list(ref_num)
    got = np.concatenate([nms.out[i, :num[i]].cpu().numpy() for i in range(n)])
    gidx = np.concatenate([nms.out_index[i, :num[i]].cpu().numpy() + i * m for i in range(n)])
    assert np.array_equal(gidx, ref_idx)
    assert np.allclose(got, ref_out, atol=1e-6)


@pytest.mark.parametrize("top_k", [1025, 3000, 10000, -1])
def test_multiclass_nms_top_k_beyond_one_pass(top_k):
    """More candidates per class than one pass holds (1024): the exporters' default nms_top_k is 10000. Boxes are
    packed so tightly that most candidates are suppressed and the later passes still add kept boxes."""
    from fastdeploy_b200.ops.nms import MulticlassNMS, multiclass_nms_reference
    rng = np.random.default_rng(11)
    n, m, c = 2, 5000, 3
    centre = rng.uniform(0, 60, (n, m, 2)).astype(np.float32)
    size = rng.uniform(20, 40, (n, m, 2)).astype(np.float32)
    boxes = np.concatenate([centre - size / 2, centre + size / 2], -1)
    scores = rng.uniform(0.05, 1.0, (n, c, m)).astype(np.float32)
    scores[:, :, ::9] = np.round(scores[:, :, ::9], 2)          # ties
    kw = dict(score_threshold=0.1, nms_threshold=0.3, nms_top_k=top_k, keep_top_k=200)
    ref_out, ref_idx, ref_num = multiclass_nms_reference(boxes, scores, normalized=True, **kw)
    nms = MulticlassNMS(torch.from_numpy(boxes).cuda(), torch.from_numpy(scores).cuda(), class_major=True, **kw)
    nms.launch()
    torch.cuda.synchronize()
    num = nms.out_num.cpu().numpy()
    assert list(num) == list(ref_num) and num.min() > 5
    gidx = np.concatenate([nms.out_index[i, :num[i]].cpu().numpy() + i * m for i in range(n)])
    assert np.array_equal(gidx, ref_idx)
    got = np.concatenate([nms.out[i, :num[i]].cpu().numpy() for i in range(n)])
    assert np.allclose(got, ref_out, atol=1e-6)


def test_multiclass_nms_keep_all_and_background():
    from fastdeploy_b200.ops.nms import MulticlassNMS, multiclass_nms_reference
    n, m, c = 1, 400, 4
    boxes, scores = _nms_inputs(n, m, c, 7, False)
    kw = dict(score_threshold=0.2, nms_threshold=0.5, nms_top_k=200, keep_top_k=-1, background_label=0)
    ref_out, ref_idx, ref_num = multiclass_nms_reference(boxes, scores, normalized=False, **kw)
    nms = MulticlassNMS(torch.from_numpy(boxes).cuda(), torch.from_numpy(scores).cuda(), class_major=True,
                        normalized=False, **kw)
    nms.launch()
    torch.cuda.synchronize()
    num = int(nms.out_num[0])
    assert num == int(ref_num[0])
    assert np.array_equal(nms.out_index[0, :num].cpu().numpy(), ref_idx)
    assert np.allclose(nms.out[0, :num].cpu().numpy(), ref_out, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("k,stride,act", [(3, 1, "relu"), (3, 2, "hard_swish"), (5, 1, None), (5, 2, "hard_sigmoid"),
                                          (3, (2, 1), "relu"), (5, (2, 1), "hard_swish"), (5, (1, 2), None),
                                          (7, 1, None)])
def test_depthwise_conv_matches_fp32_reference(dtype, k, stride, act):
    from fastdeploy_b200.ops import nhwc as K
    torch.manual_seed(0)
    n, h, w, c = 2, 23, 31, 24
    x = torch.randn(n, h, w, c, device="cuda").to(dtype)
    wt = torch.randn(c, 1, k, k, device="cuda") * 0.3
    b = torch.randn(c, device="cuda")
    pad = k // 2
    stride = (stride, stride) if isinstance(stride, int) else stride      # (rows, columns); 7x7 takes the generic kernel
    ho, wo = (h + 2 * pad - k) // stride[0] + 1, (w + 2 * pad - k) // stride[1] + 1
    y = torch.empty(n, ho, wo, c, device="cuda", dtype=dtype)
    wk = wt.reshape(c, k * k).t().contiguous()
    op = K.depthwise_conv(x, wk, b, y, n=n, h=h, w_in=w, c=c, kernel=(k, k), stride=stride, pad=(pad, pad),
                          out_hw=(ho, wo), act=act, act_alpha=0.2, act_beta=0.5)
    op.launch()
    torch.cuda.synchronize()
    ref = torch.nn.functional.conv2d(x.float().permute(0, 3, 1, 2), wt, b, stride=stride, padding=pad, groups=c)
    if act == "relu":
        ref = torch.relu(ref)
    elif act == "hard_swish":
        ref = torch.nn.functional.hardswish(ref)
    elif act == "hard_sigmoid":
        ref = torch.clamp(0.2 * ref + 0.5, 0, 1)
    ref = ref.permute(0, 2, 3, 1)
    tol = 3e-2 if dtype == torch.bfloat16 else 5e-3
    assert (y.float() - ref).abs().max().item() <= tol * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("scale_up,center", [(True, True), (False, True), (True, False)])
def test_device_letterbox_matches_host_letterbox(scale_up, center):
    from fastdeploy_b200.vision.detection.contrib import DeviceLetterbox, YOLOPreprocessor
    rng = np.random.default_rng(4)
    import cv2
    images = [cv2.GaussianBlur(rng.integers(0, 256, (h, w, 3), dtype=np.uint8), (0, 0), 2.0)
              for h, w in ((480, 640), (200, 300), (720, 405))]
    pre = YOLOPreprocessor((320, 320))
    pre.is_scale_up, pre.center = scale_up, center
    ref, ref_infos = pre.run(images)                              # [3, 3, 320, 320] fp32, RGB, / 255, padded with 114
    dst = torch.zeros(3, 320, 320, 8, dtype=torch.float16, device="cuda")
    infos = DeviceLetterbox(pre, torch.device("cuda:0")).run(images, dst)
    torch.cuda.synchronize()
    got = dst[..., :3].permute(0, 3, 1, 2).float().cpu().numpy()
    for a, b in zip(infos, ref_infos):
        assert a["pad_w"] == b["pad_w"] and a["pad_h"] == b["pad_h"] and abs(a["scale"] - b["scale"]) < 1e-9
    diff = np.abs(got - ref)
    assert diff.max() <= 2.5 / 255 and diff.mean() < 0.6 / 255          # one rounding step of the resize + fp16
    assert float(dst[..., 3:].abs().max()) == 0.0
