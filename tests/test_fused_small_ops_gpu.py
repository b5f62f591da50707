"""Fused small kernels (squeeze-excite gate, bandwidth-bound partial sums, SPP max pools) and the exact
score-floor pre-pass of the device NMS, each against a plain fp32 / NumPy statement of the same operation."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
F = torch.nn.functional


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("act", ["hard_sigmoid", "sigmoid"])
def test_gap_partial_and_ese_gate(dtype, act):
    from fastdeploy_b200.ops import nhwc as K
    torch.manual_seed(0)
    n, h, w, c, ld, cout = 5, 37, 29, 96, 136, 104
    stride = h * w * ld + 64
    buf = torch.randn(n * stride, device="cuda").to(dtype)
    x = torch.as_strided(buf, (n, h, w, c), (stride, w * ld, ld, 1), 40)
    splits = K.gap_splits_v2(h * w, n, c)
    assert splits > 1
    part = torch.full((n * splits * c,), float("nan"), device="cuda")
    K.gap_partial(x, part, n=n, hw=h * w, c=c, x_ld=ld, x_n_stride=stride, splits=splits).launch()
    sums = part.view(n, splits, c).sum(1)
    ref_sum = x.float().sum((1, 2))
    assert (sums - ref_sum).abs().max().item() <= 1e-3 * ref_sum.abs().max().item() + 1e-2
    wt = torch.zeros(cout, 104, device="cuda", dtype=dtype)
    wt[:, :c] = (torch.randn(cout, c, device="cuda") * 0.2).to(dtype)
    bias = torch.randn(cout, device="cuda")
    out = torch.zeros(n, 112, device="cuda")
    K.ese_gate(part, wt, bias, out, n=n, cin=c, cout=cout, splits=splits, hw=h * w, act=act, alpha=1 / 6.0, beta=0.5,
               out_ld=112).launch()
    torch.cuda.synchronize()
    z = x.float().mean((1, 2)) @ wt[:, :c].float().t() + bias
    ref = torch.clamp(z / 6.0 + 0.5, 0, 1) if act == "hard_sigmoid" else torch.sigmoid(z)
    assert (out[:, :cout] - ref).abs().max().item() <= 2e-3
    assert float(out[:, cout:].abs().max()) == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("hw,c", [((20, 20), 384), ((13, 17), 40), ((32, 32), 8)])
def test_spp_maxpool_matches_three_pools(dtype, hw, c):
    from fastdeploy_b200.ops import nhwc as K
    torch.manual_seed(1)
    n, (h, w) = 3, hw
    x = torch.randn(n, h, w, c, device="cuda").to(dtype)
    cat = torch.zeros(n, h, w, 4 * c, device="cuda", dtype=dtype)
    cat[..., :c] = x
    outs = [cat[..., (i + 1) * c:(i + 2) * c] for i in range(3)]
    K.spp_maxpool(x, outs, [5, 9, 13], n=n, h=h, w=w, c=c, y_lds=[4 * c] * 3,
                  y_n_strides=[h * w * 4 * c] * 3).launch()
    torch.cuda.synchronize()
    xc = x.float().permute(0, 3, 1, 2)
    for i, k in enumerate((5, 9, 13)):
        ref = F.max_pool2d(xc, k, 1, k // 2).permute(0, 2, 3, 1)
        assert torch.equal(outs[i].float(), ref), k
    assert torch.equal(cat[..., :c], x)


def _nms_case(n, m, c, seed, kind, dtype):
    rng = np.random.RandomState(seed)
    ctr = rng.rand(n, m, 2).astype(np.float32) * 600
    wh = rng.rand(n, m, 2).astype(np.float32) * (200 if kind == "crowded" else 60) + 4
    boxes = np.concatenate([ctr - wh / 2, ctr + wh / 2], -1).astype(np.float32)
    scores = rng.rand(n, c, m).astype(np.float32)
    if kind == "sparse":
        scores = scores ** 10
    elif kind == "flat":
        scores = 0.5 + 0.02 * (scores - 0.5)        # an untrained head: everything passes, everything nearly ties
    scores[:, :, ::5] = np.round(scores[:, :, ::5], 2)
    if dtype == torch.float16:
        scores = scores.astype(np.float16).astype(np.float32)
    return boxes, scores


@pytest.mark.parametrize("kind", ["dense", "sparse", "flat", "crowded"])
@pytest.mark.parametrize("dtype,class_major", [(torch.float32, True), (torch.float16, False)])
def test_nms_score_floor_prepass_is_exact(kind, dtype, class_major):
    """With many classes the pre-pass is active; the result must equal the CPU algorithm row for row, and equal
    the device result without the pre-pass."""
    from fastdeploy_b200.ops.nms import MulticlassNMS, multiclass_nms_reference
    n, m, c = 3, 2100, 40
    boxes, scores = _nms_case(n, m, c, 11, kind, dtype)
    kw = dict(score_threshold=0.01, nms_threshold=0.6, nms_top_k=400, keep_top_k=60)
    ref_out, ref_idx, ref_num = multiclass_nms_reference(boxes, scores, normalized=True, **kw)
    tb = torch.from_numpy(boxes).cuda()
    ts = torch.from_numpy(scores).cuda().to(dtype)
    if not class_major:
        ts = ts.permute(0, 2, 1).contiguous()
    results = []
    for prepass in (True, False):
        nms = MulticlassNMS(tb, ts, class_major=class_major, prepass=prepass, **kw)
        assert (nms.tau is not None) == prepass
        nms.launch()
        torch.cuda.synchronize()
        num = nms.out_num.cpu().numpy()
        assert list(num) == list(ref_num)
        got = np.concatenate([nms.out[i, :num[i]].cpu().numpy() for i in range(n)])
        gidx = np.concatenate([nms.out_index[i, :num[i]].cpu().numpy() + i * m for i in range(n)])
        assert np.array_equal(gidx, ref_idx)
        assert np.allclose(got, ref_out, atol=1e-6)
        results.append(got)
        if prepass and kind in ("flat", "dense"):
            assert float(nms.tau.min()) > 0.01       # the floor really cut the candidate lists
    assert np.array_equal(results[0], results[1])
