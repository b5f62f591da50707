"""Rotated IoU / NMS, CenterPoint decode and grid_sample_3d on the device against host statements."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rand_quads(rng, n, span=100.0):
    cx, cy = rng.uniform(10, span, n), rng.uniform(10, span, n)
    w, h = rng.uniform(4, 30, n), rng.uniform(4, 30, n)
    a = rng.uniform(-math.pi, math.pi, n)
    out = np.zeros((n, 8), np.float32)
    for k, (dx, dy) in enumerate(((-1, -1), (1, -1), (1, 1), (-1, 1))):
        out[:, 2 * k] = cx + dx * w / 2 * np.cos(a) - dy * h / 2 * np.sin(a)
        out[:, 2 * k + 1] = cy + dx * w / 2 * np.sin(a) + dy * h / 2 * np.cos(a)
    return out


def test_quad_iou_matches_polygon_clipping_oracle():
    from fastdeploy_b200.ops import perception as P
    rng = np.random.default_rng(0)
    a, b = _rand_quads(rng, 40, 60.0), _rand_quads(rng, 30, 60.0)
    b[3] = a[5]                          # identical boxes
    b[4] = a[6][[6, 7, 4, 5, 2, 3, 0, 1]]       # the same box with the opposite winding
    got = P.quad_iou(torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()).cpu().numpy()
    ref = np.array([[P.quad_iou_numpy(x, y) for y in b] for x in a])
    np.testing.assert_allclose(got, ref, atol=2e-4)
    assert abs(got[5, 3] - 1.0) < 1e-4 and abs(got[6, 4] - 1.0) < 1e-4 and (got > 0.01).sum() > 20


@pytest.mark.parametrize("keep_top_k", [100, 12])
def test_multiclass_nms_rotated_matches_oracle(keep_top_k):
    from fastdeploy_b200.ops import perception as P
    rng = np.random.default_rng(1)
    c, m = 5, 700
    boxes = _rand_quads(rng, m, 120.0)
    scores = rng.uniform(0, 1, (c, m)).astype(np.float32) ** 4          # few high scores
    ref_rows, ref_idx = P.multiclass_nms_rotated_numpy(boxes, scores, 0.3, 0.2, 60, keep_top_k, background_label=0)
    nms = P.MulticlassNMSRotated(c, m, "cuda", score_threshold=0.3, nms_threshold=0.2, nms_top_k=60, keep_top_k=keep_top_k,
                                 background_label=0, cap=1024)
    for _ in range(2):
        rows, idx = nms.run(torch.from_numpy(boxes).cuda(), torch.from_numpy(scores).cuda())
    assert len(ref_rows) > 10 and rows.shape == ref_rows.shape
    np.testing.assert_array_equal(idx, ref_idx)
    np.testing.assert_allclose(rows, ref_rows, rtol=1e-6)
    small = P.MulticlassNMSRotated(c, m, "cuda", score_threshold=0.0, cap=64)
    with pytest.raises(OverflowError):
        small.run(torch.from_numpy(boxes).cuda(), torch.from_numpy(scores).cuda())


def test_centerpoint_decode_matches_host():
    from fastdeploy_b200.ops.perception import centerpoint_decode_device
    from fastdeploy_b200.vision.perception import centerpoint_decode
    rng = np.random.default_rng(2)
    c, h, w = 3, 40, 48
    hm = rng.normal(-3.0, 1.5, (c, h, w)).astype(np.float32)
    reg = rng.uniform(0, 1, (2, h, w)).astype(np.float32)
    height = rng.uniform(-2, 1, (1, h, w)).astype(np.float32)
    dim = rng.uniform(0.2, 1.6, (3, h, w)).astype(np.float32)
    vel = rng.normal(0, 1, (2, h, w)).astype(np.float32)
    rot = rng.normal(0, 1, (2, h, w)).astype(np.float32)
    kw = dict(voxel_size=[0.2, 0.2], pc_range=[-10.0, -10.0], down_ratio=4, score_threshold=0.1, nms_iou_threshold=0.2,
              post_center_range=[-9.0, -9.0, -5.0, 25.0, 20.0, 3.0], nms_pre_max=300, nms_post_max=40)
    rb, rs, rl = centerpoint_decode(hm, reg, height, dim, vel, rot, **kw)
    t = lambda a: torch.from_numpy(a).cuda()
    gb, gs, gl = centerpoint_decode_device(t(hm), t(reg), t(height), t(dim), t(vel), t(rot), **kw)
    assert 5 < len(rs) <= 40 and len(gs) == len(rs)
    np.testing.assert_allclose(gs.cpu().numpy(), rs, rtol=1e-5)
    np.testing.assert_array_equal(gl.cpu().numpy(), rl)
    np.testing.assert_allclose(gb.cpu().numpy(), rb, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("mode", ["bilinear", "nearest"])
@pytest.mark.parametrize("padding", ["zeros", "border", "reflection"])
@pytest.mark.parametrize("align", [True, False])
def test_grid_sample_3d_matches_torch(mode, padding, align):
    from fastdeploy_b200.ops.perception import grid_sample_3d
    g = torch.Generator().manual_seed(3)
    x = torch.randn(2, 5, 6, 7, 8, generator=g)
    grid = torch.rand(2, 4, 5, 6, 3, generator=g) * 2.6 - 1.3          # some samples outside the volume
    ref = torch.nn.functional.grid_sample(x, grid, mode=mode, padding_mode=padding, align_corners=align)
    got = grid_sample_3d(x.cuda(), grid.cuda(), mode=mode, padding_mode=padding, align_corners=align).cpu()
    if mode == "nearest":
        # a sample within rounding of a cell border may snap to either side: compare where it is unambiguous
        close = (got - ref).abs() < 1e-5
        assert float(close.float().mean()) > 0.995
    else:
        torch.testing.assert_close(got, ref, rtol=1e-4, atol=1e-5)
