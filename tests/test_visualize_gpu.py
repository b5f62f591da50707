"""Device rasterisers against the host drawing code of the same module."""
import numpy as np
import pytest
import torch

from fastdeploy_b200.vision import visualize as V
from fastdeploy_b200.vision.result import DetectionResult, KeyPointDetectionResult, MattingResult, SegmentationResult

pytestmark = pytest.mark.gpu


def _img(h=97, w=131, seed=0):
    return np.random.default_rng(seed).integers(0, 255, (h, w, 3), dtype=np.uint8)


def test_boxes_match_host_rectangles():
    im = _img()
    d = DetectionResult()
    d.boxes = [[15, 16, 60, 40], [70, 50, 129, 95], [-4, -3, 10, 12]]     # edges that do not cross: boxes are drawn concurrently
    d.scores = [0.9, 0.8, 0.7]
    d.label_ids = [1, 7, 300]
    out = V.vis_detection(torch.as_tensor(im).cuda(), d, line_size=2).cpu().numpy()
    ref = im.copy()
    import cv2
    for b, l in zip(d.boxes, d.label_ids):
        c = tuple(int(v) for v in V.get_color_map()[l % 256])
        x1, y1, x2, y2 = int(b[0]), int(b[1]), int(b[2]), int(b[3])
        for t in range(2):      # thickness 2 grows inwards on the device path
            cv2.rectangle(ref, (x1 + t, y1 + t), (x2 - t, y2 - t), c, 1)
    assert (out == ref).all()


def test_label_map_blend_and_composite_and_blur():
    im = _img(seed=1)
    h, w = im.shape[:2]
    s = SegmentationResult()
    s.label_map = (np.arange(h * w) % 5).tolist()
    s.shape = [h, w]
    cpu = V.vis_segmentation(im, s, 0.4)
    gpu = V.vis_segmentation(torch.as_tensor(im).cuda(), s, 0.4).cpu().numpy()
    assert np.abs(cpu.astype(int) - gpu.astype(int)).max() <= 1
    m = MattingResult()
    m.alpha = np.random.default_rng(2).random(h * w).astype(np.float32).tolist()
    m.shape = [h, w]
    bg = _img(seed=3)
    for thr in (-1.0, 0.5):
        cpu = V.swap_background(im, bg, m, threshold=thr)
        gpu = V.swap_background(torch.as_tensor(im).cuda(), torch.as_tensor(bg).cuda(), m, threshold=thr).cpu().numpy()
        assert np.abs(cpu.astype(int) - gpu.astype(int)).max() <= 1
    cpu = V.box_blur(im, 4)
    gpu = V.box_blur(torch.as_tensor(im).cuda(), 4).cpu().numpy()
    assert (cpu == gpu).all()
    portrait = V.swap_background(torch.as_tensor(im).cuda(), None, m, blur_radius=4).cpu().numpy()
    assert portrait.shape == im.shape


def test_keypoints_draw_inside_image():
    im = np.zeros((64, 64, 3), np.uint8)
    r = KeyPointDetectionResult()
    r.num_joints = 17
    r.keypoints = [[float(3 * j + 5), float(2 * j + 8)] for j in range(17)]
    r.scores = [0.9] * 17
    out = V.vis_keypoint_detection(torch.as_tensor(im).cuda(), r).cpu().numpy()
    assert (out.sum(-1) > 0).sum() > 17 * 9
