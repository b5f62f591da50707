"""PP-TinyPose (fastdeploy/vision/keypointdet/pptinypose/): top-down key-point model. The crop of a
person box is mapped to the network size by an affine transform built from the box centre and scale
(pptinypose_utils.cc:24-84), heat-maps are decoded by arg-max with a quarter-pixel shift towards the
higher neighbour, or by the DARK Taylor refinement when ``use_dark`` is set (:86-170), and points go back
through the inverse transform."""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import numpy as np
import yaml

from ...core.types import ModelFormat
from ...runtime.model import FastDeployModel
from ...runtime.option import RuntimeOption
from ..result import DetectionResult, KeyPointDetectionResult


def get_affine(center, scale, out_size, inv: bool = False) -> np.ndarray:
    """2x3 matrix of the three-point construction: centre, a point half a scale above it, and their
    right-angle companion map to the centre of the output, its top edge and the companion."""
    src_w = scale[0]
    dst_w, dst_h = out_size
    src = np.zeros((3, 2), np.float32)
    dst = np.zeros((3, 2), np.float32)
    src[0] = center
    src[1] = [center[0], center[1] - src_w * 0.5]
    dst[0] = [dst_w * 0.5, dst_h * 0.5]
    dst[1] = [dst_w * 0.5, dst_h * 0.5 - dst_w * 0.5]

    def third(a, b):
        d = a - b
        return b + np.asarray([-d[1], d[0]], np.float32)
    src[2], dst[2] = third(src[0], src[1]), third(dst[0], dst[1])
    if inv:
        src, dst = dst, src
    a = np.concatenate([src, np.ones((3, 1), np.float32)], 1)
    return np.linalg.solve(a, dst).T.astype(np.float32)


def warp_affine(img: np.ndarray, m: np.ndarray, out_size) -> np.ndarray:
    """Bilinear warp with constant zero border (cv2.warpAffine when available)."""
    try:
        import cv2
        return cv2.warpAffine(img, m, tuple(out_size), flags=cv2.INTER_LINEAR)
    except ImportError:
        w, h = out_size
        full = np.vstack([m, [0, 0, 1]]).astype(np.float64)
        inv = np.linalg.inv(full)
        ys, xs = np.mgrid[0:h, 0:w]
        sx = inv[0, 0] * xs + inv[0, 1] * ys + inv[0, 2]
        sy = inv[1, 0] * xs + inv[1, 1] * ys + inv[1, 2]
        x0, y0 = np.floor(sx).astype(int), np.floor(sy).astype(int)
        out = np.zeros((h, w) + img.shape[2:], np.float32)
        for dy in (0, 1):
            for dx in (0, 1):
                xi, yi = x0 + dx, y0 + dy
                wgt = (1 - np.abs(sx - xi)) * (1 - np.abs(sy - yi))
                ok = (xi >= 0) & (xi < img.shape[1]) & (yi >= 0) & (yi < img.shape[0])
                v = img[np.clip(yi, 0, img.shape[0] - 1), np.clip(xi, 0, img.shape[1] - 1)].astype(np.float32)
                out += np.where(ok, wgt, 0)[..., None] * v.reshape(h, w, -1)
        return np.clip(np.rint(out), 0, 255).astype(img.dtype)


def gaussian_blur(hm: np.ndarray, k: int = 3) -> np.ndarray:
    sigma = 0.3 * ((k - 1) * 0.5 - 1) + 0.8
    ax = np.arange(k) - k // 2
    g = np.exp(-(ax ** 2) / (2 * sigma ** 2))
    g /= g.sum()
    pad = np.pad(hm, k // 2, mode="reflect")
    tmp = sum(g[i] * pad[:, i:i + hm.shape[1]] for i in range(k))
    return sum(g[i] * tmp[i:i + hm.shape[0]] for i in range(k))


def decode_heatmaps(heat: np.ndarray, center, scale, use_dark: bool = True):
    """``heat [J, h, w]`` -> (points [J, 2] in source coordinates, scores [J])."""
    j, h, w = heat.shape
    flat = heat.reshape(j, -1)
    idx = flat.argmax(1)
    scores = flat[np.arange(j), idx]
    pts = np.stack([idx % w, idx // w], 1).astype(np.float32)
    for k in range(j):
        px, py = int(pts[k, 0]), int(pts[k, 1])
        if not (0 < px < w - 1 and 0 < py < h - 1):
            continue
        if use_dark:
            m = np.log(np.maximum(gaussian_blur(heat[k]), 1e-10))
            if 1 < px < w - 2 and 1 < py < h - 2:
                dx = 0.5 * (m[py, px + 1] - m[py, px - 1])
                dy = 0.5 * (m[py + 1, px] - m[py - 1, px])
                dxx = 0.25 * (m[py, px + 2] - 2 * m[py, px] + m[py, px - 2])
                dxy = 0.25 * (m[py + 1, px + 1] - m[py - 1, px + 1] - m[py + 1, px - 1] + m[py - 1, px - 1])
                dyy = 0.25 * (m[py + 2, px] - 2 * m[py, px] + m[py - 2, px])
                det = dxx * dyy - dxy * dxy
                if abs(det) > 1e-12:
                    pts[k, 0] -= (dyy * dx - dxy * dy) / det
                    pts[k, 1] -= (dxx * dy - dxy * dx) / det
        else:
            pts[k, 0] += 0.25 * np.sign(heat[k, py, px + 1] - heat[k, py, px - 1])
            pts[k, 1] += 0.25 * np.sign(heat[k, py + 1, px] - heat[k, py - 1, px])
    sx, sy = scale[0] / w, scale[1] / h
    out = np.stack([pts[:, 0] * sx + center[0] - scale[0] * 0.5, pts[:, 1] * sy + center[1] - scale[1] * 0.5], 1)
    return out, scores


class PPTinyPose(FastDeployModel):
    def __init__(self, model_file: str, params_file: str, config_file: str,
                 runtime_option: Optional[RuntimeOption] = None, model_format: int = ModelFormat.PADDLE):
        super().__init__(runtime_option)
        self.runtime_option.set_model_path(model_file, params_file, model_format)
        self.use_dark = True
        self.normalize, self.permute = True, True
        with open(config_file) as f:
            cfg = yaml.safe_load(f)
        self.size = [192, 256]       # w, h
        self.mean, self.std = [0.485, 0.456, 0.406], [0.229, 0.224, 0.225]
        for op in cfg.get("Preprocess", []):
            if op["type"] == "TopDownEvalAffine":
                self.size = list(op["trainsize"])
            elif op["type"] == "NormalizeImage":
                self.mean, self.std = list(op["mean"]), list(op["std"])
        self.init_runtime()

    def _crop(self, im: np.ndarray, box: Optional[Sequence[float]]):
        h, w = im.shape[:2]
        if box is None:
            box = [0, 0, w - 1, h - 1]
        # expand by 0.3 like the detector-coupled pipeline, keep the model's aspect ratio
        cx, cy = (box[0] + box[2]) / 2, (box[1] + box[3]) / 2
        bw, bh = (box[2] - box[0]), (box[3] - box[1])
        aspect = self.size[0] / self.size[1]
        if bw > aspect * bh:
            bh = bw / aspect
        else:
            bw = bh * aspect
        return (cx, cy), (bw * 1.25, bh * 1.25)

    def predict(self, im: np.ndarray, detection_result: Optional[DetectionResult] = None) -> KeyPointDetectionResult:
        boxes = detection_result.boxes if detection_result is not None and detection_result.boxes else [None]
        res = KeyPointDetectionResult()
        for b in boxes:
            center, scale = self._crop(im, b)
            m = get_affine(center, scale, self.size)
            crop = warp_affine(im, m, self.size)
            x = crop[..., ::-1].astype(np.float32)
            if self.normalize:
                x = (x / 255.0 - np.asarray(self.mean, np.float32)) / np.asarray(self.std, np.float32)
            x = np.ascontiguousarray(x.transpose(2, 0, 1) if self.permute else x)[None]
            outs = self.runtime.infer({self.runtime.get_input_info(0).name: x})
            heat = np.asarray(outs[0], np.float32)[0]
            pts, sc = decode_heatmaps(heat, center, scale, self.use_dark)
            res.keypoints += pts.tolist()
            res.scores += sc.tolist()
            res.num_joints = heat.shape[0]
        return res

    def batch_predict(self, images, detection_results=None):
        return [self.predict(im, detection_results[i] if detection_results else None) for i, im in enumerate(images)]

    def disable_normalize(self) -> None:
        """The graph normalises by itself: the crop goes in as RGB float pixels
        (python/fastdeploy/vision/keypointdetection/pptinypose/__init__.py:74-86)."""
        self.normalize = False

    def disable_permute(self) -> None:
        """The crop goes in HWC."""
        self.permute = False
