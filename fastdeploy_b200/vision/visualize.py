"""Result visualisation and compositing (fastdeploy/vision/visualize/*.cc, python/fastdeploy/vision/
visualize/__init__.py:20-260).

Every function accepts a NumPy BGR image (host path, same drawing rules as the reference's OpenCV code)
or a CUDA ``uint8 [H, W, 3]`` tensor (device path: the rasterisers of csrc/kernels/visualize.cu write
into a device buffer; nothing touches a window or a graphics API). Text labels exist on the host path
only (``cv2.putText``).
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import numpy as np

from .result import (DetectionResult, FaceDetectionResult, KeyPointDetectionResult, MattingResult, MOTResult, OCRResult,
                     SegmentationResult)


def get_color_map(n: int = 256) -> np.ndarray:
    """The bit-interleaving colour table of visualize.cc:22-40 (label k -> BGR)."""
    table = np.zeros((n, 3), np.uint8)
    for i in range(n):
        lab, j = i, 0
        while lab:
            table[i, 0] |= ((lab >> 0) & 1) << (7 - j)
            table[i, 1] |= ((lab >> 1) & 1) << (7 - j)
            table[i, 2] |= ((lab >> 2) & 1) << (7 - j)
            lab >>= 3
            j += 1
    return table


_COLORS = get_color_map(256)


def _is_cuda(x) -> bool:
    return hasattr(x, "is_cuda") and x.is_cuda


def _lib():
    from .. import _native
    lib = _native.kernels()
    if not getattr(lib, "_vis_ready", False):
        vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        lib.fdb_vis_draw_boxes.argtypes = [vp, i, i, vp, vp, i, i, vp]
        lib.fdb_vis_blend_label_map.argtypes = [vp, vp, vp, i, i, i, f, i, vp]
        lib.fdb_vis_blend_masks.argtypes = [vp, vp, vp, i, i, i, f, vp]
        lib.fdb_vis_draw_points.argtypes = [vp, i, i, vp, vp, i, i, vp]
        lib.fdb_vis_draw_segments.argtypes = [vp, i, i, vp, vp, i, i, vp]
        lib.fdb_vis_box_blur.argtypes = [vp, vp, vp, i, i, i, vp]
        lib.fdb_vis_composite.argtypes = [vp, vp, vp, vp, i, i, i, f, i, i, i, i, i, vp]
        lib._vis_ready = True
    return lib


def _stream():
    from ..ops.base import current_stream_ptr
    return ctypes.c_void_p(current_stream_ptr())


def _dev(arr, dtype, device):
    import torch
    return torch.as_tensor(np.ascontiguousarray(arr), dtype=dtype).to(device)


# ------------------------------------------------------------------ detection
def vis_detection(im, result: DetectionResult, labels: Optional[Sequence[str]] = None, score_threshold: float = 0.0,
                  line_size: int = 1, font_size: float = 0.5):
    keep = [i for i, s in enumerate(result.scores) if s >= score_threshold]
    if _is_cuda(im):
        import torch
        out = im.clone()
        if keep:
            h, w = out.shape[:2]
            boxes = _dev([result.boxes[i] for i in keep], torch.float32, im.device)
            cols = _dev([_COLORS[result.label_ids[i] % 256] for i in keep], torch.uint8, im.device)
            if result.contain_masks and result.masks:
                full = np.zeros((len(keep), h, w), np.uint8)
                for k, i in enumerate(keep):
                    b = [int(v) for v in result.boxes[i]]
                    m = np.asarray(result.masks[i].data, np.uint8).reshape(result.masks[i].shape)
                    full[k, b[1]:b[1] + m.shape[0], b[0]:b[0] + m.shape[1]] = m[:h - b[1], :w - b[0]]
                _lib().fdb_vis_blend_masks(out.data_ptr(), _dev(full, torch.uint8, im.device).data_ptr(), cols.data_ptr(),
                                           len(keep), h, w, 0.5, _stream())
            _lib().fdb_vis_draw_boxes(out.data_ptr(), h, w, boxes.data_ptr(), cols.data_ptr(), len(keep), max(1, line_size), _stream())
        return out
    import cv2
    out = im.copy()
    for i in keep:
        b = [int(round(v)) for v in result.boxes[i]]
        c = tuple(int(v) for v in _COLORS[result.label_ids[i] % 256])
        if result.contain_masks and result.masks:
            m = np.asarray(result.masks[i].data, np.uint8).reshape(result.masks[i].shape) > 0
            roi = out[b[1]:b[1] + m.shape[0], b[0]:b[0] + m.shape[1]]
            mm = m[:roi.shape[0], :roi.shape[1]]
            roi[mm] = (roi[mm] * 0.5 + np.asarray(c) * 0.5).astype(np.uint8)
        cv2.rectangle(out, (b[0], b[1]), (b[2], b[3]), c, line_size)
        name = labels[result.label_ids[i]] if labels and result.label_ids[i] < len(labels) else str(result.label_ids[i])
        cv2.putText(out, f"{name},{result.scores[i]:.2f}", (b[0], max(b[1] - 2, 8)), cv2.FONT_HERSHEY_SIMPLEX, font_size, c, 1)
    return out


def vis_face_detection(im, result: FaceDetectionResult, line_size: int = 1, font_size: float = 0.5):
    k = result.landmarks_per_face
    if _is_cuda(im):
        import torch
        out = im.clone()
        n = len(result.boxes)
        if n:
            h, w = out.shape[:2]
            cols = _dev([_COLORS[(i + 1) % 256] for i in range(n)], torch.uint8, im.device)
            _lib().fdb_vis_draw_boxes(out.data_ptr(), h, w, _dev(result.boxes, torch.float32, im.device).data_ptr(), cols.data_ptr(),
                                      n, max(1, line_size), _stream())
            if k:
                pcols = _dev([_COLORS[(i // k + 1) % 256] for i in range(n * k)], torch.uint8, im.device)
                _lib().fdb_vis_draw_points(out.data_ptr(), h, w, _dev(result.landmarks, torch.float32, im.device).data_ptr(),
                                           pcols.data_ptr(), n * k, max(1, line_size + 1), _stream())
        return out
    import cv2
    out = im.copy()
    for i, b in enumerate(result.boxes):
        c = tuple(int(v) for v in _COLORS[(i + 1) % 256])
        cv2.rectangle(out, (int(b[0]), int(b[1])), (int(b[2]), int(b[3])), c, line_size)
        cv2.putText(out, f"{result.scores[i]:.2f}", (int(b[0]), max(int(b[1]) - 2, 8)), cv2.FONT_HERSHEY_SIMPLEX, font_size, c, 1)
        for j in range(k):
            p = result.landmarks[i * k + j]
            cv2.circle(out, (int(p[0]), int(p[1])), line_size + 1, c, -1)
    return out


# ------------------------------------------------------------------ segmentation
def vis_segmentation(im, result: SegmentationResult, weight: float = 0.5):
    h, w = result.shape[:2]
    if _is_cuda(im):
        import torch
        out = im.clone()
        lab = _dev(np.asarray(result.label_map, np.int32).reshape(h, w), torch.int32, im.device)
        table = _dev(_COLORS, torch.uint8, im.device)
        _lib().fdb_vis_blend_label_map(out.data_ptr(), lab.data_ptr(), table.data_ptr(), 256, h, w, weight, -1, _stream())
        return out
    lab = np.asarray(result.label_map, np.int64).reshape(h, w)
    color = _COLORS[lab % 256]
    return np.rint(im.astype(np.float32) * (1 - weight) + color.astype(np.float32) * weight).astype(np.uint8)


# ------------------------------------------------------------------ matting / background
def box_blur(im, radius: int):
    if _is_cuda(im):
        import torch
        tmp, out = torch.empty_like(im), torch.empty_like(im)
        _lib().fdb_vis_box_blur(im.data_ptr(), tmp.data_ptr(), out.data_ptr(), im.shape[0], im.shape[1], radius, _stream())
        return out

    def one(a, axis):
        acc = np.zeros(a.shape, np.int64)
        cnt = np.zeros(a.shape[:2] + (1,), np.int64)
        for d in range(-radius, radius + 1):
            sh = np.roll(a.astype(np.int64), -d, axis=axis)
            valid = np.ones(a.shape[:2] + (1,), np.int64)
            idx = [slice(None)] * 3
            if d > 0:
                idx[axis] = slice(a.shape[axis] - d, None)
            elif d < 0:
                idx[axis] = slice(0, -d)
            if d != 0:
                sh[tuple(idx)] = 0
                valid[tuple(idx[:2]) + (slice(None),)] = 0
            acc += sh
            cnt += valid
        return ((acc + cnt // 2) // cnt).astype(np.uint8)
    return one(one(im, 1), 0)


def _composite(fg, alpha, bg, alpha_mode: int, threshold: float, fg_label: int, color):
    if _is_cuda(fg):
        import torch
        out = torch.empty_like(fg)
        h, w = fg.shape[:2]
        c = color if color is not None else (0, 0, 0)
        _lib().fdb_vis_composite(fg.data_ptr(), alpha.data_ptr(), bg.data_ptr() if bg is not None else None, out.data_ptr(), h, w,
                                 alpha_mode, threshold, fg_label, 0 if bg is not None else 1, int(c[0]), int(c[1]), int(c[2]), _stream())
        return out
    if alpha_mode == 2:
        a = (np.asarray(alpha) == fg_label).astype(np.float32)
    else:
        a = np.asarray(alpha, np.float32)
        if alpha_mode == 1:
            a = (a > threshold).astype(np.float32)
        a = np.clip(a, 0, 1)
    b = bg.astype(np.float32) if bg is not None else np.broadcast_to(np.asarray(color, np.float32), fg.shape)
    return np.rint(a[..., None] * fg.astype(np.float32) + (1 - a[..., None]) * b).astype(np.uint8)


def vis_matting(im, result: MattingResult, transparent_background: bool = False, transparent_threshold: float = 0.999,
                remove_small_connected_area: bool = False):
    """The person over a green screen (matting.cc:24-100)."""
    h, w = result.shape[:2]
    alpha = np.asarray(result.alpha, np.float32).reshape(h, w)
    if remove_small_connected_area:
        alpha = remove_small_connected_area_(alpha, 0.05)
    if _is_cuda(im):
        import torch
        return _composite(im, _dev(alpha, torch.float32, im.device), None, 0, 0.0, 0, (120, 255, 155))
    return _composite(im, alpha, None, 0, 0.0, 0, (120, 255, 155))


def swap_background(im, background, result, remove_small_connected_area: bool = False, background_label: int = -1,
                    blur_radius: int = 0, threshold: float = -1.0):
    """Foreground of ``im`` over ``background`` (swap_background.cc:25-130). ``result`` is a
    :class:`MattingResult` (soft alpha, hard when ``threshold >= 0``) or a :class:`SegmentationResult`
    (pixels whose label differs from ``background_label`` are foreground). ``background=None`` with
    ``blur_radius > 0`` gives the portrait mode: the frame itself, box-blurred, is the background."""
    cuda = _is_cuda(im)
    if background is None:
        background = box_blur(im, max(1, blur_radius))
    elif tuple(background.shape[:2]) != tuple(im.shape[:2]):
        from .detection.contrib import _resize_bilinear
        bg_np = background.cpu().numpy() if _is_cuda(background) else background
        bg_np = _resize_bilinear(bg_np, im.shape[1], im.shape[0])
        if cuda:
            import torch
            background = torch.as_tensor(bg_np).to(im.device)
        else:
            background = bg_np
    h, w = im.shape[:2]
    if isinstance(result, SegmentationResult):
        lab = np.asarray(result.label_map, np.int32).reshape(h, w)
        fg_mask = (lab != background_label).astype(np.float32)
        alpha, mode, thr = fg_mask, 0, 0.0
    else:
        alpha = np.asarray(result.alpha, np.float32).reshape(h, w)
        if remove_small_connected_area:
            alpha = remove_small_connected_area_(alpha, 0.05)
        mode, thr = (1, threshold) if threshold >= 0 else (0, 0.0)
    if cuda:
        import torch
        alpha = _dev(alpha, torch.float32, im.device)
    return _composite(im, alpha, background, mode, thr, 0, None)


def remove_small_connected_area_(alpha: np.ndarray, threshold: float = 0.05) -> np.ndarray:
    """Zeroes the connected components of ``alpha > 0`` whose area is below ``threshold`` times the
    largest one (remove_small_connnected_area.cc:24-80)."""
    import cv2
    binary = (alpha > 0).astype(np.uint8)
    n, lab, stats, _ = cv2.connectedComponentsWithStats(binary, connectivity=8)
    if n <= 1:
        return alpha
    areas = stats[1:, cv2.CC_STAT_AREA]
    keep = np.zeros(n, bool)
    keep[1:] = areas >= threshold * areas.max()
    return np.where(keep[lab], alpha, 0.0).astype(alpha.dtype)


# ------------------------------------------------------------------ key points / tracking / OCR
COCO_SKELETON = [(0, 1), (0, 2), (1, 3), (2, 4), (3, 5), (4, 6), (5, 7), (6, 8), (7, 9), (8, 10), (5, 11), (6, 12),
                 (11, 13), (12, 14), (13, 15), (14, 16), (11, 12)]


def vis_keypoint_detection(im, result: KeyPointDetectionResult, conf_threshold: float = 0.5):
    nj = result.num_joints if result.num_joints > 0 else len(result.keypoints)
    persons = len(result.keypoints) // max(nj, 1)
    pts, pcol, segs, scol = [], [], [], []
    for p in range(persons):
        kp = result.keypoints[p * nj:(p + 1) * nj]
        sc = result.scores[p * nj:(p + 1) * nj]
        for j in range(nj):
            if sc[j] >= conf_threshold:
                pts.append(kp[j][:2]); pcol.append(_COLORS[(j + 1) % 256])
        if nj == 17:
            for e, (a, b) in enumerate(COCO_SKELETON):
                if sc[a] >= conf_threshold and sc[b] >= conf_threshold:
                    segs.append([kp[a][0], kp[a][1], kp[b][0], kp[b][1]]); scol.append(_COLORS[(e + 20) % 256])
    if _is_cuda(im):
        import torch
        out = im.clone()
        h, w = out.shape[:2]
        if segs:
            _lib().fdb_vis_draw_segments(out.data_ptr(), h, w, _dev(segs, torch.float32, im.device).data_ptr(),
                                         _dev(scol, torch.uint8, im.device).data_ptr(), len(segs), 2, _stream())
        if pts:
            _lib().fdb_vis_draw_points(out.data_ptr(), h, w, _dev(pts, torch.float32, im.device).data_ptr(),
                                       _dev(pcol, torch.uint8, im.device).data_ptr(), len(pts), 3, _stream())
        return out
    import cv2
    out = im.copy()
    for s, c in zip(segs, scol):
        cv2.line(out, (int(s[0]), int(s[1])), (int(s[2]), int(s[3])), tuple(int(v) for v in c), 2)
    for p, c in zip(pts, pcol):
        cv2.circle(out, (int(p[0]), int(p[1])), 3, tuple(int(v) for v in c), -1)
    return out


def vis_mot(im, result: MOTResult, score_threshold: float = 0.0, records=None):
    det = DetectionResult()
    for b, i, s in zip(result.boxes, result.ids, result.scores):
        if s >= score_threshold:
            det.boxes.append([float(v) for v in b]); det.scores.append(float(s)); det.label_ids.append(int(i))
    return vis_detection(im, det, None, 0.0, 2)


def vis_ppocr(im, result: OCRResult):
    segs, cols = [], []
    for box in result.boxes:
        p = np.asarray(box, np.float32).reshape(4, 2)
        for k in range(4):
            segs.append([*p[k], *p[(k + 1) % 4]]); cols.append([0, 0, 255])
    if _is_cuda(im):
        import torch
        out = im.clone()
        if segs:
            _lib().fdb_vis_draw_segments(out.data_ptr(), out.shape[0], out.shape[1], _dev(segs, torch.float32, im.device).data_ptr(),
                                         _dev(cols, torch.uint8, im.device).data_ptr(), len(segs), 1, _stream())
        return out
    import cv2
    out = im.copy()
    for box in result.boxes:
        cv2.polylines(out, [np.asarray(box, np.int32).reshape(4, 2)], True, (0, 0, 255), 1)
    return out


vis_ocr = vis_ppocr
