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
                  line_size: int = 1, font_size: float = 0.5, font_color: Sequence[int] = (255, 255, 255), font_thickness: int = 1):
    """Boxes (and instance masks) in the class colour; on the host path each box also gets a ``label,score`` caption in
    ``font_color`` on a patch of the class colour (fastdeploy/vision/visualize/detection.cc:27-130)."""
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
        text = f"{name},{result.scores[i]:.2f}"
        (tw, th), _ = cv2.getTextSize(text, cv2.FONT_HERSHEY_SIMPLEX, font_size, font_thickness)
        y0 = max(b[1] - th - 2, 0)
        cv2.rectangle(out, (b[0], y0), (b[0] + tw, y0 + th + 2), c, -1)
        cv2.putText(out, text, (b[0], y0 + th), cv2.FONT_HERSHEY_SIMPLEX, font_size, tuple(int(v) for v in font_color),
                    font_thickness)
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
    """Track boxes coloured by id; with ``records`` (a ``tracking.TrailRecorder``) the recorded centre points of every
    shown track are drawn as dots in the track's colour (fastdeploy/vision/visualize/mot.cc:25-78)."""
    det = DetectionResult()
    for b, i, s in zip(result.boxes, result.ids, result.scores):
        if s >= score_threshold:
            det.boxes.append([float(v) for v in b]); det.scores.append(float(s)); det.label_ids.append(int(i))
    out = vis_detection(im, det, None, 0.0, 2)
    trails = getattr(records, "records", records) if records is not None else None
    if trails:
        import cv2
        canvas, back = _host_image(out)
        for tid in det.label_ids:
            col = tuple(int(v) for v in _COLORS[tid % 256])
            for p in trails.get(tid, []):
                cv2.circle(canvas, (int(p[0]), int(p[1])), 3, col, -1)
        out = back(canvas)
    return out


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


# ------------------------------------------------------------------ face alignment, head pose, 3-D boxes
def _host_image(im):
    """(host copy as numpy, put-back function): the drawing below is a handful of primitives, done on the host."""
    if _is_cuda(im):
        import torch
        return im.cpu().numpy().copy(), lambda a: torch.as_tensor(a).to(im.device)
    return im.copy(), lambda a: a


def vis_face_alignment(im, result, line_size: int = 1):
    """A filled green dot of radius ``line_size`` on every landmark (fastdeploy/vision/visualize/face_alignment.cc:21-33)."""
    import cv2
    out, back = _host_image(im)
    for lm in result.landmarks:
        cv2.circle(out, (int(lm[0]), int(lm[1])), line_size, (0, 255, 0), -1)
    return back(out)


def headpose_axes(euler_angles: Sequence[float], size: int, centre: Sequence[int]) -> np.ndarray:
    """End points [3, 2] (x, y; integer) of the head's X, Y and Z axes drawn from ``centre``. The angles are
    (pitch, yaw, roll) in degrees as the model gives them; yaw is mirrored because the image x axis runs the other way
    (fastdeploy/vision/visualize/headpose.cc:27-49)."""
    p, y, r = (np.deg2rad(np.float32(euler_angles[0])), -np.deg2rad(np.float32(euler_angles[1])),
               np.deg2rad(np.float32(euler_angles[2])))
    sp, cp, sy, cy, sr, cr = np.sin(p), np.cos(p), np.sin(y), np.cos(y), np.sin(r), np.cos(r)
    ends = np.array([[size * cy * cr, size * (cp * sr + cr * sp * sy)],
                     [-size * cy * sr, size * (cp * cr - sp * sy * sr)],
                     [size * sy, -size * cy * sp]], np.float64)
    return np.trunc(ends).astype(np.int64) + np.asarray(centre, np.int64)[None, :]


def vis_headpose(im, result, size: int = 50, line_size: int = 1):
    """The three head axes from the image centre: X red, Y green, Z blue."""
    import cv2
    out, back = _host_image(im)
    c = (out.shape[1] // 2, out.shape[0] // 2)
    for end, col in zip(headpose_axes(result.euler_angles, size, c), ((0, 0, 255), (0, 255, 0), (255, 0, 0))):
        cv2.line(out, c, (int(end[0]), int(end[1])), col, line_size)
    return back(out)


_BOX3D_EDGES = ((1, 0), (2, 7), (3, 6), (4, 5), (1, 2), (2, 3), (3, 4), (4, 1), (0, 7), (7, 6), (6, 5), (5, 0))


def project_boxes_3d(result, k_data: Sequence[float]) -> np.ndarray:
    """Image-plane corners [N, 8, 2] of the 3-D boxes of a :class:`PerceptionResult` under the pinhole matrix ``k_data``
    (9 values, row major). A box is (h, w, l) = ``boxes[i][4:7]`` around the bottom-centre ``center[i]``, turned by
    ``yaw_angle[i]`` about the vertical axis; the rotation keeps the reference's sign convention
    (fastdeploy/vision/visualize/perception.cc:104-139)."""
    n = len(result.scores)
    if n == 0:
        return np.zeros((0, 8, 2), np.float32)
    K = np.asarray(k_data, np.float32).reshape(3, 3)
    b = np.asarray(result.boxes, np.float32).reshape(n, -1)
    h, w, l = b[:, 4:5], b[:, 5:6], b[:, 6:7]
    xs = np.array([0, 1, 1, 1, 1, 0, 0, 0], np.float32)[None] * l - l / 2
    ys = np.array([0, 0, 1, 1, 0, 0, 1, 1], np.float32)[None] * h - h
    zs = np.array([0, 0, 0, 1, 1, 1, 1, 0], np.float32)[None] * w - w / 2
    ry = np.asarray(result.yaw_angle, np.float32)[:, None]
    c, s = np.cos(ry), np.sin(ry)
    ctr = np.asarray(result.center, np.float32).reshape(n, 3)
    pts = np.stack([c * xs + s * zs + ctr[:, 0:1], ys + ctr[:, 1:2], s * xs + c * zs + ctr[:, 2:3]], axis=-1)   # [N, 8, 3]
    proj = pts @ K.T
    with np.errstate(divide="ignore", invalid="ignore"):
        return proj[..., :2] / proj[..., 2:3]


def vis_perception(im, result, config_file: str, score_threshold: float = 0.0, line_size: int = 1, font_size: float = 0.5):
    """Wire-frame 3-D boxes on the frame resized to the model's input size; the camera matrix (``k_data``) and the size
    (``Preprocess: Resize.target_size``) come from the model's yaml. Boxes below a score of 0.5 are left out, as in the
    reference, whatever ``score_threshold`` says (fastdeploy/vision/visualize/perception.cc:46-190)."""
    import cv2
    import yaml
    if not result.scores:
        return im
    with open(config_file) as f:
        cfg = yaml.safe_load(f)
    k_data = cfg.get("k_data")
    if k_data is None or len(k_data) != 9:
        raise ValueError(f"{config_file}: k_data must hold the 9 values of the camera matrix")
    target = next((op["target_size"] for op in cfg.get("Preprocess", []) if op.get("type") == "Resize"), None)
    out, back = _host_image(im)
    if target is not None:
        out = cv2.resize(out, (int(target[1]), int(target[0])), interpolation=cv2.INTER_NEAREST)
    corners = project_boxes_3d(result, k_data)
    for i, score in enumerate(result.scores):
        if score < 0.5 or not np.isfinite(corners[i]).all():
            continue
        lo, hi = corners[i].min(0), corners[i].max(0)
        if not (lo.any() or hi.any()):
            continue
        col = tuple(int(v) for v in _COLORS[result.label_ids[i] % 256])
        for a, b_ in _BOX3D_EDGES:
            cv2.line(out, tuple(int(round(v)) for v in corners[i, a]), tuple(int(round(v)) for v in corners[i, b_]), col, line_size)
        cv2.putText(out, f"{result.label_ids[i]}, {str(float(score))[:4]}", (int(lo[0]), int(lo[1])), cv2.FONT_HERSHEY_SIMPLEX,
                    font_size, (255, 255, 255), 1)
    return back(out)


# ------------------------------------------------------------------ names kept from older releases
def _deprecated(old: str, new: str) -> None:
    from ..utils import log
    log.warning(f"DEPRECATED: fastdeploy.vision.{old} is deprecated, please use fastdeploy.vision.{new} instead.")


def vis_matting_alpha(im, result: MattingResult, remove_small_connected_area: bool = False):
    _deprecated("vis_matting_alpha", "vis_matting")
    return vis_matting(im, result, remove_small_connected_area=remove_small_connected_area)


def swap_background_matting(im, background, result, remove_small_connected_area: bool = False):
    _deprecated("swap_background_matting", "swap_background")
    assert isinstance(result, MattingResult), "The result must be MattingResult type"
    return swap_background(im, background, result, remove_small_connected_area=remove_small_connected_area)


def swap_background_segmentation(im, background, background_label: int, result):
    _deprecated("swap_background_segmentation", "swap_background")
    assert isinstance(result, SegmentationResult), "The result must be SegmentationResult type"
    return swap_background(im, background, result, background_label=background_label)
