"""Rotated-box and 3-D perception ops on the device (csrc/kernels/perception_ops.cu): exact IoU of quadrilaterals,
rotated NMS (class-aware or class-agnostic), rotated multiclass NMS for PP-YOLOE-R, CenterPoint decode + bird's-eye-view
NMS, ``grid_sample_3d``; with NumPy statements of the rotated multiclass NMS as the test oracle.

Reference: fastdeploy/vision/detection/ppdet/multiclass_nms_rotated.cc:59-477,
fastdeploy/runtime/backends/paddle/ops/{centerpoint_postprocess_op.cu:43-91, iou3d_nms_kernel.cu:294-382,
grid_sample_3d.cu:96-250}."""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import _native
from .base import current_stream_ptr

_P = ctypes.c_void_p


class _CenterPointDesc(ctypes.Structure):
    _fields_ = [("hm", _P), ("reg", _P), ("height", _P), ("dim", _P), ("vel", _P), ("rot", _P),
                ("C", ctypes.c_int), ("H", ctypes.c_int), ("W", ctypes.c_int), ("with_velocity", ctypes.c_int),
                ("voxel_x", ctypes.c_float), ("voxel_y", ctypes.c_float), ("range_x", ctypes.c_float),
                ("range_y", ctypes.c_float), ("down_ratio", ctypes.c_float), ("score_thresh", ctypes.c_float),
                ("nms_thresh", ctypes.c_float), ("post_range", ctypes.c_float * 6), ("use_post_range", ctypes.c_int),
                ("pre_max", ctypes.c_int), ("post_max", ctypes.c_int)]


def _lib():
    lib = _native.kernels()
    if not getattr(lib, "_perception_ready", False):
        lib.fdb_quad_iou.argtypes = [_P, _P, ctypes.c_int, ctypes.c_int, _P, _P]
        lib.fdb_rotated_nms_workspace.restype = ctypes.c_longlong
        lib.fdb_rotated_nms_workspace.argtypes = [ctypes.c_int]
        lib.fdb_rotated_nms.argtypes = [_P, _P, _P, ctypes.c_int, ctypes.c_float, ctypes.c_int, _P, _P, ctypes.c_longlong, _P,
                                        _P, _P]
        lib.fdb_multiclass_rotated_workspace.restype = ctypes.c_longlong
        lib.fdb_multiclass_rotated_workspace.argtypes = [ctypes.c_int, ctypes.c_int]
        lib.fdb_multiclass_nms_rotated.argtypes = [_P, _P, ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_float,
                                                   ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, _P,
                                                   ctypes.c_longlong, _P, _P, _P, _P, _P]
        lib.fdb_centerpoint_workspace.restype = ctypes.c_longlong
        lib.fdb_centerpoint_workspace.argtypes = [ctypes.c_int] * 3
        lib.fdb_centerpoint_decode.argtypes = [ctypes.POINTER(_CenterPointDesc), _P, ctypes.c_longlong, _P, _P, _P, _P, _P, _P, _P]
        lib.fdb_grid_sample_3d.argtypes = [_P, _P, _P] + [ctypes.c_int] * 11 + [_P]
        lib._perception_ready = True
    return lib


def _ok(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what}: {_native.last_error()}")


def _f32(t: torch.Tensor) -> torch.Tensor:
    return t.float().contiguous()


# ---------------------------------------------------------------------------------------------- device ops
def quad_iou(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """IoU matrix ``[na, nb]`` of two sets of convex quadrilaterals ``[n, 8]`` (x1 y1 .. x4 y4, either winding)."""
    a, b = _f32(a), _f32(b)
    out = torch.empty(a.shape[0], b.shape[0], device=a.device)
    _ok(_lib().fdb_quad_iou(a.data_ptr(), b.data_ptr(), a.shape[0], b.shape[0], out.data_ptr(), current_stream_ptr()), "quad_iou")
    return out


def rotated_nms(quads: torch.Tensor, scores: torch.Tensor, thresh: float, classes: Optional[torch.Tensor] = None,
                max_keep: int = 0) -> torch.Tensor:
    """Greedy NMS over quadrilaterals ``[n, 8]``; returns the kept indices in decreasing score order. With
    ``classes`` a box only suppresses boxes of its own class."""
    n = quads.shape[0]
    if n == 0:
        return torch.zeros(0, dtype=torch.int64, device=quads.device)
    order = torch.argsort(scores.float(), descending=True, stable=True)
    q = _f32(quads)[order].contiguous()
    c = classes[order].to(torch.int32).contiguous() if classes is not None else None
    ws = torch.empty(_lib().fdb_rotated_nms_workspace(n), dtype=torch.uint8, device=quads.device)
    keep = torch.zeros(n, dtype=torch.uint8, device=quads.device)
    cnt = torch.zeros(1, dtype=torch.int32, device=quads.device)
    _ok(_lib().fdb_rotated_nms(q.data_ptr(), c.data_ptr() if c is not None else None, None, n, float(thresh), int(max_keep),
                               None, ws.data_ptr(), ws.numel(), keep.data_ptr(), cnt.data_ptr(), current_stream_ptr()),
        "rotated_nms")
    return order[keep.bool()]


class MulticlassNMSRotated:
    """Rotated multiclass NMS of one image on the device: ``boxes [M, 8]`` quadrilaterals and ``scores [C, M]`` ->
    rows ``[label, score, x1, y1, .., x4, y4]`` grouped by class, best first within a class, at most ``keep_top_k``
    overall. Buffers are allocated once for ``cap`` candidates above the score threshold."""

    def __init__(self, num_classes: int, num_boxes: int, device, *, score_threshold: float = 0.1, nms_threshold: float = 0.1,
                 nms_top_k: int = 2000, keep_top_k: int = 100, background_label: int = -1, cap: int = 4096):
        self.c, self.m, self.cap = num_classes, num_boxes, cap
        self.score_threshold, self.nms_threshold = score_threshold, nms_threshold
        self.nms_top_k, self.keep_top_k, self.background = nms_top_k, keep_top_k, background_label
        self.ws = torch.empty(_lib().fdb_multiclass_rotated_workspace(cap, num_classes), dtype=torch.uint8, device=device)
        self.out = torch.zeros(cap, 10, device=device)
        self.out_index = torch.zeros(cap, dtype=torch.int32, device=device)
        self.out_count = torch.zeros(1, dtype=torch.int32, device=device)
        self.overflow = torch.zeros(1, dtype=torch.int32, device=device)

    def run(self, boxes: torch.Tensor, scores: torch.Tensor) -> Tuple[np.ndarray, np.ndarray]:
        boxes, scores = _f32(boxes), _f32(scores)
        assert tuple(boxes.shape) == (self.m, 8) and tuple(scores.shape) == (self.c, self.m)
        _ok(_lib().fdb_multiclass_nms_rotated(boxes.data_ptr(), scores.data_ptr(), self.c, self.m, self.score_threshold,
                                              self.nms_threshold, self.nms_top_k, self.keep_top_k, self.background, self.cap,
                                              self.ws.data_ptr(), self.ws.numel(), self.out.data_ptr(),
                                              self.out_index.data_ptr(), self.out_count.data_ptr(), self.overflow.data_ptr(),
                                              current_stream_ptr()), "multiclass_nms_rotated")
        n, seen = int(self.out_count.item()), int(self.overflow.item())
        if seen > self.cap:
            raise OverflowError(f"rotated NMS: {seen} candidates above the score threshold, buffers hold {self.cap}")
        return self.out[:n].cpu().numpy(), self.out_index[:n].cpu().numpy()


def centerpoint_decode_device(hm, reg, height, dim, vel, rot, voxel_size, pc_range, down_ratio, score_threshold,
                              nms_iou_threshold, post_center_range=None, nms_pre_max=1000, nms_post_max=83,
                              with_velocity=True):
    """Device version of one CenterPoint task head: tensors ``hm [C, H, W]`` etc. on the GPU -> (boxes, scores, labels) of
    the survivors of the bird's-eye-view NMS, best first."""
    hm, reg, height, dim, rot = (_f32(t) for t in (hm, reg, height, dim, rot))
    vel = _f32(vel) if with_velocity else None
    c, h, w = hm.shape
    hw = h * w
    dev = hm.device
    nb = 9 if with_velocity else 7
    k = min(nms_pre_max, hw)
    d = _CenterPointDesc()
    d.hm, d.reg, d.height, d.dim, d.rot = hm.data_ptr(), reg.data_ptr(), height.data_ptr(), dim.data_ptr(), rot.data_ptr()
    d.vel = vel.data_ptr() if vel is not None else None
    d.C, d.H, d.W, d.with_velocity = c, h, w, int(with_velocity)
    d.voxel_x, d.voxel_y, d.range_x, d.range_y = voxel_size[0], voxel_size[1], pc_range[0], pc_range[1]
    d.down_ratio, d.score_thresh, d.nms_thresh = down_ratio, score_threshold, nms_iou_threshold
    d.use_post_range = int(post_center_range is not None)
    for i, v in enumerate(post_center_range if post_center_range is not None else [0] * 6):
        d.post_range[i] = float(v)
    d.pre_max, d.post_max = nms_pre_max, nms_post_max
    ws = torch.empty(_lib().fdb_centerpoint_workspace(h, w, nms_pre_max), dtype=torch.uint8, device=dev)
    boxes = torch.empty(hw, nb, device=dev)
    scores = torch.empty(hw, device=dev)
    labels = torch.empty(hw, dtype=torch.int32, device=dev)
    order = torch.empty(k, dtype=torch.int32, device=dev)
    keep = torch.zeros(k, dtype=torch.uint8, device=dev)
    cnt = torch.zeros(1, dtype=torch.int32, device=dev)
    _ok(_lib().fdb_centerpoint_decode(ctypes.byref(d), ws.data_ptr(), ws.numel(), boxes.data_ptr(), scores.data_ptr(),
                                      labels.data_ptr(), order.data_ptr(), keep.data_ptr(), cnt.data_ptr(),
                                      current_stream_ptr()), "centerpoint_decode")
    sel = order[keep.bool()].long()
    return boxes[sel], scores[sel], labels[sel]


def grid_sample_3d(x: torch.Tensor, grid: torch.Tensor, mode: str = "bilinear", padding_mode: str = "zeros",
                   align_corners: bool = True) -> torch.Tensor:
    """``x [N, C, D, H, W]`` sampled at ``grid [N, Do, Ho, Wo, 3]`` (x, y, z in [-1, 1]) -> ``[N, C, Do, Ho, Wo]``."""
    x, grid = _f32(x), _f32(grid)
    n, c, d, h, w = x.shape
    _, do, ho, wo, three = grid.shape
    assert three == 3 and grid.shape[0] == n
    out = torch.empty(n, c, do, ho, wo, device=x.device)
    _ok(_lib().fdb_grid_sample_3d(x.data_ptr(), grid.data_ptr(), out.data_ptr(), n, c, d, h, w, do, ho, wo,
                                  {"bilinear": 0, "trilinear": 0, "nearest": 1}[mode],
                                  {"zeros": 0, "border": 1, "reflection": 2}[padding_mode], int(align_corners),
                                  current_stream_ptr()), "grid_sample_3d")
    return out


# ---------------------------------------------------------------------------------------------- host oracle
def _clip(subject: List[np.ndarray], clip: np.ndarray) -> List[np.ndarray]:
    area2 = float(np.dot(clip[:, 0], np.roll(clip[:, 1], -1)) - np.dot(clip[:, 1], np.roll(clip[:, 0], -1)))
    sign = 1.0 if area2 >= 0 else -1.0
    out = list(subject)
    for i in range(len(clip)):
        a, b = clip[i], clip[(i + 1) % len(clip)]
        inp, out = out, []
        if not inp:
            break

        def side(p):
            return sign * ((b[0] - a[0]) * (p[1] - a[1]) - (b[1] - a[1]) * (p[0] - a[0]))
        s = inp[-1]
        ds = side(s)
        for p in inp:
            dp = side(p)
            if dp >= 0:
                if ds < 0:
                    out.append(s + ds / (ds - dp) * (p - s))
                out.append(p)
            elif ds >= 0:
                out.append(s + ds / (ds - dp) * (p - s))
            s, ds = p, dp
    return out


def quad_iou_numpy(a: Sequence[float], b: Sequence[float]) -> float:
    pa, pb = np.asarray(a, np.float64).reshape(4, 2), np.asarray(b, np.float64).reshape(4, 2)

    def area(p):
        return 0.5 * abs(np.dot(p[:, 0], np.roll(p[:, 1], -1)) - np.dot(p[:, 1], np.roll(p[:, 0], -1)))
    poly = _clip(list(pa), pb)
    inter = area(np.asarray(poly)) if len(poly) >= 3 else 0.0
    union = area(pa) + area(pb) - inter
    return float(inter / union) if union > 1e-9 else 0.0


def multiclass_nms_rotated_numpy(boxes: np.ndarray, scores: np.ndarray, score_threshold: float, nms_threshold: float,
                                 nms_top_k: int, keep_top_k: int, background_label: int = -1) -> Tuple[np.ndarray, np.ndarray]:
    """Statement of the reference's rotated multiclass NMS for one image (multiclass_nms_rotated.cc:300-477): per class
    filter by score, sort, keep ``nms_top_k``, greedy suppression by polygon IoU; then the best ``keep_top_k`` overall,
    returned grouped by class (ascending) and by score within a class. Rows: label, score, 8 coordinates."""
    c, m = scores.shape
    per_class = []
    for k in range(c):
        if k == background_label:
            continue
        idx = np.nonzero(scores[k] > score_threshold)[0]
        idx = idx[np.argsort(-scores[k, idx], kind="stable")]
        if nms_top_k > 0:
            idx = idx[:nms_top_k]
        kept: List[int] = []
        for i in idx:
            if all(quad_iou_numpy(boxes[i], boxes[j]) <= nms_threshold for j in kept):
                kept.append(int(i))
        per_class.append((k, kept))
    flat = [(float(scores[k, i]), k, i) for k, kept in per_class for i in kept]
    if keep_top_k > 0 and len(flat) > keep_top_k:
        order = sorted(range(len(flat)), key=lambda t: (-flat[t][0], t))[:keep_top_k]
        chosen = set(order)
        flat = [f for t, f in enumerate(flat) if t in chosen]
    rows = np.asarray([[k, s] + list(boxes[i]) for s, k, i in flat], np.float32).reshape(-1, 10)
    return rows, np.asarray([i for _, _, i in flat], np.int32)
