"""Device post-processing and warps (csrc/kernels/postproc_ops.cu): row top-k / arg-max, greedy CTC
decode, batched perspective / affine warps and hard voxelisation. The reference does all of these on
the host (rec_postprocessor.cc:46-83, cls_postprocessor.cc, ppcls/postprocessor.cc,
get_rotate_crop_image.cc:21-81, Paddle3D's voxelize op); here the network output never leaves the GPU
before it has been reduced to the few numbers the caller wants.
"""
from __future__ import annotations

import ctypes
import math
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import _native
from .base import current_stream_ptr, dtype_code

_P = ctypes.c_void_p


def _lib():
    lib = _native.kernels()
    if not getattr(lib, "_postproc_ready", False):
        lib.fdb_row_topk.argtypes = [_P, ctypes.c_int, ctypes.c_longlong, ctypes.c_int, ctypes.c_longlong, ctypes.c_int,
                                     _P, _P, _P]
        lib.fdb_ctc_collapse.argtypes = [_P, _P, ctypes.c_int, ctypes.c_int, _P, _P, _P, _P]
        lib.fdb_warp_batch.argtypes = [_P, ctypes.c_int, ctypes.c_int, ctypes.c_int, _P, _P, _P, ctypes.c_int,
                                       ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, _P]
        lib.fdb_hard_voxelize_workspace.restype = ctypes.c_longlong
        lib.fdb_hard_voxelize_workspace.argtypes = [ctypes.c_int]
        lib.fdb_hard_voxelize.argtypes = [_P, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_float), ctypes.c_int,
                                          ctypes.c_int, _P, _P, _P, _P, _P, ctypes.c_longlong, _P]
        lib.fdb_db_postprocess_workspace.restype = ctypes.c_longlong
        lib.fdb_db_postprocess_workspace.argtypes = [ctypes.c_int] * 4
        lib.fdb_db_postprocess.argtypes = [_P, ctypes.c_int, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_longlong,
                                           ctypes.c_int, ctypes.c_int, ctypes.c_int, _P, ctypes.c_float, ctypes.c_float,
                                           ctypes.c_float, ctypes.c_int, ctypes.c_int, ctypes.c_int, _P, ctypes.c_longlong,
                                           _P, _P, _P, _P]
        lib.fdb_warp_normalize_batch.argtypes = [_P, ctypes.c_int, ctypes.c_int, _P, ctypes.c_longlong, _P, _P, _P, _P,
                                                 ctypes.c_int, ctypes.c_int,
                                                 ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_float),
                                                 ctypes.POINTER(ctypes.c_float), _P]
        lib.fdb_cls_flip.argtypes = [_P, ctypes.c_int, ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_float, _P, _P,
                                     _P, _P]
        lib._postproc_ready = True
    return lib


def _ok(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what}: {_native.last_error()}")


def row_topk(x: torch.Tensor, k: int = 1) -> Tuple[torch.Tensor, torch.Tensor]:
    """``x [..., C]`` (fp16 / bf16 / fp32, last dim contiguous) -> ``(values fp32 [..., k], indices int32 [..., k])``
    in descending order, ties to the lower index (``numpy.argmax`` order)."""
    assert x.is_cuda and x.stride(-1) == 1
    c = x.shape[-1]
    x2 = x.reshape(-1, c)
    rows = x2.shape[0]
    idx = torch.empty(rows, k, dtype=torch.int32, device=x.device)
    val = torch.empty(rows, k, dtype=torch.float32, device=x.device)
    _ok(_lib().fdb_row_topk(x2.data_ptr(), dtype_code(x.dtype), rows, c, x2.stride(0), k, idx.data_ptr(), val.data_ptr(),
                            current_stream_ptr()), "row_topk")
    shape = tuple(x.shape[:-1]) + (k,)
    return val.view(shape), idx.view(shape)


def ctc_greedy_decode_device(probs: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``probs [B, T, C]`` on the device -> ``(ids int32 [B, T] packed to the front and padded with -1,
    lengths int32 [B], scores fp32 [B])``: per-step arg-max, blanks (class 0) and repeats dropped, score = mean
    of the kept maxima. Only ``B * (2 T + 2)`` numbers remain to be copied to the host."""
    b, t, _ = probs.shape
    val, idx = row_topk(probs, 1)
    ids = torch.empty(b, t, dtype=torch.int32, device=probs.device)
    lens = torch.empty(b, dtype=torch.int32, device=probs.device)
    score = torch.empty(b, dtype=torch.float32, device=probs.device)
    _ok(_lib().fdb_ctc_collapse(idx.data_ptr(), val.data_ptr(), b, t, ids.data_ptr(), lens.data_ptr(), score.data_ptr(),
                                current_stream_ptr()), "ctc_collapse")
    return ids, lens, score


def ctc_texts(ids: torch.Tensor, lens: torch.Tensor, scores: torch.Tensor, labels: Sequence[str]):
    """Host tail of the CTC decode: the packed ids -> strings."""
    ids_h, lens_h, sc_h = ids.cpu().numpy(), lens.cpu().numpy(), scores.cpu().numpy()
    texts = ["".join(labels[k] if k < len(labels) else "" for k in ids_h[i, :lens_h[i]]) for i in range(len(lens_h))]
    return texts, [float(s) for s in sc_h]


def perspective_matrix(src: np.ndarray, dst: np.ndarray) -> np.ndarray:
    """3x3 homography that maps the four ``src`` points onto the four ``dst`` points (the linear system
    ``cv::getPerspectiveTransform`` solves), in float64."""
    a, b = np.zeros((8, 8)), np.zeros(8)
    for i in range(4):
        x, y, u, v = src[i, 0], src[i, 1], dst[i, 0], dst[i, 1]
        a[2 * i] = [x, y, 1, 0, 0, 0, -x * u, -y * u]
        a[2 * i + 1] = [0, 0, 0, x, y, 1, -x * v, -y * v]
        b[2 * i], b[2 * i + 1] = u, v
    h = np.linalg.solve(a, b)
    return np.append(h, 1.0).reshape(3, 3)


def warp_batch(image: torch.Tensor, inv_mats: np.ndarray, out_hw: Tuple[int, int],
               sizes: Optional[np.ndarray] = None, border: str = "replicate", fill: int = 0) -> torch.Tensor:
    """``image [H, W, C]`` uint8 on the device; ``inv_mats [N, 3, 3]`` map output pixels to source pixels
    (pass ``numpy.linalg.inv`` of a forward transform; append ``[0, 0, 1]`` to a 2x3 affine). Returns
    ``[N, OH, OW, C]`` uint8; ``sizes [N, 2]`` = (w, h) of each crop inside its canvas, the rest is ``fill``."""
    assert image.is_cuda and image.dtype == torch.uint8 and image.is_contiguous()
    h, w, c = image.shape
    n = len(inv_mats)
    oh, ow = out_hw
    out = torch.empty(n, oh, ow, c, dtype=torch.uint8, device=image.device)
    if n == 0:
        return out
    m = torch.from_numpy(np.ascontiguousarray(inv_mats, np.float32).reshape(n, 9)).to(image.device)
    sz = torch.from_numpy(np.ascontiguousarray(sizes, np.int32)).to(image.device) if sizes is not None else None
    _ok(_lib().fdb_warp_batch(image.data_ptr(), h, w, c, m.data_ptr(), sz.data_ptr() if sz is not None else None,
                              out.data_ptr(), n, oh, ow, 1 if border == "replicate" else 0, int(fill),
                              current_stream_ptr()), "warp_batch")
    return out


def rotate_crop_batch(image: torch.Tensor, boxes: Sequence[Sequence[int]]) -> Tuple[torch.Tensor, List[Tuple[int, int]]]:
    """All text crops of one page in one launch: each quad ``[x0, y0, ..., x3, y3]`` is rectified to
    ``(|p0 p1|, |p0 p3|)`` and turned by 90 degrees counter-clockwise when it is at least 1.5x taller than wide
    (get_rotate_crop_image.cc:21-81). Returns the canvas batch and each crop's ``(w, h)``."""
    mats, sizes = [], []
    for box in boxes:
        p = np.asarray(box, np.float64).reshape(4, 2)
        w = max(int(np.hypot(*(p[0] - p[1]))), 1)
        h = max(int(np.hypot(*(p[0] - p[3]))), 1)
        fwd = perspective_matrix(p, np.array([[0, 0], [w, 0], [w, h], [0, h]], np.float64))
        inv = np.linalg.inv(fwd)
        if h >= w * 1.5:
            # rotated output pixel (x', y') of the (h wide, w tall) image shows upright pixel (w - 1 - y', x')
            rot = np.array([[0, -1, w - 1], [1, 0, 0], [0, 0, 1]], np.float64)
            inv = inv @ rot
            w, h = h, w
        mats.append(inv)
        sizes.append((w, h))
    ow = max((s[0] for s in sizes), default=1)
    oh = max((s[1] for s in sizes), default=1)
    out = warp_batch(image, np.asarray(mats).reshape(-1, 3, 3), (oh, ow), np.asarray(sizes, np.int32).reshape(-1, 2))
    return out, sizes


class DBPostprocess:
    """Device DB post-processing for maps of one fixed size: owns the scratch and the result buffers, so a call is
    eight launches and no allocation. ``run`` leaves everything on the device; ``boxes`` reads the results back
    (one small copy) as per-image lists of ``[x0, y0, ..., x3, y3]``.

    Counterpart of ``DBPostProcessor::BoxesFromBitmap`` (ocr_postprocess_op.cc:238-318) on the host."""

    def __init__(self, n: int, h: int, w: int, device, *, thresh: float = 0.3, box_thresh: float = 0.6,
                 unclip_ratio: float = 1.5, score_mode: str = "slow", use_dilation: bool = False, max_candidates: int = 1000):
        self.n, self.h, self.w, self.max_candidates = n, h, w, max_candidates
        self.thresh, self.box_thresh, self.unclip_ratio = thresh, box_thresh, unclip_ratio
        self.score_fast, self.dilate = int(score_mode == "fast"), int(use_dilation)
        nbytes = _lib().fdb_db_postprocess_workspace(n, h, w, max_candidates)
        self.workspace = torch.empty(nbytes, dtype=torch.uint8, device=device)
        self.out_boxes = torch.zeros(n, max_candidates, 8, dtype=torch.int32, device=device)
        self.out_scores = torch.zeros(n, max_candidates, dtype=torch.float32, device=device)
        self.out_count = torch.zeros(n, dtype=torch.int32, device=device)
        self.info = torch.zeros(n, 4, dtype=torch.int32, device=device)
        self.launches = 9          # two clears + seven kernels

    def set_info(self, infos: Sequence[Sequence[int]]) -> None:
        """``infos[i] = (source width, source height, valid map width, valid map height)``."""
        self.info.copy_(torch.tensor([list(i) for i in infos], dtype=torch.int32).reshape(self.n, 4), non_blocking=True)

    def run(self, prob: torch.Tensor) -> None:
        """``prob``: ``[n, h, w]`` view (any strides) of fp32 / fp16 / bf16 probabilities on the device."""
        assert prob.is_cuda and tuple(prob.shape) == (self.n, self.h, self.w), tuple(prob.shape)
        _ok(_lib().fdb_db_postprocess(prob.data_ptr(), dtype_code(prob.dtype), prob.stride(2), prob.stride(1),
                                      prob.stride(0), self.n, self.h, self.w, self.info.data_ptr(), self.thresh,
                                      self.box_thresh, self.unclip_ratio, self.dilate, self.score_fast, self.max_candidates,
                                      self.workspace.data_ptr(), self.workspace.numel(), self.out_boxes.data_ptr(),
                                      self.out_scores.data_ptr(), self.out_count.data_ptr(), current_stream_ptr()),
            "db_postprocess")

    def boxes(self) -> Tuple[List[List[List[int]]], List[List[float]]]:
        counts = self.out_count.cpu().tolist()
        m = max(counts) if counts else 0
        if m == 0:
            return [[] for _ in counts], [[] for _ in counts]
        b = self.out_boxes[:, :m].cpu().numpy()
        s = self.out_scores[:, :m].cpu().numpy()
        return [b[i, :c].tolist() for i, c in enumerate(counts)], [s[i, :c].tolist() for i, c in enumerate(counts)]


def warp_normalize_batch(image: torch.Tensor, mats: torch.Tensor, valid_w: torch.Tensor, out: torch.Tensor,
                         alpha: Sequence[float], beta: Sequence[float], flip: Optional[torch.Tensor] = None,
                         page: Optional[torch.Tensor] = None) -> None:
    """``out[n] = normalise(warp_n(image))``: ``image`` uint8 ``[H, W, 3]`` or a stack ``[P, H, W, 3]`` with ``page``
    int32 ``[N]`` naming each crop's frame, ``mats`` fp32 ``[N, 9]`` (output pixel -> source pixel), ``valid_w`` int32
    ``[N]`` (columns at and beyond it are zero), ``out`` ``[N, OH, OW, CP]`` 16-bit or fp32, ``flip`` int32 ``[N]``
    (non-zero: the crop is turned by 180 degrees inside its valid width). All on the device."""
    assert image.is_cuda and image.dtype == torch.uint8 and image.is_contiguous() and image.shape[-1] == 3
    assert out.is_contiguous() and mats.dtype == torch.float32 and valid_w.dtype == torch.int32
    assert image.dim() == 3 or (image.dim() == 4 and page is not None and page.dtype == torch.int32)
    n, oh, ow, cp = out.shape
    assert mats.numel() >= 9 * n and valid_w.numel() >= n
    a = (ctypes.c_float * 3)(*[float(v) for v in alpha])
    b = (ctypes.c_float * 3)(*[float(v) for v in beta])
    _ok(_lib().fdb_warp_normalize_batch(image.data_ptr(), image.shape[-3], image.shape[-2],
                                        page.data_ptr() if page is not None else None,
                                        image.stride(0) if image.dim() == 4 else 0, mats.data_ptr(), valid_w.data_ptr(), flip.data_ptr() if flip is not None else None, out.data_ptr(),
                                        dtype_code(out.dtype), n, oh, ow, cp, a, b, current_stream_ptr()),
        "warp_normalize_batch")


def cls_flip(probs: torch.Tensor, thresh: float, flip: torch.Tensor, label: Optional[torch.Tensor] = None,
             score: Optional[torch.Tensor] = None) -> None:
    """``flip[i] = 1`` when row ``i`` of ``probs [n, classes]`` has an odd arg-max class with probability above
    ``thresh``; optionally also writes the arg-max ``label`` (int32) and its ``score`` (fp32)."""
    assert probs.dim() == 2 and probs.stride(1) == 1 and flip.dtype == torch.int32
    _ok(_lib().fdb_cls_flip(probs.data_ptr(), dtype_code(probs.dtype), probs.stride(0), probs.shape[0], probs.shape[1],
                            float(thresh), flip.data_ptr(), label.data_ptr() if label is not None else None,
                            score.data_ptr() if score is not None else None, current_stream_ptr()), "cls_flip")


def crop_matrices(boxes: Sequence[Sequence[int]], out_h: int, max_w: int) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """For each quad: the 3x3 map from a pixel of its ``out_h``-high network input to the source frame (perspective
    rectification to ``(|p0 p1|, |p0 p3|)``, a 90-degree turn for crops at least 1.5x taller than wide, and the resize
    to ``out_h`` rows, composed), the valid width ``min(max_w, ceil(out_h * w / h))`` and the aspect ratio ``w / h``."""
    n = len(boxes)
    if n == 0:
        return np.zeros((0, 9), np.float32), np.zeros(0, np.int32), np.zeros(0, np.float32)
    p = np.asarray(boxes, np.float64).reshape(n, 4, 2)
    w = np.maximum(np.hypot(*(p[:, 0] - p[:, 1]).T).astype(np.int64), 1).astype(np.float64)
    h = np.maximum(np.hypot(*(p[:, 0] - p[:, 3]).T).astype(np.int64), 1).astype(np.float64)
    # homography crop -> frame, solved directly from the four corner pairs (all boxes in one batched solve)
    zero = np.zeros(n)
    crop = np.stack([np.stack([zero, zero], 1), np.stack([w, zero], 1), np.stack([w, h], 1), np.stack([zero, h], 1)], 1)
    a = np.zeros((n, 8, 8))
    rhs = np.zeros((n, 8))
    for i in range(4):
        x, y, u, v = crop[:, i, 0], crop[:, i, 1], p[:, i, 0], p[:, i, 1]
        a[:, 2 * i, 0], a[:, 2 * i, 1], a[:, 2 * i, 2] = x, y, 1.0
        a[:, 2 * i, 6], a[:, 2 * i, 7] = -x * u, -y * u
        a[:, 2 * i + 1, 3], a[:, 2 * i + 1, 4], a[:, 2 * i + 1, 5] = x, y, 1.0
        a[:, 2 * i + 1, 6], a[:, 2 * i + 1, 7] = -x * v, -y * v
        rhs[:, 2 * i], rhs[:, 2 * i + 1] = u, v
    try:
        sol = np.linalg.solve(a, rhs[..., None])[..., 0]
    except np.linalg.LinAlgError:           # a degenerate quad somewhere: solve one by one, identity for the bad ones
        sol = np.zeros((n, 8))
        for k in range(n):
            try:
                sol[k] = np.linalg.solve(a[k], rhs[k])
            except np.linalg.LinAlgError:
                sol[k] = [1, 0, 0, 0, 1, 0, 0, 0]
    inv = np.concatenate([sol, np.ones((n, 1))], 1).reshape(n, 3, 3)
    tall = h >= w * 1.5
    if tall.any():
        # turned output pixel (x', y') of the (h wide, w tall) crop shows upright pixel (w - 1 - y', x')
        rot = np.zeros((n, 3, 3))
        rot[:, 0, 1], rot[:, 0, 2], rot[:, 1, 0], rot[:, 2, 2] = -1.0, w - 1, 1.0, 1.0
        inv = np.where(tall[:, None, None], inv @ rot, inv)
        w, h = np.where(tall, h, w), np.where(tall, w, h)
    vw = np.minimum(max_w, np.ceil(out_h * w / h)).astype(np.int64)
    sx, sy = w / np.maximum(vw, 1), h / out_h
    # centre-aligned resize: input pixel (x, y) shows crop position ((x + 0.5) * sx - 0.5, (y + 0.5) * sy - 0.5)
    rs = np.zeros((n, 3, 3))
    rs[:, 0, 0], rs[:, 0, 2], rs[:, 1, 1], rs[:, 1, 2], rs[:, 2, 2] = sx, 0.5 * sx - 0.5, sy, 0.5 * sy - 0.5, 1.0
    inv = inv @ rs
    scale = np.where(np.abs(inv[:, 2, 2]) > 1e-12, inv[:, 2, 2], 1.0)
    mats = (inv / scale[:, None, None]).reshape(n, 9).astype(np.float32)
    return mats, vw.astype(np.int32), (w / h).astype(np.float32)


def hard_voxelize_device(points: torch.Tensor, voxel_size: Sequence[float], pc_range: Sequence[float],
                         max_points: int, max_voxels: int):
    """``points [N, C]`` fp32 on the device -> ``(voxels [V, max_points, C], coords [V, 3] (z, y, x), num [V])``
    with voxels in order of first appearance, like the host version in ``vision.perception``."""
    assert points.is_cuda and points.dtype == torch.float32 and points.is_contiguous()
    n, c = points.shape
    vs, r = np.asarray(voxel_size, np.float32), np.asarray(pc_range, np.float32)
    grid = np.round((r[3:] - r[:3]) / vs)
    g9 = (ctypes.c_float * 9)(*vs.tolist(), *r[:3].tolist(), *grid.tolist())
    lib = _lib()
    ws = torch.empty(lib.fdb_hard_voxelize_workspace(n), dtype=torch.uint8, device=points.device)
    voxels = torch.empty(max_voxels, max_points, c, dtype=torch.float32, device=points.device)
    coords = torch.empty(max_voxels, 3, dtype=torch.int32, device=points.device)
    num = torch.empty(max_voxels, dtype=torch.int32, device=points.device)
    count = torch.empty(1, dtype=torch.int32, device=points.device)
    _ok(lib.fdb_hard_voxelize(points.data_ptr(), n, c, g9, max_points, max_voxels, voxels.data_ptr(), coords.data_ptr(),
                              num.data_ptr(), count.data_ptr(), ws.data_ptr(), ws.numel(), current_stream_ptr()),
        "hard_voxelize")
    v = int(count.item())
    return voxels[:v], coords[:v], num[:v]
