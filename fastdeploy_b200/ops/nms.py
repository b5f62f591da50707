"""Device multiclass NMS (csrc/kernels/nms.cu) with the semantics of the reference's CPU
implementation (fastdeploy/vision/detection/ppdet/multiclass_nms.cc:29-171)."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import _native
from .base import NativeOp, dtype_code


class _NmsDesc(ctypes.Structure):
    _fields_ = [
        ("boxes", ctypes.c_void_p), ("scores", ctypes.c_void_p), ("score_dtype", ctypes.c_int),
        ("s_n", ctypes.c_longlong), ("s_c", ctypes.c_longlong), ("s_m", ctypes.c_longlong),
        ("N", ctypes.c_int), ("M", ctypes.c_int), ("C", ctypes.c_int),
        ("score_threshold", ctypes.c_float), ("nms_threshold", ctypes.c_float),
        ("nms_top_k", ctypes.c_int), ("keep_top_k", ctypes.c_int), ("normalized", ctypes.c_int),
        ("background_label", ctypes.c_int),
        ("cls_count", ctypes.c_void_p), ("cls_score", ctypes.c_void_p), ("cls_index", ctypes.c_void_p),
        ("max_keep", ctypes.c_int),
        ("out", ctypes.c_void_p), ("out_index", ctypes.c_void_p), ("out_num", ctypes.c_void_p),
        ("out_cap", ctypes.c_int), ("scores_t", ctypes.c_void_p),
        ("lead", ctypes.c_void_p), ("tau", ctypes.c_void_p),
    ]


def _lib():
    lib = _native.kernels()
    if not getattr(lib, "_nms_ready", False):
        lib.fdb_nms_create.restype = ctypes.c_void_p
        lib.fdb_nms_create.argtypes = [ctypes.POINTER(_NmsDesc)]
        lib._nms_ready = True
    return lib


class MulticlassNMS:
    """Planned NMS over fixed ``boxes [N,M,4]`` fp32 and ``scores``.

    ``scores`` may be class-major ``[N,C,M]`` (the reference layout) or anchor-major
    ``[N,M,C]`` (what an NHWC head writes); pass ``class_major`` accordingly.
    Outputs: ``out [N,cap,6]`` rows ``(label, score, x1, y1, x2, y2)``, ``out_index [N,cap]``
    and ``out_num [N]``.
    """

    MAX_KEEP = 1024          # boxes one class can contribute (min(keep_top_k, nms_top_k) must not exceed it)

    def __init__(self, boxes: torch.Tensor, scores: torch.Tensor, *, class_major: bool, score_threshold: float,
                 nms_threshold: float, nms_top_k: int = 1000, keep_top_k: int = 100, normalized: bool = True,
                 background_label: int = -1, prepass: bool = True):
        n, m, four = boxes.shape
        assert four == 4 and boxes.dtype == torch.float32 and boxes.is_contiguous()
        if class_major:
            _, c, m2 = scores.shape
            s_n, s_c, s_m = scores.stride(0), scores.stride(1), scores.stride(2)
        else:
            _, m2, c = scores.shape
            s_n, s_c, s_m = scores.stride(0), scores.stride(2), scores.stride(1)
        assert m2 == m
        # any nms_top_k (the exporters' default is 10000): the class kernel takes candidates in passes of 1024
        k = m if nms_top_k < 0 else min(nms_top_k, m)
        max_keep = min(keep_top_k, k) if keep_top_k > 0 else k
        if max_keep > self.MAX_KEEP:
            raise ValueError(f"multiclass NMS on the device keeps at most {self.MAX_KEEP} boxes per class; set keep_top_k")
        cap = keep_top_k if keep_top_k > 0 else c * max_keep
        dev = boxes.device
        self.cls_count = torch.zeros(n, c, dtype=torch.int32, device=dev)
        self.cls_score = torch.empty(n, c, max_keep, dtype=torch.float32, device=dev)
        self.cls_index = torch.empty(n, c, max_keep, dtype=torch.int32, device=dev)
        self.out = torch.zeros(n, cap, 6, dtype=torch.float32, device=dev)
        self.out_index = torch.zeros(n, cap, dtype=torch.int32, device=dev)
        self.out_num = torch.zeros(n, dtype=torch.int32, device=dev)
        d = _NmsDesc()
        d.boxes, d.scores, d.score_dtype = boxes.data_ptr(), scores.data_ptr(), dtype_code(scores.dtype)
        d.s_n, d.s_c, d.s_m = s_n, s_c, s_m
        d.N, d.M, d.C = n, m, c
        d.score_threshold, d.nms_threshold = score_threshold, nms_threshold
        d.nms_top_k, d.keep_top_k, d.normalized, d.background_label = k, keep_top_k, int(normalized), background_label
        d.cls_count, d.cls_score, d.cls_index = self.cls_count.data_ptr(), self.cls_score.data_ptr(), self.cls_index.data_ptr()
        d.max_keep = max_keep
        d.out, d.out_index, d.out_num, d.out_cap = self.out.data_ptr(), self.out_index.data_ptr(), self.out_num.data_ptr(), cap
        # anchor-major scores are transposed once so that each class reads contiguous memory
        self.scores_t = None
        if not class_major and s_c == 1 and c > 1:
            self.scores_t = torch.empty(n, c, m, dtype=scores.dtype, device=dev)
            d.scores_t = self.scores_t.data_ptr()
        # score-floor pre-pass (exact): worthwhile when the classes together can supply keep_top_k leading boxes
        self.lead = self.tau = None
        lead_n = _lib().fdb_nms_lead_per_class()
        if prepass and keep_top_k > 0 and 2 * keep_top_k <= c * lead_n <= 4096:
            self.lead = torch.zeros(n, c, lead_n, dtype=torch.float32, device=dev)
            self.tau = torch.zeros(n, dtype=torch.float32, device=dev)
            d.lead, d.tau = self.lead.data_ptr(), self.tau.data_ptr()
        self.launches = 2 + (1 if self.scores_t is not None else 0) + (2 if self.tau is not None else 0)
        self.op = NativeOp(_lib().fdb_nms_create(ctypes.byref(d)), [boxes, scores, self], "multiclass_nms")
        self.op.keep = [boxes, scores]  # avoid a reference cycle through self
        self.op.create = ("fdb_nms_create", None, d)

    def launch(self, stream: Optional[int] = None) -> None:
        self.op.launch(stream)


def multiclass_nms_reference(boxes, scores, score_threshold, nms_threshold, nms_top_k, keep_top_k, normalized=True,
                             background_label=-1, nms_eta=1.0):
    """NumPy restatement of the reference algorithm for one batch.

    ``boxes [N,M,4]``, ``scores [N,C,M]``. Returns ``(out [K,6], index [K], num [N])``.
    """
    import numpy as np
    boxes = np.asarray(boxes, dtype=np.float32)
    scores = np.asarray(scores, dtype=np.float32)
    n, c, m = scores.shape
    norm = np.float32(0.0 if normalized else 1.0)

    def area(b):
        if b[2] < b[0] or b[3] < b[1]:
            return np.float32(0)
        w, h = b[2] - b[0], b[3] - b[1]
        return w * h if normalized else (w + np.float32(1)) * (h + np.float32(1))

    def iou(a, b):
        if b[0] > a[2] or b[2] < a[0] or b[1] > a[3] or b[3] < a[1]:
            return np.float32(0)
        iw = min(a[2], b[2]) - max(a[0], b[0]) + norm
        ih = min(a[3], b[3]) - max(a[1], b[1]) + norm
        inter = np.float32(iw * ih)
        return np.float32(inter / np.float32(np.float32(area(a) + area(b)) - inter))

    outs, idxs, nums = [], [], []
    for i in range(n):
        kept = {}
        for cls in range(c):
            if cls == background_label:
                continue
            sc = scores[i, cls]
            cand = np.nonzero(sc > score_threshold)[0]
            order = cand[np.argsort(-sc[cand], kind="stable")]
            if nms_top_k > -1:
                order = order[:nms_top_k]
            keep = []
            thr = nms_threshold
            for idx in order:
                ok = True
                for kidx in keep:
                    if iou(boxes[i, idx], boxes[i, kidx]) > thr:
                        ok = False
                        break
                if ok:
                    keep.append(int(idx))
                    if nms_eta < 1.0 and thr > 0.5:
                        thr *= nms_eta
            kept[cls] = keep
        pairs = [(scores[i, cls, idx], cls, idx) for cls in sorted(kept) for idx in kept[cls]]
        if keep_top_k > -1 and len(pairs) > keep_top_k:
            order = sorted(range(len(pairs)), key=lambda t: -pairs[t][0])  # Python's sort is stable
            pairs = [pairs[t] for t in order[:keep_top_k]]
            regroup = {}
            for s, cls, idx in pairs:
                regroup.setdefault(cls, []).append((s, cls, idx))
            pairs = [p for cls in sorted(regroup) for p in regroup[cls]]
        for s, cls, idx in pairs:
            outs.append([cls, s, *boxes[i, idx]])
            idxs.append(i * m + idx)
        nums.append(len(pairs))
    return (np.asarray(outs, dtype=np.float32).reshape(-1, 6), np.asarray(idxs, dtype=np.int64),
            np.asarray(nums, dtype=np.int32))
