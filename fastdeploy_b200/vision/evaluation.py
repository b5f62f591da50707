"""Evaluation toolkit (python/fastdeploy/vision/evaluation/{classify,detection,segmentation}.py):
top-k accuracy, COCO-style box mAP (101-point interpolated AP over IoU 0.50:0.95, no pycocotools
dependency) and mIoU / pixel accuracy. Each ``eval_*`` takes a model object and an iterable of samples,
so it runs on synthetic data as well as on a dataset directory."""
from __future__ import annotations

import time
from typing import Any, Dict, Iterable, List, Sequence, Tuple

import numpy as np


def topk_accuracy(scores: np.ndarray, labels: Sequence[int], k: int = 1) -> float:
    order = np.argsort(-np.asarray(scores), axis=1, kind="stable")[:, :k]
    labels = np.asarray(labels).reshape(-1, 1)
    return float((order == labels).any(1).mean())


def eval_classify(model, samples: Iterable[Tuple[np.ndarray, int]], topk: int = 5) -> Dict[str, float]:
    hit1 = hitk = n = 0
    t0 = time.perf_counter()
    for im, label in samples:
        r = model.predict(im, topk) if "topk" in model.predict.__code__.co_varnames else model.predict(im)
        ids = list(r.label_ids)
        hit1 += int(ids[:1] == [label])
        hitk += int(label in ids[:topk])
        n += 1
    return {"topk1": hit1 / max(n, 1), f"topk{topk}": hitk / max(n, 1), "samples": n, "seconds": time.perf_counter() - t0}


def _iou(b, boxes):
    x1 = np.maximum(b[0], boxes[:, 0]); y1 = np.maximum(b[1], boxes[:, 1])
    x2 = np.minimum(b[2], boxes[:, 2]); y2 = np.minimum(b[3], boxes[:, 3])
    inter = np.maximum(x2 - x1, 0) * np.maximum(y2 - y1, 0)
    return inter / np.maximum((b[2] - b[0]) * (b[3] - b[1]) + (boxes[:, 2] - boxes[:, 0]) * (boxes[:, 3] - boxes[:, 1]) - inter, 1e-12)


def average_precision(dets: List[Tuple[int, float, Sequence[float]]], gts: Dict[int, np.ndarray], iou_thr: float) -> float:
    """``dets`` = (image id, score, box) of one class; ``gts[image id]`` = boxes ``[n, 4]`` of that class."""
    npos = sum(len(v) for v in gts.values())
    if npos == 0:
        return float("nan")
    used = {k: np.zeros(len(v), bool) for k, v in gts.items()}
    dets = sorted(dets, key=lambda d: -d[1])
    tp = np.zeros(len(dets)); fp = np.zeros(len(dets))
    for i, (img, _, box) in enumerate(dets):
        g = gts.get(img)
        if g is None or len(g) == 0:
            fp[i] = 1
            continue
        ious = _iou(np.asarray(box, float), g)
        ious[used[img]] = -1
        j = int(ious.argmax())
        if ious[j] >= iou_thr:
            tp[i] = 1
            used[img][j] = True
        else:
            fp[i] = 1
    ctp, cfp = np.cumsum(tp), np.cumsum(fp)
    rec = ctp / npos
    prec = ctp / np.maximum(ctp + cfp, 1e-12)
    for i in range(len(prec) - 2, -1, -1):
        prec[i] = max(prec[i], prec[i + 1])
    pts = np.linspace(0, 1, 101)
    idx = np.searchsorted(rec, pts, side="left")
    return float(np.mean([prec[i] if i < len(prec) else 0.0 for i in idx]))


def coco_map(predictions: List[Dict[str, Any]], ground_truth: List[Dict[str, Any]]) -> Dict[str, float]:
    """Both lists are per image: ``{"boxes": [n,4], "labels": [n], "scores": [n]}`` (scores only in predictions)."""
    classes = sorted({int(l) for g in ground_truth for l in g["labels"]})
    thrs = np.arange(0.5, 0.96, 0.05)
    per_thr = []
    for t in thrs:
        aps = []
        for c in classes:
            dets = [(i, float(s), b) for i, p in enumerate(predictions) for b, l, s in zip(p["boxes"], p["labels"], p["scores"]) if int(l) == c]
            gts = {i: np.asarray([b for b, l in zip(g["boxes"], g["labels"]) if int(l) == c], float).reshape(-1, 4)
                   for i, g in enumerate(ground_truth)}
            ap = average_precision(dets, gts, float(t))
            if ap == ap:
                aps.append(ap)
        per_thr.append(np.mean(aps) if aps else 0.0)
    return {"bbox_mAP": float(np.mean(per_thr)), "bbox_mAP50": float(per_thr[0]), "bbox_mAP75": float(per_thr[5])}


def eval_detection(model, samples: Iterable[Tuple[np.ndarray, Dict[str, Any]]]) -> Dict[str, float]:
    preds, gts = [], []
    for im, gt in samples:
        r = model.predict(im)
        preds.append({"boxes": r.boxes, "labels": r.label_ids, "scores": r.scores})
        gts.append(gt)
    return coco_map(preds, gts)


def segmentation_metrics(pred: np.ndarray, label: np.ndarray, num_classes: int, ignore_index: int = 255) -> Dict[str, float]:
    m = label != ignore_index
    p, l = pred[m].astype(np.int64), label[m].astype(np.int64)
    conf = np.bincount(l * num_classes + p, minlength=num_classes ** 2).reshape(num_classes, num_classes)
    inter = np.diag(conf).astype(float)
    union = conf.sum(0) + conf.sum(1) - inter
    present = union > 0
    return {"miou": float((inter[present] / union[present]).mean()) if present.any() else 0.0,
            "acc": float(inter.sum() / max(conf.sum(), 1))}


def eval_segmentation(model, samples: Iterable[Tuple[np.ndarray, np.ndarray]], num_classes: int) -> Dict[str, float]:
    conf = np.zeros((num_classes, num_classes), np.int64)
    for im, label in samples:
        r = model.predict(im)
        pred = np.asarray(r.label_map, np.int64).reshape(r.shape[:2])
        m = label != 255
        conf += np.bincount(label[m].astype(np.int64) * num_classes + pred[m], minlength=num_classes ** 2).reshape(num_classes, num_classes)
    inter = np.diag(conf).astype(float)
    union = conf.sum(0) + conf.sum(1) - inter
    present = union > 0
    return {"miou": float((inter[present] / union[present]).mean()) if present.any() else 0.0,
            "acc": float(inter.sum() / max(conf.sum(), 1))}


# ---------------------------------------------------------------------------- OCR (tests/acc_eval/ppocr in the reference)
def ocr_detection_hmean(predictions: List[Sequence[Sequence[float]]], ground_truth: List[Sequence[Sequence[float]]],
                        iou_thr: float = 0.5) -> Dict[str, float]:
    """ICDAR-style detection score. Both lists are per image lists of quadrilaterals (8 numbers, x0 y0 ... x3 y3).
    A prediction matches an unmatched ground-truth box when their polygon IoU is at least ``iou_thr`` (greedy, in
    prediction order, best IoU first); precision, recall and their harmonic mean are over the whole set."""
    from ..ops.perception import quad_iou_numpy
    matched = n_pred = n_gt = 0
    for preds, gts in zip(predictions, ground_truth):
        preds = [np.asarray(p, np.float64).reshape(4, 2) for p in preds]
        gts = [np.asarray(g, np.float64).reshape(4, 2) for g in gts]
        n_pred += len(preds)
        n_gt += len(gts)
        taken = set()
        for p in preds:
            best, best_j = 0.0, -1
            for j, g in enumerate(gts):
                if j in taken:
                    continue
                v = float(quad_iou_numpy(p, g))
                if v > best:
                    best, best_j = v, j
            if best_j >= 0 and best >= iou_thr:
                taken.add(best_j)
                matched += 1
    precision = matched / n_pred if n_pred else 0.0
    recall = matched / n_gt if n_gt else 0.0
    hmean = 2 * precision * recall / (precision + recall) if precision + recall > 0 else 0.0
    return {"precision": precision, "recall": recall, "hmean": hmean}


def edit_distance(a: str, b: str) -> int:
    """Levenshtein distance (insert, delete, substitute at cost one)."""
    if len(a) < len(b):
        a, b = b, a
    prev = list(range(len(b) + 1))
    for i, ca in enumerate(a, 1):
        cur = [i]
        for j, cb in enumerate(b, 1):
            cur.append(min(prev[j] + 1, cur[j - 1] + 1, prev[j - 1] + (ca != cb)))
        prev = cur
    return prev[-1]


def ocr_recognition_metrics(predictions: Sequence[str], ground_truth: Sequence[str], ignore_case: bool = False,
                            ignore_space: bool = True) -> Dict[str, float]:
    """Exact-match accuracy and 1 - normalised edit distance over text lines."""
    def norm(t: str) -> str:
        t = t.replace(" ", "") if ignore_space else t
        return t.lower() if ignore_case else t
    correct, ned = 0, 0.0
    for p, g in zip(predictions, ground_truth):
        p, g = norm(p), norm(g)
        correct += p == g
        ned += edit_distance(p, g) / max(len(p), len(g), 1)
    n = max(len(ground_truth), 1)
    return {"acc": correct / n, "norm_edit_dis": 1.0 - ned / n}


def eval_ocr(pipeline, samples: Iterable[Tuple[np.ndarray, Sequence[Sequence[float]], Sequence[str]]]) -> Dict[str, float]:
    """``samples`` yields (image, ground-truth quadrilaterals, their texts). Detection is scored over all boxes;
    recognition over the predicted boxes that matched a ground-truth box (IoU >= 0.5), text against text."""
    from ..ops.perception import quad_iou_numpy
    all_p, all_g, texts_p, texts_g = [], [], [], []
    for im, quads, texts in samples:
        r = pipeline.predict(im)
        all_p.append(r.boxes)
        all_g.append(list(quads))
        for box, text in zip(r.boxes, r.text):
            ious = [float(quad_iou_numpy(np.asarray(box, np.float64).reshape(4, 2), np.asarray(q, np.float64).reshape(4, 2)))
                    for q in quads]
            if ious and max(ious) >= 0.5:
                texts_p.append(text)
                texts_g.append(texts[int(np.argmax(ious))])
    out = ocr_detection_hmean(all_p, all_g)
    out.update({"rec_" + k: v for k, v in ocr_recognition_metrics(texts_p, texts_g).items()})
    return out


# ------------------------------------------------------------------ dataset readers and the streaming COCO metric
class CocoDetection:
    """A COCO-format detection set on disk (python/fastdeploy/vision/evaluation/utils/coco.py:35-180): ``data_dir`` holds
    the images, ``ann_file`` is the json with ``images``, ``annotations`` (``bbox`` as x, y, w, h) and ``categories``.
    ``file_list`` has one ``{"image", "im_id", "boxes" (x1, y1, x2, y2), "labels" (0-based, in category-id order),
    "is_crowd"}`` per image; iterating yields ``(BGR image, ground truth dict)`` as :func:`eval_detection` wants."""

    def __init__(self, data_dir: str, ann_file: str, num_workers: Any = "auto", shuffle: bool = False, allow_empty: bool = False,
                 empty_ratio: float = 1.0):
        import json
        import os
        self.data_dir, self.ann_file, self.shuffle, self.allow_empty, self.empty_ratio = data_dir, ann_file, shuffle, allow_empty, empty_ratio
        self.num_max_boxes = 1000
        with open(ann_file) as f:
            self.coco_gt = json.load(f)
        cats = sorted(self.coco_gt.get("categories", []), key=lambda c: c["id"])
        self.catid2clsid = {c["id"]: i for i, c in enumerate(cats)}
        self.clsid2catid = {i: c["id"] for i, c in enumerate(cats)}
        self.labels = [c.get("name", str(c["id"])) for c in cats]
        per_image: Dict[int, List[Dict[str, Any]]] = {}
        for a in self.coco_gt.get("annotations", []):
            per_image.setdefault(a["image_id"], []).append(a)
        self.file_list: List[Dict[str, Any]] = []
        for im in sorted(self.coco_gt.get("images", []), key=lambda r: r["id"]):
            anns = [a for a in per_image.get(im["id"], []) if a.get("bbox") and a["bbox"][2] > 0 and a["bbox"][3] > 0]
            if not anns and not allow_empty:
                continue
            self.file_list.append({
                "image": os.path.join(data_dir, im["file_name"]), "im_id": im["id"],
                "boxes": [[a["bbox"][0], a["bbox"][1], a["bbox"][0] + a["bbox"][2], a["bbox"][1] + a["bbox"][3]] for a in anns],
                "labels": [self.catid2clsid[a["category_id"]] for a in anns],
                "is_crowd": [int(a.get("iscrowd", 0)) for a in anns]})
        self.num_samples = len(self.file_list)

    def __len__(self) -> int:
        return self.num_samples

    def __iter__(self):
        import cv2
        for rec in self.file_list:
            yield cv2.imread(rec["image"]), {"boxes": rec["boxes"], "labels": rec["labels"]}


class COCOMetric:
    """Collects detections image by image and reports the box mAP over IoU 0.50:0.95
    (python/fastdeploy/vision/evaluation/utils/coco_metrics.py:25-120). ``update(im_id, outputs)`` takes a
    ``DetectionResult`` or ``{"boxes", "labels" | "label_ids", "scores"}``; ``get()`` returns ``{"bbox_mmap": ...}``."""

    def __init__(self, coco_gt: "CocoDetection", classwise: bool = False, **kwargs):
        self.dataset = coco_gt
        self.coco_gt = coco_gt.coco_gt
        self.clsid2catid = dict(coco_gt.clsid2catid)
        self.classwise = classwise
        self.reset()

    def reset(self) -> None:
        self.details: Dict[int, Dict[str, Any]] = {}
        self.eval_stats: Dict[str, float] = {}

    def update(self, im_id: int, outputs: Any) -> None:
        get = (lambda k, *alt: next((outputs[n] for n in (k,) + alt if n in outputs), [])) if isinstance(outputs, dict) else \
              (lambda k, *alt: next((getattr(outputs, n) for n in (k,) + alt if hasattr(outputs, n)), []))
        self.details[im_id] = {"boxes": [list(b)[:4] for b in get("boxes", "bbox")], "labels": [int(l) for l in get("labels", "label_ids")],
                               "scores": [float(s) for s in get("scores")]}

    def accumulate(self) -> Dict[str, float]:
        recs = [r for r in self.dataset.file_list if r["im_id"] in self.details]
        self.eval_stats = coco_map([self.details[r["im_id"]] for r in recs], [{"boxes": r["boxes"], "labels": r["labels"]} for r in recs]) \
            if recs else {"bbox_mAP": 0.0, "bbox_mAP50": 0.0, "bbox_mAP75": 0.0}
        return self.eval_stats

    def get(self) -> Dict[str, float]:
        if not self.eval_stats:
            self.accumulate()
        return {"bbox_mmap": self.eval_stats["bbox_mAP"], "bbox_map50": self.eval_stats["bbox_mAP50"]}


class Cityscapes:
    """The Cityscapes layout on disk (python/fastdeploy/vision/evaluation/utils/cityscapes.py:25-75):
    ``leftImg8bit/<mode>/<city>/*_leftImg8bit.png`` with labels ``gtFine/<mode>/<city>/*_gtFine_labelTrainIds.png``.
    ``file_list`` pairs them by sorted order; iterating yields ``(BGR image, label map)`` for :func:`eval_segmentation`."""
    NUM_CLASSES = 19

    def __init__(self, dataset_root: str, mode: str = "val"):
        import glob
        import os
        if mode not in ("train", "val", "test"):
            raise ValueError(f"mode should be 'train', 'val' or 'test', but got {mode}.")
        self.dataset_root, self.mode = dataset_root, mode
        self.num_classes, self.ignore_index = self.NUM_CLASSES, 255
        img_dir, label_dir = os.path.join(dataset_root, "leftImg8bit"), os.path.join(dataset_root, "gtFine")
        if not os.path.isdir(img_dir) or not os.path.isdir(label_dir):
            raise ValueError("The dataset is not Found or the folder structure is nonconfoumance.")
        labels = sorted(glob.glob(os.path.join(label_dir, mode, "*", "*_gtFine_labelTrainIds.png")))
        images = sorted(glob.glob(os.path.join(img_dir, mode, "*", "*_leftImg8bit.png")))
        self.file_list = [[i, l] for i, l in zip(images, labels)]

    def __len__(self) -> int:
        return len(self.file_list)

    def __iter__(self):
        import cv2
        for image, label in self.file_list:
            yield cv2.imread(image), cv2.imread(label, cv2.IMREAD_GRAYSCALE)
