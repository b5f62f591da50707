"""Vision utilities (fastdeploy/vision/utils/utils.h:31-118): top-k, hard NMS, result sorting, L2 normalise,
cosine similarity, five-point face alignment, crop-by-box, result -> JSON."""
from __future__ import annotations

import json
from typing import Any, List, Sequence

import numpy as np

from .result import DetectionResult, FaceDetectionResult


def topk_indices(scores: np.ndarray, k: int) -> List[int]:
    """Repeated max scan like the reference (ties resolve to the lowest index)."""
    s = np.asarray(scores, dtype=np.float64).copy()
    k = min(k, s.size)
    out = []
    for _ in range(k):
        i = int(np.argmax(s))
        out.append(i)
        s[i] = -np.inf
    return out


TopKIndices = topk_indices


def _iou_one_to_many(b, boxes):
    x1, y1 = np.maximum(b[0], boxes[:, 0]), np.maximum(b[1], boxes[:, 1])
    x2, y2 = np.minimum(b[2], boxes[:, 2]), np.minimum(b[3], boxes[:, 3])
    inter = np.maximum(x2 - x1, 0) * np.maximum(y2 - y1, 0)
    a = (b[2] - b[0]) * (b[3] - b[1])
    areas = (boxes[:, 2] - boxes[:, 0]) * (boxes[:, 3] - boxes[:, 1])
    return inter / np.maximum(a + areas - inter, 1e-12)


def nms_indices(boxes: np.ndarray, scores: np.ndarray, iou_threshold: float = 0.5, max_keep: int = 0) -> np.ndarray:
    """Indices kept by greedy hard NMS over ``boxes [n, 4]`` (x1, y1, x2, y2), visited in descending, stable score
    order. Runs in the native host library (csrc/cpu/vision_utils.cc); the numpy loop below is the fallback when the
    library is not built and the oracle of its test."""
    boxes = np.ascontiguousarray(boxes, np.float32).reshape(-1, 4)
    scores = np.ascontiguousarray(scores, np.float32).reshape(-1)
    n = len(scores)
    if n == 0:
        return np.zeros(0, np.int64)
    from .. import _native
    if _native.cpu_available():
        import ctypes
        lib = _native.cpu()
        if not getattr(lib, "_fdv_ready", False):
            P = ctypes.c_void_p
            lib.fdv_hard_nms.restype = ctypes.c_longlong
            lib.fdv_hard_nms.argtypes = [P, P, ctypes.c_longlong, ctypes.c_float, ctypes.c_longlong, P]
            lib._fdv_ready = True
        keep = np.empty(n, np.int64)
        k = lib.fdv_hard_nms(boxes.ctypes.data, scores.ctypes.data, n, float(iou_threshold), int(max_keep), keep.ctypes.data)
        return keep[:k]
    return _nms_indices_numpy(boxes, scores, iou_threshold, max_keep)


def _nms_indices_numpy(boxes: np.ndarray, scores: np.ndarray, iou_threshold: float, max_keep: int = 0) -> np.ndarray:
    order = np.argsort(-scores, kind="stable")
    sorted_boxes = boxes[order]
    keep = []
    suppressed = np.zeros(len(order), bool)
    for i in range(len(order)):
        if suppressed[i]:
            continue
        keep.append(i)
        if max_keep > 0 and len(keep) >= max_keep:
            break
        if i + 1 < len(order):
            iou = _iou_one_to_many(sorted_boxes[i], sorted_boxes[i + 1:])
            suppressed[i + 1:] |= iou > iou_threshold
    return order[keep].astype(np.int64)


def nms(result, iou_threshold: float = 0.5) -> None:
    """In-place hard NMS on a DetectionResult / FaceDetectionResult sorted by score
    (fastdeploy/vision/utils/nms.cc:24-145)."""
    if not result.boxes:
        return
    idx = nms_indices(np.asarray(result.boxes, np.float32), np.asarray(result.scores, np.float32), iou_threshold)
    result.boxes = [result.boxes[i] for i in idx]
    result.scores = [result.scores[i] for i in idx]
    if isinstance(result, DetectionResult):
        result.label_ids = [result.label_ids[i] for i in idx]
    if isinstance(result, FaceDetectionResult) and result.landmarks_per_face > 0:
        k = result.landmarks_per_face
        result.landmarks = [result.landmarks[i * k + j] for i in idx for j in range(k)]


NMS = nms


def sort_detection_result(result: DetectionResult) -> None:
    order = np.argsort(-np.asarray(result.scores), kind="stable")
    result.boxes = [result.boxes[i] for i in order]
    result.scores = [result.scores[i] for i in order]
    result.label_ids = [result.label_ids[i] for i in order]


def l2_normalize(values: Sequence[float]) -> List[float]:
    v = np.asarray(values, np.float32)
    n = float(np.sqrt((v * v).sum()))
    return (v / max(n, 1e-12)).tolist()


L2Normalize = l2_normalize


def cosine_similarity(a: Sequence[float], b: Sequence[float], normalized: bool = True) -> float:
    a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
    if normalized:
        a, b = np.asarray(l2_normalize(a)), np.asarray(l2_normalize(b))
    return float((a * b).sum())


CosineSimilarity = cosine_similarity

ARCFACE_TEMPLATE = np.array([[38.2946, 51.6963], [73.5318, 51.5014], [56.0252, 71.7366], [41.5493, 92.3655],
                             [70.7299, 92.2041]], np.float32)


def align_face_with_five_points(image: np.ndarray, result: FaceDetectionResult, output_size=(112, 112)) -> List[np.ndarray]:
    """Similarity transform of each face to the 112x112 five-point template."""
    import cv2
    out = []
    if result.landmarks_per_face != 5:
        return out
    dst = ARCFACE_TEMPLATE * (np.asarray(output_size, np.float32) / 112.0)
    for i in range(len(result.boxes)):
        src = np.asarray(result.landmarks[i * 5:(i + 1) * 5], np.float32)
        m, _ = cv2.estimateAffinePartial2D(src, dst, method=cv2.LMEDS)
        out.append(cv2.warpAffine(image, m, tuple(output_size)))
    return out


def crop_image_by_box(image: np.ndarray, box: Sequence[float]) -> np.ndarray:
    h, w = image.shape[:2]
    x1, y1 = max(int(box[0]), 0), max(int(box[1]), 0)
    x2, y2 = min(int(box[2]), w), min(int(box[3]), h)
    return image[y1:y2, x1:x2].copy()


def fd_result_to_json(result: Any) -> str:
    """Result object -> JSON text in the layout of the per-type converters below (one key per field, each instance mask a
    JSON document of its own), plus a ``type`` key with the class name (python/fastdeploy/vision/utils.py:137-172). A list
    of results gives a JSON list."""
    if isinstance(result, (list, tuple)):
        return json.dumps([json.loads(fd_result_to_json(r)) for r in result])
    if not hasattr(result, "__dict__"):
        raise TypeError(f"not a result object: {type(result).__name__}")
    d = json.loads(_fields_to_json(result))
    d["type"] = type(result).__name__
    return json.dumps(d)


# ------------------------------------------------------------------ results <-> JSON, one pair of functions per result type
# (python/fastdeploy/vision/utils.py:20-330; the serving handlers use them to put results on the wire)
def _plain(o):
    if isinstance(o, (np.floating, np.integer)):
        return o.item()
    if isinstance(o, np.ndarray):
        return o.tolist()
    if isinstance(o, (list, tuple)):
        return [_plain(v) for v in o]
    return o


def _fields_to_json(result: Any) -> str:
    out = {}
    for k, v in result.__dict__.items():
        if k == "masks":
            out[k] = [mask_to_json(m) for m in v]          # each mask is a JSON document of its own, as in the reference
        else:
            out[k] = _plain(v)
    return json.dumps(out)


def _fields_from_json(cls_name: str, data: Any) -> Any:
    from . import result as R
    if isinstance(data, (str, bytes)):
        data = json.loads(data)
    obj = getattr(R, cls_name)()
    for k, v in data.items():
        if k == "type" or not hasattr(obj, k):
            continue
        if k == "masks":
            v = [json_to_mask(m) for m in v]
        setattr(obj, k, v)
    return obj


def mask_to_json(result: Any) -> str:
    return json.dumps({"data": _plain(result.data), "shape": _plain(result.shape)})


def json_to_mask(result: Any):
    return _fields_from_json("Mask", result)


def _pair(kind: str, cls_name: str):
    def to_json(result: Any) -> str:
        return _fields_to_json(result)

    def from_json(result: Any):
        return _fields_from_json(cls_name, result)
    to_json.__name__, from_json.__name__ = f"{kind}_to_json", f"json_to_{kind}"
    to_json.__doc__ = f"``{cls_name}`` -> JSON text with one key per field."
    from_json.__doc__ = f"JSON text or the parsed dictionary -> ``{cls_name}``."
    return to_json, from_json


detection_to_json, json_to_detection = _pair("detection", "DetectionResult")
perception_to_json, json_to_perception = _pair("perception", "PerceptionResult")
classify_to_json, json_to_classify = _pair("classify", "ClassifyResult")
keypoint_to_json, json_to_keypoint = _pair("keypoint", "KeyPointDetectionResult")
ocr_to_json, json_to_ocr = _pair("ocr", "OCRResult")
mot_to_json, json_to_mot = _pair("mot", "MOTResult")
face_detection_to_json, json_to_face_detection = _pair("face_detection", "FaceDetectionResult")
face_alignment_to_json, json_to_face_alignment = _pair("face_alignment", "FaceAlignmentResult")
face_recognition_to_json, json_to_face_recognition = _pair("face_recognition", "FaceRecognitionResult")
segmentation_to_json, json_to_segmentation = _pair("segmentation", "SegmentationResult")
matting_to_json, json_to_matting = _pair("matting", "MattingResult")
head_pose_to_json, json_to_head_pose = _pair("head_pose", "HeadPoseResult")
