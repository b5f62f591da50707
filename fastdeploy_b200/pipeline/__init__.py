"""``fastdeploy.pipeline``: multi-model pipelines (python/fastdeploy/pipeline/__init__.py):
PP-OCR v2/v3/v4 (re-exported from ``vision.ocr``) and the PP-TinyPose detector + key-point pipeline
(fastdeploy/pipeline/pptinypose/pipeline.cc:22-70: detect, drop boxes below ``detection_model_score_threshold``,
run the key-point model on each box)."""
from __future__ import annotations

from typing import Any

import numpy as np

from ..vision.ocr import PPOCRv2, PPOCRv3, PPOCRv4  # noqa: F401
from ..vision.result import DetectionResult, KeyPointDetectionResult


class PPTinyPose:
    def __init__(self, det_model: Any, pptinypose_model: Any):
        self.detector = det_model
        self.pose = pptinypose_model
        self.detection_model_score_threshold = 0.0

    def predict(self, input_image: np.ndarray) -> KeyPointDetectionResult:
        det = self.detector.predict(input_image)
        kept = DetectionResult()
        for b, s, l in zip(det.boxes, det.scores, det.label_ids):
            if s > self.detection_model_score_threshold:
                kept.boxes.append(b); kept.scores.append(s); kept.label_ids.append(l)
        if not kept.boxes:
            return KeyPointDetectionResult()
        return self.pose.predict(input_image, kept)


class _Namespace:
    def __init__(self, **kw):
        self.__dict__.update(kw)


pptinypose = _Namespace(PPTinyPose=PPTinyPose)
