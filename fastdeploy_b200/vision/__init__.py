"""``fastdeploy.vision``: model zoo, processors, results, visualisation."""
from . import detection
from .result import (ClassifyResult, DetectionResult, FaceAlignmentResult, FaceDetectionResult, FaceRecognitionResult,
                     HeadPoseResult, KeyPointDetectionResult, Mask, MattingResult, MOTResult, OCRResult,
                     PerceptionResult, SegmentationResult)
