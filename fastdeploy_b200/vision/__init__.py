"""``fastdeploy.vision``: model zoo, processors, results, visualisation."""
from . import classification, common, detection, ocr, segmentation, utils
from .utils import fd_result_to_json
from .result import (ClassifyResult, DetectionResult, FaceAlignmentResult, FaceDetectionResult, FaceRecognitionResult,
                     HeadPoseResult, KeyPointDetectionResult, Mask, MattingResult, MOTResult, OCRResult,
                     PerceptionResult, SegmentationResult)
