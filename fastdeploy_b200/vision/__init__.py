"""``fastdeploy.vision``: model zoo, processors, results, visualisation."""
from . import (classification, common, detection, facealign, facedet, faceid, generation, headpose, keypointdetection,
               matting, ocr, perception, segmentation, sr, tracking, utils)
from .utils import fd_result_to_json
from .result import (ClassifyResult, DetectionResult, FaceAlignmentResult, FaceDetectionResult, FaceRecognitionResult,
                     HeadPoseResult, KeyPointDetectionResult, Mask, MattingResult, MOTResult, OCRResult,
                     PerceptionResult, SegmentationResult)
