"""``fastdeploy.vision``: model zoo, processors, results, visualisation."""
from . import (classification, common, detection, facealign, facedet, faceid, generation, headpose, keypointdetection,
               matting, ocr, perception, segmentation, sr, tracking, utils)
from .utils import fd_result_to_json
from .result import (ClassifyResult, DetectionResult, FaceAlignmentResult, FaceDetectionResult, FaceRecognitionResult,
                     HeadPoseResult, KeyPointDetectionResult, Mask, MattingResult, MOTResult, OCRResult,
                     PerceptionResult, SegmentationResult)
from . import evaluation, visualize
from .visualize import (swap_background, swap_background_matting, swap_background_segmentation, vis_detection,
                        vis_face_alignment, vis_face_detection, vis_headpose, vis_keypoint_detection, vis_matting,
                        vis_matting_alpha, vis_mot, vis_perception, vis_ppocr, vis_segmentation)

_flycv = False


def enable_flycv() -> None:
    """Kept for source compatibility (python/fastdeploy/vision/__init__.py:36-41). The reference switches its host image
    library here; this package has one host path (OpenCV / numpy) and one device path, so the switch only records the
    wish."""
    global _flycv
    _flycv = True


def disable_flycv() -> None:
    global _flycv
    _flycv = False
