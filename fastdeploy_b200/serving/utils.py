"""``fastdeploy.serving.utils`` (python/fastdeploy/serving/utils.py:23-45): predictor lock and the image <-> base64 helpers."""
from .server import base64_to_cv2, cv2_to_base64, lock_predictor  # noqa: F401
