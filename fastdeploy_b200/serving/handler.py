"""``fastdeploy.serving.handler``: the request handlers under the reference's module path
(python/fastdeploy/serving/handler/{base_handler,vision_model_handler}.py)."""
from .server import BaseModelHandler, VisionModelHandler  # noqa: F401
