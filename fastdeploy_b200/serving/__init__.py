"""Serving: data-parallel scheduler with dynamic batching, SimpleServer-compatible HTTP front end,
Triton-style model repository loader."""
from .model_repository import ModelConfig, load_model_config, parse_pbtxt, scan_repository  # noqa: F401
from .scheduler import Scheduler, Worker  # noqa: F401
from .server import BaseModelHandler, ModelManager, VisionModelHandler, base64_to_cv2, cv2_to_base64  # noqa: F401


def __getattr__(name):
    if name == "SimpleServer":
        from . import server
        return server.SimpleServer
    if name in ("BaseRouterManager", "HttpRouterManager", "RequestBase", "ResponseBase"):     # these import fastapi
        from . import router
        return getattr(router, name)
    if name in ("router", "handler", "utils"):
        import importlib
        return importlib.import_module("." + name, __name__)
    raise AttributeError(name)
