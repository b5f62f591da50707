"""fastdeploy_b200: a Blackwell-native inference deployment runtime with the public surface of
FastDeploy 1.x (python/fastdeploy/__init__.py:118-155): ``Runtime``, ``RuntimeOption``,
``FastDeployModel``, ``vision``, ``text``, ``pipeline``, ``serving``, ``encryption``."""
from __future__ import annotations

__version__ = "0.1.0"

from .core.types import (Backend, Device, FDDataType, ModelFormat, TensorInfo, get_available_backends,
                         is_backend_available)
from .runtime.option import RuntimeOption
from .runtime.runtime import Runtime
from .runtime.model import FastDeployModel
from .utils.log import set_logger
from . import vision
from . import download as _download_module  # noqa: F401
from .download import download, download_and_decompress, download_model, get_model_list  # noqa: F401
from . import c_lib_wrap as C  # noqa: F401,N812


def is_built_with_gpu() -> bool:
    from . import _native
    return _native.kernels_available()


def is_built_with_ort() -> bool:
    return True     # ONNX models are served by the native backend / reference interpreter


def is_built_with_paddle() -> bool:
    return True     # Paddle inference models are imported natively


def is_built_with_trt() -> bool:
    return is_built_with_gpu()


def is_built_with_openvino() -> bool:
    return False


def get_default_cuda_directory() -> str:
    return "/usr/local/cuda"


def __getattr__(name):
    # heavier sub-packages load on first use
    import importlib
    if name in ("text", "pipeline", "serving", "encryption", "parallel", "streamer", "tools", "function", "utils"):
        return importlib.import_module("." + name, __name__)
    raise AttributeError(name)
