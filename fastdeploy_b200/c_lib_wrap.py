"""``fastdeploy.C``: the names that user code reaches through the reference's compiled module
(python/fastdeploy/c_lib_wrap.py.in, fastdeploy/pybind/main.cc:160-210, fastdeploy/vision/vision_pybind.cc:20-60), e.g.
``fd.C.vision.FDMat()`` in a custom pre-processing chain or ``fd.C.vision.DetectionResult()`` to build a result by hand.
There is no separate compiled module here; the namespaces below point at the classes the package itself uses."""
from __future__ import annotations

import types as _types

from .core.types import Backend, Device, FDDataType, ModelFormat, TensorInfo     # noqa: F401
from .core.fd_tensor import FDTensor                                               # noqa: F401
from .runtime.option import RuntimeOption                                        # noqa: F401
from .runtime.runtime import Runtime                                             # noqa: F401


def _vision_namespace() -> _types.ModuleType:
    from . import vision as v
    from .vision import result as r, visualize as vz
    from .vision.common import processors as p
    ns = _types.ModuleType(__name__ + ".vision")
    for name in ("ClassifyResult", "DetectionResult", "FaceAlignmentResult", "FaceDetectionResult", "FaceRecognitionResult",
                 "HeadPoseResult", "KeyPointDetectionResult", "Mask", "MattingResult", "MOTResult", "OCRResult",
                 "PerceptionResult", "SegmentationResult"):
        setattr(ns, name, getattr(r, name))
    for name in dir(vz):
        if name.startswith(("vis_", "swap_background")):
            setattr(ns, name, getattr(vz, name))
    ns.FDMat, ns.FDMatBatch = p.FDMat, p.FDMatBatch
    ns.enable_flycv, ns.disable_flycv = v.enable_flycv, v.disable_flycv
    procs = _types.ModuleType(ns.__name__ + ".processors")
    for name in dir(p):
        obj = getattr(p, name)
        if isinstance(obj, type) and (issubclass(obj, p.Processor) or name == "ProcessorManager"):
            setattr(procs, name, obj)
    ns.processors = procs
    vis = _types.SimpleNamespace(**{k: getattr(ns, k) for k in dir(ns) if k.startswith(("vis_", "swap_background"))})
    ns.Visualize = vis
    return ns


def __getattr__(name: str):
    if name == "vision":
        ns = _vision_namespace()
        globals()["vision"] = ns
        return ns
    if name in ("is_built_with_gpu", "is_built_with_ort", "is_built_with_paddle", "is_built_with_trt", "is_built_with_openvino",
                "get_default_cuda_directory"):
        import fastdeploy_b200 as fd
        return getattr(fd, name)
    raise AttributeError(name)
