"""``fastdeploy.vision.classification``: PaddleClas models (any PaddleClas export incl. ViT), torchvision-style
ResNet, YOLOv5Cls, PP-ShiTuV2 recogniser (fastdeploy/vision/classification/**)."""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence

import numpy as np
import yaml

from ...core.types import ModelFormat
from ...runtime.model import FastDeployModel
from ...runtime.option import RuntimeOption
from ..common.processors import (BGR2RGB, Cast, CenterCrop, HWC2CHW, Normalize, ProcessorManager, Resize,
                                 ResizeByShort, fuse_transforms)
from ..result import ClassifyResult
from ..utils import l2_normalize, topk_indices


class PaddleClasPreprocessor(ProcessorManager):
    """``inference_cls.yaml`` ``PreProcess.transform_ops``: ResizeImage{resize_short|size}, CropImage{size},
    NormalizeImage{mean,std,scale}, ToCHWImage (fastdeploy/vision/classification/ppcls/preprocessor.cc:40-95)."""

    def __init__(self, config_file: str):
        super().__init__()
        self.config_file = config_file
        self.disable_normalize_ = False
        self.disable_permute_ = False
        self.initial_resize_on_cpu_ = False
        self._build()

    def _build(self) -> None:
        with open(self.config_file) as f:
            cfg = yaml.safe_load(f)
        ops = cfg["PreProcess"]["transform_ops"]
        procs = [BGR2RGB()]
        for op in ops:
            (name, args), = op.items()
            args = args or {}
            if name == "ResizeImage":
                if "resize_short" in args:
                    procs.append(ResizeByShort(int(args["resize_short"]), 1, False))
                else:
                    size = args["size"]
                    size = [size, size] if isinstance(size, int) else size
                    procs.append(Resize(int(size[0]), int(size[1])))
            elif name == "CropImage":
                size = args["size"]
                size = [size, size] if isinstance(size, int) else size
                procs.append(CenterCrop(int(size[0]), int(size[1])))
            elif name == "NormalizeImage":
                if not self.disable_normalize_:
                    scale = float(args.get("scale", 0.00392157))
                    if abs(scale - 0.00392157) >= 1e-6:
                        raise ValueError("Only support scale in Normalize be 0.00392157, means the pixel is in range of [0, 255].")
                    procs.append(Normalize(list(args["mean"]), list(args["std"]), True))
            elif name == "ToCHWImage":
                if not self.disable_permute_:
                    procs.append(HWC2CHW())
            else:
                raise ValueError(f"Unexcepted preprocess operator: {name}.")
        self.processors = fuse_transforms(procs)

    def disable_normalize(self) -> None:
        """For a model whose graph normalises by itself: the chain is rebuilt without NormalizeImage, so it hands over
        uint8 pixels (fastdeploy/vision/classification/ppcls/preprocessor.cc:102-110)."""
        self.disable_normalize_ = True
        self._build()

    def disable_permute(self) -> None:
        """Leaves the image HWC (preprocessor.cc:111-119)."""
        self.disable_permute_ = True
        self._build()

    def initial_resize_on_cpu(self, v: bool) -> None:
        """The reference can run the first resize on the host so that a smaller image crosses to the GPU. The device path
        here reads the source image once inside the fused kernel, so the flag is recorded and changes nothing."""
        self.initial_resize_on_cpu_ = bool(v)

    def run(self, images):
        return super().run([np.asarray(im) for im in images])


class PaddleClasPostprocessor:
    """Top-k WITHOUT softmax (fastdeploy/vision/classification/ppcls/postprocessor.cc:27-49)."""

    def __init__(self, topk: int = 1):
        self.topk = topk

    def run(self, tensors: Sequence[np.ndarray]) -> List[ClassifyResult]:
        t = tensors[0]
        if hasattr(t, "is_cuda") and t.is_cuda and 1 <= self.topk <= 16:
            # logits are still on the device: reduce them there and copy back k numbers per image
            from ...ops.postproc import row_topk
            val, idx = row_topk(t.reshape(t.shape[0], -1).contiguous(), self.topk)
            val, idx = val.cpu().numpy(), idx.cpu().numpy()
            return [ClassifyResult(label_ids=[int(i) for i in idx[r]], scores=[float(v) for v in val[r]])
                    for r in range(idx.shape[0])]
        if hasattr(t, "detach"):
            t = t.detach().float().cpu().numpy()
        scores = np.asarray(t, np.float32)
        scores = scores.reshape(scores.shape[0], -1)
        out = []
        for row in scores:
            idx = topk_indices(row, self.topk)
            out.append(ClassifyResult(label_ids=idx, scores=[float(row[i]) for i in idx]))
        return out


class _ClsBase(FastDeployModel):
    def _finish_init(self):
        self.init_runtime()

    def predict(self, im: np.ndarray, topk: int = 1) -> ClassifyResult:
        self.postprocessor.topk = topk
        return self.batch_predict([im])[0]

    def batch_predict(self, images: Sequence[np.ndarray]) -> List[ClassifyResult]:
        if self.runtime.on_gpu:
            self.preprocessor.use_cuda(gpu_id=self.runtime_option.device_id)
        x = self.preprocessor.run(images)[0]
        name = self.runtime.graph.inputs[0].name
        outs = self.infer({name: x})
        first = self.runtime.graph.outputs[0].name
        return self.postprocessor.run([outs[first]])

    def get_preprocessor(self): return self.preprocessor
    def get_postprocessor(self): return self.postprocessor


class PaddleClasModel(_ClsBase):
    def __init__(self, model_file: str, params_file: str, config_file: str,
                 runtime_option: Optional[RuntimeOption] = None, model_format: ModelFormat = ModelFormat.PADDLE):
        super().__init__(runtime_option)
        self.runtime_option.set_model_path(model_file, params_file, model_format)
        self.preprocessor = PaddleClasPreprocessor(config_file)
        self.postprocessor = PaddleClasPostprocessor()
        self._finish_init()


class ResNet(_ClsBase):
    """torchvision-style ONNX ResNet: resize -> BGR2RGB -> ImageNet mean/std -> CHW, softmax then top-k
    (fastdeploy/vision/classification/contrib/resnet.cc)."""

    def __init__(self, model_file: str, params_file: str = "", runtime_option: Optional[RuntimeOption] = None,
                 model_format: ModelFormat = ModelFormat.ONNX):
        super().__init__(runtime_option)
        self.runtime_option.set_model_path(model_file, params_file, model_format)
        self.size = [224, 224]
        self.mean_vals = [0.485, 0.456, 0.406]
        self.std_vals = [0.229, 0.224, 0.225]
        self.preprocessor = ProcessorManager()
        self._rebuild()
        self.postprocessor = _SoftmaxTopK()
        self._finish_init()

    def _rebuild(self):
        self.preprocessor.processors = fuse_transforms([
            Resize(self.size[0], self.size[1]), BGR2RGB(), Normalize(self.mean_vals, self.std_vals), HWC2CHW()])


class _SoftmaxTopK(PaddleClasPostprocessor):
    def run(self, tensors):
        x = np.asarray(tensors[0], np.float32)
        x = x.reshape(x.shape[0], -1)
        e = np.exp(x - x.max(1, keepdims=True))
        return super().run([e / e.sum(1, keepdims=True)])


class YOLOv5ClsPreprocessor:
    """Centre crop to the short side, resize to ``size`` (h, w), BGR->RGB, 1/255, ImageNet mean / std, CHW; ``run`` returns
    the batch and, per image, the input and output shapes
    (fastdeploy/vision/classification/contrib/yolov5cls/preprocessor.cc:23-90)."""

    def __init__(self):
        self.size = [224, 224]
        self.mean, self.std = [0.485, 0.456, 0.406], [0.229, 0.224, 0.225]

    def run(self, images: Sequence[np.ndarray]):
        import cv2
        if len(images) == 0:
            raise ValueError("The size of input images should be greater than 0.")
        out, infos = [], []
        for im in images:
            h, w = im.shape[:2]
            c = min(h, w)
            y, x = (h - c) // 2, (w - c) // 2
            crop = cv2.resize(np.ascontiguousarray(im[y:y + c, x:x + c]), (self.size[1], self.size[0]), interpolation=cv2.INTER_LINEAR)
            t = (crop[..., ::-1].astype(np.float32) / 255.0 - np.float32(self.mean)) / np.float32(self.std)
            out.append(np.ascontiguousarray(t.transpose(2, 0, 1)))
            infos.append({"input_shape": [float(h), float(w)], "output_shape": [float(self.size[0]), float(self.size[1])]})
        return np.stack(out), infos


class YOLOv5ClsPostprocessor(_SoftmaxTopK):
    """Softmax over the classes, then the ``topk`` best (contrib/yolov5cls/postprocessor.cc:25-58)."""

    def run(self, tensors, ims_info=None):
        return super().run(tensors)


class YOLOv5Cls(_ClsBase):
    """YOLOv5 classification model (fastdeploy/vision/classification/contrib/yolov5cls/yolov5cls.cc)."""

    def __init__(self, model_file: str, params_file: str = "", runtime_option: Optional[RuntimeOption] = None,
                 model_format: ModelFormat = ModelFormat.ONNX):
        super().__init__(runtime_option)
        self.runtime_option.set_model_path(model_file, params_file, model_format)
        self.preprocessor = YOLOv5ClsPreprocessor()
        self.postprocessor = YOLOv5ClsPostprocessor()
        self._finish_init()

    @property
    def size(self):
        return self.preprocessor.size

    @size.setter
    def size(self, v):
        self.preprocessor.size = list(v)

    def batch_predict(self, images: Sequence[np.ndarray]) -> List[ClassifyResult]:
        x, infos = self.preprocessor.run(images)
        outs = self.runtime.infer({self.runtime.get_input_info(0).name: x})
        return self.postprocessor.run([outs[0]], infos)


class PPShiTuV2RecognizerPreprocessor(PaddleClasPreprocessor):
    """The recogniser reads the same ``inference_cls.yaml`` transform list as a PaddleClas classifier
    (fastdeploy/vision/classification/ppshitu/ppshituv2_rec_preprocessor.cc:25-120)."""


class PPShiTuV2RecognizerPostprocessor:
    """Copies each row of the embedding into ``ClassifyResult.feature`` and, with ``feature_norm`` (the default),
    divides it by its L2 norm (fastdeploy/vision/classification/ppshitu/ppshituv2_rec_postprocessor.cc:24-53)."""

    def __init__(self, topk: int = 1):
        self.topk = topk            # unused by a feature extractor; kept because the classifier interface sets it
        self.feature_norm = True

    def run(self, tensors) -> List[ClassifyResult]:
        t = tensors[0]
        if hasattr(t, "detach"):
            t = t.detach().float().cpu().numpy()
        feats = np.asarray(t, np.float32)
        feats = feats.reshape(feats.shape[0], -1)
        return [ClassifyResult(feature=l2_normalize(f) if self.feature_norm else f.tolist()) for f in feats]


class PPShiTuV2Recognizer(_ClsBase):
    """Feature extractor of PP-ShiTuV2: PaddleClas pre-processing, L2-normalised embedding in ``feature``
    (fastdeploy/vision/classification/ppshitu/ppshituv2_rec.cc:22-110)."""

    def __init__(self, model_file: str, params_file: str, config_file: str,
                 runtime_option: Optional[RuntimeOption] = None, model_format: ModelFormat = ModelFormat.PADDLE):
        super().__init__(runtime_option)
        self.runtime_option.set_model_path(model_file, params_file, model_format)
        self.preprocessor = PPShiTuV2RecognizerPreprocessor(config_file)
        self.postprocessor = PPShiTuV2RecognizerPostprocessor()
        self._finish_init()

    @property
    def feature_norm(self) -> bool:
        return self.postprocessor.feature_norm

    @feature_norm.setter
    def feature_norm(self, v: bool) -> None:
        self.postprocessor.feature_norm = bool(v)

    def predict(self, im: np.ndarray) -> ClassifyResult:
        return self.batch_predict([im])[0]


from ..detection.ppdet import PicoDet as PPShiTuV2Detector   # noqa: E402  (alias, as in the reference)
