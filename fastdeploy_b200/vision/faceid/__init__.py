"""Face recognition (fastdeploy/vision/faceid/contrib/insightface/, adaface/): ArcFace, CosFace,
PartialFC, VPL share the InsightFace recipe - resize to 112x112, BGR->RGB, (x - 127.5) / 128 (alpha
1/128, beta -127.5/128), CHW - and return the embedding, optionally L2-normalised; AdaFace differs only
in keeping BGR order."""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np

from ...core.types import ModelFormat
from ...runtime.model import FastDeployModel
from ...runtime.option import RuntimeOption
from .. import utils as vutils
from ..detection.contrib import _resize_bilinear
from ..result import FaceRecognitionResult


class InsightFaceRecognitionPreprocessor:
    def __init__(self):
        self.size = [112, 112]
        self.alpha = [1.0 / 128.0] * 3
        self.beta = [-127.5 / 128.0] * 3
        self.permute = True          # BGR -> RGB
        self.normalize_ = True
        self.chw_ = True

    def disable_normalize(self) -> None:
        """The graph applies ``alpha * x + beta`` itself: hand over the resized pixels as float
        (fastdeploy/vision/faceid/contrib/insightface/preprocessor.cc:60-75)."""
        self.normalize_ = False

    def disable_permute(self) -> None:
        """Leave the image HWC."""
        self.chw_ = False

    def run(self, images: Sequence[np.ndarray]) -> np.ndarray:
        out = []
        for im in images:
            x = im if im.shape[:2] == (self.size[1], self.size[0]) else _resize_bilinear(im, self.size[0], self.size[1])
            if self.permute:
                x = x[..., ::-1]
            x = x.astype(np.float32)
            if self.normalize_:
                x = x * np.asarray(self.alpha, np.float32) + np.asarray(self.beta, np.float32)
            out.append(np.ascontiguousarray(x.transpose(2, 0, 1) if self.chw_ else x))
        return np.stack(out)


class InsightFaceRecognitionPostprocessor:
    def __init__(self):
        self.l2_normalize = False

    def run(self, embeddings: np.ndarray) -> List[FaceRecognitionResult]:
        res = []
        for e in np.asarray(embeddings, np.float32).reshape(len(embeddings), -1):
            r = FaceRecognitionResult()
            r.embedding = vutils.l2_normalize(e.tolist()) if self.l2_normalize else e.tolist()
            res.append(r)
        return res


class InsightFaceRecognitionBase(FastDeployModel):
    def __init__(self, model_file: str, params_file: str = "", runtime_option: Optional[RuntimeOption] = None,
                 model_format: int = ModelFormat.ONNX):
        super().__init__(runtime_option)
        self.runtime_option.set_model_path(model_file, params_file, model_format)
        self.preprocessor = InsightFaceRecognitionPreprocessor()
        self.postprocessor = InsightFaceRecognitionPostprocessor()
        self._configure()
        self.init_runtime()

    def _configure(self):
        pass

    def predict(self, im: np.ndarray) -> FaceRecognitionResult:
        return self.batch_predict([im])[0]

    def batch_predict(self, images: Sequence[np.ndarray]) -> List[FaceRecognitionResult]:
        x = self.preprocessor.run(images)
        out = self.runtime.infer({self.runtime.get_input_info(0).name: x})[0]
        return self.postprocessor.run(np.asarray(out))


class ArcFace(InsightFaceRecognitionBase):
    pass


class CosFace(InsightFaceRecognitionBase):
    pass


class PartialFC(InsightFaceRecognitionBase):
    pass


class VPL(InsightFaceRecognitionBase):
    pass


class AdaFacePreprocessor(InsightFaceRecognitionPreprocessor):
    """AdaFace was trained on BGR crops: no channel swap (fastdeploy/vision/faceid/contrib/adaface/preprocessor.cc:25-70)."""

    def __init__(self):
        super().__init__()
        self.permute = False


class AdaFacePostprocessor(InsightFaceRecognitionPostprocessor):
    """The embedding, optionally L2-normalised (fastdeploy/vision/faceid/contrib/adaface/postprocessor.cc)."""


class AdaFace(InsightFaceRecognitionBase):
    def _configure(self):
        self.preprocessor = AdaFacePreprocessor()
        self.postprocessor = AdaFacePostprocessor()


def cosine_similarity(a, b, normalized: bool = True) -> float:
    return vutils.cosine_similarity(a, b, normalized)
