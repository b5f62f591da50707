"""Head pose (fastdeploy/vision/headpose/contrib/fsanet.cc:70-125): FSANet takes a 64x64 crop,
(x - 127.5) / 128 in BGR order, and returns (yaw, pitch, roll) in degrees."""
from __future__ import annotations

from typing import Optional

import numpy as np

from ...core.types import ModelFormat
from ...runtime.model import FastDeployModel
from ...runtime.option import RuntimeOption
from ..detection.contrib import _resize_bilinear
from ..result import HeadPoseResult


class FSANet(FastDeployModel):
    def __init__(self, model_file: str, params_file: str = "", runtime_option: Optional[RuntimeOption] = None,
                 model_format: int = ModelFormat.ONNX):
        super().__init__(runtime_option)
        self.runtime_option.set_model_path(model_file, params_file, model_format)
        self.size = [64, 64]
        self.init_runtime()

    def predict(self, im: np.ndarray) -> HeadPoseResult:
        x = (_resize_bilinear(im, *self.size).astype(np.float32) - 127.5) / 128.0
        out = self.runtime.infer({self.runtime.get_input_info(0).name: np.ascontiguousarray(x.transpose(2, 0, 1))[None]})[0]
        r = HeadPoseResult()
        r.euler_angles = np.asarray(out, np.float32).reshape(-1)[:3].tolist()
        return r
