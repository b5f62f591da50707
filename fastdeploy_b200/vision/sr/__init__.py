"""Video super-resolution (fastdeploy/vision/sr/ppsr/): PP-MSVSR, EDVR and BasicVSR take a stack of
frames ``[1, T, 3, H, W]`` (BGR->RGB, /255) and return up-scaled frames as uint8 BGR images
(ppmsvsr.cc:60-130; EDVR returns the centre frame only, edvr.cc:30-70)."""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np

from ...core.types import ModelFormat
from ...runtime.model import FastDeployModel
from ...runtime.option import RuntimeOption


class PPMSVSR(FastDeployModel):
    def __init__(self, model_file: str, params_file: str = "", runtime_option: Optional[RuntimeOption] = None,
                 model_format: int = ModelFormat.PADDLE):
        super().__init__(runtime_option)
        self.runtime_option.set_model_path(model_file, params_file, model_format)
        self.mean, self.scale = [0.0] * 3, [1.0] * 3
        self.init_runtime()

    def preprocess(self, frames: Sequence[np.ndarray]) -> np.ndarray:
        xs = [(f[..., ::-1].astype(np.float32) / 255.0 - np.asarray(self.mean, np.float32)) / np.asarray(self.scale, np.float32)
              for f in frames]
        return np.stack([np.ascontiguousarray(x.transpose(2, 0, 1)) for x in xs])[None]

    def postprocess(self, out: np.ndarray) -> List[np.ndarray]:
        out = np.asarray(out, np.float32)
        out = out.reshape((-1,) + out.shape[-3:])
        return [np.clip(np.rint(f.transpose(1, 2, 0)[..., ::-1] * 255.0), 0, 255).astype(np.uint8) for f in out]

    def predict(self, frames: Sequence[np.ndarray]) -> List[np.ndarray]:
        out = self.runtime.infer({self.runtime.get_input_info(0).name: self.preprocess(frames)})[0]
        return self.postprocess(out)


class BasicVSR(PPMSVSR):
    pass


class EDVR(PPMSVSR):
    def postprocess(self, out):
        out = np.asarray(out, np.float32)
        return super().postprocess(out.reshape((1,) + out.shape[-3:]))
