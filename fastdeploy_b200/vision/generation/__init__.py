"""Style transfer (fastdeploy/vision/generation/contrib/animegan.cc:40-110): BGR->RGB, x / 127.5 - 1, NCHW
in; ``(y + 1) * 127.5`` clipped to uint8 and RGB->BGR out."""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np

from ...core.types import ModelFormat
from ...runtime.model import FastDeployModel
from ...runtime.option import RuntimeOption


class AnimeGANPreprocessor:
    """BGR->RGB, ``x / 127.5 - 1``; NCHW by default, NHWC for exports that want it (contrib/preprocessor.cc:22-60)."""

    def __init__(self, config_file: str = ""):
        self.config_file = config_file          # the reference's signature has it; nothing is read from it
        self.nhwc = False

    def run(self, images: Sequence[np.ndarray]) -> np.ndarray:
        x = np.stack([im[..., ::-1].astype(np.float32) / 127.5 - 1.0 for im in images])
        return np.ascontiguousarray(x if self.nhwc else x.transpose(0, 3, 1, 2))


class AnimeGANPostprocessor:
    """``(y + 1) * 127.5`` rounded and clipped to uint8, RGB->BGR, one HWC image per batch item
    (contrib/postprocessor.cc:22-60)."""

    def run(self, outputs) -> List[np.ndarray]:
        out = np.asarray(outputs[0] if isinstance(outputs, (list, tuple)) else outputs, np.float32)
        if out.shape[1] == 3 and out.shape[-1] != 3:
            out = out.transpose(0, 2, 3, 1)
        return [np.clip(np.rint((o + 1.0) * 127.5), 0, 255).astype(np.uint8)[..., ::-1].copy() for o in out]


class AnimeGAN(FastDeployModel):
    def __init__(self, model_file: str, params_file: str = "", runtime_option: Optional[RuntimeOption] = None,
                 model_format: int = ModelFormat.PADDLE):
        super().__init__(runtime_option)
        self.runtime_option.set_model_path(model_file, params_file, model_format)
        self.preprocessor = AnimeGANPreprocessor()
        self.postprocessor = AnimeGANPostprocessor()
        self.init_runtime()
        info = self.runtime.get_input_info(0)
        self.preprocessor.nhwc = len(info.shape) == 4 and info.shape[-1] == 3

    def batch_predict(self, images: Sequence[np.ndarray]) -> List[np.ndarray]:
        x = self.preprocessor.run(images)
        return self.postprocessor.run(self.runtime.infer({self.runtime.get_input_info(0).name: x}))

    def predict(self, im: np.ndarray) -> np.ndarray:
        return self.batch_predict([im])[0]
