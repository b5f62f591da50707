"""Style transfer (fastdeploy/vision/generation/contrib/animegan.cc:40-110): BGR->RGB, x / 127.5 - 1, NCHW
in; ``(y + 1) * 127.5`` clipped to uint8 and RGB->BGR out."""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np

from ...core.types import ModelFormat
from ...runtime.model import FastDeployModel
from ...runtime.option import RuntimeOption


class AnimeGAN(FastDeployModel):
    def __init__(self, model_file: str, params_file: str = "", runtime_option: Optional[RuntimeOption] = None,
                 model_format: int = ModelFormat.PADDLE):
        super().__init__(runtime_option)
        self.runtime_option.set_model_path(model_file, params_file, model_format)
        self.init_runtime()

    def batch_predict(self, images: Sequence[np.ndarray]) -> List[np.ndarray]:
        x = np.stack([np.ascontiguousarray((im[..., ::-1].astype(np.float32) / 127.5 - 1.0).transpose(2, 0, 1)) for im in images])
        info = self.runtime.get_input_info(0)
        if len(info.shape) == 4 and info.shape[-1] == 3:     # NHWC export
            x = np.ascontiguousarray(x.transpose(0, 2, 3, 1))
        out = np.asarray(self.runtime.infer({info.name: x})[0], np.float32)
        if out.shape[1] == 3:
            out = out.transpose(0, 2, 3, 1)
        return [np.clip(np.rint((o + 1.0) * 127.5), 0, 255).astype(np.uint8)[..., ::-1].copy() for o in out]

    def predict(self, im: np.ndarray) -> np.ndarray:
        return self.batch_predict([im])[0]
