"""Face alignment (fastdeploy/vision/facealign/contrib/): PFLD (106 points, output already in [0,1]),
FaceLandmark1000 (1000 points, 128x128 grey input), PIPNet (heat-map + local offsets + neighbour voting)."""
from __future__ import annotations

from typing import List, Optional

import numpy as np

from ...core.types import ModelFormat
from ...runtime.model import FastDeployModel
from ...runtime.option import RuntimeOption
from ..detection.contrib import _resize_bilinear
from ..result import FaceAlignmentResult


class _AlignBase(FastDeployModel):
    SIZE = (112, 112)

    def __init__(self, model_file: str, params_file: str = "", runtime_option: Optional[RuntimeOption] = None,
                 model_format: int = ModelFormat.ONNX):
        super().__init__(runtime_option)
        self.runtime_option.set_model_path(model_file, params_file, model_format)
        self.size = list(self.SIZE)
        self.init_runtime()

    def _run(self, x):
        return [np.asarray(o, np.float32) for o in self.runtime.infer({self.runtime.get_input_info(0).name: x})]


class PFLD(_AlignBase):
    """pfld.cc:70-130: resize 112x112, BGR->RGB, /255; output[1] holds 106 (x, y) pairs in [0,1]."""

    def predict(self, im: np.ndarray) -> FaceAlignmentResult:
        h, w = im.shape[:2]
        x = _resize_bilinear(im, *self.size)[..., ::-1].astype(np.float32) / 255.0
        outs = self._run(np.ascontiguousarray(x.transpose(2, 0, 1))[None])
        pts = outs[-1].reshape(-1, 2)
        r = FaceAlignmentResult()
        r.landmarks = (pts * np.asarray([w, h], np.float32)).tolist()
        return r


class FaceLandmark1000(_AlignBase):
    """face_landmark_1000.cc:70-125: grey 128x128 input, output 1000 (x, y) pairs scaled by the source size."""
    SIZE = (128, 128)

    def predict(self, im: np.ndarray) -> FaceAlignmentResult:
        h, w = im.shape[:2]
        g = _resize_bilinear(im, *self.size).astype(np.float32)
        g = (g[..., 0] * 0.114 + g[..., 1] * 0.587 + g[..., 2] * 0.299)[None, None]
        pts = self._run(np.ascontiguousarray(g))[0].reshape(-1, 2)
        r = FaceAlignmentResult()
        r.landmarks = (pts * np.asarray([w, h], np.float32)).tolist()
        return r


class PIPNet(_AlignBase):
    """pipnet.cc:330-630: outputs cls [1,N,8,8], x/y offsets and neighbour offsets; each landmark =
    arg-max cell + local offset, averaged with the votes of the landmarks that list it as a neighbour."""
    SIZE = (256, 256)

    def __init__(self, *a, num_landmarks: int = 19, num_nb: int = 10, **kw):
        self.num_landmarks, self.num_nb, self.net_stride = num_landmarks, num_nb, 32
        self.mean_vals, self.std_vals = [0.485, 0.456, 0.406], [0.229, 0.224, 0.225]
        self.reverse_index: Optional[np.ndarray] = None     # [N, max_len] indices into the flattened nb arrays
        super().__init__(*a, **kw)

    def set_num_landmarks(self, n: int):
        self.num_landmarks = n

    def predict(self, im: np.ndarray) -> FaceAlignmentResult:
        h, w = im.shape[:2]
        x = _resize_bilinear(im, *self.size)[..., ::-1].astype(np.float32) / 255.0
        x = (x - np.asarray(self.mean_vals, np.float32)) / np.asarray(self.std_vals, np.float32)
        cls, ox, oy, nbx, nby = self._run(np.ascontiguousarray(x.transpose(2, 0, 1))[None])[:5]
        n, fh, fw = cls.shape[1:]
        flat = cls.reshape(n, -1)
        idx = flat.argmax(1)
        gy, gx = idx // fw, idx % fw
        ar = np.arange(n)
        px = (gx + ox.reshape(n, -1)[ar, idx]) / fw
        py = (gy + oy.reshape(n, -1)[ar, idx]) / fh
        if nbx.size and self.num_nb > 0:
            nb_x = (gx[:, None] + nbx.reshape(n, self.num_nb, -1)[ar, :, idx]) / fw
            nb_y = (gy[:, None] + nby.reshape(n, self.num_nb, -1)[ar, :, idx]) / fh
            if self.reverse_index is not None:
                vx = nb_x.reshape(-1)[self.reverse_index]
                vy = nb_y.reshape(-1)[self.reverse_index]
                px = np.concatenate([px[:, None], vx], 1).mean(1)
                py = np.concatenate([py[:, None], vy], 1).mean(1)
        r = FaceAlignmentResult()
        r.landmarks = np.stack([px * w, py * h], 1).tolist()
        return r
