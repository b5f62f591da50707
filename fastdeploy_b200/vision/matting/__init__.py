"""Matting (fastdeploy/vision/matting/): MODNet (contrib/modnet.cc: 256x256, (x - 127.5) / 127.5, alpha
resized back), PPMatting (ppmatting/ppmatting.cc:161-203: limit-by-short / pad-to-32 from the yaml, alpha
cropped and resized back) and RobustVideoMatting (contrib/rvm.cc: four recurrent states carried from
frame to frame, downsample ratio as an input)."""
from __future__ import annotations

from typing import List, Optional

import numpy as np
import yaml

from ...core.types import ModelFormat
from ...runtime.model import FastDeployModel
from ...runtime.option import RuntimeOption
from ..detection.contrib import _resize_bilinear
from ..result import MattingResult


def _resize_f32(a: np.ndarray, w: int, h: int) -> np.ndarray:
    return _resize_bilinear(np.clip(a * 255.0, 0, 255).astype(np.uint8), w, h).astype(np.float32) / 255.0


class _MatBase(FastDeployModel):
    def __init__(self, model_file: str, params_file: str = "", runtime_option: Optional[RuntimeOption] = None,
                 model_format: int = ModelFormat.ONNX):
        super().__init__(runtime_option)
        self.runtime_option.set_model_path(model_file, params_file, model_format)
        self._configure()
        self.init_runtime()

    def _configure(self):
        pass

    @staticmethod
    def _result(alpha: np.ndarray, fgr: Optional[np.ndarray] = None) -> MattingResult:
        r = MattingResult()
        r.shape = list(alpha.shape[:2])
        r.alpha = alpha.reshape(-1).tolist()
        if fgr is not None:
            r.contain_foreground = True
            r.foreground = fgr.reshape(-1).tolist()
        return r


class MODNet(_MatBase):
    def _configure(self):
        self.size = [256, 256]
        self.alpha = [1.0 / 127.5] * 3
        self.beta = [-1.0] * 3
        self.swap_rb = True

    def predict(self, im: np.ndarray) -> MattingResult:
        h, w = im.shape[:2]
        x = _resize_bilinear(im, *self.size)
        if self.swap_rb:
            x = x[..., ::-1]
        x = x.astype(np.float32) * np.asarray(self.alpha, np.float32) + np.asarray(self.beta, np.float32)
        out = self.runtime.infer({self.runtime.get_input_info(0).name: np.ascontiguousarray(x.transpose(2, 0, 1))[None]})[0]
        a = np.asarray(out, np.float32).reshape(out.shape[-2], out.shape[-1])
        return self._result(_resize_f32(a, w, h))


class PPMatting(_MatBase):
    def __init__(self, model_file: str, params_file: str, config_file: str, runtime_option=None,
                 model_format: int = ModelFormat.PADDLE):
        self.config_file = config_file
        super().__init__(model_file, params_file, runtime_option, model_format)

    def _configure(self):
        with open(self.config_file) as f:
            cfg = yaml.safe_load(f)
        self.limit_short, self.limit_long, self.fixed = -1, -1, None
        self.mean, self.std = [0.5] * 3, [0.5] * 3
        for op in cfg.get("Deploy", {}).get("transforms", []):
            t = op["type"]
            if t == "LimitShort":
                self.limit_short = op.get("max_short", -1)
            elif t == "ResizeToIntMult":
                self.mult = op.get("mult_int", 32)
            elif t == "ResizeByShort":
                self.limit_short = op["short_size"]
            elif t == "Resize":
                self.fixed = list(op["target_size"])
            elif t == "Normalize":
                self.mean, self.std = list(op.get("mean", self.mean)), list(op.get("std", self.std))
        self.mult = getattr(self, "mult", 32)

    def predict(self, im: np.ndarray) -> MattingResult:
        h, w = im.shape[:2]
        rw, rh = w, h
        if self.fixed is not None:
            rw, rh = self.fixed
        elif self.limit_short > 0 and min(h, w) > self.limit_short:
            s = self.limit_short / min(h, w)
            rw, rh = int(round(w * s)), int(round(h * s))
        x = _resize_bilinear(im, rw, rh) if (rw, rh) != (w, h) else im
        pw, ph = (rw + self.mult - 1) // self.mult * self.mult, (rh + self.mult - 1) // self.mult * self.mult
        x = x[..., ::-1].astype(np.float32) / 255.0
        x = (x - np.asarray(self.mean, np.float32)) / np.asarray(self.std, np.float32)
        canvas = np.zeros((ph, pw, 3), np.float32)
        canvas[:rh, :rw] = x
        out = self.runtime.infer({self.runtime.get_input_info(0).name: np.ascontiguousarray(canvas.transpose(2, 0, 1))[None]})[0]
        a = np.asarray(out, np.float32).reshape(out.shape[-2], out.shape[-1])[:rh, :rw]
        return self._result(_resize_f32(a, w, h))


class RobustVideoMatting(_MatBase):
    def _configure(self):
        self.size = [1920, 1080]
        self.downsample_ratio = 0.25
        self.video_mode = True
        self.swap_rb = True
        self.states: List[np.ndarray] = [np.zeros((1, 1, 1, 1), np.float32) for _ in range(4)]

    def reset(self):
        self.states = [np.zeros((1, 1, 1, 1), np.float32) for _ in range(4)]

    def predict(self, im: np.ndarray) -> MattingResult:
        h, w = im.shape[:2]
        x = _resize_bilinear(im, *self.size) if (w, h) != tuple(self.size) else im
        if self.swap_rb:
            x = x[..., ::-1]
        x = x.astype(np.float32) / 255.0
        names = [self.runtime.get_input_info(i).name for i in range(self.runtime.num_inputs())]
        feeds = {names[0]: np.ascontiguousarray(x.transpose(2, 0, 1))[None]}
        for k in range(4):
            feeds[names[1 + k]] = self.states[k]
        if len(names) > 5:
            feeds[names[5]] = np.asarray([self.downsample_ratio], np.float32)
        outs = [np.asarray(o, np.float32) for o in self.runtime.infer(feeds)]
        fgr, pha = outs[0][0], outs[1][0, 0]
        if self.video_mode:
            self.states = outs[2:6]
        a = _resize_f32(pha, w, h)
        f = _resize_bilinear(np.clip(fgr.transpose(1, 2, 0)[..., ::-1] * 255.0, 0, 255).astype(np.uint8), w, h)
        return self._result(a, f.astype(np.float32))
