"""Face detectors (fastdeploy/vision/facedet/): SCRFD, RetinaFace, YOLOv5Face, YOLOv7Face, UltraFace,
BlazeFace, CenterFace. Each class restates its reference decoder - anchor / stride grids, optional 5
landmarks - and finishes with the shared hard NMS on ``FaceDetectionResult``
(fastdeploy/vision/utils/nms.cc:87-145)."""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np

from ...core.types import ModelFormat
from ...runtime.model import FastDeployModel
from ...runtime.option import RuntimeOption
from .. import utils as vutils
from ..detection.contrib import _resize_bilinear, letterbox
from ..result import FaceDetectionResult


def _finish(boxes, scores, lms, k, nms_iou, info=None, clip_hw=None) -> FaceDetectionResult:
    r = FaceDetectionResult()
    r.landmarks_per_face = k
    if len(scores) == 0:
        return r
    boxes = np.asarray(boxes, np.float32).reshape(-1, 4).copy()
    lms = np.asarray(lms, np.float32).reshape(len(scores), k, 2).copy() if k else None
    if info is not None:
        boxes[:, [0, 2]] = (boxes[:, [0, 2]] - info["pad_w"]) / info["scale"]
        boxes[:, [1, 3]] = (boxes[:, [1, 3]] - info["pad_h"]) / info["scale"]
        if k:
            lms[..., 0] = (lms[..., 0] - info["pad_w"]) / info["scale"]
            lms[..., 1] = (lms[..., 1] - info["pad_h"]) / info["scale"]
        clip_hw = info["in_hw"]
    if clip_hw is not None:
        h, w = clip_hw
        boxes[:, [0, 2]] = np.clip(boxes[:, [0, 2]], 0, w - 1.0)
        boxes[:, [1, 3]] = np.clip(boxes[:, [1, 3]], 0, h - 1.0)
        if k:
            lms[..., 0] = np.clip(lms[..., 0], 0, w - 1.0)
            lms[..., 1] = np.clip(lms[..., 1], 0, h - 1.0)
    r.boxes = boxes.tolist()
    r.scores = [float(s) for s in scores]
    if k:
        r.landmarks = lms.reshape(-1, 2).tolist()
    vutils.nms(r, nms_iou)
    return r


def _defaults(obj, size) -> None:
    """Settings every face detector has; the letterbox ones carry the names of the reference's attributes
    (python/fastdeploy/vision/facedet/contrib/scrfd.py:60-190)."""
    obj.size = list(size)
    obj.conf_threshold = 0.25
    obj.nms_iou_threshold = 0.4
    obj.padding_value = [0.0, 0.0, 0.0]
    obj.is_mini_pad = False
    obj.is_no_pad = False
    obj.is_scale_up = True
    obj.stride = 32
    obj.max_nms = 30000
    obj.normalize = True
    obj.permute = True


class _FaceProcessor:
    """Pre- or post-processing half of a face detector as a separate object
    (fastdeploy/vision/facedet/contrib/yolov7face/{preprocessor,postprocessor}.h, facedet/ppdet/blazeface/,
    facedet/contrib/centerface/). Made on its own it holds its own settings; reached through ``model.preprocessor`` /
    ``model.postprocessor`` it reads and writes the model's."""
    MODEL = None
    ROLE = "pre"

    def __init__(self, _owner=None):
        if _owner is None:
            _owner = _Settings(self.MODEL)
        object.__setattr__(self, "_state", _owner)

    @classmethod
    def view(cls, model, role: str) -> "_FaceProcessor":
        named = _NAMED.get((type(model).__name__, role))
        if named is None:
            named = type(f"{type(model).__name__}{'Preprocessor' if role == 'pre' else 'Postprocessor'}", (_FaceProcessor,),
                         {"MODEL": type(model), "ROLE": role})
        return named(model)

    def __getattr__(self, name):
        return getattr(object.__getattribute__(self, "_state"), name)

    def __setattr__(self, name, value):
        if isinstance(getattr(type(self), name, None), property):
            object.__setattr__(self, name, value)
        else:
            setattr(object.__getattribute__(self, "_state"), name, value)

    @property
    def padding_color_value(self):
        return self._state.padding_value

    @padding_color_value.setter
    def padding_color_value(self, v):
        self._state.padding_value = list(v)

    @property
    def nms_threshold(self):
        return self._state.nms_iou_threshold

    @nms_threshold.setter
    def nms_threshold(self, v):
        self._state.nms_iou_threshold = v

    def run(self, first, infos=None):
        """Pre-processor: ``run(images) -> (batch [N, 3, H, W], infos)``. Post-processor: ``run(outputs, infos) ->
        [FaceDetectionResult]`` with ``outputs`` the batched runtime outputs."""
        st, model = self._state, self.MODEL
        if self.ROLE == "pre":
            pairs = [model.preprocess(st, im) for im in first]
            return np.concatenate([p[0] for p in pairs]), [p[1] for p in pairs]
        outs = [np.asarray(o, np.float32) for o in first]
        return [model.postprocess(st, [o[i:i + 1] for o in outs], info) for i, info in enumerate(infos)]


class _Settings:
    """The attributes a detector's pre/post-processing reads, without a runtime behind them."""

    def __init__(self, model_cls):
        _defaults(self, model_cls.SIZE)
        model_cls._configure(self)

    def _letterbox(self, im, pad_value=None):
        return _FaceDetBase._letterbox(self, im, pad_value)

    def _layout(self, x):
        return _FaceDetBase._layout(self, x)


_NAMED: Dict[Tuple[str, str], type] = {}


class _FaceDetBase(FastDeployModel):
    SIZE = (640, 640)

    def __init__(self, model_file: str, params_file: str = "", runtime_option: Optional[RuntimeOption] = None,
                 model_format: int = ModelFormat.ONNX):
        super().__init__(runtime_option)
        self.runtime_option.set_model_path(model_file, params_file, model_format)
        _defaults(self, self.SIZE)
        self._configure()
        self.init_runtime()

    @property
    def preprocessor(self):
        """The pre-processing half as an object of its own; its attributes are this model's."""
        return _FaceProcessor.view(self, "pre")

    @property
    def postprocessor(self):
        return _FaceProcessor.view(self, "post")

    @property
    def downsample_strides(self):
        return self.strides

    @downsample_strides.setter
    def downsample_strides(self, v):
        self.strides = list(v)

    def disable_normalize(self) -> None:
        """The graph normalises by itself: hand over RGB pixels as float, unscaled."""
        self.normalize = False

    def disable_permute(self) -> None:
        """Hand over HWC instead of CHW."""
        self.permute = False

    def _letterbox(self, im, pad_value=None):
        return letterbox(im, self.size, tuple(self.padding_value) if pad_value is None else pad_value, mini_pad=self.is_mini_pad,
                         no_pad=self.is_no_pad, scale_up=self.is_scale_up, stride=self.stride)

    def _layout(self, x: np.ndarray) -> np.ndarray:
        return np.ascontiguousarray(x.transpose(2, 0, 1) if self.permute else x)[None]

    def _configure(self):
        pass

    def _infer(self, x: np.ndarray) -> List[np.ndarray]:
        return [np.asarray(o, np.float32) for o in self.runtime.infer({self.runtime.get_input_info(0).name: x})]

    def predict(self, im: np.ndarray, conf_threshold: Optional[float] = None, nms_iou_threshold: Optional[float] = None):
        if conf_threshold is not None:
            self.conf_threshold = conf_threshold
        if nms_iou_threshold is not None:
            self.nms_iou_threshold = nms_iou_threshold
        x, info = self.preprocess(im)
        return self.postprocess(self._infer(x), info)

    def batch_predict(self, images: Sequence[np.ndarray]):
        return [self.predict(im) for im in images]


class SCRFD(_FaceDetBase):
    """SCRFD (facedet/contrib/scrfd.cc:178-330): strides 8/16/32, 2 anchors per cell, outputs per
    stride: score [n,1], bbox distances [n,4] (x stride), optional kps [n,10] (x stride)."""

    def _configure(self):
        self.strides = [8, 16, 32]
        self.num_anchors = 2
        self.use_kps = True
        self.landmarks_per_face = 5
        self.mean, self.scale = 127.5, 1.0 / 128.0

    def preprocess(self, im):
        canvas, info = self._letterbox(im)
        x = canvas[..., ::-1].astype(np.float32)
        if self.normalize:
            x = (x - self.mean) * self.scale
        return self._layout(x), info

    def postprocess(self, outs, info):
        n_s = len(self.strides)
        boxes, scores, lms = [], [], []
        h, w = info["out_hw"]
        for i, s in enumerate(self.strides):
            sc = outs[i].reshape(-1)
            bb = outs[i + n_s].reshape(-1, 4) * s
            fh, fw = h // s, w // s
            gy, gx = np.meshgrid(np.arange(fh), np.arange(fw), indexing="ij")
            c = np.stack([gx.ravel(), gy.ravel()], 1).astype(np.float32) * s
            c = np.repeat(c, self.num_anchors, axis=0)
            m = sc > self.conf_threshold
            if not m.any():
                continue
            cm, bm = c[m], bb[m]
            boxes.append(np.stack([cm[:, 0] - bm[:, 0], cm[:, 1] - bm[:, 1], cm[:, 0] + bm[:, 2], cm[:, 1] + bm[:, 3]], 1))
            scores.append(sc[m])
            if self.use_kps and len(outs) >= 3 * n_s:
                kp = outs[i + 2 * n_s].reshape(-1, 5, 2)[m] * s
                lms.append(kp + cm[:, None, :])
        if not scores:
            return _finish([], [], [], 0, self.nms_iou_threshold)
        k = 5 if lms else 0
        return _finish(np.concatenate(boxes), np.concatenate(scores), np.concatenate(lms) if lms else [], k,
                       self.nms_iou_threshold, info)


class RetinaFace(_FaceDetBase):
    """RetinaFace (facedet/contrib/retinaface.cc:100-270): prior boxes with min sizes {16,32},{64,128},
    {256,512} on strides 8/16/32, variances (0.1, 0.2), outputs loc [n,4], conf [n,2], landms [n,10]."""

    def _configure(self):
        self.variance = [0.1, 0.2]
        self.strides = [8, 16, 32]
        self.min_sizes = [[16, 32], [64, 128], [256, 512]]
        self.landmarks_per_face = 5

    def priors(self, h, w):
        out = []
        for s, sizes in zip(self.strides, self.min_sizes):
            fh, fw = math.ceil(h / s), math.ceil(w / s)
            for i in range(fh):
                for j in range(fw):
                    for ms in sizes:
                        out.append([(j + 0.5) * s / w, (i + 0.5) * s / h, ms / w, ms / h])
        return np.asarray(out, np.float32)

    def preprocess(self, im):
        h, w = im.shape[:2]
        x = _resize_bilinear(im, self.size[0], self.size[1]).astype(np.float32) - np.asarray([104.0, 117.0, 123.0], np.float32)
        info = {"scale_w": self.size[0] / w, "scale_h": self.size[1] / h, "in_hw": (h, w)}
        return np.ascontiguousarray(x.transpose(2, 0, 1))[None], info

    def postprocess(self, outs, info):
        loc, conf, landm = outs[0].reshape(-1, 4), outs[1].reshape(-1, 2), outs[2].reshape(-1, 10)
        H, W = self.size[1], self.size[0]
        pr = self.priors(H, W)
        sc = conf[:, 1]
        m = sc > self.conf_threshold
        pr, loc, landm, sc = pr[m], loc[m], landm[m], sc[m]
        cx = pr[:, 0] + loc[:, 0] * self.variance[0] * pr[:, 2]
        cy = pr[:, 1] + loc[:, 1] * self.variance[0] * pr[:, 3]
        bw = pr[:, 2] * np.exp(loc[:, 2] * self.variance[1])
        bh = pr[:, 3] * np.exp(loc[:, 3] * self.variance[1])
        boxes = np.stack([(cx - bw / 2) * W, (cy - bh / 2) * H, (cx + bw / 2) * W, (cy + bh / 2) * H], 1)
        lm = landm.reshape(-1, 5, 2) * self.variance[0] * pr[:, None, 2:4] + pr[:, None, 0:2]
        lm = lm * np.asarray([W, H], np.float32)
        boxes[:, [0, 2]] /= info["scale_w"]
        boxes[:, [1, 3]] /= info["scale_h"]
        lm[..., 0] /= info["scale_w"]
        lm[..., 1] /= info["scale_h"]
        return _finish(boxes, sc, lm, 5, self.nms_iou_threshold, None, info["in_hw"])


class YOLOv5Face(_FaceDetBase):
    """YOLOv5-Face (facedet/contrib/yolov5face.cc:150-260): rows ``[cx, cy, w, h, obj, 5 x (lx, ly), cls]``."""

    def _configure(self):
        self.landmarks_per_face = 5
        self.padding_value = [114.0, 114.0, 114.0]

    def preprocess(self, im):
        canvas, info = self._letterbox(im)
        x = canvas[..., ::-1].astype(np.float32)
        if self.normalize:
            x = x / 255.0
        return self._layout(x), info

    def postprocess(self, outs, info):
        rows = outs[0].reshape(-1, outs[0].shape[-1])
        conf = rows[:, 4] * rows[:, 15]
        m = conf > self.conf_threshold
        rows, conf = rows[m], conf[m]
        boxes = np.stack([rows[:, 0] - rows[:, 2] / 2, rows[:, 1] - rows[:, 3] / 2, rows[:, 0] + rows[:, 2] / 2,
                          rows[:, 1] + rows[:, 3] / 2], 1)
        return _finish(boxes, conf, rows[:, 5:15].reshape(-1, 5, 2), 5, self.nms_iou_threshold, info)


class YOLOv7Face(YOLOv5Face):
    """YOLOv7-Face (facedet/contrib/yolov7face/): rows ``[cx, cy, w, h, obj, cls, 5 x (lx, ly, conf)]``."""

    def postprocess(self, outs, info):
        rows = outs[0].reshape(-1, outs[0].shape[-1])
        conf = rows[:, 4] * rows[:, 5]
        m = conf > self.conf_threshold
        rows, conf = rows[m], conf[m]
        boxes = np.stack([rows[:, 0] - rows[:, 2] / 2, rows[:, 1] - rows[:, 3] / 2, rows[:, 0] + rows[:, 2] / 2,
                          rows[:, 1] + rows[:, 3] / 2], 1)
        lm = rows[:, 6:21].reshape(-1, 5, 3)[..., :2]
        return _finish(boxes, conf, lm, 5, self.nms_iou_threshold, info)


class UltraFace(_FaceDetBase):
    """UltraFace (facedet/contrib/ultraface.cc:120-200): outputs scores [n,2] and boxes [n,4] already
    decoded and normalised to [0,1]; input 320x240, (x - 127) / 128."""
    SIZE = (320, 240)

    def _configure(self):
        self.conf_threshold = 0.7
        self.nms_iou_threshold = 0.3

    def preprocess(self, im):
        h, w = im.shape[:2]
        x = (_resize_bilinear(im, self.size[0], self.size[1])[..., ::-1].astype(np.float32) - 127.0) / 128.0
        return np.ascontiguousarray(x.transpose(2, 0, 1))[None], {"in_hw": (h, w)}

    def postprocess(self, outs, info):
        sc, bb = outs[0].reshape(-1, 2)[:, 1], outs[1].reshape(-1, 4)
        m = sc > self.conf_threshold
        h, w = info["in_hw"]
        boxes = bb[m] * np.asarray([w, h, w, h], np.float32)
        return _finish(boxes, sc[m], [], 0, self.nms_iou_threshold, None, (h, w))


class BlazeFace(_FaceDetBase):
    """BlazeFace exported by PaddleDetection (facedet/ppdet/blazeface/): the graph ends in NMS-ready
    rows ``[label, score, x1, y1, x2, y2]`` and a per-image count; only the score filter remains."""
    SIZE = (640, 640)

    def __init__(self, model_file: str, params_file: str = "", config_file: str = "", runtime_option: Optional[RuntimeOption] = None,
                 model_format: int = ModelFormat.PADDLE):
        """``config_file`` is the PaddleDetection ``infer_cfg.yml`` of the export; a ``Resize.target_size`` in it sets the
        input size (facedet/ppdet/blazeface/preprocessor.cc:30-70)."""
        if isinstance(config_file, RuntimeOption):              # older call order: (model, params, option, format)
            config_file, runtime_option = "", config_file
        self.config_file = config_file
        super().__init__(model_file, params_file, runtime_option, model_format)

    def _configure(self):
        self.conf_threshold = 0.5
        cfg_path = getattr(self, "config_file", "")
        if cfg_path:
            import yaml
            with open(cfg_path) as f:
                cfg = yaml.safe_load(f) or {}
            for op in cfg.get("Preprocess", []) or []:
                if op.get("type") == "Resize" and op.get("target_size"):
                    hh, ww = op["target_size"]
                    self.size = [int(ww), int(hh)]

    def preprocess(self, im):
        h, w = im.shape[:2]
        x = _resize_bilinear(im, self.size[0], self.size[1]).astype(np.float32)
        x = (x[..., ::-1] / 255.0 - np.asarray([0.485, 0.456, 0.406], np.float32)) / np.asarray([0.229, 0.224, 0.225], np.float32)
        return np.ascontiguousarray(x.transpose(2, 0, 1))[None], {"in_hw": (h, w), "sx": w / self.size[0], "sy": h / self.size[1]}

    def predict(self, im, conf_threshold=None, nms_iou_threshold=None):
        if conf_threshold is not None:
            self.conf_threshold = conf_threshold
        x, info = self.preprocess(im)
        feeds = {}
        for i in range(self.runtime.num_inputs()):
            name = self.runtime.get_input_info(i).name
            if name == "image" or i == 0 and self.runtime.num_inputs() == 1:
                feeds[name] = x
            elif name == "scale_factor":
                feeds[name] = np.asarray([[1.0 / info["sy"], 1.0 / info["sx"]]], np.float32)
            elif name == "im_shape":
                feeds[name] = np.asarray([[self.size[1], self.size[0]]], np.float32)
        return self.postprocess([np.asarray(self.runtime.infer(feeds)[0], np.float32)], info)

    def postprocess(self, outs, info):
        rows = np.asarray(outs[0], np.float32).reshape(-1, 6)
        rows = rows[rows[:, 1] > self.conf_threshold]
        r = FaceDetectionResult()
        r.boxes, r.scores = rows[:, 2:6].tolist(), rows[:, 1].tolist()
        return r


class CenterFace(_FaceDetBase):
    """CenterFace (facedet/contrib/centerface/): heat-map [1,1,h/4,w/4], scale [1,2,..], offset [1,2,..],
    landmarks [1,10,..]; peaks above the threshold decode to boxes of size exp(scale) * 4."""

    def _configure(self):
        self.conf_threshold = 0.5
        self.nms_iou_threshold = 0.3
        self.landmarks_per_face = 5

    def preprocess(self, im):
        canvas, info = self._letterbox(im)
        x = canvas[..., ::-1].astype(np.float32)
        return self._layout(x), info

    def postprocess(self, outs, info):
        heat, scale, offset, lms = outs[0][0, 0], outs[1][0], outs[2][0], outs[3][0]
        ys, xs = np.nonzero(heat > self.conf_threshold)
        boxes, scores, pts = [], [], []
        for y, x in zip(ys, xs):
            s0, s1 = math.exp(scale[0, y, x]) * 4, math.exp(scale[1, y, x]) * 4
            o0, o1 = offset[0, y, x], offset[1, y, x]
            x1 = max(0.0, (x + o1 + 0.5) * 4 - s1 / 2)
            y1 = max(0.0, (y + o0 + 0.5) * 4 - s0 / 2)
            boxes.append([x1, y1, x1 + s1, y1 + s0])
            scores.append(heat[y, x])
            pts.append([[lms[2 * j + 1, y, x] * s1 + x1, lms[2 * j, y, x] * s0 + y1] for j in range(5)])
        return _finish(boxes, scores, pts, 5, self.nms_iou_threshold, info)


def _named(model_cls, role: str, name: str):
    cls = type(name, (_FaceProcessor,), {"MODEL": model_cls, "ROLE": role,
                                          "__doc__": f"{'Pre' if role == 'pre' else 'Post'}-processing of :class:`{model_cls.__name__}`."})
    _NAMED[(model_cls.__name__, role)] = cls
    return cls


BlazeFacePreprocessor = _named(BlazeFace, "pre", "BlazeFacePreprocessor")
BlazeFacePostprocessor = _named(BlazeFace, "post", "BlazeFacePostprocessor")
CenterFacePreprocessor = _named(CenterFace, "pre", "CenterFacePreprocessor")
CenterFacePostprocessor = _named(CenterFace, "post", "CenterFacePostprocessor")
Yolov7FacePreprocessor = _named(YOLOv7Face, "pre", "Yolov7FacePreprocessor")
Yolov7FacePostprocessor = _named(YOLOv7Face, "post", "Yolov7FacePostprocessor")
