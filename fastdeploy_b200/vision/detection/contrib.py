"""Community detector family (fastdeploy/vision/detection/contrib/): YOLOv5 / v5Lite / v5Seg / v6 / v7 /
v7End2End / v8 / X / R, ScaledYOLOv4, NanoDetPlus, FastestDet and the RKYOLO aliases.

All of them share one pre-processing recipe - letterbox to a fixed size with value 114, BGR->RGB,
scale by 1/255, HWC->CHW (contrib/yolov5/preprocessor.cc:45-97) - and differ in how the head output
is decoded; the decoders below restate each post-processor (contrib/yolov5/postprocessor.cc:26-103,
yolov8/postprocessor.cc, yolox.cc:228-318, nanodet_plus.cc:203-300, fastestdet/postprocessor.cc,
yolov7end2end_ort.cc:190-240, yolov5seg/postprocessor.cc). Class-aware NMS is done the reference's way:
boxes are offset by ``label * max_wh`` so that one class-agnostic hard NMS separates the classes.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np

from ...core.types import ModelFormat
from ...runtime.model import FastDeployModel
from ...runtime.option import RuntimeOption
from .. import utils as vutils
from ..result import DetectionResult, Mask


def _resize_bilinear(img: np.ndarray, w: int, h: int) -> np.ndarray:
    try:
        import cv2
        return cv2.resize(img, (w, h), interpolation=cv2.INTER_LINEAR)
    except ImportError:      # OpenCV-free restatement (half-pixel centres)
        sh, sw = img.shape[:2]
        ys = np.clip((np.arange(h) + 0.5) * sh / h - 0.5, 0, sh - 1)
        xs = np.clip((np.arange(w) + 0.5) * sw / w - 0.5, 0, sw - 1)
        y0, x0 = np.floor(ys).astype(int), np.floor(xs).astype(int)
        y1, x1 = np.minimum(y0 + 1, sh - 1), np.minimum(x0 + 1, sw - 1)
        wy, wx = (ys - y0)[:, None, None], (xs - x0)[None, :, None]
        im = img.astype(np.float32).reshape(sh, sw, -1)
        out = (im[y0][:, x0] * (1 - wy) * (1 - wx) + im[y0][:, x1] * (1 - wy) * wx
               + im[y1][:, x0] * wy * (1 - wx) + im[y1][:, x1] * wy * wx)
        return np.clip(np.rint(out), 0, 255).astype(img.dtype).reshape(h, w, *img.shape[2:])


def letterbox(img: np.ndarray, size: Sequence[int], pad_value: Sequence[float] = (114, 114, 114), *, mini_pad: bool = False,
              no_pad: bool = False, scale_up: bool = True, stride: int = 32, center: bool = True):
    """Returns ``(canvas, info)`` with ``info = {scale, pad_w, pad_h, in_hw, out_hw}`` (``size`` is [w, h])."""
    h, w = img.shape[:2]
    scale = min(size[1] / h, size[0] / w)
    if not scale_up:
        scale = min(scale, 1.0)
    rw, rh = int(round(w * scale)), int(round(h * scale))
    pad_w, pad_h = size[0] - rw, size[1] - rh
    if mini_pad:
        pad_w, pad_h = pad_w % stride, pad_h % stride
    elif no_pad:
        pad_w, pad_h, rw, rh = 0, 0, size[0], size[1]
    if (rh, rw) != (h, w):
        img = _resize_bilinear(img, rw, rh)
    if center:
        half_h, half_w = pad_h / 2.0, pad_w / 2.0
        top, bottom = int(round(half_h - 0.1)), int(round(half_h + 0.1))
        left, right = int(round(half_w - 0.1)), int(round(half_w + 0.1))
    else:
        top, left, bottom, right = 0, 0, pad_h, pad_w
    canvas = np.empty((rh + top + bottom, rw + left + right, 3), dtype=img.dtype)
    canvas[...] = np.asarray(pad_value, dtype=img.dtype)
    canvas[top:top + rh, left:left + rw] = img
    return canvas, {"scale": scale, "pad_w": left, "pad_h": top, "in_hw": (h, w), "out_hw": canvas.shape[:2]}


class YOLOPreprocessor:
    def __init__(self, size: Sequence[int] = (640, 640)):
        self.size = list(size)
        self.padding_value = [114.0, 114.0, 114.0]
        self.is_mini_pad = False
        self.is_no_pad = False
        self.is_scale_up = True
        self.stride = 32
        self.center = True
        self.normalize = True       # scale by 1/255
        self.swap_rb = True

    def run(self, images: Sequence[np.ndarray]) -> Tuple[np.ndarray, List[Dict[str, Any]]]:
        outs, infos = [], []
        for im in images:
            canvas, info = letterbox(im, self.size, self.padding_value, mini_pad=self.is_mini_pad, no_pad=self.is_no_pad,
                                     scale_up=self.is_scale_up, stride=self.stride, center=self.center)
            x = canvas[..., ::-1] if self.swap_rb else canvas
            x = x.astype(np.float32)
            if self.normalize:
                x = x / 255.0
            outs.append(np.ascontiguousarray(x.transpose(2, 0, 1)))
            infos.append(info)
        return np.stack(outs), infos


def letterbox_geometry(h: int, w: int, size: Sequence[int], *, scale_up: bool = True, center: bool = True) -> Dict[str, Any]:
    """Placement of an ``h x w`` image on a ``size = [w, h]`` canvas (the fixed-size form of :func:`letterbox`)."""
    scale = min(size[1] / h, size[0] / w)
    if not scale_up:
        scale = min(scale, 1.0)
    rw, rh = int(round(w * scale)), int(round(h * scale))
    pad_w, pad_h = size[0] - rw, size[1] - rh
    if center:
        top, left = int(round(pad_h / 2.0 - 0.1)), int(round(pad_w / 2.0 - 0.1))
    else:
        top, left = 0, 0
    return {"scale": scale, "pad_w": left, "pad_h": top, "in_hw": (h, w), "out_hw": (size[1], size[0]), "rw": rw, "rh": rh}


class DeviceLetterbox:
    """Letterbox + BGR->RGB + 1/255 on the GPU in one launch per batch (csrc/kernels/preproc.cu): raw frames are copied
    to the device as they are, the kernel resizes each into its place on the padded canvas and writes the network's
    16-bit NHWC input directly. The reference's version is fastdeploy/vision/utils/yolo_preprocess.cu:37-113."""

    def __init__(self, pre: "YOLOPreprocessor", device):
        self.pre, self.device = pre, device
        self._state: Dict[Tuple, Dict[str, Any]] = {}

    def supported(self) -> bool:
        return not (self.pre.is_mini_pad or self.pre.is_no_pad)

    def run(self, images: Sequence[np.ndarray], dst) -> List[Dict[str, Any]]:
        """``dst``: the plan's input as a dense ``[n, H, W, c_phys]`` 16-bit tensor. Returns the letterbox infos."""
        import torch
        from ...ops import preproc as P
        n = len(images)
        size = self.pre.size
        infos = [letterbox_geometry(int(im.shape[0]), int(im.shape[1]), size, scale_up=self.pre.is_scale_up,
                                    center=self.pre.center) for im in images]
        sizes = [int(im.shape[0]) * int(im.shape[1]) * 3 for im in images]
        offs = np.concatenate([[0], np.cumsum([(s + 255) // 256 * 256 for s in sizes])]).astype(np.int64)
        key = (n, int(offs[-1]), dst.data_ptr(), tuple(dst.shape))
        st = self._state.get(key)
        if st is None:
            a = 1.0 / 255.0 if self.pre.normalize else 1.0
            raw = torch.empty(int(offs[-1]), dtype=torch.uint8, device=self.device)
            meta_host = torch.empty(n * P.IMAGE_META.itemsize, dtype=torch.uint8).pin_memory()
            meta_dev = torch.empty(n * P.IMAGE_META.itemsize, dtype=torch.uint8, device=self.device)
            op = P.Preprocess(raw, meta_dev, dst, n=n, out_hw=(size[1], size[0]), layout="nhwc", c_out=dst.shape[3],
                              interp="linear", swap_rb=self.pre.swap_rb, alpha=[a] * 3, beta=[0.0] * 3,
                              pad_value=[float(v) * a for v in self.pre.padding_value])
            st = self._state[key] = dict(raw=raw, meta_host=meta_host, meta_dev=meta_dev, op=op)
            if len(self._state) > 8:
                self._state.pop(next(iter(self._state)))
        meta = np.frombuffer(st["meta_host"].numpy(), dtype=P.IMAGE_META)
        for i, (im, g) in enumerate(zip(images, infos)):
            t = im if isinstance(im, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(im))
            st["raw"][int(offs[i]):int(offs[i]) + sizes[i]].copy_(t.reshape(-1), non_blocking=True)
            P.fill_meta(meta, i, src_offset=int(offs[i]), src_hw=(int(im.shape[0]), int(im.shape[1])),
                        src_stride=int(im.shape[1]) * 3, resized_hw=(g["rh"], g["rw"]), top_left=(g["pad_h"], g["pad_w"]))
        st["meta_dev"].copy_(st["meta_host"], non_blocking=True)
        st["op"].launch()
        return infos


def _xywh_to_xyxy(b: np.ndarray) -> np.ndarray:
    out = np.empty_like(b)
    out[:, 0], out[:, 1] = b[:, 0] - b[:, 2] / 2, b[:, 1] - b[:, 3] / 2
    out[:, 2], out[:, 3] = b[:, 0] + b[:, 2] / 2, b[:, 1] + b[:, 3] / 2
    return out


def finish(boxes: np.ndarray, scores: np.ndarray, labels: np.ndarray, info: Dict[str, Any], nms_threshold: float,
           max_wh: float = 7680.0, multi_label: bool = True, extra: Optional[np.ndarray] = None):
    """Class-offset hard NMS, undo the letterbox, clip to the source image. Returns a DetectionResult
    and the indices (into the inputs) of the kept rows."""
    res = DetectionResult()
    if boxes.shape[0] == 0:
        return res, np.zeros(0, int)
    off = (labels.astype(np.float32) * max_wh)[:, None] if multi_label else 0.0
    tmp = DetectionResult()
    tmp.boxes = (boxes + off).tolist()
    tmp.scores = scores.tolist()
    tmp.label_ids = list(range(len(scores)))          # carry the row index through NMS
    vutils.nms(tmp, nms_threshold)
    keep = np.asarray(tmp.label_ids, int)
    b = boxes[keep].astype(np.float32)
    b[:, [0, 2]] = (b[:, [0, 2]] - info["pad_w"]) / info["scale"]
    b[:, [1, 3]] = (b[:, [1, 3]] - info["pad_h"]) / info["scale"]
    h, w = info["in_hw"]
    b[:, [0, 2]] = np.clip(b[:, [0, 2]], 0, w)
    b[:, [1, 3]] = np.clip(b[:, [1, 3]], 0, h)
    res.boxes = b.tolist()
    res.scores = scores[keep].astype(float).tolist()
    res.label_ids = labels[keep].astype(int).tolist()
    return res, keep


class YOLOPostprocessor:
    """Decoder selected by ``kind``:

    ``v5``  rows ``[cx, cy, w, h, obj, cls...]`` (v5, v5Lite, v6 legacy, v7, R, ScaledYOLOv4)
    ``v8``  ``[4 + C, anchors]`` columns ``[cx, cy, w, h, cls...]`` (v8, v6 3.0)
    ``x``   YOLOX raw grid output ``[dx, dy, log w, log h, obj, cls...]`` per stride 8/16/32
    ``e2e`` already decoded rows ``[batch, x1, y1, x2, y2, label, score]``
    """

    def __init__(self, kind: str = "v5"):
        self.kind = kind
        self.conf_threshold = 0.25
        self.nms_threshold = 0.5
        self.multi_label = True
        self.max_wh = 7680.0
        self.strides = [8, 16, 32]
        # kept for models exported without the decode step (yolov5lite.cc:190-240); the exports handled here are decoded
        self.is_decode_exported = True
        self.anchor_config = [[10.0, 13.0, 16.0, 30.0, 33.0, 23.0], [30.0, 61.0, 62.0, 45.0, 59.0, 119.0],
                              [116.0, 90.0, 156.0, 198.0, 373.0, 326.0]]

    def _candidates(self, out: np.ndarray, info: Dict[str, Any]):
        if self.kind == "v8":
            out = out.T
            cls = out[:, 4:]
            labels = cls.argmax(1)
            conf = cls[np.arange(len(cls)), labels]
            boxes = _xywh_to_xyxy(out[:, :4])
        elif self.kind == "x":
            h, w = info["out_hw"]
            grids, strides = [], []
            for s in self.strides:
                gy, gx = np.meshgrid(np.arange(h // s), np.arange(w // s), indexing="ij")
                grids.append(np.stack([gx.ravel(), gy.ravel()], 1))
                strides.append(np.full((gx.size, 1), s))
            g, st = np.concatenate(grids), np.concatenate(strides)
            xy = (out[:, :2] + g) * st
            wh = np.exp(out[:, 2:4]) * st
            boxes = _xywh_to_xyxy(np.concatenate([xy, wh], 1))
            cls = out[:, 5:] * out[:, 4:5]
            labels = cls.argmax(1)
            conf = cls[np.arange(len(cls)), labels]
        else:
            obj = out[:, 4]
            cls = out[:, 5:]
            labels = cls.argmax(1)
            conf = obj * cls[np.arange(len(cls)), labels]
            boxes = _xywh_to_xyxy(out[:, :4])
        m = conf > self.conf_threshold
        return boxes[m].astype(np.float32), conf[m].astype(np.float32), labels[m], np.nonzero(m)[0]

    def run(self, outputs: Sequence[np.ndarray], infos: List[Dict[str, Any]]) -> List[DetectionResult]:
        out0 = np.asarray(outputs[0], dtype=np.float32)
        results = []
        if self.kind == "e2e":
            for i, info in enumerate(infos):
                rows = out0[out0[:, 0] == i]
                rows = rows[rows[:, 6] > self.conf_threshold]
                r = DetectionResult()
                b = rows[:, 1:5].copy()
                b[:, [0, 2]] = np.clip((b[:, [0, 2]] - info["pad_w"]) / info["scale"], 0, info["in_hw"][1])
                b[:, [1, 3]] = np.clip((b[:, [1, 3]] - info["pad_h"]) / info["scale"], 0, info["in_hw"][0])
                r.boxes, r.scores, r.label_ids = b.tolist(), rows[:, 6].tolist(), rows[:, 5].astype(int).tolist()
                results.append(r)
            return results
        for i, info in enumerate(infos):
            boxes, conf, labels, _ = self._candidates(out0[i], info)
            results.append(finish(boxes, conf, labels, info, self.nms_threshold, self.max_wh, self.multi_label)[0])
        return results


def _forwarded(owner: str, attr: str, doc: str = ""):
    """A model attribute of older releases that now lives on the pre- or post-processor
    (e.g. ``model.size`` -> ``model.preprocessor.size``; python/fastdeploy/vision/detection/contrib/yolov5.py:130-230)."""
    def get(self):
        return getattr(getattr(self, owner), attr)

    def put(self, value):
        setattr(getattr(self, owner), attr, value)
    return property(get, put, doc=doc)


class _YOLOModel(FastDeployModel):
    KIND = "v5"
    SIZE = (640, 640)
    PRE = None          # processor classes; a family below names its own
    POST = None

    def __init__(self, model_file: str, params_file: str = "", runtime_option: Optional[RuntimeOption] = None,
                 model_format: int = ModelFormat.ONNX):
        super().__init__(runtime_option)
        self.runtime_option.set_model_path(model_file, params_file, model_format)
        self.preprocessor = self.PRE() if self.PRE is not None else YOLOPreprocessor(self.SIZE)
        self.postprocessor = self.POST() if self.POST is not None else YOLOPostprocessor(self.KIND)
        self._configure()
        self.init_runtime()

    size = _forwarded("preprocessor", "size", "[width, height] of the network input")
    padding_value = _forwarded("preprocessor", "padding_value")
    is_mini_pad = _forwarded("preprocessor", "is_mini_pad")
    is_no_pad = _forwarded("preprocessor", "is_no_pad")
    is_scale_up = _forwarded("preprocessor", "is_scale_up")
    stride = _forwarded("preprocessor", "stride")
    max_wh = _forwarded("postprocessor", "max_wh")
    multi_label = _forwarded("postprocessor", "multi_label")
    conf_threshold = _forwarded("postprocessor", "conf_threshold")
    nms_threshold = _forwarded("postprocessor", "nms_threshold")
    downsample_strides = _forwarded("postprocessor", "strides", "strides of the head levels")
    is_decode_exported = _forwarded("postprocessor", "is_decode_exported")
    anchor_config = _forwarded("postprocessor", "anchor_config")

    @property
    def keep_ratio(self) -> bool:
        return not self.preprocessor.is_no_pad

    @keep_ratio.setter
    def keep_ratio(self, v: bool) -> None:
        self.preprocessor.is_no_pad = not v

    def _configure(self) -> None:
        pass

    def get_preprocessor(self):
        return self.preprocessor

    def get_postprocessor(self):
        return self.postprocessor

    def predict(self, im: np.ndarray, conf_threshold: Optional[float] = None, nms_iou_threshold: Optional[float] = None):
        if conf_threshold is not None:
            self.postprocessor.conf_threshold = conf_threshold
        if nms_iou_threshold is not None:
            self.postprocessor.nms_threshold = nms_iou_threshold
        return self.batch_predict([im])[0]

    def batch_predict(self, images: Sequence[np.ndarray]) -> List[DetectionResult]:
        name = self.runtime.get_input_info(0).name
        if getattr(self.runtime, "on_gpu", False) and all(im.ndim == 3 and im.shape[2] == 3 and im.dtype == np.uint8
                                                           for im in images):
            # letterbox, channel swap and scaling on the device, straight into the plan's input buffer
            import torch
            rt = self.runtime
            if getattr(self, "_device_pre", None) is None:
                self._device_pre = DeviceLetterbox(self.preprocessor, rt.device)
            if self._device_pre.supported():
                w, h = self.preprocessor.size
                with torch.cuda.device(rt.device):
                    plan = rt.plan_for_shapes({name: [len(images), 3, h, w]})
                    base = plan.inputs[name].t
                    dst = torch.as_strided(base, (base.shape[0], base.shape[1], base.shape[2], base.stride(2)), base.stride())
                    infos = self._device_pre.run(images, dst)
                    plan.run()
                    rt.gpu_launches += plan.native_kernel_launches + 1
                    outs = [rt._to_numpy(plan.outputs[vi.name].logical()) for vi in rt.graph.outputs]
                    plan.status.check("YOLO inference")
                return self.postprocessor.run(outs, infos)
        x, infos = self.preprocessor.run(images)
        outs = self.runtime.infer({name: x})
        return self.postprocessor.run(outs, infos)


def _model(name: str, kind: str, doc: str, pre=None, post=None, **cfg):
    def _configure(self):
        for k, v in cfg.items():
            target = self.preprocessor if hasattr(self.preprocessor, k) else self.postprocessor
            setattr(target, k, v)
    return type(name, (_YOLOModel,), {"KIND": kind, "__doc__": doc, "_configure": _configure, "PRE": pre, "POST": post})


def _processor_pair(family: str, kind: str, where: str):
    """The pre- and post-processor classes a family exposes under its own name (``YOLOv5Preprocessor`` ...); they are the
    shared letterbox and decoder with the family's defaults."""
    pre = type(f"{family}Preprocessor", (YOLOPreprocessor,),
               {"__doc__": f"Letterbox to 640 x 640, BGR->RGB, 1/255, CHW ({where}/preprocessor.cc)."})

    def post_init(self):
        YOLOPostprocessor.__init__(self, kind)
    post = type(f"{family}Postprocessor", (YOLOPostprocessor,),
                {"__init__": post_init, "__doc__": f"Confidence filter, class-aware NMS, boxes back to the source image ({where}/postprocessor.cc)."})
    return pre, post


YOLOv5Preprocessor, YOLOv5Postprocessor = _processor_pair("YOLOv5", "v5", "contrib/yolov5")
YOLOv7Preprocessor, YOLOv7Postprocessor = _processor_pair("YOLOv7", "v5", "contrib/yolov7")
YOLOv8Preprocessor, YOLOv8Postprocessor = _processor_pair("YOLOv8", "v8", "contrib/yolov8")
RKYOLOPreprocessor, RKYOLOPostprocessor = _processor_pair("RKYOLO", "v5", "contrib/rknpu2")


def _rk_set_anchor(self, anchors: Sequence[int], anchor_per_branch: int = 3) -> None:
    """Anchor sizes as one flat list (w, h pairs, small to large stride), ``anchor_per_branch`` pairs per head level
    (contrib/rknpu2/postprocessor.h:60-75)."""
    flat = [float(a) for a in anchors]
    per = 2 * int(anchor_per_branch)
    if per <= 0 or len(flat) % per:
        raise ValueError(f"{len(flat)} anchor values do not split into levels of {anchor_per_branch} pairs")
    self.anchor_config = [flat[i:i + per] for i in range(0, len(flat), per)]
    self.anchor_per_branch = int(anchor_per_branch)


RKYOLOPostprocessor.set_anchor = _rk_set_anchor
RKYOLOPostprocessor.class_num = 80

YOLOv5 = _model("YOLOv5", "v5", "YOLOv5 (contrib/yolov5/yolov5.cc).", YOLOv5Preprocessor, YOLOv5Postprocessor)
YOLOv5Lite = _model("YOLOv5Lite", "v5", "YOLOv5-Lite with decoded export (contrib/yolov5lite.cc).", conf_threshold=0.45)
YOLOv6 = _model("YOLOv6", "v5", "YOLOv6 (contrib/yolov6.cc).")
YOLOv7 = _model("YOLOv7", "v5", "YOLOv7 (contrib/yolov7/yolov7.cc).", YOLOv7Preprocessor, YOLOv7Postprocessor)
YOLOv8 = _model("YOLOv8", "v8", "YOLOv8 (contrib/yolov8/yolov8.cc): [4 + classes, anchors] head without objectness.",
                YOLOv8Preprocessor, YOLOv8Postprocessor)
YOLOR = _model("YOLOR", "v5", "YOLOR (contrib/yolor.cc).")
ScaledYOLOv4 = _model("ScaledYOLOv4", "v5", "Scaled-YOLOv4 (contrib/scaledyolov4.cc).")
YOLOX = _model("YOLOX", "x", "YOLOX (contrib/yolox.cc): grid decode, bottom-right padding, no 1/255 scaling.",
               center=False, normalize=False, swap_rb=False)
YOLOv7End2EndORT = _model("YOLOv7End2EndORT", "e2e", "YOLOv7 exported with the NMS plugin for ORT (yolov7end2end_ort.cc).")
YOLOv7End2EndTRT = _model("YOLOv7End2EndTRT", "e2e", "YOLOv7 exported with EfficientNMS for TensorRT (yolov7end2end_trt.cc).")
def _rk_init(self, model_file: str, runtime_option: Optional[RuntimeOption] = None, model_format: int = ModelFormat.ONNX,
             params_file: str = ""):
    """The Rockchip classes take no parameter file (python/fastdeploy/vision/detection/contrib/rkyolo/__init__.py:150-170)."""
    _YOLOModel.__init__(self, model_file, params_file, runtime_option, model_format)


RKYOLOV5 = _model("RKYOLOV5", "v5", "YOLOv5 head layout of the Rockchip export (contrib/rknpu2/rkyolo.cc).",
                  RKYOLOPreprocessor, RKYOLOPostprocessor)
RKYOLOV7 = _model("RKYOLOV7", "v5", "YOLOv7 head layout of the Rockchip export.", RKYOLOPreprocessor, RKYOLOPostprocessor)
RKYOLOX = _model("RKYOLOX", "x", "YOLOX head layout of the Rockchip export.", center=False, normalize=False, swap_rb=False)
for _cls in (RKYOLOV5, RKYOLOV7, RKYOLOX):
    _cls.__init__ = _rk_init


class NanoDetPlus(_YOLOModel):
    """NanoDet-Plus (contrib/nanodet_plus.cc:203-300): per-level GFL head, ``reg_max = 7`` integral
    regression, centre priors at ``(x + 0) * stride`` with strides 8/16/32/64, mean/std normalisation."""
    SIZE = (320, 320)

    def _configure(self) -> None:
        self.preprocessor.normalize = False
        self.preprocessor.swap_rb = False
        self.preprocessor.center = False
        self.preprocessor.is_no_pad = True
        self.mean = np.asarray([103.53, 116.28, 123.675], np.float32)
        self.std = np.asarray([57.375, 57.12, 58.395], np.float32)
        self.reg_max = 7
        self.strides = [8, 16, 32, 64]
        self.postprocessor.conf_threshold = 0.35

    def batch_predict(self, images):
        x, infos = self.preprocessor.run(images)
        x = (x - self.mean[None, :, None, None]) / self.std[None, :, None, None]
        out = np.asarray(self.runtime.infer({self.runtime.get_input_info(0).name: x})[0], np.float32)
        return [self.decode(out[i], info) for i, info in enumerate(infos)]

    def decode(self, out: np.ndarray, info: Dict[str, Any]) -> DetectionResult:
        h, w = info["out_hw"]
        nreg = 4 * (self.reg_max + 1)
        ncls = out.shape[1] - nreg
        centers, strides = [], []
        for s in self.strides:
            fh, fw = math.ceil(h / s), math.ceil(w / s)
            gy, gx = np.meshgrid(np.arange(fh), np.arange(fw), indexing="ij")
            centers.append(np.stack([gx.ravel() * s, gy.ravel() * s], 1))
            strides.append(np.full(gx.size, s))
        c, st = np.concatenate(centers).astype(np.float32), np.concatenate(strides).astype(np.float32)
        cls = out[:, :ncls]
        labels = cls.argmax(1)
        conf = cls[np.arange(len(cls)), labels]
        reg = out[:, ncls:].reshape(-1, 4, self.reg_max + 1)
        reg = np.exp(reg - reg.max(-1, keepdims=True))
        reg /= reg.sum(-1, keepdims=True)
        dist = (reg * np.arange(self.reg_max + 1)).sum(-1) * st[:, None]
        boxes = np.stack([c[:, 0] - dist[:, 0], c[:, 1] - dist[:, 1], c[:, 0] + dist[:, 2], c[:, 1] + dist[:, 3]], 1)
        m = conf > self.postprocessor.conf_threshold
        # the image was stretched, not letterboxed: undo per-axis scales
        sh, sw = info["in_hw"][0] / h, info["in_hw"][1] / w
        inf = {"scale": 1.0, "pad_w": 0, "pad_h": 0, "in_hw": (h, w)}
        res, _ = finish(boxes[m], conf[m], labels[m], inf, self.postprocessor.nms_threshold)
        b = np.asarray(res.boxes, np.float32).reshape(-1, 4)
        b[:, [0, 2]] *= sw
        b[:, [1, 3]] *= sh
        res.boxes = b.tolist()
        return res


class FastestDetPreprocessor(YOLOPreprocessor):
    """Plain resize to 352 x 352 (no letterbox), BGR kept, 1/255, CHW (contrib/fastestdet/preprocessor.cc:27-80)."""

    def __init__(self):
        super().__init__((352, 352))
        self.is_no_pad = True
        self.swap_rb = False


class FastestDetPostprocessor:
    """One 22 x 22 map of ``[obj, tanh dx, tanh dy, sigmoid w, sigmoid h, cls...]``; score = obj^0.6 * cls^0.4; boxes
    normalised to the input, scaled to the source image (contrib/fastestdet/postprocessor.cc:30-110)."""

    def __init__(self):
        self.conf_threshold = 0.65
        self.nms_threshold = 0.45

    def decode(self, out: np.ndarray, info: Dict[str, Any]) -> DetectionResult:
        c, fh, fw = out.shape
        obj = out[0]
        cls = out[5:]
        labels = cls.argmax(0)
        cmax = cls.max(0)
        score = (obj ** 0.6) * (cmax ** 0.4)
        gy, gx = np.meshgrid(np.arange(fh), np.arange(fw), indexing="ij")
        cx = (np.tanh(out[1]) + gx) / fw
        cy = (np.tanh(out[2]) + gy) / fh
        bw = 1.0 / (1.0 + np.exp(-out[3]))
        bh = 1.0 / (1.0 + np.exp(-out[4]))
        ih, iw = info["in_hw"]
        boxes = np.stack([(cx - bw / 2) * iw, (cy - bh / 2) * ih, (cx + bw / 2) * iw, (cy + bh / 2) * ih], -1).reshape(-1, 4)
        m = score.ravel() > self.conf_threshold
        inf = {"scale": 1.0, "pad_w": 0, "pad_h": 0, "in_hw": (ih, iw)}
        return finish(boxes[m], score.ravel()[m], labels.ravel()[m], inf, self.nms_threshold)[0]

    def run(self, outputs: Sequence[np.ndarray], infos: List[Dict[str, Any]]) -> List[DetectionResult]:
        out = np.asarray(outputs[0], np.float32)
        return [self.decode(out[i], info) for i, info in enumerate(infos)]


class FastestDet(_YOLOModel):
    """FastestDet (contrib/fastestdet/fastestdet.cc)."""
    SIZE = (352, 352)
    PRE = FastestDetPreprocessor
    POST = FastestDetPostprocessor

    def batch_predict(self, images):
        x, infos = self.preprocessor.run(images)
        return self.postprocessor.run(self.runtime.infer({self.runtime.get_input_info(0).name: x}), infos)

    def decode(self, out: np.ndarray, info: Dict[str, Any]) -> DetectionResult:
        return self.postprocessor.decode(out, info)


class YOLOv5SegPreprocessor(YOLOPreprocessor):
    """The YOLOv5 letterbox (contrib/yolov5seg/preprocessor.cc)."""


class YOLOv5SegPostprocessor(YOLOPostprocessor):
    """YOLOv5 instance segmentation (contrib/yolov5seg/postprocessor.cc:30-190): rows carry ``mask_nums`` mask
    coefficients after the class scores; masks = sigmoid(coeff @ protos) cropped to the box, resized to the source image
    and thresholded at ``mask_threshold``."""

    def __init__(self):
        super().__init__("v5")
        self.mask_nums = 32
        self.mask_threshold = 0.5

    def run(self, outputs: Sequence[np.ndarray], infos: List[Dict[str, Any]]) -> List[DetectionResult]:
        det, protos = np.asarray(outputs[0], np.float32), np.asarray(outputs[1], np.float32)
        res = []
        for i, info in enumerate(infos):
            rows = det[i]
            ncls = rows.shape[1] - 5 - self.mask_nums
            boxes, conf, labels, idx = self._candidates(rows[:, :5 + ncls], info)
            r, keep = finish(boxes, conf, labels, info, self.nms_threshold)
            r.contain_masks = True
            if len(keep):
                coeff = rows[idx[keep], 5 + ncls:]
                pc, ph, pw = protos[i].shape
                m = 1.0 / (1.0 + np.exp(-(coeff @ protos[i].reshape(pc, -1)))).reshape(-1, ph, pw)
                r.masks = [self._crop_mask(m[k], boxes[keep[k]], info, (ph, pw)) for k in range(len(keep))]
            res.append(r)
        return res

    def _crop_mask(self, m: np.ndarray, box_in: np.ndarray, info, proto_hw) -> Mask:
        ph, pw = proto_hw
        oh, ow = info["out_hw"]
        # letterboxed-input box -> proto grid
        x1, y1, x2, y2 = box_in * np.asarray([pw / ow, ph / oh, pw / ow, ph / oh])
        yy, xx = np.mgrid[0:ph, 0:pw]
        m = m * ((xx >= x1) & (xx < x2) & (yy >= y1) & (yy < y2))
        # strip the letterbox padding, resize to the source size
        top, left = int(info["pad_h"] * ph / oh), int(info["pad_w"] * pw / ow)
        bottom, right = ph - top, pw - left
        core = m[top:bottom, left:right]
        h, w = info["in_hw"]
        full = _resize_bilinear((core * 255).astype(np.uint8), w, h).astype(np.float32) / 255.0
        out = Mask()
        out.data = (full > self.mask_threshold).astype(np.uint8)
        out.shape = [h, w]
        return out


class YOLOv5Seg(_YOLOModel):
    """YOLOv5 instance segmentation (contrib/yolov5seg/yolov5seg.cc)."""
    PRE = YOLOv5SegPreprocessor
    POST = YOLOv5SegPostprocessor

    mask_nums = _forwarded("postprocessor", "mask_nums")
    mask_threshold = _forwarded("postprocessor", "mask_threshold")

    def batch_predict(self, images):
        x, infos = self.preprocessor.run(images)
        return self.postprocessor.run(self.runtime.infer({self.runtime.get_input_info(0).name: x}), infos)
