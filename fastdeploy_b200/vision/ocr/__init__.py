"""``fastdeploy.vision.ocr``: DBDetector, Classifier, Recognizer with their pre/post-processors and the
PP-OCRv2/v3/v4 pipelines (fastdeploy/vision/ocr/ppocr/**). Semantics restated from
det_preprocessor.cc:23-102, utils/ocr_postprocess_op.cc:23-350, utils/get_rotate_crop_image.cc:21-81,
utils/sorted_boxes.cc:21-46, cls_preprocessor.cc:37-98, rec_preprocessor.cc:40-137,
rec_postprocessor.cc:23-83, ppocr_v2.cc:108-175. The unclip step offsets the min-area rectangle
analytically (a rectangle grown by ``d`` with round joins has the min-area rectangle grown by ``d`` per side),
which replaces the vendored Clipper library."""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import numpy as np

from ...core.types import ModelFormat
from ...runtime.model import FastDeployModel
from ...runtime.option import RuntimeOption
from ..result import OCRResult


class _NormalizeSwitches:
    """``set_normalize`` / ``disable_normalize`` / ``disable_permute`` of the three OCR pre-processors
    (fastdeploy/vision/ocr/ppocr/{det,cls,rec}_preprocessor.h). These act on the host path; the device pipeline always
    feeds the network normalised CHW crops."""
    normalize_ = True
    permute_ = True

    def set_normalize(self, mean, std, is_scale=True):
        self.mean, self.scale, self.is_scale = list(mean), list(std), is_scale

    def disable_normalize(self) -> None:
        self.normalize_ = False

    def disable_permute(self) -> None:
        self.permute_ = False

    def _finish(self, batch: np.ndarray) -> np.ndarray:
        """``batch`` is NCHW as built; HWC is wanted after ``disable_permute``."""
        return batch if self.permute_ else np.ascontiguousarray(batch.transpose(0, 2, 3, 1))


def _forward(owner: str, attr: str):
    def get(self):
        return getattr(getattr(self, owner), attr)

    def put(self, value):
        setattr(getattr(self, owner), attr, value)
    return property(get, put, doc=f"``{owner}.{attr}``, under the name older releases had on the model")


# ---------------------------------------------------------------------------------- detection
class DBDetectorPreprocessor(_NormalizeSwitches):
    def __init__(self):
        self.max_side_len = 960
        self.mean = [0.485, 0.456, 0.406]
        self.scale = [0.229, 0.224, 0.225]
        self.is_scale = True
        self.static_shape_infer = False
        self.det_image_shape = [3, 960, 960]

    def target_hw(self, h: int, w: int) -> Tuple[int, int]:
        """Limit the long side, then round both sides to multiples of 32 (min 32)."""
        if self.static_shape_infer:
            return self.det_image_shape[1], self.det_image_shape[2]
        ratio = 1.0
        if max(h, w) > self.max_side_len:
            ratio = self.max_side_len / max(h, w)
        rh, rw = int(h * ratio), int(w * ratio)
        rh = max(int(round(rh / 32) * 32), 32)
        rw = max(int(round(rw / 32) * 32), 32)
        return rh, rw

    def run(self, images: Sequence[np.ndarray]):
        import cv2
        from ...ops.preproc import normalize_coeffs
        alpha, beta = normalize_coeffs(self.mean, self.scale, self.is_scale)
        infos, mats = [], []
        for im in images:
            h, w = im.shape[:2]
            rh, rw = self.target_hw(h, w)
            r = cv2.resize(im, (rw, rh)) if (rh, rw) != (h, w) else im
            mats.append(r.astype(np.float32) * np.float32(alpha) + np.float32(beta) if self.normalize_ else r.astype(np.float32))
            infos.append([w, h, rw, rh])
        mh, mw = max(m.shape[0] for m in mats), max(m.shape[1] for m in mats)
        batch = np.zeros((len(mats), 3, mh, mw), np.float32)
        for i, m in enumerate(mats):
            batch[i, :, :m.shape[0], :m.shape[1]] = m.transpose(2, 0, 1)
        return self._finish(batch), infos


def _order_clockwise(pts: np.ndarray) -> np.ndarray:
    """Mini-box point order of the reference: sort by x, left pair by y, right pair by y."""
    p = pts[np.argsort(pts[:, 0], kind="stable")]
    left, right = p[:2], p[2:]
    left = left[np.argsort(left[:, 1], kind="stable")]
    right = right[np.argsort(right[:, 1], kind="stable")]
    return np.array([left[0], right[0], right[1], left[1]], np.float32)


class DBDetectorPostprocessor:
    def __init__(self):
        self.det_db_thresh = 0.3
        self.det_db_box_thresh = 0.6
        self.det_db_unclip_ratio = 1.5
        self.det_db_score_mode = "slow"
        self.use_dilation = False
        self.max_candidates = 1000

    @staticmethod
    def _mini_box(contour):
        import cv2
        rect = cv2.minAreaRect(contour)
        pts = _order_clockwise(cv2.boxPoints(rect))
        return pts, min(rect[1]), rect

    @staticmethod
    def _score_fast(prob, box):
        import cv2
        h, w = prob.shape
        xmin = int(np.clip(np.floor(box[:, 0].min()), 0, w - 1)); xmax = int(np.clip(np.ceil(box[:, 0].max()), 0, w - 1))
        ymin = int(np.clip(np.floor(box[:, 1].min()), 0, h - 1)); ymax = int(np.clip(np.ceil(box[:, 1].max()), 0, h - 1))
        mask = np.zeros((ymax - ymin + 1, xmax - xmin + 1), np.uint8)
        b = box.copy()
        b[:, 0] -= xmin
        b[:, 1] -= ymin
        cv2.fillPoly(mask, [b.astype(np.int32)], 1)
        return float(cv2.mean(prob[ymin:ymax + 1, xmin:xmax + 1], mask)[0])

    @staticmethod
    def _score_slow(prob, contour):
        import cv2
        h, w = prob.shape
        c = contour.reshape(-1, 2).astype(np.float32)
        xmin = int(np.clip(c[:, 0].min(), 0, w - 1)); xmax = int(np.clip(c[:, 0].max(), 0, w - 1))
        ymin = int(np.clip(c[:, 1].min(), 0, h - 1)); ymax = int(np.clip(c[:, 1].max(), 0, h - 1))
        mask = np.zeros((ymax - ymin + 1, xmax - xmin + 1), np.uint8)
        cc = c.copy()
        cc[:, 0] -= xmin
        cc[:, 1] -= ymin
        cv2.fillPoly(mask, [cc.astype(np.int32)], 1)
        return float(cv2.mean(prob[ymin:ymax + 1, xmin:xmax + 1], mask)[0])

    def _unclip(self, box: np.ndarray):
        """Offset distance = area * ratio / perimeter; the grown rectangle is returned as a cv2 rect."""
        import cv2
        area = cv2.contourArea(box.astype(np.float32))
        peri = cv2.arcLength(box.astype(np.float32), True)
        if peri < 1e-6:
            return None
        d = area * self.det_db_unclip_ratio / peri
        (cx, cy), (w, h), ang = cv2.minAreaRect(box.astype(np.float32))
        return (cx, cy), (w + 2 * d, h + 2 * d), ang

    def boxes_from_bitmap(self, prob: np.ndarray, src_w: int, src_h: int, rw: int, rh: int) -> List[List[int]]:
        import cv2
        prob = prob[:rh, :rw]
        bitmap = ((prob > self.det_db_thresh) * 255).astype(np.uint8)
        if self.use_dilation:
            bitmap = cv2.dilate(bitmap, np.ones((2, 2), np.uint8))
        contours, _ = cv2.findContours(bitmap, cv2.RETR_LIST, cv2.CHAIN_APPROX_SIMPLE)
        boxes = []
        for contour in contours[:self.max_candidates]:
            if len(contour) <= 2:
                continue
            box, sside, _ = self._mini_box(contour)
            if sside < 3:
                continue
            score = self._score_slow(prob, contour) if self.det_db_score_mode == "slow" else self._score_fast(prob, box)
            if score < self.det_db_box_thresh:
                continue
            grown = self._unclip(box)
            if grown is None:
                continue
            pts = _order_clockwise(cv2.boxPoints(grown))
            if min(grown[1]) < 5:
                continue
            q = []
            for x, y in pts:
                q += [int(np.clip(round(x / rw * src_w), 0, src_w - 1)), int(np.clip(round(y / rh * src_h), 0, src_h - 1))]
            bw = int(math.hypot(q[0] - q[2], q[1] - q[3]))
            bh = int(math.hypot(q[0] - q[6], q[1] - q[7]))
            if bw <= 4 or bh <= 4:
                continue
            boxes.append(q)
        return boxes

    def run(self, prob_maps: np.ndarray, infos) -> List[List[List[int]]]:
        out = []
        for i, (w, h, rw, rh) in enumerate(infos):
            out.append(self.boxes_from_bitmap(np.asarray(prob_maps[i, 0], np.float32), w, h, rw, rh))
        return out


class _OcrStage(FastDeployModel):
    def __init__(self, model_file, params_file, runtime_option, model_format):
        super().__init__(runtime_option)
        self.runtime_option.set_model_path(model_file, params_file, model_format)
        self.init_runtime()

    def _run_net(self, x: np.ndarray) -> np.ndarray:
        outs = self.infer({self.runtime.graph.inputs[0].name: x})
        return self.runtime._to_numpy(outs[self.runtime.graph.outputs[0].name])


class DBDetector(_OcrStage):
    def __init__(self, model_file: str, params_file: str = "", runtime_option: Optional[RuntimeOption] = None,
                 model_format: ModelFormat = ModelFormat.PADDLE):
        super().__init__(model_file, params_file, runtime_option, model_format)
        self.preprocessor = DBDetectorPreprocessor()
        self.postprocessor = DBDetectorPostprocessor()

    max_side_len = _forward("preprocessor", "max_side_len")
    det_db_thresh = _forward("postprocessor", "det_db_thresh")
    det_db_box_thresh = _forward("postprocessor", "det_db_box_thresh")
    det_db_unclip_ratio = _forward("postprocessor", "det_db_unclip_ratio")
    det_db_score_mode = _forward("postprocessor", "det_db_score_mode")
    use_dilation = _forward("postprocessor", "use_dilation")

    def predict(self, im: np.ndarray) -> List[List[int]]:
        return self.batch_predict([im])[0]

    def batch_predict(self, images: Sequence[np.ndarray]) -> List[List[List[int]]]:
        x, infos = self.preprocessor.run(images)
        return self.postprocessor.run(self._run_net(x), infos)


# ---------------------------------------------------------------------------------- crops
def sort_boxes(boxes: List[List[int]]) -> List[List[int]]:
    """Top-to-bottom then left-to-right with a 10 px row tolerance (utils/sorted_boxes.cc:21-46)."""
    b = sorted(boxes, key=lambda q: (q[1], q[0]))
    for i in range(len(b) - 1):
        for j in range(i, -1, -1):
            if abs(b[j + 1][1] - b[j][1]) < 10 and b[j + 1][0] < b[j][0]:
                b[j], b[j + 1] = b[j + 1], b[j]
            else:
                break
    return b


def get_rotate_crop_image(image: np.ndarray, box: Sequence[int]) -> np.ndarray:
    """Perspective warp of the quad to (|p0p1|, |p0p3|) with replicated border; rotated by 90 degrees when
    the crop is at least 1.5x taller than wide (utils/get_rotate_crop_image.cc:21-81)."""
    import cv2
    pts = np.asarray(box, np.float32).reshape(4, 2)
    x0, y0 = pts[:, 0].min(), pts[:, 1].min()
    x1, y1 = pts[:, 0].max(), pts[:, 1].max()
    crop = image[int(y0):int(y1) + 1, int(x0):int(x1) + 1]
    p = pts - np.array([int(x0), int(y0)], np.float32)
    w = int(math.hypot(p[0, 0] - p[1, 0], p[0, 1] - p[1, 1]))
    h = int(math.hypot(p[0, 0] - p[3, 0], p[0, 1] - p[3, 1]))
    w, h = max(w, 1), max(h, 1)
    dst = np.array([[0, 0], [w, 0], [w, h], [0, h]], np.float32)
    m = cv2.getPerspectiveTransform(p, dst)
    out = cv2.warpPerspective(crop, m, (w, h), flags=cv2.INTER_LINEAR, borderMode=cv2.BORDER_REPLICATE)
    if out.shape[0] >= out.shape[1] * 1.5:
        out = np.ascontiguousarray(np.rot90(out, 1)[::-1, ::-1].transpose(0, 1, 2)) if False else cv2.rotate(
            out, cv2.ROTATE_90_COUNTERCLOCKWISE)
    return out


# ---------------------------------------------------------------------------------- classifier
class ClassifierPreprocessor(_NormalizeSwitches):
    def __init__(self):
        self.cls_image_shape = [3, 48, 192]
        self.mean, self.scale, self.is_scale = [0.5] * 3, [0.5] * 3, True

    def run(self, images: Sequence[np.ndarray]) -> np.ndarray:
        import cv2
        c, H, W = self.cls_image_shape
        out = np.zeros((len(images), 3, H, W), np.float32)
        for i, im in enumerate(images):
            ratio = im.shape[1] / im.shape[0]
            rw = W if math.ceil(H * ratio) > W else int(math.ceil(H * ratio))
            r = cv2.resize(im, (rw, H)).astype(np.float32)
            if self.normalize_:
                r = ((r / 255.0 if self.is_scale else r) - np.float32(self.mean)) / np.float32(self.scale)
            out[i, :, :, :rw] = r.transpose(2, 0, 1)
        return self._finish(out)


class ClassifierPostprocessor:
    def __init__(self):
        self.cls_thresh = 0.9

    def run(self, probs: np.ndarray) -> Tuple[List[int], List[float]]:
        p = np.asarray(probs, np.float32)
        return p.argmax(1).astype(int).tolist(), p.max(1).astype(float).tolist()


class Classifier(_OcrStage):
    def __init__(self, model_file: str, params_file: str = "", runtime_option: Optional[RuntimeOption] = None,
                 model_format: ModelFormat = ModelFormat.PADDLE):
        super().__init__(model_file, params_file, runtime_option, model_format)
        self.preprocessor = ClassifierPreprocessor()
        self.postprocessor = ClassifierPostprocessor()

    cls_image_shape = _forward("preprocessor", "cls_image_shape")
    cls_thresh = _forward("postprocessor", "cls_thresh")

    def predict(self, im):
        l, s = self.batch_predict([im])
        return l[0], s[0]

    def batch_predict(self, images):
        return self.postprocessor.run(self._run_net(self.preprocessor.run(images)))


# ---------------------------------------------------------------------------------- recogniser
class RecognizerPreprocessor(_NormalizeSwitches):
    def __init__(self):
        self.rec_image_shape = [3, 48, 320]
        self.mean, self.scale, self.is_scale = [0.5] * 3, [0.5] * 3, True
        self.static_shape_infer = False

    def run(self, images: Sequence[np.ndarray]) -> np.ndarray:
        import cv2
        c, H, W = self.rec_image_shape
        max_ratio = W / H
        for im in images:
            max_ratio = max(max_ratio, im.shape[1] / im.shape[0])
        bw = W if self.static_shape_infer else int(H * max_ratio)
        out = np.zeros((len(images), 3, H, bw), np.float32)
        for i, im in enumerate(images):
            ratio = im.shape[1] / im.shape[0]
            rw = bw if math.ceil(H * ratio) > bw else int(math.ceil(H * ratio))
            r = cv2.resize(im, (rw, H))
            canvas = np.full((H, bw, 3), 127, np.uint8)
            canvas[:, :rw] = r
            x = canvas.astype(np.float32)
            if self.normalize_:
                x = ((x / 255.0 if self.is_scale else x) - np.float32(self.mean)) / np.float32(self.scale)
            out[i] = x.transpose(2, 0, 1)
        return self._finish(out)


def ctc_greedy_decode(probs: np.ndarray, labels: Sequence[str]) -> Tuple[List[str], List[float]]:
    """argmax per step; emit when index > 0 and differs from the previous step; score = mean of the
    emitted maxima (rec_postprocessor.cc:46-83)."""
    p = np.asarray(probs, np.float32)
    idx = p.argmax(2)
    mx = p.max(2)
    texts, scores = [], []
    for b in range(p.shape[0]):
        last, chars, sc = 0, [], []
        for t in range(p.shape[1]):
            k = int(idx[b, t])
            if k > 0 and not (t > 0 and k == last):
                chars.append(labels[k] if k < len(labels) else "")
                sc.append(float(mx[b, t]))
            last = k
        texts.append("".join(chars))
        scores.append(float(np.mean(sc)) if sc else 0.0)
    return texts, scores


class RecognizerPostprocessor:
    def __init__(self, label_path: str = ""):
        self.label_list = ["#"]
        if label_path:
            with open(label_path, encoding="utf-8") as f:
                self.label_list += [l.rstrip("\n").rstrip("\r") for l in f]
        self.label_list.append(" ")

    def run(self, probs):
        if hasattr(probs, "is_cuda") and probs.is_cuda:
            # per-step arg-max and CTC collapse on the device; only the kept ids and scores come back
            from ...ops.postproc import ctc_greedy_decode_device, ctc_texts
            return ctc_texts(*ctc_greedy_decode_device(probs.contiguous()), self.label_list)
        if hasattr(probs, "detach"):
            probs = probs.detach().float().cpu().numpy()
        return ctc_greedy_decode(probs, self.label_list)


class Recognizer(_OcrStage):
    def __init__(self, model_file: str, params_file: str = "", label_path: str = "",
                 runtime_option: Optional[RuntimeOption] = None, model_format: ModelFormat = ModelFormat.PADDLE):
        super().__init__(model_file, params_file, runtime_option, model_format)
        self.preprocessor = RecognizerPreprocessor()
        self.postprocessor = RecognizerPostprocessor(label_path)

    rec_image_shape = _forward("preprocessor", "rec_image_shape")
    static_shape_infer = _forward("preprocessor", "static_shape_infer")

    def predict(self, im):
        t, s = self.batch_predict([im])
        return t[0], s[0]

    def batch_predict(self, images):
        x = self.preprocessor.run(images)
        outs = self.infer({self.runtime.graph.inputs[0].name: x})
        return self.postprocessor.run(outs[self.runtime.graph.outputs[0].name])


# ---------------------------------------------------------------------------------- pipelines
class PPOCRv2:
    """det -> sort -> crop -> (cls -> rotate) -> rec, with recognition batches sorted by aspect ratio."""

    def __init__(self, det_model: DBDetector, cls_model: Optional[Classifier] = None, rec_model: Optional[Recognizer] = None):
        if rec_model is None and cls_model is not None and isinstance(cls_model, Recognizer):
            cls_model, rec_model = None, cls_model
        self.detector, self.classifier, self.recognizer = det_model, cls_model, rec_model
        self.cls_batch_size = 1
        self.rec_batch_size = 6
        # on a GPU the pages stay on the device from the detector's input to the decoded text
        # (device_pipeline.DeviceOCR); set to False for the host path with OpenCV between the stages
        self.use_device_pipeline = True
        self._device_ocr = None

    def predict(self, im: np.ndarray) -> OCRResult:
        return self.batch_predict([im])[0]

    def _device_path(self, images):
        if not self.use_device_pipeline or self.recognizer is None or len(images) == 0:
            return None
        stages = [m for m in (self.detector, self.classifier, self.recognizer) if m is not None]
        if not all(getattr(m.runtime, "on_gpu", False) for m in stages):
            return None
        if len({m.runtime.device for m in stages}) != 1 or len({tuple(im.shape) for im in images}) != 1:
            return None
        if images[0].ndim != 3 or images[0].shape[2] != 3 or images[0].dtype != np.uint8:
            return None
        if self._device_ocr is None:
            from .device_pipeline import DeviceOCR
            self._device_ocr = DeviceOCR(self.detector, self.classifier, self.recognizer)
        return self._device_ocr

    def batch_predict(self, images: Sequence[np.ndarray]) -> List[OCRResult]:
        dev = self._device_path(images)
        if dev is not None:
            return dev.predict_pages(list(images))
        import cv2
        results = []
        all_boxes = self.detector.batch_predict(images)
        for im, boxes in zip(images, all_boxes):
            res = OCRResult()
            res.boxes = sort_boxes(boxes)
            crops = [get_rotate_crop_image(im, b) for b in res.boxes]
            if self.classifier is not None and crops:
                for s in range(0, len(crops), self.cls_batch_size):
                    labels, scores = self.classifier.batch_predict(crops[s:s + self.cls_batch_size])
                    res.cls_labels += labels
                    res.cls_scores += scores
                for i, (l, sc) in enumerate(zip(res.cls_labels, res.cls_scores)):
                    if l % 2 == 1 and sc > self.classifier.postprocessor.cls_thresh:
                        crops[i] = cv2.rotate(crops[i], cv2.ROTATE_180)
            if self.recognizer is not None and crops:
                order = np.argsort([c.shape[1] / c.shape[0] for c in crops], kind="stable")
                texts, scores = [""] * len(crops), [0.0] * len(crops)
                for s in range(0, len(order), self.rec_batch_size):
                    idx = order[s:s + self.rec_batch_size]
                    t, sc = self.recognizer.batch_predict([crops[i] for i in idx])
                    for k, i in enumerate(idx):
                        texts[i], scores[i] = t[k], sc[k]
                res.text, res.rec_scores = texts, scores
            results.append(res)
        return results

    def clone(self):
        return type(self)(self.detector.clone(), self.classifier.clone() if self.classifier else None,
                          self.recognizer.clone() if self.recognizer else None)


class PPOCRv3(PPOCRv2):
    def __init__(self, det_model, cls_model=None, rec_model=None):
        super().__init__(det_model, cls_model, rec_model)
        if self.recognizer is not None:
            self.recognizer.preprocessor.rec_image_shape = [3, 48, 320]


class PPOCRv4(PPOCRv3):
    pass


PPOCRSystemv2, PPOCRSystemv3, PPOCRSystemv4 = PPOCRv2, PPOCRv3, PPOCRv4


from .structure import (PPStructureV2Table, PPStructureV2TableSystem, StructureV2Layout,  # noqa: E402,F401
                        StructureV2LayoutPostprocessor, StructureV2LayoutPreprocessor, StructureV2Table,
                        StructureV2TablePostprocessor, StructureV2TablePreprocessor, build_html)
from .ser import (SERResult, StructureV2SERViLayoutXLM, StructureV2SERViLayoutXLMModel,  # noqa: E402,F401
                  StructureV2SERViLayoutXLMPostprocessor, StructureV2SERViLayoutXLMPreprocessor)
from .ser_ops import (KeepKeys, NormalizeImage, Resize, ToCHWImage, VQAReTokenChunk, VQASerTokenChunk,  # noqa: E402,F401
                      VQASerTokenLayoutLMPostProcess, VQATokenLabelEncode, VQATokenPad)

# names of the reference's Python classes for the same three objects
StructureV2SERViLayoutXLMModelPreprocessor = StructureV2SERViLayoutXLMPreprocessor
StructureV2SERViLayoutXLMModelPostprocessor = StructureV2SERViLayoutXLMPostprocessor
