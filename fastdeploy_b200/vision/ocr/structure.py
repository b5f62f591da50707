"""PP-StructureV2: table structure recognition and layout analysis
(fastdeploy/vision/ocr/ppocr/structurev2_table.cc + structurev2_table_{pre,post}processor.cc,
structurev2_layout.cc + structurev2_layout_postprocessor.cc, ppstructurev2_table.cc, utils/matcher.cc).

* Table: resize so that the long side is ``max_len`` (488), normalise, zero-pad bottom / right to a
  square; outputs are box regressions ``[B, T, 4 | 8]`` (normalised) and structure-token probabilities
  ``[B, T, V]``. Decoding walks the tokens by arg-max until ``eos``, skips ``beg`` / ``end``, and emits a
  box for every cell token (``<td>``, ``<td``, ``<td></td>``), scaled by the source width and height.
* Layout: PicoDet-style GFL head on strides 8/16/32/64 with ``reg_max = 8``: integral regression of the
  four distances, per-class hard NMS.
* ``PPStructureV2Table``: detector + recogniser for the cell texts, the table model for the structure,
  then each OCR box is matched to the cell with the smallest (IoU distance, corner distance) and the
  texts are spliced into the ``<td>`` tokens to give HTML.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np

from ...core.types import ModelFormat
from ...runtime.model import FastDeployModel
from ...runtime.option import RuntimeOption
from .. import utils as vutils
from ..detection.contrib import _resize_bilinear
from ..result import DetectionResult, OCRResult

TD_TOKENS = ("<td>", "<td", "<td></td>")


class StructureV2TablePreprocessor:
    def __init__(self):
        self.max_len = 488
        self.mean, self.std = [0.485, 0.456, 0.406], [0.229, 0.224, 0.225]
        self.batch_det_img_info: List[Tuple[int, int, int, int]] = []

    def run(self, images: Sequence[np.ndarray]) -> np.ndarray:
        out = []
        self.batch_det_img_info = []
        for im in images:
            h, w = im.shape[:2]
            ratio = self.max_len / float(max(h, w))
            rh, rw = int(h * ratio), int(w * ratio)
            x = _resize_bilinear(im, rw, rh).astype(np.float32) / 255.0
            x = (x - np.asarray(self.mean, np.float32)) / np.asarray(self.std, np.float32)
            canvas = np.zeros((self.max_len, self.max_len, 3), np.float32)
            canvas[:rh, :rw] = x
            out.append(np.ascontiguousarray(canvas.transpose(2, 0, 1)))
            self.batch_det_img_info.append((w, h, rw, rh))
        return np.stack(out)


class StructureV2TablePostprocessor:
    def __init__(self, dict_path: str, merge_no_span_structure: bool = True):
        with open(dict_path, encoding="utf-8") as f:
            chars = ["sos"] + [l.rstrip("\r\n") for l in f]
        if merge_no_span_structure:
            if "<td></td>" not in chars:
                chars.append("<td></td>")
            chars = [c for c in chars if c != "<td>"]
        chars.append("eos")
        self.dict_character = chars
        self.ignore_beg = chars.index("beg") if "beg" in chars else -1
        self.ignore_end = chars.index("end") if "end" in chars else -1
        self.dict_end_idx = len(chars) - 1

    def run(self, bbox_preds: np.ndarray, structure_probs: np.ndarray, img_info: Sequence[Tuple[int, int, int, int]]):
        boxes_all, tokens_all = [], []
        for b in range(structure_probs.shape[0]):
            w, h, rw, rh = img_info[b]
            boxes, toks = [], ["<html>", "<body>", "<table>"]
            for i in range(structure_probs.shape[1]):
                idx = int(structure_probs[b, i].argmax())
                if idx > 0 and idx == self.dict_end_idx:
                    break
                if idx in (self.ignore_beg, self.ignore_end):
                    continue
                text = self.dict_character[idx]
                if text in TD_TOKENS:
                    p = bbox_preds[b, i]
                    if p.shape[0] == 4:
                        q = [p[0], p[1], p[2], p[1], p[2], p[3], p[0], p[3]]
                    else:
                        q = list(p[:8])
                    # the regression is normalised by the source size (postprocessor.cc:92-113)
                    boxes.append([int(v * (w if k % 2 == 0 else h)) for k, v in enumerate(q)])
                toks.append(text)
            toks += ["</table>", "</body>", "</html>"]
            boxes_all.append(boxes)
            tokens_all.append(toks)
        return boxes_all, tokens_all


class StructureV2Table(FastDeployModel):
    def __init__(self, model_file: str, params_file: str, table_char_dict_path: str,
                 runtime_option: Optional[RuntimeOption] = None, model_format: int = ModelFormat.PADDLE):
        super().__init__(runtime_option)
        self.runtime_option.set_model_path(model_file, params_file, model_format)
        self.preprocessor = StructureV2TablePreprocessor()
        self.postprocessor = StructureV2TablePostprocessor(table_char_dict_path)
        self.init_runtime()

    def batch_predict(self, images: Sequence[np.ndarray]):
        x = self.preprocessor.run(images)
        outs = [np.asarray(o, np.float32) for o in self.runtime.infer({self.runtime.get_input_info(0).name: x})]
        return self.postprocessor.run(outs[0], outs[1], self.preprocessor.batch_det_img_info)

    def predict(self, im: np.ndarray) -> OCRResult:
        boxes, toks = self.batch_predict([im])
        r = OCRResult()
        r.table_boxes = boxes[0]
        r.table_structure = toks[0]
        return r


class StructureV2LayoutPostprocessor:
    def __init__(self):
        self.score_threshold, self.nms_threshold = 0.4, 0.5
        self.num_class, self.reg_max = 5, 8
        self.fpn_stride = [8, 16, 32, 64]

    def run(self, outs: Sequence[np.ndarray], img_info: Tuple[int, int, int, int]) -> DetectionResult:
        """``outs``: per stride a score map ``[1, A, num_class]`` followed by per stride a regression map
        ``[1, A, 4 * reg_max]``; ``img_info = (src_w, src_h, in_w, in_h)``."""
        w, h, in_w, in_h = img_info
        n = len(self.fpn_stride)
        res = DetectionResult()
        for s_idx, stride in enumerate(self.fpn_stride):
            score = np.asarray(outs[s_idx], np.float32).reshape(-1, self.num_class)
            reg = np.asarray(outs[s_idx + n], np.float32).reshape(-1, 4, self.reg_max)
            fw = int(np.ceil(in_w / stride))
            labels = score.argmax(1)
            conf = score[np.arange(len(score)), labels]
            keep = np.nonzero(conf > self.score_threshold)[0]
            if not len(keep):
                continue
            e = np.exp(reg[keep] - reg[keep].max(-1, keepdims=True))
            dist = (e / e.sum(-1, keepdims=True) * np.arange(self.reg_max)).sum(-1) * stride
            cx = (keep % fw + 0.5) * stride
            cy = (keep // fw + 0.5) * stride
            x1 = np.clip(cx - dist[:, 0], 0, in_w) * (w / in_w)
            y1 = np.clip(cy - dist[:, 1], 0, in_h) * (h / in_h)
            x2 = np.clip(cx + dist[:, 2], 0, in_w) * (w / in_w)
            y2 = np.clip(cy + dist[:, 3], 0, in_h) * (h / in_h)
            for k in range(len(keep)):
                res.boxes.append([float(x1[k]), float(y1[k]), float(x2[k]), float(y2[k])])
                res.scores.append(float(conf[keep[k]]))
                res.label_ids.append(int(labels[keep[k]]))
        # per-class hard NMS
        out = DetectionResult()
        for c in sorted(set(res.label_ids)):
            sub = DetectionResult()
            for b, s, l in zip(res.boxes, res.scores, res.label_ids):
                if l == c:
                    sub.boxes.append(b); sub.scores.append(s); sub.label_ids.append(l)
            vutils.nms(sub, self.nms_threshold)
            out.boxes += sub.boxes; out.scores += sub.scores; out.label_ids += sub.label_ids
        return out


class StructureV2LayoutPreprocessor:
    """Resize to 608 x 800 (w x h), BGR->RGB, ImageNet mean / std, CHW; remembers (w, h, resized w, resized h) per image
    for the post-processor (fastdeploy/vision/ocr/ppocr/structurev2_layout_preprocessor.cc:25-90)."""

    def __init__(self):
        self.size = [608, 800]      # w, h
        self.mean, self.std = [0.485, 0.456, 0.406], [0.229, 0.224, 0.225]
        self.batch_layout_img_info: List[Tuple[int, int, int, int]] = []

    def run(self, images: Sequence[np.ndarray]) -> np.ndarray:
        out, self.batch_layout_img_info = [], []
        for im in images:
            h, w = im.shape[:2]
            x = _resize_bilinear(im, *self.size)[..., ::-1].astype(np.float32) / 255.0
            x = (x - np.asarray(self.mean, np.float32)) / np.asarray(self.std, np.float32)
            out.append(np.ascontiguousarray(x.transpose(2, 0, 1)))
            self.batch_layout_img_info.append((w, h, self.size[0], self.size[1]))
        return np.stack(out)


class StructureV2Layout(FastDeployModel):
    def __init__(self, model_file: str, params_file: str = "", runtime_option: Optional[RuntimeOption] = None,
                 model_format: int = ModelFormat.PADDLE):
        super().__init__(runtime_option)
        self.runtime_option.set_model_path(model_file, params_file, model_format)
        self.preprocessor = StructureV2LayoutPreprocessor()
        self.postprocessor = StructureV2LayoutPostprocessor()
        self.init_runtime()

    @property
    def size(self):
        return self.preprocessor.size

    @size.setter
    def size(self, v):
        self.preprocessor.size = list(v)

    def batch_predict(self, images: Sequence[np.ndarray]) -> List[DetectionResult]:
        x = self.preprocessor.run(images)
        outs = [np.asarray(o, np.float32) for o in self.runtime.infer({self.runtime.get_input_info(0).name: x})]
        return [self.postprocessor.run([o[i:i + 1] for o in outs], info)
                for i, info in enumerate(self.preprocessor.batch_layout_img_info)]

    def predict(self, im: np.ndarray) -> DetectionResult:
        return self.batch_predict([im])[0]


def _box_distance(ocr_box: Sequence[float], cell: Sequence[float]) -> Tuple[float, float]:
    """(1 - IoU, corner distance) between an OCR box and a table cell, both ``[x1, y1, x2, y2]`` (matcher.cc)."""
    x1, y1, x2, y2 = ocr_box
    a1, b1, a2, b2 = cell
    dis = abs(a1 - x1) + abs(b1 - y1) + abs(a2 - x2) + abs(b2 - y2)
    dis2 = abs(a1 - x1) + abs(b1 - y1)
    dis3 = abs(a2 - x2) + abs(b2 - y2)
    ix1, iy1, ix2, iy2 = max(x1, a1), max(y1, b1), min(x2, a2), min(y2, b2)
    inter = max(ix2 - ix1, 0) * max(iy2 - iy1, 0)
    union = (x2 - x1) * (y2 - y1) + (a2 - a1) * (b2 - b1) - inter
    iou = inter / union if union > 0 else 0.0
    return 1.0 - iou, dis + min(dis2, dis3)


def _xyxy(poly: Sequence[float]) -> List[float]:
    xs, ys = poly[0::2], poly[1::2]
    return [min(xs), min(ys), max(xs), max(ys)]


def build_html(structure: Sequence[str], cell_boxes: Sequence[Sequence[float]], ocr_boxes: Sequence[Sequence[float]],
               texts: Sequence[str]) -> str:
    cells = [_xyxy(c) for c in cell_boxes]
    matched: Dict[int, List[int]] = {}
    for i, ob in enumerate(ocr_boxes):
        if not cells:
            break
        d = [_box_distance(_xyxy(ob), c) for c in cells]
        j = min(range(len(cells)), key=lambda k: (d[k][0], d[k][1]))
        matched.setdefault(j, []).append(i)
    html, td = [], 0
    for tok in structure:
        if "</td>" in tok:
            if tok == "<td></td>":
                html.append("<td>")
            content = "".join(texts[i] for i in matched.get(td, []))
            html.append(content)
            html.append("</td>" if tok == "<td></td>" else tok)
            td += 1
        else:
            html.append(tok)
    return "".join(html)


class PPStructureV2Table:
    def __init__(self, det_model: Any, rec_model: Any, table_model: StructureV2Table):
        self.detector, self.recognizer, self.table = det_model, rec_model, table_model

    def predict(self, im: np.ndarray) -> OCRResult:
        from . import PPOCRv3
        ocr = PPOCRv3(self.detector, None, self.recognizer).predict(im)
        t = self.table.predict(im)
        ocr.table_boxes, ocr.table_structure = t.table_boxes, t.table_structure
        ocr.table_html = build_html(t.table_structure, t.table_boxes, ocr.boxes, ocr.text)
        return ocr

    def batch_predict(self, images: Sequence[np.ndarray]) -> List[OCRResult]:
        return [self.predict(im) for im in images]

    def clone(self) -> "PPStructureV2Table":
        """A second pipeline over clones of the three models (they share weights, not buffers)."""
        return PPStructureV2Table(self.detector.clone(), self.recognizer.clone(), self.table.clone())


PPStructureV2TableSystem = PPStructureV2Table
