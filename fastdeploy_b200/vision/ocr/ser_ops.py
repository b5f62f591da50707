"""The dictionary-in, dictionary-out operators of the layout-aware token classifier's data pipeline, under the names the
reference's Python package exports from ``fastdeploy.vision.ocr`` (python/fastdeploy/vision/ocr/ppocr/utils/
ser_vi_layoutxlm/operators.py:10-95 and vqa_utils.py:47-560). A page travels as one ``dict``: ``image`` plus the OCR
lines in ``ocr_info`` (``[{"bbox" | "points": ..., "transcription": ...}]``); every operator adds or rewrites keys.

:class:`~fastdeploy_b200.vision.ocr.ser.StructureV2SERViLayoutXLMPreprocessor` does the same work in one call and is
what the model class uses; these operators are the piecewise form for code written against the reference's pipeline."""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence

import numpy as np

from ..detection.contrib import _resize_bilinear
from .ser import StructureV2SERViLayoutXLMPostprocessor, _xyxy, load_labels, order_tb_yx


def _number(v) -> float:
    """A number, or a quotient written out as the configuration files do (``"1./255."``)."""
    if isinstance(v, str) and "/" in v:
        a, b = v.split("/", 1)
        return float(a) / float(b)
    return float(v)


class Resize:
    """``image`` to ``size`` (h, w) without keeping the aspect ratio; ``bbox`` values, when present, follow."""

    def __init__(self, size=(640, 640), **kwargs):
        self.size = tuple(size)

    def __call__(self, data: Dict[str, Any]) -> Dict[str, Any]:
        im = data["image"]
        h, w = im.shape[:2]
        data["image"] = _resize_bilinear(im, self.size[1], self.size[0])
        data["resized_shape"] = [self.size[0], self.size[1]]
        if "bbox" in data and len(data["bbox"]):
            b = np.asarray(data["bbox"], np.float32)
            b[..., 0::2] *= self.size[1] / w
            b[..., 1::2] *= self.size[0] / h
            data["bbox"] = b
        return data


class NormalizeImage:
    """``(image * scale - mean) / std`` with ``mean`` / ``std`` shaped for ``order`` ("chw" or "hwc")."""

    def __init__(self, scale=None, mean=None, std=None, order: str = "chw", **kwargs):
        self.scale = np.float32(_number(scale) if scale is not None else 1.0 / 255.0)
        shape = (3, 1, 1) if order == "chw" else (1, 1, 3)
        self.mean = np.asarray(mean if mean is not None else [0.485, 0.456, 0.406], np.float32).reshape(shape)
        self.std = np.asarray(std if std is not None else [0.229, 0.224, 0.225], np.float32).reshape(shape)

    def __call__(self, data: Dict[str, Any]) -> Dict[str, Any]:
        data["image"] = (np.asarray(data["image"], np.float32) * self.scale - self.mean) / self.std
        return data


class ToCHWImage:
    def __init__(self, **kwargs):
        pass

    def __call__(self, data: Dict[str, Any]) -> Dict[str, Any]:
        data["image"] = np.ascontiguousarray(np.asarray(data["image"]).transpose(2, 0, 1))
        return data


class KeepKeys:
    """The values of ``keep_keys``, in that order, as a list: what is handed to the network."""

    def __init__(self, keep_keys: Sequence[str], **kwargs):
        self.keep_keys = list(keep_keys)

    def __call__(self, data: Dict[str, Any]) -> List[Any]:
        return [data[k] for k in self.keep_keys]


class VQATokenLabelEncode:
    """OCR lines -> token ids with one layout box per token. Lines are put in reading order, each line's text is tokenised,
    its box (scaled to 0..1000 of the page) repeated per token, and ``segment_offset_id`` records where each line ends.
    ``tokenizer.encode(text)`` returns ids or an object with ``.ids``."""

    def __init__(self, tokenizer: Any, class_path: Optional[str] = None, contains_re: bool = False, add_special_ids: bool = False,
                 use_textline_bbox_info: bool = True, order_method: Optional[str] = "tb-yx", infer_mode: bool = True,
                 cls_id: int = 0, sep_id: int = 2, pad_id: int = 1, **kwargs):
        self.tokenizer, self.contains_re, self.add_special_ids = tokenizer, contains_re, add_special_ids
        self.order_method, self.infer_mode = order_method, infer_mode
        self.cls_id, self.sep_id, self.pad_id = cls_id, sep_id, pad_id
        self.labels = load_labels(class_path) if class_path else None

    def _ids(self, text: str) -> List[int]:
        enc = self.tokenizer.encode(text)
        ids = [int(i) for i in getattr(enc, "ids", enc)]
        if ids and ids[0] == self.cls_id:
            ids = ids[1:]
        if ids and ids[-1] == self.sep_id:
            ids = ids[:-1]
        return ids

    def __call__(self, data: Dict[str, Any]) -> Optional[Dict[str, Any]]:
        h, w = data["image"].shape[:2]
        lines = [dict(r, bbox=_xyxy(r.get("bbox", r.get("points")))) for r in data.get("ocr_info", [])
                 if r.get("transcription", r.get("text", ""))]
        if self.order_method == "tb-yx":
            lines = order_tb_yx(lines)
        ids: List[int] = []
        boxes: List[List[int]] = []
        labels: List[int] = []
        seg_end: List[int] = []
        entities: List[Dict[str, int]] = []
        for r in lines:
            x1, y1, x2, y2 = r["bbox"]
            nb = [int(np.clip(x1 * 1000.0 / w, 0, 1000)), int(np.clip(y1 * 1000.0 / h, 0, 1000)),
                  int(np.clip(x2 * 1000.0 / w, 0, 1000)), int(np.clip(y2 * 1000.0 / h, 0, 1000))]
            t = self._ids(r.get("transcription", r.get("text", "")))
            if not t:
                continue
            if not self.infer_mode and self.labels is not None:
                name = str(r.get("label", "O")).upper()
                first = self.labels.index("B-" + name) if "B-" + name in self.labels else 0
                inner = self.labels.index("I-" + name) if "I-" + name in self.labels else first
                labels += [first] + [inner] * (len(t) - 1)
            entities.append({"start": len(ids), "end": len(ids) + len(t), "label": str(r.get("label", "O")).upper()})
            ids += t
            boxes += [nb] * len(t)
            seg_end.append(len(ids))
        if self.add_special_ids:
            ids = [self.cls_id] + ids + [self.sep_id]
            boxes = [[0, 0, 0, 0]] + boxes + [[1000, 1000, 1000, 1000]]
            labels = ([-100] + labels + [-100]) if labels else labels
            seg_end = [e + 1 for e in seg_end]
            entities = [{"start": e["start"] + 1, "end": e["end"] + 1, "label": e["label"]} for e in entities]
        data.update(input_ids=ids, bbox=boxes, attention_mask=[1] * len(ids), token_type_ids=[0] * len(ids),
                    segment_offset_id=seg_end, ocr_info=lines)
        if labels:
            data["labels"] = labels
        if self.contains_re:
            data["entities"], data["relations"] = entities, list(data.get("relations", []))
        return data


class VQATokenPad:
    """Pads (``pad_to_max_seq_len``) or truncates the token-level lists to ``max_seq_len`` and turns them into int64 arrays."""

    def __init__(self, max_seq_len: int = 512, pad_to_max_seq_len: bool = True, return_attention_mask: bool = True,
                 return_token_type_ids: bool = True, truncation_strategy: str = "longest_first", return_overflowing_tokens: bool = False,
                 return_special_tokens_mask: bool = False, infer_mode: bool = True, pad_token_id: int = 1, **kwargs):
        self.max_seq_len, self.pad_to_max_seq_len, self.pad_token_id = int(max_seq_len), pad_to_max_seq_len, pad_token_id
        self.return_attention_mask, self.return_token_type_ids, self.infer_mode = return_attention_mask, return_token_type_ids, infer_mode

    def __call__(self, data: Dict[str, Any]) -> Dict[str, Any]:
        n = len(data["input_ids"])
        fill = {"input_ids": self.pad_token_id, "attention_mask": 0, "token_type_ids": 0, "labels": -100}
        for key in ("input_ids", "attention_mask", "token_type_ids", "labels"):
            if key not in data:
                continue
            v = list(data[key])
            if self.pad_to_max_seq_len and n < self.max_seq_len:
                v += [fill[key]] * (self.max_seq_len - n)
            data[key] = np.asarray(v, np.int64)
        b = [list(x) for x in data["bbox"]]
        if self.pad_to_max_seq_len and n < self.max_seq_len:
            b += [[0, 0, 0, 0]] * (self.max_seq_len - n)
        data["bbox"] = np.asarray(b, np.int64).reshape(-1, 4)
        if not self.return_attention_mask:
            data.pop("attention_mask", None)
        if not self.return_token_type_ids:
            data.pop("token_type_ids", None)
        return data


_TOKEN_KEYS = ("input_ids", "attention_mask", "token_type_ids", "bbox", "labels")


class VQASerTokenChunk:
    """Cuts the token-level arrays into windows of ``max_seq_len``; in ``infer_mode`` all windows come back stacked (one
    row per window), otherwise the first one (the training pipeline samples one window per page)."""

    def __init__(self, max_seq_len: int = 512, infer_mode: bool = True, **kwargs):
        self.max_seq_len, self.infer_mode = int(max_seq_len), infer_mode

    def __call__(self, data: Dict[str, Any]) -> Dict[str, Any]:
        n = len(data["input_ids"])
        windows = []
        for at in range(0, max(n, 1), self.max_seq_len):
            windows.append({k: np.asarray(data[k])[at:at + self.max_seq_len] for k in _TOKEN_KEYS if k in data})
        if not self.infer_mode:
            data.update(windows[0])
            return data
        last = windows[-1]
        short = self.max_seq_len - len(last["input_ids"])
        if len(windows) > 1 and short > 0:                   # the tail window is padded so that the windows stack
            for k, v in last.items():
                pad = np.zeros((short,) + v.shape[1:], v.dtype)
                if k == "labels":
                    pad -= 100
                last[k] = np.concatenate([v, pad])
        for k in windows[0]:
            data[k] = np.stack([w[k] for w in windows])
        return data


class VQAReTokenChunk:
    """The relation-extraction form of the cut: the first window of ``max_seq_len`` tokens, with the entities that lie
    wholly inside it (renumbered) and the relations whose two ends survived."""

    def __init__(self, max_seq_len: int = 512, entities_labels: Optional[Dict[str, int]] = None, infer_mode: bool = True, **kwargs):
        self.max_seq_len, self.infer_mode = int(max_seq_len), infer_mode
        self.entities_labels = entities_labels or {"HEADER": 0, "QUESTION": 1, "ANSWER": 2}

    def __call__(self, data: Dict[str, Any]) -> Dict[str, Any]:
        for k in _TOKEN_KEYS:
            if k in data:
                data[k] = np.asarray(data[k])[:self.max_seq_len]
        kept: Dict[int, int] = {}
        entities = []
        for i, e in enumerate(data.get("entities", [])):
            if e["end"] <= self.max_seq_len:
                kept[i] = len(entities)
                label = e["label"]
                entities.append({"start": e["start"], "end": e["end"], "label": self.entities_labels.get(label, label)})
        relations = [{"head": kept[r["head"]], "tail": kept[r["tail"]]} for r in data.get("relations", [])
                     if r["head"] in kept and r["tail"] in kept]
        data["entities"] = {"start": [e["start"] for e in entities], "end": [e["end"] for e in entities],
                            "label": [e["label"] for e in entities]}
        data["relations"] = {"head": [r["head"] for r in relations], "tail": [r["tail"] for r in relations]}
        return data


class VQASerTokenLayoutLMPostProcess:
    """Token logits -> one class per OCR line by majority vote over the line's tokens
    (vqa_utils.py:491-560). ``preds`` is ``[windows, max_seq_len, classes]``; ``segment_offset_ids`` and ``ocr_infos``
    are the lists the encoder produced for each page."""

    def __init__(self, class_path: Optional[str] = None, labels: Optional[Sequence[str]] = None, **kwargs):
        self._post = StructureV2SERViLayoutXLMPostprocessor(class_path, labels)
        self.id2label_map_for_show = dict(enumerate(self._post.draw_names))

    def __call__(self, preds, batch=None, segment_offset_ids=None, ocr_infos=None, special_ids: bool = False, **kwargs):
        preds = np.asarray(preds[0] if isinstance(preds, (tuple, list)) else preds, np.float32)
        if preds.ndim == 2:
            preds = preds[None]
        results = []
        for seg, lines in zip(segment_offset_ids, ocr_infos):
            windows, length = preds.shape[0], preds.shape[1]
            body = length - 2 if special_ids else length
            logits = preds if special_ids else np.pad(preds, ((0, 0), (1, 1), (0, 0)))       # the vote skips one slot per end
            seg = [s - (1 if special_ids else 0) for s in seg] if special_ids else list(seg)
            res = self._post.run(logits, {"body": body, "ocr_info": [dict(r, bbox=_xyxy(r.get("bbox", r.get("points")))) for r in lines],
                                          "segment_offset_id": seg})
            out = []
            for r, pid, name in zip(lines, res.pred_id, res.pred):
                out.append(dict(r, pred_id=pid, pred=name))
            results.append(out)
            del windows
        return results
