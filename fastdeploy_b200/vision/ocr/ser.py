"""PP-StructureV2 semantic entity recognition with a visual-feature-independent LayoutXLM
(fastdeploy/vision/ocr/ppocr/structurev2_ser_vi_layoutxlm.cc and the Python wrapper
python/fastdeploy/vision/ocr/ppocr/__init__.py:1142-1345).

The network takes four token-level inputs, ``input_ids``, ``bbox``, ``attention_mask``, ``token_type_ids``
(each ``[B, 512]``, ``bbox`` ``[B, 512, 4]``), and returns per-token class logits. Around it:

* text lines come from an OCR pass (``PPOCRv3`` of this package, or lines the caller already has);
* lines are put in reading order (top to bottom, then left to right for lines less than 20 px apart);
* every line is tokenised, each token inherits the line's box scaled to the 0..1000 grid, ``[CLS]``/``[SEP]``
  get the boxes ``[0, 0, 0, 0]`` / ``[1000, 1000, 1000, 1000]``, and the page is cut into windows of 512 tokens;
* per line, the majority class of its tokens (``I-x`` counted as ``B-x``) is the line's entity label.

The reference delegates all of this to the ``paddleocr`` package; here it is written out, so the class runs
with the tokenizer of this package (or any object with ``encode(text) -> ids``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence

import numpy as np

from ...core.types import ModelFormat
from ...runtime.model import FastDeployModel
from ...runtime.option import RuntimeOption


@dataclass
class SERResult:
    """One entry per OCR line: its box ``[x1, y1, x2, y2]``, text, entity label and label id."""
    boxes: List[List[int]] = field(default_factory=list)
    text: List[str] = field(default_factory=list)
    pred: List[str] = field(default_factory=list)
    pred_id: List[int] = field(default_factory=list)

    def __str__(self) -> str:
        return "\n".join(f"{b} {t!r}: {p}" for b, t, p in zip(self.boxes, self.text, self.pred))


def load_labels(class_path: str) -> List[str]:
    """``O`` plus ``B-x`` / ``I-x`` for every class name in the file (one per line, ``OTHER`` is ``O``)."""
    with open(class_path, encoding="utf-8") as f:
        names = [ln.strip() for ln in f if ln.strip()]
    labels = ["O"]
    for n in names:
        if n.upper() in ("O", "OTHER", "OTHERS", "IGNORE"):
            continue
        labels += ["B-" + n.upper(), "I-" + n.upper()]
    return labels


def order_tb_yx(lines: Sequence[Dict[str, Any]]) -> List[Dict[str, Any]]:
    """Reading order: by top edge, then lines whose tops are within 20 px are swapped into left-to-right order."""
    out = sorted(lines, key=lambda r: (r["bbox"][1], r["bbox"][0]))
    for i in range(len(out) - 1):
        for j in range(i, -1, -1):
            a, b = out[j], out[j + 1]
            if abs(b["bbox"][1] - a["bbox"][1]) < 20 and b["bbox"][0] < a["bbox"][0]:
                out[j], out[j + 1] = b, a
            else:
                break
    return out


def _xyxy(box: Sequence[float]) -> List[int]:
    b = np.asarray(box, np.float32).reshape(-1)
    if b.size == 4:
        return [int(b[0]), int(b[1]), int(b[2]), int(b[3])]
    xs, ys = b[0::2], b[1::2]
    return [int(xs.min()), int(ys.min()), int(xs.max()), int(ys.max())]


class StructureV2SERViLayoutXLMPreprocessor:
    """OCR lines -> windows of ``max_seq_len`` tokens. ``tokenizer.encode(text)`` may return a list of ids or an
    object with ``.ids``; ids equal to ``cls_id`` / ``sep_id`` at the ends are dropped (they are added once per
    window here)."""

    def __init__(self, tokenizer: Any, max_seq_len: int = 512, cls_id: int = 0, sep_id: int = 2, pad_id: int = 1):
        self.tokenizer, self.max_seq_len = tokenizer, int(max_seq_len)
        self.cls_id, self.sep_id, self.pad_id = cls_id, sep_id, pad_id

    def _ids(self, text: str) -> List[int]:
        enc = self.tokenizer.encode(text)
        ids = list(getattr(enc, "ids", enc))
        if ids and ids[0] == self.cls_id:
            ids = ids[1:]
        if ids and ids[-1] == self.sep_id:
            ids = ids[:-1]
        return [int(i) for i in ids]

    def run(self, lines: Sequence[Dict[str, Any]], height: int, width: int) -> Dict[str, Any]:
        lines = order_tb_yx([dict(r, bbox=_xyxy(r["bbox"] if "bbox" in r else r["points"])) for r in lines])
        ids: List[int] = []
        boxes: List[List[int]] = []
        seg_end: List[int] = []
        for r in lines:
            x1, y1, x2, y2 = r["bbox"]
            nb = [int(np.clip(x1 * 1000.0 / width, 0, 1000)), int(np.clip(y1 * 1000.0 / height, 0, 1000)),
                  int(np.clip(x2 * 1000.0 / width, 0, 1000)), int(np.clip(y2 * 1000.0 / height, 0, 1000))]
            t = self._ids(r.get("transcription", r.get("text", "")))
            ids += t
            boxes += [nb] * len(t)
            seg_end.append(len(ids))
        body = self.max_seq_len - 2
        n_win = max(1, (len(ids) + body - 1) // body)
        input_ids = np.full((n_win, self.max_seq_len), self.pad_id, np.int64)
        bbox = np.zeros((n_win, self.max_seq_len, 4), np.int64)
        mask = np.zeros((n_win, self.max_seq_len), np.int64)
        for w in range(n_win):
            part = ids[w * body:(w + 1) * body]
            n = len(part)
            input_ids[w, 0] = self.cls_id
            input_ids[w, 1:1 + n] = part
            input_ids[w, 1 + n] = self.sep_id
            bbox[w, 1:1 + n] = boxes[w * body:(w + 1) * body] if n else 0
            bbox[w, 1 + n] = 1000
            mask[w, :n + 2] = 1
        return {"input_ids": input_ids, "bbox": bbox, "attention_mask": mask,
                "token_type_ids": np.zeros_like(input_ids), "segment_offset_id": seg_end, "ocr_info": lines,
                "body": body}


class StructureV2SERViLayoutXLMPostprocessor:
    def __init__(self, class_path: Optional[str] = None, labels: Optional[Sequence[str]] = None):
        self.labels = list(labels) if labels is not None else load_labels(class_path)
        # for the line-level vote I-x counts as B-x; the vote's classes are O and the entity names
        self.draw_names = ["O"] + sorted({l[2:] for l in self.labels if l != "O"}, key=lambda n: self.labels.index("B-" + n))
        self.to_draw = [0 if l == "O" else self.draw_names.index(l[2:]) for l in self.labels]

    def run(self, logits: np.ndarray, batch: Dict[str, Any]) -> SERResult:
        """``logits`` ``[windows, max_seq_len, classes]`` of ONE page as cut by the preprocessor."""
        body = batch["body"]
        cls = np.argmax(np.asarray(logits, np.float32), axis=-1)               # [W, L]
        flat = cls[:, 1:1 + body].reshape(-1)                                    # token i of the page at flat[i]
        to_draw = np.asarray(self.to_draw)
        res = SERResult()
        start = 0
        for r, end in zip(batch["ocr_info"], batch["segment_offset_id"]):
            votes = to_draw[flat[start:end]] if end > start else np.zeros(0, np.int64)
            pid = int(np.argmax(np.bincount(votes, minlength=len(self.draw_names)))) if votes.size else 0
            res.boxes.append(list(r["bbox"]))
            res.text.append(r.get("transcription", r.get("text", "")))
            res.pred_id.append(pid)
            res.pred.append(self.draw_names[pid])
            start = end
        return res


class StructureV2SERViLayoutXLM(FastDeployModel):
    """``predict(image)`` runs the OCR pipeline given as ``ocr`` for the lines; ``predict(image, lines)`` takes
    ``[{"bbox": [x1, y1, x2, y2] | 8 numbers, "transcription": str}, ...]`` from the caller."""

    def __init__(self, model_file: str, params_file: str = "", class_path: Optional[str] = None, *,
                 tokenizer: Any = None, ocr: Any = None, labels: Optional[Sequence[str]] = None,
                 runtime_option: Optional[RuntimeOption] = None, model_format: int = ModelFormat.PADDLE,
                 max_seq_len: int = 512):
        super().__init__(runtime_option)
        if tokenizer is None:
            raise ValueError("StructureV2SERViLayoutXLM needs a tokenizer (an object with encode(text) -> ids)")
        self.runtime_option.set_model_path(model_file, params_file, model_format)
        self.preprocessor = StructureV2SERViLayoutXLMPreprocessor(tokenizer, max_seq_len)
        self.postprocessor = StructureV2SERViLayoutXLMPostprocessor(class_path, labels)
        self.ocr = ocr
        self.init_runtime()

    def model_name(self) -> str:
        return "ppocr/structurev2_ser_vi_layoutxlm"

    def _lines(self, im: np.ndarray) -> List[Dict[str, Any]]:
        if self.ocr is None:
            raise ValueError("no OCR pipeline was given: pass the text lines to predict()")
        r = self.ocr.predict(im)
        return [{"bbox": b, "transcription": t} for b, t in zip(r.boxes, r.text)]

    def predict(self, im: np.ndarray, lines: Optional[Sequence[Dict[str, Any]]] = None) -> SERResult:
        return self.batch_predict([im], None if lines is None else [lines])[0]

    def batch_predict(self, images: Sequence[np.ndarray],
                      lines: Optional[Sequence[Sequence[Dict[str, Any]]]] = None) -> List[SERResult]:
        batches = []
        for i, im in enumerate(images):
            ls = lines[i] if lines is not None else self._lines(im)
            batches.append(self.preprocessor.run(ls, im.shape[0], im.shape[1]))
        names = [self.runtime.get_input_info(i).name for i in range(self.runtime.num_inputs())]
        by_key = {"input_ids": None, "bbox": None, "attention_mask": None, "token_type_ids": None}
        for key in by_key:
            by_key[key] = np.concatenate([b[key] for b in batches], axis=0)
        # inputs are matched by name where the graph uses these names, else in the reference's order
        order = ["input_ids", "bbox", "attention_mask", "token_type_ids"]
        feeds = {n: by_key[n] if n in by_key else by_key[order[i]] for i, n in enumerate(names)}
        logits = np.asarray(self.runtime.infer(feeds)[0], np.float32)
        out, at = [], 0
        for b in batches:
            w = b["input_ids"].shape[0]
            out.append(self.postprocessor.run(logits[at:at + w], b))
            at += w
        return out


class StructureV2SERViLayoutXLMModel(StructureV2SERViLayoutXLM):
    """The same model under the reference's class name and constructor order
    (python/fastdeploy/vision/ocr/ppocr/__init__.py:1241-1300): ``(model_file, params_file, ser_dict_path, class_path,
    config_file, runtime_option, model_format)``. The reference builds its tokenizer and its OCR engine from external
    packages; here they are arguments: ``tokenizer`` (any object with ``encode(text)``), or a SentencePiece model file
    named ``sentencepiece.bpe.model`` beside the model file, read in the XLM-R convention; ``ocr`` is a PP-OCR pipeline
    for ``predict(image)`` without lines (``ser_dict_path`` is the recogniser dictionary the reference hands to its own
    engine and is kept on the object)."""

    def __init__(self, model_file: str, params_file: str = "", ser_dict_path: str = "", class_path: Optional[str] = None,
                 config_file: str = "", runtime_option: Optional[RuntimeOption] = None, model_format: int = ModelFormat.PADDLE,
                 *, tokenizer: Any = None, ocr: Any = None, labels: Optional[Sequence[str]] = None, max_seq_len: int = 512):
        import os
        if tokenizer is None:
            spm_file = os.path.join(os.path.dirname(os.path.abspath(model_file)), "sentencepiece.bpe.model")
            if not os.path.exists(spm_file):
                raise ValueError(f"no tokenizer given and {spm_file} does not exist")
            from ...text.spm_tokenizer import XLMRobertaTokenizer
            tokenizer = XLMRobertaTokenizer(spm_file, max_seq_len)
        self.ser_dict_path, self.config_file = ser_dict_path, config_file
        super().__init__(model_file, params_file, class_path, tokenizer=tokenizer, ocr=ocr, labels=labels,
                         runtime_option=runtime_option, model_format=model_format, max_seq_len=max_seq_len)

    @property
    def postprocesser(self):                # the reference's spelling of the attribute
        return self.postprocessor
