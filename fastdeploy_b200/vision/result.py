"""Result types of the vision API with the reference's fields and ``Str()`` formats
(fastdeploy/vision/common/result.h:24-433, result.cc)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import numpy as np


def _f(v: float) -> str:
    return f"{v:.6f}"


class _Base:
    def Str(self) -> str:
        return self.__str__()

    def clear(self) -> None:
        for k, v in self.__dict__.items():
            if isinstance(v, list):
                v.clear()

    Clear = clear
    Free = clear


@dataclass
class ClassifyResult(_Base):
    label_ids: List[int] = field(default_factory=list)
    scores: List[float] = field(default_factory=list)
    feature: List[float] = field(default_factory=list)

    def __str__(self) -> str:
        out = "ClassifyResult(\nlabel_ids: " + "".join(f"{i}, " for i in self.label_ids)
        out += "\nscores: " + "".join(f"{_f(s)}, " for s in self.scores)
        if self.feature:
            out += f"\nfeature: size ({len(self.feature)}), only show first 100 values.\n"
            for i, v in enumerate(self.feature[:100]):
                out += f"{_f(v)}, "
                if (i + 1) % 10 == 0 and (i + 1) < 100:
                    out += "\n"
                if i + 1 == 100:
                    out += "\n......"
        return out + "\n)"


@dataclass
class Mask(_Base):
    data: List[int] = field(default_factory=list)
    shape: List[int] = field(default_factory=list)

    def __str__(self) -> str:
        return "Mask(" + ",".join(str(s) for s in self.shape) + ")\n"


@dataclass
class DetectionResult(_Base):
    boxes: List[List[float]] = field(default_factory=list)
    rotated_boxes: List[List[float]] = field(default_factory=list)
    scores: List[float] = field(default_factory=list)
    label_ids: List[int] = field(default_factory=list)
    masks: List[Mask] = field(default_factory=list)
    contain_masks: bool = False

    def __str__(self) -> str:
        rot = bool(self.rotated_boxes)
        head = "x1, y1, x2, y2, x3, y3, x4, y4" if rot else "xmin, ymin, xmax, ymax"
        out = f"DetectionResult: [{head}, score, label_id" + (", mask_shape]\n" if self.contain_masks else "]\n")
        rows = self.rotated_boxes if rot else self.boxes
        for i, b in enumerate(rows):
            out += ",".join(_f(v) for v in b) + f", {_f(self.scores[i])}, {self.label_ids[i]}"
            if self.contain_masks:
                out += ", " + str(self.masks[i])
            else:
                out += "\n"
        return out

    def reserve(self, n: int) -> None:
        pass

    def resize(self, n: int) -> None:
        self.boxes = [[0.0] * 4 for _ in range(n)]
        self.scores = [0.0] * n
        self.label_ids = [0] * n


@dataclass
class PerceptionResult(_Base):
    scores: List[float] = field(default_factory=list)
    label_ids: List[int] = field(default_factory=list)
    boxes: List[List[float]] = field(default_factory=list)          # 7 values
    center: List[List[float]] = field(default_factory=list)
    observation_angle: List[float] = field(default_factory=list)
    yaw_angle: List[float] = field(default_factory=list)
    velocity: List[List[float]] = field(default_factory=list)
    valid: List[bool] = field(default_factory=list)

    def __str__(self) -> str:
        out = "PerceptionResult: ["
        keys = ["xmin, ymin, xmax, ymax, w, h, l,", "cx, cy, cz,", "yaw_angle,", "ob_angle,", "score,", "label_id"]
        out += " ".join(keys) + "]\n"
        for i in range(len(self.label_ids)):
            parts = []
            if i < len(self.boxes): parts += [_f(v) for v in self.boxes[i]]
            if i < len(self.center): parts += [_f(v) for v in self.center[i]]
            if i < len(self.yaw_angle): parts.append(_f(self.yaw_angle[i]))
            if i < len(self.observation_angle): parts.append(_f(self.observation_angle[i]))
            if i < len(self.scores): parts.append(_f(self.scores[i]))
            parts.append(str(self.label_ids[i]))
            out += ", ".join(parts) + "\n"
        return out


@dataclass
class KeyPointDetectionResult(_Base):
    keypoints: List[List[float]] = field(default_factory=list)
    scores: List[float] = field(default_factory=list)
    num_joints: int = -1

    def __str__(self) -> str:
        out = f"KeyPointDetectionResult: [x, y, conf]\nnum_joints:{self.num_joints}\n"
        for k, s in zip(self.keypoints, self.scores):
            out += f"{_f(k[0])},{_f(k[1])}, {_f(s)}\n"
        return out + "\n"


@dataclass
class OCRResult(_Base):
    boxes: List[List[int]] = field(default_factory=list)           # 8 ints per box
    text: List[str] = field(default_factory=list)
    rec_scores: List[float] = field(default_factory=list)
    cls_scores: List[float] = field(default_factory=list)
    cls_labels: List[int] = field(default_factory=list)
    table_boxes: List[List[int]] = field(default_factory=list)
    table_structure: List[str] = field(default_factory=list)
    table_html: str = ""

    def __str__(self) -> str:
        out = ""
        if self.boxes:
            for n, b in enumerate(self.boxes):
                out += "det boxes: [" + ",".join(f"[{b[2 * i]},{b[2 * i + 1]}]" for i in range(4)) + "]"
                if self.rec_scores:
                    out += f"rec text: {self.text[n]} rec score:{_f(self.rec_scores[n])} "
                if self.cls_labels:
                    out += f"cls label: {self.cls_labels[n]} cls score: {_f(self.cls_scores[n])}"
                out += "\n"
            if self.table_boxes:
                for b in self.table_boxes:
                    out += "table boxes: [" + ",".join(f"[{b[2 * i]},{b[2 * i + 1]}]" for i in range(len(b) // 2)) + "]\n"
                out += "\ntable structure: \n" + "".join(self.table_structure)
            if self.table_html:
                out += "\n" + "table html: \n" + self.table_html
            return out
        if self.rec_scores and self.cls_scores:
            for i in range(len(self.rec_scores)):
                out += f"rec text: {self.text[i]} rec score:{_f(self.rec_scores[i])} "
                out += f"cls label: {self.cls_labels[i]} cls score: {_f(self.cls_scores[i])}\n"
            return out
        if self.cls_scores:
            for i in range(len(self.cls_scores)):
                out += f"cls label: {self.cls_labels[i]} cls score: {_f(self.cls_scores[i])}\n"
            return out
        if self.rec_scores:
            for i in range(len(self.rec_scores)):
                out += f"rec text: {self.text[i]} rec score:{_f(self.rec_scores[i])}\n"
            return out
        return "No Results!"


@dataclass
class MOTResult(_Base):
    boxes: List[List[int]] = field(default_factory=list)
    ids: List[int] = field(default_factory=list)
    scores: List[float] = field(default_factory=list)
    class_ids: List[int] = field(default_factory=list)

    def __str__(self) -> str:
        out = "MOTResult:\nall boxes counts: " + str(len(self.boxes)) + "\n[xmin\tymin\txmax\tymax\tid\tscore]\n"
        for b, i, s in zip(self.boxes, self.ids, self.scores):
            out += f"[{b[0]}\t{b[1]}\t{b[2]}\t{b[3]}\t{i}\t{s}]\n"
        return out


@dataclass
class FaceDetectionResult(_Base):
    boxes: List[List[float]] = field(default_factory=list)
    landmarks: List[List[float]] = field(default_factory=list)
    scores: List[float] = field(default_factory=list)
    landmarks_per_face: int = 0

    def __str__(self) -> str:
        if self.landmarks_per_face > 0:
            out = f"FaceDetectionResult: [xmin, ymin, xmax, ymax, score, (x, y) x {self.landmarks_per_face}]\n"
        else:
            out = "FaceDetectionResult: [xmin, ymin, xmax, ymax, score]\n"
        for i, b in enumerate(self.boxes):
            out += ",".join(_f(v) for v in b) + f", {_f(self.scores[i])}, "
            for j in range(self.landmarks_per_face):
                lm = self.landmarks[i * self.landmarks_per_face + j]
                out += f"({_f(lm[0])},{_f(lm[1])})" + (", " if j < self.landmarks_per_face - 1 else "")
            out += "\n"
        return out


@dataclass
class FaceAlignmentResult(_Base):
    landmarks: List[List[float]] = field(default_factory=list)

    def __str__(self) -> str:
        out = f"FaceAlignmentResult: [x, y]\nThere are {len(self.landmarks)} landmarks, the coordinates are listed below\n"
        for lm in self.landmarks:
            out += f"{_f(lm[0])},{_f(lm[1])}\n"
        return out + "\n"


@dataclass
class SegmentationResult(_Base):
    label_map: List[int] = field(default_factory=list)
    score_map: List[float] = field(default_factory=list)
    shape: List[int] = field(default_factory=list)
    contain_score_map: bool = False

    def __str__(self) -> str:
        out = f"SegmentationResult Image masks 10 rows x 10 cols: \n"
        h, w = (self.shape + [0, 0])[:2]
        for i in range(min(10, h)):
            out += "[" + ", ".join(str(self.label_map[i * w + j]) for j in range(min(10, w))) + ", .....]\n"
        out += "...........\n"
        if self.contain_score_map:
            out += "SegmentationResult Score map 10 rows x 10 cols: \n"
            for i in range(min(10, h)):
                out += "[" + ", ".join(_f(self.score_map[i * w + j]) for j in range(min(10, w))) + ", .....]\n"
            out += "...........\n"
        return out + f"result shape is: [{h} {w}]\n"


@dataclass
class FaceRecognitionResult(_Base):
    embedding: List[float] = field(default_factory=list)

    def __str__(self) -> str:
        e = np.asarray(self.embedding, dtype=np.float32)
        if e.size == 0:
            return "FaceRecognitionResult: [Dim(0), Min(0), Max(0), Mean(0)]\n"
        return (f"FaceRecognitionResult: [Dim({e.size}), Min({_f(float(e.min()))}), Max({_f(float(e.max()))}), "
                f"Mean({_f(float(e.mean()))})]\n")


@dataclass
class MattingResult(_Base):
    alpha: List[float] = field(default_factory=list)
    foreground: List[float] = field(default_factory=list)
    shape: List[int] = field(default_factory=list)
    contain_foreground: bool = False

    def __str__(self) -> str:
        out = "MattingResult["
        out += "Foreground(true)" if self.contain_foreground else "Foreground(false)"
        out += ", Alpha(Numel(" + str(len(self.alpha)) + "), Shape(" + ",".join(str(s) for s in self.shape) + ")"
        a = np.asarray(self.alpha, dtype=np.float32)
        if a.size:
            out += f", Min({_f(float(a.min()))}), Max({_f(float(a.max()))}), Mean({_f(float(a.mean()))})"
        return out + ")]\n"


@dataclass
class HeadPoseResult(_Base):
    euler_angles: List[float] = field(default_factory=list)

    def __str__(self) -> str:
        out = "HeadPoseResult: [yaw, pitch, roll]\n"
        names = ["yaw", "pitch", "roll"]
        for n, v in zip(names, self.euler_angles):
            out += f"{n}: {_f(v)}\n"
        return out + "\n"
