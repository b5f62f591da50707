"""3-D perception (fastdeploy/vision/perception/paddle3d/): SMOKE, PETR and CADDN copy the network's
``[N, 7 | 9]`` boxes, scores and labels into :class:`PerceptionResult` (smoke/postprocessor.cc:40-90,
petr/postprocessor.cc, caddn/postprocessor.cc); CenterPoint runs on a point cloud with voxelisation,
head decode and rotated BEV NMS (the reference registers those as custom ops inside Paddle Inference,
fastdeploy/runtime/backends/paddle/ops/{voxelize_op,postprocess,iou3d_nms}*). The three ops are restated
here on the host; their inputs and outputs keep the reference's layouts."""
from __future__ import annotations

import math
from typing import Any, List, Optional, Sequence, Tuple

import numpy as np
import yaml

from ...core.types import ModelFormat
from ...runtime.model import FastDeployModel
from ...runtime.option import RuntimeOption
from ..detection.contrib import _resize_bilinear
from ..result import PerceptionResult


# ------------------------------------------------------------------ ops
def hard_voxelize(points: np.ndarray, voxel_size: Sequence[float], pc_range: Sequence[float], max_points: int,
                  max_voxels: int):
    """Points ``[N, C]`` -> (voxels ``[V, max_points, C]``, coords ``[V, 3]`` as (z, y, x), points per
    voxel ``[V]``). Voxels are created in the order their first point appears; points beyond
    ``max_points`` in a voxel and voxels beyond ``max_voxels`` are dropped (voxelize_op.cc)."""
    vs, r = np.asarray(voxel_size, np.float32), np.asarray(pc_range, np.float32)
    grid = np.round((r[3:] - r[:3]) / vs).astype(np.int64)
    c = np.floor((points[:, :3] - r[:3]) / vs).astype(np.int64)
    ok = ((c >= 0) & (c < grid)).all(1)
    voxels = np.zeros((max_voxels, max_points, points.shape[1]), np.float32)
    coords = np.zeros((max_voxels, 3), np.int32)
    num = np.zeros(max_voxels, np.int32)
    index = {}
    for i in np.nonzero(ok)[0]:
        key = (int(c[i, 2]), int(c[i, 1]), int(c[i, 0]))
        v = index.get(key)
        if v is None:
            if len(index) >= max_voxels:
                continue
            v = len(index)
            index[key] = v
            coords[v] = key
        if num[v] < max_points:
            voxels[v, num[v]] = points[i]
            num[v] += 1
    n = len(index)
    return voxels[:n], coords[:n], num[:n]


def _rot_corners(b):
    x, y, w, l, a = b
    c, s = math.cos(a), math.sin(a)
    pts = np.asarray([[-w / 2, -l / 2], [w / 2, -l / 2], [w / 2, l / 2], [-w / 2, l / 2]])
    return pts @ np.asarray([[c, s], [-s, c]]) + [x, y]


def _poly_clip(subject, clip):
    def inside(p, a, b):
        return (b[0] - a[0]) * (p[1] - a[1]) - (b[1] - a[1]) * (p[0] - a[0]) >= 0

    def inter(p, q, a, b):
        d1, d2 = q - p, b - a
        den = d1[0] * d2[1] - d1[1] * d2[0]
        t = ((a[0] - p[0]) * d2[1] - (a[1] - p[1]) * d2[0]) / (den if abs(den) > 1e-12 else 1e-12)
        return p + t * d1
    out = list(subject)
    for i in range(len(clip)):
        a, b = clip[i], clip[(i + 1) % len(clip)]
        inp, out = out, []
        if not inp:
            break
        s = inp[-1]
        for e in inp:
            if inside(e, a, b):
                if not inside(s, a, b):
                    out.append(inter(s, e, a, b))
                out.append(e)
            elif inside(s, a, b):
                out.append(inter(s, e, a, b))
            s = e
    return out


def rotated_iou_bev(a, b) -> float:
    """IoU of two BEV boxes ``(x, y, w, l, angle)`` by polygon clipping."""
    pa, pb = _rot_corners(a), _rot_corners(b)
    poly = _poly_clip(list(pa), list(pb))
    if len(poly) < 3:
        return 0.0
    p = np.asarray(poly)
    inter = 0.5 * abs(np.dot(p[:, 0], np.roll(p[:, 1], -1)) - np.dot(p[:, 1], np.roll(p[:, 0], -1)))
    return float(inter / max(a[2] * a[3] + b[2] * b[3] - inter, 1e-9))


def nms_bev(boxes: np.ndarray, scores: np.ndarray, thresh: float, pre_max: int = 1000, post_max: int = 83) -> List[int]:
    order = np.argsort(-scores, kind="stable")[:pre_max]
    keep: List[int] = []
    for i in order:
        if all(rotated_iou_bev(boxes[i], boxes[k]) <= thresh for k in keep):
            keep.append(int(i))
            if len(keep) >= post_max:
                break
    return keep


def centerpoint_decode(hm, reg, height, dim, vel, rot, voxel_size, pc_range, down_ratio, score_threshold,
                       nms_iou_threshold, post_center_range=None, nms_pre_max=1000, nms_post_max=83, with_velocity=True):
    """One task head of CenterPoint: ``hm [C, H, W]`` logits, ``reg [2,..]``, ``height [1,..]``, ``dim
    [3,..]`` (log), ``vel [2,..]``, ``rot [2,..]`` (sin, cos) -> boxes ``[n, 9 | 7]`` as
    (x, y, z, w, l, h, (vx, vy,) yaw), scores, labels (postprocess.cc)."""
    c, h, w = hm.shape
    prob = 1.0 / (1.0 + np.exp(-hm))
    labels = prob.argmax(0).reshape(-1)
    scores = prob.max(0).reshape(-1)
    ys, xs = np.divmod(np.arange(h * w), w)
    x = (xs + reg[0].reshape(-1)) * down_ratio * voxel_size[0] + pc_range[0]
    y = (ys + reg[1].reshape(-1)) * down_ratio * voxel_size[1] + pc_range[1]
    z = height.reshape(-1)
    d = np.exp(dim.reshape(3, -1))
    yaw = np.arctan2(rot[0].reshape(-1), rot[1].reshape(-1))
    cols = [x, y, z, d[0], d[1], d[2]]
    if with_velocity:
        cols += [vel[0].reshape(-1), vel[1].reshape(-1)]
    cols.append(yaw)
    boxes = np.stack(cols, 1).astype(np.float32)
    m = scores > score_threshold
    if post_center_range is not None:
        pr = np.asarray(post_center_range, np.float32)
        m &= (boxes[:, :3] >= pr[:3]).all(1) & (boxes[:, :3] <= pr[3:]).all(1)
    boxes, scores, labels = boxes[m], scores[m], labels[m]
    bev = np.stack([boxes[:, 0], boxes[:, 1], boxes[:, 3], boxes[:, 4], boxes[:, -1]], 1)
    keep = nms_bev(bev, scores, nms_iou_threshold, nms_pre_max, nms_post_max)
    return boxes[keep], scores[keep], labels[keep]


# ------------------------------------------------------------------ models
def _fill(boxes: np.ndarray, scores: np.ndarray, labels: np.ndarray, with_velocity: bool = False) -> PerceptionResult:
    r = PerceptionResult()
    for b, s, l in zip(np.asarray(boxes, np.float32), np.asarray(scores, np.float32), np.asarray(labels).reshape(-1)):
        r.scores.append(float(s))
        r.label_ids.append(int(l))
        if with_velocity and len(b) >= 9:
            r.boxes.append([float(v) for v in (b[0], b[1], b[2], b[3], b[4], b[5], b[8])])
            r.velocity.append([float(b[6]), float(b[7])])
        else:
            r.boxes.append([float(v) for v in b[:7]])
        r.center.append([float(b[0]), float(b[1]), float(b[2])])
        r.yaw_angle.append(float(b[-1]))
        r.valid.append(True)
    return r


class _ImagePreprocessor:
    """Image half of the camera models' inputs, from the model's yaml: resize to ``Resize.target_size``, BGR->RGB, 1/255,
    ``NormalizeImage`` mean / std, CHW (fastdeploy/vision/perception/paddle3d/{smoke,petr,caddn}/preprocessor.cc)."""

    def __init__(self, config_file: str):
        with open(config_file) as f:
            cfg = yaml.safe_load(f) or {}
        self.config_file = config_file
        self.size = [1280, 384]
        self.mean, self.std = [0.485, 0.456, 0.406], [0.229, 0.224, 0.225]
        for op in cfg.get("Preprocess", []) or []:
            if op.get("type") == "Resize":
                hh, ww = op["target_size"]
                self.size = [ww, hh]
            elif op.get("type") == "NormalizeImage":
                self.mean, self.std = list(op["mean"]), list(op["std"])

    def image_tensor(self, im: np.ndarray) -> np.ndarray:
        x = _resize_bilinear(im, *self.size)[..., ::-1].astype(np.float32) / 255.0
        x = (x - np.asarray(self.mean, np.float32)) / np.asarray(self.std, np.float32)
        return np.ascontiguousarray(x.transpose(2, 0, 1))

    def run(self, images: Sequence[np.ndarray]) -> np.ndarray:
        return np.stack([self.image_tensor(im) for im in images])


class SmokePreprocessor(_ImagePreprocessor):
    pass


class PetrPreprocessor(_ImagePreprocessor):
    pass


class CaddnPreprocessor(_ImagePreprocessor):
    def run(self, input_ims: Sequence[np.ndarray], cam_data: Optional[Sequence[float]] = None,
            lidar_data: Optional[Sequence[float]] = None):
        """``[images [N, 3, H, W], cam2img [N, 3, 4], lidar2cam [N, 4, 4]]``: the two matrices (12 and 16 numbers, row
        major) are shared by the images of the batch (caddn/preprocessor.cc:95-140)."""
        x = _ImagePreprocessor.run(self, input_ims)
        if cam_data is None and lidar_data is None:
            return x
        n = len(input_ims)
        cam = np.eye(3, 4, dtype=np.float32) if cam_data is None else np.asarray(cam_data, np.float32).reshape(3, 4)
        lidar = np.eye(4, dtype=np.float32) if lidar_data is None else np.asarray(lidar_data, np.float32).reshape(4, 4)
        return [x, np.repeat(cam[None], n, 0), np.repeat(lidar[None], n, 0)]


class SmokePostprocessor:
    """Rows ``[label, alpha, x1, y1, x2, y2, h, w, l, x, y, z, yaw, score]`` above the score threshold
    (smoke/postprocessor.cc:40-90)."""

    def __init__(self):
        self.score_threshold = 0.25

    def run(self, outputs: Sequence[np.ndarray]) -> List[PerceptionResult]:
        rows = np.asarray(outputs[0], np.float32).reshape(-1, 14)
        rows = rows[rows[:, 13] > self.score_threshold]
        r = PerceptionResult()
        for row in rows:
            r.label_ids.append(int(row[0])); r.observation_angle.append(float(row[1]))
            r.boxes.append([float(v) for v in (row[2], row[3], row[4], row[5], row[6], row[7], row[8])])
            r.center.append([float(row[9]), float(row[10]), float(row[11])])
            r.yaw_angle.append(float(row[12])); r.scores.append(float(row[13])); r.valid.append(True)
        return [r]


class PetrPostprocessor:
    """Boxes ``[n, 9]`` (with velocity), scores, labels (petr/postprocessor.cc:30-80)."""

    def __init__(self):
        self.score_threshold = 0.25

    def run(self, outputs: Sequence[np.ndarray]) -> List[PerceptionResult]:
        b, s, l = (np.asarray(o) for o in outputs[:3])
        m = s.reshape(-1) > self.score_threshold
        return [_fill(b.reshape(len(m), -1)[m], s.reshape(-1)[m], l.reshape(-1)[m], with_velocity=True)]


class CaddnPostprocessor:
    """Boxes ``[n, 7]``, labels, scores (caddn/postprocessor.cc:30-75)."""

    def __init__(self):
        self.score_threshold = 0.25

    def run(self, outputs: Sequence[np.ndarray]) -> List[PerceptionResult]:
        b, l, s = (np.asarray(o) for o in outputs[:3])
        m = s.reshape(-1) > self.score_threshold
        return [_fill(b.reshape(len(m), -1)[m], s.reshape(-1)[m], l.reshape(-1)[m])]


class _ImagePerception(FastDeployModel):
    PRE = _ImagePreprocessor
    POST = None

    def __init__(self, model_file: str, params_file: str, config_file: str,
                 runtime_option: Optional[RuntimeOption] = None, model_format: int = ModelFormat.PADDLE):
        super().__init__(runtime_option)
        self.runtime_option.set_model_path(model_file, params_file, model_format)
        self.preprocessor = self.PRE(config_file)
        self.postprocessor = self.POST()
        self.init_runtime()

    size = property(lambda self: self.preprocessor.size, lambda self, v: setattr(self.preprocessor, "size", list(v)))
    mean = property(lambda self: self.preprocessor.mean)
    std = property(lambda self: self.preprocessor.std)
    score_threshold = property(lambda self: self.postprocessor.score_threshold,
                               lambda self, v: setattr(self.postprocessor, "score_threshold", v))

    def _image_tensor(self, im: np.ndarray) -> np.ndarray:
        return self.preprocessor.image_tensor(im)

    def batch_predict(self, items: Sequence[Any], *extras) -> List[PerceptionResult]:
        """One :meth:`predict` per item; ``extras`` (camera matrices ...) are either one value for all items or a sequence
        with one value per item."""
        out = []
        for i, it in enumerate(items):
            args = [e[i] if isinstance(e, (list, tuple)) and len(e) == len(items) else e for e in extras]
            out.append(self.predict(it, *args))
        return out


class Smoke(_ImagePerception):
    PRE, POST = SmokePreprocessor, SmokePostprocessor
    __doc__ = """Monocular SMOKE: inputs image, camera intrinsics ``K [1,3,3]`` and ``down_ratios [1,2]``; output rows
    ``[label, alpha, x1, y1, x2, y2, h, w, l, x, y, z, yaw, score]`` (smoke/postprocessor.cc:40-90)."""

    def predict(self, im: np.ndarray, k: Optional[np.ndarray] = None) -> PerceptionResult:
        h, w = im.shape[:2]
        k = np.eye(3, dtype=np.float32) if k is None else np.asarray(k, np.float32).reshape(3, 3)
        feeds = {}
        for i in range(self.runtime.num_inputs()):
            name = self.runtime.get_input_info(i).name
            if i == 0:
                feeds[name] = self._image_tensor(im)[None]
            elif "K" in name or i == 1:
                feeds[name] = k[None]
            else:
                feeds[name] = np.asarray([[w / self.size[0] * 4.0, h / self.size[1] * 4.0]], np.float32)
        return self.postprocessor.run(self.runtime.infer(feeds))[0]


class Petr(_ImagePerception):
    PRE, POST = PetrPreprocessor, PetrPostprocessor
    __doc__ = """Multi-camera PETR: six images stacked ``[1, 6, 3, H, W]`` plus ``img2lidars [1, 6, 4, 4]``; outputs
    boxes ``[n, 9]``, scores, labels."""

    def predict(self, images: Sequence[np.ndarray], img2lidars: Optional[np.ndarray] = None) -> PerceptionResult:
        x = np.stack([self._image_tensor(im) for im in images])[None]
        names = [self.runtime.get_input_info(i).name for i in range(self.runtime.num_inputs())]
        feeds = {names[0]: x}
        if len(names) > 1:
            t = np.tile(np.eye(4, dtype=np.float32), (1, len(images), 1, 1)) if img2lidars is None else np.asarray(img2lidars, np.float32)
            feeds[names[1]] = t.reshape(1, len(images), 4, 4)
        return self.postprocessor.run(self.runtime.infer(feeds))[0]


class Caddn(_ImagePerception):
    PRE, POST = CaddnPreprocessor, CaddnPostprocessor
    __doc__ = """CaDDN: image plus camera-to-image and lidar-to-camera matrices; outputs boxes ``[n, 7]``, labels, scores."""

    def predict(self, input_image: np.ndarray, cam_data: Optional[Sequence[float]] = None,
                lidar_data: Optional[Sequence[float]] = None, *, cam2img=None, lidar2cam=None):
        """``cam_data``: the 3 x 4 camera-to-image matrix (12 numbers), ``lidar_data``: the 4 x 4 lidar-to-camera matrix
        (``cam2img`` / ``lidar2cam`` are the same two under the names of earlier versions of this class)."""
        cam_data = cam2img if cam_data is None else cam_data
        lidar_data = lidar2cam if lidar_data is None else lidar_data
        names = [self.runtime.get_input_info(i).name for i in range(self.runtime.num_inputs())]
        feeds = {names[0]: self._image_tensor(input_image)[None]}
        if len(names) > 1:
            feeds[names[1]] = (np.eye(3, 4, dtype=np.float32) if cam_data is None else np.asarray(cam_data, np.float32)).reshape(1, 3, 4)
        if len(names) > 2:
            feeds[names[2]] = (np.eye(4, dtype=np.float32) if lidar_data is None else np.asarray(lidar_data, np.float32)).reshape(1, 4, 4)
        return self.postprocessor.run(self.runtime.infer(feeds))[0]


class CenterpointPreprocessor:
    """Voxelisation settings of the lidar model and the host voxeliser (centerpoint/preprocessor.cc:25-90)."""

    def __init__(self, config_file: str = ""):
        self.config_file = config_file
        self.voxel_size = [0.2, 0.2, 8.0]
        self.point_cloud_range = [-51.2, -51.2, -5.0, 51.2, 51.2, 3.0]
        self.max_points_in_voxel, self.max_voxel_num = 20, 30000

    def voxelize(self, points: np.ndarray):
        return hard_voxelize(np.asarray(points, np.float32), self.voxel_size, self.point_cloud_range, self.max_points_in_voxel,
                             self.max_voxel_num)

    @staticmethod
    def read_points(point_dir, num_point_dim: int = 5, with_timelag: int = 0) -> np.ndarray:
        """One sweep ``[N, num_point_dim]`` from a file of packed float32 values (or an array, passed through). The fifth
        column is the time lag; it is zeroed when the file has one but the model was trained without it, and for sweeps
        with more than five columns (centerpoint/preprocessor.cc:25-95)."""
        if num_point_dim < 4:
            raise ValueError(f"Point dimension must not be less than 4, but received num_point_dim is {num_point_dim}")
        if isinstance(point_dir, (str, bytes)) or hasattr(point_dir, "__fspath__"):
            data = np.fromfile(point_dir, dtype=np.float32)
            if data.size % num_point_dim:
                raise ValueError(f"Loaded file size ({data.size * 4}) is not evenly divisible by num_point_dim ({num_point_dim})")
            pts = data.reshape(-1, num_point_dim).copy()
        else:
            pts = np.array(point_dir, np.float32, copy=True).reshape(-1, num_point_dim)
        if (not with_timelag and num_point_dim == 5) or num_point_dim > 5:
            pts[:, 4] = 0.0
        return pts

    def run(self, point_dirs, num_point_dim: int = 5, with_timelag: int = 0) -> List[np.ndarray]:
        """Files (or arrays) -> one ``[N, num_point_dim]`` array per sweep."""
        if isinstance(point_dirs, (str, bytes)) or isinstance(point_dirs, np.ndarray):
            point_dirs = [point_dirs]
        return [self.read_points(p, num_point_dim, with_timelag) for p in point_dirs]


class Centerpoint(FastDeployModel):
    """CenterPoint on a lidar sweep ``[N, 4 | 5]``: voxelise on the host, run the network on
    (voxels, coords, num_points), decode + rotated NMS per task head."""

    def __init__(self, model_file: str, params_file: str, config_file: str = "",
                 runtime_option: Optional[RuntimeOption] = None, model_format: int = ModelFormat.PADDLE):
        super().__init__(runtime_option)
        self.runtime_option.set_model_path(model_file, params_file, model_format)
        self.preprocessor = CenterpointPreprocessor(config_file)
        self.down_ratio, self.score_threshold, self.nms_iou_threshold = 4, 0.1, 0.2
        self.with_velocity = True
        self.num_point_dim, self.with_timelag = 5, 0
        self.init_runtime()

    voxel_size = property(lambda self: self.preprocessor.voxel_size, lambda self, v: setattr(self.preprocessor, "voxel_size", list(v)))
    point_cloud_range = property(lambda self: self.preprocessor.point_cloud_range,
                                 lambda self, v: setattr(self.preprocessor, "point_cloud_range", list(v)))
    max_points_in_voxel = property(lambda self: self.preprocessor.max_points_in_voxel,
                                   lambda self, v: setattr(self.preprocessor, "max_points_in_voxel", int(v)))
    max_voxel_num = property(lambda self: self.preprocessor.max_voxel_num, lambda self, v: setattr(self.preprocessor, "max_voxel_num", int(v)))

    @property
    def postprocessor(self):
        """Decoding is part of :meth:`predict` (it needs the voxel grid); the thresholds live on the model."""
        return self

    def batch_predict(self, sweeps: Sequence[np.ndarray]) -> List[PerceptionResult]:
        return [self.predict(p) for p in sweeps]

    def predict(self, points) -> PerceptionResult:
        """``points``: a sweep ``[N, 4 | 5]`` or the path of a file of packed float32 values."""
        if isinstance(points, (str, bytes)) or hasattr(points, "__fspath__"):
            points = self.preprocessor.read_points(points, self.num_point_dim, self.with_timelag)
        pts = np.asarray(points, np.float32)
        voxels, coords, num = hard_voxelize(pts, self.voxel_size, self.point_cloud_range, self.max_points_in_voxel,
                                            self.max_voxel_num)
        names = [self.runtime.get_input_info(i).name for i in range(self.runtime.num_inputs())]
        if len(names) == 1:      # exports with the voxeliser inside the graph take the raw points
            outs = self.runtime.infer({names[0]: pts})
        else:
            outs = self.runtime.infer(dict(zip(names, [voxels, coords, num])))
        outs = [np.asarray(o, np.float32) for o in outs]
        if len(outs) == 3 and outs[0].ndim == 2:   # already decoded: boxes, scores, labels
            return _fill(outs[0], outs[1].reshape(-1), outs[2].reshape(-1), self.with_velocity)
        hm, reg, height, dim, vel, rot = (o[0] for o in outs[:6])
        if getattr(self.runtime, "on_gpu", False):
            # decode, candidate sort and rotated bird's-eye-view NMS on the device
            import torch
            from ...ops.perception import centerpoint_decode_device
            dev = self.runtime.device
            t = [torch.from_numpy(np.ascontiguousarray(a)).to(dev) for a in (hm, reg, height, dim, vel, rot)]
            b, s, l = centerpoint_decode_device(*t, self.voxel_size, self.point_cloud_range, self.down_ratio,
                                                self.score_threshold, self.nms_iou_threshold,
                                                with_velocity=self.with_velocity)
            return _fill(b.cpu().numpy(), s.cpu().numpy(), l.cpu().numpy(), self.with_velocity)
        b, s, l = centerpoint_decode(hm, reg, height, dim, vel, rot, self.voxel_size, self.point_cloud_range,
                                     self.down_ratio, self.score_threshold, self.nms_iou_threshold,
                                     with_velocity=self.with_velocity)
        return _fill(b, s, l, self.with_velocity)
