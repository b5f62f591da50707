"""Multi-object tracking.

* :class:`JDETracker` / :class:`PPTracking` - the FairMOT / JDE association of
  fastdeploy/vision/tracking/pptracking/tracker.cc:49-170: Kalman prediction (constant-velocity
  ``x, y, a, h`` state, trajectory.cc), then three matching stages solved as linear assignments -
  embedding distance fused with the motion gate (threshold 0.7, chi-square gating, lambda 0.98), IoU
  on the remaining tracked ones (0.5), IoU on unconfirmed ones (0.7) - with ``max_lost_time = 30`` and
  ``det_thresh = 0.3`` for new tracks.
* :class:`OCSortTracker` - the observation-centric SORT used by the streamer's tracker element
  (streamer/src/gstreamer/plugin/fdtracker/src/ocsort.cpp): IoU + velocity-direction consistency,
  a second association against the last observations, and re-update of the filter along the virtual
  trajectory when a lost track is found again.

Assignments use ``scipy.optimize.linear_sum_assignment`` (the reference ships LAPJV; both return an
optimal assignment).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import yaml

from ...core.types import ModelFormat
from ...runtime.model import FastDeployModel
from ...runtime.option import RuntimeOption
from ..detection.contrib import letterbox
from ..result import MOTResult

CHI2INV95 = {1: 3.8415, 2: 5.9915, 3: 7.8147, 4: 9.4877, 5: 11.070, 6: 12.592, 7: 14.067, 8: 15.507, 9: 16.919}


def linear_assignment(cost: np.ndarray, thresh: float):
    """Returns (matches [(row, col)], unmatched rows, unmatched cols); pairs above ``thresh`` are dropped."""
    if cost.size == 0:
        return [], list(range(cost.shape[0])), list(range(cost.shape[1]))
    from scipy.optimize import linear_sum_assignment
    c = np.where(cost > thresh, thresh + 1e-4, cost)
    rows, cols = linear_sum_assignment(c)
    matches = [(int(r), int(k)) for r, k in zip(rows, cols) if cost[r, k] <= thresh]
    mr, mc = {m[0] for m in matches}, {m[1] for m in matches}
    return matches, [i for i in range(cost.shape[0]) if i not in mr], [j for j in range(cost.shape[1]) if j not in mc]


def iou_matrix(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    if len(a) == 0 or len(b) == 0:
        return np.zeros((len(a), len(b)), np.float32)
    a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
    x1 = np.maximum(a[:, None, 0], b[None, :, 0]); y1 = np.maximum(a[:, None, 1], b[None, :, 1])
    x2 = np.minimum(a[:, None, 2], b[None, :, 2]); y2 = np.minimum(a[:, None, 3], b[None, :, 3])
    inter = np.maximum(x2 - x1, 0) * np.maximum(y2 - y1, 0)
    aa = (a[:, 2] - a[:, 0]) * (a[:, 3] - a[:, 1])
    ab = (b[:, 2] - b[:, 0]) * (b[:, 3] - b[:, 1])
    return inter / np.maximum(aa[:, None] + ab[None, :] - inter, 1e-9)


class KalmanFilterXYAH:
    """Constant-velocity filter over (cx, cy, aspect, height) with height-proportional noise."""

    def __init__(self):
        self.F = np.eye(8)
        for i in range(4):
            self.F[i, i + 4] = 1.0
        self.H = np.eye(4, 8)
        self.wp, self.wv = 1.0 / 20, 1.0 / 160

    def initiate(self, z):
        mean = np.r_[z, np.zeros(4)]
        h = z[3]
        std = [2 * self.wp * h, 2 * self.wp * h, 1e-2, 2 * self.wp * h, 10 * self.wv * h, 10 * self.wv * h, 1e-5, 10 * self.wv * h]
        return mean, np.diag(np.square(std))

    def predict(self, mean, cov):
        h = mean[3]
        std = [self.wp * h, self.wp * h, 1e-2, self.wp * h, self.wv * h, self.wv * h, 1e-5, self.wv * h]
        return self.F @ mean, self.F @ cov @ self.F.T + np.diag(np.square(std))

    def project(self, mean, cov):
        h = mean[3]
        std = [self.wp * h, self.wp * h, 1e-1, self.wp * h]
        return self.H @ mean, self.H @ cov @ self.H.T + np.diag(np.square(std))

    def update(self, mean, cov, z):
        pm, pc = self.project(mean, cov)
        k = np.linalg.solve(pc, (cov @ self.H.T).T).T
        return mean + k @ (z - pm), cov - k @ pc @ k.T

    def gating_distance(self, mean, cov, zs):
        pm, pc = self.project(mean, cov)
        d = np.asarray(zs) - pm
        l = np.linalg.cholesky(pc)
        y = np.linalg.solve(l, d.T)
        return (y * y).sum(0)


def _tlbr_to_xyah(b):
    w, h = b[2] - b[0], b[3] - b[1]
    return np.asarray([b[0] + w / 2, b[1] + h / 2, w / max(h, 1e-6), h], np.float64)


class Track:
    NEW, TRACKED, LOST, REMOVED = range(4)
    _count = 0

    def __init__(self, tlbr, score, feat, cls_id=0):
        self.tlbr_det = np.asarray(tlbr, np.float64)
        self.score, self.cls_id = float(score), cls_id
        self.feat = None
        self.alpha = 0.9
        self.update_feat(feat)
        self.mean = self.cov = None
        self.state, self.activated = Track.NEW, False
        self.id, self.frame_id, self.start_frame, self.tracklet_len = 0, 0, 0, 0

    @staticmethod
    def next_id():
        Track._count += 1
        return Track._count

    def update_feat(self, f):
        if f is None:
            return
        f = np.asarray(f, np.float64)
        f = f / max(np.linalg.norm(f), 1e-12)
        self.feat = f if self.feat is None else self.alpha * self.feat + (1 - self.alpha) * f
        self.feat = self.feat / max(np.linalg.norm(self.feat), 1e-12)

    @property
    def tlbr(self):
        if self.mean is None:
            return self.tlbr_det
        cx, cy, a, h = self.mean[:4]
        w = a * h
        return np.asarray([cx - w / 2, cy - h / 2, cx + w / 2, cy + h / 2])

    def activate(self, kf, frame_id):
        self.id = Track.next_id()
        self.mean, self.cov = kf.initiate(_tlbr_to_xyah(self.tlbr_det))
        self.state, self.frame_id, self.start_frame = Track.TRACKED, frame_id, frame_id
        self.activated = frame_id == 1

    def re_activate(self, kf, det: "Track", frame_id):
        self.mean, self.cov = kf.update(self.mean, self.cov, _tlbr_to_xyah(det.tlbr_det))
        self.update_feat(det.feat)
        self.tracklet_len = 0
        self.state, self.activated, self.frame_id, self.score = Track.TRACKED, True, frame_id, det.score

    def update(self, kf, det: "Track", frame_id):
        self.frame_id = frame_id
        self.tracklet_len += 1
        self.mean, self.cov = kf.update(self.mean, self.cov, _tlbr_to_xyah(det.tlbr_det))
        self.state, self.activated, self.score = Track.TRACKED, True, det.score
        self.update_feat(det.feat)


class JDETracker:
    def __init__(self, det_thresh: float = 0.3, track_buffer: int = 30, min_box_area: float = 200,
                 tracked_thresh: float = 0.7, r_tracked_thresh: float = 0.5, unconfirmed_thresh: float = 0.7,
                 motion_lambda: float = 0.98):
        self.kf = KalmanFilterXYAH()
        self.det_thresh, self.max_lost, self.min_box_area = det_thresh, track_buffer, min_box_area
        self.t1, self.t2, self.t3, self.lam = tracked_thresh, r_tracked_thresh, unconfirmed_thresh, motion_lambda
        self.tracked: List[Track] = []
        self.lost: List[Track] = []
        self.frame_id = 0

    def update(self, boxes: np.ndarray, scores: np.ndarray, feats: Optional[np.ndarray], cls_ids=None) -> List[Track]:
        self.frame_id += 1
        dets = [Track(b, s, feats[i] if feats is not None else None, int(cls_ids[i]) if cls_ids is not None else 0)
                for i, (b, s) in enumerate(zip(boxes, scores))]
        unconfirmed = [t for t in self.tracked if not t.activated]
        tracked = [t for t in self.tracked if t.activated]
        pool = tracked + [t for t in self.lost if t not in tracked]
        for t in pool:
            if t.state != Track.TRACKED:
                t.mean[7] = 0
            t.mean, t.cov = self.kf.predict(t.mean, t.cov)
        # stage 1: embedding distance fused with motion
        if pool and dets and feats is not None:
            tf = np.stack([t.feat for t in pool]); df = np.stack([d.feat for d in dets])
            cost = np.maximum(0.0, 1.0 - tf @ df.T)
            zs = [_tlbr_to_xyah(d.tlbr_det) for d in dets]
            for r, t in enumerate(pool):
                g = self.kf.gating_distance(t.mean, t.cov, zs)
                cost[r, g > CHI2INV95[4]] = np.inf
                cost[r] = self.lam * cost[r] + (1 - self.lam) * g
            cost = np.where(np.isfinite(cost), cost, 1e5)
        else:
            cost = 1.0 - iou_matrix([t.tlbr for t in pool], [d.tlbr_det for d in dets]) if pool and dets else np.zeros((len(pool), len(dets)))
        matches, u_track, u_det = linear_assignment(cost, self.t1)
        activated, refind = [], []
        for r, c in matches:
            t, d = pool[r], dets[c]
            if t.state == Track.TRACKED:
                t.update(self.kf, d, self.frame_id); activated.append(t)
            else:
                t.re_activate(self.kf, d, self.frame_id); refind.append(t)
        # stage 2: IoU for the tracked ones that are left
        rest_dets = [dets[i] for i in u_det]
        r_tracked = [pool[i] for i in u_track if pool[i].state == Track.TRACKED]
        cost = 1.0 - iou_matrix([t.tlbr for t in r_tracked], [d.tlbr_det for d in rest_dets])
        matches, u_track2, u_det2 = linear_assignment(cost, self.t2)
        for r, c in matches:
            r_tracked[r].update(self.kf, rest_dets[c], self.frame_id); activated.append(r_tracked[r])
        newly_lost = []
        for i in u_track2:
            t = r_tracked[i]
            if t.state != Track.LOST:
                t.state = Track.LOST; newly_lost.append(t)
        # stage 3: unconfirmed tracks
        rest_dets = [rest_dets[i] for i in u_det2]
        cost = 1.0 - iou_matrix([t.tlbr for t in unconfirmed], [d.tlbr_det for d in rest_dets])
        matches, u_unc, u_det3 = linear_assignment(cost, self.t3)
        for r, c in matches:
            unconfirmed[r].update(self.kf, rest_dets[c], self.frame_id); activated.append(unconfirmed[r])
        removed = [unconfirmed[i] for i in u_unc]
        for i in u_det3:
            d = rest_dets[i]
            if d.score >= self.det_thresh:
                d.activate(self.kf, self.frame_id); activated.append(d)
        for t in self.lost:
            if self.frame_id - t.frame_id > self.max_lost:
                t.state = Track.REMOVED; removed.append(t)
        self.tracked = activated + refind
        gone = {id(t) for t in removed} | {id(t) for t in self.tracked}
        self.lost = [t for t in self.lost if id(t) not in gone] + newly_lost
        return [t for t in self.tracked if t.activated]


class TrailRecorder:
    """Per track id, the centre points of its boxes frame after frame (fastdeploy/vision/tracking/pptracking/model.h:24-40);
    ``vis_mot(..., records=recorder)`` draws them as trails."""

    def __init__(self):
        self.records: Dict[int, List[List[int]]] = {}

    def add(self, track_id: int, point: Sequence[int]) -> None:
        self.records.setdefault(int(track_id), []).append([int(point[0]), int(point[1])])

    Add = add


class PPTracking(FastDeployModel):
    """FairMOT / JDE models exported by PaddleDetection (pptracking/model.cc:150-330): letterbox to the
    yaml's ``target_size`` with value 127.5, /255 normalise, outputs ``pred_dets [n, 6]`` and embeddings."""

    def __init__(self, model_file: str, params_file: str, config_file: str,
                 runtime_option: Optional[RuntimeOption] = None, model_format: int = ModelFormat.PADDLE):
        super().__init__(runtime_option)
        self.runtime_option.set_model_path(model_file, params_file, model_format)
        with open(config_file) as f:
            cfg = yaml.safe_load(f)
        self.size = [1088, 608]
        for op in cfg.get("Preprocess", []):
            if op["type"] == "LetterBoxResize":
                hh, ww = op["target_size"]
                self.size = [ww, hh]
        tr = cfg.get("tracker", {})
        self.conf_thresh = tr.get("conf_thres", 0.4)
        self.tracker = JDETracker(det_thresh=tr.get("tracked_thresh", 0.4), min_box_area=tr.get("min_box_area", 200))
        self.recorder: Optional[TrailRecorder] = None
        self.init_runtime()

    def bind_recorder(self, recorder: TrailRecorder) -> None:
        """From now on every returned track adds its box centre to ``recorder`` (model.cc:330-345)."""
        self.recorder = recorder

    def unbind_recorder(self) -> None:
        self.recorder = None

    def predict(self, im: np.ndarray) -> MOTResult:
        canvas, info = letterbox(im, self.size, (127.5, 127.5, 127.5))
        x = canvas[..., ::-1].astype(np.float32) / 255.0
        feeds = {}
        for i in range(self.runtime.num_inputs()):
            name = self.runtime.get_input_info(i).name
            if name == "image":
                feeds[name] = np.ascontiguousarray(x.transpose(2, 0, 1))[None]
            elif name == "im_shape":
                feeds[name] = np.asarray([[self.size[1], self.size[0]]], np.float32)
            elif name == "scale_factor":
                feeds[name] = np.asarray([[info["scale"], info["scale"]]], np.float32)
        outs = self.runtime.infer(feeds)
        dets, emb = np.asarray(outs[0], np.float32).reshape(-1, 6), np.asarray(outs[1], np.float32)
        m = dets[:, 1] > self.conf_thresh
        dets, emb = dets[m], emb.reshape(len(m), -1)[m]
        boxes = dets[:, 2:6].copy()
        boxes[:, [0, 2]] = (boxes[:, [0, 2]] - info["pad_w"]) / info["scale"]
        boxes[:, [1, 3]] = (boxes[:, [1, 3]] - info["pad_h"]) / info["scale"]
        tracks = self.tracker.update(boxes, dets[:, 1], emb, dets[:, 0])
        r = MOTResult()
        for t in tracks:
            b = t.tlbr
            if (b[2] - b[0]) * (b[3] - b[1]) <= self.tracker.min_box_area:
                continue
            r.boxes.append([int(v) for v in b]); r.ids.append(t.id); r.scores.append(t.score); r.class_ids.append(t.cls_id)
            if self.recorder is not None:
                self.recorder.add(t.id, [(int(b[0]) + int(b[2])) // 2, (int(b[1]) + int(b[3])) // 2])
        return r


# ------------------------------------------------------------------ OC-SORT
class _KalmanXYSR:
    """SORT's filter: state (x, y, s, r, vx, vy, vs) with s = area and r = aspect ratio."""

    def __init__(self, z):
        self.F = np.eye(7)
        self.F[0, 4] = self.F[1, 5] = self.F[2, 6] = 1.0
        self.H = np.eye(4, 7)
        self.R = np.diag([1.0, 1.0, 10.0, 10.0])
        self.P = np.diag([10.0, 10.0, 10.0, 10.0, 1e4, 1e4, 1e4])
        self.Q = np.diag([1.0, 1.0, 1.0, 1.0, 0.01, 0.01, 1e-4])
        self.x = np.r_[z, np.zeros(3)]

    def predict(self):
        if self.x[6] + self.x[2] <= 0:
            self.x[6] = 0.0
        self.x = self.F @ self.x
        self.P = self.F @ self.P @ self.F.T + self.Q

    def update(self, z):
        s = self.H @ self.P @ self.H.T + self.R
        k = self.P @ self.H.T @ np.linalg.inv(s)
        self.x = self.x + k @ (z - self.H @ self.x)
        self.P = (np.eye(7) - k @ self.H) @ self.P


def _to_z(b):
    w, h = b[2] - b[0], b[3] - b[1]
    return np.asarray([b[0] + w / 2, b[1] + h / 2, w * h, w / max(h, 1e-6)])


def _to_box(x):
    w = np.sqrt(max(x[2] * x[3], 0.0))
    h = x[2] / max(w, 1e-6)
    return np.asarray([x[0] - w / 2, x[1] - h / 2, x[0] + w / 2, x[1] + h / 2])


class _OCTrack:
    count = 0

    def __init__(self, box, score, cls_id, delta_t):
        self.kf = _KalmanXYSR(_to_z(box))
        _OCTrack.count += 1
        self.id = _OCTrack.count
        self.time_since_update, self.hits, self.hit_streak, self.age = 0, 0, 0, 0
        self.last_obs = np.r_[box, score]
        self.obs: Dict[int, np.ndarray] = {}
        self.velocity = None
        self.delta_t, self.score, self.cls_id = delta_t, score, cls_id
        self.lost_since: Optional[Tuple[int, np.ndarray]] = None

    def predict(self):
        self.kf.predict()
        self.age += 1
        if self.time_since_update > 0:
            self.hit_streak = 0
        self.time_since_update += 1
        return _to_box(self.kf.x)

    def update(self, box, score):
        if self.time_since_update > 1 and self.lost_since is not None:
            # observation-centric re-update: walk the filter along the straight line between the last
            # observation before the gap and this one
            t0, b0 = self.lost_since
            gap = self.time_since_update
            for k in range(1, gap):
                virt = b0 + (np.asarray(box) - b0) * k / gap
                self.kf.update(_to_z(virt))
                self.kf.predict()
        prev = None
        for dt in range(self.delta_t, 0, -1):
            if self.age - dt in self.obs:
                prev = self.obs[self.age - dt]
                break
        if prev is None and self.last_obs is not None:
            prev = self.last_obs[:4]
        if prev is not None:
            c0 = np.asarray([(prev[0] + prev[2]) / 2, (prev[1] + prev[3]) / 2])
            c1 = np.asarray([(box[0] + box[2]) / 2, (box[1] + box[3]) / 2])
            d = c1 - c0
            self.velocity = d / (np.linalg.norm(d) + 1e-6)
        self.last_obs = np.r_[box, score]
        self.obs[self.age] = np.asarray(box, np.float64)
        self.lost_since = (self.age, np.asarray(box, np.float64))
        self.time_since_update = 0
        self.hits += 1
        self.hit_streak += 1
        self.score = score
        self.kf.update(_to_z(box))


class OCSortTracker:
    def __init__(self, det_thresh: float = 0.6, max_age: int = 30, min_hits: int = 3, iou_threshold: float = 0.3,
                 delta_t: int = 3, inertia: float = 0.2):
        self.det_thresh, self.max_age, self.min_hits = det_thresh, max_age, min_hits
        self.iou_threshold, self.delta_t, self.inertia = iou_threshold, delta_t, inertia
        self.tracks: List[_OCTrack] = []
        self.frame = 0

    def update(self, boxes: np.ndarray, scores: np.ndarray, cls_ids=None):
        """Returns rows ``[x1, y1, x2, y2, id, score, cls]`` of the confirmed tracks of this frame."""
        self.frame += 1
        boxes, scores = np.asarray(boxes, np.float64).reshape(-1, 4), np.asarray(scores, np.float64).reshape(-1)
        cls_ids = np.zeros(len(scores), int) if cls_ids is None else np.asarray(cls_ids, int)
        keep = scores > self.det_thresh
        boxes, scores, cls_ids = boxes[keep], scores[keep], cls_ids[keep]
        preds = np.asarray([t.predict() for t in self.tracks]).reshape(-1, 4)
        iou = iou_matrix(preds, boxes)
        cost = -iou
        if len(self.tracks) and len(boxes):
            # velocity-direction consistency between each track's motion and the direction to each detection
            ang = np.zeros_like(iou)
            for r, t in enumerate(self.tracks):
                if t.velocity is None:
                    continue
                prev = t.last_obs[:4]
                c0 = np.asarray([(prev[0] + prev[2]) / 2, (prev[1] + prev[3]) / 2])
                c1 = np.stack([(boxes[:, 0] + boxes[:, 2]) / 2, (boxes[:, 1] + boxes[:, 3]) / 2], 1)
                d = c1 - c0
                d = d / (np.linalg.norm(d, axis=1, keepdims=True) + 1e-6)
                diff = np.arccos(np.clip(d @ t.velocity, -1, 1))
                ang[r] = (np.pi / 2 - np.abs(diff)) / np.pi * scores
            cost = -(iou + self.inertia * ang)
        matches, u_trk, u_det = linear_assignment(cost, 1e3) if cost.size else ([], list(range(len(self.tracks))), list(range(len(boxes))))
        good = []
        for r, c in matches:
            if iou[r, c] < self.iou_threshold:
                u_trk.append(r); u_det.append(c)
            else:
                good.append((r, c))
        for r, c in good:
            self.tracks[r].update(boxes[c], scores[c])
        # second pass: last observations of the unmatched tracks against the unmatched detections
        if u_trk and u_det:
            last = np.asarray([self.tracks[r].last_obs[:4] for r in u_trk])
            iou2 = iou_matrix(last, boxes[u_det])
            m2, _, _ = linear_assignment(-iou2, 1e3)
            done_t, done_d = set(), set()
            for r, c in m2:
                if iou2[r, c] >= self.iou_threshold:
                    self.tracks[u_trk[r]].update(boxes[u_det[c]], scores[u_det[c]])
                    done_t.add(u_trk[r]); done_d.add(u_det[c])
            u_trk = [r for r in u_trk if r not in done_t]
            u_det = [c for c in u_det if c not in done_d]
        for c in u_det:
            self.tracks.append(_OCTrack(boxes[c], scores[c], int(cls_ids[c]), self.delta_t))
        out = []
        alive = []
        for t in self.tracks:
            if t.time_since_update < 1 and (t.hit_streak >= self.min_hits or self.frame <= self.min_hits):
                out.append(np.r_[t.last_obs[:4], t.id, t.score, t.cls_id])
            if t.time_since_update <= self.max_age:
                alive.append(t)
        self.tracks = alive
        return np.asarray(out).reshape(-1, 7)
