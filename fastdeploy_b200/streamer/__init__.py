"""Streamer: multi-stream video analytics driven by a YAML file.

The reference (streamer/src/app/{yaml_parser,base_app,video_analytics}.cc) turns the YAML into a
``gst-launch`` string of DeepStream / GStreamer elements and runs the main loop with a bus watch and an
FPS probe. The element names are kept as configuration vocabulary, the pipeline itself is native:

``nvurisrcbin_list`` / ``filesrc`` / ``appsrc`` -> frame sources (video files through OpenCV, NumPy
frame lists, synthetic generators) · ``nvstreammux`` -> batcher (batch-size, batched-push-timeout) ·
``nvinfer`` / ``fdinfer`` -> a model object's ``batch_predict`` · ``nvtracker`` / ``fdtracker`` ->
OC-SORT per stream · ``nvmultistreamtiler`` + ``nvosdbin`` -> tiled overlay drawn by the visualisation
kernels (or on the host) · sinks: ``appsink`` collects results / frames in memory, ``filesink`` writes
an ``.mp4`` or ``.npy``. There is no window or display sink: output always lands in a buffer or a file.
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterator, List, Optional, Sequence

import numpy as np
import yaml

from ..vision.result import DetectionResult, MOTResult
from ..vision.tracking import OCSortTracker


@dataclass
class Frame:
    stream_id: int
    index: int
    image: np.ndarray
    pts: float = 0.0
    result: Any = None
    tracks: Optional[np.ndarray] = None


class FrameSource:
    """Iterator of BGR frames. ``uri`` may be ``file://...`` (decoded with OpenCV), ``synthetic://WxHxN``
    (moving rectangles, deterministic) or a list / array of frames."""

    def __init__(self, uri: Any, stream_id: int = 0):
        self.uri, self.stream_id = uri, stream_id

    def __iter__(self) -> Iterator[Frame]:
        u = self.uri
        if isinstance(u, str) and u.startswith("synthetic://"):
            w, h, n = (int(v) for v in u[len("synthetic://"):].split("x"))
            rng = np.random.default_rng(self.stream_id)
            base = rng.integers(0, 60, (h, w, 3), dtype=np.uint8)
            for i in range(n):
                img = base.copy()
                x = (10 + 7 * i + 31 * self.stream_id) % max(w - 60, 1)
                img[h // 4:h // 4 + 50, x:x + 50] = (40, 200, 240)
                yield Frame(self.stream_id, i, img, i / 30.0)
        elif isinstance(u, str):
            import cv2
            path = u[len("file://"):] if u.startswith("file://") else u
            cap = cv2.VideoCapture(path)
            fps = cap.get(cv2.CAP_PROP_FPS) or 30.0
            i = 0
            while True:
                ok, img = cap.read()
                if not ok:
                    break
                yield Frame(self.stream_id, i, img, i / fps)
                i += 1
            cap.release()
        else:
            for i, img in enumerate(u):
                yield Frame(self.stream_id, i, np.asarray(img), i / 30.0)


class StreamMux:
    """Round-robin batcher over the sources: emits lists of up to ``batch_size`` frames; a source that
    ends drops out, the last batches are smaller (the timeout of the reference's mux becomes 'whatever
    is available', there is no wall-clock pacing in file mode)."""

    def __init__(self, sources: Sequence[FrameSource], batch_size: int):
        self.sources, self.batch_size = list(sources), max(1, batch_size)

    def __iter__(self) -> Iterator[List[Frame]]:
        its = [iter(s) for s in self.sources]
        batch: List[Frame] = []
        while its:
            for it in list(its):
                try:
                    batch.append(next(it))
                except StopIteration:
                    its.remove(it)
                    continue
                if len(batch) == self.batch_size:
                    yield batch
                    batch = []
        if batch:
            yield batch


@dataclass
class PerfMeasurement:
    interval_s: float = 5.0
    frames: int = 0
    t0: float = field(default_factory=time.perf_counter)
    history: List[float] = field(default_factory=list)

    def tick(self, n: int) -> Optional[float]:
        self.frames += n
        dt = time.perf_counter() - self.t0
        if dt >= self.interval_s:
            fps = self.frames / dt
            self.history.append(fps)
            self.frames, self.t0 = 0, time.perf_counter()
            return fps
        return None


def tile_frames(frames: Sequence[np.ndarray], rows: int, cols: int, width: int, height: int) -> np.ndarray:
    from ..vision.detection.contrib import _resize_bilinear
    tw, th = width // cols, height // rows
    canvas = np.zeros((th * rows, tw * cols, 3), np.uint8)
    for k, f in enumerate(frames[:rows * cols]):
        r, c = divmod(k, cols)
        canvas[r * th:(r + 1) * th, c * tw:(c + 1) * tw] = _resize_bilinear(f, tw, th)
    return canvas


class FDStreamer:
    """``FDStreamer(config).Run()`` as in the Python binding (streamer/python/streamer/fd_streamer.py:19-30), or
    ``FDStreamer().Init(config); Run()`` as in C++ (streamer/src/fd_streamer.cc:22-110). ``config`` is a YAML path or a dict."""

    def __init__(self, config_file: Any = None, model: Any = None):
        self._construct()
        if config_file is not None:
            self.Init(config_file, model)

    def _construct(self) -> None:
        self.cfg: Dict[str, Any] = {}
        self.model = None
        self.results: List[Frame] = []
        self.tiled: List[np.ndarray] = []
        self.perf: Optional[PerfMeasurement] = None
        self._thread: Optional[threading.Thread] = None
        self._stop = threading.Event()
        self.on_batch: Optional[Callable[[List[Frame]], None]] = None
        self.error: Optional[BaseException] = None

    # -- configuration
    def Init(self, config: Any, model: Any = None) -> bool:
        if isinstance(config, str):
            with open(config) as f:
                config = yaml.safe_load(f)
        self.cfg = dict(config or {})
        self.model = model
        app = self.cfg.get("app", {}) or {}
        if app.get("enable-perf-measurement"):
            self.perf = PerfMeasurement(float(app.get("perf-measurement-interval-sec", 5)))
        return True

    init = Init

    def _sources(self) -> List[FrameSource]:
        out: List[FrameSource] = []
        lst = self.cfg.get("nvurisrcbin_list") or {}
        for i, u in enumerate(lst.get("uri-list", []) or []):
            out.append(FrameSource(u, i))
        for key in ("filesrc", "nvurisrcbin"):
            if key in self.cfg:
                u = self.cfg[key].get("location") or self.cfg[key].get("uri")
                out.append(FrameSource(u, len(out)))
        if "appsrc" in self.cfg:
            for frames in self.cfg["appsrc"].get("streams", []):
                out.append(FrameSource(frames, len(out)))
        if not out:
            raise ValueError("streamer config has no source element")
        return out

    def describe(self) -> str:
        """The element chain as text, the analogue of the reference's generated launch string."""
        parts = []
        for key in ("nvurisrcbin_list", "filesrc", "appsrc", "nvstreammux", "nvinfer", "fdinfer", "nvtracker", "fdtracker",
                    "nvmultistreamtiler", "nvosdbin", "appsink", "filesink", "nvvideoencfilesinkbin"):
            if key in self.cfg:
                props = " ".join(f"{k}={v}" for k, v in (self.cfg[key] or {}).items() if not isinstance(v, (list, dict)))
                parts.append((key + " " + props).strip())
        return " ! ".join(parts)

    # -- execution
    def Run(self) -> bool:
        self._loop()
        if self.error is not None:
            raise self.error
        return True

    run = Run

    def RunAsync(self) -> None:
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self._thread.start()

    def Stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=10)

    def _loop(self) -> None:
        try:
            mux_cfg = self.cfg.get("nvstreammux", {}) or {}
            sources = self._sources()
            mux = StreamMux(sources, int(mux_cfg.get("batch-size", len(sources))))
            trk_cfg = self.cfg.get("fdtracker", self.cfg.get("nvtracker"))
            trackers: Dict[int, OCSortTracker] = {}
            tiler = self.cfg.get("nvmultistreamtiler")
            osd = "nvosdbin" in self.cfg
            sink = self.cfg.get("filesink") or self.cfg.get("nvvideoencfilesinkbin")
            keep_frames = bool((self.cfg.get("appsink") or {}).get("keep-frames", False))
            writer = None
            for batch in mux:
                if self._stop.is_set():
                    break
                if self.model is not None:
                    res = self.model.batch_predict([f.image for f in batch])
                    for f, r in zip(batch, res):
                        f.result = r
                if trk_cfg is not None:
                    for f in batch:
                        if isinstance(f.result, DetectionResult):
                            t = trackers.setdefault(f.stream_id, OCSortTracker(
                                det_thresh=float((trk_cfg or {}).get("det-thresh", 0.3)),
                                max_age=int((trk_cfg or {}).get("max-age", 30))))
                            f.tracks = t.update(np.asarray(f.result.boxes, float).reshape(-1, 4), np.asarray(f.result.scores, float),
                                                f.result.label_ids)
                if osd:
                    from ..vision import visualize as V
                    for f in batch:
                        if f.tracks is not None and len(f.tracks):
                            m = MOTResult()
                            m.boxes = f.tracks[:, :4].astype(int).tolist()
                            m.ids = f.tracks[:, 4].astype(int).tolist()
                            m.scores = f.tracks[:, 5].tolist()
                            f.image = V.vis_mot(f.image, m)
                        elif isinstance(f.result, DetectionResult):
                            f.image = V.vis_detection(f.image, f.result)
                if tiler:
                    tiled = tile_frames([f.image for f in batch], int(tiler.get("rows", 1)), int(tiler.get("columns", len(batch))),
                                        int(tiler.get("width", mux_cfg.get("width", 1280))), int(tiler.get("height", mux_cfg.get("height", 720))))
                    self.tiled.append(tiled)
                    if sink and str(sink.get("output-file", sink.get("location", ""))).endswith(".mp4"):
                        import cv2
                        if writer is None:
                            writer = cv2.VideoWriter(sink.get("output-file", sink.get("location")), cv2.VideoWriter_fourcc(*"mp4v"),
                                                     30.0, (tiled.shape[1], tiled.shape[0]))
                        writer.write(tiled)
                if self.on_batch is not None:
                    self.on_batch(batch)
                for f in batch:
                    if not keep_frames:
                        f.image = None
                    self.results.append(f)
                if self.perf is not None:
                    self.perf.tick(len(batch))
            if writer is not None:
                writer.release()
            if sink and str(sink.get("output-file", sink.get("location", ""))).endswith(".npy") and self.tiled:
                np.save(sink.get("output-file", sink.get("location")), np.stack(self.tiled))
        except BaseException as e:      # surfaces in Run(); RunAsync callers read .error
            self.error = e
