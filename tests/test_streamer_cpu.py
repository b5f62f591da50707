import numpy as np

from fastdeploy_b200.streamer import FDStreamer, FrameSource, StreamMux
from fastdeploy_b200.vision.result import DetectionResult


class BlobDetector:
    """Finds the bright rectangle the synthetic source draws."""

    def batch_predict(self, images):
        out = []
        for im in images:
            r = DetectionResult()
            ys, xs = np.nonzero(im[..., 1] > 150)
            if len(xs):
                r.boxes = [[float(xs.min()), float(ys.min()), float(xs.max()), float(ys.max())]]
                r.scores, r.label_ids = [0.9], [0]
            out.append(r)
        return out


def test_mux_round_robin_and_tail():
    mux = StreamMux([FrameSource("synthetic://64x48x5", 0), FrameSource("synthetic://64x48x3", 1)], 4)
    batches = list(mux)
    assert sum(len(b) for b in batches) == 8
    assert [f.stream_id for f in batches[0]] == [0, 1, 0, 1]


def test_pipeline_tracks_across_frames(tmp_path):
    cfg = {
        "app": {"type": "video_analytics", "enable-perf-measurement": True, "perf-measurement-interval-sec": 0},
        "nvurisrcbin_list": {"uri-list": ["synthetic://160x120x12", "synthetic://160x120x12"]},
        "nvstreammux": {"batch-size": 2, "width": 160, "height": 120},
        "fdinfer": {"model": "blob"},
        "fdtracker": {"det-thresh": 0.3},
        "nvmultistreamtiler": {"rows": 1, "columns": 2, "width": 160, "height": 60},
        "nvosdbin": {},
        "filesink": {"location": str(tmp_path / "out.npy")},
    }
    s = FDStreamer()
    assert s.Init(cfg, BlobDetector())
    assert "nvstreammux batch-size=2" in s.describe() and " ! " in s.describe()
    s.Run()
    assert len(s.results) == 24 and len(s.tiled) == 12 and s.tiled[0].shape == (60, 160, 3)
    for sid in (0, 1):
        ids = [int(f.tracks[0, 4]) for f in s.results if f.stream_id == sid and f.tracks is not None and len(f.tracks)]
        assert len(ids) >= 9 and len(set(ids)) == 1          # one identity per stream, kept over time
    assert np.load(str(tmp_path / "out.npy")).shape == (12, 60, 160, 3)
    assert s.perf.history and s.perf.history[0] > 0
