"""Pieces of the vision package's public surface with no test elsewhere: perception processors, trail recorder, evaluation
dataset readers, face-recognition and style-transfer processor classes, segmentation / key-point switches."""
import json
import os

import numpy as np
import pytest

import fastdeploy_b200 as fd

V = fd.vision


def test_perception_processors_and_batches(tmp_path):
    cfg = tmp_path / "infer_cfg.yml"
    cfg.write_text("Preprocess:\n- type: Resize\n  target_size: [32, 64]\n- type: NormalizeImage\n  mean: [0.5, 0.5, 0.5]\n  std: [0.5, 0.5, 0.5]\n")
    pre = V.perception.SmokePreprocessor(str(cfg))
    assert pre.size == [64, 32]
    x = pre.run([np.full((48, 96, 3), 255, np.uint8)] * 2)
    assert x.shape == (2, 3, 32, 64) and np.allclose(x, 1.0)
    rows = np.zeros((3, 14), np.float32)
    rows[0] = [2, 0.1, 10, 20, 30, 40, 1.5, 1.6, 4.0, 1, 2, 30, 0.3, 0.9]
    rows[1, 13] = 0.1
    post = V.perception.SmokePostprocessor()
    r = post.run([rows])[0]
    assert r.label_ids == [2] and r.boxes[0] == pytest.approx([10, 20, 30, 40, 1.5, 1.6, 4.0]) and r.center[0] == [1, 2, 30]
    assert r.yaw_angle[0] == pytest.approx(0.3) and r.observation_angle[0] == pytest.approx(0.1)
    b = np.arange(18, dtype=np.float32).reshape(2, 9)
    r = V.perception.PetrPostprocessor().run([b, np.array([0.9, 0.1], np.float32), np.array([3, 4])])[0]
    assert r.label_ids == [3] and r.velocity == [[6.0, 7.0]] and r.boxes[0][-1] == 8.0
    r = V.perception.CaddnPostprocessor().run([b[:, :7], np.array([1, 2]), np.array([0.9, 0.8], np.float32)])[0]
    assert r.label_ids == [1, 2] and len(r.boxes[0]) == 7
    # batches: one predict per item, extras per item or shared
    calls = []

    class Fake(V.perception.Smoke):
        def __init__(self): pass
        def predict(self, im, k=None):
            calls.append((im, k))
            return len(calls)

    assert Fake().batch_predict(["a", "b"], ["k1", "k2"]) == [1, 2] and calls == [("a", "k1"), ("b", "k2")]
    cp = V.perception.CenterpointPreprocessor()
    pts = np.array([[0.05, 0.05, 0.0, 1.0], [0.06, 0.04, 0.1, 1.0], [10.0, 10.0, 0.0, 1.0], [999.0, 0, 0, 1.0]], np.float32)
    voxels, coords, num = cp.voxelize(pts)
    assert int(np.asarray(num).sum()) == 3 and len(np.asarray(num)) == 2          # two voxels, the far point dropped
    sweep = np.arange(20, dtype=np.float32).reshape(4, 5)
    path = tmp_path / "sweep.bin"
    sweep.tofile(path)
    got = cp.run([str(path)], 5, 0)[0]
    assert got.shape == (4, 5) and np.array_equal(got[:, :4], sweep[:, :4]) and (got[:, 4] == 0).all()
    assert np.array_equal(cp.run([str(path)], 5, 1)[0], sweep)                    # the model uses the time lag: kept
    with pytest.raises(ValueError, match="divisible"):
        cp.run([str(path)], 6, 0)
    imgs, cam, lidar = V.perception.CaddnPreprocessor(str(cfg)).run([np.zeros((48, 96, 3), np.uint8)] * 2, list(range(12)), list(range(16)))
    assert imgs.shape == (2, 3, 32, 64) and cam.shape == (2, 3, 4) and lidar.shape == (2, 4, 4) and cam[1, 2, 3] == 11


def test_trail_recorder_and_mot_drawing():
    rec = V.tracking.TrailRecorder()
    rec.add(7, [10, 12]); rec.Add(7, (14, 16)); rec.add(9, [40, 40])
    assert rec.records == {7: [[10, 12], [14, 16]], 9: [[40, 40]]}
    m = V.tracking.PPTracking.__new__(V.tracking.PPTracking)
    m.recorder = None
    m.bind_recorder(rec)
    assert m.recorder is rec
    m.unbind_recorder()
    assert m.recorder is None
    res = V.MOTResult()
    res.boxes, res.ids, res.scores, res.class_ids = [[30, 30, 50, 50]], [7], [0.9], [0]
    im = np.zeros((64, 64, 3), np.uint8)
    plain = V.vis_mot(im, res)
    trails = V.vis_mot(im, res, records=rec)
    assert plain[12, 10].sum() == 0 and trails[12, 10].sum() > 0 and trails[16, 14].sum() > 0
    assert trails[40, 40].sum() == plain[40, 40].sum()                            # id 9 is not on this frame


def test_coco_and_cityscapes_readers(tmp_path):
    import cv2
    ev = V.evaluation
    img_dir = tmp_path / "images"
    img_dir.mkdir()
    for i in range(3):
        cv2.imwrite(str(img_dir / f"{i}.png"), np.full((20, 30, 3), 10 * i, np.uint8))
    ann = {"images": [{"id": 5 + i, "file_name": f"{i}.png", "height": 20, "width": 30} for i in range(3)],
           "categories": [{"id": 18, "name": "dog"}, {"id": 3, "name": "car"}],
           "annotations": [{"id": 1, "image_id": 5, "category_id": 18, "bbox": [2, 3, 10, 8], "iscrowd": 0},
                           {"id": 2, "image_id": 5, "category_id": 3, "bbox": [1, 1, 5, 5]},
                           {"id": 3, "image_id": 6, "category_id": 3, "bbox": [4, 4, 6, 6]},
                           {"id": 4, "image_id": 7, "category_id": 3, "bbox": [0, 0, 0, 6]}]}
    (tmp_path / "ann.json").write_text(json.dumps(ann))
    ds = ev.CocoDetection(str(img_dir), str(tmp_path / "ann.json"))
    assert len(ds) == 2 and ds.labels == ["car", "dog"] and ds.clsid2catid == {0: 3, 1: 18}     # the empty image is left out
    assert ds.file_list[0]["boxes"] == [[2, 3, 12, 11], [1, 1, 6, 6]] and ds.file_list[0]["labels"] == [1, 0]
    assert len(ev.CocoDetection(str(img_dir), str(tmp_path / "ann.json"), allow_empty=True)) == 3
    im, gt = next(iter(ds))
    assert im.shape == (20, 30, 3) and gt["labels"] == [1, 0]
    metric = ev.COCOMetric(ds)
    for rec in ds.file_list:                              # perfect detections
        metric.update(rec["im_id"], {"boxes": rec["boxes"], "labels": rec["labels"], "scores": [0.9] * len(rec["labels"])})
    assert metric.get()["bbox_mmap"] == pytest.approx(1.0)
    metric.reset()
    d = V.DetectionResult()
    d.boxes, d.label_ids, d.scores = [[0, 0, 1, 1]], [0], [0.9]
    metric.update(5, d)
    assert metric.get()["bbox_mmap"] == pytest.approx(0.0)
    root = tmp_path / "city"
    for sub, suffix in (("leftImg8bit", "_leftImg8bit.png"), ("gtFine", "_gtFine_labelTrainIds.png")):
        d_ = root / sub / "val" / "aachen"
        d_.mkdir(parents=True)
        for n in ("a_000", "a_001"):
            cv2.imwrite(str(d_ / (n + suffix)), np.full((8, 8, 3) if sub == "leftImg8bit" else (8, 8), 3, np.uint8))
    cs = ev.Cityscapes(str(root), "val")
    assert len(cs) == 2 and cs.num_classes == 19 and cs.ignore_index == 255
    assert os.path.basename(cs.file_list[1][0]) == "a_001_leftImg8bit.png" and cs.file_list[1][1].endswith("a_001_gtFine_labelTrainIds.png")
    image, label = next(iter(cs))
    assert image.shape == (8, 8, 3) and label.shape == (8, 8) and int(label[0, 0]) == 3
    with pytest.raises(ValueError, match="mode"):
        ev.Cityscapes(str(root), "all")


def test_face_recognition_and_style_transfer_processors():
    fid = V.faceid
    im = np.random.default_rng(0).integers(0, 255, (112, 112, 3), dtype=np.uint8)
    base = fid.InsightFaceRecognitionPreprocessor().run([im])
    ada = fid.AdaFacePreprocessor().run([im])
    assert np.allclose(ada[:, ::-1], base)                      # same numbers, channels not swapped
    p = fid.InsightFaceRecognitionPreprocessor(); p.disable_normalize(); p.disable_permute()
    raw = p.run([im])
    assert raw.shape == (1, 112, 112, 3) and np.array_equal(raw[0], im[..., ::-1].astype(np.float32))
    post = fid.AdaFacePostprocessor(); post.l2_normalize = True
    assert np.allclose(post.run(np.array([[3.0, 4.0]], np.float32))[0].embedding, [0.6, 0.8])
    g = V.generation
    x = g.AnimeGANPreprocessor().run([im])
    assert x.shape == (1, 3, 112, 112) and -1.0 <= x.min() and x.max() <= 1.0
    back = g.AnimeGANPostprocessor().run([x])
    assert np.array_equal(back[0], im)                          # the two halves are inverses of each other
    nhwc = g.AnimeGANPreprocessor(); nhwc.nhwc = True
    assert nhwc.run([im]).shape == (1, 112, 112, 3)


def test_segmentation_preprocessor_switches(tmp_path):
    cfg = tmp_path / "deploy.yaml"
    cfg.write_text("Deploy:\n  transforms:\n  - type: Resize\n    target_size: [32, 16]\n  - type: Normalize\n    mean: [0.5, 0.5, 0.5]\n    std: [0.5, 0.5, 0.5]\n")
    from fastdeploy_b200.vision.segmentation import PaddleSegPreprocessor
    im = np.random.default_rng(1).integers(0, 255, (40, 50, 3), dtype=np.uint8)
    base = PaddleSegPreprocessor(str(cfg)).run([im])[0]
    assert base.shape == (1, 3, 16, 32)
    p = PaddleSegPreprocessor(str(cfg)); p.disable_permute()
    assert np.allclose(p.run([im])[0].transpose(0, 3, 1, 2), base, atol=1e-6)
    p = PaddleSegPreprocessor(str(cfg)); p.disable_normalize()
    raw = p.run([im])[0]
    assert np.allclose((raw.astype(np.float32) / 255.0 - 0.5) / 0.5, base, atol=1e-5)
