"""The import-compatible public surface: top-level names, the ``C`` namespace, visualisers, custom Python processors."""
import math
import os

import numpy as np
import pytest

import fastdeploy_b200 as fd
from fastdeploy_b200.vision.result import (FaceAlignmentResult, HeadPoseResult, MattingResult, PerceptionResult,
                                           SegmentationResult)


def test_names_of_the_reference_package_resolve():
    top = ("ModelFormat Backend FDDataType TensorInfo Device is_built_with_gpu is_built_with_ort is_built_with_paddle "
           "is_built_with_trt get_default_cuda_directory set_logger Runtime RuntimeOption FastDeployModel C vision pipeline "
           "text encryption download download_and_decompress download_model get_model_list serving __version__").split()
    assert [n for n in top if not hasattr(fd, n)] == []
    vision = ("detection classification segmentation tracking keypointdetection matting facedet facealign faceid ocr headpose "
              "sr evaluation generation perception fd_result_to_json enable_flycv disable_flycv vis_detection vis_perception "
              "vis_keypoint_detection vis_face_detection vis_face_alignment vis_segmentation vis_matting_alpha vis_matting "
              "swap_background_matting swap_background_segmentation swap_background vis_ppocr vis_mot vis_headpose").split()
    assert [n for n in vision if not hasattr(fd.vision, n)] == []
    from fastdeploy_b200.vision.common import manager, processors
    assert hasattr(manager, "ProcessorManager") and hasattr(manager, "PyProcessorManager")
    for n in "ResizeByShort CenterCrop Pad NormalizeAndPermute Cast HWC2CHW Normalize PadToSize Resize StridePad".split():
        assert hasattr(processors, n), n
    assert fd.C.vision.DetectionResult is fd.vision.DetectionResult and fd.C.Runtime is fd.Runtime
    assert fd.C.vision.processors.Resize is processors.Resize
    assert fd.C.vision.Visualize.swap_background_matting is fd.vision.swap_background_matting
    fd.vision.enable_flycv(); fd.vision.disable_flycv()


def test_custom_python_processor_runs_on_a_batch(capsys):
    from fastdeploy_b200.vision.common.manager import PyProcessorManager
    from fastdeploy_b200.vision.common.processors import CenterCrop, NormalizeAndPermute, Pad, PadToSize, ResizeByShort

    class Custom(PyProcessorManager):
        def __init__(self):
            super().__init__()
            self.short = ResizeByShort(target_size=100, interp=1, use_scale=True, max_hw=[500, 500])
            self.crop = CenterCrop(width=50, height=50)
            self.pad = Pad(top=5, bottom=5, left=5, right=5, value=[225, 225, 225])
            self.to_size = PadToSize(height=160, width=160, value=[225, 225, 225])
            self.norm = NormalizeAndPermute(mean=[0.485, 0.456, 0.406], std=[0.229, 0.224, 0.225], is_scale=True)

        def apply(self, image_batch):
            for op in (self.short, self.crop, self.pad, self.to_size, self.norm):
                assert op(image_batch)
            return [m for m in image_batch.mats]

    rng = np.random.default_rng(0)
    mats = [fd.C.vision.FDMat().from_numpy(rng.integers(0, 255, (120, 200, 3), dtype=np.uint8)),
            fd.C.vision.FDMat().from_numpy(rng.integers(0, 255, (300, 150, 3), dtype=np.uint8))]
    mats[0].print_info("images0")
    assert "images0: DataType=uint8, Channel=3, Height=120, Width=200, Mean=" in capsys.readouterr().out
    pre = Custom()
    pre.use_cuda(True, -1)
    assert pre.cuda_used()
    outs = pre(mats)
    assert len(outs) == 2 and all(o.mat.shape == (3, 160, 160) and o.mat.dtype == np.float32 for o in outs)
    # the padded border is the pad value, normalised
    want = (225 / 255 - 0.485) / 0.229
    assert abs(float(outs[0].mat[0, -1, -1]) - want) < 1e-5
    outs[0].print_info("out")
    assert "Channel=3, Height=160, Width=160" in capsys.readouterr().out
    with pytest.raises(TypeError):
        PyProcessorManager()                     # abstract


def test_headpose_axes_and_landmark_dots():
    from fastdeploy_b200.vision import visualize as V
    ends = V.headpose_axes([0.0, 0.0, 0.0], 50, (100, 80))
    assert ends.tolist() == [[150, 80], [100, 130], [100, 80]]
    ends = V.headpose_axes([0.0, 90.0, 0.0], 50, (100, 80))       # yaw turns the Z axis into the image plane, mirrored
    assert ends[2].tolist() == [50, 80] and abs(ends[0][0] - 100) <= 1
    p, y, r = 10.0, 20.0, 30.0
    pr, yr, rr = math.radians(p), -math.radians(y), math.radians(r)
    ends = V.headpose_axes([p, y, r], 40, (0, 0))
    assert ends[0].tolist() == [int(40 * math.cos(yr) * math.cos(rr)),
                                int(40 * (math.cos(pr) * math.sin(rr) + math.cos(rr) * math.sin(pr) * math.sin(yr)))]
    im = np.zeros((60, 60, 3), np.uint8)
    hp = HeadPoseResult(); hp.euler_angles = [0.0, 0.0, 0.0]
    out = fd.vision.vis_headpose(im, hp, size=20, line_size=1)
    assert out[30, 45].tolist() == [0, 0, 255] and out[45, 30].tolist() == [0, 255, 0] and im.sum() == 0
    fa = FaceAlignmentResult(); fa.landmarks = [[10.7, 20.2], [40, 41]]
    out = fd.vision.vis_face_alignment(im, fa, line_size=2)
    assert out[20, 10].tolist() == [0, 255, 0] and out[41, 40].tolist() == [0, 255, 0] and out[0, 0].sum() == 0


def test_perception_boxes_project_through_the_camera_matrix(tmp_path):
    from fastdeploy_b200.vision import visualize as V
    r = PerceptionResult()
    r.scores, r.label_ids = [0.9, 0.2], [1, 2]
    r.boxes = [[0, 0, 0, 0, 1.5, 1.6, 4.0], [0, 0, 0, 0, 1.0, 1.0, 1.0]]       # h, w, l in columns 4..6
    r.center = [[1.0, 1.0, 10.0], [0.0, 0.0, 5.0]]
    r.yaw_angle = [0.0, 0.3]
    k = [700.0, 0, 320, 0, 700.0, 180, 0, 0, 1]
    c = V.project_boxes_3d(r, k)
    assert c.shape == (2, 8, 2)
    # yaw 0: corner 0 is (-l/2, -h, -w/2) from the bottom centre
    x, y, z = 1.0 - 2.0, 1.0 - 1.5, 10.0 - 0.8
    assert np.allclose(c[0, 0], [700 * x / z + 320, 700 * y / z + 180], atol=1e-3)
    # the turned box against a per-corner evaluation of the same rotation
    ry, (h, w, l) = 0.3, (1.0, 1.0, 1.0)
    xs = np.array([0, l, l, l, l, 0, 0, 0]) - l / 2
    ys = np.array([0, 0, h, h, 0, 0, h, h]) - h
    zs = np.array([0, 0, 0, w, w, w, w, 0]) - w / 2
    rot = np.array([[math.cos(ry), 0, math.sin(ry)], [0, 1, 0], [math.sin(ry), 0, math.cos(ry)]])
    pts = rot @ np.stack([xs, ys, zs]) + np.array([[0.0], [0.0], [5.0]])
    proj = np.array(k).reshape(3, 3) @ pts
    assert np.allclose(c[1], (proj[:2] / proj[2]).T, atol=1e-3)
    cfg = tmp_path / "infer_cfg.yml"
    cfg.write_text("k_data: [700.0, 0, 320, 0, 700.0, 180, 0, 0, 1]\nPreprocess:\n- type: Resize\n  target_size: [360, 640]\n")
    im = np.zeros((720, 1280, 3), np.uint8)
    out = fd.vision.vis_perception(im, r, str(cfg))
    assert out.shape == (360, 640, 3) and out.any()
    lo, hi = c[0].min(0), c[0].max(0)
    ys_, xs_ = np.nonzero(out.any(2))
    assert xs_.min() >= int(lo[0]) - 1 and xs_.max() <= max(int(hi[0]) + 1, int(lo[0]) + 80)     # drawing + caption only
    only_low = PerceptionResult()
    only_low.scores, only_low.label_ids, only_low.boxes, only_low.center, only_low.yaw_angle = [0.2], [2], [r.boxes[1]], [r.center[1]], [0.3]
    assert not fd.vision.vis_perception(im, only_low, str(cfg)).any()
    bad = tmp_path / "bad.yml"
    bad.write_text("k_data: [1, 2, 3]\n")
    with pytest.raises(ValueError, match="k_data"):
        fd.vision.vis_perception(im, r, str(bad))


def test_deprecated_visualiser_names_still_work(capsys):
    im = np.full((8, 8, 3), 200, np.uint8)
    bg = np.zeros((8, 8, 3), np.uint8)
    m = MattingResult(); m.alpha = [1.0] * 32 + [0.0] * 32; m.shape = [8, 8]
    a = fd.vision.swap_background_matting(im, bg, m)
    assert np.array_equal(a, fd.vision.swap_background(im, bg, m)) and a[0, 0, 0] == 200 and a[7, 7, 0] == 0
    s = SegmentationResult(); s.label_map = [0] * 32 + [3] * 32; s.shape = [8, 8]
    b = fd.vision.swap_background_segmentation(im, bg, 0, s)
    assert b[0, 0, 0] == 0 and b[7, 7, 0] == 200
    assert np.array_equal(fd.vision.vis_matting_alpha(im, m), fd.vision.vis_matting(im, m))
    assert capsys.readouterr().out.count("DEPRECATED") == 3
    with pytest.raises(AssertionError):
        fd.vision.swap_background_matting(im, bg, s)


def test_model_list_comes_from_the_local_cache(tmp_path, monkeypatch):
    monkeypatch.setenv("FASTDEPLOY_MODEL_CACHE", str(tmp_path))
    assert fd.get_model_list() == {}
    (tmp_path / "ppyoloe_crn_l_300e_coco").mkdir()
    (tmp_path / "ResNet50_vd_infer.tgz").write_bytes(b"")
    assert fd.get_model_list() == {"local": [{"name": "ResNet50_vd_infer"}, {"name": "ppyoloe_crn_l_300e_coco"}]}
    (tmp_path / "index.json").write_text('{"detection": [{"name": "ppyoloe_crn_l_300e_coco", "format": "paddle"}], "ocr": []}')
    assert list(fd.get_model_list()) == ["detection", "ocr"]
    assert fd.get_model_list("detection") == {"detection": [{"name": "ppyoloe_crn_l_300e_coco", "format": "paddle"}]}
    with pytest.raises(ValueError, match="No pretrained model in category"):
        fd.get_model_list("audio")


def test_example_image_and_hub_directories(tmp_path, monkeypatch):
    import importlib
    import cv2
    monkeypatch.setenv("HUB_HOME", str(tmp_path / "hub"))
    monkeypatch.setenv("FASTDEPLOY_MODEL_CACHE", str(tmp_path / "cache"))
    from fastdeploy_b200.utils import hub_env
    importlib.reload(hub_env)
    assert hub_env.MODEL_HOME == str(tmp_path / "hub" / "models") and not os.path.exists(hub_env.HUB_HOME)   # nothing created
    p = fd.utils.get_detection_test_image()
    assert p == str(tmp_path / "hub" / "resources" / "detection_test_image.jpg") and cv2.imread(p).shape == (720, 1280, 3)
    first = os.path.getmtime(p)
    assert fd.utils.get_detection_test_image() == p and os.path.getmtime(p) == first                           # kept, not redrawn
    (tmp_path / "cache").mkdir()
    cv2.imwrite(str(tmp_path / "cache" / "detection_test_image.jpg"), np.zeros((8, 8, 3), np.uint8))
    q = fd.utils.get_detection_test_image(str(tmp_path / "elsewhere"))
    assert cv2.imread(q).shape == (8, 8, 3)                                                                    # the cached file wins
    monkeypatch.delenv("HUB_HOME")
    importlib.reload(hub_env)


def test_results_round_trip_through_json():
    import json
    U = fd.vision.utils
    R = fd.vision
    d = R.DetectionResult()
    d.boxes, d.scores, d.label_ids, d.contain_masks = [[1.0, 2.0, 3.0, 4.0]], [0.5], [7], True
    m = R.Mask(); m.data, m.shape = [0, 1, 1, 0], [2, 2]
    d.masks = [m]
    text = U.detection_to_json(d)
    parsed = json.loads(text)
    assert parsed["boxes"] == [[1.0, 2.0, 3.0, 4.0]] and json.loads(parsed["masks"][0]) == {"data": [0, 1, 1, 0], "shape": [2, 2]}
    back = U.json_to_detection(parsed)
    assert back.boxes == d.boxes and back.label_ids == [7] and back.masks[0].shape == [2, 2] and back.contain_masks
    assert U.json_to_detection(text).scores == [0.5]                      # the text form is taken as well
    o = R.OCRResult()
    o.boxes, o.text, o.rec_scores = [[0, 0, 5, 0, 5, 5, 0, 5]], ["héllo"], [0.9]
    assert U.json_to_ocr(U.ocr_to_json(o)).text == ["héllo"]
    s = R.SegmentationResult()
    s.label_map, s.shape = np.array([0, 1, 2, 1], np.uint8).tolist(), [2, 2]
    assert U.json_to_segmentation(U.segmentation_to_json(s)).label_map == [0, 1, 2, 1]
    for kind, cls in (("perception", "PerceptionResult"), ("classify", "ClassifyResult"), ("keypoint", "KeyPointDetectionResult"),
                      ("mot", "MOTResult"), ("face_detection", "FaceDetectionResult"), ("face_alignment", "FaceAlignmentResult"),
                      ("face_recognition", "FaceRecognitionResult"), ("matting", "MattingResult"), ("head_pose", "HeadPoseResult")):
        obj = getattr(R, cls)()
        again = getattr(U, f"json_to_{kind}")(getattr(U, f"{kind}_to_json")(obj))
        assert type(again) is type(obj) and again.__dict__ == obj.__dict__, kind
    h = R.HeadPoseResult(); h.euler_angles = [np.float32(1.5), 2.0, 3.0]
    assert json.loads(U.head_pose_to_json(h))["euler_angles"] == [1.5, 2.0, 3.0]


def test_generic_result_serialiser_uses_the_per_type_layout():
    import json
    U, R = fd.vision.utils, fd.vision
    d = R.DetectionResult()
    d.boxes, d.scores, d.label_ids, d.contain_masks = [[1.0, 2.0, 3.0, 4.0]], [np.float32(0.5)], [7], True
    m = R.Mask(); m.data, m.shape = [1, 0], [1, 2]
    d.masks = [m]
    parsed = json.loads(U.fd_result_to_json(d))
    assert parsed["type"] == "DetectionResult" and isinstance(parsed["masks"][0], str) and parsed["scores"] == [0.5]
    assert U.json_to_detection(parsed).masks[0].data == [1, 0]
    both = json.loads(U.fd_result_to_json([d, R.ClassifyResult(label_ids=[1], scores=[0.25])]))
    assert [b["type"] for b in both] == ["DetectionResult", "ClassifyResult"]
    with pytest.raises(TypeError):
        U.fd_result_to_json(3)
