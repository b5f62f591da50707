"""The YOLO-family classes through the CPU runtime: named pre/post-processors, the attributes older releases had on the
model, FastestDet and YOLOv5Seg with their own post-processors."""
import numpy as np
import pytest

import fastdeploy_b200 as fd
from fastdeploy_b200.importer.onnx_format import save_onnx
from fastdeploy_b200.ir.graph import Graph

det = fd.vision.detection


def _opt():
    o = fd.RuntimeOption()
    o.use_cpu()
    return o


def _head_model(path, size, rows, outputs=1, seed=0):
    """A graph whose output does not depend on the picture: `rows` [n, c] (and optional protos) added to 0 * mean(input)."""
    g = Graph("head", opset=13)
    x = g.add_input("images", "float32", ["N", 3, size, size])
    zero = g.op("Mul", g.op("ReduceMean", x, axes=[1, 2, 3], keepdims=1), g.add_initializer("zero", np.zeros(1, np.float32)))
    names = []
    for k, r in enumerate(rows if outputs > 1 else [rows]):
        r = np.asarray(r, np.float32)
        flat = g.op("Reshape", zero, g.add_initializer(f"shape{k}", np.array([-1] + [1] * r.ndim, np.int64)))
        y = g.op("Add", flat, g.add_initializer(f"rows{k}", r[None]))
        g.nodes[-1].outputs = [f"out{k}"]
        g.add_output(f"out{k}", "float32", ["N"] + list(r.shape))
        names.append(y)
    with open(path, "wb") as f:
        f.write(save_onnx(g))
    return path


def test_yolov5_named_processors_and_legacy_attributes(tmp_path):
    rows = np.zeros((6, 85), np.float32)
    rows[0, :5] = [160, 160, 60, 40, 0.9]; rows[0, 5 + 2] = 0.9
    rows[1, :5] = [60, 80, 30, 30, 0.8]; rows[1, 5 + 5] = 0.7
    m = det.YOLOv5(_head_model(str(tmp_path / "y5.onnx"), 320, rows), runtime_option=_opt())
    assert isinstance(m.preprocessor, det.YOLOv5Preprocessor) and isinstance(m.postprocessor, det.YOLOv5Postprocessor)
    assert m.size == [640, 640] and m.padding_value == [114.0, 114.0, 114.0] and m.stride == 32 and m.max_wh == 7680.0
    assert m.is_scale_up and not m.is_mini_pad and not m.is_no_pad and m.multi_label
    m.size = [320, 320]
    assert m.preprocessor.size == [320, 320]
    m.is_scale_up = False
    assert m.preprocessor.is_scale_up is False
    im = np.zeros((320, 320, 3), np.uint8)
    r = m.predict(im)
    assert sorted(r.label_ids) == [2, 5]
    assert np.allclose(r.boxes[r.label_ids.index(2)], [130, 140, 190, 180], atol=1e-3)
    r = m.predict(im, conf_threshold=0.7)
    assert r.label_ids == [2] and m.conf_threshold == 0.7
    # the processors also work on their own, as in the reference's two-step usage
    x, infos = det.YOLOv5Preprocessor().run([np.zeros((480, 640, 3), np.uint8)])
    assert x.shape == (1, 3, 640, 640) and infos[0]["pad_h"] == 80
    post = det.YOLOv5Postprocessor()
    assert post.kind == "v5" and post.conf_threshold == 0.25 and det.YOLOv8Postprocessor().kind == "v8"
    assert det.YOLOX.downsample_strides.fget is not None and det.YOLOv5Lite.anchor_config.fget is not None
    assert isinstance(det.NMSRotatedOption().nms_top_k, int) and det.NMSRotatedOption().nms_threshold == 0.1


def test_fastestdet_post_processor_decodes_the_grid(tmp_path):
    out = np.full((5 + 3, 22, 22), -10.0, np.float32)       # logits already through sigmoid in the export: use small values
    out[:] = 0.0
    out[0, 11, 11] = 0.95                                     # objectness
    out[3, 11, 11] = 0.0; out[4, 11, 11] = 0.0               # sigmoid(0) = 0.5 of the image in w and h
    out[5 + 1, 11, 11] = 0.9
    m = det.FastestDet(_head_model(str(tmp_path / "fd.onnx"), 352, out), runtime_option=_opt())
    assert isinstance(m.preprocessor, det.FastestDetPreprocessor) and isinstance(m.postprocessor, det.FastestDetPostprocessor)
    assert m.size == [352, 352] and m.conf_threshold == pytest.approx(0.65)
    r = m.predict(np.zeros((200, 400, 3), np.uint8))
    assert r.label_ids == [1] and len(r.boxes) == 1
    cx, cy = (11 + 0.0) / 22 * 400, (11 + 0.0) / 22 * 200
    assert np.allclose(r.boxes[0], [cx - 100, cy - 50, cx + 100, cy + 50], atol=1e-3)
    assert r.scores[0] == pytest.approx(0.95 ** 0.6 * 0.9 ** 0.4, rel=1e-5)


def test_yolov5seg_masks_come_from_the_post_processor(tmp_path):
    ncls, nm = 2, 32
    rows = np.zeros((4, 5 + ncls + nm), np.float32)
    rows[0, :5] = [32, 32, 32, 32, 0.9]; rows[0, 5 + 1] = 0.9; rows[0, 5 + ncls] = 8.0     # coefficient on proto 0
    protos = np.zeros((nm, 16, 16), np.float32)
    protos[0] = 1.0
    path = _head_model(str(tmp_path / "seg.onnx"), 64, [rows, protos], outputs=2)
    m = det.YOLOv5Seg(path, runtime_option=_opt())
    m.size = [64, 64]
    assert isinstance(m.postprocessor, det.YOLOv5SegPostprocessor) and m.mask_nums == 32 and m.mask_threshold == 0.5
    r = m.predict(np.zeros((64, 64, 3), np.uint8))
    assert r.label_ids == [1] and r.contain_masks and len(r.masks) == 1
    mask = np.asarray(r.masks[0].data).reshape(r.masks[0].shape)
    assert mask.shape == (64, 64) and mask[32, 32] == 1 and mask[2, 2] == 0 and mask[60, 60] == 0
    assert 700 < int(mask.sum()) < 1400                       # about the 32 x 32 box


def test_face_detector_processors_alone_and_through_the_model(tmp_path):
    fdet = fd.vision.facedet
    # standalone: CenterFace decode of one peak
    pre = fdet.CenterFacePreprocessor()
    assert pre.size == [640, 640]
    pre.size = [64, 64]
    x, infos = pre.run([np.zeros((64, 64, 3), np.uint8), np.zeros((32, 64, 3), np.uint8)])
    assert x.shape == (2, 3, 64, 64) and infos[1]["pad_h"] == 16
    heat = np.zeros((2, 1, 16, 16), np.float32); heat[0, 0, 8, 8] = 0.9
    scale = np.zeros((2, 2, 16, 16), np.float32)                      # exp(0) * 4 = 4 pixels
    offset = np.zeros((2, 2, 16, 16), np.float32)
    lms = np.full((2, 10, 16, 16), 0.5, np.float32)
    post = fdet.CenterFacePostprocessor()
    assert post.conf_threshold == 0.5 and post.nms_threshold == pytest.approx(0.3)
    res = post.run([heat, scale, offset, lms], infos)
    assert len(res) == 2 and len(res[0].boxes) == 1 and len(res[1].boxes) == 0
    assert np.allclose(res[0].boxes[0], [32, 32, 36, 36]) and np.allclose(res[0].landmarks[0], [34, 34])
    assert fdet.Yolov7FacePreprocessor().padding_value == [114.0, 114.0, 114.0]
    # through a model: the processors are views of the model's settings
    rows = np.array([[0, 0.9, 10, 12, 40, 44], [0, 0.3, 1, 1, 5, 5]], np.float32)
    cfg = tmp_path / "infer_cfg.yml"
    cfg.write_text("Preprocess:\n- type: Resize\n  target_size: [64, 64]\n")
    m = fdet.BlazeFace(_head_model(str(tmp_path / "bf.onnx"), 64, rows), "", str(cfg), runtime_option=_opt(),
                       model_format=fd.ModelFormat.ONNX)
    assert m.size == [64, 64]                               # from the yaml
    assert isinstance(m.preprocessor, fdet.BlazeFacePreprocessor) and isinstance(m.postprocessor, fdet.BlazeFacePostprocessor)
    m.postprocessor.conf_threshold = 0.2
    assert m.conf_threshold == 0.2
    r = m.predict(np.zeros((64, 64, 3), np.uint8))
    assert len(r.boxes) == 2
    m.postprocessor.conf_threshold = 0.5
    assert len(m.predict(np.zeros((64, 64, 3), np.uint8)).boxes) == 1
    # attributes of older releases
    s = fdet.SCRFD.__new__(fdet.SCRFD)
    fdet._defaults(s, s.SIZE); s._configure()
    assert s.downsample_strides == [8, 16, 32] and s.max_nms == 30000 and s.stride == 32 and not s.is_mini_pad
    a = s.preprocess(np.full((40, 64, 3), 255, np.uint8))[0]
    s.disable_normalize(); s.disable_permute()
    b = s.preprocess(np.full((40, 64, 3), 255, np.uint8))[0]
    assert a.shape == (1, 3, 640, 640) and b.shape == (1, 640, 640, 3) and b.max() == 255.0 and a.max() < 1.0
