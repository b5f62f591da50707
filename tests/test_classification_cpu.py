"""PaddleClas classifier, PP-ShiTuV2 recogniser and the ONNX ResNet through the CPU runtime."""
import numpy as np
import pytest

import fastdeploy_b200 as fd
from fastdeploy_b200.models.vit import write_vit


@pytest.fixture(scope="module")
def vit(tmp_path_factory):
    return write_vit(str(tmp_path_factory.mktemp("vit")), "tiny", image=32, num_classes=10, seed=3)


def _opt():
    o = fd.RuntimeOption()
    o.use_cpu()
    return o


def _images(n=3):
    rng = np.random.default_rng(0)
    return [rng.integers(0, 255, (40 + 7 * i, 60 - 5 * i, 3), dtype=np.uint8) for i in range(n)]


def test_paddleclas_model_topk_matches_the_graph_on_preprocessed_pixels(vit):
    m = fd.vision.classification.PaddleClasModel(vit["model"], vit["params"], vit["config"], runtime_option=_opt())
    ims = _images()
    res = m.batch_predict(ims)
    assert len(res) == 3
    x = m.preprocessor.run(ims)[0]
    assert x.shape == (3, 3, 32, 32) and x.dtype == np.float32
    logits = fd.Runtime(_rt_opt(vit)).infer({m.runtime.get_input_info(0).name: x})[0]
    for r, row in zip(res, logits):
        assert r.label_ids == [int(np.argmax(row))] and abs(r.scores[0] - float(row.max())) < 1e-5      # no softmax
    top3 = m.predict(ims[0], topk=3)
    assert top3.label_ids == np.argsort(-logits[0], kind="stable")[:3].tolist()
    assert "ClassifyResult" in str(top3)


def _rt_opt(vit):
    o = _opt()
    o.set_model_path(vit["model"], vit["params"], fd.ModelFormat.PADDLE)
    return o


def test_preprocessor_switches(vit):
    from fastdeploy_b200.vision.classification import PaddleClasPreprocessor
    ims = _images(1)
    base = PaddleClasPreprocessor(vit["config"]).run(ims)[0]
    p = PaddleClasPreprocessor(vit["config"])
    p.disable_permute()
    hwc = p.run(ims)[0]
    assert hwc.shape == (1, 32, 32, 3) and np.allclose(hwc.transpose(0, 3, 1, 2), base, atol=1e-6)
    p = PaddleClasPreprocessor(vit["config"])
    p.disable_normalize()
    raw = p.run(ims)[0]
    assert raw.shape == (1, 3, 32, 32)
    assert np.allclose((raw.astype(np.float32) / 255 - 0.5) / 0.5, base, atol=1e-5)     # the yaml's mean / std are 0.5
    p.initial_resize_on_cpu(True)
    assert np.array_equal(p.run(ims)[0], raw)


def test_ppshitu_recognizer_gives_unit_features(vit):
    cls = fd.vision.classification
    m = cls.PPShiTuV2Recognizer(vit["model"], vit["params"], vit["config"], runtime_option=_opt())
    assert isinstance(m.preprocessor, cls.PPShiTuV2RecognizerPreprocessor)
    assert isinstance(m.postprocessor, cls.PPShiTuV2RecognizerPostprocessor)
    ims = _images(2)
    res = m.batch_predict(ims)
    feats = np.asarray([r.feature for r in res], np.float32)
    assert feats.shape == (2, 10) and np.allclose(np.linalg.norm(feats, axis=1), 1.0, atol=1e-5)
    m.feature_norm = False
    raw = np.asarray([r.feature for r in m.batch_predict(ims)], np.float32)
    assert np.allclose(raw / np.linalg.norm(raw, axis=1, keepdims=True), feats, atol=1e-5)
    assert not np.allclose(np.linalg.norm(raw, axis=1), 1.0, atol=1e-3)
    one = m.predict(ims[0])
    assert len(one.feature) == 10 and one.label_ids == []
    post = cls.PPShiTuV2RecognizerPostprocessor()
    out = post.run([np.array([[3.0, 4.0]], np.float32)])
    assert np.allclose(out[0].feature, [0.6, 0.8])


def test_onnx_resnet_softmax_topk(tmp_path):
    from fastdeploy_b200.models.resnet import resnet18_like_onnx
    path = str(tmp_path / "r.onnx")
    resnet18_like_onnx(path, seed=1, num_classes=7, width=8)
    m = fd.vision.classification.ResNet(path, runtime_option=_opt())
    m.size = [64, 64]
    m._rebuild()
    r = m.predict(_images(1)[0], topk=7)
    assert sorted(r.label_ids) == list(range(7)) and abs(sum(r.scores) - 1.0) < 1e-4
    assert r.scores == sorted(r.scores, reverse=True)


def test_yolov5cls_centre_crops_before_resizing(tmp_path):
    from fastdeploy_b200.models.resnet import resnet18_like_onnx
    cls = fd.vision.classification
    pre = cls.YOLOv5ClsPreprocessor()
    pre.size = [32, 32]
    im = np.zeros((40, 100, 3), np.uint8)
    im[:, 30:70] = 255                                   # the centre 40 x 40 square is white, the sides black
    x, infos = pre.run([im])
    assert x.shape == (1, 3, 32, 32) and infos[0] == {"input_shape": [40.0, 100.0], "output_shape": [32.0, 32.0]}
    assert np.allclose(x[0, 0], (1.0 - 0.485) / 0.229, atol=1e-5)          # only the white square is left
    path = str(tmp_path / "c.onnx")
    resnet18_like_onnx(path, seed=2, num_classes=5, width=8)
    m = cls.YOLOv5Cls(path, runtime_option=_opt())
    assert isinstance(m.postprocessor, cls.YOLOv5ClsPostprocessor)
    m.size = [64, 64]
    r = m.predict(_images(1)[0], topk=5)
    assert sorted(r.label_ids) == list(range(5)) and abs(sum(r.scores) - 1.0) < 1e-4
