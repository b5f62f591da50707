"""Public API on the CPU path: Runtime / RuntimeOption, PPYOLOE model class, NMS reference, results."""
import numpy as np
import pytest


def test_runtime_cpu_onnx(tmp_path):
    import fastdeploy_b200 as fd
    from fastdeploy_b200.models.resnet import resnet18_like_onnx
    path = str(tmp_path / "m.onnx")
    resnet18_like_onnx(path)
    opt = fd.RuntimeOption()
    opt.set_model_path(path, model_format=fd.ModelFormat.ONNX)
    opt.use_cpu()
    opt.use_ort_backend()
    rt = fd.Runtime(opt)
    assert rt.num_inputs() == 1 and rt.num_outputs() == 1
    info = rt.get_input_info(0)
    assert info.name == "input" and info.shape == [-1, 3, 64, 64] and info.dtype == fd.FDDataType.FP32
    x = np.random.RandomState(0).rand(2, 3, 64, 64).astype(np.float32)
    out = rt.infer({"input": x})
    assert out[0].shape == (2, 10)
    assert np.array_equal(out[0], rt.forward(x)[0])
    rt2 = rt.clone()
    assert np.array_equal(out[0], rt2.infer([x])[0])


def test_fddatatype_codes_match_paddle():
    import fastdeploy_b200 as fd
    assert [int(fd.FDDataType[n]) for n in ("BOOL", "INT16", "INT32", "INT64", "FP16", "FP32", "FP64", "UINT8", "INT8")] \
        == [0, 1, 2, 3, 4, 5, 6, 20, 21]


def test_ppyoloe_cpu_predict(tmp_path):
    import fastdeploy_b200 as fd
    from fastdeploy_b200.models.ppyoloe import write_ppyoloe
    paths = write_ppyoloe(str(tmp_path), "tiny", image=96, num_classes=6, score_threshold=0.005)
    opt = fd.RuntimeOption()
    opt.use_cpu()
    m = fd.vision.detection.PPYOLOE(paths["model"], paths["params"], paths["config"], runtime_option=opt)
    ims = [np.random.RandomState(i).randint(0, 256, (60 + 10 * i, 120, 3), dtype=np.uint8) for i in range(2)]
    rs = m.batch_predict(ims)
    assert len(rs) == 2
    for r in rs:
        assert len(r.boxes) == len(r.scores) == len(r.label_ids) <= 100
        assert r.Str().startswith("DetectionResult: [xmin, ymin, xmax, ymax, score, label_id]")
        assert all(0 <= l < 6 for l in r.label_ids)
    # grouped by class ascending, descending score inside a class
    r = rs[0]
    assert r.label_ids == sorted(r.label_ids)
    one = m.predict(ims[0])
    assert np.allclose(one.scores, rs[0].scores, atol=1e-6)


def test_preprocessor_matches_manual_pipeline(tmp_path):
    import cv2
    from fastdeploy_b200.models.ppyoloe import write_ppyoloe
    from fastdeploy_b200.vision.detection import PaddleDetPreprocessor
    paths = write_ppyoloe(str(tmp_path), "tiny", image=64, num_classes=4)
    pre = PaddleDetPreprocessor(paths["config"])
    im = np.random.RandomState(0).randint(0, 256, (90, 160, 3), dtype=np.uint8)
    img, sf, shape = pre.run([im])
    ref = cv2.resize(np.ascontiguousarray(im[..., ::-1]), (64, 64), interpolation=2).astype(np.float32) / 255.0
    assert img.shape == (1, 3, 64, 64)
    assert np.allclose(img[0].transpose(1, 2, 0), ref, atol=1e-6)
    assert np.allclose(sf, [[64 / 90, 64 / 160]])


def test_nms_reference_ties_and_topk():
    from fastdeploy_b200.ops.nms import multiclass_nms_reference
    boxes = np.array([[[0, 0, 10, 10], [1, 1, 11, 11], [20, 20, 30, 30], [20, 20, 30, 30], [50, 50, 60, 60]]], np.float32)
    scores = np.array([[[0.9, 0.8, 0.7, 0.7, 0.05], [0.1, 0.1, 0.6, 0.2, 0.95]]], np.float32)
    out, idx, num = multiclass_nms_reference(boxes, scores, 0.06, 0.5, 10, 3)
    # class 0 keeps boxes 0 and 2 (1 overlaps 0; 3 ties with 2 and is suppressed by it), class 1 keeps 4, 2, 0/1...
    assert num.tolist() == [3]
    assert out[:, 1].tolist() == pytest.approx([0.9, 0.7, 0.95])
    assert out[:, 0].tolist() == [0, 0, 1]
    assert idx.tolist() == [0, 2, 4]


def test_nonzero_device_status_raises_on_every_inference_path():
    """A kernel that gives up on a bounded wait writes a code to the plan's status word instead of trapping;
    ``Runtime.infer`` and ``FastDeployModel.infer`` must turn that into an exception for every model kind,
    not only for graphs with padded NMS outputs. Driven with a fake plan: no GPU involved."""
    import torch
    from fastdeploy_b200.ops.base import StatusWord
    from fastdeploy_b200.runtime.runtime import Runtime
    from fastdeploy_b200.runtime.model import FastDeployModel

    class FakeEvent:
        def synchronize(self):
            pass

    class FakePlan:
        def __init__(self):
            self.status = StatusWord.__new__(StatusWord)
            self.status.t = torch.zeros(1, dtype=torch.int32)

    rt = Runtime.__new__(Runtime)
    rt.on_gpu = True
    rt._last_plan = FakePlan()
    rt._status_event = FakeEvent()
    rt._status_host = torch.zeros(1, dtype=torch.int32)
    rt._check_status()                                  # zero word: fine
    rt._status_host[0] = 4
    with pytest.raises(RuntimeError, match="peer signal wait timed out"):
        rt._check_status()

    class Graph:
        inputs, outputs = [], []
    rt.graph = Graph()
    rt._infer_dict = lambda data: {}
    rt._status_host[0] = 2
    with pytest.raises(RuntimeError, match="device status 2"):
        rt.infer({})
    m = FastDeployModel.__new__(FastDeployModel)
    m.runtime, m._record_time = rt, False
    rt._status_host[0] = 3
    with pytest.raises(RuntimeError, match="epilogue wait timed out"):
        m.infer({})


def test_cpu_runtime_fast_path_matches_plain_interpreter(tmp_path):
    """The CPU runtime (optimised graph, channel-innermost operands, packed fused convolutions) returns what the plain
    interpreter returns on the imported graph."""
    import numpy as np
    import fastdeploy_b200 as fd
    from fastdeploy_b200.ir.interp import Interpreter
    from fastdeploy_b200.models.resnet import resnet18_like_onnx
    path = tmp_path / "r.onnx"
    path.write_bytes(resnet18_like_onnx())
    opt = fd.RuntimeOption()
    opt.use_cpu()
    opt.set_model_path(str(path), "", fd.ModelFormat.ONNX)
    rt = fd.Runtime(opt)
    for n in (1, 3):                                   # two input shapes: the packed weights are kept per shape
        x = np.random.RandomState(n).rand(n, 3, 64, 64).astype(np.float32)
        ref = Interpreter(rt.graph).run({"input": x})["output"].numpy()
        got = rt.infer({"input": x})[0]
        assert got.shape == ref.shape and np.abs(got - ref).max() < 1e-4 * max(1.0, np.abs(ref).max())


def test_initialized_reads_as_property_and_as_method():
    import fastdeploy_b200 as fd
    m = fd.FastDeployModel()
    assert not m.initialized and m.initialized() is False and repr(m.initialized) == "False"
    m.initialized_ = True
    assert m.initialized and m.initialized() is True
