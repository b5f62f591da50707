import json
import os

import numpy as np

from fastdeploy_b200 import tools
from fastdeploy_b200.vision import evaluation as EV


def test_convert_and_compress_and_benchmark(tmp_path, capsys):
    from fastdeploy_b200.models.resnet import resnet18_like_onnx
    src = str(tmp_path / "m.onnx")
    resnet18_like_onnx(src, seed=0)
    assert tools.main(["convert", "--model", src, "--save_dir", str(tmp_path / "conv")]) == 0
    assert os.path.getsize(tmp_path / "conv" / "model.onnx") > 1000
    assert tools.main(["compress", "--model", src, "--save_dir", str(tmp_path / "q"), "--calib_batches", "2"]) == 0
    q = json.load(open(tmp_path / "q" / "quant_scales.json"))
    assert q["format"] == "e4m3" and len(q["layers"]) > 5
    layer = next(iter(q["layers"].values()))
    assert layer["act_absmax"] > 0 and len(layer["weight_scale"]) > 0
    assert tools.main(["benchmark", "--model", src, "--repeat", "2", "--warmup", "1"]) == 0
    line = [l for l in capsys.readouterr().out.splitlines() if l.startswith("{")][-1]
    assert json.loads(line)["runtime_ms"] > 0


def test_e4m3_grid():
    x = np.array([0.0, 1.0, 1.06, 1.07, 447.0, 500.0, -3.3, 0.001], np.float32)
    r = tools.e4m3_round(x)
    assert r[0] == 0 and r[1] == 1.0 and r[2] == 1.0 and r[3] == 1.125 and r[4] == 448.0 and r[5] == 448.0 and r[6] == -3.25


def test_coco_map_and_miou():
    gt = [{"boxes": [[0, 0, 10, 10], [20, 20, 40, 40]], "labels": [0, 1]}]
    perfect = [{"boxes": [[0, 0, 10, 10], [20, 20, 40, 40]], "labels": [0, 1], "scores": [0.9, 0.8]}]
    assert abs(EV.coco_map(perfect, gt)["bbox_mAP"] - 1.0) < 1e-9
    shifted = [{"boxes": [[0, 0, 10, 8], [20, 20, 40, 40]], "labels": [0, 1], "scores": [0.9, 0.8]}]     # IoU 0.8 on class 0
    m = EV.coco_map(shifted, gt)
    assert m["bbox_mAP50"] == 1.0 and 0.7 < m["bbox_mAP"] < 1.0
    pred = np.array([[0, 0, 1], [1, 1, 1]])
    label = np.array([[0, 0, 0], [1, 1, 255]])
    s = EV.segmentation_metrics(pred, label, 2)
    assert abs(s["acc"] - 0.8) < 1e-9 and abs(s["miou"] - (2 / 3 + 2 / 3) / 2) < 1e-9
    assert EV.topk_accuracy(np.array([[0.1, 0.9], [0.8, 0.2]]), [1, 1], 1) == 0.5


def test_model_zoo_benchmark_driver_on_cpu(tmp_path):
    from fastdeploy_b200.benchmarks import model_zoo
    cfg_file = tmp_path / "config.cpu.txt"
    cfg_file.write_text("device: cpu\ncpu_thread_nums: 1\nwarmup: 1\nrepeat: 2\nprofile_mode: end2end\n"
                        "collect_memory_info: true\nsampling_interval: 1\nresult_path: %s\n" % (tmp_path / "result.txt"))
    cfg = model_zoo.load_benchmark_config(str(cfg_file))
    assert cfg["device"] == "cpu" and cfg["repeat"] == "2" and cfg["use_fp16"] == "true"
    assert model_zoo.main(["--model", "ppocr_cls", "--config_path", str(cfg_file)]) == 0
    text = (tmp_path / "result.txt").read_text()
    assert "End2End(ms):" in text and "cpu_rss_mb:" in text
    res = model_zoo.run_benchmark("ernie", dict(cfg, profile_mode="runtime", collect_memory_info="false", warmup="1", repeat="2"))
    assert res["Runtime(ms)"] > 0
