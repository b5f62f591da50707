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


def test_ocr_evaluation_metrics():
    sq = lambda x, y, s: [x, y, x + s, y, x + s, y + s, x, y + s]
    gt = [[sq(0, 0, 10), sq(20, 0, 10)], [sq(5, 5, 10)]]
    pred = [[sq(1, 0, 10), sq(50, 50, 10), sq(20, 1, 10)], []]            # two hits, one false alarm, one image missed
    m = EV.ocr_detection_hmean(pred, gt)
    assert abs(m["precision"] - 2 / 3) < 1e-9 and abs(m["recall"] - 2 / 3) < 1e-9 and abs(m["hmean"] - 2 / 3) < 1e-9
    assert EV.ocr_detection_hmean([[sq(0, 0, 10)]], [[sq(6, 0, 10)]])["hmean"] == 0.0       # IoU 0.25 < 0.5
    assert EV.edit_distance("kitten", "sitting") == 3 and EV.edit_distance("", "abc") == 3
    r = EV.ocr_recognition_metrics(["he llo", "wrld", "X"], ["hello", "world", "x"])
    assert abs(r["acc"] - 1 / 3) < 1e-9 and abs(r["norm_edit_dis"] - (1 - (0 + 0.2 + 1.0) / 3)) < 1e-9
    assert EV.ocr_recognition_metrics(["X"], ["x"], ignore_case=True)["acc"] == 1.0

    class FakeOCR:
        def predict(self, im):
            from fastdeploy_b200.vision.result import OCRResult
            r = OCRResult()
            r.boxes, r.text = [sq(0, 0, 10), sq(40, 40, 8)], ["abc", "zzz"]
            return r
    out = EV.eval_ocr(FakeOCR(), [(np.zeros((64, 64, 3), np.uint8), [sq(0, 1, 10)], ["abd"])])
    assert out["recall"] == 1.0 and out["precision"] == 0.5 and out["rec_acc"] == 0.0 and abs(out["rec_norm_edit_dis"] - 2 / 3) < 1e-9


def test_cpu_resnet50_benchmark_line(tmp_path):
    """`bench.py --config resnet50_cpu` prints the benchmark line with the keys every configuration prints."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--config", "resnet50_cpu", "--steps", "5", "--warmup",
                        "3", "--model-dir", str(tmp_path)], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    line = json.loads(p.stdout.strip().splitlines()[-1])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "dtype", "data",
                "config", "vs_baseline", "impl"):
        assert key in line, key
    assert line["unit"] == "ms" and line["higher_is_better"] is False and line["n_gpus"] == 0 and line["value"] > 0
    assert set(line["by_threads"]) >= {"1"} and line["by_threads"]["1"]["runtime_ms"] <= line["by_threads"]["1"]["e2e_ms"] * 1.2
    ref = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference"], capture_output=True, text=True,
                         timeout=120)
    out = json.loads(ref.stdout.strip().splitlines()[-1])
    assert ref.returncode == 0 and out["impl"] == "reference" and "unavailable" in out


def test_subcommands_without_a_counterpart_say_so(capsys):
    from fastdeploy_b200.tools import main
    assert main(["paddle2coreml", "--p2c_paddle_model_dir", "x", "--p2c_coreml_model_name", "m"]) == 2
    assert "CoreML" in capsys.readouterr().err
    assert main(["convert", "--framework", "caffe", "--prototxt", "a", "--weight", "b"]) == 2
    assert "x2paddle" in capsys.readouterr().err
