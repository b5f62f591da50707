"""Builds a C program against the C API header and library and runs it as a child process."""
import os
import shutil
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "fastdeploy_b200", "_native", "libfastdeploy_capi.so")


@pytest.mark.skipif(shutil.which("gcc") is None, reason="no C compiler")
def test_c_program_runs_a_model(tmp_path):
    if not os.path.exists(LIB):
        from fastdeploy_b200._native import build
        if not build.build_capi():
            pytest.skip("interpreter headers not available")
    import fastdeploy_b200 as fd
    from fastdeploy_b200.core.types import ModelFormat
    from fastdeploy_b200.models.resnet import resnet18_like_onnx
    model = str(tmp_path / "m.onnx")
    resnet18_like_onnx(model, seed=0)
    opt = fd.RuntimeOption(); opt.use_cpu(); opt.set_model_path(model, "", ModelFormat.ONNX)
    rt = fd.Runtime(opt)
    info = rt.get_input_info(0)
    shape = [d if isinstance(d, int) and d > 0 else 1 for d in info.shape]
    n, c, hw = shape[0], shape[1], shape[2]
    count = n * c * hw * hw
    x = ((np.arange(count, dtype=np.uint64) * np.uint64(2654435761)) % np.uint64(1000)).astype(np.float32) / np.float32(1000.0) - np.float32(0.5)
    ref = float(np.asarray(rt.infer({info.name: x.reshape(n, c, hw, hw)})[0], np.float64).sum())
    exe = str(tmp_path / "capi_smoke")
    subprocess.run(["gcc", os.path.join(ROOT, "tests", "capi_smoke.c"), "-I", os.path.join(ROOT, "csrc", "capi"), "-o", exe,
                    "-L", os.path.dirname(LIB), "-lfastdeploy_capi", f"-Wl,-rpath,{os.path.dirname(LIB)}"], check=True)
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.pathsep.join(p for p in sys.path if p), PYTHONHOME="")
    env.pop("PYTHONHOME")
    p = subprocess.run([exe, model, info.name, str(n), str(c), str(hw)], capture_output=True, text=True, env=env, timeout=300)
    assert p.returncode == 0, p.stdout + p.stderr
    lines = p.stdout.strip().splitlines()
    assert lines[0].startswith("inputs=1 outputs=1")
    chk = float(lines[1].split("checksum=")[1])
    assert abs(chk - ref) <= 1e-3 * max(1.0, abs(ref)), (chk, ref)
    assert lines[2] == "bad=null err=set"


@pytest.mark.skipif(shutil.which("gcc") is None, reason="no C compiler")
def test_plan_runner_header_links_and_reports_errors(tmp_path):
    """The plan runner is a plain C library: a C program links it without Python and gets messages, not crashes."""
    from fastdeploy_b200 import _native
    from fastdeploy_b200._native import build
    if not os.path.exists(build.RUNNER_LIB):
        build.build_runner()
    exe = str(tmp_path / "plan_runner_smoke")
    subprocess.run(["gcc", os.path.join(ROOT, "tests", "plan_runner_smoke.c"), "-I", os.path.join(ROOT, "csrc", "runner"),
                    "-o", exe, "-L", os.path.dirname(build.RUNNER_LIB), "-lfdb200_runner",
                    f"-Wl,-rpath,{os.path.dirname(build.RUNNER_LIB)}"], check=True)
    junk = tmp_path / "junk.fdplan"
    junk.write_bytes(b"not a plan file at all")
    p = subprocess.run([exe, _native.KERNEL_LIB, str(tmp_path / "absent.fdplan"), str(junk)], capture_output=True,
                       text=True, timeout=120)
    assert p.returncode == 0, p.stdout + p.stderr
    lines = p.stdout.strip().splitlines()
    assert lines[0].startswith("missing: null | cannot open") and lines[1] == "garbage: null | not a plan file"
    assert lines[2] == "nolib: null | message"
    # the library itself does not depend on the interpreter
    deps = subprocess.run(["ldd", build.RUNNER_LIB], capture_output=True, text=True).stdout
    assert "python" not in deps.lower()


@pytest.mark.skipif(shutil.which("gcc") is None, reason="no C compiler")
def test_c_program_uses_models_by_name_batches_text_and_image_files(tmp_path):
    from fastdeploy_b200._native import build
    if not build.build_capi():
        pytest.skip("interpreter headers not available")
    import fastdeploy_b200 as fd
    from fastdeploy_b200.models.ppyoloe import write_ppyoloe
    from fastdeploy_b200.models.vit import write_vit
    det = write_ppyoloe(str(tmp_path / "det"), "tiny", image=96, num_classes=6, score_threshold=0.005)
    cls = write_vit(str(tmp_path / "cls"), "tiny", image=32, num_classes=10, seed=3)
    exe = str(tmp_path / "capi_models")
    subprocess.run(["gcc", "-Wall", "-Werror", os.path.join(ROOT, "tests", "capi_models.c"), "-I", os.path.join(ROOT, "csrc", "capi"),
                    "-o", exe, "-L", os.path.dirname(LIB), "-lfastdeploy_capi", f"-Wl,-rpath,{os.path.dirname(LIB)}"], check=True)
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.pathsep.join(p for p in sys.path if p))
    env.pop("PYTHONHOME", None)
    png = str(tmp_path / "drawn.png")
    p = subprocess.run([exe, det["model"], det["params"], det["config"], cls["model"], cls["params"], cls["config"], png],
                       capture_output=True, text=True, env=env, timeout=600)
    assert p.returncode == 0, p.stdout + p.stderr
    out = dict(line.split("=", 1) for line in p.stdout.strip().splitlines() if "=" in line)
    assert out["options"] == "ok" and out["initialized"] == "1"
    assert out["boxes"].endswith("batch_equals_single=1")
    n0 = int(out["boxes"].split(",")[0])
    # the same two images through the Python class
    opt = fd.RuntimeOption(); opt.use_cpu()
    m = fd.vision.detection.PicoDet(det["model"], det["params"], det["config"], runtime_option=opt)

    def image(h, w, seed):
        vals = []
        for _ in range(h * w * 3):
            seed = (seed * 1664525 + 1013904223) & 0xFFFFFFFF
            vals.append(seed >> 24)
        return np.asarray(vals, np.uint8).reshape(h, w, 3)

    ims = [image(60, 120, 1), image(70, 120, 2)]
    want = m.batch_predict(ims)
    assert n0 == len(want[0].scores)
    text = str(want[0])
    assert out["str_need"].startswith(f"{len(text.encode()) + 1} head=DetectionResult: [xmin, ymin, xmax, ymax")
    assert out["tiny"] == "Detecti"                                   # 7 characters and the terminator
    assert out["png_roundtrip"] == "1" and os.path.getsize(png) > 0
    assert out["missing"] == "null err=set" and out["yolov5"] == "null"
    c = fd.vision.classification.PaddleClasModel(cls["model"], cls["params"], cls["config"], runtime_option=opt)
    labels = [r.label_ids[0] for r in c.batch_predict(ims)]
    assert out["cls_initialized"] == f"1 labels={labels[0]},{labels[1]} single={labels[0]}"
    assert out["cls_str"] == "ClassifyResult("
    assert int(out["empty_ocr_str_len"]) >= 0


@pytest.mark.skipif(shutil.which("gcc") is None, reason="no C compiler")
def test_c_program_runs_the_ocr_stages_one_by_one(tmp_path):
    from fastdeploy_b200._native import build
    if not build.build_capi():
        pytest.skip("interpreter headers not available")
    import fastdeploy_b200 as fd
    from fastdeploy_b200.models.ppocr import write_ppocr
    paths = write_ppocr(str(tmp_path / "ocr"), vocab=64)
    exe = str(tmp_path / "capi_ocr_stages")
    subprocess.run(["gcc", "-Wall", "-Werror", os.path.join(ROOT, "tests", "capi_ocr_stages.c"), "-I", os.path.join(ROOT, "csrc", "capi"),
                    "-o", exe, "-L", os.path.dirname(LIB), "-lfastdeploy_capi", f"-Wl,-rpath,{os.path.dirname(LIB)}"], check=True)
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.pathsep.join(p for p in sys.path if p))
    env.pop("PYTHONHOME", None)
    p = subprocess.run([exe, paths["det_model"], paths["det_params"], paths["cls_model"], paths["cls_params"], paths["rec_model"],
                        paths["rec_params"], paths["dict"]], capture_output=True, text=True, env=env, timeout=600)
    assert p.returncode == 0, p.stdout + p.stderr
    out = dict(line.split("=", 1) for line in p.stdout.strip().splitlines() if "=" in line)
    assert out["initialized"] == "111" and out["bad"] == "null"
    vals = []
    seed = 7
    for _ in range(64 * 160 * 3):
        seed = (seed * 1664525 + 1013904223) & 0xFFFFFFFF
        vals.append(seed >> 24)
    page = np.asarray(vals, np.uint8).reshape(64, 160, 3)
    opt = fd.RuntimeOption(); opt.use_cpu()
    ocr = fd.vision.ocr
    boxes = ocr.DBDetector(paths["det_model"], paths["det_params"], runtime_option=opt).predict(page)
    assert out["boxes"] == f"{len(boxes)} all_have_8=1"
    label, score = ocr.Classifier(paths["cls_model"], paths["cls_params"], runtime_option=opt).predict(page)
    got_label, got_score = out["cls"].split()
    assert int(got_label) == label and abs(float(got_score) - score) < 1e-5
    text, rscore = ocr.Recognizer(paths["rec_model"], paths["rec_params"], paths["dict"], runtime_option=opt).predict(page)
    nbytes, got_rscore = out["rec_bytes"].split()
    assert int(nbytes) == len(text.encode()) and abs(float(got_rscore) - rscore) < 1e-5 and out.get("rec_text", "") == text
